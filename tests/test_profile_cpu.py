"""Profiles: tunables by operator shape, applied as an operator is made (no GPU).

The behaviours iron/tests/common/test_declare.py:344-390 pins for the reference's ``Profile``:
the most specific matching entry gives each open tunable, what the call gives wins and is
pinned, a tunable given as None is left to the profile, equally specific entries that disagree
are an error, entries are checked as they are added, files are checked as they are read, and a
graph makes its steps through its profile.
"""

import json

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.declare import In, Operator, Out, param, tunable
from iron_b200.profile import Profile


class MV(Operator):
    """A toy operator with two tunables, one of which has a declared default."""

    M: int = param()
    K: int = param()
    columns: int = tunable()
    tile_out: int = tunable(default=64)
    A = In(M, K)
    x = In(K)
    y = Out(M)


def test_a_profile_fills_the_tunables_a_call_leaves_open():
    p = Profile()
    p.add(MV, columns=4, tile_out=32)   # any MV: a declared default counts as open
    p.add(MV, K=256, tile_out=16)       # more specific: it names K
    a = p.make(MV, M=1024, K=128)
    assert (a.columns, a.tile_out) == (4, 32)
    b = p.make(MV, M=1024, K=256)
    assert (b.columns, b.tile_out) == (4, 16)
    c = p.make(MV, M=1024, K=256, tile_out=8)   # what the call gives wins, and is pinned
    assert c.tile_out == 8 and c.pinned == {"tile_out"}
    plain = MV(M=1024, K=128)                   # plain construction reads no profile
    assert plain.columns is None and plain.tile_out == 64
    assert p.tunables_for(MV, dict(M=1024, K=256)) == {"columns": 4, "tile_out": 16}
    assert len(p) == 2 and repr(p) == "Profile(MV)"


def test_a_tunable_given_as_none_is_left_to_the_profile():
    p = Profile()
    p.add(MV, columns=4, tile_out=32)
    op = p.make(MV, M=1024, K=128, columns=None, tile_out=None)
    assert (op.columns, op.tile_out, op.pinned) == (4, 32, set())


def test_a_base_class_entry_serves_its_subclasses():
    class Wide(MV):
        pass

    p = Profile()
    p.add(MV, columns=2)
    assert p.make(Wide, M=8, K=8).columns == 2


def test_a_profile_is_checked_as_it_is_written_and_ambiguity_is_an_error():
    p = Profile()
    with pytest.raises(TypeError, match="declares no field"):
        p.add(MV, rows=4, columns=2)
    with pytest.raises(TypeError, match="must give a tunable"):
        p.add(MV, M=1024)
    p.add(MV, M=1024, columns=2)
    p.add(MV, K=128, columns=8)     # as specific as the first: a clash for (1024, 128)
    assert p.make(MV, M=512, K=128).columns == 8
    with pytest.raises(ValueError, match="ambiguous"):
        p.make(MV, M=1024, K=128)


def test_profiles_round_trip_through_json_and_files_are_checked(tmp_path):
    from iron_b200.operators import GEMV, MHA

    p = Profile()
    p.add(MHA, seq_len=1, key_splits=8)
    p.add(MHA, seq_len=1, kv_len=256, key_splits=2)
    p.add(GEMV, M=2048, K=8192, num_aie_columns=4)   # an AIE tunable: accepted, ignored by the launch
    path = tmp_path / "b200.json"
    p.save(path)
    data = json.loads(path.read_text())
    assert set(data) == {"entries"} and data["entries"][1] == {"operator": "MHA", "seq_len": 1, "kv_len": 256,
                                                               "key_splits": 2}
    q = Profile.load(path)
    assert [(c.__name__, d, t) for c, d, t in q] == [(c.__name__, d, t) for c, d, t in p]
    op = q.make(MHA, num_heads=32, num_KV_heads=8, seq_len=1, kv_len=256, heads_interleaved=True,
                kv_interleaved=True)
    assert op.key_splits == 2
    assert q.make(MHA, num_heads=32, num_KV_heads=8, seq_len=1, kv_len=4096).key_splits == 8
    assert q.make(MHA, num_heads=32, num_KV_heads=8, seq_len=2048, kv_len=4096).key_splits is None
    other = Profile()
    other.add(MV, columns=4)
    with pytest.raises(ValueError, match="MV is not in the catalogue"):
        other.save(tmp_path / "x.json")
    (tmp_path / "bad.json").write_text('{"rows": []}')
    with pytest.raises(ValueError, match="a profile is"):
        Profile.load(tmp_path / "bad.json")
    (tmp_path / "unknown.json").write_text('{"entries": [{"operator": "Nope", "columns": 1}]}')
    with pytest.raises(ValueError, match="no operator 'Nope'"):
        Profile.load(tmp_path / "unknown.json")


def test_a_graph_makes_its_steps_through_its_profile():
    """The Llama graph's decode step records its one-query MHA with the key split the shipped
    B200 profile gives a 256-row cache; a graph without a profile leaves it open."""
    from iron_b200.applications.llama.model import Llama
    from oracle import model as M
    from tests.test_engine_gpu import toy_config

    weights = M.filled_random(M.llama_shapes(M.SCALED), 0)
    model = Llama(toy_config(), weights)
    steps = [s.op for s in model.record().steps if type(s.op).__name__ == "MHA"]
    assert steps and all(op.key_splits == 2 and op.pinned == set() for op in steps)
    chunk = model.record(ids=((256,), np.int32))
    assert all(s.op.key_splits is None for s in chunk.steps if type(s.op).__name__ == "MHA")

    class Bare(Llama):
        profile = None

    assert all(s.op.key_splits is None for s in Bare(toy_config(), weights).record().steps
               if type(s.op).__name__ == "MHA")
