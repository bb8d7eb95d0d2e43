"""The reference's own model files, unmodified, on this package (no GPU).

``iron/applications/llama/model.py``, ``granite/model.py`` and ``granite_hybrid/model.py`` are
loaded from the reference checkout as they lie there -- nothing is copied or edited -- with
``iron`` resolving to this repository's alias package, so their ``from iron import ...``,
``from iron.lm import ...`` and ``from iron.operators... import ...`` bind to this package's
declaration layer, graph layer and model library.  Their classes are then built on the toys'
drawn weights, recorded, and run on the host: the recorded steps are the ones this package's
own model files record, and the logits lie inside the reference's bound of its golden rows.
Skipped where the reference checkout is not mounted.
"""

import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import model as M
from tests.test_oracle_golden import assert_close

# a checkout of amd/IRON: IRON_REFERENCE, or a `reference` directory beside this repository
REFERENCE = Path(os.environ.get("IRON_REFERENCE") or Path(__file__).resolve().parents[2] / "reference")
pytestmark = pytest.mark.skipif(not (REFERENCE / "iron" / "applications").is_dir(),
                                reason="the reference checkout is not mounted")
GOLDENS = Path(__file__).parent / "golden"


def reference_module(relative: str, name: str):
    """Execute a reference source file in place under module ``name``."""
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import iron  # noqa: F401  (installs the alias finder)

    spec = importlib.util.spec_from_file_location(name, REFERENCE / relative)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def golden_rows(fixture):
    with np.load(GOLDENS / fixture) as z:
        return {k: z[k] for k in z.files}


def signature(recording):
    """What a recording is made of: each step's operator and its construction fields."""
    out = []
    for s in recording.steps:
        fields = {n: getattr(s.op, n) for n, f in type(s.op).declaration.params.items() if f.kind == "param"}
        out.append((type(s.op).__name__, tuple(sorted((k, repr(v)) for k, v in fields.items()))))
    return out


def test_the_reference_llama_model_file_records_and_runs_on_this_package():
    ref = reference_module("iron/applications/llama/model.py", "reference_llama_model")
    from iron_b200.applications.llama.model import Llama, Llama3RopeScaling, LlamaConfig

    kw = dict(vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=16, num_key_value_heads=4,
              head_dim=64, intermediate_size=2048, rope_theta=500000.0, max_seq_len=256, eps=1e-5, prefill_chunk=256)
    theirs = ref.Llama(ref.LlamaConfig(rope_scaling=ref.Llama3RopeScaling(8.0, 1.0, 4.0, 64), **kw),
                       M.filled_random(M.llama_shapes(M.SCALED), 0))
    ours = Llama(LlamaConfig(rope_scaling=Llama3RopeScaling(8.0, 1.0, 4.0, 64), **kw),
                 M.filled_random(M.llama_shapes(M.SCALED), 0))
    assert type(theirs).__module__ == "reference_llama_model" and isinstance(theirs, type(ours).__mro__[1])
    for shapes in ({}, dict(ids=((256,), np.int32))):       # the decode step and the prompt chunk
        assert signature(theirs.record(**shapes)) == signature(ours.record(**shapes))
    golden = golden_rows("llama_small.npz")
    prompt = np.random.default_rng(7).integers(0, 1024, 8)
    got = theirs.reference_logits(prompt)
    assert_close(got, golden[M.golden_key(prompt)])
    assert np.array_equal(got, ours.reference_logits(prompt))
    tokens = np.append(prompt, got.argmax())
    assert_close(theirs.reference_logits(tokens[-1:], len(prompt)), golden[M.golden_key(tokens)])


def test_the_reference_granite_and_hybrid_model_files_run_on_this_package():
    granite = reference_module("iron/applications/granite/model.py", "reference_granite_model")
    # the hybrid's file imports Granite from its application path: give it the reference's own
    saved = sys.modules.get("iron.applications.granite.model")
    sys.modules["iron.applications.granite.model"] = granite
    try:
        hybrid = reference_module("iron/applications/granite_hybrid/model.py", "reference_granite_hybrid_model")
    finally:
        if saved is None:
            sys.modules.pop("iron.applications.granite.model", None)
        else:
            sys.modules["iron.applications.granite.model"] = saved
    assert hybrid.GraniteHybrid.__mro__[1] is granite.Granite

    c = M.GRANITE_TOY
    config = granite.GraniteConfig(
        vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
        intermediate_size=1024, rope_theta=10000.0, max_seq_len=256, prefill_chunk=256, tie_word_embeddings=False,
        attention_multiplier=0.0625, residual_multiplier=0.22, embedding_multiplier=12.0, logits_scaling=8.0)
    weights = M.filled_random(M.decoder_shapes(c), 0)
    model = granite.Granite(config, weights)
    golden = golden_rows("granite_toy.npz")
    prompt = np.random.default_rng(0).integers(0, 1024, 8)
    got = model.reference_logits(prompt)
    assert_close(got, golden[M.golden_key(prompt)])
    assert np.array_equal(got, M.NumpyDecoder(c, weights).forward(prompt, 0).astype(np.float32))

    c = M.HYBRID_TOY
    config = hybrid.GraniteHybridConfig(
        vocab_size=1024, hidden_size=512, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=2,
        intermediate_size=256, max_seq_len=256, prefill_chunk=64, attention_multiplier=0.0625,
        residual_multiplier=0.22, embedding_multiplier=12.0, logits_scaling=8.0, tie_word_embeddings=False,
        layer_types=("mamba", "attention", "mamba", "mamba"), position_embedding_type="nope",
        shared_intermediate_size=512, num_local_experts=0, num_experts_per_tok=2, mamba_n_heads=16, mamba_d_head=64,
        mamba_d_state=64, mamba_n_groups=2)
    weights = M.hybrid_redraw(c, M.filled_random(M.decoder_shapes(c), 0))
    model = hybrid.GraniteHybrid(config, weights)
    golden = golden_rows("granite_hybrid_dense.npz")
    prompt = np.random.default_rng(2).integers(0, 1024, 8)
    oracle = M.NumpyDecoder(c, weights)
    got = model.reference_logits(prompt)
    assert_close(got, golden[M.golden_key(prompt)])
    assert np.array_equal(got, oracle.forward(prompt, 0).astype(np.float32))
    tokens = np.append(prompt, got.argmax())
    got = model.reference_logits(tokens[-1:], len(prompt))       # a decode step: the mixers' states carry on
    assert_close(got, golden[M.golden_key(tokens)])
    assert np.array_equal(got, oracle.forward(tokens[-1:], len(prompt)).astype(np.float32))
    long = np.random.default_rng(3).integers(0, 1024, 64 + 150)  # several 64-row chunks
    model = hybrid.GraniteHybrid(hybrid.dataclasses.replace(config, max_seq_len=256), weights)
    assert_close(model.reference_logits(long), golden[M.golden_key(long)])


def test_the_reference_import_paths_resolve_to_this_packages_objects():
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    import iron
    import iron.functional as F
    from iron import Graph, Precision, Profile, carry, param, state, weight  # noqa: F401
    from iron.common.declare.precision import Precision as P2
    from iron.common.graph import CompiledGraph, Handle  # noqa: F401
    from iron.common.graph.compiled import walk  # noqa: F401
    from iron.common.graph.handle import State  # noqa: F401
    from iron.lm import CausalConv1d, CausalLM, Checkpoints, DecoderConfig, Linear, RMSNorm, residual_add  # noqa: F401
    from iron.operators.copy import Copy
    from iron.operators.flm.gemm.design import Epilogue  # noqa: F401
    from iron.operators.flm.gemm.op import ProjectionGEMM  # noqa: F401
    from iron.operators.gemv import GEMV
    from iron.operators.selective_scan import SelectiveScan  # noqa: F401

    import iron_b200.functional
    import iron_b200.operators.copy
    import iron_b200.operators.gemv

    assert F is iron_b200.functional and GEMV is iron_b200.operators.gemv.GEMV and Copy is iron_b200.operators.copy.Copy
    assert P2 is Precision and iron.lm.CausalLM is CausalLM


def test_importing_iron_loads_no_torch():
    """iron/tests/infrastructure/test_no_torch_on_import.py:56-58: ``import iron`` stays light."""
    import subprocess

    root = str(Path(__file__).resolve().parents[1])
    code = ("import sys; sys.path.insert(0, %r); import iron, iron.functional, iron.lm; "
            "from iron.lm import CausalLM, DecoderConfig; from iron.operators.gemv import GEMV; "
            "assert 'torch' not in sys.modules, sorted(m for m in sys.modules if m.startswith('torch'))[:3]") % root
    subprocess.run([sys.executable, "-c", code], check=True)
