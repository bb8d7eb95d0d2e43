"""Checkpoints without a device: the safetensors reader, trees, fills, the staging uploader.

The contracts of iron/lm/checkpoint.py (:31-118 the file format and its refusals, :220-294
``Checkpoint``, :297-424 trees) and of iron/common/graph/fill.py; the random fill is held
bit for bit to the oracle's restatement, which the golden logits pin.
"""

import json
import struct

import numpy as np
import pytest
from ml_dtypes import bfloat16

from iron_b200.lm import Checkpoint, leaves, nest, renamed, save_file, subtree, weights_file
from iron_b200.lm.checkpoint import Uploader, filled
from oracle import model as M


def small(seed=0):
    rng = np.random.default_rng(seed)
    return {"model.embed_tokens.weight": rng.standard_normal((32, 16)).astype(bfloat16),
            "model.layers.0.mlp.up_proj.weight": rng.standard_normal((24, 16)).astype(bfloat16),
            "model.layers.1.mlp.up_proj.weight": rng.standard_normal((24, 16)).astype(np.float32),
            "model.layers.1.mlp.up_proj.bias": rng.standard_normal((24,)).astype(np.float16),
            "model.norm.weight": np.ones(16, bfloat16),
            "steps": np.arange(3, dtype=np.int64)}


def bits(a):
    return np.ascontiguousarray(a).view(np.uint8)


def test_a_file_round_trips_every_dtype_and_views_stay_lazy_and_read_only(tmp_path):
    t = small()
    c = Checkpoint(save_file(t, tmp_path / "model.safetensors", {"format": "pt"}))
    assert list(c.tensors) == list(t)
    for n, a in t.items():
        assert c.tensors[n].dtype == a.dtype and c.tensors[n].shape == a.shape
        assert np.array_equal(bits(c.tensors[n]), bits(a))
        assert not c.tensors[n].flags.writeable
    c.release(c.tensors["model.embed_tokens.weight"])        # pages dropped, bytes still there
    assert np.array_equal(bits(c.tensors["model.embed_tokens.weight"]), bits(t["model.embed_tokens.weight"]))
    c.release(np.zeros(4))                                   # not a view of the file: left alone
    assert weights_file(tmp_path) == tmp_path / "model.safetensors"


def test_a_sharded_checkpoint_merges_its_shards_and_checks_them_against_the_index(tmp_path):
    t = small()
    names = list(t)
    save_file({n: t[n] for n in names[:3]}, tmp_path / "a.safetensors")
    save_file({n: t[n] for n in names[3:]}, tmp_path / "b.safetensors")
    index = {"weight_map": {n: ("a.safetensors" if i < 3 else "b.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    assert weights_file(tmp_path).name == "model.safetensors.index.json"
    c = Checkpoint(weights_file(tmp_path))
    assert set(c.tensors) == set(t) and all(np.array_equal(bits(c.tensors[n]), bits(t[n])) for n in t)
    index["weight_map"]["model.norm.weight"] = "a.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(ValueError, match="the index does not name"):
        Checkpoint(tmp_path / "model.safetensors.index.json")
    index["weight_map"]["model.norm.weight"] = "../b.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(ValueError, match="not a file beside the index"):
        Checkpoint(tmp_path / "model.safetensors.index.json")


def _write(path, header: dict, data: bytes):
    blob = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(blob)) + blob + data)
    return path


def test_malformed_files_are_refused_by_name(tmp_path):
    p = tmp_path / "x.safetensors"
    with pytest.raises(ValueError, match="w is F8"):
        Checkpoint(_write(p, {"w": {"dtype": "F8", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 4))
    with pytest.raises(ValueError, match="no data_offsets or shape"):
        Checkpoint(_write(p, {"w": {"dtype": "F32", "data_offsets": [0, 4]}}, b"\0" * 4))
    with pytest.raises(ValueError, match="spans bytes"):
        Checkpoint(_write(p, {"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 8))
    with pytest.raises(ValueError, match="spans bytes"):
        Checkpoint(_write(p, {"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError, match="a header of"):
        Checkpoint(p)
    with pytest.raises(ValueError, match="safetensors here holds"):
        save_file({"w": np.zeros(3, np.int8)}, p)


def test_trees_nest_at_the_dots_and_say_where_a_missing_name_is(tmp_path):
    t = small()
    c = Checkpoint(save_file(t, tmp_path / "model.safetensors"))
    tree = c.tree()
    assert np.array_equal(bits(tree.model.layers[1].mlp.up_proj.bias), bits(t["model.layers.1.mlp.up_proj.bias"]))
    assert dict(leaves(tree)).keys() == t.keys()
    with pytest.raises(AttributeError, match=r"model\.layers\.0\.mlp\.down_proj is not in .*it has up_proj"):
        tree.model.layers[0].mlp.down_proj
    with pytest.raises(IndexError, match=r"model\.layers\.2 is not in .*it has 2"):
        tree.model.layers[2]
    moved = renamed(tree, {"model.layers": "decoder.blocks", "mlp.up_proj": "ffn.up"})
    assert "decoder.blocks.1.mlp.up_proj.bias" in dict(leaves(moved)) and "model.norm.weight" in dict(leaves(moved))
    assert dict(leaves(tree)).keys() == t.keys()             # the original is left as it was
    part = subtree(tree, text=tree.model, head=tree.model.norm)
    assert part.text.layers[0] is tree.model.layers[0] and part.head.weight is tree.model.norm.weight
    # a skipped index is an empty module; a far index is refused
    sparse = nest({"seq.0.weight": 1, "seq.2.weight": 2})
    assert len(sparse.seq) == 3 and not dict(leaves(sparse.seq[1]))
    with pytest.raises(ValueError, match="past its 1 layers"):
        nest({"seq.1000.weight": 1})


def test_fills_read_nothing_and_the_random_draw_is_the_pinned_one(tmp_path):
    shapes = M.llama_shapes(M.SCALED)
    zeros = {n: np.zeros(s, bfloat16) for n, s in shapes.items()}
    c = Checkpoint(save_file(zeros, tmp_path / "model.safetensors"))
    drawn = c.named("random", seed=0)
    want = M.filled_random(shapes, 0)
    assert drawn.keys() == want.keys()
    assert all(np.array_equal(bits(drawn[n]), bits(want[n])) for n in want)
    assert not any(a.any() for a in c.named("unread").values())
    assert c.tree("random", 3).model.norm.weight.shape == shapes["model.norm.weight"]
    with pytest.raises(ValueError, match="read, random or unread"):
        c.named("ones")
    assert filled("random", {"b.bias": ((4,), np.float32)}, 1)["b.bias"].mean() < 0.5   # a bias without the one


def test_a_fingerprint_tells_a_changed_tensor_without_reading_the_whole(tmp_path):
    t = small()
    a = Checkpoint(save_file(t, tmp_path / "a.safetensors")).fingerprint()
    assert a == Checkpoint(save_file(t, tmp_path / "b.safetensors")).fingerprint()
    t["model.norm.weight"] = t["model.norm.weight"].copy()
    t["model.norm.weight"][-1] = 2
    assert a != Checkpoint(save_file(t, tmp_path / "c.safetensors")).fingerprint()


def test_the_uploader_stages_in_pieces_casts_and_fills_strided_rows():
    import torch

    rng = np.random.default_rng(0)
    released = []
    up = Uploader("cpu", slot_bytes=96, slots=2, release=released.append)
    a = rng.standard_normal((7, 40)).astype(np.float32)            # 560 bytes of bf16: six pieces
    out = torch.zeros(7, 40, dtype=torch.bfloat16)
    up.put(a, out)
    assert torch.equal(out, torch.from_numpy(a).to(torch.bfloat16)) and released[-1] is a
    packed = torch.zeros(7, 64, dtype=torch.bfloat16)
    up.put(a.astype(bfloat16), packed[:, 8:48])                    # a column run of a wider matrix
    assert torch.equal(packed[:, 8:48], out) and not packed[:, :8].any() and not packed[:, 48:].any()
    up.put(a[:, ::2], out.view(-1)[:140].view(7, 20))              # a strided source is gathered first
    assert torch.equal(out.view(-1)[:140].view(7, 20), torch.from_numpy(a[:, ::2].copy()).to(torch.bfloat16))
    with pytest.raises(ValueError, match="does not fill"):
        up.put(a, torch.zeros(3, dtype=torch.bfloat16))
    up.finish()


def test_the_command_line_refuses_what_it_cannot_do_before_loading(tmp_path, capsys):
    from iron_b200.applications.llama.model import Llama
    from iron_b200.lm.cli import main

    for argv, said in ((["x", "--check-determinism", "1"], "give 2 or more"),
                       (["x", "--top-k", "100"], "not one the device draws"),
                       (["x", "--temperature", "-1"], "is negative"),
                       (["x", "--check-accuracy", "--check-determinism", "2"], "not allowed with")):
        with pytest.raises(SystemExit):
            main(Llama, argv)
        assert said in capsys.readouterr().err
