"""Tensor-parallel sharding and its one exchange step, on two CPU ranks over gloo.

The kernels need a GPU; what is checked here is the host-side logic the N > 1 path rests on:
``shard_layout`` splits heads and MLP rows, each rank's partial o_proj / down_proj products
sum (one all-reduce each) to the unsharded layer's, and replicas of a batch split evenly.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from iron_b200.applications.llama.model import LLAMA_3B, LlamaConfig


def _config():
    return LlamaConfig(vocab_size=256, hidden_size=128, num_hidden_layers=1, num_attention_heads=8,
                       num_key_value_heads=4, head_dim=16, intermediate_size=256, rope_theta=500000.0,
                       max_seq_len=64)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _layer(x, w, heads_slice=None, ffn_slice=None):
    """Attention-free stand-in for one layer's two row-parallel products (float64)."""
    q = w["q"][heads_slice] @ x if heads_slice is not None else w["q"] @ x
    wo = w["o"][:, heads_slice] if heads_slice is not None else w["o"]
    att = wo @ q
    g = w["g"][ffn_slice] if ffn_slice is not None else w["g"]
    u = w["u"][ffn_slice] if ffn_slice is not None else w["u"]
    d = w["d"][:, ffn_slice] if ffn_slice is not None else w["d"]
    return att, d @ ((g @ x) * (u @ x))


def _rank(rank: int, size: int, port: int, out):
    from iron_b200.lm.engine import shard_layout

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=size)
    c = _config()
    rng = np.random.default_rng(0)
    E, Q, F = c.hidden_size, c.num_attention_heads * c.head_dim, c.intermediate_size
    w = {"q": rng.standard_normal((Q, E)), "o": rng.standard_normal((E, Q)), "g": rng.standard_normal((F, E)),
         "u": rng.standard_normal((F, E)), "d": rng.standard_normal((E, F))}
    x = rng.standard_normal(E)
    lay = shard_layout(c, rank, size)
    att, mlp = _layer(x, w, lay.q_rows, lay.ffn_rows)
    t = torch.from_numpy(np.stack([att, mlp]))
    dist.all_reduce(t)
    if rank == 0:
        full = np.stack(_layer(x, w))
        out.put(float(np.abs(t.numpy() - full).max() / np.abs(full).max()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_partial_products_all_reduce_to_the_whole():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out.get(timeout=10) < 1e-12


def test_shard_layout_covers_every_row_once_and_refuses_uneven_splits():
    from iron_b200.lm.engine import shard_layout

    c = LLAMA_3B
    for size in (1, 2, 4, 8):
        q, kv, f = [], [], []
        for r in range(size):
            lay = shard_layout(c, r, size)
            assert lay.heads * size == 24 and lay.kv_heads * size == 8 and lay.ffn * size == 8192
            q += list(range(*lay.q_rows.indices(10 ** 9)))
            kv += list(range(*lay.kv_rows.indices(10 ** 9)))
            f += list(range(*lay.ffn_rows.indices(10 ** 9)))
        assert q == list(range(24 * 128)) and kv == list(range(8 * 128)) and f == list(range(8192))
    with pytest.raises(ValueError):
        shard_layout(c, 0, 16)       # 8 KV heads do not split 16 ways
    with pytest.raises(ValueError):
        shard_layout(c, 3, 2)


def test_batch_shards_split_sequences_evenly():
    from iron_b200.lm.engine import batch_shard

    for n in (1, 2, 4, 8):
        parts = [batch_shard(64, r, n) for r in range(n)]
        assert sum(len(p) for p in parts) == 64 and sorted(sum(map(list, parts), [])) == list(range(64))
        assert len({len(p) for p in parts}) == 1
    assert [len(batch_shard(10, r, 4)) for r in range(4)] == [3, 3, 2, 2]
