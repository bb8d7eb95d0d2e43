"""The Llama-architecture decoder as fused sm_100a kernels over one device arena.

This is what a compiled ``CausalLM`` graph of the reference becomes on B200
(iron/lm/causal.py:271-349 recorded over iron/lm/blocks.py:627-733): the reference's 18
operator steps per layer run as five kernels,

    1. RMSNorm + fused q/k/v GEMV + RoPE + KV-cache write      (iron_decode_qkv_rope_bf16)
    2. one-query attention, split over the keys                (iron_mha_decode_bf16)
    3. o_proj GEMV + residual add                              (iron_gemv_bf16)
    4. RMSNorm + gate/up GEMV + SiLU + multiply                (iron_gemv_swiglu_bf16)
    5. down_proj GEMV + residual add                           (iron_gemv_bf16)

-- and where a CTA's share of o_proj fits an SM's shared memory (one sequence, one GPU),
kernels 2 and 3 are one launch, a thread-block cluster per KV group whose weights and keys
are staged while kernel 1 still runs (iron_decode_attn_oproj_bf16) --

between an embedding-row gather and the final norm + tied-head GEMV + greedy draw, all
captured in one CUDA graph.  The per-call values (token, position) live in a small device
buffer the last kernel updates, so ``generate`` replays the graph once per token with no
host round trip, as the reference's device-carried loop does
(iron/common/graph/carried.py:189-276).

Weights, KV caches and intermediates are slices of one HBM allocation planned by
``iron_b200.arena.ArenaPlan``.
"""

from __future__ import annotations

import dataclasses
import math
import os

import numpy as np
import torch

from .. import kernels as K
from ..arena import ArenaPlan
from ..tensor import capturing
from .config import DecoderConfig

BF16 = torch.bfloat16


def _as_device_bf16(a, out: torch.Tensor) -> None:
    """Copy ``a`` (numpy bf16 via ml_dtypes, or a torch tensor) into arena slice ``out``."""
    if isinstance(a, torch.Tensor):
        out.copy_(a.to(BF16).reshape(out.shape))
        return
    a = np.ascontiguousarray(a)
    if a.dtype.name == "bfloat16":
        t = torch.from_numpy(a.view(np.int16)).view(BF16)
    else:
        t = torch.from_numpy(a.astype(np.float32)).to(BF16)
    out.copy_(t.reshape(out.shape))


@dataclasses.dataclass(frozen=True)
class ShardLayout:
    """What one tensor-parallel rank holds of each projection."""

    heads: int
    kv_heads: int
    ffn: int
    q_rows: slice      # rows of q_proj (and columns of o_proj)
    kv_rows: slice     # rows of k_proj and v_proj
    ffn_rows: slice    # rows of gate/up_proj (and columns of down_proj)


def shard_layout(c: DecoderConfig, rank: int, size: int) -> ShardLayout:
    """Split heads and MLP rows ``size`` ways; raises ``ValueError`` when they do not divide."""
    H, G, D, F = c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.intermediate_size
    if not 0 <= rank < size:
        raise ValueError(f"rank {rank} is outside 0..{size - 1}")
    if H % size or G % size or F % size or (F // size) % 8:
        raise ValueError(f"{H} heads, {G} KV heads and {F} MLP rows do not split {size} ways")
    h, g, f = H // size, G // size, F // size
    return ShardLayout(h, g, f, slice(rank * h * D, (rank + 1) * h * D),
                       slice(rank * g * D, (rank + 1) * g * D), slice(rank * f, (rank + 1) * f))


class LlamaEngine:
    """A decoder of ``config``'s shape on ``weights`` (Hugging Face checkpoint names).

    ``batch`` independent sequences share the weights and hold a KV cache each.
    """

    def __init__(self, config: DecoderConfig, weights: dict, device="cuda", batch: int = 1,
                 kv_len_hint: int | None = None, tp_rank: int = 0, tp_size: int = 1, tp_group=None,
                 release=None):
        c = config
        # what the fused kernels do not compute is refused, not skipped
        if getattr(c, "attention_bias", False) or getattr(c, "mlp_bias", False):
            raise ValueError("LlamaEngine: projections with biases run on the recorded graph (CausalLM), "
                             "not on the fused engine")
        if getattr(c, "hidden_act", "silu") != "silu":
            raise ValueError(f"LlamaEngine: the gated MLP's activation is silu, not {c.hidden_act!r}")
        if c.rope_theta is None or c.rope_width != c.head_dim:
            raise ValueError("LlamaEngine: RoPE over the whole head (rope_width == head_dim) is the only form")
        if not torch.cuda.is_available():
            raise RuntimeError("LlamaEngine needs a CUDA device: there is no CPU path")
        self.c, self.device, self.batch = config, torch.device(device), batch
        E, V, L = c.hidden_size, c.vocab_size, c.num_hidden_layers
        D, S = c.head_dim, c.max_seq_len
        # Tensor parallelism: this rank holds heads [rank*H/t, ...) of q/k/v and o_proj's
        # matching columns, rows [rank*F/t, ...) of gate/up and down_proj's matching
        # columns; o_proj and down_proj produce partial sums that one all-reduce completes.
        self.tp_rank, self.tp_size, self.tp_group = tp_rank, tp_size, tp_group
        layout = shard_layout(c, tp_rank, tp_size)
        H, G, F = layout.heads, layout.kv_heads, layout.ffn
        self.H, self.G, self.F = H, G, F
        self.kv_len_hint = kv_len_hint or S
        # which launches carry an L2 prefetch hint (bit 0: QKV -> o_proj weights, bit 1:
        # attention -> gate/up, bit 2: gate/up -> down, bit 3: down -> next layer's QKV)
        self.prefetch_hints = int(os.environ.get("IRON_PREFETCH_HINTS", "0"))
        # One sequence on one GPU can decode in one persistent kernel per step
        # (IRON_DECODE_STEP=1); batches and tensor-parallel shards always take the separate
        # launches.  The two paths are compared by the tests.
        self.fused_step = (batch == 1 and tp_size == 1 and D in (64, 128) and L <= 64
                           and E % 32 == 0 and F % 32 == 0 and V % 8 == 0 and max(E, F, H * D) <= 8192
                           and os.environ.get("IRON_DECODE_STEP", "0") == "1")
        self._fused_step_wanted = self.fused_step
        # One sequence on one GPU runs a layer's attention, o_proj and residual add as one
        # launch (a cluster per KV group) where a CTA's rows of Wo fit an SM's shared memory;
        # IRON_ATTN_OPROJ=0 keeps the two separate kernels.
        self.attn_oproj = (batch == 1 and tp_size == 1 and os.environ.get("IRON_ATTN_OPROJ", "1") != "0"
                           and K.attn_oproj_supported(E, H, G, D) > 0)

        # ---- plan the arena: residents first, then the decode step's transients ----
        plan = ArenaPlan()
        sizes: dict[str, int] = {}

        def res(name, shape, dtype_bytes=2):
            sizes[name] = int(np.prod(shape)) * dtype_bytes
            return name

        res("embed", (V, E)); res("norm", (E,)); res("angles", (S, D))
        if not c.tie_word_embeddings:
            res("head", (V, E))
        for i in range(L):
            res(f"l{i}.ln1", (E,)); res(f"l{i}.wqkv", ((H + 2 * G) * D, E))
            res(f"l{i}.wo", (E, H * D)); res(f"l{i}.ln2", (E,))
            res(f"l{i}.wg", (F, E)); res(f"l{i}.wu", (F, E)); res(f"l{i}.wd", (E, F))
            res(f"l{i}.k", (batch, S, G, D)); res(f"l{i}.v", (batch, S, G, D))
        res("values", (16,), 4); res("drawn", (batch, S), 4)
        # used by every version (decode step, prompt chunk, batched step): resident too
        res("x0", (batch, E)); res("logits", (batch, V)); res("b.values", (2, max(batch, 8)), 4)
        residents = {n: n for n in sizes}
        trans = {"x1": (batch, E), "q": (batch, H * D), "att": (batch, H * D),
                 "act": (batch, F), "part": (batch, E)}
        for n, shape in trans.items():
            sizes[n] = int(np.prod(shape)) * 2
        # the decode step touches every transient in each layer: all live together
        spans = plan.place_version([list(trans)], sizes, residents)
        # The prompt-chunk version: the same residents at the same offsets, its own
        # transients (one batch entry at a time) placed by live range, so the attention
        # buffers share bytes with the gated MLP's.
        C = min(c.prefill_chunk, S)
        self.chunk = C
        QKV = (H + 2 * G) * D
        ptrans = {"p.ids": (C, 2), "p.x": (C, E), "p.h": (C, E), "p.y": (C, E), "p.qkv": (C, QKV),
                  "p.att": (C, H * D), "p.gate": (C, F), "p.up": (C, F), "p.part": (C, E)}
        psizes = dict(sizes)
        for n in trans:
            psizes.pop(n)
        for n, shape in ptrans.items():
            psizes[n] = int(np.prod(shape)) * 2
        psteps = [["p.ids", "p.x"], ["p.x", "p.h"], ["p.h", "p.qkv"], ["p.qkv", "p.att"],
                  ["p.att", "p.x", "p.y"], ["p.y", "p.h"], ["p.h", "p.gate"], ["p.h", "p.up"],
                  ["p.gate", "p.up"], ["p.gate", "p.y", "p.x"]]
        # within a layer p.x and p.y stay live across the loop: mark them touched last too
        psteps.append(["p.x", "p.y", "p.part"])
        psteps[4].append("p.part")
        spans.update(plan.place_version(psteps, psizes, {n: n for n in residents}))
        # The batched decode step (one row per sequence): the prompt chunk's recipe on
        # `batch` rows, with a dense q for the packed attention.
        if batch > 1:
            btrans = {"b.x": (batch, E), "b.h": (batch, E), "b.y": (batch, E), "b.qkv": (batch, QKV),
                      "b.q": (batch, H * D), "b.att": (batch, H * D), "b.gate": (batch, F), "b.up": (batch, F),
                      "b.part": (batch, E)}
            bsizes = {n: sizes[n] for n in residents}
            for n, shape in btrans.items():
                bsizes[n] = int(np.prod(shape)) * 2
            bsteps = [["b.x"], ["b.x", "b.h"], ["b.h", "b.qkv"], ["b.qkv", "b.q"], ["b.q", "b.att"],
                      ["b.att", "b.x", "b.y", "b.part"], ["b.y", "b.h"], ["b.h", "b.gate"], ["b.h", "b.up"],
                      ["b.gate", "b.up"], ["b.gate", "b.y", "b.x", "b.part"], ["b.x", "b.y"]]
            spans.update(plan.place_version(bsteps, bsizes, {n: n for n in residents}))
        self.plan = plan
        self.arena = torch.empty(plan.size, dtype=torch.uint8, device=self.device)
        self.arena.zero_()

        def view(name, shape, dtype=BF16):
            s = spans[name]
            return self.arena[s.offset : s.offset + s.size].view(dtype).view(*shape)

        self.embed, self.norm, self.angles = view("embed", (V, E)), view("norm", (E,)), view("angles", (S, D))
        self.head = self.embed if c.tie_word_embeddings else view("head", (V, E))
        self.layers = []
        for i in range(L):
            self.layers.append(dict(
                ln1=view(f"l{i}.ln1", (E,)), wqkv=view(f"l{i}.wqkv", ((H + 2 * G) * D, E)),
                wo=view(f"l{i}.wo", (E, H * D)), ln2=view(f"l{i}.ln2", (E,)),
                wg=view(f"l{i}.wg", (F, E)), wu=view(f"l{i}.wu", (F, E)), wd=view(f"l{i}.wd", (E, F)),
                k=view(f"l{i}.k", (batch, S, G, D)), v=view(f"l{i}.v", (batch, S, G, D))))
        self.values = view("values", (16,), torch.int32)   # [token, position, ...]
        self.drawn = view("drawn", (batch, S), torch.int32)
        self.x0, self.x1 = view("x0", (batch, E)), view("x1", (batch, E))
        self.q, self.att = view("q", (batch, H, D)), view("att", (batch, H, D))
        self.act, self.logits_buf = view("act", (batch, F)), view("logits", (batch, V))
        self.part, self.p_part = view("part", (batch, E)), view("p.part", (C, E))
        self.p_ids = view("p.ids", (C,), torch.int32)
        self.p_x, self.p_h, self.p_y = view("p.x", (C, E)), view("p.h", (C, E)), view("p.y", (C, E))
        self.p_qkv, self.p_att = view("p.qkv", (C, QKV)), view("p.att", (C, H * D))
        self.p_gate, self.p_up = view("p.gate", (C, F)), view("p.up", (C, F))
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        bv = view("b.values", (2, max(batch, 8)), torch.int32)
        self.b_tokens, self.b_pos = bv[0, :batch], bv[1, :batch]   # per-sequence (token, position)
        if batch > 1:
            self.b_x, self.b_h, self.b_y = view("b.x", (batch, E)), view("b.h", (batch, E)), view("b.y", (batch, E))
            self.b_qkv, self.b_q = view("b.qkv", (batch, QKV)), view("b.q", (batch, H, D))
            self.b_att = view("b.att", (batch, H, D))
            self.b_gate, self.b_up = view("b.gate", (batch, F)), view("b.up", (batch, F))
            self.b_part = view("b.part", (batch, E))
        # A batched step's projections can take their neighbours into the launch where the
        # weight-streaming kernel covers the shapes: RoPE and the cache write after q/k/v
        # (IRON_BATCH_FOLD=rope), the RMSNorms before q/k/v and gate/up (=norm), both (=1).  Off unless
        # asked for: measured, the step is as long either way (the norm's latency moves into the
        # projection), and 128-wide heads at small batches lose a few percent.
        fold = os.environ.get("IRON_BATCH_FOLD", "0")
        foldable = (1 < batch <= 64 and tp_size == 1 and E % 64 == 0 and E <= 8192 and D in (64, 128)
                    and (H * D) % 128 == 0 and (G * D) % 128 == 0
                    and os.environ.get("IRON_GEMM_SKINNY", "1") != "0"
                    and min(K.gemm_rows_parts(batch, E, H * D), K.gemm_rows_parts(batch, E, F),
                            K.gemm_rows_parts(batch, QKV, E), K.gemm_rows_parts(batch, F, E, True)) > 0)
        self.fold_norm = foldable and fold in ("1", "norm")
        self.fold_rope = foldable and fold in ("1", "rope")
        if self.fold_norm:
            self.b_sq_x, self.b_sq_y = K.rowsq_buffer(self.device), K.rowsq_buffer(self.device)
            self.b_parts_o, self.b_parts_d = K.gemm_rows_parts(batch, E, H * D), K.gemm_rows_parts(batch, E, F)

        self._load(weights, release)
        self._peer_exchange_setup()
        self.nsplit = K.mha_decode_splits(batch, G, self.kv_len_hint)
        self.argmax_ws = K.argmax_workspace(self.device)
        # Under tensor parallelism the output head is split by vocabulary rows as well (one
        # sequence, greedy draw): a rank multiplies its V / t rows, reduces them to one 64-bit
        # (value, index) key, the keys are gathered and the largest names the token -- the head
        # is most of a rank's bytes once the layers are split.  IRON_TP_SHARD_HEAD=0 keeps every
        # rank on the whole head.
        self.head_sharded = (tp_size > 1 and batch == 1 and V % (8 * tp_size) == 0
                             and os.environ.get("IRON_TP_SHARD_HEAD", "1") != "0")
        if self.head_sharded:
            self.head_rows = slice(tp_rank * (V // tp_size), (tp_rank + 1) * (V // tp_size))
            self.head_key = torch.zeros(1, dtype=torch.int64, device=self.device)
            self.head_keys = torch.zeros(tp_size, dtype=torch.int64, device=self.device)
        self.ab_scratch = K.attn_oproj_scratch(E, G, self.device) if self.attn_oproj else None
        self.draws = None   # (batch, S, 4) int32 draw rows once a sampler is set
        self.fuse_rope = os.environ.get("IRON_PREFILL_FUSED_ROPE", "1") != "0"
        self._chunk_launches: int | None = None
        self.step_ws = K.decode_step_workspace(E, H, G, D, self.device)
        self.step_table = K.decode_step_table(
            [dict(l, k=l["k"][0], v=l["v"][0]) for l in self.layers], self.device)
        self.step_maps = None
        if self.fused_step:
            self.step_maps = K.decode_step_maps(self.step_table, E=E, F=F, H=H, G=G, D=D, V=V, head=self.head)
        self._graph: torch.cuda.CUDAGraph | None = None
        # Per-call values are staged in a ring of pinned slots: a slot is rewritten only
        # after the copy that read it has completed, so calls can be queued without a
        # host synchronisation between them.
        self._ring = [torch.zeros(16, dtype=torch.int32).pin_memory() for _ in range(32)]
        self._ring_done: list[torch.cuda.Event | None] = [None] * len(self._ring)
        self._ring_at = 0
        self._h_token = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._h_in = torch.zeros(16, dtype=torch.int32).pin_memory()   # the host loop's per-call values
        self._h_b = torch.zeros((2, batch), dtype=torch.int32).pin_memory()
        self._h_b_np = self._h_b.numpy()
        self._h_b_out = torch.zeros(batch, dtype=torch.int32).pin_memory()
        self._h_b_out_np = self._h_b_out.numpy()
        self._h_in_np = self._h_in.numpy()
        self._graph_host: torch.cuda.CUDAGraph | None = None
        self._h_ids = torch.zeros(self.chunk, dtype=torch.int32).pin_memory()
        self._h_ids_done: torch.cuda.Event | None = None
        self._h_status = torch.zeros(1, dtype=torch.int32).pin_memory()
        # the position the next replayed step runs at (the largest over a batch), mirrored on
        # the host so that a replay past the end of the caches is refused before any launch
        self._next_position = 0
        self._last_call_sharded = False

    # ------------------------------------------------------------------ weights
    @classmethod
    def from_checkpoint(cls, path, *, random_weights: int | None = None, max_seq_len: int | None = None,
                        config_class=None, **kwargs) -> "LlamaEngine":
        """The engine on a checkpoint directory (``config.json`` beside ``model.safetensors`` or
        its shard index), as ``Model.from_checkpoint`` loads one (iron/lm/model.py:125-234).

        ``random_weights`` draws weights at that seed in the checkpoint's shapes, reading only
        its header; ``max_seq_len`` lowers the context served and refuses to raise it.
        """
        from pathlib import Path

        from .checkpoint import Checkpoint, weights_file

        if config_class is None:
            from ..applications.llama.model import LlamaConfig as config_class
        path = Path(path)
        directory = path if path.is_dir() else path.parent
        config = config_class.from_checkpoint(directory)
        if max_seq_len is not None:
            if max_seq_len > config.max_seq_len:
                raise ValueError(f"max_seq_len {max_seq_len} is past the checkpoint's {config.max_seq_len}")
            config = dataclasses.replace(config, max_seq_len=max_seq_len)
        checkpoint = Checkpoint(weights_file(directory) if path.is_dir() else path)
        weights = checkpoint.named("read" if random_weights is None else "random", seed=random_weights or 0)
        engine = cls(config, weights, release=checkpoint.release if random_weights is None else None, **kwargs)
        engine.checkpoint = checkpoint
        return engine

    def _load(self, w: dict, release=None) -> None:
        """Every weight into its arena slice through the pinned staging ring; ``release`` drops
        a mapped checkpoint's pages behind the copies."""
        from .checkpoint import Uploader

        c = self.c
        up = Uploader(self.device, release=release)

        def put(a, out):
            if isinstance(a, torch.Tensor):
                _as_device_bf16(a, out)
            else:
                up.put(a, out)

        put(w["model.embed_tokens.weight"], self.embed)
        put(w["model.norm.weight"], self.norm)
        if not c.tie_word_embeddings:
            put(w["lm_head.weight"], self.head)
        put(c.angles().astype(np.float32), self.angles)
        lay = shard_layout(c, self.tp_rank, self.tp_size)
        Q, KV = lay.heads * c.head_dim, lay.kv_heads * c.head_dim
        for i, l in enumerate(self.layers):
            p = f"model.layers.{i}"
            put(w[f"{p}.input_layernorm.weight"], l["ln1"])
            put(w[f"{p}.self_attn.q_proj.weight"][lay.q_rows], l["wqkv"][:Q])
            put(w[f"{p}.self_attn.k_proj.weight"][lay.kv_rows], l["wqkv"][Q : Q + KV])
            put(w[f"{p}.self_attn.v_proj.weight"][lay.kv_rows], l["wqkv"][Q + KV :])
            put(w[f"{p}.self_attn.o_proj.weight"][:, lay.q_rows], l["wo"])
            put(w[f"{p}.post_attention_layernorm.weight"], l["ln2"])
            put(w[f"{p}.mlp.gate_proj.weight"][lay.ffn_rows], l["wg"])
            put(w[f"{p}.mlp.up_proj.weight"][lay.ffn_rows], l["wu"])
            put(w[f"{p}.mlp.down_proj.weight"][:, lay.ffn_rows], l["wd"])
        up.finish()
        self.uploaded_bytes = up.bytes

    def _all_reduce(self, t: torch.Tensor) -> None:
        """Sum ``t`` over the tensor-parallel ranks in place (NCCL; stream-ordered, capturable)."""
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.tp_group)

    def _peer_exchange_setup(self) -> None:
        """Map one small exchange buffer per rank into every rank's address space
        (torch symmetric memory over NVLink peer access), for the decode step's fused
        all-reduce + residual add.  IRON_TP_PEER=0 keeps the NCCL all-reduce."""
        self.peer_buffers = None
        self.tp_fused = False
        if self.tp_size == 1 or os.environ.get("IRON_TP_PEER", "1") == "0":
            return
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        # plain peer loads and stores only: no multicast object is bound to the buffer
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        # one slot holds a decode step's rows: the vector of one sequence, or a few sequences'
        # (one CTA moves a slot: larger batches take NCCL)
        self.peer_slot_elems = self.c.hidden_size * min(self.batch, 8)
        nbytes = K.tp_buffer_bytes(self.tp_size, self.peer_slot_elems)
        group = self.tp_group if self.tp_group is not None else dist.group.WORLD
        self._peer_mem = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        self._peer_mem.zero_()
        self._peer_handle = symm.rendezvous(self._peer_mem, group)
        ptrs = [int(q) for q in self._peer_handle.buffer_ptrs]
        self.peer_buffers = (ctypes.c_void_p * self.tp_size)(*ptrs)
        self.peer_seq = torch.zeros(1, dtype=torch.int32, device=self.device)
        # a one-sequence step folds each exchange into the GEMVs on either side of it
        # (IRON_TP_FUSED=0 keeps the all-reduce kernel of its own)
        self.tp_fused = self.batch == 1 and os.environ.get("IRON_TP_FUSED", "1") != "0"
        self.peer_state = torch.zeros(8, dtype=torch.int32, device=self.device)
        # an exchange that is a launch of its own: many CTAs over tagged words (IRON_TP_TAGGED=0: the one-CTA
        # kernel with a fence and flags)
        self.tp_tagged = os.environ.get("IRON_TP_TAGGED", "1") != "0"
        torch.cuda.synchronize()
        dist.barrier(group=group)   # every rank's buffer is zeroed before anyone stores into it

    @property
    def exchange_path(self) -> str:
        """How a decode step's partial sums meet under tensor parallelism."""
        if self.tp_size == 1:
            return "none"
        if self.tp_fused:
            return ("peer memory, no launch of its own (the producing GEMV stores its rows into every rank's slot, "
                    "the consuming GEMV waits, bounded, and sums in rank order)")
        if self.peer_buffers is not None and self.c.hidden_size * self.batch <= self.peer_slot_elems:
            if self.tp_tagged:
                return ("peer-memory kernel (tagged 32-bit words to every rank's slot, bounded re-reads, "
                        "rank-ordered f32 sum; no fence, no flag)")
            return "peer-memory kernel (stores to every rank's slot, bounded flag wait, rank-ordered f32 sum)"
        return "nccl all-reduce"

    def _reduce_add(self, part: torch.Tensor, residual: torch.Tensor, out: torch.Tensor) -> None:
        """out = residual + (sum of ``part`` over the ranks): one kernel over peer memory
        for a decode step's vector, NCCL and an add otherwise."""
        if (self.peer_buffers is not None and part.numel() <= self.peer_slot_elems and part.is_contiguous()
                and self.tp_tagged):
            K.tp_allreduce_tagged(part, out, residual=residual, peer_buffers=self.peer_buffers,
                                  slot_elems=self.peer_slot_elems, rank=self.tp_rank, world=self.tp_size,
                                  state=self.peer_state, status=self.status)
        elif self.peer_buffers is not None and part.numel() <= self.peer_slot_elems and part.is_contiguous():
            K.tp_allreduce(part, out, residual=residual, peer_buffers=self.peer_buffers,
                           slot_elems=self.peer_slot_elems, rank=self.tp_rank, world=self.tp_size,
                           seq=self.peer_seq, status=self.status)
        else:
            self._all_reduce(part)
            K.elementwise("add", residual, part, out)

    # ------------------------------------------------------------------ decode step
    @property
    def launches_per_step(self) -> int:
        """This package's kernels in one decode step: one persistent kernel, or gather, four or
        five per layer, head, draw; a batched step takes gather, eight per layer, norm, head, draw.
        Tensor parallelism adds two exchange kernels a layer unless the exchanges ride on the GEMVs,
        and a key and a pick in place of the draw when the head is split."""
        if self.batch > 1:
            per_layer = 8 - (1 if self.fold_rope else 0) - (2 if self.fold_norm else 0)
            return 1 + per_layer * self.c.num_hidden_layers + (1 if self.fold_norm else 0) + 3
        if self.fused_step:
            return 1
        per_layer = 4 if self.attn_oproj else 5
        if self.tp_size > 1 and self.peer_buffers is not None and not self.tp_fused:
            per_layer += 2
        return 1 + per_layer * self.c.num_hidden_layers + (3 if self.head_sharded else 2)

    @property
    def weight_bytes_per_token(self) -> int:
        """Bytes of weights one decode step streams (the HBM roofline's numerator)."""
        c = self.c
        E, F, V = c.hidden_size, c.intermediate_size, c.vocab_size
        Q, KV = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
        layer = ((Q + 2 * KV) * E + E * Q + 3 * F * E) * 2
        head = V * E * 2 // (self.tp_size if getattr(self, "head_sharded", False) else 1)
        return c.num_hidden_layers * layer // self.tp_size + head

    def _batch_launches(self) -> None:
        """Launch one decode step of every sequence of the batch: row b reads
        (b_tokens[b], b_pos[b]) and leaves (drawn token, position + 1) there.  The
        projections are skinny GEMMs on the tensor cores (the weights cross HBM once for the
        whole batch); RoPE, the cache writes, the attention and the draw are per sequence."""
        c = self.c
        H, G, D, E, V = self.H, self.G, c.head_dim, c.hidden_size, c.vocab_size
        n = self.batch
        x, h, y = self.b_x, self.b_h, self.b_y
        tp, part = self.tp_size > 1, self.b_part
        K.copy_rows(self.embed, x, ids=self.b_tokens, nrows=n, row_bytes=E * 2, src_rows=V)
        fold_norm, fold_rope = self.fold_norm, self.fold_rope
        for i, l in enumerate(self.layers):
            # the layer's input is normalised inside the q/k/v projection when the projection before it left
            # the rows' sums of squares (the embedding rows come with none: the first norm is a launch)
            normed = dict(norm_weight=l["ln1"], rowsq_in=self.b_sq_x, rowsq_parts=self.b_parts_d,
                          eps=c.eps) if fold_norm and i > 0 else None
            if normed is None:
                K.rms_norm(x, l["ln1"], h, eps=c.eps)
            if fold_rope:
                K.gemm_rows_qkv_rope(h if normed is None else x, l["wqkv"], self.angles, self.b_q, l["k"], l["v"],
                                     self.b_pos, H=H, G=G, D=D, status=self.status, **(normed or {}))
            else:
                if normed is None:
                    K.gemm(h, l["wqkv"], self.b_qkv, b_col_maj=True, status=self.status)
                else:
                    K.gemm_rows(x, l["wqkv"], self.b_qkv, status=self.status, **normed)
                K.rope_kv_scatter(self.b_qkv, self.angles, self.b_q, l["k"], l["v"], self.b_pos, H=H, G=G, D=D)
            K.mha_decode(self.b_q, l["k"], l["v"], self.b_att, d_kv_valid=self.b_pos, per_batch=True,
                         kv_valid_add=1, window=c.window, scale=c.attention_scale)
            if tp:   # row-parallel: this rank's partial sums meet the others', then the residual
                K.gemm(self.b_att.view(n, H * D), l["wo"], part, b_col_maj=True, status=self.status)
                self._reduce_add(part, x, y)
            elif fold_norm:
                K.gemm_rows(self.b_att.view(n, H * D), l["wo"], y, residual=x, rowsq_out=self.b_sq_y, status=self.status)
            else:
                K.gemm(self.b_att.view(n, H * D), l["wo"], y, b_col_maj=True, residual=x, status=self.status)
            if fold_norm:
                K.gemm_rows(y, l["wg"], self.b_gate, W2=l["wu"], norm_weight=l["ln2"], rowsq_in=self.b_sq_y,
                            rowsq_parts=self.b_parts_o, eps=c.eps, status=self.status)
            else:
                K.rms_norm(y, l["ln2"], h, eps=c.eps)
                K.gemm_swiglu(h, l["wg"], l["wu"], self.b_gate, status=self.status)
            if tp:
                K.gemm(self.b_gate, l["wd"], part, b_col_maj=True, status=self.status)
                self._reduce_add(part, y, x)
            elif fold_norm:
                K.gemm_rows(self.b_gate, l["wd"], x, residual=y, rowsq_out=self.b_sq_x, status=self.status)
            else:
                K.gemm(self.b_gate, l["wd"], x, b_col_maj=True, residual=y, status=self.status)
        K.rms_norm(x, self.norm, h, eps=c.eps)
        K.gemm(h, self.head, self.logits_buf, b_col_maj=True, status=self.status)
        if self.draws is None:
            K.argmax_rows(self.logits_buf, self.b_tokens, self.b_pos, self.drawn)
        else:
            K.sample_rows(self.logits_buf, self.draws, self.b_tokens, self.b_pos, self.drawn)

    def _decode_launches(self) -> None:
        """Launch one decode step on the current stream, reading (token, position) from
        the device values buffer and leaving (drawn token, position + 1) there."""
        if self.batch > 1:
            return self._batch_launches()
        c = self.c
        H, G, D = self.H, self.G, c.head_dim
        d_token, d_pos = self.values[0:1], self.values[1:2]
        if self.fused_step:
            K.decode_step(self.step_table, self.step_maps, L=c.num_hidden_layers, E=c.hidden_size, F=self.F, H=H, G=G,
                          D=D, V=c.vocab_size, S=c.max_seq_len, embed=self.embed, head=self.head,
                          final_norm=self.norm, angles=self.angles, eps=c.eps,
                          scale=c.attention_scale or 1.0 / math.sqrt(D), window=c.window,
                          values=self.values, drawn=self.drawn[0],
                          xa=self.x0[0], xb=self.x1[0], act=self.act[0],
                          logits=self.logits_buf[0], workspace=self.step_ws)
            return
        E2 = c.hidden_size * 2
        x, y, part = self.x0[0], self.x1[0], self.part[0]
        tp = self.tp_size > 1
        K.copy_rows(self.embed, x, ids=d_token, nrows=1, row_bytes=E2, src_rows=c.vocab_size)
        hints = 0 if tp else self.prefetch_hints
        if tp and self.tp_fused:
            # Each exchange rides on its neighbours: the row-parallel GEMV pushes its rows to every
            # rank, the next GEMV pulls the ranks' sum plus the residual as its input.
            link = dict(peer_buffers=self.peer_buffers, slot_elems=self.peer_slot_elems, rank=self.tp_rank,
                        world=self.tp_size, state=self.peer_state, status=self.status)
            pushed = False
            for l in self.layers:
                if pushed:
                    K.tp_pull_next(**link, residual=y, x_out=x)
                K.decode_qkv_rope(l["wqkv"], x, self.angles, l["k"][0], l["v"][0], self.q[0],
                                  H=H, G=G, D=D, d_position=d_pos, norm_weight=l["ln1"], eps=c.eps)
                K.mha_decode(self.q, l["k"], l["v"], self.att, d_kv_valid=d_pos, kv_valid_add=1,
                             window=c.window, scale=c.attention_scale, nsplit=self.nsplit, stable_prefix=True)
                K.tp_push_next(**link)
                K.gemv(l["wo"], self.att[0].view(-1), part)
                K.tp_pull_next(**link, residual=x, x_out=y)
                K.gemv_swiglu(l["wg"], l["wu"], y, self.act[0], norm_weight=l["ln2"], eps=c.eps)
                K.tp_push_next(**link)
                K.gemv(l["wd"], self.act[0], part)
                pushed = True
            K.tp_pull_next(**link, residual=y, x_out=x)   # consumed by the head projection below
        for i, l in enumerate(self.layers if not (tp and self.tp_fused) else ()):
            if self.attn_oproj and not hints:
                K.decode_qkv_rope(l["wqkv"], x, self.angles, l["k"][0], l["v"][0], self.q[0],
                                  H=H, G=G, D=D, d_position=d_pos, norm_weight=l["ln1"], eps=c.eps)
                K.decode_attn_oproj(self.q[0], l["wo"], x, l["k"][0], l["v"][0], y, G=G, scratch=self.ab_scratch,
                                    d_position=d_pos, window=c.window, scale=c.attention_scale, status=self.status)
                K.gemv_swiglu(l["wg"], l["wu"], y, self.act[0], norm_weight=l["ln2"], eps=c.eps)
                K.gemv(l["wd"], self.act[0], x, residual=y)
                continue
            # Each launch is told which weights follow it, so the latency-bound kernels keep
            # HBM busy pulling the next projections into L2.
            if hints & 1:
                K.prefetch_hint(l["wo"])
            K.decode_qkv_rope(l["wqkv"], x, self.angles, l["k"][0], l["v"][0], self.q[0],
                              H=H, G=G, D=D, d_position=d_pos, norm_weight=l["ln1"], eps=c.eps)
            if hints & 2:
                K.prefetch_hint(l["wg"], l["wu"])
            K.mha_decode(self.q, l["k"], l["v"], self.att, d_kv_valid=d_pos, kv_valid_add=1,
                         window=c.window, scale=c.attention_scale, nsplit=self.nsplit,
                         stable_prefix=True)
            if hints:
                K.gemv(l["wo"], self.att[0].view(-1), y, residual=x)
                if hints & 4:
                    K.prefetch_hint(l["wd"])
                K.gemv_swiglu(l["wg"], l["wu"], y, self.act[0], norm_weight=l["ln2"], eps=c.eps)
                if hints & 8:
                    K.prefetch_hint(self.layers[i + 1]["wqkv"] if i + 1 < len(self.layers) else self.head[:4096])
                K.gemv(l["wd"], self.act[0], x, residual=y)
                continue
            if tp:   # partial sums meet in an all-reduce before each residual add
                K.gemv(l["wo"], self.att[0].view(-1), part)
                self._reduce_add(part, x, y)
                K.gemv_swiglu(l["wg"], l["wu"], y, self.act[0], norm_weight=l["ln2"], eps=c.eps)
                K.gemv(l["wd"], self.act[0], part)
                self._reduce_add(part, y, x)
                continue
            K.gemv(l["wo"], self.att[0].view(-1), y, residual=x)
            K.gemv_swiglu(l["wg"], l["wu"], y, self.act[0], norm_weight=l["ln2"], eps=c.eps)
            K.gemv(l["wd"], self.act[0], x, residual=y)
        if self.head_sharded and self.draws is None:
            import torch.distributed as dist

            rows = self.head_rows
            K.gemv(self.head[rows], x, self.logits_buf[0, rows], norm_weight=self.norm, eps=c.eps)
            K.argmax_key(self.logits_buf[0, rows], self.head_key, self.argmax_ws, index_offset=rows.start)
            dist.all_gather_into_tensor(self.head_keys, self.head_key, group=self.tp_group)
            K.argmax_pick(self.head_keys, self.drawn[0], d_out_index=d_pos, carry_token=d_token, carry_position=d_pos)
            return
        K.gemv(self.head, x, self.logits_buf[0], norm_weight=self.norm, eps=c.eps)
        self._draw(0, d_token, d_pos)

    def _draw(self, seq: int, d_token, d_pos) -> None:
        """The draw after a head projection: greedy, or by the draw row of the position when a
        sampler is set; writes drawn[seq][position] and carries (token, position + 1)."""
        if self.draws is None:
            K.argmax(self.logits_buf[seq], self.drawn[seq], self.argmax_ws, d_out_index=d_pos,
                     carry_token=d_token, carry_position=d_pos)
        else:
            K.sample_rows(self.logits_buf[seq], self.draws[seq], d_token, d_pos, self.drawn[seq : seq + 1])

    def set_sampler(self, sampler, start: int = 0, count: int | None = None, seq: int | None = None) -> None:
        """Draw with ``sampler`` (an ``iron_b200.lm.generation.Sampler``) at positions
        ``start .. start + count`` of sequence ``seq`` (every sequence when None, each taking
        its own uniforms in turn): the device gets the uniforms the sampler's host draws would
        use, one draw row per position (iron/lm/causal.py:340-347 keeps them in its ``draws``
        state).  ``sampler`` None returns to the greedy draw.  Captured graphs are dropped."""
        self._graph = None
        self._graph_host = None
        if sampler is None:
            self.draws = None
            self.fused_step = self._fused_step_wanted
            return
        S = self.c.max_seq_len
        count = S - start if count is None else count
        if start < 0 or start + count > S:
            raise IndexError(f"positions {start}..{start + count} leave the {S}-row caches")
        if self.draws is None:
            self.draws = torch.zeros((self.batch, S, 4), dtype=torch.int32, device=self.device)
        self.fused_step = False   # the one-kernel step draws greedily
        for b in (range(self.batch) if seq is None else (seq,)):
            rows = torch.from_numpy(sampler.rows(count, K.sample_k_max()))
            self.draws[b, start : start + count].copy_(rows)

    # ------------------------------------------------------------------ prompt chunk
    @property
    def launches_per_chunk(self) -> int:
        """Kernels the last prompt chunk launched (a full chunk's count before any ran): gather,
        per layer two norms, the q/k/v projection (with RoPE and the cache write in its output
        stage, or followed by the RoPE kernel), attention, o_proj, the gated gate/up GEMM and
        down_proj, then row pick, head and draw; tensor-parallel chunks add two adds a layer."""
        if self._chunk_launches is not None:
            return self._chunk_launches
        per_layer = 7 + (0 if self.fuse_rope else 1) + (2 if self.tp_size > 1 else 0)
        return 1 + per_layer * self.c.num_hidden_layers + 3

    def prefill_chunk(self, tokens, start: int, seq: int = 0) -> None:
        """Run one prompt chunk (at most ``prefill_chunk`` tokens) at positions ``start...``.

        What the reference's prompt-chunk version records (iron/lm/causal.py:289-332):
        embedding rows, then per layer RMSNorm, the fused q/k/v projection on the tensor
        cores, RoPE and the bounded cache write, causal attention of the chunk's rows over
        the cache, o_proj with the residual, RMSNorm, gate and up projections, SiLU and
        product, down_proj with the residual; only the last row goes through the head.
        Leaves (drawn token, start + rows) in the per-call values.
        """
        c = self.c
        tokens = np.asarray(tokens).reshape(-1)
        n = len(tokens)
        if not 0 < n <= self.chunk:
            raise ValueError(f"a prompt chunk holds 1 to {self.chunk} tokens, not {n}")
        if start < 0 or start + n > c.max_seq_len:
            raise IndexError(f"positions {start}..{start + n} leave the {c.max_seq_len}-row caches")
        if tokens.min() < 0 or tokens.max() >= c.vocab_size:
            raise IndexError("a token id is outside the vocabulary")
        H, G, D, E, F = self.H, self.G, c.head_dim, c.hidden_size, self.F
        tp = self.tp_size > 1
        part = self.p_part[:n]
        # token ids go through one pinned buffer, reused once the copy that read it has run
        if self._h_ids_done is not None:
            self._h_ids_done.synchronize()
        self._h_ids[:n].copy_(torch.from_numpy(tokens.astype(np.int32)))
        self.p_ids[:n].copy_(self._h_ids[:n], non_blocking=True)
        self._h_ids_done = torch.cuda.Event()
        self._h_ids_done.record()
        x, h, y = self.p_x[:n], self.p_h[:n], self.p_y[:n]
        qkv, att, gate, up = self.p_qkv[:n], self.p_att[:n], self.p_gate[:n], self.p_up[:n]
        K.copy_rows(self.embed, x, ids=self.p_ids, nrows=n, row_bytes=E * 2, src_rows=c.vocab_size)
        launches = 4 + (7 + (2 if tp else 0)) * len(self.layers)
        for l in self.layers:
            K.rms_norm(x, l["ln1"], h, eps=c.eps)
            # one launch where the CTA-pair GEMM takes the shape (RoPE and the cache write in its
            # output stage), the projection and the RoPE kernel otherwise
            if not (self.fuse_rope and K.gemm_qkv_rope(h, l["wqkv"], qkv, self.angles, l["k"][seq], l["v"][seq],
                                                       H=H, G=G, D=D, start=start, status=self.status)):
                launches += 1
                K.gemm(h, l["wqkv"], qkv, b_col_maj=True, status=self.status)
                K.rope_kv_write(qkv, self.angles, l["k"][seq], l["v"][seq], rows=n, H=H, G=G, D=D, start=start)
            K.mha_prefill(qkv.view(n, H + 2 * G, D)[:, :H], l["k"][seq], l["v"][seq], att.view(n, H, D),
                          q_tokens=n, kv_tokens=start + n, window=c.window, scale=c.attention_scale,
                          q_row_stride=qkv.stride(0))
            if tp:
                K.gemm(att, l["wo"], part, b_col_maj=True, status=self.status)
                self._all_reduce(part)
                K.elementwise("add", x, part, y)
            else:
                K.gemm(att, l["wo"], y, b_col_maj=True, residual=x, status=self.status)
            K.rms_norm(y, l["ln2"], h, eps=c.eps)
            K.gemm_swiglu(h, l["wg"], l["wu"], gate, status=self.status)
            if tp:
                K.gemm(gate, l["wd"], part, b_col_maj=True, status=self.status)
                self._all_reduce(part)
                K.elementwise("add", y, part, x)
            else:
                K.gemm(gate, l["wd"], x, b_col_maj=True, residual=y, status=self.status)
        last = self.x0[seq]
        K.copy_rows(x, last, nrows=1, row_bytes=E * 2, src_row0=n - 1)
        K.gemv(self.head, last, self.logits_buf[seq], norm_weight=self.norm, eps=c.eps)
        self.set_call(0, start + n - 1)
        self._draw(seq, self.values[0:1], self.values[1:2])
        self._next_position = start + n
        self._last_call_sharded = False
        self._chunk_launches = launches

    def prefill(self, tokens, start: int = 0, seq: int = 0) -> np.ndarray:
        """Run a prompt of any length in chunks from ``start``; the logits after its last token."""
        tokens = np.asarray(tokens).reshape(-1)
        for s in range(0, len(tokens), self.chunk):
            self.prefill_chunk(tokens[s : s + self.chunk], start + s, seq)
        out = self.logits_buf[seq].float().cpu().numpy()
        if int(self.status.item()) != 0:
            raise RuntimeError("a GEMM pipeline wait gave up (IRON_ERR_TIMEOUT)")
        if int(K.prefill_status(self.device).item()) != 0:
            raise RuntimeError("a prompt-attention pipeline wait gave up (IRON_ERR_TIMEOUT)")
        return out

    def complete(self, prompt, steps: int) -> list[int]:
        """Greedy continuation: prompt in chunks, then ``steps - 1`` device-carried decode steps.

        Returns the ``steps`` tokens drawn (the first comes from the prompt's last row).
        """
        prompt = np.asarray(prompt).reshape(-1)
        n = len(prompt)
        if n + steps > self.c.max_seq_len:
            raise IndexError("the run would pass the end of the caches")
        self.prefill(prompt)
        return self.generate_from_prompt(n, steps)

    def generate_from_prompt(self, n: int, steps: int) -> list[int]:
        """After a prompt of ``n`` tokens has run: the token its last row drew, then ``steps - 1``
        device-carried decode steps."""
        if n + steps > self.c.max_seq_len:
            raise IndexError("the run would pass the end of the caches")
        self.capture()
        self._next_position = n
        self._advance(steps - 1)
        for _ in range(steps - 1):
            self._replay()
        out = self.drawn[0, n - 1 : n - 1 + steps].cpu().tolist()
        self.check()
        return out

    def capture(self) -> None:
        """Capture the decode step as one CUDA graph (idempotent)."""
        if self._graph is not None:
            return
        # the warm-up and the capture run a step at position 0: keep what they overwrite
        saved = self.values.clone()
        saved_next = self._next_position
        saved_logits = self.logits_buf.clone()   # the warm-up step overwrites the last call's logits
        saved_b = (self.b_tokens.clone(), self.b_pos.clone())
        rows = [(l["k"][:, 0].clone(), l["v"][:, 0].clone()) for l in self.layers]
        drawn0 = self.drawn[:, 0].clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # warm up outside capture: lazy module loading
            self.set_call(0, 0)
            self.b_tokens.zero_(); self.b_pos.zero_()
            self._decode_launches()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        self.set_call(0, 0)
        self.b_tokens.zero_(); self.b_pos.zero_()
        with capturing(g):
            self._decode_launches()
        self._graph = g
        self.values.copy_(saved)
        self.b_tokens.copy_(saved_b[0]); self.b_pos.copy_(saved_b[1])
        for l, (k0, v0) in zip(self.layers, rows):
            l["k"][:, 0].copy_(k0); l["v"][:, 0].copy_(v0)
        self.drawn[:, 0].copy_(drawn0)
        self.logits_buf.copy_(saved_logits)
        self._next_position = saved_next
        torch.cuda.synchronize()

    def _capture_host(self) -> None:
        """The step a host loop drives, as one graph: the per-call values in from pinned
        memory, the decode launches, the drawn tokens (and a status word) out to pinned memory,
        so a call is one launch and one stream synchronisation.  Built on first use."""
        self.capture()
        if self._graph_host is not None:
            return
        gh = torch.cuda.CUDAGraph()
        with capturing(gh):
            if self.batch > 1:
                self.b_tokens.copy_(self._h_b[0], non_blocking=True)
                self.b_pos.copy_(self._h_b[1], non_blocking=True)
                self._decode_launches()
                self._h_b_out.copy_(self.b_tokens, non_blocking=True)
                self._h_status.copy_(self.status.view(-1)[:1], non_blocking=True)
            else:
                self.values.copy_(self._h_in, non_blocking=True)
                self._decode_launches()
                self._h_token.copy_(self.values[0:1], non_blocking=True)
                if self.fused_step:
                    self._h_status.copy_(self.step_ws[128:132].view(torch.int32), non_blocking=True)
        self._graph_host = gh

    def set_call(self, token: int, position: int) -> None:
        """Write the per-call values (one small pinned-host to device copy)."""
        if not 0 <= position < self.c.max_seq_len:
            raise IndexError(f"position {position} is outside the {self.c.max_seq_len}-row caches")
        if not 0 <= token < self.c.vocab_size:
            raise IndexError(f"token {token} is outside the {self.c.vocab_size}-row vocabulary")
        i = self._ring_at
        self._ring_at = (i + 1) % len(self._ring)
        if self._ring_done[i] is not None:
            self._ring_done[i].synchronize()
        slot = self._ring[i]
        slot[0], slot[1] = int(token), int(position)
        self.values.copy_(slot, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self._ring_done[i] = done
        self._next_position = int(position)

    def _advance(self, steps: int = 1) -> None:
        """Refuse ``steps`` more device-carried steps when they would leave the caches."""
        if self._next_position + steps > self.c.max_seq_len:
            raise IndexError(f"{steps} more step(s) from position {self._next_position} leave the "
                             f"{self.c.max_seq_len}-row caches")
        self._next_position += steps

    def step(self) -> None:
        """Replay one decode step (stream-ordered; no host synchronisation).  Raises
        ``IndexError`` at the end of the caches, before anything is launched."""
        self.capture()
        self._advance()
        self._replay()

    def _replay(self) -> None:
        """One replay of the captured step; notes whether its logits are split over the ranks."""
        self._graph.replay()
        self._last_call_sharded = self.head_sharded and self.draws is None

    def decode(self, token: int, position: int) -> int:
        """One decode step from the host: token in, drawn token out (both cross PCIe)."""
        if not 0 <= position < self.c.max_seq_len:
            raise IndexError(f"position {position} is outside the {self.c.max_seq_len}-row caches")
        if not 0 <= token < self.c.vocab_size:
            raise IndexError(f"token {token} is outside the {self.c.vocab_size}-row vocabulary")
        self._capture_host()
        self._h_in_np[0], self._h_in_np[1] = token, position
        self._next_position = position + 1
        self._graph_host.replay()
        torch.cuda.current_stream().synchronize()
        if int(self._h_status[0]) != 0:
            raise RuntimeError("the decode step's grid barrier gave up (IRON_ERR_TIMEOUT)")
        return int(self._h_token[0])

    def step_trace(self) -> np.ndarray:
        """CTA 0's timestamps of the last one-kernel decode step, nanoseconds: one row per
        phase (five per layer -- q/k/v, attention, o_proj, gate/up, down_proj -- then the
        head), columns (barrier wait over, staging done, own weight items done)."""
        if not self.fused_step:
            raise RuntimeError("the phase trace belongs to the one-kernel decode step (IRON_DECODE_STEP=1)")
        c = self.c
        off = 256 + 512 * 8 + self.H * 16 * (c.head_dim + 4) * 4
        n = 5 * c.num_hidden_layers + 1
        raw = self.step_ws[off : off + 3 * n * 8].view(torch.int64).cpu().numpy()
        return raw.reshape(n, 3).astype(np.int64)

    def check(self) -> None:
        """Raise if a kernel's bounded wait gave up since the last check (reads two words)."""
        if int(self.status.item()) != 0:
            raise RuntimeError("a GEMM pipeline wait gave up (IRON_ERR_TIMEOUT)")
        if K.decode_step_status(self.step_ws) != 0:
            raise RuntimeError("the decode step's grid barrier gave up (IRON_ERR_TIMEOUT)")
        if int(K.prefill_status(self.device).item()) != 0:
            raise RuntimeError("a prompt-attention pipeline wait gave up (IRON_ERR_TIMEOUT)")

    # ------------------------------------------------------------------ batched decode
    def set_batch(self, tokens, positions) -> None:
        """Write every sequence's (token, position) for the next batched step."""
        tokens = np.asarray(tokens, dtype=np.int64).reshape(-1)
        positions = np.asarray(positions, dtype=np.int64).reshape(-1)
        if len(tokens) != self.batch or len(positions) != self.batch:
            raise ValueError(f"a batched step takes {self.batch} tokens and positions")
        if positions.min() < 0 or positions.max() >= self.c.max_seq_len:
            raise IndexError(f"a position is outside the {self.c.max_seq_len}-row caches")
        if tokens.min() < 0 or tokens.max() >= self.c.vocab_size:
            raise IndexError(f"a token is outside the {self.c.vocab_size}-row vocabulary")
        if getattr(self, "_h_set_batch", None) is None:      # one pinned staging buffer for the engine's life
            self._h_set_batch = torch.empty((2, self.batch), dtype=torch.int32).pin_memory()
        host = self._h_set_batch
        host.copy_(torch.from_numpy(np.stack([tokens, positions]).astype(np.int32)))
        self.b_tokens.copy_(host[0], non_blocking=True)
        self.b_pos.copy_(host[1], non_blocking=True)
        torch.cuda.current_stream().synchronize()   # the staging buffer may be rewritten after this
        self._next_position = int(positions.max())

    def decode_batch(self, tokens, positions) -> list[int]:
        """One decode step of every sequence from the host: tokens in, drawn tokens out, the
        copies being nodes of the step's graph (one launch and one synchronisation a call)."""
        tokens = np.asarray(tokens, dtype=np.int64).reshape(-1)
        positions = np.asarray(positions, dtype=np.int64).reshape(-1)
        if len(tokens) != self.batch or len(positions) != self.batch:
            raise ValueError(f"a batched step takes {self.batch} tokens and positions")
        if positions.min() < 0 or positions.max() >= self.c.max_seq_len:
            raise IndexError(f"a position is outside the {self.c.max_seq_len}-row caches")
        if tokens.min() < 0 or tokens.max() >= self.c.vocab_size:
            raise IndexError(f"a token is outside the {self.c.vocab_size}-row vocabulary")
        if self.batch == 1:
            return [self.decode(int(tokens[0]), int(positions[0]))]
        self._capture_host()
        self._h_b_np[0], self._h_b_np[1] = tokens, positions
        self._next_position = int(positions.max()) + 1
        self._graph_host.replay()
        torch.cuda.current_stream().synchronize()
        if int(self._h_status[0]) != 0:
            raise RuntimeError("a GEMM pipeline wait gave up (IRON_ERR_TIMEOUT)")
        return self._h_b_out_np.tolist()

    def generate_batch(self, tokens, positions, steps: int) -> np.ndarray:
        """``steps`` greedy tokens per sequence, the loop carried on the device; (batch, steps)."""
        positions = np.asarray(positions).reshape(-1)
        if positions.max() + steps > self.c.max_seq_len:
            raise IndexError("the run would pass the end of the caches")
        self.set_batch(tokens, positions)
        self.capture()
        self._advance(steps)
        for _ in range(steps):
            self._graph.replay()
        drawn = self.drawn.cpu().numpy()
        self.check()
        return np.stack([drawn[b, p : p + steps] for b, p in enumerate(positions)])

    def logits_batch(self) -> np.ndarray:
        """The last batched step's logits, (batch, vocab) float32 on the host."""
        return self.logits_buf.float().cpu().numpy()

    def logits(self) -> np.ndarray:
        """The last step's logits as float32 on the host (with a vocabulary-split head, every
        rank's rows are gathered first: a collective, every rank calls it)."""
        if self.head_sharded and self._last_call_sharded:
            import torch.distributed as dist

            rows = self.head_rows
            whole = torch.empty_like(self.logits_buf[0])
            dist.all_gather_into_tensor(whole, self.logits_buf[0, rows].contiguous(), group=self.tp_group)
            return whole.float().cpu().numpy()
        return self.logits_buf[0].float().cpu().numpy()

    def generate(self, token: int, position: int, steps: int) -> list[int]:
        """``steps`` greedy tokens, the loop carried on the device: one replay per token."""
        if position + steps > self.c.max_seq_len:
            raise IndexError("the run would pass the end of the caches")
        self.set_call(token, position)
        self.capture()
        self._advance(steps)
        for _ in range(steps):
            self._replay()
        out = self.drawn[0, position : position + steps].cpu()
        self.check()
        return out.tolist()

    def feed(self, tokens, start: int = 0) -> np.ndarray:
        """Run ``tokens`` one decode step at a time from ``start`` (teacher-forced);
        returns the logits after the last."""
        for i, t in enumerate(tokens):
            self.set_call(int(t), start + i)
            self.step()
        return self.logits()


def batch_shard(sequences: int, rank: int, size: int) -> range:
    """The sequences rank ``rank`` of ``size`` decodes when a batch is split with no collective:
    contiguous runs whose lengths differ by at most one."""
    base, extra = divmod(sequences, size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))
