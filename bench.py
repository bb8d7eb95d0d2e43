"""Headline benchmark: Llama-3.2-1B-architecture greedy decode, tokens per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode token of the random-init 1B-architecture model (bf16 weights
N(0, 0.02), 16 layers, hidden 2048, 32/8 heads of 64, MLP 8192, vocabulary 128256, tied
head) at context 2048 and growing.  `value` is tokens/s with the loop carried on the
device (CUDA-graph replays, per-call values in HBM); `e2e` is the same through the
host-facing call (`LlamaEngine.decode`: token in from pinned host memory, drawn token read
back, every step).  With N > 1 every rank holds a full replica and decodes its own
sequence (no collective; weak scaling).

`--impl reference` times the CPU restatement of the reference's host graph
(`oracle.model.NumpyLlama`: numpy float32 arithmetic on bf16 tensors, one rounding per
operator) on the host cores for a bounded number of tokens.

The default run's line also carries, under `sharded`, the two workloads whose work really is
split over the N ranks: `llama1b-batch64` (64 sequences, 64 / N per rank, no collective) and
`llama3b-tp` (the 3B architecture tensor-parallel over the N ranks, batch 1 and 8).  Other
workloads print their own line:

    --workload gemm2048       one bf16 GEMM, M = N = K = 2048 (B both ways), tensor roofline
    --workload decode-chain   RMSNorm -> q/k/v GEMV -> RoPE -> gate/up + SwiGLU -> down at hidden 2048
    --workload mamba2         the Mamba2 layer at d_model 1536, 8 x 4096 rows: scan, conv, whole layer
    --workload llama1b-batch64 | llama3b-tp   the sharded workloads on their own
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONTEXT = 2048          # positions already in the caches when decode starts
MAX_SEQ = 4096
METRIC = "llama-3.2-1b-arch decode throughput (batch 1, greedy, context 2048+)"
UNIT = "tokens/s"


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return dict(json.loads(path.read_text()), kind="measured")
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


def timed_loops(run, rewind, steps: int, barrier, min_seconds: float = 0.5, max_loops: int = 64,
                agree=None) -> list[float]:
    """Time ``run()`` (which launches exactly ``steps`` steps) with CUDA events, a barrier and a
    synchronisation on both sides, again and again until ``min_seconds`` have been timed;
    ``rewind()`` puts the inputs back between loops, outside the timed region.  ``agree`` turns a
    rank's timed total into the one every rank stops by (the maximum over the ranks), so that
    all ranks run the same number of loops.  Returns every loop's milliseconds."""
    import torch

    out: list[float] = []
    while True:
        rewind()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        run()
        stop.record()
        barrier()
        out.append(start.elapsed_time(stop))
        total = sum(out) if agree is None else agree(sum(out))
        if total >= min_seconds * 1e3 or len(out) >= max_loops:
            return out


def median(xs) -> float:
    xs = sorted(xs)
    return xs[len(xs) // 2]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._thread = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                     "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.rows.append(parts)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": float(self.rows[0][1]) if self.rows[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(self.rows)}


def build_config():
    import dataclasses

    from iron_b200.applications.llama.model import LLAMA_1B

    return dataclasses.replace(LLAMA_1B, max_seq_len=MAX_SEQ)


def device_weights(config, seed: int, device):
    """Random-init weights N(0, 0.02) (norms one), drawn on the device from ``seed``."""
    from iron_b200.applications.llama.model import random_device_weights

    return random_device_weights(config, seed, device)


def prompt_tokens(seed: int):
    """The 2048-token prompt: uniform-random token ids."""
    import numpy as np

    return np.random.default_rng(seed).integers(0, 128256, CONTEXT)


def time_prefill(engine, tokens, reps: int = 3) -> dict:
    """TTFT of the 2048-token prompt: ids from pinned host memory in, first drawn token out."""
    import torch

    c = engine.c
    engine.prefill(tokens)  # warm-up (module load, tensor-map encode paths)
    times, device_ms = [], []
    for _ in range(reps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        start.record()
        engine.prefill_chunk(tokens, 0)
        stop.record()
        first = int(engine.values[0:1].cpu()[0])
        times.append(time.perf_counter() - t0)
        device_ms.append(start.elapsed_time(stop))
    ttft = min(times)
    n = len(tokens)
    E, F, V = c.hidden_size, c.intermediate_size, c.vocab_size
    Q, KV = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
    linear = c.num_hidden_layers * 2 * n * ((Q + 2 * KV) * E + E * Q + 3 * F * E)
    attn = c.num_hidden_layers * 4 * c.num_attention_heads * c.head_dim * (n * (n + 1) // 2)
    flops = linear + attn + 2 * V * E
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    return {"ttft_ms": round(ttft * 1e3, 3), "device_ms": round(min(device_ms), 3), "tokens": n, "first_token": first,
            "tflops": round(flops / ttft / 1e12, 1), "peak_tflops": peak,
            "frac": round(flops / ttft / 1e12 / peak, 4),
            "launches": engine.launches_per_chunk}


def time_dominant_kernel(engine, peak_gbs: float, peak_kind: str) -> dict:
    """CUDA-event timing of the gate/up SwiGLU GEMV (43 % of the step's bytes), cycling
    through the 16 layers' weights so every launch streams from HBM."""
    import torch

    from iron_b200 import kernels as K
    from iron_b200.tensor import capturing

    c = engine.c
    x, act = engine.x1[0], engine.act[0]
    x.copy_(torch.randn(c.hidden_size, device=engine.device).to(torch.bfloat16))

    def sweep():
        for l in engine.layers:
            K.gemv_swiglu(l["wg"], l["wu"], x, act, norm_weight=l["ln2"], eps=c.eps)

    for _ in range(3):
        sweep()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 20
    g = torch.cuda.CUDAGraph()
    with capturing(g):
        sweep()
    g.replay()
    torch.cuda.synchronize()
    start.record()
    for _ in range(reps):
        g.replay()
    stop.record()
    torch.cuda.synchronize()
    per_launch_s = start.elapsed_time(stop) / 1e3 / (reps * len(engine.layers))
    bytes_per_launch = 2 * c.intermediate_size * c.hidden_size * 2
    achieved = bytes_per_launch / per_launch_s / 1e9
    return {"bound": "hbm", "kernel": "gemv_ring_kernel<SWIGLU> (gate/up GEMV + SiLU + mul, TMA-fed)",
            "achieved": round(achieved, 1), "peak": peak_gbs, "peak_kind": peak_kind,
            "unit": "GB/s", "frac": round(achieved / peak_gbs, 4),
            "bytes_per_launch": bytes_per_launch, "us_per_launch": round(per_launch_s * 1e6, 2),
            # dram__bytes_read.sum + dram__bytes_write.sum per launch of this kernel on these
            # shapes, from one ncu capture (mean of two launches)
            "traffic": 67_480_000 if (c.intermediate_size, c.hidden_size) == (8192, 2048) else None,
            "traffic_from": "profiles/gemv_swiglu_llama1b_ncu.md"}


def cpu_baseline(tokens: int = 2) -> dict:
    """The oracle decoder on the host cores for a bounded number of decode tokens."""
    import numpy as np

    from oracle import model as M

    shape = M.LlamaShape(max_seq_len=CONTEXT + 64)
    t0 = time.perf_counter()
    weights = M.filled_normal(M.llama_shapes(shape), 3001)
    model = M.NumpyLlama(shape, weights)
    rng = np.random.default_rng(3002)
    for k, v in zip(model.keys, model.values):
        k[:CONTEXT] = rng.standard_normal(k[:CONTEXT].shape, dtype=np.float32).astype(k.dtype)
        v[:CONTEXT] = k[:CONTEXT]
    setup = time.perf_counter() - t0
    tok = 1
    model.forward([tok], CONTEXT)  # warm-up: page in, BLAS threads up
    t0 = time.perf_counter()
    for i in range(tokens):
        logits = model.forward([tok], CONTEXT + 1 + i)
        tok = int(np.argmax(logits.astype(np.float32)))
    dt = time.perf_counter() - t0
    cores = len(os.sched_getaffinity(0))
    return {"value": round(tokens / dt, 4), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{tokens} greedy decode tokens of the same 1B-architecture model at context "
                      f"{CONTEXT} (numpy float32 restatement of the reference's host graph, "
                      f"{setup:.0f}s weight draw excluded)"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    timed = max(1, min(args.steps, 3))   # a bounded sample: a token costs about a second on the host
    base = cpu_baseline(tokens=timed)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
            "n_gpus": args.gpus, "steps": args.steps, "steps_timed": timed, "warmup": args.warmup,
            "ms_per_step": round(1e3 / base["value"], 2), "timed_ms": round(timed * 1e3 / base["value"], 1),
            "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, f32 arithmetic",
            "data": "synthetic", "config": workload_config(args.gpus),
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(n_gpus: int) -> dict:
    return {"workload": "configs[2]: Llama-3.2-1B architecture, random-init bf16 N(0,0.02), tied head; "
                        "decode after a 2048-position context, batch 1 per GPU",
            "context": CONTEXT, "replicas": n_gpus,
            "l2": "every step streams 2.47 GB of weights, far more than the 126 MB L2",
            "prompt": "2048 uniform-random token ids run as one prompt chunk; decode continues from its caches"}


def make_barrier(world: int):
    import torch
    import torch.distributed as dist

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    return barrier


def make_agree(world: int, device):
    """The maximum of a number over the ranks (every rank gets the same answer)."""
    return lambda x: max_over_ranks([x], world, device)[0]


def max_over_ranks(values, world: int, device):
    import torch
    import torch.distributed as dist

    t = torch.tensor(list(values), device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def measure_tp(args, rank: int, world: int, device, nb: int, steps: int) -> dict:
    """Llama-3.2-3B architecture, decode of ``nb`` sequences at position 4096 and on, the
    QKV/O/MLP weights tensor-parallel over the ranks with one exchange after o_proj and
    down_proj.  Every rank draws the same full weights from one seed and keeps its shard."""
    import dataclasses

    import torch

    from iron_b200.applications.llama.model import LLAMA_3B
    from iron_b200.lm.engine import LlamaEngine

    ctx = 4096
    config = dataclasses.replace(LLAMA_3B, max_seq_len=ctx + 512)
    weights = device_weights(config, 4001, device)
    engine = LlamaEngine(config, weights, device=device, kv_len_hint=ctx + steps, tp_rank=rank, tp_size=world,
                         batch=nb)
    del weights
    gen = torch.Generator(device=device).manual_seed(4002)
    for l in engine.layers:
        for name in ("k", "v"):
            l[name][:, :ctx].copy_(torch.randn(l[name][:, :ctx].shape, generator=gen, device=device).to(torch.bfloat16))
    engine.capture()
    warm = max(args.warmup, 3)

    def rewind():
        if nb == 1:
            engine.set_call(1, ctx)
        else:
            engine.set_batch([1 + b for b in range(nb)], [ctx] * nb)

    def run():
        for _ in range(steps):
            engine.step()

    rewind()
    for _ in range(warm):
        engine.step()
    loops = timed_loops(run, rewind, steps, make_barrier(world), agree=make_agree(world, device))
    (ms,) = max_over_ranks([median(loops)], world, device)
    engine.check()
    pk = peaks()
    G = config.num_key_value_heads // world
    step_bytes = engine.weight_bytes_per_token + nb * (ctx + steps // 2) * 2 * config.num_hidden_layers * G * config.head_dim * 2
    gbs = step_bytes / (ms / steps / 1e3) / 1e9
    out = {
        "metric": f"llama-3.2-3b-arch decode throughput (batch {nb}, context 4096, tensor parallel)",
        "value": round(nb * steps / (ms / 1e3), 1), "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warm, "loops": len(loops), "ms_per_step": round(ms / steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "configs[3]: Llama-3.2-3B architecture decode, 4096-token KV cache N(0,1), "
                               f"batch {nb}, tensor parallel with one exchange after o_proj and down_proj",
                   "tp": world, "batch": nb},
        "gpu_launches": (engine.launches_per_step + (4 * config.num_hidden_layers if world > 1 else 0)) * steps,
        "exchange": "none" if world == 1 else engine.exchange_path,
        "per_rank_roofline": {"bound": "hbm", "bytes_per_step": step_bytes, "achieved": round(gbs, 1),
                              "peak": pk["hbm_gbs"], "peak_kind": pk["kind"], "unit": "GB/s",
                              "frac": round(gbs / pk["hbm_gbs"], 4)},
        "all_reduces_per_step": 2 * config.num_hidden_layers if world > 1 else 0}
    del engine
    torch.cuda.empty_cache()
    return out


def measure_batch(args, rank: int, world: int, device, total: int, steps: int, e2e: bool = True) -> dict:
    """Llama-3.2-1B architecture, ``total`` independent sequences decoded in lockstep after a
    2048-token context each, the batch split over the ranks with no collective (every rank
    holds the full weights and total / world sequences)."""
    import numpy as np
    import torch

    from iron_b200.lm.engine import LlamaEngine, batch_shard

    mine = batch_shard(total, rank, world)
    config = build_config()
    weights = device_weights(config, 3001, device)
    engine = LlamaEngine(config, weights, device=device, batch=len(mine), kv_len_hint=CONTEXT + steps)
    del weights
    for b, seq in enumerate(mine):
        engine.prefill(np.random.default_rng(3100 + seq).integers(0, config.vocab_size, CONTEXT), 0, seq=b)
    first = engine.drawn[:, CONTEXT - 1].cpu().numpy()       # the token each prompt drew
    engine.capture()
    warm = max(args.warmup, 3)
    positions = [CONTEXT] * len(mine)
    barrier = make_barrier(world)

    def run():
        for _ in range(steps):
            engine.step()

    engine.set_batch(first, positions)
    for _ in range(warm):
        engine.step()
    with ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) as clocks:
        loops = timed_loops(run, lambda: engine.set_batch(first, positions), steps, barrier,
                            agree=make_agree(world, device))
    ms_e2e = None
    if e2e:
        # host-facing: every step's tokens go in from pinned host memory and come back
        state = {}

        def rewind_host():
            state["toks"] = list(first)

        def run_host():
            toks = state["toks"]
            for i in range(steps):
                toks = engine.decode_batch(toks, [CONTEXT + i] * len(mine))

        rewind_host()
        for i in range(warm):
            state["toks"] = engine.decode_batch(state["toks"], [CONTEXT + i] * len(mine))
        ms_e2e = median(timed_loops(run_host, rewind_host, steps, barrier, agree=make_agree(world, device)))
    ms, ms_e2e = max_over_ranks([median(loops), ms_e2e or 0.0], world, device)
    engine.check()
    pk = peaks()
    kv = (CONTEXT + steps // 2) * 32768 * len(mine)
    step_bytes = engine.weight_bytes_per_token + kv
    gbs = step_bytes / (ms / steps / 1e3) / 1e9
    out = {
        "metric": f"llama-3.2-1b-arch decode throughput ({total} sequences, greedy, context 2048+)",
        "value": round(total * steps / (ms / 1e3), 1), "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warm, "loops": len(loops), "ms_per_step": round(ms / steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"configs[2] batch {total}: Llama-3.2-1B architecture, {total} independent sequences after a "
                               "2048-token prompt each, split over the ranks with no collective",
                   "sequences_per_gpu": len(mine), "context": CONTEXT,
                   "l2": "every step streams 2.47 GB of weights and 67 MB of KV cache per sequence"},
        "gpu_launches": engine.launches_per_step * steps,
        "clocks": clocks.summary(),
        "per_rank_roofline": {"bound": "hbm", "bytes_per_step": step_bytes, "achieved": round(gbs, 1),
                              "peak": pk["hbm_gbs"], "peak_kind": pk["kind"], "unit": "GB/s",
                              "frac": round(gbs / pk["hbm_gbs"], 4)}}
    if e2e:
        out["e2e"] = {"value": round(total * steps / (ms_e2e / 1e3), 1), "unit": UNIT,
                      "h2d_bytes_per_step": 8 * len(mine), "d2h_bytes_per_step": 4 * len(mine),
                      "ms_per_step": round(ms_e2e / steps, 4)}
    del engine
    torch.cuda.empty_cache()
    return out


def sharded_workloads(args, rank: int, world: int, device) -> dict:
    """The two partitionings of the work over the ranks, measured after the headline: their
    results ride on the headline's JSON line under ``sharded``."""
    steps = min(args.steps, 32)
    out = {}
    for name, fn in (("llama1b-batch64", lambda: measure_batch(args, rank, world, device, 64, steps, e2e=False)),
                     ("llama3b-tp batch 1", lambda: measure_tp(args, rank, world, device, 1, steps)),
                     ("llama3b-tp batch 8", lambda: measure_tp(args, rank, world, device, 8, steps))):
        try:
            r = fn()
            out[name] = {k: r[k] for k in ("value", "unit", "ms_per_step", "steps", "loops", "scaling",
                                           "per_rank_roofline", "exchange", "all_reduces_per_step", "gpu_launches")
                         if k in r}
        except Exception as e:   # the headline stands on its own
            out[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
    return out


def time_prompt_attention(device, n: int = CONTEXT, heads: int = 32, kv_heads: int = 8, head_dim: int = 64) -> None:
    """CUDA-event time of the prompt-chunk attention kernel on its own: ``n`` queries over ``n``
    keys, causal, random bf16 inputs (17.2 GFLOP at the defaults)."""
    import torch

    from iron_b200 import kernels as K

    g = torch.Generator(device=device).manual_seed(7)
    q = torch.randn(n, heads, head_dim, device=device, generator=g).to(torch.bfloat16)
    k = torch.randn(n, kv_heads, head_dim, device=device, generator=g).to(torch.bfloat16)
    v = torch.randn(n, kv_heads, head_dim, device=device, generator=g).to(torch.bfloat16)
    o = torch.empty_like(q)
    for _ in range(3):
        K.mha_prefill(q, k, v, o, q_tokens=n, kv_tokens=n)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 20
    start.record()
    for _ in range(reps):
        K.mha_prefill(q, k, v, o, q_tokens=n, kv_tokens=n)
    stop.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(stop) * 1e3 / reps
    flops = 4 * heads * head_dim * n * (n + 1) // 2
    print(json.dumps({"kernel": "prompt attention", "tokens": n, "heads": heads, "kv_heads": kv_heads,
                      "head_dim": head_dim, "us_per_launch": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                      "tensor_memory_kernel": os.environ.get("IRON_MHA_PREFILL_TC", "1") != "0",
                      "status": int(K.prefill_status(device).item())}))


def event_us(launch, reps: int, sets: int = 1) -> float:
    """Microseconds per ``launch(i)`` over ``reps`` launches timed as one CUDA-event bracket
    after three warm-up rounds; ``i`` cycles through ``sets`` input sets so that consecutive
    launches do not find their inputs in L2."""
    import torch

    for i in range(3 * sets):
        launch(i % sets)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(reps):
        launch(i % sets)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / reps


def run_gemm2048(args, device) -> None:
    """configs[0]: one bf16 GEMM, M = N = K = 2048, A and B N(0,1)/sqrt(K) (seeds 1001, 1002),
    f32 accumulation, bf16 output; B row-major (K, N) and as (N, K) (``b_col_maj``)."""
    import numpy as np
    import torch

    from iron_b200 import kernels as K

    n, sets = 2048, 8    # 8 x 25 MB of operands: launches do not re-read their inputs from the 126 MB L2
    gen = torch.Generator(device=device)
    A = [(torch.randn(n, n, generator=gen.manual_seed(1001 + 10 * i), device=device) / n ** 0.5).to(torch.bfloat16)
         for i in range(sets)]
    B = [(torch.randn(n, n, generator=gen.manual_seed(1002 + 10 * i), device=device) / n ** 0.5).to(torch.bfloat16)
         for i in range(sets)]
    C = [torch.empty(n, n, dtype=torch.bfloat16, device=device) for _ in range(sets)]
    status = torch.zeros(1, dtype=torch.int32, device=device)
    reps = max(args.steps, 200)
    flops = 2 * n ** 3
    pk = peaks()
    res = {}
    with ClockSampler(device.index or 0) as clocks:
        for name, col in (("b_row_major", False), ("b_col_maj", True)):
            us = event_us(lambda i: K.gemm(A[i], B[i], C[i], b_col_maj=col, status=status), reps, sets)
            res[name] = {"us_per_launch": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                         "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 4)}
    best = max(res.values(), key=lambda r: r["tflops"])
    # the CPU restatement (numpy float32 matmul of the bf16 operands, rounded once) beside it
    a, b = A[0].float().cpu().numpy(), B[0].float().cpu().numpy()
    a @ b
    t0 = time.perf_counter()
    for _ in range(3):
        a @ b
    cpu = (time.perf_counter() - t0) / 3
    print(json.dumps({
        "metric": "bf16 GEMM 2048^3 throughput", "value": best["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
        "steps": reps, "warmup": 3 * sets, "ms_per_step": round(best["us_per_launch"] / 1e3, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "configs[0]: bf16 GEMM M=N=K=2048, A,B ~ N(0,1)/sqrt(K), f32 accumulate, bf16 out",
                   "l2": f"{sets} operand sets cycled (201 MB), more than the 126 MB L2"},
        "gpu_launches": 2 * reps, "clocks": clocks.summary(), "layouts": res,
        "roofline": {"bound": "tensor", "kernel": "gemm_pair_kernel / gemm_bf16_kernel (tcgen05)",
                     "achieved": best["tflops"], "peak": pk["bf16_tflops"], "peak_kind": pk["kind"] + " (burst)",
                     "unit": "TFLOP/s", "frac": best["frac"], "flops_per_launch": flops,
                     "us_per_launch": best["us_per_launch"], "traffic": None},
        "status": int(status.item()),
        "cpu_baseline": {"value": round(flops / cpu / 1e12, 4), "unit": "TFLOP/s",
                         "cores": len(os.sched_getaffinity(0)), "kind": "port",
                         "sample": "3 numpy float32 matmuls of the same 2048^3 operands (the reference's GEMM.reference)"}}))


def run_decode_chain(args, device) -> None:
    """configs[1]: the decode-step operator chain at hidden 2048, batch 1, position 1023:
    RMSNorm -> fused q/k/v GEMV (3072 x 2048) -> RoPE -> gate/up GEMV (2 x 8192 x 2048) + SwiGLU ->
    down GEMV (2048 x 8192), as three fused kernels in one CUDA graph."""
    import numpy as np
    import torch

    from iron_b200 import kernels as K
    from iron_b200.lm.config import rope_angles
    from iron_b200.tensor import capturing

    E, H, G, D, F, pos, sets = 2048, 32, 8, 64, 8192, 1023, 4   # 4 x 113 MB of weights cycled
    gen = torch.Generator(device=device).manual_seed(2001)
    rnd = lambda *shape, std=0.02: (torch.randn(*shape, generator=gen, device=device) * std).to(torch.bfloat16)
    x = rnd(E, std=1.0)
    w = [dict(norm=(1 + torch.randn(E, generator=gen, device=device) * 0.02).to(torch.bfloat16),
              qkv=rnd((H + 2 * G) * D, E), gate=rnd(F, E), up=rnd(F, E), down=rnd(E, F)) for _ in range(sets)]
    angles = torch.from_numpy(rope_angles(D, 1024, 500000.0).astype(np.float32)).to(device).to(torch.bfloat16)
    kc = torch.zeros(1024, G, D, dtype=torch.bfloat16, device=device)
    vc = torch.zeros_like(kc)
    q = torch.empty(H, D, dtype=torch.bfloat16, device=device)
    act = torch.empty(F, dtype=torch.bfloat16, device=device)
    o = torch.empty(E, dtype=torch.bfloat16, device=device)

    def chain(i):
        s = w[i]
        K.decode_qkv_rope(s["qkv"], x, angles, kc, vc, q, H=H, G=G, D=D, position=pos, norm_weight=s["norm"], eps=1e-5)
        K.gemv_swiglu(s["gate"], s["up"], x, act, norm_weight=s["norm"], eps=1e-5)
        K.gemv(s["down"], act, o)

    for i in range(sets):
        chain(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with capturing(g):
        for i in range(sets):
            chain(i)
    reps = max(args.steps // sets, 50)
    with ClockSampler(device.index or 0) as clocks:
        us = event_us(lambda i: g.replay(), reps) / sets
    nbytes = ((H + 2 * G) * D * E + 2 * F * E + E * F) * 2
    pk = peaks()
    gbs = nbytes / us / 1e3
    # the same chain through the restated numpy references on the host
    from iron_b200.tensor import torch_to_numpy as to_numpy
    from oracle import ops

    hx, hw = to_numpy(x), {k: to_numpy(v) for k, v in w[0].items()}
    def host():
        h = ops.rms_norm(hx[None], hw["norm"], 1e-5)[0]
        ops.gemv(hw["qkv"], h)
        a = ops.mul(ops.silu(ops.gemv(hw["gate"], h)), ops.gemv(hw["up"], h))
        return ops.gemv(hw["down"], a)
    host()
    t0 = time.perf_counter()
    for _ in range(5):
        host()
    cpu = (time.perf_counter() - t0) / 5
    print(json.dumps({
        "metric": "decode-step operator chain latency (hidden 2048, batch 1)", "value": round(us, 2), "unit": "us",
        "n_gpus": 1, "steps": reps * sets, "warmup": 3, "ms_per_step": round(us / 1e3, 5),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "configs[1]: RMSNorm -> QKV GEMV 2048->3072 -> RoPE (theta 5e5, position 1023) -> "
                               "gate/up GEMV 2048->2x8192 + SwiGLU -> down GEMV 8192->2048; weights N(0,0.02)",
                   "l2": f"{sets} weight sets cycled (453 MB), more than the 126 MB L2",
                   "kernels": "iron_decode_qkv_rope_bf16, iron_gemv_swiglu_bf16, iron_gemv_bf16 in one CUDA graph"},
        "gpu_launches": 3 * reps * sets, "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": "the chain's three GEMV kernels", "achieved": round(gbs, 1),
                     "peak": pk["hbm_gbs"], "peak_kind": pk["kind"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4), "bytes_per_launch": nbytes,
                     "us_per_launch": round(us, 2), "traffic": None},
        "cpu_baseline": {"value": round(cpu * 1e6, 1), "unit": "us", "cores": len(os.sched_getaffinity(0)),
                         "kind": "port", "sample": "5 passes of the same chain through the numpy references"}}))


def run_mamba2(args, device) -> None:
    """configs[4]: the Mamba2 layer at d_model 1536, d_inner 3072 (48 heads of 64), d_state 128,
    one group, conv width 4, 8 sequences of 4096 rows: the selective scan and the causal conv on
    their own (HBM rooflines) and the whole mixer (projections on the tensor cores)."""
    import numpy as np
    import torch

    from iron_b200 import kernels as K
    from iron_b200.lm.mamba import MambaMixer

    B, R, E, H, P, N, Kc = args.mamba_batch, args.mamba_rows, 1536, 48, 64, 128, 4
    inner, C = H * P, H * P + 2 * N
    gen = torch.Generator(device=device).manual_seed(5001)
    rnd = lambda *shape, std=1.0: (torch.randn(*shape, generator=gen, device=device) * std).to(torch.bfloat16)
    xbc, taps, bias = rnd(B, R, C), rnd(Kc, C, std=0.5), torch.zeros(C, dtype=torch.bfloat16, device=device)
    dt = (torch.randn(B, R, H, generator=gen, device=device) - 4).to(torch.bfloat16)
    A = -torch.exp(torch.rand(H, generator=gen, device=device) * 2.7)
    head = torch.stack([torch.zeros(H, device=device), A, torch.ones(H, device=device)], 1).contiguous()
    y = torch.empty(B, R, inner, dtype=torch.bfloat16, device=device)
    final = torch.empty(B, H, P, N, dtype=torch.float32, device=device)
    conv_out = torch.empty_like(xbc)
    reps = max(min(args.steps, 50), 10)
    pk = peaks()
    with ClockSampler(device.index or 0) as clocks:
        scan_us = event_us(lambda i: K.selective_scan(xbc, dt, head, None, heads=H, head_dim=P, state_size=N,
                                                     y=y, final=final), reps)
        conv_us = event_us(lambda i: K.causal_conv1d(xbc, taps, bias=bias, out=conv_out, silu=True), reps)
        w = {"in_proj.weight": rnd(inner + C + H, E, std=0.02), "conv1d.weight": rnd(C, 1, Kc, std=0.5),
             "conv1d.bias": bias, "dt_bias": torch.zeros(H, device=device), "A_log": torch.log(-A),
             "D": torch.ones(H, device=device), "norm.weight": torch.ones(inner, device=device),
             "out_proj.weight": rnd(E, inner, std=0.02)}
        mixer = MambaMixer(w, hidden_size=E, heads=H, head_dim=P, state_size=N, batch=B, rows=R, device=device)
        x = rnd(B, R, E)
        layer_us = event_us(lambda i: mixer.forward(x), max(reps // 2, 5))
        mixer.check()
    scan_bytes = B * (R * C * 2 + R * H * 2 + R * inner * 2 + H * P * N * 4 + H * 12)
    conv_bytes = B * 2 * R * C * 2
    proj_flops = 2 * B * R * E * (inner + C + H) + 2 * B * R * inner * E
    scan_gbs, conv_gbs = scan_bytes / scan_us / 1e3, conv_bytes / conv_us / 1e3
    mode = os.environ.get("IRON_SCAN_CHUNKED", "2")[:1]
    if mode == "2" and R >= 128:
        scan_kernel = "ssd_scan_tc_kernel (128-row chunks, tcgen05 products with tensor-memory accumulators)"
    elif mode in "12" and R >= 32:
        scan_kernel = "ssd_scan_kernel (64-row chunks, warp MMAs)"
    else:
        scan_kernel = "selective_scan_kernel (step by step)"
    # CPU: the sequential numpy scan on a bounded sample of one sequence
    from iron_b200.tensor import torch_to_numpy as to_numpy
    from oracle import ops

    rows = min(512, R)
    hx, hd, hh = to_numpy(xbc[0, :rows]), to_numpy(dt[0, :rows]), head.cpu().numpy()
    t0 = time.perf_counter()
    ops.selective_scan(hx, hd, hh, np.zeros((H, P, N), np.float32), heads=H, head_dim=P, state_size=N)
    cpu = time.perf_counter() - t0
    print(json.dumps({
        "metric": f"Mamba2 layer time (d_model 1536, {B} x {R} rows)", "value": round(layer_us, 1), "unit": "us",
        "n_gpus": 1, "steps": reps, "warmup": 3, "ms_per_step": round(layer_us / 1e3, 4), "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, f32 scan state", "data": "synthetic",
        "config": {"workload": "configs[4]: Mamba2 layer, d_model 1536, d_inner 3072, 48 heads x 64, d_state 128, "
                               f"1 group, conv 4, sequence {R}, batch {B}; inputs N(0,1), dt softplus(N(-4,1)), "
                               "A = -exp(U(0,2.7))",
                   "l2": "the scan reads 448 MB and the layer's activations are 200 MB each: nothing stays in L2"},
        "gpu_launches": reps * 2 + max(reps // 2, 5) * MambaMixer.launches_per_call, "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": scan_kernel, "achieved": round(scan_gbs, 1),
                     "peak": pk["hbm_gbs"], "peak_kind": pk["kind"], "unit": "GB/s",
                     "frac": round(scan_gbs / pk["hbm_gbs"], 4), "bytes_per_launch": scan_bytes,
                     "us_per_launch": round(scan_us, 1),
                     # dram bytes of one launch at this shape under ncu (the summary named beside it)
                     "traffic": 392400000 if (mode == "2" and (B, R) == (8, 4096)) else None,
                     "traffic_from": "profiles/ssd_scan_tc_mamba2_ncu.md"},
        "conv_roofline": {"bound": "hbm", "kernel": "causal_conv_kernel (+ bias + SiLU)", "achieved": round(conv_gbs, 1),
                          "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(conv_gbs / pk["hbm_gbs"], 4),
                          "bytes_per_launch": conv_bytes, "us_per_launch": round(conv_us, 1),
                          "traffic": 399600000 if (B, R) == (8, 4096) else None,
                          "traffic_from": "profiles/causal_conv_mamba2_ncu.md"},
        "layer": {"us": round(layer_us, 1), "launches": MambaMixer.launches_per_call,
                  "projection_tflop": round(proj_flops / 1e12, 3),
                  "projection_floor_us": round(proj_flops / pk["bf16_tflops_sustained"] / 1e6, 1)},
        "cpu_baseline": {"value": round(cpu * R / rows * B * 1e6, 0), "unit": "us", "cores": 1, "kind": "port",
                         "sample": f"the sequential numpy scan on {rows} rows of one sequence ({cpu:.2f} s), "
                                   f"scaled to {B} x {R} rows"}}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sharded", action="store_true",
                    help="llama1b: leave the sharded workloads (batch 64, 3B tensor parallel) off the line")
    ap.add_argument("--sequences", type=int, default=64,
                    help="llama1b-batch64: sequences in the whole job (split over the ranks)")
    ap.add_argument("--decode-step-trace", action="store_true",
                    help="with IRON_DECODE_STEP=1: print the one-kernel step's per-phase timeline and exit")
    ap.add_argument("--tp-batch", type=int, default=1,
                    help="llama3b-tp: sequences decoded in lockstep (1, 2, 4, ... 32)")
    ap.add_argument("--mamba-batch", type=int, default=8, help="mamba2: sequences (8 in the named config)")
    ap.add_argument("--mamba-rows", type=int, default=4096,
                    help="mamba2: rows per sequence (4096 in the named config; a profiler capture takes fewer)")
    ap.add_argument("--prompt-attention", action="store_true",
                    help="time the prompt-chunk attention kernel alone (2048 x 2048 causal, the 1B head "
                         "shape; IRON_MHA_PREFILL_TC=0 for the warp-MMA kernel), print one JSON line and exit")
    ap.add_argument("--workload", default="llama1b",
                    choices=["llama1b", "llama3b-tp", "llama1b-batch64", "gemm2048", "decode-chain", "mamba2"],
                    help="llama1b: the headline decode, one replica per GPU (plus the sharded workloads on "
                         "the same line); the others print their own line (see the module docstring)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from __graft_entry__ import build

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU path); "
                           "use --impl reference for the CPU baseline")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import datetime

        # a rank that failed must not leave the others in a collective for long
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=180))
    if rank == 0:
        build()
    if world > 1:
        dist.barrier()

    def leave():
        # captured graphs may hold NCCL work: leave without tearing the group down under them
        sys.stdout.flush()
        torch.cuda.synchronize()
        os._exit(0)

    from iron_b200.lm.engine import LlamaEngine

    if args.prompt_attention:
        time_prompt_attention(device)
        return
    single = {"gemm2048": run_gemm2048, "decode-chain": run_decode_chain, "mamba2": run_mamba2}
    if args.workload in single:
        if rank == 0:
            single[args.workload](args, device)
        leave()
    if args.workload == "llama1b-batch64":
        line = measure_batch(args, rank, world, device, args.sequences, args.steps)
        if rank == 0:
            print(json.dumps(line))
        leave()
    if args.workload == "llama3b-tp":
        line = measure_tp(args, rank, world, device, max(1, args.tp_batch), args.steps)
        if rank == 0:
            print(json.dumps(line))
        leave()
    config = build_config()
    weights = device_weights(config, 3001, device)
    engine = LlamaEngine(config, weights, device=device, kv_len_hint=CONTEXT + args.steps)
    del weights
    tokens = prompt_tokens(3002 + rank)
    prefill = time_prefill(engine, tokens)
    engine.capture()
    if args.decode_step_trace:
        engine.set_call(1, CONTEXT)
        for _ in range(max(args.steps, 1)):
            engine.step()
        torch.cuda.synchronize()
        t = engine.step_trace()
        L = config.num_hidden_layers
        names = ["qkv", "attention", "o_proj", "gate_up", "down_proj"]
        out = {}
        for j, name in enumerate(names):
            rows = [5 * l + j for l in range(L)]
            wait = [t[p, 0] - (t[p - 1, 2] if p else t[p, 0]) for p in rows]
            out[name] = {"wait_us": round(float(np.mean(wait)) / 1e3, 2),
                         "stage_us": round(float(np.mean([t[p, 1] - t[p, 0] for p in rows])) / 1e3, 2),
                         "items_us": round(float(np.mean([t[p, 2] - t[p, 1] for p in rows])) / 1e3, 2)}
        p = 5 * L
        out["head"] = {"wait_us": round((t[p, 0] - t[p - 1, 2]) / 1e3, 2), "stage_us": round((t[p, 1] - t[p, 0]) / 1e3, 2),
                       "items_us": round((t[p, 2] - t[p, 1]) / 1e3, 2)}
        out["step_us"] = round((t[p, 2] - t[0, 0]) / 1e3, 1)
        print(json.dumps({"decode_step_trace": out}))
        return
    warm = max(args.warmup, 3)
    barrier = make_barrier(world)
    steps = args.steps

    # ---- device-carried loop: inputs resident, one graph replay per token.  The K-step loop
    # is timed again and again (from the same position) until half a second has been timed;
    # the line reports the median loop. ----
    def run():
        for _ in range(steps):
            engine.step()

    engine.set_call(1, CONTEXT)
    for _ in range(warm):
        engine.step()
    with ClockSampler(local) as clocks:
        loops = timed_loops(run, lambda: engine.set_call(1, CONTEXT), steps, barrier, agree=make_agree(world, device))

        # ---- host-facing call: token from pinned host memory in, drawn token out ----
        def run_host():
            tok = 1
            for i in range(steps):
                tok = engine.decode(tok, CONTEXT + i)

        tok = 1
        for i in range(warm):
            tok = engine.decode(tok, CONTEXT + i)
        loops_e2e = timed_loops(run_host, lambda: None, steps, barrier, agree=make_agree(world, device))
    ms, ms_e2e = max_over_ranks([median(loops), median(loops_e2e)], world, device)
    pk = peaks()
    peak, kind = pk["hbm_gbs"], pk["kind"]
    value = world * steps / (ms / 1e3)
    e2e = world * steps / (ms_e2e / 1e3)
    step_bytes = engine.weight_bytes_per_token + (CONTEXT + steps // 2) * 32768
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world,
        "steps": steps, "warmup": warm, "ms_per_step": round(ms / steps, 4),
        "loops": len(loops), "loop_ms": {"median": round(median(loops), 4), "min": round(min(loops), 4),
                                         "max": round(max(loops), 4), "timed_s": round(sum(loops) / 1e3, 3)},
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(world),
        "e2e": {"value": round(e2e, 1), "unit": UNIT, "h2d_bytes_per_step": 64,
                "d2h_bytes_per_step": 4, "ms_per_step": round(ms_e2e / steps, 4), "loops": len(loops_e2e)},
        "gpu_launches": engine.launches_per_step * steps,
        "clocks": clocks.summary(),
        "prefill": prefill,
    }
    step_gbs = step_bytes / (ms / steps / 1e3) / 1e9
    gemv = time_dominant_kernel(engine, peak, kind)
    if engine.fused_step:
        # the whole step is one launch of the persistent kernel: it IS the dominant kernel
        line["roofline"] = {
            "bound": "hbm", "kernel": "decode_step_kernel (all layers, head and draw in one launch)",
            "achieved": round(step_gbs, 1), "peak": peak, "peak_kind": kind, "unit": "GB/s",
            "frac": round(step_gbs / peak, 4), "bytes_per_launch": step_bytes,
            "us_per_launch": round(ms / steps * 1e3, 2), "traffic": None}
        line["gemv_roofline"] = gemv
    else:
        line["roofline"] = gemv
        line["step_roofline"] = {"bound": "hbm", "bytes_per_step": step_bytes,
                                 "achieved": round(step_gbs, 1), "peak": peak, "unit": "GB/s",
                                 "frac": round(step_gbs / peak, 4),
                                 "weights_only_frac": round(engine.weight_bytes_per_token / (ms / steps / 1e3) / 1e9 / peak, 4)}
    del engine
    torch.cuda.empty_cache()
    if not args.no_sharded and os.environ.get("IRON_BENCH_SHARDED", "1") != "0":
        line["sharded"] = sharded_workloads(args, rank, world, device)
    if rank != 0:
        leave()
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line))
    leave()


if __name__ == "__main__":
    main()
