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


def measured_peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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
    base = cpu_baseline(tokens=max(1, min(args.steps, 3)))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(1e3 / base["value"], 2), "higher_is_better": True,
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


def run_tp(args, rank: int, world: int, device) -> None:
    """Llama-3.2-3B architecture, decode of one token at position 4096 and on, batch 1,
    QKV/O/MLP weights tensor-parallel over the ranks with an all-reduce after o_proj and
    down_proj.  Every rank draws the same full weights from one seed and keeps its shard."""
    import dataclasses

    import torch
    import torch.distributed as dist

    from iron_b200.applications.llama.model import LLAMA_3B
    from iron_b200.lm.engine import LlamaEngine

    ctx = 4096
    config = dataclasses.replace(LLAMA_3B, max_seq_len=ctx + 512)
    weights = device_weights(config, 4001, device)
    nb = max(1, args.tp_batch)
    engine = LlamaEngine(config, weights, device=device, kv_len_hint=ctx + args.steps, tp_rank=rank, tp_size=world,
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

    rewind()
    for _ in range(warm):
        engine.step()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rewind()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.steps):
        engine.step()
    stop.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([start.elapsed_time(stop)], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    if rank != 0:
        return
    peak, kind = measured_peaks()
    step_bytes = engine.weight_bytes_per_token + nb * (ctx + args.steps // 2) * 2 * 28 * (8 // world) * 128 * 2
    print(json.dumps({
        "metric": f"llama-3.2-3b-arch decode throughput (batch {nb}, context 4096, tensor parallel)",
        "value": round(nb * args.steps / (ms / 1e3), 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "configs[3]: Llama-3.2-3B architecture decode, 4096-token KV cache N(0,1), "
                               f"batch {nb}, tensor parallel with one exchange after o_proj and down_proj",
                   "tp": world, "batch": nb},
        "gpu_launches": (engine.launches_per_step + (4 * 28 if world > 1 else 0)) * args.steps,
        "per_rank_roofline": {"bound": "hbm", "bytes_per_step": step_bytes,
                              "achieved": round(step_bytes / (ms / args.steps / 1e3) / 1e9, 1),
                              "peak": peak, "unit": "GB/s",
                              "frac": round(step_bytes / (ms / args.steps / 1e3) / 1e9 / peak, 4)},
        "all_reduces_per_step": 56 if world > 1 else 0}))


def run_batch(args, rank: int, world: int, device) -> None:
    """Llama-3.2-1B architecture, 64 independent sequences decoded in lockstep after a
    2048-token context each, the batch split over the ranks with no collective (every rank
    holds the full weights and 64 / world sequences)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from iron_b200.lm.engine import LlamaEngine, batch_shard

    total = args.sequences
    mine = batch_shard(total, rank, world)
    config = build_config()
    weights = device_weights(config, 3001, device)
    engine = LlamaEngine(config, weights, device=device, batch=len(mine), kv_len_hint=CONTEXT + args.steps)
    del weights
    for b, seq in enumerate(mine):
        engine.prefill(np.random.default_rng(3100 + seq).integers(0, config.vocab_size, CONTEXT), 0, seq=b)
    first = engine.drawn[:, CONTEXT - 1].cpu().numpy()       # the token each prompt drew
    engine.capture()
    warm = max(args.warmup, 3)
    positions = [CONTEXT] * len(mine)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    engine.set_batch(first, positions)
    for _ in range(warm):
        engine.step()
    engine.set_batch(first, positions)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) as clocks:
        start.record()
        for _ in range(args.steps):
            engine.step()
        stop.record()
        barrier()
    ms = start.elapsed_time(stop)
    # host-facing: every step's tokens go in from pinned host memory and come back
    toks = list(first)
    for i in range(warm):
        toks = engine.decode_batch(toks, [CONTEXT + i] * len(mine))
    barrier()
    toks = list(first)
    start.record()
    for i in range(args.steps):
        toks = engine.decode_batch(toks, [CONTEXT + i] * len(mine))
    stop.record()
    barrier()
    ms_e2e = start.elapsed_time(stop)
    t = torch.tensor([ms, ms_e2e], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = t.tolist()
    if rank != 0:
        return
    peak, kind = measured_peaks()
    kv = (CONTEXT + args.steps // 2) * 32768 * len(mine)
    step_bytes = engine.weight_bytes_per_token + kv
    gbs = step_bytes / (ms / args.steps / 1e3) / 1e9
    print(json.dumps({
        "metric": f"llama-3.2-1b-arch decode throughput ({total} sequences, greedy, context 2048+)",
        "value": round(total * args.steps / (ms / 1e3), 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"configs[2] batch {total}: Llama-3.2-1B architecture, {total} independent sequences after a "
                               "2048-token prompt each, split over the ranks with no collective",
                   "sequences_per_gpu": len(mine), "context": CONTEXT,
                   "l2": "every step streams 2.47 GB of weights and 67 MB of KV cache per sequence"},
        "e2e": {"value": round(total * args.steps / (ms_e2e / 1e3), 1), "unit": UNIT,
                "h2d_bytes_per_step": 8 * len(mine), "d2h_bytes_per_step": 4 * len(mine),
                "ms_per_step": round(ms_e2e / args.steps, 4)},
        "gpu_launches": engine.launches_per_step * args.steps,
        "clocks": clocks.summary(),
        "per_rank_roofline": {"bound": "hbm", "bytes_per_step": step_bytes, "achieved": round(gbs, 1),
                              "peak": peak, "peak_kind": kind, "unit": "GB/s", "frac": round(gbs / peak, 4)}}))


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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sequences", type=int, default=64,
                    help="llama1b-batch64: sequences in the whole job (split over the ranks)")
    ap.add_argument("--decode-step-trace", action="store_true",
                    help="with IRON_DECODE_STEP=1: print the one-kernel step's per-phase timeline and exit")
    ap.add_argument("--tp-batch", type=int, default=1,
                    help="llama3b-tp: sequences decoded in lockstep (1, 2, 4, ... 32)")
    ap.add_argument("--prompt-attention", action="store_true",
                    help="time the prompt-chunk attention kernel alone (2048 x 2048 causal, the 1B head "
                         "shape; IRON_MHA_PREFILL_TC=0 for the warp-MMA kernel), print one JSON line and exit")
    ap.add_argument("--workload", default="llama1b", choices=["llama1b", "llama3b-tp", "llama1b-batch64"],
                    help="llama1b: the headline decode, one replica per GPU; llama3b-tp: the 3B "
                         "architecture tensor-parallel over --gpus ranks at context 4096")
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
        dist.init_process_group("nccl", device_id=device)
    if rank == 0:
        build()
    if world > 1:
        dist.barrier()

    from iron_b200.lm.engine import LlamaEngine

    if args.prompt_attention:
        time_prompt_attention(device)
        return
    if args.workload == "llama1b-batch64":
        run_batch(args, rank, world, device)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "llama3b-tp":
        run_tp(args, rank, world, device)
        # the captured graphs hold NCCL work: leave without tearing the group down under them
        sys.stdout.flush()
        torch.cuda.synchronize()
        os._exit(0)
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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-carried loop: inputs resident, one graph replay per token ----
    engine.set_call(1, CONTEXT)
    for _ in range(warm):
        engine.step()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    engine.set_call(1, CONTEXT)
    barrier()
    with ClockSampler(local) as clocks:
        start.record()
        for _ in range(args.steps):
            engine.step()
        stop.record()
        barrier()
    ms = start.elapsed_time(stop)

    # ---- host-facing call: token from pinned host memory in, drawn token out ----
    tok = 1
    for i in range(warm):
        tok = engine.decode(tok, CONTEXT + i)
    barrier()
    tok = 1
    start.record()
    for i in range(args.steps):
        tok = engine.decode(tok, CONTEXT + i)
    stop.record()
    barrier()
    ms_e2e = start.elapsed_time(stop)

    times = torch.tensor([ms, ms_e2e], device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = times.tolist()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, kind = measured_peaks()
    value = world * args.steps / (ms / 1e3)
    e2e = world * args.steps / (ms_e2e / 1e3)
    step_bytes = engine.weight_bytes_per_token + (CONTEXT + args.steps // 2) * 32768
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": round(ms / args.steps, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(world),
        "e2e": {"value": round(e2e, 1), "unit": UNIT, "h2d_bytes_per_step": 64,
                "d2h_bytes_per_step": 4, "ms_per_step": round(ms_e2e / args.steps, 4)},
        "gpu_launches": engine.launches_per_step * args.steps,
        "clocks": clocks.summary(),
        "prefill": prefill,
    }
    step_gbs = step_bytes / (ms / args.steps / 1e3) / 1e9
    gemv = time_dominant_kernel(engine, peak, kind)
    if engine.fused_step:
        # the whole step is one launch of the persistent kernel: it IS the dominant kernel
        line["roofline"] = {
            "bound": "hbm", "kernel": "decode_step_kernel (all layers, head and draw in one launch)",
            "achieved": round(step_gbs, 1), "peak": peak, "peak_kind": kind, "unit": "GB/s",
            "frac": round(step_gbs / peak, 4), "bytes_per_launch": step_bytes,
            "us_per_launch": round(ms / args.steps * 1e3, 2), "traffic": None}
        line["gemv_roofline"] = gemv
    else:
        line["roofline"] = gemv
        line["step_roofline"] = {"bound": "hbm", "bytes_per_step": step_bytes,
                                 "achieved": round(step_gbs, 1), "peak": peak, "unit": "GB/s",
                                 "frac": round(step_gbs / peak, 4)}
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
