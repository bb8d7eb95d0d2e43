"""``main``, a model's command line (iron/lm/cli.py:83-208).

``python -m iron_b200.applications.llama.model DIR`` loads the checkpoint in ``DIR`` into
the fused engine and samples from it, or checks it: ``--check-accuracy`` compares each
step's logits with the host reference's (every recorded operator's numpy ``reference()``),
``--check-determinism`` counts runs whose logits differ bitwise.  The flags are the
reference's; the ones that choose an NPU packaging (``--full-elf``) have nothing to choose
here and are not taken.  ``--temperature`` / ``--top-k`` draw on the device by the rule of
``iron_b200.lm.generation``; ``--compare-host`` repeats the run drawing on the host.
"""

from __future__ import annotations

import argparse
import inspect
import logging
import time
from pathlib import Path

import numpy as np

from .generation import Sampler

#: Flags the command line and the test fixtures read alike (iron/lm/cli.py:19-42).
FLAGS = (
    (("--random-weights",), dict(type=int, default=None, metavar="SEED",
                                 help="in place of the checkpoint's weights and the tokenizer, weights drawn at "
                                      "SEED in its shapes (only its header is read) and prompts of random tokens")),
    (("--max-seq-len",), dict(type=int, default=None,
                              help="the longest context served, prompt and generated tokens together "
                                   "(default: the checkpoint's max_position_embeddings)")),
)


def parse_args(parser: argparse.ArgumentParser, args=None) -> argparse.Namespace:
    parser.add_argument("-v", "--verbose", action="store_true", help="log iron_b200's INFO lines")
    ns = parser.parse_args(args)
    if ns.verbose:
        logging.basicConfig()
        logging.getLogger("iron_b200").setLevel(logging.INFO)
    return ns


def open_tokenizer(directory: Path):
    """The tokenizer beside a checkpoint (``tokenizer.json``), or None without one."""
    if not (Path(directory) / "tokenizer.json").exists():
        return None
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(str(directory), local_files_only=True)


def random_prompt(vocab_size: int, n: int, seed: int = 0, skip: int = 0) -> list[int]:
    """``n`` token ids drawn at ``seed``, after ``skip`` others of the same stream."""
    return np.random.default_rng(seed).integers(0, vocab_size, skip + n)[skip:].tolist()


def kl_stats(results) -> dict[str, float]:
    kls = np.asarray([kl for kl, _ in results], np.float64)
    return {"Mean": float(kls.mean()), "Max": float(kls.max())}


def _log_softmax(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float64)
    x = x - x.max()
    return x - np.log(np.exp(x).sum())


def accuracy(engine, reference, tokens, steps: int):
    """Per step, KL(reference || device) of the next-token distributions and whether the
    greedy tokens agree; both are fed the reference's greedy token (iron/lm/generation.py)."""
    results = []
    tokens = list(tokens)
    dev = engine.prefill(tokens)
    ref = reference.reference_logits(tokens, 0)
    for step in range(steps):
        lp, lq = _log_softmax(ref), _log_softmax(dev)
        results.append((float((np.exp(lp) * (lp - lq)).sum()), int(np.argmax(ref)) == int(np.argmax(dev))))
        if step == steps - 1:
            break
        nxt, at = int(np.argmax(ref)), len(tokens)
        tokens.append(nxt)
        dev = engine.feed([nxt], at)
        ref = reference.reference_logits([nxt], at)
    return results


def host_draws(engine, tokens, steps: int, sampler) -> list[int]:
    """The ``steps`` tokens drawn on the host from the engine's logits: the prompt, then each
    drawn token fed back (iron/lm/generation.py:102-107 over an incremental model)."""
    logits = engine.prefill(tokens)
    out = []
    for i in range(steps):
        out.append(sampler(logits))
        if i + 1 < steps:
            logits = engine.feed([out[-1]], len(tokens) + i)
    return out


def determinism(engine, prompts, steps: int, rounds: int) -> int:
    """Run each prompt ``rounds`` times, alternating; count the runs whose logits differ
    bitwise from the prompt's first run."""
    first: dict[int, list[np.ndarray]] = {}
    differ = 0
    for _ in range(rounds):
        for i, prompt in enumerate(prompts):
            rows = [engine.prefill(prompt).copy()]
            for t in range(steps - 1):
                engine.feed([int(np.argmax(rows[-1]))], len(prompt) + t)
                rows.append(engine.logits().copy())
            if i not in first:
                first[i] = rows
            else:
                differ += any(not np.array_equal(a.view(np.uint32), b.view(np.uint32)) for a, b in zip(first[i], rows))
    return differ


def main(model_class, args=None, out=print) -> int:
    """The command line of ``model_class`` (a ``CausalLM`` with a ``config_class``)."""
    from .engine import LlamaEngine

    parser = argparse.ArgumentParser(description=f"{model_class.__name__} on a B200")
    parser.add_argument("path", help="a directory holding config.json, the checkpoint and the tokenizer")
    for flags, kwargs in FLAGS:
        parser.add_argument(*flags, **kwargs)
    parser.add_argument("--prompt", metavar="TEXT", help="the text to continue")
    parser.add_argument("--prompt-len", type=int, default=2048,
                        help="without --prompt, a third as many random tokens to prompt with (default: 2048)")
    parser.add_argument("--num-tokens", type=int, default=40, help="tokens to generate (default: 40)")
    defaults = inspect.signature(Sampler).parameters
    parser.add_argument("--temperature", type=float, default=defaults["temperature"].default)
    parser.add_argument("--top-k", type=int, default=defaults["top_k"].default)
    parser.add_argument("--compare-host", action="store_true",
                        help="after drawing on the device, generate again drawing on the host from the same "
                             "seed and count the tokens that differ")
    check = parser.add_mutually_exclusive_group()
    check.add_argument("--check-accuracy", action="store_true",
                       help="instead of sampling, compare each step's logits with the host reference's, "
                            "feeding both the reference's greedy token")
    check.add_argument("--check-determinism", type=int, metavar="ROUNDS",
                       help="instead of sampling, run two prompts ROUNDS times each, alternating, and count "
                            "the runs whose logits differ bitwise")
    ns = parse_args(parser, args)
    if ns.check_determinism is not None and ns.check_determinism < 2:
        parser.error("--check-determinism compares rounds: give 2 or more")
    try:
        Sampler(ns.temperature, ns.top_k).rows(0)
    except ValueError as e:
        parser.error(str(e))
    config_class = getattr(model_class, "config_class", None)
    try:
        engine = LlamaEngine.from_checkpoint(ns.path, random_weights=ns.random_weights,
                                             max_seq_len=ns.max_seq_len, config_class=config_class)
    except ValueError as e:
        parser.error(str(e))
    config = engine.c
    tokenizer = None if ns.random_weights is not None else open_tokenizer(Path(ns.path))
    if ns.prompt is not None:
        if tokenizer is None:
            parser.error("--prompt takes the checkpoint's tokenizer: no --random-weights")
        tokens = tokenizer(ns.prompt)["input_ids"]
    else:
        tokens = random_prompt(config.vocab_size, max(1, ns.prompt_len // 3))
    if len(tokens) + ns.num_tokens > config.max_seq_len:
        parser.error(f"a {len(tokens)}-token prompt and {ns.num_tokens} more exceed {config.max_seq_len} rows")

    if ns.check_accuracy:
        reference = model_class(config, engine.checkpoint.named(
            "read" if ns.random_weights is None else "random", seed=ns.random_weights or 0))
        results = accuracy(engine, reference, tokens, ns.num_tokens)
        worst = int(np.argmax([kl for kl, _ in results]))
        for stat, value in kl_stats(results).items():
            out(f"[Accuracy] {stat} KL: {value:.6f}" + (f" (step {worst})" if stat == "Max" else ""))
        out(f"[Accuracy] Top-1 mismatches: {sum(not t for _, t in results)}")
    elif ns.check_determinism is not None:
        n = len(tokens)
        prompts = [tokens, random_prompt(config.vocab_size, n, skip=n)]
        differ = determinism(engine, prompts, ns.num_tokens, ns.check_determinism)
        out(f"[Determinism] Differing runs: {differ}/{2 * (ns.check_determinism - 1)}")
    else:
        import torch

        # draw rows for the positions this run draws at: the prompt's last row, then each new token's
        engine.set_sampler(Sampler(ns.temperature, ns.top_k), start=len(tokens) - 1, count=ns.num_tokens)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        engine.prefill(tokens)
        ttft = time.perf_counter() - t0
        t1 = time.perf_counter()
        drawn = engine.generate_from_prompt(len(tokens), ns.num_tokens)
        decode_s = time.perf_counter() - t1
        if tokenizer is None:
            out(" ".join(str(t) for t in drawn))
        else:
            out(tokenizer.decode(drawn))
        out(f"\n[Prefill] Time to first token: {ttft:7.3f} s")
        if ns.num_tokens > 1:
            out(f"[Decode]  Tokens per second:   {(ns.num_tokens - 1) / decode_s:7.3f}")
        if ns.compare_host:
            host = host_draws(engine, tokens, ns.num_tokens, Sampler(ns.temperature, ns.top_k))
            differ = sum(a != b for a, b in zip(drawn, host))
            out(f"[Device] Tokens differing from the host loop: {differ}/{len(host)}")
    return 0
