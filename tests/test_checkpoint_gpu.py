"""A checkpoint directory through ``from_checkpoint`` and the command line (B200)."""

import dataclasses
import json

import numpy as np
import pytest

from iron_b200.lm import save_file
from oracle import model as M
from tests.test_engine_gpu import toy_config

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def directory(tmp_path_factory):
    """``config.json`` and ``model.safetensors`` of the scaled-down Llama at the pinned draw."""
    d = tmp_path_factory.mktemp("llama-small")
    (d / "config.json").write_text(json.dumps(toy_config().to_json()))
    save_file(M.filled_random(M.llama_shapes(M.SCALED), 0), d / "model.safetensors", {"format": "pt"})
    return d


def test_from_checkpoint_gives_the_engine_the_files_weights(directory):
    from iron_b200.lm.engine import LlamaEngine

    prompt = np.random.default_rng(7).integers(0, 1024, 24)
    want = LlamaEngine(toy_config(), M.filled_random(M.llama_shapes(M.SCALED), 0)).prefill(prompt)
    engine = LlamaEngine.from_checkpoint(directory)
    assert dataclasses.asdict(engine.c) == dataclasses.asdict(toy_config())
    assert np.array_equal(engine.prefill(prompt).view(np.uint32), want.view(np.uint32))
    assert engine.uploaded_bytes > 2 * sum(int(np.prod(s)) for s in M.llama_shapes(M.SCALED).values()) * 0.99
    # the mapped file is still readable after its pages were dropped behind the copies
    assert engine.checkpoint.fingerprint() == type(engine.checkpoint)(directory / "model.safetensors").fingerprint()
    # a seed in place of the weights: the same shapes, other logits; the context only shrinks
    other = LlamaEngine.from_checkpoint(directory, random_weights=3, max_seq_len=64)
    assert other.c.max_seq_len == 64 and not np.array_equal(other.prefill(prompt), want)
    with pytest.raises(ValueError, match="past the checkpoint's 256"):
        LlamaEngine.from_checkpoint(directory, max_seq_len=512)


def test_the_command_line_samples_and_checks_itself(directory, capsys):
    from iron_b200.applications.llama.model import Llama
    from iron_b200.lm.cli import main

    lines = []
    assert main(Llama, [str(directory), "--prompt-len", "48", "--num-tokens", "6", "--temperature", "0"],
                out=lines.append) == 0
    drawn = [int(t) for t in lines[0].split()]
    assert len(drawn) == 6 and all(0 <= t < 1024 for t in drawn)
    assert "[Prefill] Time to first token" in lines[1] and "[Decode]  Tokens per second" in lines[2]
    # the tokens are the greedy continuation the engine gives through its own API
    from iron_b200.lm.cli import random_prompt
    from iron_b200.lm.engine import LlamaEngine

    assert LlamaEngine.from_checkpoint(directory).complete(random_prompt(1024, 16), 6) == drawn

    # temperature and top-k on the device, then the same draws on the host from the same seed
    lines.clear()
    main(Llama, [str(directory), "--prompt-len", "48", "--num-tokens", "12", "--temperature", "0.9", "--top-k", "40",
                 "--compare-host"], out=lines.append)
    sampled = [int(t) for t in lines[0].split()]
    assert len(sampled) == 12 and sampled != drawn + sampled[6:]
    assert lines[-1] == "[Device] Tokens differing from the host loop: 0/12"

    lines.clear()
    main(Llama, [str(directory), "--prompt-len", "24", "--num-tokens", "4", "--check-accuracy"], out=lines.append)
    mean = float(lines[0].split("KL:")[1].split()[0])
    assert lines[0].startswith("[Accuracy] Mean KL") and 0 <= mean < 1e-2
    assert lines[2] == "[Accuracy] Top-1 mismatches: 0"

    lines.clear()
    main(Llama, [str(directory), "--random-weights", "5", "--prompt-len", "24", "--num-tokens", "3",
                 "--check-determinism", "3"], out=lines.append)
    assert lines == ["[Determinism] Differing runs: 0/4"]

    with pytest.raises(SystemExit):
        main(Llama, [str(directory), "--prompt", "hello"])          # no tokenizer beside this checkpoint
    assert "--prompt takes the checkpoint's tokenizer" in capsys.readouterr().err
    with pytest.raises(SystemExit):
        main(Llama, [str(directory), "--prompt-len", "600", "--num-tokens", "100"])
    assert "exceed 256 rows" in capsys.readouterr().err
