"""Copy the reference's recorded float32 Hugging Face logits into ``tests/golden/``.

Run once in a container that has the reference tree mounted; the GPU box has no copy of
it, so the rows travel as this small fixture.  The rows are data the reference's own
tests judge by (iron/tests/common/goldens/small.npz, keyed by sha256 of the int64 token
ids, iron/lm/golden.py:88-92): the toy ``SCALED`` Llama on ``filled("random", seed 0)``
weights, prompt ``default_rng(7).integers(0, 1024, 8)`` then six greedy steps, and the
multi-chunk prompts of seeds 3 and 4 (iron/tests/support/llama_reference.py:134, :219-224).
The other three files are the same rows for the reference's other toy decoders: Llama with
projection biases (prompt seed 1), Granite with its four scalars (seed 0) and the Granite
4.0-H hybrid with three Mamba2 layers (seed 2), the only fixture of the reference that pins
the selective scan and the causal convolution through a model.

    python tests/golden/make_golden.py <path to the reference checkout>
"""

import sys
from pathlib import Path

import numpy as np

SOURCES = {
    "llama_small.npz": "iron/tests/common/goldens/small.npz",
    "llama_biased.npz": "tests/applications/llama/reference/goldens/biased.npz",
    "granite_toy.npz": "tests/applications/granite/reference/goldens/toy.npz",
    "granite_hybrid_dense.npz": "tests/applications/granite_hybrid/reference/goldens/dense.npz",
}


def main(reference: str) -> None:
    here = Path(__file__).resolve().parent
    for name, rel in SOURCES.items():
        with np.load(Path(reference) / rel) as z:
            rows = {k: z[k] for k in z.files}
        np.savez_compressed(here / name, **rows)
        print(name, len(rows), "rows")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
