"""Sample (iron/operators/sample.py:106): the token drawn from a row of logits.

An all-zero draw row is greedy (iron/lm/generation.py:97-99): the first index of the largest
logit.  A non-zero row (temperature bits, top_k, a 53-bit uniform) draws by the rule of
``iron_b200.lm.generation``: the reference's own arithmetic (``sample_ref``) is mlir-aie's and
not in its tree, so the rule is this package's, the same on host and device.
"""

import numpy as np

from ..declare import In, InOut, Operator, Out, param, per_call
from ..testing import Case, Testing
from ..verify import Tolerance

from ..lm.generation import ROW_WORDS, draw_row, sample_ref  # noqa: E402  (row: temperature bits, top_k, uniform lo / hi)


def _rows(op) -> np.ndarray:
    """Greedy rows for the default cases; the third case draws at temperature 0.7, top-k 50."""
    rows = np.zeros(op.draws.shape, np.int32)
    if op.vocab == 32000:
        rng = np.random.default_rng(4)
        for r in range(op.rows):
            rows[r] = draw_row(0.7, 50, int(rng.integers(0, 2 ** 53)))
    return rows


class Sample(Operator):
    """``drawn[at]`` = the token draw row ``row`` picks from ``logits[:drawable]``."""

    test = Testing([Case(dict(vocab=1024, rows=16)), Case(dict(vocab=128256, rows=8), bench=True),
                    Case(dict(vocab=32000, rows=4), id="temperature_top_k")],
                   draw=lambda op: dict(centered=(op.logits,),
                                        given={op.draws: _rows(op),
                                               op.drawn: np.zeros(op.drawn.shape, np.int32)}))

    vocab: int = param()
    rows: int = param()
    drawable: int = param(default=lambda op: op.vocab)

    logits = In(vocab)
    draws = In(rows, ROW_WORDS, dtype=np.int32)
    drawn = InOut(rows, dtype=np.int32)
    row = per_call()
    at = per_call()

    def __getattr__(self, name):
        if name in ("row", "at"):
            return self.__dict__.get("bound_extents", {}).get(name, 0)
        return super().__getattr__(name)

    def ops(self) -> int:
        return self.vocab

    def reference(self, logits, draws, drawn):
        row = np.asarray(draws).reshape(-1, ROW_WORDS)[self.row].view(np.uint32)
        out = np.array(drawn, np.int32)
        out[self.at] = sample_ref(np.asarray(logits)[: self.drawable], row[:1].view(np.float32)[0], int(row[1]),
                                  int(row[2]) | (int(row[3]) << 32))
        return out

    def tolerance(self):
        return Tolerance.exact(note="a token id")

    def launch(self, buffers, values):
        import torch

        from .. import kernels as K

        logits, draws, drawn = buffers["logits"], buffers["draws"], buffers["drawn"]
        dev = logits.device

        def index(name, host):
            v = values.get(f"d_{name}")
            # a fill, not a copy from the host: this may run inside a stream capture
            return torch.full((1,), int(host), dtype=torch.int32, device=dev) if v is None else v

        row, at = index("row", self.row), index("at", self.at)
        # the kernel reads the draw row at the position it writes: put row `row` at `at`
        table = torch.zeros_like(draws).view(-1, ROW_WORDS)
        table.index_copy_(0, at.long(), draws.view(-1, ROW_WORDS).index_select(0, row.long()))
        token = torch.empty(1, dtype=torch.int32, device=dev)
        K.sample_rows(logits[: self.drawable], table, token, at.clone(), drawn.view(1, -1))
