"""Sample (iron/operators/sample.py:106): the token drawn from a row of logits.

Only the greedy draw is exact here: an all-zero draw row is greedy in the reference
(iron/lm/generation.py:97-99), and greedy is the first index of the largest logit.
Temperature / top-k draws follow mlir-aie's ``sample_ref`` tie rules, which are not in the
reference tree; a non-zero draw row is refused.
"""

import numpy as np

from ..declare import In, InOut, Operator, Out, param, per_call
from ..testing import Case, Testing
from ..verify import Tolerance

ROW_WORDS = 4  # temperature bits, top_k, 53-bit uniform lo / hi


class Sample(Operator):
    """``drawn[at] = argmax(logits[:drawable])`` for a greedy draw row."""

    test = Testing([Case(dict(vocab=1024, rows=16)), Case(dict(vocab=128256, rows=8), bench=True)],
                   draw=lambda op: dict(centered=(op.logits,),
                                        given={op.draws: np.zeros(op.draws.shape, np.int32),
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
        if np.asarray(draws).reshape(-1, ROW_WORDS)[self.at].any():
            raise NotImplementedError("only the greedy draw (an all-zero draw row) is defined here")
        out = np.array(drawn, np.int32)
        out[self.at] = int(np.argmax(np.asarray(logits[: self.drawable], np.float32)))
        return out

    def tolerance(self):
        return Tolerance.exact(note="a token id")

    def launch(self, buffers, values):
        import torch

        from .. import kernels as K

        ws = K.argmax_workspace(buffers["logits"].device)
        at = values.get("d_at")
        if at is None:
            at = torch.tensor([self.at], dtype=torch.int32, device=buffers["logits"].device)
        K.argmax(buffers["logits"][: self.drawable], buffers["drawn"], ws, d_out_index=at)
