"""Sampling: temperature, then top-k, then a draw from the softmax, the same on host and device.

The reference's ``Sampler`` (iron/lm/generation.py:24-94) delegates its arithmetic --
``sample_ref``, ``sample_weights``, ``draw_row`` -- to mlir-aie, which is not in the reference
tree, so its tie rules and roundings cannot be pinned here.  This module therefore states
its own rule in full, and the device kernel (``iron_sample_rows_bf16``) follows it operation
for operation, so that a host ``Sampler`` and the device draw pick the same token from the
same logits and uniform (the property the reference's class promises):

1. Candidates: the ``k = min(top_k, K_MAX, len)`` largest logits, ordered by value
   (descending, as bf16 bit patterns in the total order -NaN.. < -0 < +0 < ..; NaN ranks
   last) and, among equal values, by index (ascending).
2. Weights, float32, every operation rounded to nearest and none fused:
   ``z = (l_i - l_0) * (log2(e) / T)``; ``n = rint(z)``; ``f = z - n``;
   ``w = poly7(f) * 2**n`` with ``poly7`` the degree-7 Taylor polynomial of ``2**f``
   (Horner, multiply then add); ``w = 0`` once ``n < -120``; a ``z`` that is not ``>= -1000`` (a NaN
   too) is taken as ``-1000``.
3. The draw: ``u = n53 * 2**-53`` for a 53-bit integer ``n53`` (what ``Generator.random()``
   holds); the weights are summed in float64 in rank order; the token is the first
   candidate whose running sum exceeds ``u * total`` (the last one if rounding leaves none).

``temperature == 0`` (or ``top_k == 1``) is the greedy draw: the first index of the largest
logit.  A draw row is ``ROW_WORDS`` int32: temperature bits, top_k, the low 32 and the high
21 bits of ``n53``; an all-zero row is greedy.
"""

from __future__ import annotations

import math

import numpy as np
from ml_dtypes import bfloat16

#: Seeds the sampler, so a run's text is reproducible (iron/lm/generation.py:21).
SEED = 1608560892
ROW_WORDS = 4
#: The device's largest top-k.
K_MAX = 64

_F = np.float32
_LOG2E = _F(1.4426950408889634)
#: (ln 2)**k / k! for k = 7 .. 0, rounded to float32 once.
POLY7 = tuple(_F(math.log(2.0) ** k / math.factorial(k)) for k in range(7, -1, -1))


def ordered_keys(logits) -> np.ndarray:
    """bf16 logits as uint16 keys whose integer order is the value order (NaN lowest)."""
    bits = np.asarray(logits).astype(bfloat16).reshape(-1).view(np.uint16)
    keys = np.where(bits & 0x8000, ~bits, bits | 0x8000).astype(np.uint16)
    nan = (bits & 0x7FFF) > 0x7F80
    return np.where(nan, np.uint16(0), keys)


def candidates(logits, k: int) -> np.ndarray:
    """Indices of the ``k`` largest logits: value descending, then index ascending."""
    keys = ordered_keys(logits).astype(np.int64)
    order = np.lexsort((np.arange(keys.size), -keys))
    return order[:k]


def exp2_det(z: np.ndarray) -> np.ndarray:
    """``2**z`` for ``z <= 0`` by rule 2: float32, round to nearest, nothing fused."""
    z = np.asarray(z, _F)
    z = np.where(z >= _F(-1000), z, _F(-1000)).astype(_F)   # also what a NaN becomes
    n = np.rint(z).astype(_F)
    f = (z - n).astype(_F)
    p = np.full(z.shape, POLY7[0], _F)
    for c in POLY7[1:]:
        p = (p * f).astype(_F)
        p = (p + c).astype(_F)
    w = np.ldexp(p, n.astype(np.int32)).astype(_F)
    return np.where(n < _F(-120), _F(0), w).astype(_F)


def sample_weights(logits, temperature, top_k: int):
    """The candidates (rule 1) and their float32 weights (rule 2)."""
    logits = np.asarray(logits).astype(bfloat16).reshape(-1)
    k = max(1, min(int(top_k), K_MAX if top_k is not None else logits.size, logits.size))
    cand = candidates(logits, k)
    vals = logits[cand].astype(_F)
    c = _F(_LOG2E / _F(temperature))
    with np.errstate(invalid="ignore"):   # inf - inf, or a NaN logit: rule 2 makes them -1000
        z = ((vals - vals[0]).astype(_F) * c).astype(_F)
    return cand, exp2_det(z)


def sample_ref(logits, temperature, top_k: int, n53: int) -> int:
    """The token rules 1-3 pick from one row of logits."""
    logits = np.asarray(logits).reshape(-1)
    if float(temperature) == 0.0 or top_k == 1:
        return int(candidates(logits, 1)[0])
    cand, w = sample_weights(logits, temperature, top_k)
    w64 = w.astype(np.float64)
    total = np.float64(0.0)
    for x in w64:
        total = total + x
    target = np.float64(n53) * np.float64(2.0 ** -53) * total
    acc = np.float64(0.0)
    for i, x in enumerate(w64):
        acc = acc + x
        if target < acc:
            return int(cand[i])
    return int(cand[-1])


def draw_row(temperature, top_k: int, n53: int) -> np.ndarray:
    """One device draw: temperature bits, top_k, the uniform's low 32 and high 21 bits."""
    row = np.empty(ROW_WORDS, np.uint32)
    row[0] = np.asarray(temperature, _F).view(np.uint32)
    row[1] = top_k
    row[2] = n53 & 0xFFFFFFFF
    row[3] = n53 >> 32
    return row.view(np.int32)


class Sampler:
    """Temperature, then top-k, then a draw from the softmax, exactly as the device draws
    (iron/lm/generation.py:24-94; the arithmetic is this module's, see its docstring).

    ``top_k`` None keeps the whole row, on the host only: the device's top-k is bounded.
    """

    def __init__(self, temperature: float = 0.7, top_k: int | None = 50, seed: int = SEED):
        if temperature < 0:
            raise ValueError(f"temperature {temperature} is negative")
        if top_k is not None and top_k < 1:
            raise ValueError(f"top_k {top_k} keeps no token")
        self.temperature = _F(temperature)
        self.top_k = top_k
        self.rng = np.random.default_rng(seed)

    def _top_k(self, size: int) -> int:
        return size if self.top_k is None else self.top_k

    def _n53(self) -> int:
        # random() is n53 * 2^-53 for the generator's next 53 bits, exactly
        return int(self.rng.random() * 2.0 ** 53)

    def probabilities(self, logits) -> np.ndarray:
        """The distribution a token is drawn from, float64, over ``logits`` (1-D)."""
        size = np.asarray(logits).size
        probs = np.zeros(size, np.float64)
        if self.temperature == 0:
            probs[sample_ref(logits, self.temperature, 1, 0)] = 1.0
            return probs
        if self.top_k is None:
            cand = candidates(logits, size)
            vals = np.asarray(logits).astype(bfloat16).reshape(-1)[cand].astype(_F)
            w = exp2_det(((vals - vals[0]).astype(_F) * _F(_LOG2E / self.temperature)).astype(_F))
        else:
            cand, w = sample_weights(logits, self.temperature, self.top_k)
        probs[cand] = w.astype(np.float64) / w.astype(np.float64).sum()
        return probs

    def __call__(self, logits) -> int:
        """One token id drawn from a row of logits (any shape of one row)."""
        n53 = self._n53()
        if self.top_k is None and self.temperature != 0:
            p = self.probabilities(logits)
            order = candidates(logits, p.size)
            acc = np.cumsum(p[order])
            return int(order[min(int(np.searchsorted(acc, n53 * 2.0 ** -53 * acc[-1], side="right")), p.size - 1)])
        return sample_ref(logits, self.temperature, self._top_k(np.asarray(logits).size), n53)

    def rows(self, count: int, k_max: int = K_MAX) -> np.ndarray:
        """``count`` draws for the device, ``(count, ROW_WORDS)`` int32, one per position, taking
        the uniforms ``count`` host draws would, in order.  ``top_k`` must be one the device
        draws (1..``k_max``): it would be clamped, not honoured, otherwise."""
        if self.top_k is None or self.top_k > k_max:
            raise ValueError(f"top_k {self.top_k} is not one the device draws (1..{k_max})")
        rows = np.empty((count, ROW_WORDS), np.int32)
        for i in range(count):
            rows[i] = draw_row(self.temperature, self.top_k, self._n53())
        return rows


def greedy(logits) -> int:
    """The id of the largest of ``logits`` (the first of equals)."""
    return int(np.argmax(np.asarray(logits, np.float32).reshape(-1)))


def generate_on_host(model, tokens, num_tokens: int, sample) -> list[int]:
    """The ``num_tokens`` drawn after ``tokens``, each from ``model.logits(history)``."""
    history = [int(t) for t in tokens]
    for _ in range(num_tokens):
        history.append(sample(model.logits(history)))
    return history[-num_tokens:]
