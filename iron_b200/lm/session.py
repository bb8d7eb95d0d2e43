"""One conversation over a causal model's versions (iron/lm/session.py:25-193).

A session remembers which tokens the model's caches hold.  ``logits(history)`` then runs only
what is new: one more token than last time is a decode step; anything else restarts from the
first token the caches do not hold -- or, where a layer carries a recurrent state that can only
be re-entered at a prompt-chunk boundary (a Mamba2 mixer's ``Checkpoints``), from the boundary
before it.  Several sessions may share one model; its caches hold one session's tokens at a
time, so a session another one displaced runs its history again from the first token.  Token ids
outside the vocabulary and histories longer than the caches are refused before anything is
dispatched, so a refused call leaves the caches as they were.
"""

from __future__ import annotations

from typing import Iterator

import numpy as np

from .generation import Sampler

NOTHING = np.empty(0, dtype=np.int64)


class Session:
    """A conversation over ``lm``, a ``CausalLM``."""

    def __init__(self, lm):
        self.lm = lm
        self._seen = NOTHING        # the tokens the caches hold for this session

    # ---- what the caches hold ----
    def _take(self) -> None:
        if self.lm.holder is not self:   # what another session left there is none of this one's
            self.lm.holder, self._seen = self, NOTHING

    def _tokens(self, tokens) -> np.ndarray:
        tokens = np.asarray(tokens, dtype=np.int64).reshape(-1)
        V = self.lm.config.vocab_size
        bad = (tokens < 0) | (tokens >= V)
        if bad.any():
            raise IndexError(f"tokens {tokens[bad]} are outside [0, {V})")
        return tokens

    def _held(self, tokens: np.ndarray) -> int:
        """How many leading tokens of ``tokens`` the caches hold; never the last one."""
        n = min(tokens.size - 1, self._seen.size)
        differ = np.flatnonzero(tokens[:n] != self._seen[:n])
        return int(differ[0]) if differ.size else n

    def resume(self, held: int) -> int:
        """Where calls start so that the tokens from ``held`` on are run: ``held`` itself, or
        the earliest restart point among the model's recurrent states."""
        ran = self._seen.size
        return min([held, *(state.restart(held, ran) for state in self.lm.recurrent)])

    def forget(self, position: int) -> None:
        """Hold nothing from ``position`` on: the next call runs from there, or from the restart
        boundary before it."""
        held = self._seen[:position].size
        self._seen = self._seen[: self.resume(held)]

    # ---- running ----
    def _chunks(self, tokens: np.ndarray, start: int):
        """Each prompt call from ``start``: (ids padded to the chunk, per-call values).  With a
        recurrent state a call ends at the next chunk boundary."""
        n, C = tokens.size, self.lm.config.prefill_chunk
        end = start
        while end < n:
            begin, end = end, min(end + C, n)
            if self.lm.recurrent:
                end = min(end, (begin // C + 1) * C)
            ids = np.zeros(C, dtype=np.int32)
            ids[: end - begin] = tokens[begin:end]
            yield ids, dict(position=end - 1, start=begin, rows=end - begin)

    def logits(self, tokens) -> np.ndarray:
        """Float32 logits after the last of ``tokens``, the whole history."""
        tokens = self._tokens(tokens)
        n, L = tokens.size, self.lm.config.max_seq_len
        if not 0 < n <= L:
            raise ValueError(f"{n} tokens do not fit {L} rows")
        self._take()
        held = self._held(tokens)
        if held == n - 1 == self._seen.size:
            out, _ = self.lm.call_version(token=int(tokens[-1]), position=n - 1)
        else:
            start = self.resume(held)
            self._seen = tokens[:start]
            out = None
            for ids, values in self._chunks(tokens, start):
                out, _ = self.lm.call_version(ids, **values)
        self._seen = tokens
        return np.array(out, np.float32).reshape(-1)[: self.lm.config.vocab_size]

    def draw(self, tokens, max_tokens: int, sampler: Sampler | None = None) -> Iterator[int]:
        """``max_tokens`` tokens drawn after ``tokens``, each yielded as it is drawn: the draw
        happens on the device (or in the host graph's ``Sample`` step) from the draw rows the
        sampler's uniforms fill, the token carried into the next decode step."""
        tokens = self._tokens(tokens)
        n, L = tokens.size, self.lm.config.max_seq_len
        if not (0 < n and 0 < max_tokens and n + max_tokens - 1 <= L):
            raise ValueError(f"{n} tokens and {max_tokens} more to draw do not fit {L} rows")
        self._take()
        self.lm.write_draws(n - 1, max_tokens, sampler)
        start = self.resume(self._held(tokens))
        self._seen = NOTHING        # a caller may stop early: until the end the caches hold nothing known
        carried = None
        for ids, values in self._chunks(tokens, start):
            _, carried = self.lm.call_version(ids, **values)
        drawn = [int(carried["token"])]
        yield drawn[-1]
        for _ in range(max_tokens - 1):
            _, carried = self.lm.call_version(**carried)
            drawn.append(int(carried["token"]))
            yield drawn[-1]
        self._seen = np.concatenate([tokens, drawn[:-1]]).astype(np.int64)   # the last drawn was never run
