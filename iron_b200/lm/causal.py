"""``CausalLM``: a decoder and its head as one graph with two versions
(iron/lm/causal.py:166-400): the decode step (no inputs: the token and position are
per-call values) and the prompt chunk (``ids`` of ``prefill_chunk`` int32, bounded per call
by ``rows``).  Both write the same KV-cache states.

``logits(tokens)`` runs the compiled versions on the device; ``reference_logits(tokens)``
runs the same recordings on the host with every operator's numpy reference (the
reference's ``OnHost``, iron/lm/model.py:667-695); ``engine()`` returns the fused decoder
the same weights run on when throughput matters.
"""

from __future__ import annotations

import numpy as np
from ml_dtypes import bfloat16

import dataclasses

from .. import functional as F
from ..graph import Carried, Graph, Scratchpad, carry, param, state, walk
from ..graph.handle import State
from ..operators.copy import Copy
from ..operators.sample import ROW_WORDS, Sample
from .blocks import Call, DecoderLayer, Embedding, Linear, RMSNorm, Rope
from .config import DecoderConfig


@dataclasses.dataclass(frozen=True)
class Checkpoints:
    """A state carried from position to position, one slot per prompt-chunk boundary
    (iron/lm/causal.py:71-121): slot ``k`` holds it after the first ``k * chunk`` positions
    (or the positions run so far, for the chunk in progress); slot 0, never written, is the
    state before the sequence.  A call reads the slot before its first position and writes
    the slot after its last, so a sequence can restart at any chunk boundary."""

    slots: State
    chunk: int

    @classmethod
    def of(cls, shape, max_seq_len: int, chunk: int, dtype=bfloat16) -> "Checkpoints":
        if chunk < 1 or chunk & (chunk - 1):
            raise ValueError(f"Checkpoints: a {chunk}-position chunk is no power of two")
        return cls(state(((max_seq_len - 1) // chunk + 2, *shape), dtype), chunk)

    def at(self, call: Call):
        """(the slot ``call`` reads, the slot it writes), inside a body."""
        C = self.chunk
        return self.slots[(call.start - 1) // C + 1], self.slots[call.position // C + 1]

    def restart(self, held: int, ran: int) -> int:
        """Where a call may start so that the positions from ``held`` on change, after ``ran``
        ran: where the last call ended, else the chunk boundary before ``held``."""
        return held if held == ran else held // self.chunk * self.chunk

    def slot(self, position: int) -> int:
        """The slot holding the state after the first ``position`` positions."""
        return 0 if position == 0 else (position - 1) // self.chunk + 1


class CausalConv1d(Graph):
    """A depth-wise causal convolution of ``kernel`` taps over a call's rows
    (iron/lm/causal.py:124-163): ``weight`` as torch stores it, ``(channels, 1, kernel)``,
    an optional ``bias``, and the ``kernel - 1`` rows before a call as ``state``, a slot per
    prompt-chunk boundary."""

    def __init__(self, c, channels: int, kernel: int, bias: bool = False):
        if c.prefill_chunk < kernel - 1:
            raise ValueError(f"CausalConv1d: prefill_chunk {c.prefill_chunk} is smaller than "
                             f"kernel - 1 ({kernel - 1})")
        self.weight = param(channels, 1, kernel)
        self.bias = param(channels) if bias else None
        self.state = Checkpoints.of((kernel - 1, channels), c.max_seq_len, c.prefill_chunk)
        self.taps = None

    def load_state_dict(self, tree, *, path: str = "") -> None:
        super().load_state_dict(tree, path=path)
        C, _, K = self.weight.shape   # one row per tap
        self.taps = param(np.ascontiguousarray(np.asarray(self.weight).reshape(C, K).T))

    def body(self, x, call: Call):
        read, write = self.state.at(call)
        y = F.causal_conv1d(x, self.taps, F.ConvState(read, write))
        return y if self.bias is None else y + self.bias


class Decoder(Graph):
    def __init__(self, c: DecoderConfig, layer_class=DecoderLayer):
        self.embed_tokens = Embedding(c.vocab_size, c.hidden_size)
        self.layers = [layer_class(c, i) for i in range(c.num_hidden_layers)]
        self.norm = RMSNorm(c.hidden_size, c.eps)


class CausalLM(Graph):
    """A causal language model on ``config``'s shape and a checkpoint's ``weights`` (by name)."""

    layer_class = DecoderLayer

    def __init__(self, config: DecoderConfig, weights: dict):
        self.config = config
        self.rotary_emb = None if config.rope_theta is None else Rope(config)
        self.draws = state((config.max_seq_len, ROW_WORDS), np.int32)
        self.drawn = state((config.max_seq_len,), np.int32)
        self.model = Decoder(config, self.layer_class)
        for layer in self.model.layers:
            layer.rope = self.rotary_emb
        self.lm_head = Linear(config.hidden_size, config.vocab_size, False, precision=config.precision)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.load_state_dict(weights)
        self._weights = weights
        # the session whose tokens the caches hold, and the one ``history_logits`` / ``generate`` run in
        from .session import Session

        self.holder = None
        self.session = Session(self)

    def body(self, ids=None, *, token: Carried[np.int32] = np.int32(0), position: Carried[np.int32] = np.int32(0),
             start: Scratchpad[np.int32] = np.int32(0), rows: Scratchpad[np.int32] = np.int32(1)):
        c = self.config
        prompt = ids is not None
        call = Call(prompt=prompt, start=start if prompt else position, rows=rows, position=position,
                    ids=ids[:rows] if prompt else token, token=token)
        x = self.lookup(call.ids) if prompt else self.lookup(token).reshape(1, c.hidden_size)
        if self.rotary_emb is not None:
            call.ropes[self.rotary_emb] = self.rotary_emb.rows(call)
        for layer in self.model.layers:
            x = layer(x, call)
        if prompt:
            x = Copy.step(x[rows - 1]).reshape(1, c.hidden_size)   # the last row's logits alone
        logits = self.head(x)
        drawn = Sample.step(logits.reshape(c.vocab_size), self.draws, self.drawn, row=position, at=position,
                            vocab=c.vocab_size)
        return logits, carry(token=drawn[position], position=position + 1)

    def lookup(self, ids):
        """The embedding rows of ``ids`` (bounded as ``ids`` is), or of the decode step's token
        (iron/lm/causal.py:262-268); a model that scales its embedding overrides it."""
        if hasattr(ids, "shape") and len(ids.shape) == 1:
            return self.model.embed_tokens(ids)
        return Copy.step(self.model.embed_tokens.weight[ids])

    def head(self, x):
        """The final norm, then the output head (iron/lm/causal.py:253-255)."""
        return self.lm_head(self.model.norm(x))

    # ---- running ----
    def shapes(self) -> list[dict]:
        return [{}, dict(ids=((self.config.prefill_chunk,), np.int32))]

    def _chunks(self, n: int, start: int):
        C = self.config.prefill_chunk
        s = start
        while s < start + n:
            e = min(start + n, (s // C + 1) * C)
            yield s, e
            s = e

    def _run(self, tokens, start: int, on_host: bool):
        c = self.config
        tokens = np.asarray(tokens).reshape(-1)
        if start + len(tokens) > c.max_seq_len:
            raise IndexError(f"{start + len(tokens)} positions do not fit the {c.max_seq_len}-row caches")
        out = None
        if len(tokens) == 1:
            kw = dict(token=int(tokens[0]), position=start)
            out = self.reference(**kw) if on_host else self.compile()(**kw)
        else:
            C = c.prefill_chunk
            for s, e in self._chunks(len(tokens), start):
                ids = np.zeros(C, np.int32)
                ids[: e - s] = tokens[s - start : e - start]
                kw = dict(position=e - 1, start=s, rows=e - s)
                out = self.reference(ids, **kw) if on_host else self.compile(ids=((C,), np.int32))(ids, **kw)
        logits, carried = out
        logits = logits if isinstance(logits, np.ndarray) else logits.numpy()
        return np.asarray(logits, np.float32).reshape(-1), carried

    #: ``OnHost`` turns this on: the versions are stood in by the graph's host reference
    on_host = False

    @property
    def recurrent(self) -> list:
        """Each state a layer carries from position to position that restarts only at some
        positions (iron/lm/causal.py:229-243): the mixers' ``Checkpoints``."""
        found = {}
        for layer in self.model.layers:
            for _, value in self._walk_checkpoints(layer):
                found.setdefault(id(value), value)
        return list(found.values())

    @staticmethod
    def _walk_checkpoints(node, seen=None):
        seen = set() if seen is None else seen
        if id(node) in seen:
            return
        seen.add(id(node))
        if isinstance(node, Checkpoints):
            yield None, node
            return
        children = []
        if isinstance(node, Graph):
            children = [v for k, v in vars(node).items() if not k.startswith("_")]
        elif isinstance(node, (list, tuple)):
            children = list(node)
        for child in children:
            if isinstance(child, (Graph, Checkpoints, list, tuple)):
                yield from CausalLM._walk_checkpoints(child, seen)

    def call_version(self, ids=None, **values):
        """Run one call -- the prompt chunk when ``ids`` is given, else the decode step -- on the
        device (compiled versions) or on the host (``on_host``); ``(float32 logits, carried)``."""
        if self.on_host:
            logits, carried = self.reference(ids, **values) if ids is not None else self.reference(**values)
        elif ids is not None:
            logits, carried = self.compile(ids=((self.config.prefill_chunk,), np.int32))(ids, **values)
        else:
            logits, carried = self.compile()(**values)
        logits = logits if isinstance(logits, np.ndarray) else logits.numpy()
        return np.asarray(logits, np.float32).reshape(-1), carried

    def write_draws(self, first: int, count: int, sampler) -> None:
        """Fill the draw rows of positions ``first .. first + count`` from ``sampler``'s
        uniforms (rows of zeros draw greedily), as iron/lm/session.py:83-92 writes them."""
        rows = np.zeros((self.config.max_seq_len, ROW_WORDS), np.int32)
        if sampler is not None and sampler.temperature != 0:
            rows[first : first + count] = sampler.rows(count)
        if self.on_host:
            self.draws.host = rows.reshape(-1).copy()
        else:
            for version in self.__dict__.get("_versions", {}).values():
                version.write(self.draws, rows)
            if not self.__dict__.get("_versions"):
                self.compile().write(self.draws, rows)

    def history_logits(self, tokens) -> np.ndarray:
        """Logits after the whole history ``tokens``, running only what the caches do not hold
        (``Session.logits``)."""
        return self.session.logits(tokens)

    def generate(self, tokens, max_tokens: int, sampler=None) -> list[int]:
        """``max_tokens`` tokens drawn after ``tokens`` (greedy without a sampler)."""
        return list(self.session.draw(tokens, max_tokens, sampler))

    def stream(self, tokens, max_tokens: int, sampler=None):
        """``generate`` as an iterator, each token yielded as it is drawn."""
        return self.session.draw(tokens, max_tokens, sampler)

    def forget(self, position: int) -> None:
        self.session.forget(position)

    def logits(self, tokens, start: int = 0) -> np.ndarray:
        """Float32 logits after the last of ``tokens`` run at positions ``start...`` on the device."""
        return self._run(tokens, start, on_host=False)[0]

    def reference_logits(self, tokens, start: int = 0) -> np.ndarray:
        """The same on the host: every recorded step's numpy reference."""
        return self._run(tokens, start, on_host=True)[0]

    def engine(self, **kwargs):
        """The fused decoder on the same weights (five kernels a layer, one CUDA graph a step)."""
        from .engine import LlamaEngine

        return LlamaEngine(self.config, self._weights, **kwargs)


class OnHost:
    """A model with its versions stood in by its graph's host reference (iron/lm/model.py:667-695):
    mixed in before the model's own class, it compiles nothing and needs no GPU --

        class HostLlama(OnHost, Llama): pass
    """

    on_host = True

    def logits(self, tokens, start: int | None = None) -> np.ndarray:
        """With ``start``: the tokens run at those positions; without: the whole history, resuming
        from what the caches hold (``Session.logits``), as the reference's ``Model.logits`` does."""
        if start is None:
            return self.session.logits(tokens)
        return self._run(tokens, start, on_host=True)[0]
