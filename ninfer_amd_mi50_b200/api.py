"""The Python entry point, in the manner of the reference's ctypes wrapper.

The reference's ``tools/ninfer_ctypes.py`` exposes ``Ninfer(model_dir, max_context,
prefill_chunk, num_sequences, ...)`` with ``tokenize / detokenize / session() /
decode_batch(sessions, tokens) / sample(...) / close()`` and ``Session`` with
``prefill(tokens) / decode(token) / reset() / slot / length / close()`` over the C API of
``src/api/ninfer_c_api.h:32-82``.  Names, argument order, defaults and meanings are kept
(``gpus``, ``quant`` and ``parallel`` are gone: one GPU, no quantisation); logits come back
as NumPy float32 arrays instead of Python lists.  Added: ``step`` (a mixed batch with
chosen logit rows), ``generate`` (the scheduler), ``stats``, ``pages_free``.

    from ninfer_amd_mi50_b200.api import Ninfer
    eng = Ninfer("/path/to/Qwen1.5-MoE-A2.7B", num_sequences=4)
    with eng.session() as s:
        logits = s.prefill(ids)
        tok = eng.sample(logits, temperature=0.7)
        logits = s.decode(tok)
"""

from __future__ import annotations

import itertools
from typing import Any, Dict, Iterable, List, Optional, Sequence

import numpy as np
import torch

from .config.engine_options import EngineOptions
from .engine.batch import StepEntry
from .engine.engine import Engine
from .sampling.params import SamplingParams
from .sampling.sampler import sample_reference, uniform_draw


class NinferError(RuntimeError):
    pass


class Session:
    """One request's place in the cache: a state slot, pages, a length."""

    def __init__(self, engine: "Ninfer", key: int):
        self._engine, self._key = engine, key
        self._open = True
        engine._runner.open(key)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def slot(self) -> int:
        return self._engine._runner.cache.slot(self._key)

    @property
    def length(self) -> int:
        return self._engine._runner.cache.length(self._key)

    def reset(self) -> None:
        """Forget everything; pages go back to the pool (``ninfer_session_reset``)."""
        r = self._engine._runner
        r.close(self._key)
        r.open(self._key)

    def prefill(self, tokens: Sequence[int]) -> np.ndarray:
        """Run the tokens in portions of ``prefill_chunk``; logits of the last one.

        Positions continue from the session's length, so a second call extends the first
        (the reference's ``ninfer_prefill`` does not advance the position between its
        chunks, src/api/ninfer_c_api.cpp:171-198; that defect is not kept)."""
        if len(tokens) == 0:
            raise NinferError("prefill: no tokens")
        if self.length + len(tokens) > self._engine.max_context:
            raise NinferError("prefill: capacity too small")      # the reference's -3
        chunk = self._engine.prefill_chunk
        out = None
        for i in range(0, len(tokens), chunk):
            part = list(tokens[i:i + chunk])
            last = i + chunk >= len(tokens)
            out = self._engine._runner.step([StepEntry(self._key, part, [len(part) - 1] if last else [])])
        return out[0].cpu().numpy()

    def decode(self, token: int) -> np.ndarray:
        return self._engine._runner.step([StepEntry(self._key, [int(token)], [0])])[0].cpu().numpy()

    def close(self) -> None:
        if self._open:
            self._engine._runner.close(self._key)
            self._open = False


class Ninfer:
    def __init__(self, model_dir: Optional[str] = None, max_context: int = 32768,
                 prefill_chunk: int = 2048, num_sequences: int = 1, *, dtype: str = "bfloat16",
                 page_size: int = 64, cache_tokens: Optional[int] = None,
                 max_batched_tokens: Optional[int] = None, use_graph: bool = True,
                 run_ahead: bool = True,
                 config: Optional[Dict[str, Any]] = None, random_weights: Optional[int] = None,
                 device: str = "cuda:0"):
        opts = EngineOptions(dtype=dtype, max_context=max_context, prefill_chunk=prefill_chunk,
                             num_sequences=num_sequences, page_size=page_size, cache_tokens=cache_tokens,
                             max_batched_tokens=max_batched_tokens, use_graph=use_graph, run_ahead=run_ahead,
                             device=device)
        self._engine = Engine(model_dir, config=config, random_seed=random_weights, options=opts)
        self._runner = self._engine.runner
        self.vocab = self._engine.vocab_size
        self.max_context, self.prefill_chunk = opts.max_context, opts.prefill_chunk
        self.num_sequences = opts.num_sequences
        self._keys = itertools.count()
        self._tokenizer = None
        self._model_dir = model_dir

    # ---- queries (ninfer_c_api.h:40-52) ----
    @property
    def devices(self) -> int:
        return 1

    @property
    def kv_bytes_per_token(self) -> int:
        return self._runner.cache.bytes_per_token()

    @property
    def kv_total_bytes(self) -> int:
        return self._runner.cache.total_bytes()

    @property
    def pages_free(self) -> List[int]:
        return self._runner.cache.pages_free()

    def stats(self) -> Dict[str, Any]:
        return self._engine.stats()

    # ---- tokenizer ----
    def _tok(self):
        if self._tokenizer is None:
            from .frontend.tokenizer import Tokenizer
            import os
            path = os.path.join(self._model_dir or "", "tokenizer.json")
            if not self._model_dir or not os.path.exists(path):
                raise NinferError("no tokenizer.json beside the model; pass token ids instead")
            self._tokenizer = Tokenizer(path)
        return self._tokenizer

    def tokenize(self, text: str, special: bool = False) -> List[int]:
        """Raw text -> ids; with `special`, chat markers written in the text (``<|im_start|>`` ...)
        become their own ids, as a rendered chat prompt needs (src/runtime/engine.cpp:115-120)."""
        return self._tok().encode_with_special(text) if special else self._tok().encode(text)

    def detokenize(self, ids: Sequence[int]) -> str:
        return self._tok().decode(ids)

    # ---- sessions ----
    def session(self) -> Session:
        try:
            return Session(self, ("session", next(self._keys)))
        except Exception as e:
            raise NinferError(f"session: {e}") from None

    def decode_batch(self, sessions: Sequence[Session], tokens: Sequence[int]) -> np.ndarray:
        """One step for N live requests, one token each -> logits [N, vocab]."""
        if len(sessions) != len(tokens):
            raise NinferError("decode_batch: sessions and tokens differ in length")
        out = self._runner.step([StepEntry(s._key, [int(t)], [0]) for s, t in zip(sessions, tokens)])
        return out.cpu().numpy()

    def step(self, entries: Sequence[tuple]) -> np.ndarray:
        """A mixed batch: ``(session, tokens, want)`` triples -> logits [wanted rows, vocab]."""
        out = self._runner.step([StepEntry(s._key, list(t), list(w)) for s, t, w in entries])
        return out.cpu().numpy()

    # ---- sampling (ninfer_sample, ninfer_c_api.cpp:248-260) ----
    def sample(self, logits, temperature: float = 0.7, top_k: int = 50, top_p: float = 0.95,
               repetition_penalty: float = 1.0, seed: int = 0, recent: Sequence[int] = ()) -> int:
        p = SamplingParams(temperature, top_k, top_p, repetition_penalty, seed)
        return sample_reference(np.asarray(logits, dtype=np.float32), p, recent, uniform_draw(seed, 0))

    # ---- whole generations through the scheduler ----
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 512,
                 temperature: float = 0.7, top_k: int = 50, top_p: float = 0.95,
                 repetition_penalty: float = 1.0, seed: int = 0,
                 stop_ids: Iterable[int] = ()) -> List[List[int]]:
        p = SamplingParams(temperature, top_k, top_p, repetition_penalty, seed, max_new_tokens)
        return self._engine.generate(prompts, p, stop_ids)

    def stream(self, prompt: Sequence[int], max_new_tokens: int = 512, temperature: float = 0.7,
               top_k: int = 50, top_p: float = 0.95, repetition_penalty: float = 1.0, seed: int = 0,
               stop_ids: Iterable[int] = ()):
        """Token ids of one generation, each as soon as it exists."""
        p = SamplingParams(temperature, top_k, top_p, repetition_penalty, seed, max_new_tokens)
        return self._engine.stream(prompt, p, stop_ids)

    def close(self) -> None:
        self._engine = None
        self._runner = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
