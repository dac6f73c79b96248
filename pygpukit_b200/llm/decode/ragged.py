"""Batch scheduler of the token-major models (net-new; the reference's scheduler is its Rust crate, outside this
package's scope -- this is the Python loop that drives `LayeredCausalModel.step_device`).

Requests are admitted at any time.  A step is either a PREFILL step -- every request that still has prompt tokens
feeds its next portion (the whole rest, or `prefill_chunk` tokens), requests of different lengths side by side in
one ragged batch -- or a DECODE step, in which every running request feeds the token it sampled last.  A request
that finishes gives its cache pages and slot back at once.  Greedy sampling is a row argmax on the device (4 bytes
per request come back); temperature / top-k / top-p go through `llm.sampling.sample_token` on the host logits.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from ..._lib import api
from ...core.array import GPUArray
from ...core.dtypes import int32
from ...core.stream import current_stream_handle as _st
from ..sampling import sample_token


@dataclass
class Request:
    id: object
    prompt: list[int]
    max_new_tokens: int
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    eos_token_id: int | None = None
    fed: int = 0                                   # prompt tokens already in the cache
    tokens: list[int] = field(default_factory=list)
    generated: int = 0


class RaggedScheduler:
    def __init__(self, model, prefill_chunk: int | None = None):
        if prefill_chunk is not None and prefill_chunk < 1:
            raise ValueError("prefill_chunk must be positive")
        self.model, self.prefill_chunk = model, prefill_chunk
        self.running: dict = {}
        self.finished: dict = {}
        self._argmax: GPUArray | None = None

    def add_request(self, req_id, prompt: list[int], max_new_tokens: int = 20, temperature: float = 0.0, top_k: int = 0,
                    top_p: float = 1.0, eos_token_id: int | None = None) -> None:
        if req_id in self.running or req_id in self.finished:
            raise ValueError(f"request {req_id!r} already exists")
        if not prompt:
            raise ValueError("empty prompt")
        r = Request(req_id, [int(t) for t in prompt], int(max_new_tokens), float(temperature), int(top_k), float(top_p),
                    eos_token_id)
        r.tokens = list(r.prompt)
        if r.max_new_tokens <= 0:
            self.finished[req_id] = r.tokens
        else:
            self.running[req_id] = r

    def _sample(self, reqs: list[Request], logits: GPUArray) -> list[int]:
        n, V = len(reqs), self.model.config.vocab_size
        if all(r.temperature == 0 for r in reqs):
            if self._argmax is None or self._argmax.size < n:
                self._argmax = GPUArray((max(n, 16),), int32)
            api.argmax_rows(logits.device_ptr, self._argmax.device_ptr, None, n, V, 0, _st())
            return [int(t) for t in self._argmax.to_numpy()[:n]]
        host = np.empty((n, V), np.float32)
        api.memcpy_d2h(host.ctypes.data, logits.device_ptr, host.nbytes, _st())
        api.stream_sync(_st()) if _st() is not None else api.device_sync()
        return [sample_token(host[i], r.temperature, r.top_k, r.top_p) for i, r in enumerate(reqs)]

    def step(self) -> list[tuple[object, int]]:
        """One model step; returns the (request id, token) pairs sampled in it."""
        pending = [r for r in self.running.values() if r.fed < len(r.prompt)]
        entries, sampled = [], []
        if pending:                                   # prefill step: next portion of every unfinished prompt
            for r in pending:
                n = len(r.prompt) - r.fed
                if self.prefill_chunk is not None:
                    n = min(n, self.prefill_chunk)
                last = r.fed + n == len(r.prompt)
                entries.append((r.id, r.prompt[r.fed:r.fed + n], [n - 1] if last else []))
                r.fed += n
                if last:
                    sampled.append(r)
        else:                                         # decode step: one token per running request
            for r in self.running.values():
                entries.append((r.id, [r.tokens[-1]], [0]))
                sampled.append(r)
        if not entries:
            return []
        logits, n = self.model.step_device(entries)
        out = []
        if n:
            for r, tok in zip(sampled, self._sample(sampled, logits)):
                r.tokens.append(tok)
                r.generated += 1
                out.append((r.id, tok))
                if r.generated >= r.max_new_tokens or (r.eos_token_id is not None and tok == r.eos_token_id):
                    self.model.release(r.id)
                    self.finished[r.id] = r.tokens
                    del self.running[r.id]
        return out

    def run(self) -> dict:
        """Step until every request has finished; {request id: prompt + generated tokens}."""
        while self.running:
            self.step()
        return self.finished


__all__ = ["Request", "RaggedScheduler"]
