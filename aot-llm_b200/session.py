"""The callers either side of the forward pass, as the reference's generated binary runs
them (crates/aot-kernels/src/app.rs): KV rows that need no evaluation (a saved run or the
compile-time prefix, app.rs:458-471), prompt evaluation in batches with logits for the
last token only (app.rs:473-486), the greedy loop (app.rs:553-610 with sampler.rs:99-109),
and the saved run written afterwards (app.rs:629-640). Host logic only; every number
comes from the `Gpu` it drives.
"""
from __future__ import annotations

import struct

import numpy as np

from .lib import AotCudaError


def blob_tokens(blob: bytes):
    """Token ids of an "AOTP" blob without touching a device (prefix.rs:45-61), or None when
    the header is not one."""
    if len(blob) < 24 or blob[:4] != b"AOTP":
        return None
    version, n = struct.unpack_from("<II", blob, 4)
    if version not in (1, 2) or n == 0 or len(blob) < 24 + 4 * n:
        return None
    return list(struct.unpack_from(f"<{n}I", blob, 24))


class Session:
    def __init__(self, gpu, batch: int = 64):
        self.g = gpu
        self.batch = max(1, min(batch, gpu.max_batch))
        self.tokens: list[int] = []     # every token of the run, in order
        self.pos = 0                    # positions whose KV rows are in the cache

    # ---- KV rows that need no evaluation -------------------------------------------------
    def load_saved(self, blob: bytes) -> int:
        """`--load-kv` (app.rs:396-413, 461-463): the saved tokens come first; returns how
        many of them have cache rows. Raises AotCudaError when the blob is not a cache of
        this model."""
        if self.tokens:
            raise ValueError("the session is not empty")       # capi.rs:527-529
        toks, cached = self.g.kv_load(blob)
        if len(toks) >= self.g.n_ctx:
            raise ValueError(f"saved sequence has {len(toks)} tokens, context is {self.g.n_ctx}")   # capi.rs:534-536
        self.tokens, self.pos = list(toks), cached
        return cached

    def try_prefix(self, blob: bytes, prompt) -> int:
        """The compile-time prefix (app.rs:464-470): used only when the prompt is longer than
        the prefix and starts with its tokens; a blob that is not of this model is ignored,
        as `Prefix::parse` returning None is. Returns the cached positions (0: not used)."""
        if self.tokens or not blob:
            return 0
        pre = blob_tokens(blob)
        prompt = [int(t) for t in prompt]
        if pre is None or not (len(prompt) > len(pre) and prompt[:len(pre)] == pre):
            return 0
        try:
            _, cached = self.g.kv_load(blob)
        except AotCudaError:
            return 0
        self.pos = cached
        return cached

    # ---- prompt evaluation ---------------------------------------------------------------
    def feed(self, prompt) -> np.ndarray:
        """Appends `prompt` to the run and evaluates every token that has no cache row yet, in
        batches, with logits for the last one only (app.rs:473-486). Returns the logits."""
        self.tokens += [int(t) for t in prompt]
        n = len(self.tokens)
        if n == 0:
            raise ValueError("empty prompt")                    # app.rs:421-424
        if n > self.g.n_ctx:
            raise ValueError(f"prompt has {n} tokens but the context is {self.g.n_ctx}")   # app.rs:430-433
        done = self.pos
        if done >= n:
            done = n - 1                                         # re-evaluate the last token for its logits
        while done < n:
            end = min(done + self.batch, n)
            last = end == n
            if end - done == 1:
                self.g.forward(self.tokens[done], done, last)
            else:
                self.g.forward_batch(self.tokens[done:end], done, last)
            done = end
        self.pos = n
        return self.g.logits()

    # ---- generation ------------------------------------------------------------------------
    def generate_greedy(self, n_tokens: int):
        """Greedy decoding after `feed`: the first token from the current logits, the rest on
        the device. The last generated token is never fed back (app.rs:629-632)."""
        if n_tokens <= 0:
            return []
        n_tokens = min(n_tokens, self.g.n_ctx - self.pos)
        if n_tokens <= 0:
            return []
        first = int(np.argmax(self.g.logits()))                  # first maximum, sampler.rs:99-109
        out = [first]
        if n_tokens > 1:
            ids, _ = self.g.generate(first, self.pos, n_tokens - 1)
            out += [int(i) for i in ids]
            self.pos += n_tokens - 1
        self.tokens += out
        return out

    def save(self) -> bytes:
        """`--save-kv` (app.rs:629-640): every token of the run, cache rows for the evaluated ones."""
        return self.g.kv_save(self.tokens, self.pos)
