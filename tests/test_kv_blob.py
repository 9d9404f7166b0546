"""Saved KV cache ("AOTP" blob): the oracle's restatement against a hand-written header and
the reference's end-to-end property (crates/aot-llm/tests/e2e.rs:797-805), then the CUDA
library's aotcu_kv_save / aotcu_kv_load against the oracle, byte for byte."""
import struct

import numpy as np
import pytest

from conftest import assert_bits_equal
from oracle import prefix as op


def _caches(n_layer, ctx, kv, seed=3):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(n_layer * ctx * kv).astype(np.float32), rng.standard_normal(n_layer * ctx * kv).astype(np.float32))


def test_blob_layout_written_out_by_hand():
    n_layer, ctx, kv = 2, 8, 4
    k, v = _caches(n_layer, ctx, kv)
    tokens, n_cached = [7, 300, 0xFFFFFFFF, 12, 5], 3
    blob = op.serialize(k, v, ctx, n_layer, kv, tokens, n_cached)
    want = b"AOTP" + struct.pack("<I", 2) + struct.pack("<I", 5) + struct.pack("<I", 2) + struct.pack("<I", 4) + struct.pack("<I", 3)
    want += b"".join(struct.pack("<I", t) for t in tokens)
    assert len(want) == 44
    want += b"\0" * 20                                   # to the 64-byte boundary
    for layer in range(n_layer):
        at = layer * ctx * kv
        want += k[at:at + n_cached * kv].tobytes() + v[at:at + n_cached * kv].tobytes()
    assert blob == want
    assert len(blob) == 64 + n_layer * 2 * n_cached * kv * 4
    # exactly on a boundary: 10 tokens end at byte 64, no padding
    assert op.data_offset(10) == 64 and op.data_offset(11) == 128
    # n_cached is clamped to the token count
    assert op.serialize(k, v, ctx, n_layer, kv, tokens, 99) == op.serialize(k, v, ctx, n_layer, kv, tokens, 5)


def test_parse_accepts_and_rejects():
    n_layer, ctx, kv = 2, 8, 4
    k, v = _caches(n_layer, ctx, kv)
    tokens = [1, 2, 3, 4]
    blob = op.serialize(k, v, ctx, n_layer, kv, tokens, 3)
    p = op.parse(blob, n_layer, kv)
    assert p is not None and p.tokens == tokens and p.cached() == 3 and len(p) == 4
    k2, v2 = np.zeros_like(k), np.zeros_like(v)
    p.load_into(k2, v2, ctx)
    for layer in range(n_layer):
        at = layer * ctx * kv
        assert_bits_equal(k2[at:at + 3 * kv], k[at:at + 3 * kv], "k rows")
        assert_bits_equal(v2[at:at + 3 * kv], v[at:at + 3 * kv], "v rows")
        assert not k2[at + 3 * kv:at + ctx * kv].any()   # rows beyond the cached ones stay untouched
    # a different context length on the loading side only moves the layer bases
    k3, v3 = np.zeros(n_layer * 16 * kv, np.float32), np.zeros(n_layer * 16 * kv, np.float32)
    p.load_into(k3, v3, 16)
    assert_bits_equal(k3[16 * kv:16 * kv + 3 * kv], k[ctx * kv:ctx * kv + 3 * kv], "layer 1 rows at the new base")
    assert op.parse(b"", n_layer, kv) is None
    assert op.parse(b"AOTQ" + blob[4:], n_layer, kv) is None
    assert op.parse(blob[:4] + struct.pack("<I", 3) + blob[8:], n_layer, kv) is None          # unknown version
    assert op.parse(blob, n_layer + 1, kv) is None and op.parse(blob, n_layer, kv * 2) is None
    assert op.parse(blob[:-1], n_layer, kv) is None                                           # truncated rows
    assert op.parse(blob[:30], n_layer, kv) is None                                           # truncated ids
    assert op.parse(blob[:20] + struct.pack("<I", 5) + blob[24:], n_layer, kv) is None        # n_cached > n_tokens
    assert op.parse(blob[:8] + struct.pack("<I", 0) + blob[12:], n_layer, kv) is None         # no tokens
    # version 1: every token has rows, the sixth header word is not a count
    full = op.serialize(k, v, ctx, n_layer, kv, tokens, 4)
    v1 = full[:4] + struct.pack("<I", 1) + full[8:20] + struct.pack("<I", 0xDEAD) + full[24:]
    p1 = op.parse(v1, n_layer, kv)
    assert p1 is not None and p1.cached() == 4


def _tiny(pkg):
    return pkg.model.tiny("qwen3", n_layer=2)


def test_oracle_continuation_equals_whole_prompt(pkg, ob):
    """e2e.rs:797-805 on the oracle's model: save after the first part of a prompt, load into
    a fresh model, evaluate the rest; the logits are those of the whole prompt."""
    spec = _tiny(pkg)
    d = spec.head.dims
    kv, ctx = d.n_kv_head * d.head_dim, 48
    first, rest = [5, 17, 300, 42, 7], [9, 1, 250, 33]
    whole = ob.model_from_spec(spec, ctx, 16, n_threads=2)
    whole.forward_batch(first + rest, 0, True)
    a = ob.model_from_spec(spec, ctx, 16, n_threads=2)
    a.forward_batch(first, 0, False)
    blob = op.serialize(a.buf("k_cache"), a.buf("v_cache"), ctx, d.n_layer, kv, first, len(first))
    b = ob.model_from_spec(spec, 64, 16, n_threads=2)     # another context length on the loading side
    p = op.parse(blob, d.n_layer, kv)
    p.load_into(b.buf("k_cache"), b.buf("v_cache"), 64)
    b.forward_batch(rest, p.cached(), True)
    assert_bits_equal(b.logits(), whole.logits(), "continued logits")


@pytest.mark.gpu
def test_gpu_blob_is_the_oracle_blob_and_continues(pkg, ob, ctx):
    spec = _tiny(pkg)
    d = spec.head.dims
    kv, n_ctx = d.n_kv_head * d.head_dim, 48
    first, rest = [5, 17, 300, 42, 7], [9, 1, 250, 33]
    om = ob.model_from_spec(spec, n_ctx, 8, n_threads=2)
    om.forward_batch(first, 0, True)
    tok = ob.argmax(om.logits())
    om.forward(tok, len(first), True)                        # one decoded position on top of the prompt
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 8)
    g.forward_batch(first, 0, True)
    g.forward(tok, len(first), True)
    run = first + [tok, 11]                                   # the last token was never fed back (app.rs:629-632)
    blob = g.kv_save(run, len(first) + 1)
    want = op.serialize(om.buf("k_cache"), om.buf("v_cache"), n_ctx, d.n_layer, kv, run, len(first) + 1)
    assert blob == want
    # a second Gpu with a longer context continues the run
    g2 = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 64, 8)
    toks, cached = g2.kv_load(blob)
    assert toks == run and cached == len(first) + 1
    g2.forward_batch(toks[cached:] + rest, cached, True)
    whole = ob.model_from_spec(spec, 64, 16, n_threads=2)
    whole.forward_batch(first, 0, False)
    whole.forward(tok, len(first), False)
    whole.forward_batch([11] + rest, len(first) + 1, True)
    assert_bits_equal(g2.logits(), whole.logits(), "logits after continuing the saved run")
    # then through the one-kernel decode step on the restored cache
    nxt = ob.argmax(whole.logits())
    pos = cached + 1 + len(rest)
    g2.forward(nxt, pos, True)
    whole.forward(nxt, pos, True)
    assert_bits_equal(g2.logits(), whole.logits(), "decode step on the restored cache")
    # version 1 blobs load; blobs of another model or damaged ones fail and change nothing
    full = g.kv_save(first, len(first))
    v1 = full[:4] + struct.pack("<I", 1) + full[8:20] + struct.pack("<I", 77) + full[24:]
    assert g2.kv_load(v1) == (first, len(first))
    before = g2.kv_save(first, len(first))
    for bad in (b"", b"AOTQ" + blob[4:], blob[:4] + struct.pack("<I", 3) + blob[8:], blob[:-1], blob[:30],
                blob[:12] + struct.pack("<I", d.n_layer + 1) + blob[16:], blob[:16] + struct.pack("<I", kv * 2) + blob[20:],
                blob[:20] + struct.pack("<I", len(run) + 1) + blob[24:], blob[:8] + struct.pack("<I", 0) + blob[12:]):
        with pytest.raises(pkg.AotCudaError):
            g2.kv_load(bad)
    assert g2.kv_save(first, len(first)) == before
    # a cache longer than the loading context is refused (capi.rs:534-536)
    small = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 4, 4)
    with pytest.raises(pkg.AotCudaError):
        small.kv_load(blob)
    # n_cached is clamped to the token count; zero cached rows give a header-only blob
    assert g.kv_save(first, 99) == g.kv_save(first, len(first))
    assert len(g.kv_save(first, 0)) == op.data_offset(len(first))
    for x in (g, g2, small):
        x.close()


class _FakeGpu:
    """Records the calls a Session makes (no device)."""

    def __init__(self, n_ctx=64, max_batch=8, vocab=16):
        self.n_ctx, self.max_batch, self.vocab, self.calls, self.loaded = n_ctx, max_batch, vocab, [], None

    def forward(self, tok, pos, want):
        self.calls.append(("step", [tok], pos, bool(want)))

    def forward_batch(self, toks, pos, want):
        self.calls.append(("batch", list(toks), pos, bool(want)))

    def logits(self):
        v = np.zeros(self.vocab, np.float32)
        v[3] = v[7] = 1.0                      # a tie: the first maximum wins
        return v

    def generate(self, tok, pos, n):
        self.calls.append(("generate", [tok], pos, n))
        return np.arange(n, dtype=np.uint32) + 100, 0.0

    def kv_load(self, blob):
        toks = list(struct.unpack_from(f"<{struct.unpack_from('<I', blob, 8)[0]}I", blob, 24))
        self.loaded = blob
        return toks, struct.unpack_from("<I", blob, 20)[0]

    def kv_save(self, toks, n_cached):
        return ("saved", list(toks), n_cached)


def test_session_follows_the_reference_run_loop(pkg):
    S = pkg.session.Session
    # batches of 8, a single trailing token as a plain step, logits only for the last (app.rs:473-486)
    g = _FakeGpu()
    s = S(g, batch=8)
    s.feed(list(range(17)))
    assert g.calls == [("batch", list(range(8)), 0, False), ("batch", list(range(8, 16)), 8, False), ("step", [16], 16, True)]
    out = s.generate_greedy(4)
    assert out == [3, 100, 101, 102] and g.calls[-1] == ("generate", [3], 17, 3)
    assert s.pos == 20 and len(s.tokens) == 21                      # the last token was never fed back
    assert s.save() == ("saved", s.tokens, 20)
    # a saved run: its tokens come first and only the uncached ones are evaluated (app.rs:396-413)
    blob = b"AOTP" + struct.pack("<5I", 2, 5, 2, 64, 4) + struct.pack("<5I", 9, 8, 7, 6, 5) + b"\0" * 64
    g = _FakeGpu()
    s = S(g, batch=8)
    assert s.load_saved(blob) == 4
    s.feed([1, 2])
    assert g.calls == [("batch", [5, 1, 2], 4, True)] and s.tokens == [9, 8, 7, 6, 5, 1, 2]
    with pytest.raises(ValueError):
        s.load_saved(blob)                                            # not empty (capi.rs:527-529)
    # loading alone and asking for logits re-evaluates the last token
    g = _FakeGpu()
    s = S(g, batch=8)
    full = b"AOTP" + struct.pack("<5I", 2, 3, 2, 64, 3) + struct.pack("<3I", 4, 5, 6) + b"\0" * 64
    s.load_saved(full)
    s.feed([])
    assert g.calls == [("step", [6], 2, True)]
    # the compile-time prefix: only for a longer prompt that starts with it (app.rs:464-470)
    g = _FakeGpu()
    s = S(g, batch=8)
    assert s.try_prefix(full, [4, 5, 6]) == 0 and g.loaded is None    # not longer
    assert s.try_prefix(full, [4, 5, 7, 8]) == 0 and g.loaded is None  # another start
    assert s.try_prefix(b"junk", [4, 5, 6, 7]) == 0
    assert s.try_prefix(full, [4, 5, 6, 7, 8]) == 3 and g.loaded is full
    s.feed([4, 5, 6, 7, 8])
    assert g.calls == [("batch", [7, 8], 3, True)]
    # errors of the run loop
    with pytest.raises(ValueError):
        S(_FakeGpu(), 8).feed([])
    with pytest.raises(ValueError):
        S(_FakeGpu(n_ctx=4), 8).feed([1, 2, 3, 4, 5])
    assert pkg.session.blob_tokens(full) == [4, 5, 6] and pkg.session.blob_tokens(b"AOTQ" + full[4:]) is None


@pytest.mark.gpu
def test_session_saved_run_and_prefix_on_the_gpu(pkg, ob, ctx):
    """Two turns through save / load and a compile-time prefix give the tokens and logits of
    one uninterrupted run (e2e.rs:797-805 with generation in between)."""
    spec = _tiny(pkg)
    S = pkg.session.Session
    turn1, turn2 = [5, 17, 300, 42, 7], [9, 1, 250]
    whole = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 64, 8)
    w = S(whole, batch=8)
    w.feed(turn1)
    gen1 = w.generate_greedy(4)
    lw = w.feed(turn2)
    a = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 64, 8)
    sa = S(a, batch=4)
    sa.feed(turn1)
    assert sa.generate_greedy(4) == gen1
    blob = sa.save()
    b = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 48, 8)
    sb = S(b, batch=3)
    assert sb.load_saved(blob) == len(turn1) + 3
    lb = sb.feed(turn2)
    assert sb.tokens == w.tokens
    assert_bits_equal(lb, lw, "logits after the second turn of a saved run")
    # the compile-time prefix of the first turn
    pre = a.kv_save(turn1, len(turn1))
    c = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 64, 8)
    sc = S(c, batch=8)
    assert sc.try_prefix(pre, turn1 + [11, 12]) == len(turn1)
    n0 = c.dispatches()                      # launches are counted per context
    lc = sc.feed(turn1 + [11, 12])
    n1 = c.dispatches()
    d = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 64, 8)
    ld = S(d, batch=8).feed(turn1 + [11, 12])
    n2 = d.dispatches()
    assert_bits_equal(lc, ld, "logits with and without the prefix cache")
    assert n1 - n0 <= n2 - n1                # two tokens evaluated instead of seven
    for x in (whole, a, b, c, d):
        x.close()
