"""Pins the CPU oracle against the known answers and invariants that the reference's
own tests hold for this path (the reference is Rust and cannot be built here, so its
test expectations are re-expressed against the restatement)."""
import math

import numpy as np
import pytest

from conftest import XorShift64, assert_bits_equal, make_weights

ALL = list(range(9))
F32, F16, BF16, Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K = ALL


# crates/aot-kernels/src/quant.rs:445-466
def test_f16_known_answers(ob):
    L = ob.lib()
    for v in [0.0, 1.0, -1.0, 0.5, 65504.0, 1e-5, 6.1e-5, 1.2345, -0.333, 1e-7]:
        back = L.orc_f16_to_f32(L.orc_f32_to_f16(v))
        assert abs(back - v) <= abs(v) * 1e-3 + 1e-7
    assert L.orc_f16_to_f32(0x3C00) == 1.0
    assert L.orc_f16_to_f32(0xC000) == -2.0
    assert L.orc_f16_to_f32(0x0001) == np.float32(5.9604645e-8)
    assert math.isinf(L.orc_f16_to_f32(0x7C00))
    assert math.isnan(L.orc_f16_to_f32(0x7E00))
    assert L.orc_f32_to_f16(1.0) == 0x3C00
    assert L.orc_f32_to_f16(float("inf")) == 0x7C00
    assert L.orc_f32_to_f16(1e-8) == 0


def test_f16_all_patterns_match_numpy(ob):
    L = ob.lib()
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([L.orc_f16_to_f32(int(x)) for x in h], dtype=np.float32)
    ok = (got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))
    assert ok.all()


# quant.rs:468-490
def test_q8_0_activation(ob):
    x = np.array([(i - 32.0) / 7.0 for i in range(64)], dtype=np.float32)
    out = ob.quantize_q8_0(x)
    assert out.size == 2
    for i in range(2):
        v = out[i]["qs"].astype(np.float32) * out[i]["d"]
        assert np.all(np.abs(v - x[i * 32:(i + 1) * 32]) < 0.05)


def test_q8_k_activation_bsums(ob):
    x = np.array([((i * 37) % 101) - 50.0 for i in range(256)], dtype=np.float32)
    blk = ob.quantize_q8_k(x)[0]
    for j in range(16):
        assert int(blk["qs"][j * 16:(j + 1) * 16].astype(np.int32).sum()) == int(blk["bsums"][j])
    # the signed extreme maps to -127 exactly; an all-zero block stays zero
    assert blk["qs"][np.argmax(np.abs(x))] == -127
    z = ob.quantize_q8_k(np.zeros(256, dtype=np.float32))[0]
    assert z["d"] == 0 and not z["qs"].any() and not z["bsums"].any()


# crates/aot-kernels/src/ops.rs:233-241
def test_rmsnorm_unit_weights(ob):
    out = ob.rmsnorm([3.0, 4.0], [1.0, 1.0], 0.0)
    rms = math.sqrt(25.0 / 2.0)
    assert abs(out[0] - 3.0 / rms) < 1e-6 and abs(out[1] - 4.0 / rms) < 1e-6


# ops.rs:244-279
def test_rope_rotations(ob):
    cs = ob.rope_cos_sin([1.0, 0.5], math.pi / 2)
    x = ob.rope([1.0, 0.0, 1.0, 0.0], 1, 4, 4, cs)
    r = 1 / math.sqrt(2)
    assert abs(x[0]) < 1e-6 and abs(x[1] - 1) < 1e-6 and abs(x[2] - r) < 1e-6 and abs(x[3] - r) < 1e-6
    y = ob.rope([1.0, 1.0, 0.0, 0.0], 1, 4, 4, cs, neox=True)
    assert abs(y[0]) < 1e-6 and abs(y[2] - 1) < 1e-6 and abs(y[1] - r) < 1e-6 and abs(y[3] - r) < 1e-6
    cs8 = ob.rope_cos_sin([1.0, 0.7, 0.4, 0.1], 3.0)
    src = np.array([i * 0.37 - 1.0 for i in range(8)], dtype=np.float32)
    neox = ob.rope(src, 1, 8, 8, cs8, neox=True)
    perm = ob.rope(np.array([[src[i], src[i + 4]] for i in range(4)]).ravel(), 1, 8, 8, cs8)
    for i in range(4):
        assert abs(neox[i] - perm[2 * i]) < 1e-6 and abs(neox[i + 4] - perm[2 * i + 1]) < 1e-6


# ops.rs:282-294
def test_rmsnorm_heads(ob):
    x = ob.rmsnorm_heads([3.0, 4.0, 0.5, 0.5], [2.0, 1.0], 2, 2, 0.0)
    rms0 = math.sqrt(12.5)
    assert abs(x[0] - 6 / rms0) < 1e-5 and abs(x[1] - 4 / rms0) < 1e-5 and abs(x[2] - 2.0) < 1e-5 and abs(x[3] - 1.0) < 1e-5


def _dims(ob, **kw):
    d = ob.Dims()
    for k, v in dict(dim=8, hidden=8, n_layer=1, n_head=2, n_kv_head=1, head_dim=4, rot_dim=4, vocab=1, n_ctx_train=4,
                     eps=1e-5, rope_base=10000.0, rope_scale=1.0, rope_base_local=10000.0, rope_scale_local=1.0).items():
        setattr(d, k, v)
    for k, v in kw.items():
        setattr(d, k, v)
    return d


# ops.rs:297-340
def test_attention_small_cases(ob):
    d = _dims(ob)
    ctx = 4
    pool = ob.Pool(2)
    q = np.ones(8, dtype=np.float32)
    kc = np.zeros(ctx * 4, dtype=np.float32)
    vc = np.zeros(ctx * 4, dtype=np.float32)
    kc[:4] = [1, 2, 3, 4]
    vc[:4] = [5, 6, 7, 8]
    out = ob.attention(pool, q, kc, vc, d, ctx, 0, 0)
    assert out.tolist() == [5, 6, 7, 8, 5, 6, 7, 8]
    kc[4:8] = [1, 2, 3, 4]
    vc[4:8] = [1, 1, 1, 1]
    assert ob.attention(pool, q, kc, vc, d, ctx, 0, 1, window=1)[:4].tolist() == [1, 1, 1, 1]
    w2 = ob.attention(pool, q, kc, vc, d, ctx, 0, 1, window=2)
    assert w2[:4].tolist() == [3.0, 3.5, 4.0, 4.5]
    assert_bits_equal(ob.attention(pool, q, kc, vc, d, ctx, 0, 1, window=0), w2, "window 0 == window 2")
    rows = ob.attention_rows(pool, q, kc, vc, d, ctx, 0, 1, 1, window=1)
    assert_bits_equal(rows, ob.attention(pool, q, kc, vc, d, ctx, 0, 1, window=1), "rows == single")


# ops.rs:343-349
def test_gelu(ob):
    L = ob.lib()
    assert abs(L.orc_gelu(0.0)) < 1e-7
    assert abs(L.orc_gelu(1.0) - 0.841192) < 1e-5 and abs(L.orc_gelu(-1.0) + 0.158808) < 1e-5
    h = ob.gelu_mul([1.0, -1.0], [2.0, 2.0])
    assert abs(h[0] - 1.682384) < 1e-5 and abs(h[1] + 0.317616) < 1e-5


def test_softmax_and_argmax(ob):
    v = ob.softmax([1.0, 2.0, 3.0, -1.0])
    assert abs(v.sum() - 1) < 1e-6 and v[2] > v[1] > v[0] > v[3]
    assert ob.argmax([0.1, 5.0, 2.0]) == 1          # sampler.rs:123-127
    assert ob.argmax([1.0, 7.0, 7.0, 3.0]) == 1     # the first maximum wins
    assert ob.argmax([float("nan"), -1.0]) == 1     # NaN never wins
    assert ob.argmax([float("-inf")] * 3) == 0


# crates/aot-kernels/tests/dots.rs:52-134
@pytest.mark.parametrize("kind,cols,seed", [
    (Q4_0, 32, 1), (Q4_0, 64, 2), (Q4_0, 96, 3), (Q4_0, 2048, 4), (Q4_0, 5632, 5),
    (Q5_0, 32, 11), (Q5_0, 2048, 14), (Q8_0, 32, 11), (Q8_0, 64, 12), (Q8_0, 96, 13), (Q8_0, 2048, 14),
    (Q4_K, 256, 21), (Q4_K, 512, 22), (Q4_K, 2048, 23), (Q4_K, 5632, 24),
    (Q5_K, 256, 31), (Q5_K, 512, 32), (Q5_K, 2048, 33),
    (Q6_K, 256, 41), (Q6_K, 512, 42), (Q6_K, 2048, 43), (Q6_K, 8192, 44),
    (F16, 8, 51), (F16, 12, 52), (F16, 2053, 55), (BF16, 64, 53), (BF16, 2053, 55), (F32, 2048, 54), (F32, 2053, 55)])
def test_dot_tables_agree(pkg, ob, kind, cols, seed):
    rng = XorShift64(seed)
    w = rng.floats(cols)
    x = rng.floats(cols, 3.0)
    wq = np.empty(pkg.lib.row_bytes(kind, cols), dtype=np.uint8)
    pkg.lib.check(pkg.lib.synth().aotcu_synth_quantize_row(kind, pkg.lib.ptr(w), cols, pkg.lib.ptr(wq)))
    fref = float(np.dot(ob.dequant_row(kind, wq, cols).astype(np.float32), x))
    tol = float(np.abs(x).sum()) * 0.02 + 1e-3
    xq = ob.quantize_act(kind, x)
    vals = [ob.dot(t, kind, wq, xq, cols) for t in (ob.SCALAR, ob.AVX2, ob.AVX2_F16C)]
    for v in vals:
        assert abs(v - fref) < tol
    for v in vals[1:]:
        assert abs(v - vals[0]) <= abs(vals[0]) * 1e-4 + 1e-3
    if kind in (Q4_K, Q5_K, Q6_K):
        # the K-quant float formula is identical across tables (simd_avx2.rs:169, 264)
        assert vals[0].view(np.uint32) == vals[1].view(np.uint32)


# dots.rs:159-203
@pytest.mark.parametrize("kind", [Q4_0, Q5_0, Q8_0, Q4_K, Q6_K])
def test_x4_matches_singles_bitwise(pkg, ob, kind):
    cols = 2048
    rng = np.random.default_rng(777 + kind)
    wq = make_weights(pkg, kind, 1, cols, 3 + kind)
    xs = [ob.quantize_act(kind, (rng.random(cols, dtype=np.float32) * 4 - 2)) for _ in range(4)]
    got = ob.dot_x4(ob.AVX2, kind, wq, xs, cols)
    assert got is not None
    for i in range(4):
        assert got[i].view(np.uint32) == ob.dot(ob.AVX2, kind, wq, xs[i], cols).view(np.uint32)
    assert ob.dot_x4(ob.AVX2, Q5_K, wq, xs, cols) is None  # matvec.rs:541


# dots.rs:136-157 and 205-266
@pytest.mark.parametrize("kind", [Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K, F16])
def test_matmul_matches_matvec_bitwise(pkg, ob, kind):
    rows, cols = 37, 512
    rng = np.random.default_rng(4242 + kind)
    wq = make_weights(pkg, kind, rows, cols, 9 + kind)
    pool1, pool3 = ob.Pool(1), ob.Pool(3)
    tab = ob.detect_table()
    for m in (1, 3, 4, 7, 9):
        xs = rng.random(m * cols, dtype=np.float32) * 2 - 1
        q = ob.quantize_act(kind, xs)
        batched = ob.matmul(pool3, tab, kind, wq, q, m, rows, cols)
        per = q.reshape(m, -1)
        for i in range(m):
            single = ob.matvec(pool1, tab, kind, wq, np.ascontiguousarray(per[i]), rows, cols)
            assert_bits_equal(batched[i], single, f"kind {kind} m {m} row {i}")
            assert_bits_equal(ob.matvec(pool3, tab, kind, wq, np.ascontiguousarray(per[i]), rows, cols), single,
                              "1 vs 3 threads")


def test_matvec2_matvec3_match_matvec(pkg, ob):
    cols, tab, pool = 512, ob.detect_table(), ob.Pool(4)
    x = ob.quantize_q8_k(np.random.default_rng(5).standard_normal(cols).astype(np.float32))
    ws = [make_weights(pkg, Q4_K, r, cols, 20 + i) for i, r in enumerate((64, 16, 16))]
    outs = ob.matvec3(pool, tab, Q4_K, ws, x, (64, 16, 16), cols)
    for w, o, r in zip(ws, outs, (64, 16, 16)):
        assert_bits_equal(o, ob.matvec(pool, tab, Q4_K, w, x, r, cols), "matvec3")
    a, b = ob.matvec2(pool, tab, Q4_K, ws[1], ws[2], x, 16, cols)
    assert_bits_equal(a, outs[1], "matvec2 a")
    assert_bits_equal(b, outs[2], "matvec2 b")


# crates/aot-kernels/src/quantize.rs:322-333
@pytest.mark.parametrize("kind,tol", [(F32, 1e-7), (F16, 1e-3), (BF16, 1e-2), (Q8_0, 1e-2), (Q4_0, 0.1), (Q5_0, 0.05),
                                      (Q4_K, 0.08), (Q5_K, 0.04), (Q6_K, 0.02)])
def test_encoder_roundtrip_error(pkg, ob, kind, tol):
    x = (np.random.default_rng(kind + 1).random(512, dtype=np.float32) * 2 - 1).astype(np.float32)
    enc = np.empty(pkg.lib.row_bytes(kind, 512), dtype=np.uint8)
    pkg.lib.check(pkg.lib.synth().aotcu_synth_quantize_row(kind, pkg.lib.ptr(x), 512, pkg.lib.ptr(enc)))
    dec = ob.dequant_row(kind, enc, 512)
    assert float(np.abs(x - dec).mean()) < tol


def _numpy_forward(ob, spec, tokens):
    """An independent float64 forward pass with the same activation quantization, in the
    spirit of the reference's in-test model (crates/aot-llm/tests/e2e.rs:156-189, 260-343)."""
    d = spec.head.dims
    W = spec.weights

    def mat(t):
        rb = ob.row_bytes(t.kind, t.cols)
        return np.stack([ob.dequant_row(t.kind, W[t.off + r * rb: t.off + (r + 1) * rb], t.cols) for r in range(t.rows)]).astype(np.float64)

    def vec(t):
        return W[t.off:t.off + 4 * t.cols].view(np.float32).astype(np.float64)

    def act(kind, x):
        a = ob.activation(kind)
        x = x.astype(np.float32)
        if a == "q8_k":
            q = ob.quantize_q8_k(x)
            return (q["qs"].astype(np.float64) * q["d"].astype(np.float64)[:, None]).ravel()
        if a == "q8_0":
            q = ob.quantize_q8_0(x)
            return (q["qs"].astype(np.float64) * q["d"].astype(np.float64)[:, None]).ravel()
        return x.astype(np.float64)

    def rms(x, w, eps):
        return x / np.sqrt((x * x).mean() + eps) * w

    hd, nh, nkv = d.head_dim, d.n_head, d.n_kv_head
    embd = spec.head.token_embd
    rb = ob.row_bytes(embd.kind, embd.cols)
    kc = [[] for _ in range(d.n_layer)]
    vc = [[] for _ in range(d.n_layer)]
    mats = [{n: mat(getattr(l, n)) for n in ("wq", "wk", "wv", "wo", "gate", "up", "down")} for l in spec.layers]
    out_m = mat(spec.head.output)
    logits = None
    for pos, t in enumerate(tokens):
        x = ob.dequant_row(embd.kind, W[embd.off + t * rb: embd.off + (t + 1) * rb], d.dim).astype(np.float64)
        for li, l in enumerate(spec.layers):
            xb = rms(x, vec(l.attn_norm), d.eps)
            q = mats[li]["wq"] @ act(l.wq.kind, xb)
            k = mats[li]["wk"] @ act(l.wk.kind, xb)
            v = mats[li]["wv"] @ act(l.wv.kind, xb)
            if d.qkv_bias:
                q, k, v = q + vec(l.bq), k + vec(l.bk), v + vec(l.bv)
            if d.qk_norm:
                q = np.concatenate([rms(q[h * hd:(h + 1) * hd], vec(l.q_norm), d.eps) for h in range(nh)])
                k = np.concatenate([rms(k[h * hd:(h + 1) * hd], vec(l.k_norm), d.eps) for h in range(nkv)])
            inv = np.array([d.rope_base ** (-(2.0 * i) / d.rot_dim) for i in range(d.rot_dim // 2)])
            ang = pos * inv

            def rope(z, n):
                z = z.copy().reshape(n, hd)
                c, s = np.cos(ang), np.sin(ang)
                if d.rope_neox:
                    a, b = z[:, :hd // 2].copy(), z[:, hd // 2:].copy()
                    z[:, :hd // 2], z[:, hd // 2:] = a * c - b * s, a * s + b * c
                else:
                    a, b = z[:, 0::2].copy(), z[:, 1::2].copy()
                    z[:, 0::2], z[:, 1::2] = a * c - b * s, a * s + b * c
                return z.ravel()

            q, k = rope(q, nh), rope(k, nkv)
            kc[li].append(k)
            vc[li].append(v)
            att = np.zeros(nh * hd)
            for h in range(nh):
                kvh = h // (nh // nkv)
                sc = np.array([q[h * hd:(h + 1) * hd] @ kk[kvh * hd:(kvh + 1) * hd] for kk in kc[li]]) / math.sqrt(hd)
                p = np.exp(sc - sc.max())
                p /= p.sum()
                att[h * hd:(h + 1) * hd] = sum(pp * vv[kvh * hd:(kvh + 1) * hd] for pp, vv in zip(p, vc[li]))
            x = x + mats[li]["wo"] @ act(l.wo.kind, att)
            xb = rms(x, vec(l.ffn_norm), d.eps)
            g = mats[li]["gate"] @ act(l.gate.kind, xb)
            u = mats[li]["up"] @ act(l.up.kind, xb)
            x = x + mats[li]["down"] @ act(l.down.kind, g / (1 + np.exp(-g)) * u)
        if pos + 1 == len(tokens):
            logits = out_m @ act(spec.head.output.kind, rms(x, vec(spec.head.output_norm), d.eps))
    return logits


# crates/aot-llm/tests/e2e.rs:488-502
@pytest.mark.parametrize("arch", ["llama", "qwen3", "qwen2"])
def test_oracle_forward_matches_independent_float_model(pkg, ob, arch):
    spec = pkg.model.tiny(arch, n_layer=2)
    tokens = [5, 17, 300, 42, 7]
    want = _numpy_forward(ob, spec, tokens)
    om = ob.model_from_spec(spec, 16, 8, n_threads=3)
    for pos, t in enumerate(tokens):
        assert om.forward(t, pos, pos + 1 == len(tokens)) == 0
    got = om.logits().astype(np.float64)
    tol = 2e-3 * np.abs(want).max() + 1e-3
    assert np.abs(got - want).max() <= tol
    assert int(np.argmax(got)) == int(np.argmax(want))
    # batch == single, bitwise (the reference's --batch 1 vs --batch 128 check)
    ob2 = ob.model_from_spec(spec, 16, 8, n_threads=2)
    assert ob2.forward_batch(tokens, 0, True) == 0
    assert_bits_equal(ob2.logits(), om.logits(), "forward_batch vs forward")
    # bounds asserted by the generated code (emit.rs:467-468, 493-494)
    assert om.forward(spec.head.dims.vocab, 0, True) == -1
    assert om.forward(1, 16, True) == -1
    assert ob2.forward_batch([1] * 9, 0, True) == -1
