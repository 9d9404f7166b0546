"""Parity of every kernel-level entry point of the C-ABI library with the CPU oracle.
Bit-exact: integer block sums, quantized activations and all f32 outputs."""
import numpy as np
import pytest

from conftest import assert_bits_equal, make_weights

pytestmark = pytest.mark.gpu

F32, F16, BF16, Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K = range(9)
QUANT = [Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K]


def _x(cols, seed, scale=2.0):
    return (np.random.default_rng(seed).standard_normal(cols) * scale).astype(np.float32)


def test_quantizers_bit_exact(pkg, ob, ctx):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(9 * 2048) * 3).astype(np.float32)
    x[256:512] = 0.0                      # an all-zero block
    x[512:768] = np.abs(x[512:768])       # positive extreme
    x[768] = x[769] = 7.5                 # tie on |v|: the first one is the extreme
    x[1030] = -9.25
    x[1031] = 9.25                        # tie with opposite signs
    for act, want in (("q8_k", ob.quantize_q8_k(x)), ("q8_0", ob.quantize_q8_0(x))):
        got = ctx.host_quantize(act, x)
        assert got.tobytes() == want.tobytes(), act


@pytest.mark.parametrize("mode", ["enc", "uniform"])
@pytest.mark.parametrize("kind", QUANT)
def test_block_sums_bit_exact(pkg, ob, ctx, kind, mode):
    rows, cols = 5, 1024
    w = make_weights(pkg, kind, rows, cols, 100 + kind, mode)
    xq = ob.quantize_act(kind, _x(cols, kind))
    nb = cols // pkg.lib.BLOCK[kind]
    dw, dx = ctx.to_device(w), ctx.to_device(xq.view(np.uint8))
    dsi, dsm = ctx.alloc(rows * nb * 4), ctx.alloc(rows * nb * 4)
    ctx.block_sums(kind, dw, dx, rows, cols, dsi, dsm)
    si = dsi.download(np.int32, rows * nb).reshape(rows, nb)
    sm = dsm.download(np.int32, rows * nb).reshape(rows, nb)
    rb = pkg.lib.row_bytes(kind, cols)
    for r in range(rows):
        osi, osm = ob.block_sums(kind, w[r * rb:(r + 1) * rb].copy(), xq, cols)
        assert np.array_equal(si[r], osi), (kind, r)
        if kind in (Q4_K, Q5_K):
            assert np.array_equal(sm[r], osm), (kind, r)


SHAPES = {
    Q4_0: [(5, 32), (37, 96), (300, 2048), (64, 5632)],
    Q5_0: [(5, 32), (37, 96), (300, 2048)],
    Q8_0: [(5, 32), (37, 64), (300, 2048), (33, 4096)],
    Q4_K: [(1, 256), (37, 512), (5632, 2048), (2048, 5632), (3, 12288)],
    Q5_K: [(1, 256), (37, 512), (700, 2048)],
    Q6_K: [(1, 256), (37, 512), (2048, 5632), (1500, 2048), (7, 8192)],
    F16: [(5, 8), (9, 12), (37, 2053), (300, 2048)],
    BF16: [(5, 64), (37, 2053), (300, 2048)],
    F32: [(5, 8), (37, 2053), (300, 2048)],
}


@pytest.mark.parametrize("mode", ["enc", "uniform"])
@pytest.mark.parametrize("kind", list(range(9)))
def test_matvec_bit_exact(pkg, ob, ctx, kind, mode):
    if mode == "uniform" and kind < 3:
        pytest.skip("float kinds have no block fields")
    pool, tab = ob.Pool(4), ob.detect_table()
    for rows, cols in SHAPES[kind]:
        w = make_weights(pkg, kind, rows, cols, 7 * kind + rows, mode)
        x = _x(cols, rows + cols)
        xq = ob.quantize_act(kind, x)
        want = ob.matvec(pool, tab, kind, w, xq, rows, cols)
        dw, dx, dout = ctx.to_device(w), ctx.to_device(xq.view(np.uint8)), ctx.alloc(rows * 4)
        ctx.matvec(kind, dout, dw, dx, rows, cols)
        assert_bits_equal(dout.download(np.float32, rows), want, f"matvec kind {kind} {rows}x{cols} {mode}")
    ctx.device_status()


def test_config0_single_q4k_matvec(pkg, ob, ctx):
    """Field-uniform Q4_K blocks, 5632 x 2048 (TinyLlama ffn_up), x ~ N(0,1)."""
    rows, cols = 5632, 2048
    w = make_weights(pkg, Q4_K, rows, cols, 1, "uniform")
    x = np.random.default_rng(2).standard_normal(cols).astype(np.float32)
    got = ctx.host_matmul(Q4_K, w, x, 1, rows, cols)[0]
    want = ob.matvec(ob.Pool(8), ob.detect_table(), Q4_K, w, ob.quantize_q8_k(x), rows, cols)
    assert_bits_equal(got, want, "config 0")


@pytest.mark.parametrize("kind", [Q4_K, Q6_K, Q8_0, F16])
def test_matvec2_matvec3(pkg, ob, ctx, kind):
    cols, rows3 = 512, (96, 40, 24)
    pool, tab = ob.Pool(3), ob.detect_table()
    ws = [make_weights(pkg, kind, r, cols, 50 + i) for i, r in enumerate(rows3)]
    xq = ob.quantize_act(kind, _x(cols, 9))
    dx = ctx.to_device(xq.view(np.uint8))
    dws = [ctx.to_device(w) for w in ws]
    douts = [ctx.alloc(r * 4) for r in rows3]
    ctx.matvec3([kind] * 3, douts, dws, dx, rows3, cols)
    for w, o, r in zip(ws, douts, rows3):
        assert_bits_equal(o.download(np.float32, r), ob.matvec(pool, tab, kind, w, xq, r, cols), "matvec3")
    wb = make_weights(pkg, kind, rows3[0], cols, 77)
    da, db_ = ctx.alloc(rows3[0] * 4), ctx.alloc(rows3[0] * 4)
    ctx.matvec2(kind, da, db_, dws[0], ctx.to_device(wb), dx, rows3[0], cols)
    oa, ob_ = ob.matvec2(pool, tab, kind, ws[0], wb, xq, rows3[0], cols)
    assert_bits_equal(da.download(np.float32, rows3[0]), oa, "matvec2 a")
    assert_bits_equal(db_.download(np.float32, rows3[0]), ob_, "matvec2 b")


def test_matvec3_mixed_k_quants(pkg, ob, ctx):
    """q/k in Q4_K and v in Q6_K share Q8_K activations and run as one launch."""
    cols, rows3, kinds = 2048, (2048, 256, 256), (Q4_K, Q4_K, Q6_K)
    pool, tab = ob.Pool(4), ob.detect_table()
    ws = [make_weights(pkg, k, r, cols, 60 + i) for i, (k, r) in enumerate(zip(kinds, rows3))]
    xq = ob.quantize_q8_k(_x(cols, 4))
    douts = [ctx.alloc(r * 4) for r in rows3]
    ctx.matvec3(kinds, douts, [ctx.to_device(w) for w in ws], ctx.to_device(xq.view(np.uint8)), rows3, cols)
    for k, w, o, r in zip(kinds, ws, douts, rows3):
        assert_bits_equal(o.download(np.float32, r), ob.matvec(pool, tab, k, w, xq, r, cols), f"mixed kind {k}")


# crates/aot-kernels/tests/dots.rs:205-266: batched == per-token, bitwise
@pytest.mark.parametrize("kind", [Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K, F16, BF16, F32])
def test_matmul_bit_exact(pkg, ob, ctx, kind):
    rows, cols = 37, 512
    pool, tab = ob.Pool(3), ob.detect_table()
    w = make_weights(pkg, kind, rows, cols, 31 + kind)
    dw = ctx.to_device(w)
    for m in (1, 3, 4, 7, 9, 64):
        xs = _x(m * cols, m, 1.0)
        q = ob.quantize_act(kind, xs)
        want = ob.matmul(pool, tab, kind, w, q, m, rows, cols)
        dout = ctx.alloc(m * rows * 4)
        ctx.matmul(kind, dout, dw, ctx.to_device(q.view(np.uint8)), m, rows, cols)
        got = dout.download(np.float32, m * rows).reshape(m, rows)
        assert_bits_equal(got, want, f"matmul kind {kind} m {m}")
        assert_bits_equal(ctx.host_matmul(kind, w, xs, m, rows, cols), want, "host-buffer path")


# Prompt chunks of 8..64 tokens on K-quant matrices run on int8 tensor-core tiles; results
# must still equal the per-token products bit for bit (crates/aot-kernels/tests/dots.rs:205-266).
@pytest.mark.parametrize("kind", [Q4_K, Q5_K, Q6_K])
@pytest.mark.parametrize("rows,cols", [(37, 512), (160, 2048), (48, 5632)])
def test_matmul_tensor_core_tiles_bit_exact(pkg, ob, ctx, kind, rows, cols):
    pool, tab = ob.Pool(4), ob.detect_table()
    w = make_weights(pkg, kind, rows, cols, 77 + kind)
    dw = ctx.to_device(w)
    for m in (8, 13, 16, 40, 64):
        xs = _x(m * cols, 100 + m, 1.0)
        q = ob.quantize_act(kind, xs)
        want = ob.matmul(pool, tab, kind, w, q, m, rows, cols)
        dout = ctx.alloc(m * rows * 4)
        ctx.matmul(kind, dout, dw, ctx.to_device(q.view(np.uint8)), m, rows, cols)
        got = dout.download(np.float32, m * rows).reshape(m, rows)
        assert_bits_equal(got, want, f"matmul kind {kind} {rows}x{cols} m {m} (reference-layout blocks)")
        assert_bits_equal(ctx.host_matmul(kind, w, xs, m, rows, cols), want, f"kind {kind} m {m} host-buffer path")
    ctx.device_status()


# matmul2 (crates/aot-kernels/src/matvec.rs:571-583): gate and up of a prompt chunk in one call
@pytest.mark.parametrize("kind", [Q8_0, Q4_K, Q6_K, F16])
def test_matmul2_bit_exact(pkg, ob, ctx, kind):
    rows, cols = 40, 512
    pool, tab = ob.Pool(3), ob.detect_table()
    wa, wb = make_weights(pkg, kind, rows, cols, 201 + kind), make_weights(pkg, kind, rows, cols, 301 + kind)
    dwa, dwb = ctx.to_device(wa), ctx.to_device(wb)
    for m in (1, 5, 8, 33):
        xs = _x(m * cols, 40 + m, 1.0)
        q = ob.quantize_act(kind, xs)
        da, db = ctx.alloc(m * rows * 4), ctx.alloc(m * rows * 4)
        ctx.matmul2(kind, da, db, dwa, dwb, ctx.to_device(q.view(np.uint8)), m, rows, cols)
        assert_bits_equal(da.download(np.float32, m * rows).reshape(m, rows), ob.matmul(pool, tab, kind, wa, q, m, rows, cols), f"matmul2 a kind {kind} m {m}")
        assert_bits_equal(db.download(np.float32, m * rows).reshape(m, rows), ob.matmul(pool, tab, kind, wb, q, m, rows, cols), f"matmul2 b kind {kind} m {m}")
    ctx.device_status()


# Wide rows: the activation images of all rows do not fit in shared memory at once, so the
# streaming kernel (Q8_0 family) and the float kernel work through them in groups.
@pytest.mark.parametrize("kind", [Q4_0, Q8_0, BF16])
def test_matmul_wide_rows_in_groups_bit_exact(pkg, ob, ctx, kind):
    rows, cols, m = 24, 8192, 61
    pool, tab = ob.Pool(4), ob.detect_table()
    w = make_weights(pkg, kind, rows, cols, 400 + kind)
    xs = _x(m * cols, 77, 1.0)
    q = ob.quantize_act(kind, xs)
    want = ob.matmul(pool, tab, kind, w, q, m, rows, cols)
    dout = ctx.alloc(m * rows * 4)
    ctx.matmul(kind, dout, ctx.to_device(w), ctx.to_device(q.view(np.uint8)), m, rows, cols)
    assert_bits_equal(dout.download(np.float32, m * rows).reshape(m, rows), want, f"matmul kind {kind} {rows}x{cols} m {m}")
    ctx.device_status()


# The chunk-streaming kernels (Q8_0 family and float kinds: rows in fours, 16-byte aligned
# rows) in each of their shapes: one or two rows per lane, a CTA with more rows than one
# stage holds, a last chunk that is not full, and 1, 8 or 16 activation rows per lane with
# one or two token groups. Both they and the whole-row kernels they replace must give the
# oracle's bits.
@pytest.mark.parametrize("kind", [Q4_0, Q5_0, Q8_0, F16, BF16, F32])
def test_chunk_streaming_products_bit_exact(pkg, ob, ctx, kind):
    spec = pkg.model.tiny("llama", n_layer=1)
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 16, 2)   # only to reach the process-wide switches
    pool, tab = ob.Pool(8), ob.detect_table()
    cols = 2304 if kind >= Q4_0 else 2056                     # 4.5 chunks of 16 blocks / 7.6 and 14.3 chunks of columns
    switch = "q80_chunks" if kind >= Q4_0 else "float_chunks"
    try:
        for on in (1, 0):
            g.set_option(switch, on)
            # rows per CTA (148 SMs): 1 quad; 7 quads; 14 quads; 33 quads (two groups of 30)
            for rows, ms in ((600, (1, 5)), (4000, (1, 9, 16)), (8000, (1, 33)), (19000, (1, 17))):
                if not on and rows > 4000:
                    continue
                w = make_weights(pkg, kind, rows, cols, 500 + kind + rows)
                dw = ctx.to_device(w)
                for m in ms:
                    xs = _x(m * cols, 60 + m, 1.0)
                    q = ob.quantize_act(kind, xs)
                    want = ob.matmul(pool, tab, kind, w, q, m, rows, cols)
                    dout = ctx.alloc(m * rows * 4)
                    ctx.matmul(kind, dout, dw, ctx.to_device(q.view(np.uint8)), m, rows, cols)
                    assert_bits_equal(dout.download(np.float32, m * rows).reshape(m, rows), want,
                                      f"kind {kind} {rows}x{cols} m {m} chunks {on}")
                    dout.free()
                dw.free()
            # gate/up pair and three matrices in one launch
            rows = 2400
            wa, wb = make_weights(pkg, kind, rows, cols, 700 + kind), make_weights(pkg, kind, rows, cols, 800 + kind)
            dwa, dwb = ctx.to_device(wa), ctx.to_device(wb)
            for m in (1, 12):
                xs = _x(m * cols, 90 + m, 1.0)
                q = ob.quantize_act(kind, xs)
                da, db = ctx.alloc(m * rows * 4), ctx.alloc(m * rows * 4)
                ctx.matmul2(kind, da, db, dwa, dwb, ctx.to_device(q.view(np.uint8)), m, rows, cols)
                assert_bits_equal(da.download(np.float32, m * rows).reshape(m, rows), ob.matmul(pool, tab, kind, wa, q, m, rows, cols), f"pair a kind {kind} m {m} chunks {on}")
                assert_bits_equal(db.download(np.float32, m * rows).reshape(m, rows), ob.matmul(pool, tab, kind, wb, q, m, rows, cols), f"pair b kind {kind} m {m} chunks {on}")
            rows3 = (2048, 256, 512)
            ws = [make_weights(pkg, kind, r, cols, 900 + i) for i, r in enumerate(rows3)]
            xq = ob.quantize_act(kind, _x(cols, 4))
            douts = [ctx.alloc(r * 4) for r in rows3]
            ctx.matvec3((kind,) * 3, douts, [ctx.to_device(w) for w in ws], ctx.to_device(xq.view(np.uint8)), rows3, cols)
            for w, o, r in zip(ws, douts, rows3):
                assert_bits_equal(o.download(np.float32, r), ob.matvec(pool, tab, kind, w, xq, r, cols), f"three matrices, kind {kind} chunks {on}")
    finally:
        g.set_option(switch, 1)
    ctx.device_status()


# Short batches of K-quant products run with one lane per super-block against every activation
# row (gemv_stream_kernel<3>): here the switch point is raised so that batches up to 64 rows
# take that path, for every K-quant kind, a q/k/v launch of mixed kinds, residual adds through
# the model path being covered by the model tests; then the same shapes with the path off.
@pytest.mark.parametrize("kind", [Q4_K, Q5_K, Q6_K])
def test_short_batches_one_lane_per_block_bit_exact(pkg, ob, ctx, kind):
    spec = pkg.model.tiny("llama", n_layer=1)
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 16, 2)   # only to reach the process-wide switches
    pool, tab = ob.Pool(8), ob.detect_table()
    try:
        for on in (1, 0):
            g.set_option("wide_multi", on)
            g.set_option("wide_multi_work", 1 << 30)
            for rows, cols in ((37, 512), (600, 2048), (300, 5632), (2048, 768)):
                w = make_weights(pkg, kind, rows, cols, 40 + kind + rows)
                dw = ctx.to_device(w)
                for m in (2, 3, 7, 8, 17, 33, 64):
                    xs = _x(m * cols, 70 + m, 1.0)
                    q = ob.quantize_act(kind, xs)
                    want = ob.matmul(pool, tab, kind, w, q, m, rows, cols)
                    dout = ctx.alloc(m * rows * 4)
                    ctx.matmul(kind, dout, dw, ctx.to_device(q.view(np.uint8)), m, rows, cols)
                    assert_bits_equal(dout.download(np.float32, m * rows).reshape(m, rows), want, f"kind {kind} {rows}x{cols} m {m} on {on}")
                    dout.free()
                dw.free()
    finally:
        g.set_option("wide_multi", 1)
        g.set_option("wide_multi_work", 57344)
    ctx.device_status()


def test_matmul_large_tile_loop(pkg, ob, ctx):
    rows, cols, m = 1200, 2048, 5
    w = make_weights(pkg, Q4_K, rows, cols, 5)
    xs = _x(m * cols, 8, 1.0)
    want = ob.matmul(ob.Pool(8), ob.detect_table(), Q4_K, w, ob.quantize_q8_k(xs), m, rows, cols)
    assert_bits_equal(ctx.host_matmul(Q4_K, w, xs, m, rows, cols), want, "matmul 1200x2048 m5")


def test_dequant_rows(pkg, ob, ctx):
    cols, rows = 512, 11
    ids = np.array([0, 10, 3, 3, 7], dtype=np.int32)
    for kind in range(9):
        w = make_weights(pkg, kind, rows, cols, 90 + kind)
        rb = pkg.lib.row_bytes(kind, cols)
        dout = ctx.alloc(ids.size * cols * 4)
        ctx.dequant_rows(kind, ctx.to_device(w), ctx.to_device(ids), ids.size, cols, dout)
        got = dout.download(np.float32, ids.size * cols).reshape(ids.size, cols)
        for i, r in enumerate(ids):
            assert_bits_equal(got[i], ob.dequant_row(kind, w[r * rb:(r + 1) * rb].copy(), cols), f"dequant kind {kind}")


def test_rmsnorm_and_heads(pkg, ob, ctx):
    rng = np.random.default_rng(12)
    for n, m in ((2048, 1), (4096, 3), (256, 9), (8, 2)):
        x = (rng.standard_normal(n * m) * 3).astype(np.float32)
        w = (1 + rng.random(n) * 0.5).astype(np.float32)
        dx, dout = ctx.to_device(x), ctx.alloc(n * m * 4)
        ctx.rmsnorm(dout, dx, ctx.to_device(w), n, m, 1e-5)
        got = dout.download(np.float32, n * m).reshape(m, n)
        for i in range(m):
            assert_bits_equal(got[i], ob.rmsnorm(x[i * n:(i + 1) * n], w, 1e-5), f"rmsnorm n {n}")
    for hd, nh in ((64, 36), (128, 40), (32, 3)):
        x = (rng.standard_normal(hd * nh) * 2).astype(np.float32)
        w = (1 + rng.random(hd) * 0.5).astype(np.float32)
        dx = ctx.to_device(x)
        ctx.rmsnorm_heads(dx, ctx.to_device(w), nh, hd, 1e-6)
        assert_bits_equal(dx.download(np.float32, hd * nh), ob.rmsnorm_heads(x, w, nh, hd, 1e-6), "rmsnorm_heads")


def test_rope_silu_add(pkg, ob, ctx):
    rng = np.random.default_rng(13)
    for neox in (False, True):
        for hd, rot, nh, m in ((64, 64, 32, 1), (128, 128, 8, 5), (32, 16, 4, 3)):
            inv = ob.inv_freq(rot, 10000.0)
            cs = np.concatenate([ob.rope_cos_sin(inv, float(7 + i)) for i in range(m)])
            x = rng.standard_normal(m * nh * hd).astype(np.float32)
            dx = ctx.to_device(x)
            ctx.rope(dx, m, nh, hd, rot, ctx.to_device(cs), neox)
            want = np.concatenate([ob.rope(x[i * nh * hd:(i + 1) * nh * hd], nh, hd, rot, cs[i * rot:(i + 1) * rot], neox)
                                   for i in range(m)])
            assert_bits_equal(dx.download(np.float32, x.size), want, f"rope neox={neox} hd={hd}")
    h = (rng.standard_normal(5632 * 3) * 4).astype(np.float32)
    h[:4] = [0.0, -0.0, 88.5, -104.0]
    up = rng.standard_normal(h.size).astype(np.float32)
    dh = ctx.to_device(h)
    ctx.silu_mul(dh, ctx.to_device(up), h.size)
    assert_bits_equal(dh.download(np.float32, h.size), ob.silu_mul(h, up), "silu_mul")
    dx = ctx.to_device(h)
    ctx.add_inplace(dx, ctx.to_device(up), h.size)
    assert_bits_equal(dx.download(np.float32, h.size), ob.add_inplace(h, up), "add_inplace")


def test_gelu_mul_correctly_rounded_tanh(pkg, ob, ctx):
    """GeGLU gating (ops.rs:122-134). With tanh rounded correctly (the value a correctly
    rounded libm gives) device and oracle agree bit for bit over a dense sweep; against this
    host's own tanhf, which the reference would call here, they stay within one ulp of the
    gated value wherever tanhf itself is within one ulp."""
    L = ob.lib()
    v = np.concatenate([np.linspace(-12.0, 12.0, 1 << 19, dtype=np.float32),
                        np.array([0.0, -0.0, 1.0, -1.0, 1e-20, -1e-20, 30.0, -30.0, 1e30, -1e30], dtype=np.float32)])
    up = np.random.default_rng(2).standard_normal(v.size).astype(np.float32)
    dh = ctx.to_device(v)
    ctx.gelu_mul(dh, ctx.to_device(up), v.size)
    got = dh.download(np.float32, v.size)
    L.orc_set_tanh_mode(1)
    try:
        assert_bits_equal(got, ob.gelu_mul(v, up), "gelu_mul, correctly rounded tanh")
    finally:
        L.orc_set_tanh_mode(0)
    host = ob.gelu_mul(v, up)
    ulp = np.abs(got.view(np.int32).astype(np.int64) - host.view(np.int32).astype(np.int64))
    same = float(np.mean(ulp == 0))
    assert same > 0.9, same                      # this host's tanhf is usually the rounded value
    # known answers of the reference's own test (ops.rs:343-350)
    one = ctx.to_device(np.array([1.0, -1.0], dtype=np.float32))
    ctx.gelu_mul(one, ctx.to_device(np.array([2.0, 2.0], dtype=np.float32)), 2)
    r = one.download(np.float32, 2)
    assert abs(r[0] - 1.682384) < 1e-5 and abs(r[1] + 0.317616) < 1e-5


def test_expf_matches_host_libm(pkg, ob, ctx):
    """silu(v)*1 exposes expf(-v): compare the device expf with the oracle's libm over a
    dense sweep of the range softmax and SiLU use."""
    v = np.linspace(-104.0, 89.0, 1 << 20, dtype=np.float32)
    dh = ctx.to_device(v)
    ctx.silu_mul(dh, ctx.to_device(np.ones_like(v)), v.size)
    assert_bits_equal(dh.download(np.float32, v.size), ob.silu_mul(v, np.ones_like(v)), "expf sweep")


# crates/aot-kernels/src/ops.rs:602-636 plus GQA shapes of both configured models
@pytest.mark.parametrize("n_head,n_kv,hd", [(32, 4, 64), (32, 8, 128), (2, 1, 4), (40, 8, 64), (6, 2, 32), (3, 3, 16), (24, 2, 32), (4, 2, 80),
                                            (2, 1, 160), (2, 2, 256), (3, 1, 200)])
def test_attention_bit_exact(pkg, ob, ctx, n_head, n_kv, hd):
    ctxlen = 128
    kvd = n_kv * hd
    rng = np.random.default_rng(7)
    kc = (rng.random(ctxlen * kvd, dtype=np.float32) * 2 - 1)
    vc = (rng.random(ctxlen * kvd, dtype=np.float32) * 2 - 1)
    d = ob.Dims()
    d.n_head, d.n_kv_head, d.head_dim = n_head, n_kv, hd
    pool = ob.Pool(3)
    dk, dv = ctx.to_device(kc), ctx.to_device(vc)
    for pos in (0, 1, 7, 51, 52, 53, 100, 127):
        q = (rng.random(n_head * hd, dtype=np.float32) * 8 - 4)
        dout = ctx.alloc(n_head * hd * 4)
        for window in (0, 5):
            ctx.attention(dout, ctx.to_device(q), dk, dv, n_head, n_kv, hd, ctxlen, pos, 1, window)
            assert_bits_equal(dout.download(np.float32, n_head * hd),
                              ob.attention(pool, q, kc, vc, d, ctxlen, 0, pos, window), f"attention pos {pos} w {window}")
    # several rows per call: a CTA serves consecutive rows of one KV head (row counts that do
    # and do not fill the CTAs, a window that cuts differently into each row, a chunk
    # boundary inside the rows' ranges)
    for m, pos0, window in ((9, 40, 0), (1, 3, 0), (16, 0, 0), (7, 60, 5), (13, 57, 64), (64, 64, 0), (5, 123, 100)):
        q = (rng.random(m * n_head * hd, dtype=np.float32) * 8 - 4)
        dout = ctx.alloc(q.size * 4)
        ctx.attention(dout, ctx.to_device(q), dk, dv, n_head, n_kv, hd, ctxlen, pos0, m, window)
        assert_bits_equal(dout.download(np.float32, q.size), ob.attention_rows(pool, q, kc, vc, d, ctxlen, 0, pos0, m, window),
                          f"attention_rows m {m} pos0 {pos0} window {window}")


def test_argmax_first_maximum(pkg, ob, ctx):
    rng = np.random.default_rng(1)
    dtok = ctx.alloc(4)
    cases = [rng.standard_normal(32000).astype(np.float32), rng.standard_normal(151936).astype(np.float32),
             np.full(5000, -np.inf, dtype=np.float32), np.array([1.0, 7.0, 7.0, 3.0], dtype=np.float32)]
    tie = rng.standard_normal(40000).astype(np.float32)
    tie[[31999, 1234, 20000]] = 99.0
    cases.append(tie)
    nan = rng.standard_normal(3000).astype(np.float32)
    nan[5] = np.nan
    cases.append(nan)
    for x in cases:
        ctx.argmax(ctx.to_device(x), x.size, dtok)
        assert int(dtok.download(np.int32, 1)[0]) == ob.argmax(x)


def test_bad_arguments_are_reported_not_fatal(pkg, ctx):
    L = pkg.lib
    d = ctx.alloc(4096)
    with pytest.raises(pkg.AotCudaError) as e:
        ctx.matvec(Q4_K, d, d, d, 4, 100)  # cols not a multiple of 256
    assert e.value.status == L.ERR_BAD_ARG
    with pytest.raises(pkg.AotCudaError):
        ctx.matvec(Q4_K, d, d.at(8), d, 4, 256)  # misaligned weights
    with pytest.raises(pkg.AotCudaError):
        ctx.quantize_q8_k(d, 100, d)
    ctx.device_status()  # the context is still usable


# north_star: "integer per-block dot products are bit-exact" -- checked on the integers the
# production kernels themselves form (the streaming single-row product and the tcgen05 prompt
# product write them out while they compute), not on a separate checker kernel.
@pytest.mark.parametrize("kind", [Q4_K, Q5_K, Q6_K])
def test_streaming_product_exports_exact_block_sums(pkg, ob, ctx, kind):
    rows, cols = 300, 2048
    nb = cols // 256
    w = make_weights(pkg, kind, rows, cols, 900 + kind, "uniform")
    xq = ob.quantize_q8_k(_x(cols, 5 + kind))
    dsi, dsm = ctx.alloc(rows * nb * 4), ctx.alloc(rows * nb * 4)
    ctx.block_sums_of(0, kind, ctx.to_device(w), ctx.to_device(xq.view(np.uint8)), 1, rows, cols, dsi, dsm)
    si = dsi.download(np.int32, rows * nb).reshape(rows, nb)
    sm = dsm.download(np.int32, rows * nb).reshape(rows, nb)
    rb = pkg.lib.row_bytes(kind, cols)
    for r in range(rows):
        osi, osm = ob.block_sums(kind, w[r * rb:(r + 1) * rb].copy(), xq, cols)
        assert np.array_equal(si[r], osi), (kind, r)
        if kind != Q6_K:
            assert np.array_equal(sm[r], osm), (kind, r)
    ctx.device_status()


@pytest.mark.parametrize("kind", [Q4_K, Q5_K])
def test_tcgen05_product_exports_exact_block_sums(pkg, ob, ctx, kind):
    rows, cols, m = 150, 1024, 21   # a full and a partial 128-row tile, a partial token tile
    nb = cols // 256
    w = make_weights(pkg, kind, rows, cols, 950 + kind, "uniform")
    xs = _x(m * cols, 31 + kind)
    xq = ob.quantize_q8_k(xs)
    dsi, dsm = ctx.alloc(m * rows * nb * 4), ctx.alloc(m * rows * nb * 4)
    ctx.block_sums_of(1, kind, ctx.to_device(w), ctx.to_device(xq.view(np.uint8)), m, rows, cols, dsi, dsm)
    si = dsi.download(np.int32, m * rows * nb).reshape(m, rows, nb)
    sm = dsm.download(np.int32, m * rows * nb).reshape(m, rows, nb)
    rb = pkg.lib.row_bytes(kind, cols)
    for t in (0, 7, m - 1):
        xt = xq[t * nb:(t + 1) * nb]
        for r in (0, 1, 63, 127, 128, rows - 1):
            osi, osm = ob.block_sums(kind, w[r * rb:(r + 1) * rb].copy(), xt, cols)
            assert np.array_equal(si[t, r], osi) and np.array_equal(sm[t, r], osm), (kind, t, r)
    ctx.device_status()


# Prompt chunks through the tcgen05 kernel whatever the launch size (the library picks it by
# itself only when a launch fills the GPU): batched == per-token, bit for bit.
@pytest.mark.parametrize("kind", [Q4_K, Q5_K])
def test_tcgen05_product_bit_exact_when_forced(pkg, ob, ctx, kind):
    spec = pkg.model.tiny("llama", n_layer=1)
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 16, 4)   # any Gpu: the switch is process-wide
    g.set_option("tc_gemm", 2)
    try:
        pool, tab = ob.Pool(4), ob.detect_table()
        for rows, cols in ((37, 512), (300, 2048), (130, 5632)):
            w = make_weights(pkg, kind, rows, cols, 70 + kind + rows)
            for m in (8, 33, 64):
                xs = _x(m * cols, 60 + m, 1.0)
                q = ob.quantize_act(kind, xs)
                dout = ctx.alloc(m * rows * 4)
                ctx.matmul(kind, dout, ctx.to_device(w), ctx.to_device(q.view(np.uint8)), m, rows, cols)
                assert_bits_equal(dout.download(np.float32, m * rows).reshape(m, rows), ob.matmul(pool, tab, kind, w, q, m, rows, cols),
                                  f"tcgen05 matmul kind {kind} {rows}x{cols} m {m}")
    finally:
        g.set_option("tc_gemm", 1)
        g.close()
    ctx.device_status()


def test_scale_inplace(pkg, ctx):
    # ops.rs:138-142: x[i] *= s
    x = _x(5000, 77)
    d = ctx.to_device(x)
    ctx.scale_inplace(d, 0.37, 5000)
    assert_bits_equal(d.download(np.float32, 5000), x * np.float32(0.37), "scale_inplace")


# The shapes of the kernel sweep (4096 x 14336 for every kind at M = 1 and M = 64, and the
# 128256 x 4096 output-head shape for three kinds at M = 1), field-uniform blocks.
@pytest.mark.parametrize("kind", list(range(9)))
def test_sweep_shape_4096x14336_bit_exact(pkg, ob, ctx, kind):
    rows, cols = 4096, 14336
    pool, tab = ob.Pool(8), ob.detect_table()
    w = make_weights(pkg, kind, rows, cols, 500 + kind, "uniform")
    dw = ctx.to_device(w)
    for m in (1, 64):
        xs = _x(m * cols, 90 + m, 1.0)
        q = ob.quantize_act(kind, xs)
        want = ob.matmul(pool, tab, kind, w, q, m, rows, cols)
        dout = ctx.alloc(m * rows * 4)
        ctx.matmul(kind, dout, dw, ctx.to_device(q.view(np.uint8)), m, rows, cols)
        assert_bits_equal(dout.download(np.float32, m * rows).reshape(m, rows), want, f"kind {kind} 4096x14336 m {m}")
    ctx.device_status()


@pytest.mark.parametrize("kind", [Q4_K, Q6_K, Q8_0])
def test_sweep_shape_128256x4096_matvec_bit_exact(pkg, ob, ctx, kind):
    rows, cols = 128256, 4096
    w = make_weights(pkg, kind, rows, cols, 600 + kind, "uniform")
    xq = ob.quantize_act(kind, _x(cols, 3))
    want = ob.matvec(ob.Pool(8), ob.detect_table(), kind, w, xq, rows, cols)
    dout = ctx.alloc(rows * 4)
    ctx.matvec(kind, dout, ctx.to_device(w), ctx.to_device(xq.view(np.uint8)), rows, cols)
    assert_bits_equal(dout.download(np.float32, rows), want, f"kind {kind} 128256x4096")
    ctx.device_status()


def test_single_row_products_one_lane_per_block(pkg, ob, ctx):
    """The streaming kernel's two row arithmetics, one lane per super-block (the default for
    single matrices and q/k/v launches) and four lanes per super-block (gate/up pairs; here
    forced for everything by raising the switch point), against the oracle: every K-quant
    kind, block counts that are and are not powers of two, more blocks than lanes, a mixed
    q/k/v launch, and the 14336 x 4096 shape."""
    spec = pkg.model.tiny("llama", n_layer=1)
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 16, 2)   # only to reach the process-wide switch
    pool, tab = ob.Pool(4), ob.detect_table()
    try:
        for switch in (1, 1 << 30):
            g.set_option("wide_rows", switch)
            for kind in (Q4_K, Q5_K, Q6_K):
                for rows, cols in ((1, 256), (37, 512), (700, 2048), (300, 5632), (96, 768), (40, 12288)):
                    for mode in ("enc", "uniform"):
                        w = make_weights(pkg, kind, rows, cols, 3 * kind + rows, mode)
                        xq = ob.quantize_act(kind, _x(cols, rows + cols))
                        dout = ctx.alloc(rows * 4)
                        ctx.matvec(kind, dout, ctx.to_device(w), ctx.to_device(xq.view(np.uint8)), rows, cols)
                        assert_bits_equal(dout.download(np.float32, rows), ob.matvec(pool, tab, kind, w, xq, rows, cols),
                                          f"switch {switch}: kind {kind} {rows}x{cols} {mode}")
            cols, rows3, kinds = 2048, (2048, 256, 256), (Q4_K, Q5_K, Q6_K)
            ws = [make_weights(pkg, k, r, cols, 60 + i) for i, (k, r) in enumerate(zip(kinds, rows3))]
            xq = ob.quantize_q8_k(_x(cols, 4))
            douts = [ctx.alloc(r * 4) for r in rows3]
            ctx.matvec3(kinds, douts, [ctx.to_device(w) for w in ws], ctx.to_device(xq.view(np.uint8)), rows3, cols)
            for k, w, o, r in zip(kinds, ws, douts, rows3):
                assert_bits_equal(o.download(np.float32, r), ob.matvec(pool, tab, k, w, xq, r, cols), f"switch {switch}: mixed kinds, kind {k}")
    finally:
        g.set_option("wide_rows", 1)
    rows, cols = 14336, 4096
    for kind in (Q4_K, Q6_K):
        w = make_weights(pkg, kind, rows, cols, 11 + kind, "uniform")
        xq = ob.quantize_act(kind, _x(cols, 5))
        dout = ctx.alloc(rows * 4)
        ctx.matvec(kind, dout, ctx.to_device(w), ctx.to_device(xq.view(np.uint8)), rows, cols)
        assert_bits_equal(dout.download(np.float32, rows), ob.matvec(pool, tab, kind, w, xq, rows, cols), f"14336 x 4096 kind {kind}")
    g.close()
    ctx.device_status()
