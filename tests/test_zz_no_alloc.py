"""The allocation-free K-quant product (aotcu_matvec_k_static) against the ordinary
two-call route (aotcu_quantize_q8_k into a caller-owned buffer, then aotcu_matvec).

Some users of this library run inside a process that committed all of its device memory
at start-up and may not call the CUDA allocator afterwards; for them the quantized
activations live in an array inside the library itself. Both routes must give the same
bits, call after call, because the array keeps whatever the previous call left in it.

Collected last on purpose: a run that stops at the first failure has then already
exercised everything else.
"""
import numpy as np
import pytest

from conftest import assert_bits_equal, make_weights

pytestmark = pytest.mark.gpu

Q4_K, Q5_K, Q6_K = 6, 7, 8


@pytest.mark.parametrize("kind", [Q4_K, Q5_K, Q6_K])
def test_static_area_product_matches_two_call_route(pkg, ob, ctx, kind):
    rng = np.random.default_rng(100 + kind)
    pool, tab = ob.Pool(4), ob.detect_table()
    # Calls in a row with different widths: the widest vector the built-in area takes
    # (16384 columns, where a Q6_K row is 13,440 bytes), then narrower ones that read fewer
    # blocks than the call before wrote, so stale images sit behind them in the shared array.
    for rows, cols in ((33, 16384), (300, 5632), (257, 2048)):
        w = make_weights(pkg, kind, rows, cols, 40 + kind + cols)
        x = (rng.standard_normal(cols) * 2).astype(np.float32)
        dw, dx = ctx.to_device(w), ctx.to_device(x)
        # ordinary route: the caller owns the quantized copy
        xq = ctx.alloc(cols // 256 * 292)
        want_buf = ctx.alloc(rows * 4)
        ctx.quantize_q8_k(dx, cols, xq)
        ctx.matvec(kind, want_buf, dw, xq, rows, cols)
        want = want_buf.download(np.float32, rows)
        # ... and both must be the CPU oracle's bits, not merely each other's
        assert_bits_equal(want, ob.matvec(pool, tab, kind, w, ob.quantize_q8_k(x), rows, cols), f"two-call route vs oracle, kind {kind}")
        # allocation-free route, twice: same input, same answer, both times
        out = ctx.alloc(rows * 4)
        for _ in range(2):
            ctx.matvec_k_static(kind, out, dw, dx, rows, cols)
            assert_bits_equal(out.download(np.float32, rows), want, f"kind {kind} {rows}x{cols}")
    ctx.device_status()


def test_static_area_rejects_oversized_vectors(pkg, ctx):
    d = ctx.alloc(1 << 16)
    with pytest.raises(pkg.AotCudaError) as e:
        ctx.matvec_k_static(Q4_K, d, d, d, 1, 16384 + 256)
    assert e.value.status == pkg.lib.ERR_BAD_ARG and "16384" in str(e.value)
    with pytest.raises(pkg.AotCudaError):
        ctx.matvec_k_static(5, d, d, d, 1, 256)  # Q8_0 is not a K-quant
    ctx.device_status()
