"""Whole-step parity: the interpreted forward pass on the GPU against the oracle's."""
import os

import numpy as np
import pytest

from conftest import assert_bits_equal

pytestmark = pytest.mark.gpu


def _run_both(pkg, ob, ctx, spec, tokens, n_ctx=64, max_batch=16):
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, max_batch)
    om = ob.model_from_spec(spec, n_ctx, max_batch, n_threads=4)
    return g, om


@pytest.mark.parametrize("arch", ["llama", "qwen3", "qwen2"])
def test_tiny_models_all_kinds_bit_exact(pkg, ob, ctx, arch):
    spec = pkg.model.tiny(arch, n_layer=3)
    tokens = [5, 17, 300, 42, 7, 7, 1]
    g, om = _run_both(pkg, ob, ctx, spec, tokens)
    for graph in (0, 1):
        g.set_option("graph", graph)
        for pos, t in enumerate(tokens):
            g.forward(t, pos, True)
            om.forward(t, pos, True)
            assert_bits_equal(g.read("X"), om.buf("x"), f"{arch} x pos {pos} graph {graph}")
            assert_bits_equal(g.logits(), om.logits(), f"{arch} logits pos {pos} graph {graph}")
    d = spec.head.dims
    kvd = d.n_kv_head * d.head_dim
    assert_bits_equal(g.read("KCache", len(tokens) * kvd), om.buf("k_cache")[:len(tokens) * kvd], "k cache layer 0")
    assert_bits_equal(g.read("VCache", len(tokens) * kvd), om.buf("v_cache")[:len(tokens) * kvd], "v cache layer 0")
    # batched prompt path == oracle's batched path == single-token path
    g2, om2 = _run_both(pkg, ob, ctx, spec, tokens)
    g2.forward_batch(tokens, 0, True)
    om2.forward_batch(tokens, 0, True)
    assert_bits_equal(g2.logits(), om2.logits(), f"{arch} forward_batch")
    assert_bits_equal(g2.logits(), g.logits(), f"{arch} batch vs single")
    assert_bits_equal(g2.read("Bx", len(tokens) * d.dim), om2.buf("bx")[:len(tokens) * d.dim], "bx")
    # continue token by token after a batch, then another batch at an offset
    g2.forward(9, len(tokens), True)
    om2.forward(9, len(tokens), True)
    assert_bits_equal(g2.logits(), om2.logits(), "decode after batch")
    g2.forward_batch([4, 5, 6], len(tokens) + 1, True)
    om2.forward_batch([4, 5, 6], len(tokens) + 1, True)
    assert_bits_equal(g2.logits(), om2.logits(), "second batch")
    ctx.device_status()


def test_greedy_generate_on_device_matches_oracle(pkg, ob, ctx):
    spec = pkg.model.tiny("llama", n_layer=3)
    prompt = [3, 99, 250, 8]
    g, om = _run_both(pkg, ob, ctx, spec, prompt, n_ctx=64)
    g.forward_batch(prompt, 0, True)
    om.forward_batch(prompt, 0, True)
    first = ob.argmax(om.logits())
    assert int(np.argmax(g.logits())) == first
    n = 40
    ids, ms = g.generate(first, len(prompt), n)
    want, tok = [], first
    for i in range(n):
        om.forward(tok, len(prompt) + i, True)
        tok = ob.argmax(om.logits())
        want.append(tok)
    assert ids.tolist() == want
    assert ms > 0 and g.dispatches() > 0


def test_operator_level_api_matches_step(pkg, ob, ctx):
    """Driving one block through the Gpu operator calls (the sequence the reference's
    emit_gpu_forwards writes) gives the same bits as aotcu_forward."""
    spec = pkg.model.tiny("llama", n_layer=1, kinds=lambda l, t: 6 if t != "output" else 8)
    d = spec.head.dims
    g, om = _run_both(pkg, ob, ctx, spec, [])
    om.forward(11, 0, False)
    om.forward(12, 1, False)
    g.forward(11, 0, False)
    l = spec.layers[0]
    x0 = ob.dequant_row(spec.head.token_embd.kind,
                        spec.weights[spec.head.token_embd.off + 12 * pkg.lib.row_bytes(6, d.dim):][:pkg.lib.row_bytes(6, d.dim)].copy(), d.dim)
    g.begin()
    g.write("X", x0)
    g.rmsnorm("Xb", "X", l.attn_norm, d.dim, 1, d.eps)
    g.mv3(["Q", "K", "V"], [l.wq, l.wk, l.wv], "Xb")
    g.qk_post(0, 1)
    g.attention("Xb", "Q", 0, 1)
    g.mv("X", l.wo, "Xb", accumulate=True)
    g.rmsnorm("Xb", "X", l.ffn_norm, d.dim, 1, d.eps)
    g.gate_up("Hb", l.gate, l.up, "Xb")
    g.mv("X", l.down, "Hb", accumulate=True)
    g.finish()
    assert_bits_equal(g.read("X"), om.buf("x"), "operator-level block")


def test_forward_bounds_match_generated_asserts(pkg, ctx):
    spec = pkg.model.tiny("llama", n_layer=1)
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 8, 4)
    for bad in (lambda: g.forward(spec.head.dims.vocab, 0), lambda: g.forward(1, 8),
                lambda: g.forward_batch([1] * 5, 0), lambda: g.forward_batch([1, 2], 7)):
        with pytest.raises(pkg.AotCudaError):
            bad()
    g.forward(1, 0)


def test_tinyllama_shape_greedy_128_identical(pkg, ob, ctx):
    """Benchmark configuration 1: TinyLlama-shaped Q4_K_M model, 6-token prompt, 128 greedy tokens."""
    spec = pkg.model.tinyllama()
    prompt = np.random.default_rng(7).integers(0, 32000, 6).tolist()
    n_ctx, n_gen = 160, 128
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 8)
    om = ob.model_from_spec(spec, n_ctx, 8)
    g.forward_batch(prompt, 0, True)
    om.forward_batch(prompt, 0, True)
    assert_bits_equal(g.logits(), om.logits(), "prompt logits")
    first = ob.argmax(om.logits())
    ids, ms = g.generate(first, len(prompt), n_gen - 1)
    want, tok = [], first
    for i in range(n_gen - 1):
        om.forward(tok, len(prompt) + i, True)
        tok = ob.argmax(om.logits())
        want.append(tok)
    assert ids.tolist() == want
    assert_bits_equal(g.logits(), om.logits(), "final logits")
    print(f"\n[tinyllama-shape] {n_gen - 1} decode steps in {ms:.1f} ms -> {(n_gen - 1) / ms * 1e3:.0f} tok/s")


def _kquant_kinds(layer, tensor):
    if tensor == "output":
        return 8
    name = "gate" if tensor == "up" else tensor  # gate and up share a kind (fused launch)
    return [6, 8, 7][(layer + len(name)) % 3]  # Q4_K / Q6_K / Q5_K mix


@pytest.mark.parametrize("arch", ["llama", "qwen3"])
def test_one_kernel_decode_step_bit_exact(pkg, ob, ctx, arch):
    """The persistent one-kernel decode step against the oracle and against the
    per-operator path, position by position, then a greedy run on the device."""
    spec = pkg.model.tiny(arch, n_layer=3, kinds=_kquant_kinds, dim=512, hidden=768, vocab=600)
    n_ctx = 96
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 8)
    om = ob.model_from_spec(spec, n_ctx, 8, n_threads=4)
    tokens = [5, 17, 300, 42, 7, 7, 1, 599, 0]
    for mega in (1, 0):
        g.set_option("mega", mega)
        for graph in (0, 1):
            g.set_option("graph", graph)
            om2 = ob.model_from_spec(spec, n_ctx, 8, n_threads=4)
            for pos, t in enumerate(tokens):
                g.forward(t, pos, True)
                om2.forward(t, pos, True)
                assert_bits_equal(g.read("X"), om2.buf("x"), f"{arch} x pos {pos} mega {mega} graph {graph}")
                assert_bits_equal(g.logits(), om2.logits(), f"{arch} logits pos {pos} mega {mega} graph {graph}")
    g.set_option("mega", 1)
    g.set_option("graph", 1)
    prompt = tokens[:4]
    g.forward_batch(prompt, 0, True)
    om.forward_batch(prompt, 0, True)
    first = ob.argmax(om.logits())
    n = 70
    ids, ms = g.generate(first, len(prompt), n)
    want, tok = [], first
    for i in range(n):
        om.forward(tok, len(prompt) + i, True)
        tok = ob.argmax(om.logits())
        want.append(tok)
    assert ids.tolist() == want
    assert_bits_equal(g.logits(), om.logits(), "logits after the greedy run")
    ctx.device_status()


@pytest.mark.gpu
@pytest.mark.parametrize("arch", ["llama", "qwen3"])
def test_prompt_chunks_on_tensor_core_tiles_bit_exact(pkg, ob, ctx, arch):
    """Prompt chunks of 8..64 tokens (q/k/v, gate/up pair, accumulate epilogues on the
    tensor-core kernel) against the oracle, then decode from the cache they left."""
    spec = pkg.model.tiny(arch, n_layer=2, kinds=_kquant_kinds, dim=512, hidden=768, vocab=600)
    n_ctx = 160
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 64)
    om = ob.model_from_spec(spec, n_ctx, 64, n_threads=4)
    rng = np.random.default_rng(11)
    pos = 0
    for n in (64, 21, 8, 40):
        toks = rng.integers(0, 600, n).tolist()
        g.forward_batch(toks, pos, True)
        om.forward_batch(toks, pos, True)
        assert_bits_equal(g.logits(), om.logits(), f"{arch} logits after a chunk of {n} at {pos}")
        pos += n
    for t in (3, 9):
        g.forward(t, pos, True)
        om.forward(t, pos, True)
        assert_bits_equal(g.logits(), om.logits(), f"{arch} decode at {pos} after the prompt chunks")
        pos += 1
    ctx.device_status()


@pytest.mark.gpu
def test_prepared_tensor_core_operands_bit_exact(pkg, ob, ctx):
    """Q4_K / Q5_K layer matrices expanded once into tensor-core operand tiles (the default
    when memory allows) against the per-launch unpacking and against the oracle: ragged
    row counts (rows that do not fill a 128-row tile), Q5_K high bits, chunks of 8..64
    tokens, accumulate and gate/up epilogues."""
    Q4_K, Q5_K, Q6_K = pkg.lib.Q4_K, pkg.lib.Q5_K, pkg.lib.Q6_K
    kinds = lambda l, t: {"wv": Q6_K, "wo": Q5_K, "down": Q5_K if l % 2 else Q4_K, "output": Q6_K}.get(t, Q4_K)
    spec = pkg.model.build("prep", dim=512, hidden=1280, n_layer=2, n_head=8, n_kv_head=1, head_dim=64, vocab=600, seed=9,
                           kinds=kinds, n_ctx_train=256)
    n_ctx = 160
    om = ob.model_from_spec(spec, n_ctx, 64, n_threads=4)
    g1 = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 64)
    g0 = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 64)
    g1.set_option("tc_gemm", 2)      # the model is small: send every Q4_K / Q5_K launch to the tensor-core kernels
    g0.set_option("prepared_operands", 0)
    rng = np.random.default_rng(12)
    pos = 0
    for n in (64, 9, 33, 8):
        toks = rng.integers(0, 600, n).tolist()
        for g in (g1, g0):
            g.forward_batch(toks, pos, True)
        om.forward_batch(toks, pos, True)
        assert_bits_equal(g1.logits(), om.logits(), f"prepared operands: logits after a chunk of {n} at {pos}")
        assert_bits_equal(g0.logits(), om.logits(), f"per-launch unpacking: logits after a chunk of {n} at {pos}")
        assert_bits_equal(g1.read("KCache"), g0.read("KCache"), "K cache")
        pos += n
    assert g1.set_option("prepared_bytes", 0) > 0 and g0.set_option("prepared_bytes", 0) == 0
    # switching the operands off frees them and keeps the results
    g1.set_option("prepared_operands", 0)
    assert g1.set_option("prepared_bytes", 0) == 0
    toks = rng.integers(0, 600, 16).tolist()
    g1.forward_batch(toks, pos, True)
    om.forward_batch(toks, pos, True)
    assert_bits_equal(g1.logits(), om.logits(), "after switching prepared operands off")
    g1.set_option("tc_gemm", 1)      # back to the default: by size
    g1.close()
    g0.close()
    ctx.device_status()


@pytest.mark.gpu
@pytest.mark.parametrize("n_head,n_kv,hd", [(4, 1, 128), (16, 4, 80), (40, 8, 64)])
def test_heads_shared_by_several_ctas_bit_exact(pkg, ob, ctx, n_head, n_kv, hd):
    """Once a head's cached rows outgrow one CTA's staging area, the one-kernel step deals
    each head's positions (scores) and dimensions (value mix) out to several CTAs. Few heads
    of 128 (the per-rank shape of a sharded 8B model: 37 CTAs per head, 16-wide slices), a
    head width that is not a power of two (five slices of 16), and a head count that leaves
    three CTAs per head of which two mix values."""
    spec = pkg.model.build("split", dim=512, hidden=768, n_layer=2, n_head=n_head, n_kv_head=n_kv, head_dim=hd, vocab=600,
                           seed=31, kinds=_kquant_kinds, n_ctx_train=512, qk_norm=(hd == 128), rope_neox=(hd == 128))
    n_ctx, n_prompt, n_gen = 384, 320, 5
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 64)
    assert g.set_option("mega_available", 0)
    om = ob.model_from_spec(spec, n_ctx, 64, n_threads=min(8, os.cpu_count() or 1))
    toks = np.random.default_rng(hd).integers(0, 600, n_prompt).tolist()
    for c0 in range(0, n_prompt, 64):
        g.forward_batch(toks[c0:c0 + 64], c0, c0 + 64 == n_prompt)
        om.forward_batch(toks[c0:c0 + 64], c0, c0 + 64 == n_prompt)
    tok = ob.argmax(om.logits())
    for i in range(n_gen):
        g.forward(tok, n_prompt + i, True)
        om.forward(tok, n_prompt + i, True)
        assert_bits_equal(g.read("X"), om.buf("x"), f"x at position {n_prompt + i}")
        assert_bits_equal(g.logits(), om.logits(), f"logits at position {n_prompt + i}")
        tok = ob.argmax(om.logits())
    ids, _ = g.generate(tok, n_prompt + n_gen, 4)
    want = []
    for i in range(4):
        om.forward(tok, n_prompt + n_gen + i, True)
        tok = ob.argmax(om.logits())
        want.append(tok)
    assert ids.tolist() == want
    ctx.device_status()


@pytest.mark.gpu
@pytest.mark.timeout(600)
def test_long_context_decode_bit_exact(pkg, ob, ctx):
    """Near the end of a 2048-position context: prompt chunks of 64 fill the cache, then the
    one-kernel step decodes with ~2000 cached positions per head (many staged K/V chunks, the
    exact softmax sum over two thousand terms). Four layers of the TinyLlama shape keep the
    CPU side of the comparison short."""
    spec = pkg.model.tinyllama(n_layer=4)
    n_ctx, n_prompt, n_gen = 2048, 1984, 6
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 64)
    om = ob.model_from_spec(spec, n_ctx, 64, n_threads=min(16, os.cpu_count() or 1))
    toks = np.random.default_rng(21).integers(0, 32000, n_prompt).tolist()
    for c0 in range(0, n_prompt, 64):
        last = c0 + 64 == n_prompt
        g.forward_batch(toks[c0:c0 + 64], c0, last)
        om.forward_batch(toks[c0:c0 + 64], c0, last)
    assert_bits_equal(g.logits(), om.logits(), "logits after the 1984-token prompt")
    first = ob.argmax(om.logits())
    ids, _ = g.generate(first, n_prompt, n_gen)
    want, tok = [], first
    for i in range(n_gen):
        om.forward(tok, n_prompt + i, True)
        tok = ob.argmax(om.logits())
        want.append(tok)
    assert ids.tolist() == want
    assert_bits_equal(g.logits(), om.logits(), "logits at position 1989")
    ctx.device_status()


@pytest.mark.gpu
@pytest.mark.parametrize("arch", ["llama", "qwen2", "qwen3"])
def test_dependent_launch_switch_keeps_results(pkg, ob, ctx, arch):
    """The "pdl" switch lets every kernel of the per-operator path start while its predecessor
    drains; each kernel waits for the predecessor's results before it touches them, so the
    output is unchanged bit for bit (prompt chunk, per-token steps, with and without graphs)."""
    spec = pkg.model.tiny(arch, n_layer=3)
    n_ctx = 96
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 16)
    om = ob.model_from_spec(spec, n_ctx, 16, n_threads=4)
    g.set_option("pdl", 1)
    if g.set_option("mega_available", 0):
        g.set_option("mega", 0)
    prompt = [5, 17, 300, 42, 7, 7, 1, 250, 0, 33, 91, 2]
    g.forward_batch(prompt, 0, True)
    om.forward_batch(prompt, 0, True)
    assert_bits_equal(g.logits(), om.logits(), f"{arch} prompt logits with dependent launches")
    tok, pos = ob.argmax(om.logits()), len(prompt)
    for graph in (0, 1):
        g.set_option("graph", graph)
        for _ in range(6):
            g.forward(tok, pos, True)
            om.forward(tok, pos, True)
            assert_bits_equal(g.logits(), om.logits(), f"{arch} logits at {pos} graph {graph} with dependent launches")
            tok, pos = ob.argmax(om.logits()), pos + 1
    g.set_option("pdl", 0)
    ctx.device_status()


@pytest.mark.gpu
@pytest.mark.timeout(900)
def test_qwen3_8b_shape_prompt_and_decode_bit_exact(pkg, ob, ctx):
    """Benchmark configuration 3's shape (dim 4096, hidden 12288, 32 query / 8 KV heads of 128,
    per-head q/k RMSNorm, NEOX RoPE, vocabulary 151936, Q4_K_M mix) with three layers: a
    64-token prompt chunk, then greedy tokens through the one-kernel step, bit-equal to the
    oracle at every step."""
    spec = pkg.model.qwen3_8b(n_layer=3)
    n_ctx, n_prompt, n_gen = 128, 64, 12
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 64)
    assert g.set_option("mega_available", 0) == 1, "the one-kernel step must accept the 8B shape"
    om = ob.model_from_spec(spec, n_ctx, 64, n_threads=min(16, os.cpu_count() or 1))
    toks = np.random.default_rng(9).integers(0, 151936, n_prompt).tolist()
    g.forward_batch(toks, 0, True)
    om.forward_batch(toks, 0, True)
    assert_bits_equal(g.logits(), om.logits(), "logits after the prompt chunk")
    tok = ob.argmax(om.logits())
    for i in range(3):   # step by step, comparing the residual stream as well
        g.forward(tok, n_prompt + i, True)
        om.forward(tok, n_prompt + i, True)
        assert_bits_equal(g.read("X"), om.buf("x"), f"x at {n_prompt + i}")
        assert_bits_equal(g.logits(), om.logits(), f"logits at {n_prompt + i}")
        tok = ob.argmax(om.logits())
    ids, _ = g.generate(tok, n_prompt + 3, n_gen)
    want = []
    for i in range(n_gen):
        om.forward(tok, n_prompt + 3 + i, True)
        tok = ob.argmax(om.logits())
        want.append(tok)
    assert ids.tolist() == want
    assert_bits_equal(g.logits(), om.logits(), "final logits")
    ctx.device_status()


@pytest.mark.gpu
def test_bounded_wait_expires_and_the_context_stays_usable(pkg, ob, ctx):
    """Every wait inside the one-kernel step is bounded. With the limit lowered to a single
    poll the step cannot finish: it must return (nothing hangs), report a timeout, and leave
    the context usable: with the limit restored the same position decodes bit-equal to the
    oracle, and steps queued behind a failed one drain without working."""
    spec = pkg.model.tiny("llama", n_layer=3, kinds=_kquant_kinds, dim=512, hidden=768, vocab=600)
    n_ctx = 64
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 8)
    om = ob.model_from_spec(spec, n_ctx, 8, n_threads=4)
    prompt = [5, 17, 300, 42]
    g.forward_batch(prompt, 0, True)
    om.forward_batch(prompt, 0, True)
    tok = ob.argmax(om.logits())
    g.set_option("spin_limit", 1)
    with pytest.raises(pkg.AotCudaError) as e:
        g.generate(tok, len(prompt), 5)      # five queued steps: the first gives up, the rest drain
    assert e.value.status == pkg.lib.ERR_TIMEOUT, e.value
    g.set_option("spin_limit", 1 << 21)
    ctx.device_status()                       # the error word was consumed with the failed call
    for i in range(3):
        g.forward(tok, len(prompt) + i, True)
        om.forward(tok, len(prompt) + i, True)
        assert_bits_equal(g.logits(), om.logits(), f"logits at {len(prompt) + i} after the expired wait")
        tok = ob.argmax(om.logits())
    ctx.device_status()


@pytest.mark.gpu
def test_context_closed_before_its_gpu(pkg):
    """Closing a context releases the Gpus still alive on it; closing (or collecting) such a
    Gpu afterwards is a no-op instead of a use after free."""
    spec = pkg.model.tiny("llama", n_layer=1)
    ctx2 = pkg.Context(0)
    g = pkg.Gpu(ctx2, spec.head, spec.layers, spec.weights, 32, 4)
    g.forward(1, 0, True)
    first = g.logits().copy()
    ctx2.close()
    assert g.h is None
    g.close()
    del g
    ctx3 = pkg.Context(0)
    g3 = pkg.Gpu(ctx3, spec.head, spec.layers, spec.weights, 32, 4)
    g3.forward(1, 0, True)
    assert_bits_equal(g3.logits(), first, "same model on a fresh context")
    g3.close()
    ctx3.close()


@pytest.mark.gpu
def test_gemma_shape_geglu_post_norms_sliding_window(pkg, ob, ctx):
    """The Gemma switches together: GeGLU gating, norms after attention and FFN, scaled
    embedding, q/k norm, a tied output head and sliding-window layers with their own RoPE
    base (window 16, so positions beyond it drop out of the local layers). With tanh
    correctly rounded on both sides every buffer is bit-identical; with this host's tanhf
    (what the reference would call here) the logits agree to the floating-point tolerance."""
    spec = pkg.model.tiny("gemma", n_layer=3)
    assert [l.local_attn for l in spec.layers] == [1, 1, 0]
    n_ctx = 64
    toks = np.random.default_rng(5).integers(0, 384, 40).tolist()
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, 16)
    L = ob.lib()
    for mode in (1, 0):
        L.orc_set_tanh_mode(mode)
        try:
            om = ob.model_from_spec(spec, n_ctx, 16, n_threads=4)
            for c0 in range(0, 32, 16):
                g.forward_batch(toks[c0:c0 + 16], c0, True)
                om.forward_batch(toks[c0:c0 + 16], c0, True)
            for pos in range(32, 40):
                g.forward(toks[pos], pos, True)
                om.forward(toks[pos], pos, True)
                lg, lo = g.logits(), om.logits()
                if mode == 1:
                    assert_bits_equal(g.read("X"), om.buf("x"), f"x at position {pos}")
                    assert_bits_equal(lg, lo, f"logits at position {pos}")
                else:
                    assert float(np.max(np.abs(lg - lo))) <= 1e-3 * float(np.max(np.abs(lo)))   # tolerance for f32 outputs
                    assert int(np.argmax(lg)) == int(np.argmax(lo))
        finally:
            L.orc_set_tanh_mode(0)
    g.close()
    ctx.device_status()


@pytest.mark.gpu
def test_rope_variants_partial_rotation_linear_scale_frequency_factors(pkg, ob, ctx):
    """RoPE as the remaining model files use it: only part of each head rotated
    (rope.dimension_count < head_dim), positions divided by a linear scale factor, and the
    per-frequency divisors of Llama 3 files (rope_freqs.weight); both pair layouts. Prompt
    chunk, per-operator steps and the one-kernel step against the oracle."""
    for neox in (False, True):
        spec = pkg.model.build("rope", dim=512, hidden=768, n_layer=2, n_head=8, n_kv_head=2, head_dim=64, vocab=600, seed=21,
                               kinds=_kquant_kinds, n_ctx_train=256, rot_dim=32, rope_scale=4.0, rope_freqs=True, rope_neox=neox,
                               rope_base=500000.0)
        assert spec.head.rope_freqs.present and spec.head.dims.rot_dim == 32
        g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 64, 16)
        om = ob.model_from_spec(spec, 64, 16, n_threads=4)
        toks = np.random.default_rng(3).integers(0, 600, 20).tolist()
        g.forward_batch(toks[:12], 0, True)
        om.forward_batch(toks[:12], 0, True)
        assert_bits_equal(g.logits(), om.logits(), f"prompt chunk, neox={neox}")
        for mega in (1, 0):
            g.set_option("mega", mega)
            for pos in range(12 + 4 * (1 - mega), 16 + 4 * (1 - mega)):
                g.forward(toks[pos], pos, True)
                om.forward(toks[pos], pos, True)
                assert_bits_equal(g.logits(), om.logits(), f"decode at {pos}, neox={neox}, one-kernel step {mega}")
        g.close()
    ctx.device_status()
