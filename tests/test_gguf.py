"""GGUF reader / writer (aot-llm_b200/gguf.py) against a header written out by hand, the
reference's parsing rules (crates/aot-gguf/src/lib.rs:156-222) and its model checks
(crates/aot-codegen/src/model.rs:240-400); on a GPU, a model loaded from a file gives the
results of the model it was written from."""
import importlib
import struct

import numpy as np
import pytest

from conftest import assert_bits_equal


@pytest.fixture(scope="module")
def gg(pkg):
    return importlib.import_module("aot_llm_b200.gguf")


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def test_header_written_out_by_hand(gg):
    # magic, version 3, 1 tensor, 3 metadata pairs
    raw = b"GGUF" + struct.pack("<IQQ", 3, 1, 3)
    raw += _s("general.architecture") + struct.pack("<I", 8) + _s("llama")
    raw += _s("general.alignment") + struct.pack("<II", 4, 64)
    raw += _s("tokenizer.ggml.tokens") + struct.pack("<IIQ", 9, 8, 2) + _s("a") + _s("bc")
    raw += _s("blk.0.attn_q.weight") + struct.pack("<I", 2) + struct.pack("<QQ", 256, 3) + struct.pack("<IQ", 12, 0)
    pad = -len(raw) % 64
    data = bytes(range(256)) * 2
    blob = raw + b"\0" * pad + data[:3 * 144]
    g = gg.parse(blob)
    assert (g.version, g.alignment, g.data_offset) == (3, 64, len(raw) + pad)
    assert g.get("general.architecture") == "llama" and g.get("tokenizer.ggml.tokens") == ["a", "bc"]
    t = g.tensor("blk.0.attn_q.weight")
    assert (t.dims, t.ty, t.offset, t.cols(), t.rows(), t.n_bytes()) == ([256, 3], 12, 0, 256, 3, 3 * 144)
    # a prefix that covers the descriptors parses when the file length is given
    assert gg.parse(blob[:len(raw)], len(blob)).tensor("blk.0.attn_q.weight").n_bytes() == 432
    # the writer emits the same bytes for the same content
    again = gg.write([("general.architecture", "llama"), ("general.alignment", 64), ("tokenizer.ggml.tokens", ["a", "bc"])],
                     [("blk.0.attn_q.weight", [256, 3], 12, data[:3 * 144])], alignment=64)
    assert again[:len(blob)] == blob and not any(again[len(blob):])


def test_parse_rejects_what_the_reference_rejects(gg):
    ok = gg.write([("general.architecture", "llama")], [("t", [32], 0, b"\0" * 128)])
    assert gg.parse(ok).tensor("t").n_elements() == 32
    with pytest.raises(gg.GgufError):
        gg.parse(b"GGUX" + ok[4:])                                           # magic
    with pytest.raises(gg.GgufError):
        gg.parse(ok[:4] + struct.pack("<I", 1) + ok[8:])                     # version 1
    with pytest.raises(gg.GgufError):
        gg.parse(ok[:-1])                                                    # tensor out of bounds
    with pytest.raises(gg.GgufError):
        gg.parse(ok[:30])                                                    # truncated descriptors
    with pytest.raises(gg.GgufError):
        gg.parse(gg.write([("general.alignment", 48)], []))                  # not a power of two
    five = b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + _s("t") + struct.pack("<I", 5)
    with pytest.raises(gg.GgufError):
        gg.parse(five + b"\0" * 64)                                          # five dimensions
    unknown = b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + _s("t") + struct.pack("<IQIQ", 1, 32, 99, 0)
    with pytest.raises(gg.GgufError):
        gg.parse(unknown + b"\0" * 256)                                      # unknown tensor type
    badval = b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + _s("k") + struct.pack("<I", 13)
    with pytest.raises(gg.GgufError):
        gg.parse(badval + b"\0" * 64)                                        # unknown value type
    # version 2 files parse like version 3
    assert gg.parse(ok[:4] + struct.pack("<I", 2) + ok[8:]).version == 2


@pytest.mark.parametrize("arch,gguf_arch", [("llama", "llama"), ("qwen2", "qwen2"), ("qwen3", "qwen3"), ("gemma", "gemma3"),
                                            ("llama3", "llama")])
def test_model_round_trip(pkg, gg, arch, gguf_arch, tmp_path):
    kw = dict(n_layer=6) if arch == "gemma" else dict(n_layer=2)
    if arch == "llama3":
        # partial rotation, linear position scale and the frequency-factor tensor
        spec = pkg.model.build("llama3-file", dim=256, hidden=512, n_layer=2, n_head=8, n_kv_head=2, head_dim=32, vocab=384, seed=13,
                               rot_dim=16, rope_scale=8.0, rope_freqs=True, rope_base=500000.0, n_ctx_train=512)
    else:
        spec = pkg.model.tiny(arch, **kw)
    if arch == "gemma":
        # the file format fixes the pattern: every sixth layer is global (model.rs:190)
        spec = pkg.model.build("gemma-file", dim=256, hidden=512, n_layer=6, n_head=8, n_kv_head=2, head_dim=32, vocab=384, seed=11,
                               gelu=True, post_norms=True, embd_scale=True, qk_norm=True, rope_neox=True, rope_base=1e6, eps=1e-6,
                               swa_window=16, swa_pattern=6, tied_output=True, n_ctx_train=512)
    path = tmp_path / "m.gguf"
    path.write_bytes(gg.spec_to_gguf(spec, gguf_arch))
    got = gg.load_model(str(path))
    a, b = spec.head.dims, got.head.dims
    for f, _ in type(a)._fields_:
        va, vb = getattr(a, f), getattr(b, f)
        assert va == pytest.approx(vb, rel=1e-7), f
    assert [l.local_attn for l in got.layers] == [l.local_attn for l in spec.layers]
    assert bool(got.head.output.present) == bool(spec.head.output.present)

    def same(ta, tb, what):
        assert (ta.present, ta.kind, ta.rows, ta.cols, ta.len) == (tb.present, tb.kind, tb.rows, tb.cols, tb.len), what
        if ta.present:
            assert np.array_equal(spec.weights[ta.off:ta.off + ta.len], got.weights[tb.off:tb.off + tb.len]), what
            assert tb.off % 32 == 0

    for f in ("token_embd", "output_norm", "output", "rope_freqs"):
        same(getattr(spec.head, f), getattr(got.head, f), f)
    for i, (la, lb) in enumerate(zip(spec.layers, got.layers)):
        for f in pkg.lib.LAYER_TENSORS:
            same(getattr(la, f), getattr(lb, f), f"layer {i} {f}")


def test_model_checks(pkg, gg):
    spec = pkg.model.tiny("llama", n_layer=1)
    blob = gg.spec_to_gguf(spec, "llama")
    g = gg.parse(blob)
    w = np.frombuffer(blob, dtype=np.uint8, offset=g.data_offset)
    assert gg.model_spec(g, w).head.dims.n_layer == 1
    with pytest.raises(gg.GgufError):
        gg.model_spec(gg.parse(gg.spec_to_gguf(spec, "falcon")), w)          # unsupported architecture
    # a missing tensor, a wrong shape, LongRoPE factors, an odd rope dimension count
    md = list(g.metadata)
    ts = [(t.name, t.dims, t.ty, bytes(w[t.offset:t.offset + t.n_bytes()])) for t in g.tensors]
    with pytest.raises(gg.GgufError):
        g2 = gg.parse(gg.write(md, [t for t in ts if t[0] != "blk.0.ffn_down.weight"]))
        gg.model_spec(g2, w)
    with pytest.raises(gg.GgufError):
        g2 = gg.parse(gg.write(md, [(n, d[::-1] if n == "blk.0.ffn_up.weight" else d, ty, b) for n, d, ty, b in ts]))
        gg.model_spec(g2, w)
    with pytest.raises(gg.GgufError):
        g2 = gg.parse(gg.write(md, ts + [("rope_factors_long.weight", [16], 0, b"\0" * 64)]))
        gg.model_spec(g2, w)
    with pytest.raises(gg.GgufError):
        g2 = gg.parse(gg.write([(k, 31 if k == "llama.rope.dimension_count" else v) for k, v in md], ts))
        gg.model_spec(g2, w)
    # a fused q/k/v and gate/up file (Phi-3) is read as row views of the fused matrices
    d = spec.head.dims
    l = spec.layers[0]
    if l.wq.kind == l.wk.kind == l.wv.kind and l.gate.kind == l.up.kind:
        pass  # (kinds of the tiny model differ per matrix; the view arithmetic is checked below on offsets)
    t = pkg.lib.Tensor(kind=pkg.lib.Q4_K, present=1, off=1024, len=10 * 144, rows=10, cols=256)
    v = gg._rows_view(t, 3, 4)
    assert (v.off, v.len, v.rows, v.cols) == (1024 + 3 * 144, 4 * 144, 4, 256)


@pytest.mark.gpu
def test_model_from_file_runs_like_the_model_it_was_written_from(pkg, gg, ob, ctx, tmp_path):
    spec = pkg.model.tiny("qwen3", n_layer=2)
    path = tmp_path / "m.gguf"
    path.write_bytes(gg.spec_to_gguf(spec, "qwen3"))
    got = gg.load_model(str(path))
    toks = [5, 17, 300, 42, 7, 9, 1, 250, 33]
    om = ob.model_from_spec(spec, 32, 16, n_threads=2)
    om.forward_batch(toks, 0, True)
    g = pkg.Gpu(ctx, got.head, got.layers, got.weights, 32, 16)
    g.forward_batch(toks, 0, True)
    assert_bits_equal(g.logits(), om.logits(), "logits of the model loaded from a GGUF file")
    g.forward(int(np.argmax(g.logits())), len(toks), True)
    om.forward(ob.argmax(om.logits()), len(toks), True)
    assert_bits_equal(g.logits(), om.logits(), "decode step of the model loaded from a GGUF file")
    g.close()
