"""A host written in C against include/aot_cuda.h alone (aot-llm_b200/bindings/c/client.c):
the header is valid C11, the library links from C, the struct layouts are the ones the
ctypes binding uses, and on a GPU a model driven from C gives the Python binding's results."""
import ctypes as C
import os
import shutil
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "aot-llm_b200" / "bindings" / "c" / "client.c"


def _fnv1a(b: bytes) -> int:
    h = 1469598103934665603
    for x in b:
        h = ((h ^ x) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


@pytest.fixture(scope="module")
def client(pkg, tmp_path_factory):
    gcc = shutil.which("gcc")
    if not gcc:
        pytest.skip("no C compiler")
    libdir = Path(pkg.lib.load()._name).resolve().parent
    exe = tmp_path_factory.mktemp("cclient") / "client"
    cmd = [gcc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", f"-I{ROOT / 'include'}", "-o", str(exe), str(SRC),
           f"-L{libdir}", "-l:libaot_cuda.so", f"-Wl,-rpath,{libdir}", "-Wl,--allow-shlib-undefined"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_header_is_c11_and_layouts_match_the_ctypes_binding(pkg, client):
    r = subprocess.run([str(client), "--abi"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.splitlines()
    assert lines[0].startswith("version ") and pkg.lib.load().aotcu_version().decode() in lines[0]
    sizes = dict(zip(lines[1].split()[1::2], map(int, lines[1].split()[2::2])))
    assert sizes == {"tensor": C.sizeof(pkg.lib.Tensor), "dims": C.sizeof(pkg.lib.Dims), "layer": C.sizeof(pkg.lib.Layer),
                     "head": C.sizeof(pkg.lib.ModelHead)}
    assert lines[2] in ("init 0", "init -2")      # a device, or AOTCU_ERR_CUDA without one: never a crash


@pytest.mark.gpu
def test_c_host_matches_python_host(pkg, ctx, client, tmp_path):
    spec = pkg.model.tiny("qwen3", n_layer=2)
    path = tmp_path / "model.bin"
    with open(path, "wb") as f:
        f.write(bytes(spec.head))
        for l in spec.layers:
            f.write(bytes(l))
        f.write(spec.weights.tobytes())
    prompt, n_decode, n_ctx = [5, 17, 300, 42, 7], 6, 32
    r = subprocess.run([str(client), str(path), str(n_ctx), str(n_decode), *map(str, prompt)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = dict(l.split(": ", 1) for l in r.stdout.strip().splitlines())
    g = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, n_ctx, len(prompt))
    g.forward_batch(prompt, 0, True)
    toks = list(prompt)
    for _ in range(n_decode):
        toks.append(int(np.argmax(g.logits())))
        g.forward(toks[-1], len(toks) - 1, True)
    assert out["tokens"].split() == [str(t) for t in toks[len(prompt):]]
    assert int(out["logits"], 16) == _fnv1a(g.logits().tobytes())
    blob = g.kv_save(toks, len(toks) - 1)
    h, n = out["kv"].split()
    assert int(h, 16) == _fnv1a(blob) and int(n) == len(blob)
    g.close()
