"""Generates tests/golden/dots.npz: for every weight kind a few rows of seeded blocks, one
activation vector, and what the CPU oracle computes for them (quantized activations,
integer block sums, f32 dot products of the AVX2+F16C table, dequantized rows).

Run from the repository root:  python tests/golden/make_golden.py
The reference itself holds no literal output vectors for this path (its tests draw
seeded random data), so these pins are produced by the restatement in oracle/ after it
passed the reference's known-answer tests (tests/test_oracle_pins.py).
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as graft  # noqa: E402

graft.build()
pkg = graft.import_package()
from oracle import binding as ob  # noqa: E402

L = pkg.lib
out = {}
rows = 4
for kind in range(9):
    cols = 512 if L.BLOCK[kind] > 1 else 72
    for mode in ("enc", "uniform"):
        if mode == "uniform" and kind < 3:
            continue
        w = np.empty(rows * L.row_bytes(kind, cols), dtype=np.uint8)
        if mode == "enc":
            L.check(L.load().aotcu_synth_tensor(kind, rows, cols, 1.0, 0.0, 1000 + kind, L.ptr(w)))
        else:
            L.check(L.load().aotcu_synth_blocks(kind, rows * cols // L.BLOCK[kind], 2000 + kind, L.ptr(w)))
        x = (np.random.default_rng(3000 + kind).standard_normal(cols) * 1.5).astype(np.float32)
        xq = ob.quantize_act(kind, x)
        key = f"{L.KIND_NAMES[kind]}_{mode}"
        out[key + "_w"] = w
        out[key + "_x"] = x
        out[key + "_xq"] = np.frombuffer(xq.tobytes(), dtype=np.uint8)
        rb = L.row_bytes(kind, cols)
        out[key + "_dot"] = np.array([ob.dot(ob.AVX2_F16C, kind, w[r * rb:(r + 1) * rb].copy(), xq, cols) for r in range(rows)], dtype=np.float32)
        out[key + "_deq"] = np.stack([ob.dequant_row(kind, w[r * rb:(r + 1) * rb].copy(), cols) for r in range(rows)])
        if kind >= 3:
            s = [ob.block_sums(kind, w[r * rb:(r + 1) * rb].copy(), xq, cols) for r in range(rows)]
            out[key + "_sumi"] = np.stack([a for a, _ in s])
            out[key + "_summ"] = np.stack([b for _, b in s])
np.savez_compressed(Path(__file__).parent / "dots.npz", **out)
print("wrote", len(out), "arrays")
