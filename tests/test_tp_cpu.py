"""Tensor-parallel sharding on the CPU: the shards are byte-exact slices, per-block integer
sums do not change, the ranks' partial products add up to the unsharded product, and two
`gloo` ranks reduce them with an all-reduce as the GPU path does with NCCL."""
import json
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


Q4_K, Q5_K, Q6_K = 6, 7, 8  # kind ids of include/aot_cuda.h


def _kinds(layer, tensor):
    return {"wv": Q6_K, "down": Q6_K if layer % 2 == 0 else Q4_K, "output": Q6_K, "wo": Q5_K}.get(tensor, Q4_K)


def _model(pkg, arch, n_layer, world_max=4):
    """8 query / 4 KV heads of 128 (q width 1024), FFN 2048: splits 2 and 4 ways on block boundaries."""
    kw = dict(dim=512, hidden=2048, n_layer=n_layer, n_head=8, n_kv_head=4, head_dim=128, vocab=300, seed=5,
              kinds=_kinds, n_ctx_train=256)
    if arch == "qwen3":
        kw.update(qk_norm=True, rope_neox=True, rope_base=1e6, eps=1e-6)
    return pkg.model.build(f"tp-{arch}", **kw)


def test_shards_are_exact_slices(pkg):
    spec = _model(pkg, "qwen3", 2)
    d = spec.head.dims
    world = 2
    shards = [pkg.tp.shard_spec(spec, r, world) for r in range(world)]
    for r, sh in enumerate(shards):
        sd = sh.head.dims
        assert (sd.n_head, sd.n_kv_head, sd.hidden) == (d.n_head // world, d.n_kv_head // world, d.hidden // world)
        assert sd.dim == d.dim and sd.vocab == d.vocab and sd.head_dim == d.head_dim
    for i, l in enumerate(spec.layers):
        full = spec.weights
        rb = pkg.lib.row_bytes(l.wq.kind, l.wq.cols)
        got = np.concatenate([sh.weights[sh.layers[i].wq.off:sh.layers[i].wq.off + sh.layers[i].wq.len] for sh in shards])
        assert np.array_equal(got, full[l.wq.off:l.wq.off + l.wq.len])          # row slices, back to back
        # column slices: row by row, the shards' bytes side by side give the full row
        rbf = pkg.lib.row_bytes(l.down.kind, l.down.cols)
        rows_full = full[l.down.off:l.down.off + l.down.len].reshape(l.down.rows, rbf)
        parts = [sh.weights[sh.layers[i].down.off:sh.layers[i].down.off + sh.layers[i].down.len].reshape(l.down.rows, rbf // world)
                 for sh in shards]
        assert np.array_equal(np.concatenate(parts, axis=1), rows_full)
    # the output head: vocabulary rows dealt out in rank order; the greedy choice over the
    # shards' best (logit, id) pairs, lowest id on ties, is the first maximum of the whole
    out = spec.head.output
    got = np.concatenate([sh.weights[sh.head.output.off:sh.head.output.off + sh.head.output.len] for sh in shards])
    assert np.array_equal(got, spec.weights[out.off:out.off + out.len])
    assert all(sh.head.output.rows * world == d.vocab for sh in shards)
    logits = np.random.default_rng(1).integers(-3, 4, d.vocab).astype(np.float32)   # many ties
    per = d.vocab // world
    best = [(float(logits[r * per:(r + 1) * per].max()), r * per + int(np.argmax(logits[r * per:(r + 1) * per]))) for r in range(world)]
    pick = min(best, key=lambda b: (-b[0], b[1]))[1]
    assert pick == int(np.argmax(logits))
    whole = pkg.tp.shard_spec(spec, 1, world, shard_head=False)
    assert whole.head.output.rows == d.vocab
    with pytest.raises(ValueError):
        pkg.tp.shard_spec(spec, 0, 3)                      # heads do not split three ways
    assert pkg.tp.shard_spec(spec, 0, 1) is spec


def test_partial_products_add_up(pkg, ob):
    """attn_output and ffn_down of every layer: sum over ranks of (shard x its slice of the
    activations) equals the full product to f32 rounding, and the integer block sums of a
    shard are the matching columns of the full matrix's block sums."""
    spec = _model(pkg, "llama", 2)
    world = 4
    shards = [pkg.tp.shard_spec(spec, r, world) for r in range(world)]
    pool, tab = ob.Pool(2), ob.detect_table()
    rng = np.random.default_rng(3)
    for i, l in enumerate(spec.layers):
        for name in ("wo", "down"):
            t = getattr(l, name)
            x = rng.standard_normal(t.cols).astype(np.float32)
            w = spec.weights[t.off:t.off + t.len].copy()
            want = ob.matvec(pool, tab, t.kind, w, ob.quantize_act(t.kind, x), t.rows, t.cols)
            rbf = pkg.lib.row_bytes(t.kind, t.cols)
            si_full = ob.block_sums(t.kind, w[:rbf].copy(), ob.quantize_act(t.kind, x), t.cols)[0]  # row 0
            total = np.zeros(t.rows, dtype=np.float64)
            cw = t.cols // world
            for r, sh in enumerate(shards):
                ts = getattr(sh.layers[i], name)
                ws = sh.weights[ts.off:ts.off + ts.len].copy()
                xq = ob.quantize_act(ts.kind, x[r * cw:(r + 1) * cw])
                total += ob.matvec(pool, tab, ts.kind, ws, xq, ts.rows, ts.cols)
                rbs = pkg.lib.row_bytes(ts.kind, ts.cols)
                si = ob.block_sums(ts.kind, ws[:rbs].copy(), xq, ts.cols)[0]
                nbs = ts.cols // 256
                assert np.array_equal(si, si_full[r * nbs:(r + 1) * nbs])
            assert np.allclose(total, want, rtol=2e-5, atol=1e-5)


WORKER = textwrap.dedent("""
    import json, os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    sys.path.insert(0, {root!r} + "/tests")
    import __graft_entry__ as graft
    import torch, torch.distributed as dist
    pkg = graft.import_package()
    from oracle import binding as ob
    info = pkg.ranks.RankInfo.from_env()
    ranks = pkg.ranks.Ranks(info, backend="gloo")
    Q4_K, Q6_K = pkg.lib.Q4_K, pkg.lib.Q6_K
    spec = pkg.model.build("tp", dim=512, hidden=2048, n_layer=1, n_head=8, n_kv_head=4, head_dim=128, vocab=300, seed=5,
                           kinds=lambda l, t: Q6_K if t in ("down", "output") else Q4_K, n_ctx_train=256)
    sh = pkg.tp.shard_spec(spec, info.rank, info.world)
    pool, tab = ob.Pool(2), ob.detect_table()
    x = np.random.default_rng(9).standard_normal(spec.head.dims.hidden).astype(np.float32)
    t, ts = spec.layers[0].down, sh.layers[0].down
    cw = t.cols // info.world
    part = ob.matvec(pool, tab, ts.kind, sh.weights[ts.off:ts.off + ts.len].copy(),
                     ob.quantize_act(ts.kind, x[info.rank * cw:(info.rank + 1) * cw]), ts.rows, ts.cols)
    buf = torch.from_numpy(part.copy())
    dist.all_reduce(buf)                      # what aotcu_tp_attach arranges on the GPU with NCCL
    # the vocabulary-sharded head: every rank's slice of the logits, gathered in rank order, is
    # the whole vector bit for bit (rows are independent), and the best {{logit, id}} over the
    # ranks' slices (highest logit, lowest id on ties) is the first maximum of the whole
    xh = np.random.default_rng(10).standard_normal(spec.head.dims.dim).astype(np.float32)
    oh, os_ = spec.head.output, sh.head.output
    mine = ob.matvec(pool, tab, os_.kind, sh.weights[os_.off:os_.off + os_.len].copy(), ob.quantize_act(os_.kind, xh), os_.rows, os_.cols)
    mine[::7] = np.float32(3.0)               # ties across the ranks
    parts = [torch.zeros(os_.rows) for _ in range(info.world)]
    dist.all_gather(parts, torch.from_numpy(mine.copy()))
    gathered = torch.cat(parts).numpy()
    best = torch.tensor([float(mine.max()), float(info.rank * os_.rows + int(np.argmax(mine)))], dtype=torch.float64)
    bests = [torch.zeros(2, dtype=torch.float64) for _ in range(info.world)]
    dist.all_gather(bests, best)
    pick = min(((float(b[0]), int(b[1])) for b in bests), key=lambda b: (-b[0], b[1]))[1]
    if ranks.is_root:
        want = ob.matvec(pool, tab, t.kind, spec.weights[t.off:t.off + t.len].copy(), ob.quantize_act(t.kind, x), t.rows, t.cols)
        err = float(np.max(np.abs(buf.numpy() - want) / (np.abs(want) + 1e-3)))
        full = ob.matvec(pool, tab, oh.kind, spec.weights[oh.off:oh.off + oh.len].copy(), ob.quantize_act(oh.kind, xh), oh.rows, oh.cols)
        for r in range(info.world):
            full[r * os_.rows:(r + 1) * os_.rows:7] = np.float32(3.0)
        print(json.dumps({{"world": info.world, "max_rel_err": err, "head_rows": int(os_.rows),
                          "gathered_equal": bool(np.array_equal(gathered.view(np.uint32), full.view(np.uint32))),
                          "pick": pick, "argmax": int(np.argmax(full))}}))
    ranks.close()
""")


@pytest.mark.timeout(240)
def test_two_gloo_ranks_reduce_partial_ffn_down(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
         "--master-port", "29741", str(script)],
        capture_output=True, text=True, env=env, timeout=230)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout
    out = json.loads(lines[0])
    assert out["world"] == 2 and out["max_rel_err"] < 1e-4
    assert out["head_rows"] == 150 and out["gathered_equal"] and out["pick"] == out["argmax"]
