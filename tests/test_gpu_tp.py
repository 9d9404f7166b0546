"""Tensor-parallel decode on two GPUs: each rank holds a shard, the partial attn_output /
ffn_down rows are summed over NCCL inside the forward pass, and the logits match the
single-device path to f32 rounding (the order of additions over blocks differs)."""
import json
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu

WORKER = textwrap.dedent("""
    import json, os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    import __graft_entry__ as graft
    pkg = graft.import_package()
    info = pkg.ranks.RankInfo.from_env()
    ranks = pkg.ranks.Ranks(info, backend="nccl")
    Q4_K, Q5_K, Q6_K = pkg.lib.Q4_K, pkg.lib.Q5_K, pkg.lib.Q6_K
    kinds = lambda l, t: {{"wv": Q6_K, "down": Q6_K if l % 2 == 0 else Q4_K, "output": Q6_K, "wo": Q5_K}}.get(t, Q4_K)
    out = {{}}
    for arch, fused in (("llama", True), ("qwen3", True), ("llama", False)):
        kw = dict(dim=512, hidden=2048, n_layer=3, n_head=8, n_kv_head=4, head_dim=128, vocab=600, seed=5, kinds=kinds, n_ctx_train=256)
        if arch == "qwen3":
            kw.update(qk_norm=True, rope_neox=True, rope_base=1e6, eps=1e-6)
        spec = pkg.model.build("tp-" + arch, **kw)
        ctx = pkg.Context(info.local_rank)
        sh = pkg.tp.shard_spec(spec, info.rank, info.world)
        g = pkg.Gpu(ctx, sh.head, sh.layers, sh.weights, 128, 16)
        # fused: partial rows cross NVLink inside the one-kernel step; else NCCL all-reduces
        pkg.tp.join(g, ranks, fused=fused)
        one_kernel = bool(g.set_option("mega_available", 0))
        full = pkg.Gpu(ctx, spec.head, spec.layers, spec.weights, 128, 16) if ranks.is_root else None
        prompt = [5, 17, 300, 42, 7, 7, 1, 599, 0, 12, 13]
        worst, agree, total = 0.0, 0, 0
        g.forward_batch(prompt, 0, True)
        lg = g.logits()
        if full:
            full.forward_batch(prompt, 0, True)
            lf = full.logits()
            worst = max(worst, float(np.max(np.abs(lg - lf)) / np.max(np.abs(lf))))
        tok, pos = int(np.argmax(lg)), len(prompt)
        for step in range(24):
            g.forward(tok, pos, True)              # every rank feeds the same token
            lg = g.logits()
            if full:
                full.forward(tok, pos, True)
                lf = full.logits()
                worst = max(worst, float(np.max(np.abs(lg - lf)) / np.max(np.abs(lf))))
                agree += int(np.argmax(lg) == np.argmax(lf))
                total += 1
            tok, pos = int(np.argmax(lg)), pos + 1
        ids, ms = g.generate(tok, pos, 16)         # the device-side greedy loop, all ranks in step
        ctx.device_status()
        out[arch + ("-fused" if fused else "-nccl")] = {{"worst_rel": worst, "agree": agree, "total": total,
                                                         "ids": [int(i) for i in ids], "one_kernel": one_kernel, "fused": fused}}
        ranks.barrier()
    if ranks.is_root:
        print(json.dumps(out))
    ranks.close()
""")


@pytest.mark.timeout(600)
def test_two_ranks_match_single_device(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
         "--master-port", "29751", str(script)],
        capture_output=True, text=True, env=env, timeout=580)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-3000:])
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout
    out = json.loads(lines[0])
    for arch, res in out.items():
        assert res["worst_rel"] < 1e-3, (arch, res)      # north-star tolerance for f32 outputs
        assert res["agree"] == res["total"], (arch, res)  # same greedy choice at every compared step
        assert len(res["ids"]) == 16
        assert res["one_kernel"] == res["fused"], (arch, res)  # the fused exchange keeps the one-kernel step
