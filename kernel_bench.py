"""Per-kernel microbenchmarks through the session's C ABI (a measurement harness beside
bench.py, not part of the package).

    python kernel_bench.py gemm 6304 768 2304 [--mode 0|1|2] [--iters 10] [--bias] [--gelu] [--residual]
    python kernel_bench.py micrograph [--batch 64] [--no-fuse]
    python kernel_bench.py attention 32 197 12     # batch, tokens, heads (head dim 64): the core alone, fp32 operands
    python kernel_bench.py layers 32 2             # batch, depth: ViT-B/16 encoder layers as in the model (the
                                                   # CTA-pair GEMMs with their epilogues, the TMA-fed attention kernel,
                                                   # the LayerNorm chains writing fp16 halves)
    python kernel_bench.py conv 16 64 112 [--k 1] [--depthwise] [--batch 32]   # c_in, c_out, H = W

Builds a one-node (or micrograph) session with per-kernel CUDA-event profiling
and prints, per kernel kind, the mean device time and the achieved algorithmic
TFLOP/s or GB/s. Inputs live on the device; the weight of `gemm` is a constant
(the form the models have). The event times include the host's launch latency of each step
(the steps are launched one by one, not as a graph): compare variants, not absolutes.
"""
import argparse
import json
import sys

import numpy as np

import os

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from altius_b200 import configs, ir  # noqa: E402
from altius_b200.session import CudaSessionBuilder  # noqa: E402


def _run(model, feeds, mode, fuse, iters, cold=False, pairs=False):
    import torch
    sess = (CudaSessionBuilder(model).with_gemm_mode(mode).with_fusion(fuse).with_gemm_pairs(pairs)
            .with_profiling_enabled(True, cold_l2=cold).build())
    ins = [torch.from_numpy(np.ascontiguousarray(v)).cuda() for v in feeds]
    outs = [torch.empty(tuple(shape), dtype=torch.float32, device="cuda") for shape, _ in sess.output_info]
    for it in range(iters + 2):
        if it == 2:
            sess.profile_reset()
        sess.run_device([t.data_ptr() for t in ins], [t.data_ptr() for t in outs])
    rows = {}
    steps = {}
    for e in sess.schedule():
        steps[e["kind"]] = steps.get(e["kind"], 0) + 1
    for kind, p in sess.profile().items():
        n = steps.get(kind, 1) * iters                 # executions of this kind of step
        us = 1e3 * p["total_ms"] / n
        rows[kind] = {"us": round(us, 2), "steps_per_run": steps.get(kind, 1),
                      "launches_per_run": p["launches"] // iters,
                      "GBps": round(p["bytes"] / n / us / 1e3, 1),
                      "TFLOPs": round(p["flops"] / n / us / 1e6, 2)}
    sess.close()
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "micrograph", "attention", "conv", "layers"])
    ap.add_argument("dims", nargs="*", type=int)
    ap.add_argument("--mode", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--no-fuse", action="store_true")
    ap.add_argument("--pairs", type=int, default=0, help="fp16-split GEMM on clusters of two CTAs: 1 A staged through registers, 2 A pre-split")
    ap.add_argument("--bias", action="store_true", help="gemm: + bias[n] in the epilogue")
    ap.add_argument("--gelu", action="store_true", help="gemm: Gelu after the bias")
    ap.add_argument("--residual", action="store_true", help="gemm: + residual[m, n] in the epilogue")
    ap.add_argument("--k", type=int, default=1, help="conv: square filter size (stride 1, same padding)")
    ap.add_argument("--depthwise", action="store_true", help="conv: one filter per channel (c_out is ignored)")
    ap.add_argument("--cold-l2", action="store_true", help="sweep L2 before every kernel (micrograph)")
    a = ap.parse_args(argv)
    rng = np.random.default_rng(0)
    if a.what == "gemm":
        m, k, n = a.dims
        x = rng.standard_normal((m, k)).astype(np.float32)
        w = (0.02 * rng.standard_normal((k, n))).astype(np.float32)
        g = ir.Graph()
        xi = g.add_input("x", x.shape)
        out = g.op("MatMul", xi, g.new_init(w))
        feeds = [x]
        if a.bias or a.gelu:
            out = g.op("Add", out, g.new_init((0.1 * rng.standard_normal(n)).astype(np.float32)))
        if a.gelu:
            out = g.op("Gelu", out)
        if a.residual:
            r = rng.standard_normal((m, n)).astype(np.float32)
            out = g.op("Add", g.add_input("r", r.shape), out)
            feeds.append(r)
        g.outputs.append(out)
        rows = _run(ir.Model(g, 13), feeds, a.mode, True, a.iters, pairs=a.pairs)
    elif a.what == "conv":
        cin, cout, hw = a.dims
        batch = a.batch if a.batch != 64 else 32
        group = cin if a.depthwise else 1
        cout = cin if a.depthwise else cout
        x = rng.standard_normal((batch, cin, hw, hw)).astype(np.float32)
        w = (rng.standard_normal((cout, cin // group, a.k, a.k)) / np.sqrt(cin // group * a.k * a.k)).astype(np.float32)
        g = ir.Graph()
        pad = a.k // 2
        y = g.op("Conv2d", g.add_input("x", x.shape), g.new_init(w),
                 g.new_init(rng.standard_normal(cout).astype(np.float32)), kernel_shape=[a.k, a.k], strides=[1, 1],
                 padding=[pad, pad, pad, pad], dilations=[1, 1], group=group, auto_pad="")
        g.outputs.append(g.op("ReLU", y))
        rows = _run(ir.Model(g, 13), [x], a.mode, True, a.iters)
    elif a.what == "attention":
        B, T, H = a.dims
        hd, D = 64, 64 * H
        qkv = rng.standard_normal((B, T, 3 * D)).astype(np.float32)
        g = ir.Graph()
        x = g.add_input("qkv", qkv.shape)
        i64 = lambda v: g.new_init(np.asarray(v, np.int64))
        q, k, v = g.add_node("Split", [x, i64([D, D, D])], 3, axis=2)

        def heads(t):
            t = g.op("Reshape", t, i64([B, T, H, hd]))
            t = g.op("Transpose", t, perm=[0, 2, 1, 3])
            return g.op("Reshape", t, i64([B * H, T, hd]))
        q, k, v = heads(q), heads(k), heads(v)
        s_ = g.op("MatMul", q, g.op("Transpose", k, perm=[0, 2, 1]))
        s_ = g.op("Mul", s_, g.new_init(np.array([hd ** -0.5], np.float32)))
        o = g.op("MatMul", g.op("Softmax", s_, axis=-1), v)
        o = g.op("Reshape", o, i64([B, H, T, hd]))
        o = g.op("Transpose", o, perm=[0, 2, 1, 3])
        g.outputs.append(g.op("Reshape", o, i64([B, T, D])))
        rows = _run(ir.Model(g, 13), [qkv], a.mode, not a.no_fuse, a.iters)
    elif a.what == "layers":
        batch, depth = a.dims
        model, feeds = configs.vit_base_16(batch=batch, depth=depth)
        rows = _run(model, list(feeds.values()), a.mode, not a.no_fuse, a.iters, pairs=a.pairs)
    else:
        model, feeds = configs.micrograph(batch=a.batch)
        rows = _run(model, list(feeds.values()), a.mode, not a.no_fuse, a.iters, cold=a.cold_l2)
    for kind, row in rows.items():
        print(json.dumps({kind: row}))


if __name__ == "__main__":
    main()
