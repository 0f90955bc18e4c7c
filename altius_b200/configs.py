"""Synthetic graphs for the benchmark configurations.

No model files or datasets are available offline, so each configuration is
built programmatically in the form the graphs have after altius's fusion
passes (`LayerNormalization`, `Gelu` already fused; BatchNorm folded into the
preceding Conv2d) with seeded random weights and inputs of the shapes and value
distributions the configurations name. The same bytes feed the CPU oracle and
the CUDA session.

Shapes stay inside what the reference interpreter accepts where it can
(3-D batched MatMul rather than 4-D, last-axis Split, last-axis Softmax and
LayerNormalization); the class-token select uses Gather on axis 1 with a
batch larger than one, which the reference asserts against and is noted as an
extension.
"""
from __future__ import annotations

from typing import Dict, Tuple

import numpy as np

from .ir import Graph, Model, I64


def _i64(g: Graph, vals) -> int:
    return g.new_init(np.asarray(vals, dtype=np.int64))


class _W:
    """Seeded weight source: ~N(mean, std) float32."""

    def __init__(self, seed: int, std: float):
        self.rng = np.random.default_rng(seed)
        self.std = std

    def __call__(self, *shape, mean: float = 0.0, std: float = None) -> np.ndarray:
        std = self.std if std is None else std
        return (mean + std * self.rng.standard_normal(shape)).astype(np.float32)


# ---------------------------------------------------------------------------
def mnist_cnn(seed: int = 0) -> Tuple[Model, Dict[str, np.ndarray]]:
    """mnist-8 shaped CNN, batch 1. Structure as pinned by the reference's
    `mnist_model` test (crates/core/src/model.rs:187-350): Conv 5x5 SAME_UPPER
    -> Add bias [8,1,1] -> ReLU -> MaxPool 2x2/2 -> Conv 5x5 -> Add [16,1,1] ->
    ReLU -> MaxPool 3x3/3 -> Reshape [1,256]; Reshape of the [16,4,4,10] weight
    to [256,10] -> MatMul -> Add [1,10]. Weights ~N(0, 0.1)."""
    w = _W(seed, 0.1)
    g = Graph()
    x = g.add_input("Input3", (1, 1, 28, 28))
    c0 = g.op("Conv2d", x, g.new_init(w(8, 1, 5, 5)), auto_pad="SAME_UPPER", kernel_shape=[5, 5],
              strides=[1, 1], dilations=[1, 1], group=1, padding=[])
    a0 = g.op("Add", c0, g.new_init(w(8, 1, 1)))
    r0 = g.op("ReLU", a0)
    p0 = g.op("MaxPool", r0, auto_pad="NOTSET", padding=[0, 0, 0, 0], kernel_shape=[2, 2],
              strides=[2, 2])
    c1 = g.op("Conv2d", p0, g.new_init(w(16, 8, 5, 5)), auto_pad="SAME_UPPER", kernel_shape=[5, 5],
              strides=[1, 1], dilations=[1, 1], group=1, padding=[])
    a1 = g.op("Add", c1, g.new_init(w(16, 1, 1)))
    r1 = g.op("ReLU", a1)
    p1 = g.op("MaxPool", r1, auto_pad="NOTSET", padding=[0, 0, 0, 0], kernel_shape=[3, 3],
              strides=[3, 3])
    f0 = g.op("Reshape", p1, _i64(g, [1, 256]))
    wr = g.op("Reshape", g.new_init(w(16, 4, 4, 10)), _i64(g, [256, 10]))
    mm = g.op("MatMul", f0, wr)
    out = g.op("Add", mm, g.new_init(w(1, 10)))
    g.values[out].name = "Plus214_Output_0"
    g.outputs.append(out)
    rng = np.random.default_rng(seed + 1)
    return Model(g, 13), {"Input3": rng.random((1, 1, 28, 28), dtype=np.float32)}


# ---------------------------------------------------------------------------
def micrograph(batch: int = 64, tokens: int = 197, dim: int = 768, heads: int = 12,
               seed: int = 0) -> Tuple[Model, Dict[str, np.ndarray]]:
    """Tensor-op micrograph: X + bias -> Gelu -> + X -> LayerNormalization
    (eps 1e-6); S * 0.125 -> Softmax; ReduceMean and ReduceMax over the last
    axis of X. Four outputs in that order."""
    rng = np.random.default_rng(seed)
    g = Graph()
    x = g.add_input("X", (batch, tokens, dim))
    s = g.add_input("S", (batch, heads, tokens, tokens))
    bias = g.new_init(rng.standard_normal(dim).astype(np.float32))
    gamma = g.new_init((1 + 0.02 * rng.standard_normal(dim)).astype(np.float32))
    beta = g.new_init((0.02 * rng.standard_normal(dim)).astype(np.float32))
    a = g.op("Add", x, bias)
    ge = g.op("Gelu", a)
    r = g.op("Add", ge, x)
    ln = g.op("LayerNormalization", r, gamma, beta, axis=-1, epsilon=1e-6, stash_type=1)
    sc = g.op("Mul", s, g.new_init(np.array([0.125], np.float32)))
    sm = g.op("Softmax", sc, axis=-1)
    mean = g.op("ReduceMean", x, axes=[-1], keep_dims=True)
    mx = g.op("ReduceMax", x, axes=[-1], keep_dims=True)
    for name, v in (("ln", ln), ("softmax", sm), ("mean", mean), ("max", mx)):
        g.values[v].name = name
        g.outputs.append(v)
    X = rng.standard_normal((batch, tokens, dim)).astype(np.float32)
    S = rng.standard_normal((batch, heads, tokens, tokens)).astype(np.float32)
    return Model(g, 13), {"X": X, "S": S}


# ---------------------------------------------------------------------------
def _linear(g: Graph, w: _W, x: int, din: int, dout: int) -> int:
    y = g.op("MatMul", x, g.new_init(w(din, dout)))
    return g.op("Add", y, g.new_init(w(dout)))


def _f32(g: Graph, v: float) -> int:
    return g.new_init(np.array(v, dtype=np.float32))


def _ln(g: Graph, w: _W, x: int, dim: int, eps: float, fused: bool = True) -> int:
    gamma, beta = g.new_init(w(dim, mean=1.0)), g.new_init(w(dim))
    if fused:
        return g.op("LayerNormalization", x, gamma, beta, axis=-1, epsilon=eps, stash_type=1)
    # The nine nodes an opset < 17 export spells LayerNorm with, the pattern `fuse_layer_norm`
    # recognises (crates/core/src/optimize/layer_norm_fusion.rs:9-15).
    mean = g.op("ReduceMean", x, axes=[-1], keep_dims=True)
    d = g.op("Sub", x, mean)
    var = g.op("ReduceMean", g.op("Pow", d, _f32(g, 2.0)), axes=[-1], keep_dims=True)
    n = g.op("Div", d, g.op("Sqrt", g.op("Add", var, _f32(g, eps))))
    return g.op("Add", g.op("Mul", n, gamma), beta)


def _gelu(g: Graph, x: int, fused: bool = True, form: str = "erf") -> int:
    if fused:
        return g.op("Gelu", x)
    if form == "erf":
        # x * 0.5 * (1 + erf(x / sqrt(2))) as exporters write it: the pattern of `fuse_gelu`
        # (crates/core/src/optimize/gelu_fusion.rs:12-82).
        e = g.op("Erf", g.op("Div", x, _f32(g, np.sqrt(2.0))))
        return g.op("Mul", g.op("Mul", x, g.op("Add", e, _f32(g, 1.0))), _f32(g, 0.5))
    # The tanh form: the pattern of `fuse_fast_gelu` (fast_gelu_fusion.rs:5-167).
    c = g.op("Mul", g.op("Pow", x, _f32(g, 3.0)), _f32(g, 0.044715))
    t = g.op("Tanh", g.op("Mul", g.op("Add", x, c), _f32(g, np.sqrt(2.0 / np.pi))))
    return g.op("Mul", g.op("Mul", x, _f32(g, 0.5)), g.op("Add", t, _f32(g, 1.0)))


def _encoder_layer(g: Graph, w: _W, x: int, B: int, T: int, D: int, H: int, mlp: int,
                   eps: float, fused: bool = True, gelu_form: str = "erf") -> int:
    hd = D // H
    h = _ln(g, w, x, D, eps, fused)
    qkv = _linear(g, w, h, D, 3 * D)                                   # [B,T,3D]
    q, k, v = g.add_node("Split", [qkv, _i64(g, [D, D, D])], 3, axis=2)

    def heads(t: int) -> int:
        t = g.op("Reshape", t, _i64(g, [B, T, H, hd]))
        t = g.op("Transpose", t, perm=[0, 2, 1, 3])                    # [B,H,T,hd]
        return g.op("Reshape", t, _i64(g, [B * H, T, hd]))

    q, k, v = heads(q), heads(k), heads(v)
    kt = g.op("Transpose", k, perm=[0, 2, 1])                          # [BH,hd,T]
    s = g.op("MatMul", q, kt)                                          # [BH,T,T]
    s = g.op("Mul", s, g.new_init(np.array([hd ** -0.5], np.float32)))
    p = g.op("Softmax", s, axis=-1)
    o = g.op("MatMul", p, v)                                           # [BH,T,hd]
    o = g.op("Reshape", o, _i64(g, [B, H, T, hd]))
    o = g.op("Transpose", o, perm=[0, 2, 1, 3])
    o = g.op("Reshape", o, _i64(g, [B, T, D]))
    o = _linear(g, w, o, D, D)
    x = g.op("Add", x, o)
    h = _ln(g, w, x, D, eps, fused)
    h = _linear(g, w, h, D, mlp)
    h = _gelu(g, h, fused, gelu_form)
    h = _linear(g, w, h, mlp, D)
    return g.op("Add", x, h)


def vision_transformer(batch: int, dim: int, depth: int, heads: int, mlp: int, n_prefix: int,
                       eps: float = 1e-6, n_classes: int = 1000, img: int = 224, patch: int = 16,
                       seed: int = 0, fused: bool = True, gelu_form: str = "erf"
                       ) -> Tuple[Model, Dict[str, np.ndarray]]:
    """ViT / DeiT encoder: patch-embed Conv 16x16/16 -> tokens (+cls[, dist]) +
    pos-embed -> `depth` pre-LN layers -> LN -> class-token select -> Gemm.
    With two prefix tokens (DeiT distilled) the two heads' logits are averaged
    (Add, Mul 0.5). Weights ~N(0, 0.02), LN gamma ~N(1, 0.02). `fused=False` spells every
    LayerNormalization and Gelu as the node chains a raw export has (the same weights: the
    graph passes turn it back into the fused form)."""
    w = _W(seed, 0.02)
    B, D = batch, dim
    n_patch = (img // patch) ** 2
    T = n_patch + n_prefix
    g = Graph()
    x = g.add_input("input", (B, 3, img, img))
    pe = g.op("Conv2d", x, g.new_init(w(D, 3, patch, patch)), g.new_init(w(D)), auto_pad="",
              kernel_shape=[patch, patch], strides=[patch, patch], dilations=[1, 1], group=1,
              padding=[0, 0, 0, 0])                                    # [B,D,14,14]
    t = g.op("Reshape", pe, _i64(g, [B, D, n_patch]))
    t = g.op("Transpose", t, perm=[0, 2, 1])                           # [B,196,D]
    # The prefix tokens arrive expanded over the batch, as constant folding of
    # the exporter's `cls_token.expand(B, -1, -1)` leaves them.
    prefix = g.new_init(np.broadcast_to(w(1, n_prefix, D), (B, n_prefix, D)).copy())
    t = g.op("Concat", prefix, t, axis=1)                              # [B,T,D]
    t = g.op("Add", t, g.new_init(w(1, T, D)))
    for _ in range(depth):
        t = _encoder_layer(g, w, t, B, T, D, heads, mlp, eps, fused, gelu_form)
    t = _ln(g, w, t, D, eps, fused)
    logits = None
    for i in range(n_prefix):
        tok = g.op("Gather", t, g.new_init(np.array(i, dtype=np.int64)), axis=1)     # [B,D]
        li = g.op("Gemm", tok, g.new_init(w(n_classes, D)), g.new_init(w(n_classes)), alpha=1.0,
                  beta=1.0, trans_a=False, trans_b=True)
        logits = li if logits is None else g.op("Add", logits, li)
    if n_prefix > 1:
        logits = g.op("Mul", logits, g.new_init(np.array([1.0 / n_prefix], np.float32)))
    g.values[logits].name = "output"
    g.outputs.append(logits)
    rng = np.random.default_rng(seed + 1)
    return Model(g, 13), {"input": rng.standard_normal((B, 3, img, img)).astype(np.float32)}


def vit_base_16(batch: int = 32, seed: int = 0, depth: int = 12, fused: bool = True, gelu_form: str = "erf"):
    """ViT-B/16: 197 tokens, dim 768, 12 heads, MLP 3072, LN eps 1e-6."""
    return vision_transformer(batch, 768, depth, 12, 3072, 1, 1e-6, seed=seed, fused=fused, gelu_form=gelu_form)


def deit_small_distilled_16(batch: int = 64, seed: int = 0, depth: int = 12, fused: bool = True):
    """DeiT-Small/16 distilled: 198 tokens, dim 384, 6 heads, MLP 1536."""
    return vision_transformer(batch, 384, depth, 6, 1536, 2, 1e-6, seed=seed, fused=fused)


# ---------------------------------------------------------------------------
def _make_divisible(v: float, divisor: int = 8) -> int:
    new_v = max(divisor, int(v + divisor / 2) // divisor * divisor)
    if new_v < 0.9 * v:
        new_v += divisor
    return new_v


# kernel, expanded channels, output channels, squeeze-excite, HardSwish?, stride
_MBV3_LARGE = (
    (3, 16, 16, False, False, 1), (3, 64, 24, False, False, 2), (3, 72, 24, False, False, 1),
    (5, 72, 40, True, False, 2), (5, 120, 40, True, False, 1), (5, 120, 40, True, False, 1),
    (3, 240, 80, False, True, 2), (3, 200, 80, False, True, 1), (3, 184, 80, False, True, 1),
    (3, 184, 80, False, True, 1), (3, 480, 112, True, True, 1), (3, 672, 112, True, True, 1),
    (5, 672, 160, True, True, 2), (5, 960, 160, True, True, 1), (5, 960, 160, True, True, 1),
)


def mobilenet_v3_large(batch: int = 32, seed: int = 0, img: int = 224, n_classes: int = 1000):
    """MobileNetV3-Large with BatchNorm folded into the convolutions (weight +
    bias only). HardSwish is HardSigmoid(alpha 1/6, beta 0.5) followed by Mul,
    the form an opset < 14 export has; squeeze-excite is GlobalAveragePool ->
    1x1 Conv -> ReLU -> 1x1 Conv -> HardSigmoid -> broadcast Mul."""
    w = _W(seed, 0.02)
    g = Graph()
    x = g.add_input("input", (batch, 3, img, img))

    def conv(t, cin, cout, k, s, group=1):
        p = (k - 1) // 2
        return g.op("Conv2d", t, g.new_init(w(cout, cin // group, k, k)), g.new_init(w(cout)),
                    auto_pad="", kernel_shape=[k, k], strides=[s, s], dilations=[1, 1], group=group,
                    padding=[p, p, p, p])

    def hsig(t):
        return g.op("HardSigmoid", t, alpha=1.0 / 6.0, beta=0.5)

    def act(t, hs):
        return g.op("Mul", t, hsig(t)) if hs else g.op("ReLU", t)

    t = act(conv(x, 3, 16, 3, 2), True)
    cin = 16
    for k, exp, cout, se, hs, s in _MBV3_LARGE:
        inp = t
        if exp != cin:
            t = act(conv(t, cin, exp, 1, 1), hs)
        t = act(conv(t, exp, exp, k, s, group=exp), hs)
        if se:
            sq = _make_divisible(exp // 4, 8)
            z = g.op("GlobalAveragePool", t)
            z = g.op("ReLU", conv(z, exp, sq, 1, 1))
            z = hsig(conv(z, sq, exp, 1, 1))
            t = g.op("Mul", t, z)
        t = conv(t, exp, cout, 1, 1)
        if s == 1 and cin == cout:
            t = g.op("Add", t, inp)
        cin = cout
    t = act(conv(t, cin, 960, 1, 1), True)
    t = g.op("GlobalAveragePool", t)
    t = g.op("Flatten", t, axis=1)
    t = g.op("Gemm", t, g.new_init(w(1280, 960)), g.new_init(w(1280)), alpha=1.0, beta=1.0,
             trans_a=False, trans_b=True)
    t = g.op("Mul", t, hsig(t))
    t = g.op("Gemm", t, g.new_init(w(n_classes, 1280)), g.new_init(w(n_classes)), alpha=1.0,
             beta=1.0, trans_a=False, trans_b=True)
    g.values[t].name = "output"
    g.outputs.append(t)
    rng = np.random.default_rng(seed + 1)
    return Model(g, 13), {"input": rng.standard_normal((batch, 3, img, img)).astype(np.float32)}
