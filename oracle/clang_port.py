"""CPU restatement of the reference's generated-C backend (test infrastructure and a timed
baseline, never shipped code).

The reference's second CPU backend translates a graph into one C function per node, compiles
the file with `clang -O3 -march=native -fopenmp`, and calls `model_entry` through a trampoline
(crates/session_clang/src/translator.rs:288-531). Dense contractions call `cblas_sgemm` (BLIS
there); everything else is a loop nest written into the C text with OpenMP pragmas. This module
restates that translator for the operators of the benchmark graphs (the vision transformer and
the tensor-op micrograph): same loop nests, same constants, same threading pragmas, same
region-reusing arena. What differs, because the toolchain here differs:

  * the compiler is gcc; `#pragma clang loop vectorize(enable)` becomes `#pragma omp simd`
    (with a reduction clause where the loop reduces), the same permission to vectorise;
  * `cblas_sgemm` is the OpenBLAS bundled with scipy / numpy, bound through a function pointer
    (no BLIS in this image);
  * ReduceMax over the last axis is added (the reference's template only reduces over all
    axes, crates/session_clang/src/translator.rs:2792-2819) in the style of its ReduceMean.

Parity of this restatement is checked against the interpreter oracle in the tests.
"""
import ctypes
import glob
import hashlib
import os
import subprocess
import time
from typing import Dict, List, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_CACHE = os.path.join(_HERE, "_clang")
CFLAGS = ["-O3", "-march=native", "-fno-math-errno", "-fopenmp", "-ftree-vectorize", "-shared", "-fPIC",
          "-w"]


# ---- cblas_sgemm from the OpenBLAS that ships with scipy / numpy ---------------------------------
def _find_sgemm():
    import numpy
    site = os.path.dirname(os.path.dirname(numpy.__file__))
    for pattern, sym, setter, blasint in (
            ("scipy.libs/libscipy_openblas-*.so", "scipy_cblas_sgemm", "scipy_openblas_set_num_threads", "int"),
            ("numpy.libs/libscipy_openblas64_-*.so", "scipy_cblas_sgemm64_",
             "scipy_openblas_set_num_threads64_", "long")):
        for path in sorted(glob.glob(os.path.join(site, pattern))):
            lib = ctypes.CDLL(path)
            if hasattr(lib, sym):
                return lib, ctypes.cast(getattr(lib, sym), ctypes.c_void_p).value, getattr(lib, setter), blasint
    raise RuntimeError("no OpenBLAS with a cblas_sgemm entry point was found beside numpy / scipy")


# ---- shapes (crates/core/src/analysis/shape.rs, the operators translated below) ------------------
def _strides(dims):
    out, s = [], 1
    for d in reversed(dims):
        out.append(s)
        s *= d
    return list(reversed(out))


def _broadcast(a, b):
    n = max(len(a), len(b))
    a = [1] * (n - len(a)) + list(a)
    b = [1] * (n - len(b)) + list(b)
    return [max(x, y) for x, y in zip(a, b)]


def _bcast_strides(dims, out):
    """Strides of `dims` viewed as `out` with 0 on broadcast axes (crates/core/src/dim.rs
    strides_for_broadcasting_to)."""
    pad = [1] * (len(out) - len(dims)) + list(dims)
    st = _strides(pad)
    return [0 if d == 1 and o != 1 else s for d, o, s in zip(pad, out, st)]


def _infer(node, ins, inits):
    op, a = node.op, node.attrs
    if op in ("Add", "Sub", "Mul", "Div"):
        return [_broadcast(ins[0], ins[1])]
    if op in ("Gelu", "Softmax", "LayerNormalization"):
        return [list(ins[0])]
    if op == "MatMul":
        return [list(ins[0][:-1]) + [ins[1][-1]]]
    if op == "Gemm":
        m = ins[0][1] if a.get("trans_a") else ins[0][0]
        n = ins[1][0] if a.get("trans_b") else ins[1][1]
        return [[m, n]]
    if op == "Conv2d":
        kh, kw = a["kernel_shape"]
        sh, sw = a.get("strides", [1, 1])
        pad = list(a.get("padding", [0, 0, 0, 0]))
        assert not a.get("auto_pad"), "auto_pad is not translated"
        assert list(a.get("dilations", [1, 1])) == [1, 1]
        oh = (ins[0][2] + pad[0] + pad[2] - kh) // sh + 1
        ow = (ins[0][3] + pad[1] + pad[3] - kw) // sw + 1
        return [[ins[0][0], ins[1][0], oh, ow]]
    if op == "Reshape":
        want = [int(v) for v in inits[node.inputs[1]].reshape(-1)]
        total = int(np.prod(ins[0]))
        want = [ins[0][i] if d == 0 else d for i, d in enumerate(want)]
        if -1 in want:
            known = int(np.prod([d for d in want if d != -1]))
            want[want.index(-1)] = total // known
        return [want]
    if op == "Transpose":
        return [[ins[0][p] for p in a["perm"]]]
    if op == "Concat":
        ax = a["axis"] % len(ins[0])
        out = list(ins[0])
        out[ax] = sum(s[ax] for s in ins)
        return [out]
    if op == "Split":
        ax = a["axis"] % len(ins[0])
        parts = [int(v) for v in inits[node.inputs[1]].reshape(-1)]
        return [[*ins[0][:ax], p, *ins[0][ax + 1:]] for p in parts]
    if op == "Gather":
        ax = a.get("axis", 0)
        # a shape of [] or [1] is a scalar to the reference (crates/core/src/dim.rs is_scalar)
        idx = [] if list(ins[1]) in ([], [1]) else list(ins[1])
        return [list(ins[0][:ax]) + idx + list(ins[0][ax + 1:])]
    if op in ("ReduceMean", "ReduceMax"):
        axes = [x % len(ins[0]) for x in a["axes"]]
        assert a.get("keep_dims", True)
        return [[1 if i in axes else d for i, d in enumerate(ins[0])]]
    raise NotImplementedError(f"the generated-C restatement does not translate {op}")


# ---- one C body per node ------------------------------------------------------------------------
_SOFTMAX_CONSTS = """
const float LOWER_RANGE = -88.37626f, ROUNDING_BIAS = 12582912.0f, LOG2RECIPROCAL = 1.44269504088896341f;
const float LOG2HIGH = -6.93145752e-1f, LOG2LOW = -1.42860677e-6f;
const float POLY_0 = 0.0013780593872f, POLY_1 = 0.0083731245250f, POLY_2 = 0.0416695363820f;
const float POLY_3 = 0.1666647195816f, POLY_4 = 0.4999998509884f, POLY_56 = 1.0f;
const int32_t MAXIMUM_EXPONENT = 0x3F800000;
"""

_GELU_CONSTS = """
const float B = 0.7978845608028654f, C = 0.035677408136300125f, LOWER_RANGE = -9.f, UPPER_RANGE = 9.f;
const float ALPHA_13 = -2.76076847742355e-16f, ALPHA_11 = 2.00018790482477e-13f, ALPHA_9 = -8.60467152213735e-11f;
const float ALPHA_7 = 5.12229709037114e-08f, ALPHA_5 = 1.48572235717979e-05f, ALPHA_3 = 6.37261928875436e-04f;
const float ALPHA_1 = 4.89352455891786e-03f, BETA_6 = 1.19825839466702e-06f, BETA_4 = 1.18534705686654e-04f;
const float BETA_2 = 2.26843463243900e-03f, BETA_0 = 4.89352518554385e-03f;
"""


class _Translator:
    def __init__(self, model, threads):
        self.m, self.g, self.th = model, model.graph, threads
        self.shapes: Dict[int, List[int]] = {}

    def name(self, v):
        return f"v{v}"

    def body(self, node):
        fn = getattr(self, "t_" + node.op.lower(), None)
        if fn is None:
            raise NotImplementedError(node.op)
        ins = [self.shapes[i] for i in node.inputs]
        outs = [self.shapes[o] for o in node.outputs]
        names = [self.name(i) for i in node.inputs] + [self.name(o) for o in node.outputs]
        return fn(node, names, ins, outs)

    # crates/session_clang/src/translator.rs:1145-1240
    def _bin(self, sym, names, ins, outs):
        a, b, o = names
        total = int(np.prod(outs[0]))
        if list(ins[0]) == list(ins[1]):
            return (f"#pragma omp parallel for simd num_threads({self.th})\n"
                    f"for (int i = 0; i < {total}; i++) {o}[i] = {a}[i] {sym} {b}[i];")
        od = outs[0]
        rank = len(od)
        ost, s0, s1 = _strides(od), _bcast_strides(ins[0], od), _bcast_strides(ins[1], od)
        i = rank - 1
        text = (f"#pragma omp simd\nfor (int i{i} = 0; i{i} < {od[i]}; i{i}++)\n"
                f"    *(o{i} + {ost[i]} * i{i}) = *(a{i} + {s0[i]} * i{i}) {sym} *(b{i} + {s1[i]} * i{i});")
        # The outer loops of a broadcast operation run on one thread in the reference.
        for i in reversed(range(rank - 1)):
            inner = text.replace("\n", "\n    ")
            text = (f"for (int i{i} = 0; i{i} < {od[i]}; i{i}++) {{\n"
                    f"    const float *a{i + 1} = a{i} + {s0[i]} * i{i};\n"
                    f"    const float *b{i + 1} = b{i} + {s1[i]} * i{i};\n"
                    f"    float *o{i + 1} = o{i} + {ost[i]} * i{i};\n    {inner}\n}}")
        return f"const float *a0 = {a}; const float *b0 = {b}; float *o0 = {o};\n" + text

    def t_add(self, n, names, ins, outs): return self._bin("+", names, ins, outs)
    def t_sub(self, n, names, ins, outs): return self._bin("-", names, ins, outs)
    def t_mul(self, n, names, ins, outs): return self._bin("*", names, ins, outs)
    def t_div(self, n, names, ins, outs): return self._bin("/", names, ins, outs)

    # crates/session_clang/src/translator.rs:3020-3082
    def t_gelu(self, n, names, ins, outs):
        x, y = names
        return (f"{_GELU_CONSTS}\n#pragma omp parallel for simd num_threads({self.th})\n"
                f"for (int i = 0; i < {int(np.prod(outs[0]))}; i++) {{\n"
                f"    const float x = {x}[i];\n"
                "    const float y = fminf(fmaxf(x * fmaf(C * x, x, B), LOWER_RANGE), UPPER_RANGE);\n"
                "    const float y2 = y * y;\n"
                "    float p = fmaf(y2, ALPHA_13, ALPHA_11);\n"
                "    p = fmaf(p, y2, ALPHA_9); p = fmaf(p, y2, ALPHA_7); p = fmaf(p, y2, ALPHA_5);\n"
                "    p = fmaf(p, y2, ALPHA_3); p = fmaf(p, y2, ALPHA_1); p = p * y;\n"
                "    float q = fmaf(y2, BETA_6, BETA_4);\n"
                "    q = fmaf(q, y2, BETA_2); q = fmaf(q, y2, BETA_0);\n"
                f"    {y}[i] = (p / q + 1.f) * (x * 0.5f);\n}}")

    # crates/session_clang/src/translator.rs:2821-2895
    def t_softmax(self, n, names, ins, outs):
        x, y = names
        axis = n.attrs.get("axis", -1)
        assert axis in (-1, len(ins[0]) - 1)
        L = ins[0][-1]
        rows = int(np.prod(ins[0])) // L
        return (f"{_SOFTMAX_CONSTS}\n#pragma omp parallel for num_threads({self.th})\n"
                f"for (int i = 0; i < {rows}; i++) {{\n"
                f"    const float *in = {x} + (size_t)i * {L};\n    float *out = {y} + (size_t)i * {L};\n"
                f"    float max = -INFINITY;\n    for (int j = 0; j < {L}; j++) max = fmaxf(in[j], max);\n"
                f"    float sum = 0.0f;\n    #pragma omp simd reduction(+:sum)\n    for (int j = 0; j < {L}; j++) {{\n"
                "        const float val0 = fmaxf(in[j] - max, LOWER_RANGE);\n"
                "        const float biased = fmaf(val0, LOG2RECIPROCAL, ROUNDING_BIAS);\n"
                "        const float m = biased - ROUNDING_BIAS;\n"
                "        const float val2 = fmaf(m, LOG2LOW, fmaf(m, LOG2HIGH, val0));\n"
                "        union { float f; int32_t i; } bits, scale;\n        bits.f = biased;\n"
                "        scale.i = (int32_t)((uint32_t)bits.i << 23) + MAXIMUM_EXPONENT;\n"
                "        float p = fmaf(POLY_0, val2, POLY_1);\n"
                "        p = fmaf(p, val2, POLY_2); p = fmaf(p, val2, POLY_3); p = fmaf(p, val2, POLY_4);\n"
                "        p = fmaf(p, val2, POLY_56); p = fmaf(p, val2, POLY_56);\n"
                "        p = p * scale.f;\n        sum += p;\n        out[j] = p;\n    }\n"
                f"    const float recip = 1.0f / sum;\n    #pragma omp simd\n"
                f"    for (int j = 0; j < {L}; j++) out[j] = out[j] * recip;\n}}")

    # crates/session_clang/src/translator.rs:2961-3018
    def t_layernormalization(self, n, names, ins, outs):
        x, gamma, beta, y = names[0], names[1], names[2], names[3]
        L = ins[0][-1]
        rows = int(np.prod(ins[0])) // L
        inv = repr(float(np.float32(1.0) / np.float32(L)))
        eps = repr(float(np.float32(n.attrs.get("epsilon", 1e-5))))
        return (f"#pragma omp parallel for num_threads({self.th})\nfor (int i = 0; i < {rows}; i++) {{\n"
                f"    const float *data = {x} + (size_t)i * {L};\n    float *out = {y} + (size_t)i * {L};\n"
                f"    float sum = 0.0f;\n    #pragma omp simd reduction(+:sum)\n"
                f"    for (int j = 0; j < {L}; j++) sum = sum + data[j];\n"
                f"    const float mean = sum * {inv}f;\n    float ss = 0.0f;\n    #pragma omp simd reduction(+:ss)\n"
                f"    for (int j = 0; j < {L}; j++) {{ const float d = data[j] - mean; out[j] = d; ss += d * d; }}\n"
                f"    const float inv_std = 1.0f / sqrtf(ss * {inv}f + {eps}f);\n    #pragma omp simd\n"
                f"    for (int j = 0; j < {L}; j++) out[j] = out[j] * inv_std * {gamma}[j] + {beta}[j];\n}}")

    # crates/session_clang/src/translator.rs:2745-2790 (ReduceMax over the last axes: this
    # restatement's extension in the same style)
    def _reduce(self, n, names, ins, outs, is_max):
        x, y = names
        axes = sorted(a % len(ins[0]) for a in n.attrs["axes"])
        assert axes[0] >= len(ins[0]) - len(axes), "axes must be the innermost dimensions"
        L = int(np.prod(ins[0][axes[0]:]))
        rows = int(np.prod(outs[0]))
        if is_max:
            return (f"for (int i = 0; i < {rows}; i++) {{\n    const float *p = {x} + (size_t)i * {L};\n"
                    f"    float max = -INFINITY;\n    #pragma omp simd reduction(max:max)\n"
                    f"    for (int j = 0; j < {L}; j++) max = fmaxf(p[j], max);\n    {y}[i] = max;\n}}")
        return (f"for (int i = 0; i < {rows}; i++) {{\n    const float *p = {x} + (size_t)i * {L};\n"
                f"    float sum = 0.f;\n    #pragma omp simd reduction(+:sum)\n"
                f"    for (int j = 0; j < {L}; j++) sum += p[j];\n    {y}[i] = sum * (1.f / {L});\n}}")

    def t_reducemean(self, n, names, ins, outs): return self._reduce(n, names, ins, outs, False)
    def t_reducemax(self, n, names, ins, outs): return self._reduce(n, names, ins, outs, True)

    # crates/session_clang/src/translator.rs:1670-1801
    def t_matmul(self, n, names, ins, outs):
        a, b, o = names
        if len(ins[1]) == 2:
            rows = int(np.prod(ins[0][:-1]))
            k, nn = ins[1]
            return (f"cblas_sgemm(CblasRowMajor, CblasNoTrans, CblasNoTrans, {rows}, {nn}, {k}, 1.f, "
                    f"{a}, {k}, {b}, {nn}, 0.f, {o}, {nn});")
        assert len(ins[0]) == len(ins[1]) and list(ins[0][:-2]) == list(ins[1][:-2])
        batch = int(np.prod(ins[0][:-2]))
        m, k = ins[0][-2:]
        nn = ins[1][-1]
        return (f"for (int i = 0; i < {batch}; i++)\n"
                f"    cblas_sgemm(CblasRowMajor, CblasNoTrans, CblasNoTrans, {m}, {nn}, {k}, 1.f,\n"
                f"        {a} + (size_t)i * {m * k}, {k}, {b} + (size_t)i * {k * nn}, {nn}, 0.f, "
                f"{o} + (size_t)i * {m * nn}, {nn});")

    # crates/session_clang/src/translator.rs:1820-1890
    def t_gemm(self, n, names, ins, outs):
        a, b = names[0], names[1]
        o = names[-1]
        ta, tb = bool(n.attrs.get("trans_a", 0)), bool(n.attrs.get("trans_b", 0))
        m = ins[0][1] if ta else ins[0][0]
        k = ins[0][0] if ta else ins[0][1]
        nn = ins[1][0] if tb else ins[1][1]
        fill, beta = "", 0.0
        if len(ins) > 2:
            beta = float(n.attrs.get("beta", 1.0))
            if len(ins[2]) == 1:
                fill = (f"for (int i = 0; i < {m * nn}; i += {nn}) memcpy({o} + i, {names[2]}, "
                        f"{nn} * sizeof(float));\n")
            else:
                fill = f"memcpy({o}, {names[2]}, {m * nn} * sizeof(float));\n"
        return (f"{fill}cblas_sgemm(CblasRowMajor, {'CblasTrans' if ta else 'CblasNoTrans'}, "
                f"{'CblasTrans' if tb else 'CblasNoTrans'}, {m}, {nn}, {k}, {float(n.attrs.get('alpha', 1.0))!r}f, "
                f"{a}, {m if ta else k}, {b}, {k if tb else nn}, {beta!r}f, {o}, {nn});")

    # crates/session_clang/src/translator.rs:716-948 (unit dilation)
    def t_conv2d(self, n, names, ins, outs):
        x, w = names[0], names[1]
        o = names[-1]
        at = n.attrs
        B, C, H, W = ins[0]
        OC, OH, OW = outs[0][1], outs[0][2], outs[0][3]
        kh, kw = at["kernel_shape"]
        sh, sw = at.get("strides", [1, 1])
        pad = list(at.get("padding", [0, 0, 0, 0]))
        pt, pl = pad[0], pad[1]
        group = int(at.get("group", 1))
        icg, ocg = C // group, OC // group
        if len(ins) > 2:
            fill = (f"{{ float *op = {o};\n  for (int b = 0; b < {B}; b++) for (int oc = 0; oc < {OC}; oc++) {{\n"
                    f"      const float bias = {names[2]}[oc];\n"
                    f"      for (int i = 0; i < {OH * OW}; i++) op[i] = bias;\n      op += {OH * OW}; }} }}")
        else:
            fill = f"for (int i = 0; i < {int(np.prod(outs[0]))}; i++) {o}[i] = 0.0f;"
        col_elems = B * C * OH * OW * kh * kw
        im2col = (f"float *col = (float *)malloc(sizeof(float) * {col_elems});\n"
                  f"#pragma omp parallel for num_threads({self.th})\n"
                  f"for (int outer = 0; outer < {B * C}; outer++) {{\n"
                  f"    const float *ip = {x} + (size_t)outer * {H * W};\n"
                  f"    float *cp = col + (size_t)outer * {OH * OW * kh * kw};\n"
                  f"    for (int fy = 0; fy < {kh}; fy++) for (int fx = 0; fx < {kw}; fx++) {{\n"
                  f"        for (int oh = 0; oh < {OH}; oh++) {{\n"
                  f"            float *c = cp + oh * {OW};\n            const int ih = fy + oh * {sh};\n"
                  f"            if ({pt} > ih || ih >= {H} + {pt}) {{ for (int i = 0; i < {OW}; i++) c[i] = 0.f; continue; }}\n"
                  f"            int ow = 0, iw = fx;\n"
                  f"            while (iw < {pl} && ow < {OW}) {{ c[ow] = 0.f; iw += {sw}; ow++; }}\n"
                  f"            const int base = (ih - {pt}) * {W};\n"
                  f"            while (iw < {W} + {pl} && ow < {OW}) {{ c[ow] = ip[base + iw - {pl}]; iw += {sw}; ow++; }}\n"
                  f"            for (; ow < {OW}; ow++) c[ow] = 0.f;\n        }}\n        cp += {OH * OW};\n    }}\n}}")
        k = icg * kh * kw
        gemm = (f"{{ const float *wp = {w}; float *op = {o}; const float *cp = col;\n"
                f"  for (int b = 0; b < {B}; b++) {{\n    wp = {w};\n    for (int g = 0; g < {group}; g++) {{\n"
                f"      cblas_sgemm(CblasRowMajor, CblasNoTrans, CblasNoTrans, {ocg}, {OH * OW}, {k}, 1.f,\n"
                f"          wp, {k}, cp, {OH * OW}, 1.f, op, {OH * OW});\n"
                f"      wp += {ocg * k}; op += {ocg * OH * OW}; cp += {k * OH * OW}; }} }} }}")
        return f"{fill}\n{im2col}\n{gemm}\nfree(col);"

    # crates/session_clang/src/translator.rs:1892-2045: blocks of the contiguous suffix are
    # copied from source offsets computed at translation time.
    def t_transpose(self, n, names, ins, outs):
        x, y = names
        perm = [int(p) for p in n.attrs["perm"]]
        dims = ins[0]
        ist = _strides(dims)
        block, r = 1, len(dims)
        while r > 0 and perm[r - 1] == r - 1:
            block *= dims[r - 1]
            r -= 1
        if r == 0:
            return f"memcpy({y}, {x}, sizeof(float) * {block});"
        od = [dims[p] for p in perm[:r]]
        st = [ist[p] for p in perm[:r]]
        idx = np.zeros((), dtype=np.int64)
        for d, s in zip(od, st):
            idx = (idx[..., None] + np.arange(d, dtype=np.int64) * s)
        table = ", ".join(str(int(v)) for v in np.asarray(idx).reshape(-1))
        nblk = int(np.prod(od))
        copy = (f"{y}[i] = {x}[src_indices[i]];" if block == 1 else
                f"memcpy({y} + (size_t)i * {block}, {x} + src_indices[i], sizeof(float) * {block});")
        return f"static const int src_indices[{nblk}] = {{ {table} }};\nfor (int i = 0; i < {nblk}; i++) {copy}"

    # crates/session_clang/src/translator.rs:2351-2399
    def t_concat(self, n, names, ins, outs):
        o = names[-1]
        ax = n.attrs["axis"] % len(outs[0])
        outer = int(np.prod(outs[0][:ax]))
        lines = []
        for nm, shp in zip(names[:-1], ins):
            ne = int(np.prod(shp[ax:]))
            lines.append(f"    memcpy({o} + offset, {nm} + (size_t)i * {ne}, sizeof(float) * {ne}); offset += {ne};")
        return f"size_t offset = 0;\nfor (int i = 0; i < {outer}; i++) {{\n" + "\n".join(lines) + "\n}"

    # crates/session_clang/src/translator.rs:3084-3155 (opset >= 13: sizes come as an input)
    def t_split(self, n, names, ins, outs):
        x, sp = names[0], names[1]
        onames = names[2:]
        assert n.attrs["axis"] % len(ins[0]) == len(ins[0]) - 1
        L = ins[0][-1]
        rows = int(np.prod(ins[0])) // L
        k = len(onames)
        return (f"size_t offsets[{k}] = {{0}};\nfloat *outputs[] = {{ {', '.join(onames)} }};\n"
                f"for (int i = 0; i < {rows}; i++) {{\n    int s = 0;\n    for (int j = 0; j < {k}; j++) {{\n"
                f"        const int n = (int){sp}[j];\n"
                f"        memcpy(outputs[j] + offsets[j], {x} + (size_t)i * {L} + s, n * sizeof(float));\n"
                f"        offsets[j] += n; s += n;\n    }}\n}}")

    # crates/session_clang/src/translator.rs:2522-2574. The reference's template copies one
    # slice (scalar index, leading axes of extent 1) or rows of a 2-D table; here the same copy
    # runs under an outer loop so that a batch axis before `axis` is covered as well.
    def t_gather(self, n, names, ins, outs):
        data, ind, o = names
        ax = int(n.attrs.get("axis", 0))
        st = _strides(ins[0])[ax]
        outer = int(np.prod(ins[0][:ax]))
        span = ins[0][ax] * st
        count = int(np.prod(ins[1])) if len(ins[1]) else 1
        return (f"for (int i = 0; i < {outer}; i++) for (int j = 0; j < {count}; j++)\n"
                f"    memcpy({o} + ((size_t)i * {count} + j) * {st}, "
                f"{data} + (size_t)i * {span} + {st} * (size_t)({ind}[j]), sizeof(float) * {st});")


class _Regions:
    """First-fit arena with reuse of freed ranges (crates/session_clang/src/translator.rs
    `Regions`): a value's bytes are handed back after its last user."""

    def __init__(self):
        self.live: Dict[int, tuple] = {}
        self.free: List[tuple] = []
        self.top = 0

    def alloc(self, key, size):
        size = (size + 63) // 64 * 64
        for i, (start, length) in enumerate(self.free):
            if length >= size:
                self.free[i] = (start + size, length - size)
                if self.free[i][1] == 0:
                    self.free.pop(i)
                self.live[key] = (start, size)
                return start
        start = self.top
        self.top += size
        self.live[key] = (start, size)
        return start

    def release(self, key):
        start, size = self.live.pop(key)
        self.free.append((start, size))
        self.free.sort()
        merged = []
        for s, l in self.free:
            if merged and merged[-1][0] + merged[-1][1] == s:
                merged[-1] = (merged[-1][0], merged[-1][1] + l)
            else:
                merged.append((s, l))
        self.free = merged


_HEADER = """#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
enum { CblasRowMajor = 101, CblasNoTrans = 111, CblasTrans = 112 };
typedef BLASINT blasint;
typedef void (*sgemm_fn)(int, int, int, blasint, blasint, blasint, float, const float *, blasint,
                         const float *, blasint, float, float *, blasint);
static sgemm_fn cblas_sgemm;
static char *global_memory;
void set_sgemm(void *fn) { cblas_sgemm = (sgemm_fn)fn; }
"""


def translate(model, threads: int, blasint: str = "int"):
    """The C text of the model and the order of its initializers (bound by `set_init`)."""
    g = model.graph
    tr = _Translator(model, threads)
    for v, arr in g.inits.items():
        tr.shapes[v] = list(arr.shape)
    graph_inputs = [i for i in g.inputs if i not in g.inits]
    for v in graph_inputs:
        tr.shapes[v] = list(g.values[v].shape)
    order = model.topo_sort_nodes()
    alias: Dict[int, int] = {}          # Reshape outputs share their input's bytes

    def root(v):
        while v in alias:
            v = alias[v]
        return v

    last_use: Dict[int, int] = {}
    for pos, nid in enumerate(order):
        node = g.nodes[nid]
        outs = _infer(node, [tr.shapes[i] for i in node.inputs], g.inits)
        for o, s in zip(node.outputs, outs):
            tr.shapes[o] = [int(d) for d in s]
        if node.op == "Reshape":
            alias[node.outputs[0]] = node.inputs[0]
    for pos, nid in enumerate(order):
        for i in g.nodes[nid].inputs:
            last_use[root(i)] = pos

    def ctype(v):
        arr = g.inits.get(v)
        if arr is not None and arr.dtype == np.int64:
            return "int64_t"
        if arr is not None and arr.dtype == np.int32:
            return "int32_t"
        return "float"

    regions = _Regions()
    kernels, calls, decls = [], [], []
    init_order = list(g.inits.keys())
    for v in init_order:
        decls.append(f"static const {ctype(v)} *v{v};")
    produced = set()
    for pos, nid in enumerate(order):
        node = g.nodes[nid]
        if node.op == "Reshape":
            o = node.outputs[0]
            if o in g.outputs:
                calls.append(f"memcpy(v{o}, v{node.inputs[0]}, {int(np.prod(tr.shapes[o]))} * sizeof(float));")
            else:
                decls.append(f"static float *v{o};")
                calls.append(f"v{o} = (float *)v{node.inputs[0]};")
        else:
            for o in node.outputs:
                if o in g.outputs:
                    continue
                decls.append(f"static float *v{o};")
                off = regions.alloc(o, 4 * int(np.prod(tr.shapes[o])))
                produced.add(o)
                calls.append(f"v{o} = (float *)(global_memory + {off});")
            kernels.append(f"static void node_{nid}(void) {{\n{tr.body(node)}\n}}\n")
            calls.append(f"node_{nid}();")
        for key in [k for k in list(regions.live) if last_use.get(k, -1) <= pos and k in produced]:
            regions.release(key)
    io = [f"static const float *v{v};" for v in graph_inputs] + [f"static float *v{v};" for v in g.outputs]
    setters = ("void set_init(int i, const void *p) {\n    switch (i) {\n"
               + "".join(f"    case {i}: v{v} = (const {ctype(v)} *)p; break;\n" for i, v in enumerate(init_order))
               + "    }\n}\n")
    entry = ("void initialize(void) { global_memory = (char *)aligned_alloc(64, %d); }\n\n"
             "void trampoline(const void **ins, void **outs) {\n" % max(regions.top, 64)
             + "".join(f"    v{v} = (const float *)ins[{i}];\n" for i, v in enumerate(graph_inputs))
             + "".join(f"    v{v} = (float *)outs[{i}];\n" for i, v in enumerate(g.outputs))
             + "".join(f"    {c}\n" for c in calls) + "}\n")
    text = (_HEADER.replace("BLASINT", blasint) + "\n".join(io + decls) + "\n\n" + "\n".join(kernels)
            + "\n" + setters + "\n" + entry)
    return text, init_order, tr.shapes


class ClangPortSession:
    """Translate, compile (gcc), load, bind the weights; `run(inputs)` like the reference's
    session (crates/session_clang/src/session.rs:30-86)."""

    def __init__(self, model, intra_op_num_threads: int = 1):
        self._model = model
        self.threads = intra_op_num_threads
        self._blas, sgemm_addr, set_threads, blasint = _find_sgemm()
        set_threads(int(intra_op_num_threads))
        text, init_order, self.shapes = translate(model, intra_op_num_threads, blasint)
        os.makedirs(_CACHE, exist_ok=True)
        tag = hashlib.sha1((text + " ".join(CFLAGS)).encode()).hexdigest()[:16]
        so = os.path.join(_CACHE, f"model_{tag}.so")
        if not os.path.exists(so):
            src = os.path.join(_CACHE, f"model_{tag}.c")
            with open(src, "w") as f:
                f.write(text)
            try:
                subprocess.check_call(["gcc", *CFLAGS, "-o", so + ".tmp", src, "-lm"])
                os.replace(so + ".tmp", so)
            finally:
                os.remove(src)      # the index tables of the transposes make it tens of megabytes
        self._lib = ctypes.CDLL(so)
        self._lib.set_sgemm(ctypes.c_void_p(sgemm_addr))
        self._keep = []
        for i, v in enumerate(init_order):
            arr = np.ascontiguousarray(model.graph.inits[v])
            self._keep.append(arr)
            self._lib.set_init(ctypes.c_int(i), ctypes.c_void_p(arr.ctypes.data))
        self._lib.initialize()

    def model(self):
        return self._model

    def run(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        g = self._model.graph
        ins = [np.ascontiguousarray(x, dtype=np.float32) for x in inputs]
        outs = [np.empty(self.shapes[o], dtype=np.float32) for o in g.outputs]
        in_ptrs = (ctypes.c_void_p * len(ins))(*[x.ctypes.data for x in ins])
        out_ptrs = (ctypes.c_void_p * len(outs))(*[y.ctypes.data for y in outs])
        self._lib.trampoline(in_ptrs, out_ptrs)
        return outs


def time_vit(batch: int, threads: int):
    """images/s of the generated-C restatement on ViT-B/16 at `batch`: translation and the gcc
    build are outside the timed region; one warm-up run, then runs for about ten seconds."""
    from altius_b200 import configs
    model, feeds = configs.vit_base_16(batch=batch)
    t0 = time.perf_counter()
    sess = ClangPortSession(model, threads)
    build_s = time.perf_counter() - t0
    x = list(feeds.values())
    sess.run(x)
    runs, t0 = 0, time.perf_counter()
    while True:
        sess.run(x)
        runs += 1
        dt = time.perf_counter() - t0
        if dt > 10.0 or runs >= 50:
            break
    return dict(value=batch * runs / dt, unit="images/s", cores=threads, kind="port",
                sample=f"{runs} forward passes of ViT-B/16 at batch {batch} in {dt:.1f} s; restatement of the "
                       f"reference's generated-C backend, gcc -O3 -march=native -fopenmp, OpenBLAS sgemm, "
                       f"{threads} threads (translate + compile {build_s:.1f} s, not timed)")
