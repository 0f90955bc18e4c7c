// Topological order and static shape inference for the session's graph.
// The rules restate `Model::compute_output_shapes`
// (crates/core/src/analysis/shape.rs:23-654) for the operators this backend
// lowers; `infer_shapes` there (:659-719) is the driver being replaced.
// Failures surface as AC_ERR_SHAPE from altius_cuda_create, never mid-run.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <set>
#include <sstream>

#include "session.h"

namespace ac {

[[noreturn]] void fail(int status, const std::string& msg) { throw BuildError{status, msg}; }

namespace {

const char* kOpNames[] = {
    "Identity", "Conv2d", "Add", "Sub", "Mul", "Div", "Pow", "Greater", "Sqrt", "ReLU", "Gelu",
    "LeakyReLU", "Sigmoid", "Erf", "Tanh", "Clip", "Where", "Softmax", "Cast", "MaxPool",
    "GlobalAveragePool", "Reshape", "Flatten", "Resize", "Concat", "Transpose", "Squeeze",
    "Unsqueeze", "ReduceMin", "ReduceMax", "ReduceMean", "Round", "Exp", "Expand", "Range", "Loop",
    "Tile", "Split", "Slice", "Gather", "Shape", "NonMaxSuppression", "MatMul", "Gemm",
    "BatchNormalization", "LayerNormalization", "HardSigmoid", "Constant", "FusedElemwise"};

std::string dims_str(const Value& v) {
  std::ostringstream o;
  o << "[";
  for (int i = 0; i < v.rank; ++i) o << (i ? ", " : "") << v.dims[i];
  o << "]";
  return o.str();
}

void set_shape(Value& v, int elem_ty, const std::vector<int64_t>& d) {
  if (d.size() > AC_MAX_RANK) fail(AC_ERR_SHAPE, "rank above 8 is not supported");
  if (v.rank >= 0) {  // a shape given in the description must agree
    bool same = v.rank == (int)d.size();
    for (int i = 0; same && i < v.rank; ++i) same = v.dims[i] == d[i];
    if (!same) fail(AC_ERR_SHAPE, "inferred shape disagrees with the described one");
  }
  v.elem_ty = elem_ty;
  v.rank = (int)d.size();
  for (size_t i = 0; i < d.size(); ++i) {
    if (d[i] < 0) fail(AC_ERR_SHAPE, "negative dimension");
    v.dims[i] = d[i];
  }
}

std::vector<int64_t> dims_of(const Value& v) { return std::vector<int64_t>(v.dims, v.dims + v.rank); }

// crates/core/src/fixed_dim.rs:108-133 `broadcast`
std::vector<int64_t> broadcast(const Value& x, const Value& y, const char* op) {
  const int r = std::max(x.rank, y.rank);
  std::vector<int64_t> out(r);
  for (int i = 0; i < r; ++i) {
    const int64_t a = i < x.rank ? x.dims[x.rank - 1 - i] : 1;
    const int64_t b = i < y.rank ? y.dims[y.rank - 1 - i] : 1;
    if (a != b && a != 1 && b != 1)
      fail(AC_ERR_SHAPE, std::string(op) + ": cannot broadcast " + dims_str(x) + " with " + dims_str(y));
    out[r - 1 - i] = a == 1 ? b : a;
  }
  return out;
}

const int64_t* host_i64(const AcSession& s, int vid, const char* what) {
  const Value& v = s.values[vid];
  if (!v.host || v.elem_ty != AC_I64)
    fail(AC_ERR_UNSUPPORTED, std::string(what) + " must be a constant i64 tensor");
  return static_cast<const int64_t*>(v.host);
}

// crates/core/src/analysis/shape.rs:50-61: SAME_UPPER padding.
void same_upper(int64_t ih, int64_t iw, const int64_t* k, const int64_t* st, int64_t* pads) {
  const int64_t out0 = (int64_t)std::ceil((float)ih / (float)st[0]);
  const int64_t out1 = (int64_t)std::ceil((float)iw / (float)st[1]);
  const int64_t pad0 = std::max<int64_t>((out0 - 1) * st[0] + k[0] - ih, 0);
  const int64_t pad1 = std::max<int64_t>((out1 - 1) * st[1] + k[1] - iw, 0);
  pads[0] = pad0 / 2; pads[1] = pad1 / 2; pads[2] = pad0 - pad0 / 2; pads[3] = pad1 - pad1 / 2;
}

}  // namespace

const char* op_name(int op) { return (op >= 0 && op < AC_OP_COUNT) ? kOpNames[op] : "?"; }

// Resolves the 4 pads of a Conv2d / MaxPool node in place (ints layout in the
// public header) and returns them. shape.rs:47-75 and :112-125.
void resolve_pads(Node& n, int pad_pos /* index of auto_pad */, int64_t ih, int64_t iw,
                  int64_t pads[4]) {
  const int64_t* k = &n.ints[0];
  const int64_t* st = &n.ints[2];
  const int64_t auto_pad = n.ints[pad_pos];
  const int npos = n.op == AC_OP_CONV2D ? pad_pos + 2 : pad_pos + 1;
  const int64_t np = n.ints[npos];
  if (auto_pad == 1) {
    same_upper(ih, iw, k, st, pads);
  } else if (np == 2) {
    pads[0] = n.ints[npos + 1]; pads[1] = n.ints[npos + 2]; pads[2] = pads[0]; pads[3] = pads[1];
  } else if (np == 4) {
    for (int i = 0; i < 4; ++i) pads[i] = n.ints[npos + 1 + i];
  } else if (np == 0 && n.op == AC_OP_MAXPOOL) {
    pads[0] = pads[1] = pads[2] = pads[3] = 0;
  } else {
    fail(AC_ERR_SHAPE, "Conv2d: Unknown padding pattern");
  }
}

static void topo_sort(AcSession& s) {
  // Kahn's algorithm with the LIFO work list of `Model::topo_sort_nodes`
  // (crates/core/src/model.rs:61-102).
  const int nn = (int)s.nodes.size();
  std::vector<int> parent(s.values.size(), -1);
  for (int i = 0; i < nn; ++i)
    for (int o : s.nodes[i].outputs) parent[o] = i;
  std::vector<std::vector<int>> users(s.values.size());
  std::vector<int> pending(nn, 0), work;
  for (int i = 0; i < nn; ++i) {
    std::set<int> ins;
    for (int v : s.nodes[i].inputs)
      if (v >= 0 && parent[v] >= 0) ins.insert(v);
    pending[i] = (int)ins.size();
    for (int v : ins) users[v].push_back(i);
    if (ins.empty()) work.push_back(i);
  }
  while (!work.empty()) {
    const int id = work.back();
    work.pop_back();
    s.order.push_back(id);
    for (int o : s.nodes[id].outputs)
      for (int u : users[o])
        if (--pending[u] == 0) work.push_back(u);
  }
  if ((int)s.order.size() != nn) fail(AC_ERR_INVALID, "graph has a cycle or an undefined value");
}

void infer_shapes(AcSession& s) {
  topo_sort(s);
  for (int nid : s.order) {
    Node& n = s.nodes[nid];
    auto in = [&](int i) -> Value& {
      if (i >= (int)n.inputs.size() || n.inputs[i] < 0)
        fail(AC_ERR_INVALID, std::string(op_name(n.op)) + ": missing input");
      Value& v = s.values[n.inputs[i]];
      if (v.rank < 0) fail(AC_ERR_SHAPE, std::string(op_name(n.op)) + ": input shape unknown");
      return v;
    };
    auto has_in = [&](int i) { return i < (int)n.inputs.size() && n.inputs[i] >= 0; };
    auto out = [&](int i) -> Value& { return s.values[n.outputs[i]]; };
    auto need_ints = [&](size_t k) {
      if (n.ints.size() < k) fail(AC_ERR_INVALID, std::string(op_name(n.op)) + ": attributes missing");
    };
    switch (n.op) {
      case AC_OP_IDENTITY:
      case AC_OP_SQRT: case AC_OP_RELU: case AC_OP_LEAKYRELU: case AC_OP_GELU: case AC_OP_SIGMOID:
      case AC_OP_ERF: case AC_OP_TANH: case AC_OP_HARDSIGMOID: case AC_OP_SOFTMAX:
      case AC_OP_BATCHNORMALIZATION: case AC_OP_LAYERNORMALIZATION: {
        if (n.op == AC_OP_LAYERNORMALIZATION && n.outputs.size() != 1)
          fail(AC_ERR_UNSUPPORTED, "LayerNormalization: one output only");  // shape.rs:584
        set_shape(out(0), in(0).elem_ty, dims_of(in(0)));
        break;
      }
      case AC_OP_CAST:
        need_ints(1);
        set_shape(out(0), (int)n.ints[0], dims_of(in(0)));
        break;
      case AC_OP_ADD: case AC_OP_SUB: case AC_OP_MUL: case AC_OP_DIV: case AC_OP_POW:
        set_shape(out(0), in(0).elem_ty, broadcast(in(0), in(1), op_name(n.op)));
        break;
      case AC_OP_GREATER:
        set_shape(out(0), AC_BOOL, broadcast(in(0), in(1), "Greater"));
        break;
      case AC_OP_WHERE: {
        // The reference broadcasts x with y (its two patterns keep the condition inside that
        // shape); the condition takes part here as ONNX defines it.
        Value xy;
        const std::vector<int64_t> d = broadcast(in(1), in(2), "Where");
        xy.rank = (int)d.size();
        for (size_t i = 0; i < d.size(); ++i) xy.dims[i] = d[i];
        set_shape(out(0), in(1).elem_ty, broadcast(xy, in(0), "Where"));
        break;
      }
      case AC_OP_EXPAND: {
        // shape.rs:148-160: the output shape is the `shape` input, taken as it is.
        const Value& sh = in(1);
        if (!sh.host || sh.elem_ty != AC_I64) fail(AC_ERR_UNSUPPORTED, "Expand: shape must be a constant i64 tensor");
        const int64_t* d = static_cast<const int64_t*>(sh.host);
        const int64_t r = sh.numel();
        if (r > AC_MAX_RANK) fail(AC_ERR_SHAPE, "rank above 8 is not supported");
        set_shape(out(0), in(0).elem_ty, std::vector<int64_t>(d, d + r));
        break;
      }
      case AC_OP_RESIZE: {
        // shape.rs:209-254: sizes (4 inputs) or floor(dims * scales) (3 inputs; asymmetric,
        // nearest, floor only).
        need_ints(3);
        const Value& x = in(0);
        if (x.rank != 4) fail(AC_ERR_SHAPE, "Resize: 4-D input expected");
        if (n.inputs.size() == 4) {
          const Value& sz = in(3);
          if (!sz.host || sz.elem_ty != AC_I64 || sz.rank != 1 || sz.dims[0] != 4)
            fail(AC_ERR_UNSUPPORTED, "Resize: sizes must be a constant i64[4]");
          const int64_t* d = static_cast<const int64_t*>(sz.host);
          set_shape(out(0), x.elem_ty, {d[0], d[1], d[2], d[3]});
        } else if (n.inputs.size() == 3) {
          if (n.ints[0] != 0 || n.ints[1] != 0 || n.ints[2] != 0)
            fail(AC_ERR_UNSUPPORTED, "Resize: Unsupported pattern");
          const Value& sc = in(2);
          if (!sc.host || sc.elem_ty != AC_F32 || sc.numel() != 4)
            fail(AC_ERR_UNSUPPORTED, "Resize: scales must be a constant f32[4]");
          const float* f = static_cast<const float*>(sc.host);
          std::vector<int64_t> d(4);
          for (int k = 0; k < 4; ++k) d[k] = (int64_t)std::floor((float)x.dims[k] * f[k]);
          set_shape(out(0), x.elem_ty, d);
        } else {
          fail(AC_ERR_UNSUPPORTED, "Resize: Unsupported pattern");
        }
        break;
      }
      case AC_OP_CONV2D: {
        need_ints(10);
        const Value& x = in(0);
        const Value& w = in(1);
        if (x.rank != 4 || w.rank != 4) fail(AC_ERR_SHAPE, "Conv2d: 4-D input and weight expected");
        int64_t pads[4];
        resolve_pads(n, 7, x.dims[2], x.dims[3], pads);
        const int64_t* k = &n.ints[0]; const int64_t* st = &n.ints[2]; const int64_t* d = &n.ints[4];
        const int64_t oh = (x.dims[2] + pads[0] + pads[2] - d[0] * (k[0] - 1) - 1) / st[0] + 1;
        const int64_t ow = (x.dims[3] + pads[1] + pads[3] - d[1] * (k[1] - 1) - 1) / st[1] + 1;
        set_shape(out(0), x.elem_ty, {x.dims[0], w.dims[0], oh, ow});
        break;
      }
      case AC_OP_MAXPOOL: {
        need_ints(6);
        const Value& x = in(0);
        if (x.rank != 4) fail(AC_ERR_SHAPE, "MaxPool: 4-D input expected");
        int64_t pads[4];
        resolve_pads(n, 4, x.dims[2], x.dims[3], pads);
        const int64_t* k = &n.ints[0]; const int64_t* st = &n.ints[2];
        const int64_t oh = (x.dims[2] + pads[0] + pads[2] - (k[0] - 1) - 1) / st[0] + 1;
        const int64_t ow = (x.dims[3] + pads[1] + pads[3] - (k[1] - 1) - 1) / st[1] + 1;
        set_shape(out(0), x.elem_ty, {x.dims[0], x.dims[1], oh, ow});
        break;
      }
      case AC_OP_GLOBALAVERAGEPOOL: {
        const Value& x = in(0);
        if (x.rank != 4) fail(AC_ERR_SHAPE, "Input must be four dimensions");
        set_shape(out(0), x.elem_ty, {x.dims[0], x.dims[1], 1, 1});
        break;
      }
      case AC_OP_RESHAPE: {
        const Value& x = in(0);
        const Value& sh = in(1);
        const int64_t* spec = host_i64(s, n.inputs[1], "Reshape: shape");
        const int64_t ns = sh.numel();
        int64_t other = 1;
        for (int64_t i = 0; i < ns; ++i)
          if (spec[i] != -1) other *= spec[i];
        std::vector<int64_t> d(ns);
        for (int64_t i = 0; i < ns; ++i) d[i] = spec[i] == -1 ? (other ? x.numel() / other : 0) : spec[i];
        int64_t tot = 1;
        for (int64_t v : d) tot *= v;
        if (tot != x.numel()) fail(AC_ERR_SHAPE, "Reshape: element count changes");
        set_shape(out(0), x.elem_ty, d);
        break;
      }
      case AC_OP_FLATTEN: {
        need_ints(1);
        const Value& x = in(0);
        const int64_t axis = n.ints[0];
        if (axis < 0 || axis > x.rank) fail(AC_ERR_SHAPE, "Flatten: bad axis");
        int64_t a = 1, b = 1;
        for (int i = 0; i < x.rank; ++i) (i < axis ? a : b) *= x.dims[i];
        set_shape(out(0), x.elem_ty, {a, b});
        break;
      }
      case AC_OP_SQUEEZE: case AC_OP_UNSQUEEZE: {
        const Value& x = in(0);
        std::vector<int64_t> axes;
        const bool from_input = n.op == AC_OP_SQUEEZE ? s.opset >= 12 : s.opset >= 13;
        if (from_input && has_in(1)) {
          const int64_t* a = host_i64(s, n.inputs[1], "axes");
          axes.assign(a, a + s.values[n.inputs[1]].numel());
        } else {
          axes = n.ints;
        }
        std::vector<int64_t> d;
        if (n.op == AC_OP_SQUEEZE) {
          for (int i = 0; i < x.rank; ++i)
            if (std::find(axes.begin(), axes.end(), (int64_t)i) == axes.end()) d.push_back(x.dims[i]);
        } else {
          d = dims_of(x);
          for (int64_t a : axes) {
            if (a < 0 || a > (int64_t)d.size()) fail(AC_ERR_SHAPE, "Unsqueeze: bad axis");
            d.insert(d.begin() + a, 1);
          }
        }
        set_shape(out(0), x.elem_ty, d);
        break;
      }
      case AC_OP_CONCAT: {
        need_ints(1);
        std::vector<int64_t> d = dims_of(in(0));
        int64_t axis = n.ints[0];
        if (axis < 0) axis += (int64_t)d.size();
        if (axis < 0 || axis >= (int64_t)d.size()) fail(AC_ERR_SHAPE, "Concat: bad axis");
        int64_t sum = 0;
        for (size_t i = 0; i < n.inputs.size(); ++i) {
          const Value& v = in((int)i);
          if (v.rank != (int)d.size()) fail(AC_ERR_SHAPE, "Concat: rank mismatch");
          sum += v.dims[axis];
        }
        d[axis] = sum;
        set_shape(out(0), in(0).elem_ty, d);
        break;
      }
      case AC_OP_TRANSPOSE: {
        const Value& x = in(0);
        if ((int)n.ints.size() != x.rank) fail(AC_ERR_SHAPE, "Transpose: perm length");
        std::vector<int64_t> d(x.rank);
        for (int i = 0; i < x.rank; ++i) {
          if (n.ints[i] < 0 || n.ints[i] >= x.rank) fail(AC_ERR_SHAPE, "Transpose: bad perm");
          d[i] = x.dims[n.ints[i]];
        }
        set_shape(out(0), x.elem_ty, d);
        break;
      }
      case AC_OP_REDUCEMAX: case AC_OP_REDUCEMEAN: {
        need_ints(1);
        const Value& x = in(0);
        const bool keep = n.ints[0] != 0;
        std::vector<int> axes;
        for (size_t i = 1; i < n.ints.size(); ++i)
          axes.push_back((int)(n.ints[i] < 0 ? n.ints[i] + x.rank : n.ints[i]));
        if (axes.empty() && n.op == AC_OP_REDUCEMAX)
          for (int i = 0; i < x.rank; ++i) axes.push_back(i);
        std::vector<int64_t> d;
        for (int i = 0; i < x.rank; ++i) {
          const bool red = std::find(axes.begin(), axes.end(), i) != axes.end();
          if (!red) d.push_back(x.dims[i]);
          else if (keep) d.push_back(1);
        }
        if (d.empty()) d.push_back(1);
        set_shape(out(0), x.elem_ty, d);
        break;
      }
      case AC_OP_SPLIT: {
        need_ints(1);
        const Value& x = in(0);
        int64_t axis = n.ints[0];
        if (axis < 0) axis += x.rank;
        std::vector<int64_t> sizes;
        if (s.opset >= 13 && has_in(1)) {
          const int64_t* a = host_i64(s, n.inputs[1], "Split: split");
          sizes.assign(a, a + s.values[n.inputs[1]].numel());
        } else {
          sizes.assign(n.ints.begin() + 1, n.ints.end());
        }
        if (sizes.size() != n.outputs.size()) fail(AC_ERR_SHAPE, "Split: sizes vs outputs");
        int64_t tot = 0;
        for (size_t i = 0; i < sizes.size(); ++i) {
          std::vector<int64_t> d = dims_of(x);
          d[axis] = sizes[i];
          tot += sizes[i];
          set_shape(out((int)i), x.elem_ty, d);
        }
        if (tot != x.dims[axis]) fail(AC_ERR_SHAPE, "Split: sizes do not cover the axis");
        break;
      }
      case AC_OP_SLICE: {
        const Value& x = in(0);
        const int64_t* starts = host_i64(s, n.inputs[1], "Slice: starts");
        const int64_t* ends = host_i64(s, n.inputs[2], "Slice: ends");
        const int64_t* axes = host_i64(s, n.inputs[3], "Slice: axes");
        const int64_t na = s.values[n.inputs[3]].numel();
        const int64_t* steps = has_in(4) ? host_i64(s, n.inputs[4], "Slice: steps") : nullptr;
        std::vector<int64_t> d = dims_of(x);
        for (int64_t i = 0; i < na; ++i) {
          const int64_t ax = axes[i] < 0 ? axes[i] + x.rank : axes[i];
          const int64_t st = steps ? steps[i] : 1;
          if (starts[i] < 0 || ends[i] < 0 || st <= 0 || ax < 0 || ax >= x.rank)
            fail(AC_ERR_UNSUPPORTED, "Slice: negative starts/ends/steps are not supported");
          const int64_t end = std::min(ends[i], x.dims[ax]);
          const int64_t od = (end - starts[i] + st - 1) / st;
          if (od <= 0) fail(AC_ERR_SHAPE, "Slice: empty result");
          d[ax] = od;
        }
        set_shape(out(0), x.elem_ty, d);
        break;
      }
      case AC_OP_GATHER: {
        need_ints(1);
        const Value& x = in(0);
        const Value& idx = in(1);
        const int64_t axis = n.ints[0];
        if (axis < 0 || axis >= x.rank) fail(AC_ERR_SHAPE, "Gather: bad axis");
        std::vector<int64_t> d = dims_of(x);
        const bool scalar = idx.rank == 0 || (idx.rank == 1 && idx.dims[0] <= 1);
        if (scalar) {
          d.erase(d.begin() + axis);
        } else if (idx.rank == 2 && idx.dims[0] == 1 && axis == 0) {
          d.erase(d.begin());
          d.insert(d.begin(), idx.dims[1]);
          d.insert(d.begin(), 1);
        } else {
          fail(AC_ERR_UNSUPPORTED, "Gather: Unsupported indices shape");
        }
        set_shape(out(0), x.elem_ty, d);
        break;
      }
      case AC_OP_SHAPE:
        // shape.rs:516-524 asserts start == 0 and no end.
        if (n.ints.size() >= 2 && (n.ints[0] != 0 || n.ints[1] != 0))
          fail(AC_ERR_UNSUPPORTED, "Shape: start / end are not supported");
        set_shape(out(0), AC_I64, {(int64_t)in(0).rank});
        break;
      case AC_OP_MATMUL: {
        const Value& a = in(0);
        const Value& b = in(1);
        std::vector<int64_t> d;
        if (a.rank == 2 && b.rank == 2 && a.dims[1] == b.dims[0]) d = {a.dims[0], b.dims[1]};
        else if (a.rank == 3 && b.rank == 2 && a.dims[2] == b.dims[0]) d = {a.dims[0], a.dims[1], b.dims[1]};
        else if (a.rank == 3 && b.rank == 3 && a.dims[0] == b.dims[0] && a.dims[2] == b.dims[1])
          d = {a.dims[0], a.dims[1], b.dims[2]};
        else if (a.rank == 4 && b.rank == 4 && a.dims[0] == b.dims[0] && a.dims[1] == b.dims[1] &&
                 a.dims[3] == b.dims[2])
          d = {a.dims[0], a.dims[1], a.dims[2], b.dims[3]};
        else
          fail(AC_ERR_SHAPE, "MatMul: A shape: " + dims_str(a) + ", B shape: " + dims_str(b));
        set_shape(out(0), a.elem_ty, d);
        break;
      }
      case AC_OP_GEMM: {
        need_ints(2);
        const Value& a = in(0);
        const Value& b = in(1);
        if (a.rank != 2 || b.rank != 2) fail(AC_ERR_SHAPE, "Gemm: 2-D operands expected");
        const int64_t m = n.ints[0] ? a.dims[1] : a.dims[0], ka = n.ints[0] ? a.dims[0] : a.dims[1];
        const int64_t kb = n.ints[1] ? b.dims[1] : b.dims[0], nn = n.ints[1] ? b.dims[0] : b.dims[1];
        if (ka != kb) fail(AC_ERR_SHAPE, "Gemm: inner dimensions differ");
        set_shape(out(0), a.elem_ty, {m, nn});
        break;
      }
      default:
        fail(AC_ERR_UNSUPPORTED, std::string(op_name(n.op)) + ": Kernel not implemented");
    }
    // Host evaluation of constant shape tensors (Shape of a static value).
    if (n.op == AC_OP_SHAPE) {
      Value& o = out(0);
      o.host_owned.resize(sizeof(int64_t) * in(0).rank);
      int64_t* d = reinterpret_cast<int64_t*>(o.host_owned.data());
      for (int i = 0; i < in(0).rank; ++i) d[i] = in(0).dims[i];
      o.host = o.host_owned.data();
    }
  }
  for (int o : s.outputs)
    if (s.values[o].rank < 0) fail(AC_ERR_SHAPE, "graph output shape could not be inferred");
}

}  // namespace ac
