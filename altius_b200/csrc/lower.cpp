// Lowering: op graph (after altius's fusion passes and shape inference) ->
// static schedule of kernel launches over storages.
//
//  1. values get storages; Reshape / Flatten / Squeeze / Unsqueeze / Identity
//     alias their input (the reference shares the buffer too: `copy_data_from`
//     is an Arc clone, crates/core/src/tensor.rs:340-342);
//  2. producer/consumer folds are detected (disabled by options.disable_fusion):
//       MatMul|Gemm|Conv2d -> bias Add -> ReLU|Gelu|HardSigmoid|HardSwish -> residual Add
//       Mul|Div by a scalar -> Softmax
//       bias Add -> Gelu -> residual Add -> LayerNormalization
//       HardSigmoid -> Mul (HardSwish), Transpose(last two) -> MatMul rhs
//  3. every remaining node becomes one or more kernel launches;
//  4. steps are ordered by their data dependencies.
//
// What each node computes follows `run_node`'s dispatch
// (crates/session_interpreter/src/session.rs:168-249).
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <set>

#include "session.h"

namespace ac {
namespace {

struct Ctx {
  AcSession& s;
  std::vector<int> producer;                 // value -> node
  std::vector<std::vector<int>> consumers;   // value -> node ids (one entry per use)
  std::vector<char> is_output;
  std::vector<char> absorbed;                // node folded into another node's kernel
  // Values that a CTA-pair GEMM takes as its A operand already split into fp16 hi / lo halves
  // (scratch values `hi`, `lo`). `produced`: a step emitted so far writes the halves (the kernel
  // that computes the value, or a split kernel); `fp32_needed`: someone still reads the value
  // itself, so its producer writes it as well.
  // The halves are on the fixed scale (f16_split_fixed): X = x * 2^8, hi = rn(X), lo = rn(X - hi).
  struct Split { int hi = -1, lo = -1; bool produced = false, fp32_needed = true; };
  std::map<int, Split> split;
  explicit Ctx(AcSession& s_) : s(s_) {}

  Value& val(int v) { return s.values[v]; }
  bool single_use(int v) const { return consumers[v].size() == 1 && !is_output[v]; }
  int only_consumer(int v) const { return consumers[v][0]; }
  Node& node(int n) { return s.nodes[n]; }

  int new_storage(size_t bytes, bool weight = false, bool pinned = false) {
    Storage st;
    st.bytes = std::max<size_t>(bytes, 4);
    st.weight = weight;
    st.pinned_live = pinned;
    s.storages.push_back(st);
    return (int)s.storages.size() - 1;
  }
};

bool same_dims(const Value& a, const Value& b) {
  if (a.rank != b.rank) return false;
  for (int i = 0; i < a.rank; ++i)
    if (a.dims[i] != b.dims[i]) return false;
  return true;
}

// True when `v` broadcasts against [.., n] as a vector along the last axis.
bool is_last_axis_vector(const Value& v, int64_t n) {
  if (v.rank < 1 || v.numel() != n || v.dims[v.rank - 1] != n) return false;
  return true;
}
// True when `v` is a per-channel vector for an NCHW tensor: [c,1,1] or [1,c,1,1].
bool is_channel_vector(const Value& v, int64_t c) {
  if (v.numel() != c) return false;
  if (v.rank == 3) return v.dims[0] == c;
  if (v.rank == 4) return v.dims[1] == c;
  return false;
}

double f32_bytes(const Value& v) { return (double)v.bytes(); }

// ---- fused-group descriptions ----------------------------------------------------
struct Epilogue {
  int bias = -1;          // value id of the bias vector
  int act = ACT_NONE;
  float act_alpha = 0, act_beta = 0;
  int residual = -1;
  int out = -1;           // final value written
  int trans_b_src = -1;   // MatMul rhs taken from the input of an absorbed Transpose
};

struct LnFusion {
  int x = -1, pre_bias = -1, residual = -1, sum_val = -1;
  int gelu = 0;
};

struct HeadView {       // a [B*H, T, hd] operand that is a strided view of a [B, T, C] tensor
  int src = -1;         // the [B, T, C] value
  int64_t col = 0;      // first column of this operand inside C
  int64_t B = 0, H = 0, T = 0, hd = 0, C = 0;
};

struct AttentionFusion {
  HeadView q, k, v;
  int scale = -1, scale_mode = 0;
  int out = -1;         // the [B, T, H*hd] result
};

struct Plan {
  std::map<int, AttentionFusion> attention;  // Softmax node -> whole attention core
  std::map<int, Epilogue> epi;      // base node (MatMul/Gemm/Conv2d) -> epilogue
  std::map<int, int> softmax_scale; // Softmax node -> Mul/Div node folded in
  std::map<int, int> softmax_mask;  // Softmax node -> Where(mask, x, c) node folded in
  std::map<int, LnFusion> ln;       // LayerNormalization node -> folded producers
  std::map<int, int> hardswish;     // Mul node -> HardSigmoid node folded in
  std::map<int, int> reduce_sibling; // ReduceMean node -> ReduceMax node of the same rows computed with it
  struct SeGate { int x, gate; };
  std::map<int, SeGate> se_gate;    // pointwise Conv2d node -> squeeze-excite Mul folded into its input
};

// Recognises `hs = HardSigmoid(t); m = Mul(t, hs)` hanging off value t whose only
// uses are those two nodes. Returns the Mul node or -1.
int match_hardswish_pair(Ctx& c, int t, int* hs_node) {
  if (c.is_output[t] || c.consumers[t].size() != 2) return -1;
  for (int k = 0; k < 2; ++k) {
    const int h = c.consumers[t][k], m = c.consumers[t][1 - k];
    if (c.absorbed[h] || c.absorbed[m]) continue;
    if (c.node(h).op != AC_OP_HARDSIGMOID || c.node(m).op != AC_OP_MUL) continue;
    const int hv = c.node(h).outputs[0];
    if (!c.single_use(hv) || c.only_consumer(hv) != m) continue;
    const Node& mul = c.node(m);
    if (!((mul.inputs[0] == t && mul.inputs[1] == hv) || (mul.inputs[1] == t && mul.inputs[0] == hv)))
      continue;
    *hs_node = h;
    return m;
  }
  return -1;
}


// Walks back from a [B*H, T, hd] MatMul operand through
//   Reshape <- Transpose[0,2,1,3] <- Reshape <- (Split output | plain [B,T,C] value)
// collecting the nodes; every intermediate must have exactly one user.
bool trace_head_view(Ctx& c, int v, HeadView* out, std::vector<int>* nodes) {
  const Value& v3 = c.val(v);
  if (v3.rank != 3 || !c.single_use(v)) return false;
  const int r2 = c.producer[v];
  if (r2 < 0 || c.absorbed[r2] || c.node(r2).op != AC_OP_RESHAPE) return false;
  const int t1 = c.node(r2).inputs[0];
  const Value& v4 = c.val(t1);
  if (v4.rank != 4 || !c.single_use(t1) || v4.dims[0] * v4.dims[1] != v3.dims[0] ||
      v4.dims[2] != v3.dims[1] || v4.dims[3] != v3.dims[2]) return false;
  const int tr = c.producer[t1];
  if (tr < 0 || c.absorbed[tr] || c.node(tr).op != AC_OP_TRANSPOSE) return false;
  const Node& tn = c.node(tr);
  if (tn.ints.size() != 4 || tn.ints[0] != 0 || tn.ints[1] != 2 || tn.ints[2] != 1 || tn.ints[3] != 3) return false;
  const int t0 = tn.inputs[0];
  if (!c.single_use(t0)) return false;
  const int r1 = c.producer[t0];
  if (r1 < 0 || c.absorbed[r1] || c.node(r1).op != AC_OP_RESHAPE) return false;
  const int s0 = c.node(r1).inputs[0];
  const Value& sv = c.val(s0);
  const int64_t B = v4.dims[0], H = v4.dims[1], T = v4.dims[2], hd = v4.dims[3];
  if (sv.rank != 3 || sv.dims[0] != B || sv.dims[1] != T || sv.dims[2] != H * hd) return false;
  out->B = B; out->H = H; out->T = T; out->hd = hd;
  nodes->push_back(r2); nodes->push_back(tr); nodes->push_back(r1);
  // Optional Split on the last axis: read in place from its input.
  const int sp = c.producer[s0];
  if (sp >= 0 && !c.absorbed[sp] && c.node(sp).op == AC_OP_SPLIT && c.single_use(s0)) {
    const Node& sn = c.node(sp);
    const Value& in = c.val(sn.inputs[0]);
    int64_t axis = sn.ints[0] < 0 ? sn.ints[0] + in.rank : sn.ints[0];
    if (in.rank == 3 && axis == 2 && !in.is_const) {
      int64_t col = 0;
      for (int o : sn.outputs) {
        if (o == s0) break;
        col += c.val(o).dims[2];
      }
      out->src = sn.inputs[0]; out->col = col; out->C = in.dims[2];
      nodes->push_back(-1 - sp);   // marks the Split: absorbed only if all its outputs are
      return true;
    }
  }
  out->src = s0; out->col = 0; out->C = sv.dims[2];
  return true;
}

// MatMul(q, Transpose(k)) -> [Mul|Div scalar] -> Softmax -> MatMul(., v) -> Reshape ->
// Transpose[0,2,1,3] -> Reshape, with q, k, v head views of [B,T,C] tensors.
void detect_attention(Ctx& c, Plan& plan) {
  for (int nid : c.s.order) {
    Node& sm = c.node(nid);
    if (c.absorbed[nid] || sm.op != AC_OP_SOFTMAX) continue;
    std::vector<int> nodes;
    AttentionFusion f;
    int x = sm.inputs[0];
    if (c.val(x).rank != 3 || !c.single_use(x)) continue;
    const int64_t sm_axis = sm.ints.empty() ? -1 : sm.ints[0];
    if (!(sm_axis == -1 || sm_axis == c.val(x).rank - 1)) continue;   // the fused kernel is a last-axis softmax
    int px = c.producer[x];
    if (px < 0 || c.absorbed[px]) continue;
    if (c.node(px).op == AC_OP_MUL || c.node(px).op == AC_OP_DIV) {
      Node& m = c.node(px);
      const bool b_scalar = c.val(m.inputs[1]).numel() == 1;
      const bool a_scalar = c.val(m.inputs[0]).numel() == 1 && m.op == AC_OP_MUL;
      if (!b_scalar && !a_scalar) continue;
      f.scale = b_scalar ? m.inputs[1] : m.inputs[0];
      f.scale_mode = m.op == AC_OP_MUL ? 1 : 2;
      nodes.push_back(px);
      x = b_scalar ? m.inputs[0] : m.inputs[1];
      if (!c.single_use(x)) continue;
      px = c.producer[x];
      if (px < 0 || c.absorbed[px]) continue;
    }
    if (c.node(px).op != AC_OP_MATMUL) continue;
    Node& m1 = c.node(px);
    nodes.push_back(px);
    // rhs must be Transpose[0,2,1] of k
    const int kt = m1.inputs[1];
    const int tp = c.producer[kt];
    if (tp < 0 || c.absorbed[tp] || c.node(tp).op != AC_OP_TRANSPOSE || !c.single_use(kt)) continue;
    const Node& tn = c.node(tp);
    if (tn.ints.size() != 3 || tn.ints[0] != 0 || tn.ints[1] != 2 || tn.ints[2] != 1) continue;
    nodes.push_back(tp);
    if (!trace_head_view(c, m1.inputs[0], &f.q, &nodes)) continue;
    if (!trace_head_view(c, tn.inputs[0], &f.k, &nodes)) continue;
    // Softmax -> MatMul(P, v)
    const int pv = sm.outputs[0];
    if (!c.single_use(pv)) continue;
    const int m2n = c.only_consumer(pv);
    Node& m2 = c.node(m2n);
    if (c.absorbed[m2n] || m2.op != AC_OP_MATMUL || m2.inputs[0] != pv) continue;
    nodes.push_back(m2n);
    if (!trace_head_view(c, m2.inputs[1], &f.v, &nodes)) continue;
    if (f.q.B != f.k.B || f.q.B != f.v.B || f.q.H != f.k.H || f.q.H != f.v.H || f.q.T != f.k.T ||
        f.q.T != f.v.T || f.q.hd != f.k.hd || f.q.hd != f.v.hd || f.q.C != f.k.C || f.q.C != f.v.C)
      continue;
    if (f.q.hd != 64 || f.q.T > 256 || f.q.B * f.q.H > 65535 || (f.q.C % 4) || (f.q.col % 4) ||
        (f.k.col % 4) || (f.v.col % 4))
      continue;
    // O [BH,T,hd] -> Reshape [B,H,T,hd] -> Transpose [0,2,1,3] -> Reshape [B,T,D]
    const int o3 = m2.outputs[0];
    if (!c.single_use(o3)) continue;
    const int r1 = c.only_consumer(o3);
    if (c.absorbed[r1] || c.node(r1).op != AC_OP_RESHAPE) continue;
    const int o4 = c.node(r1).outputs[0];
    const Value& o4v = c.val(o4);
    if (o4v.rank != 4 || o4v.dims[0] != f.q.B || o4v.dims[1] != f.q.H || o4v.dims[2] != f.q.T ||
        o4v.dims[3] != f.q.hd || !c.single_use(o4)) continue;
    const int tr = c.only_consumer(o4);
    if (c.absorbed[tr] || c.node(tr).op != AC_OP_TRANSPOSE) continue;
    const Node& otn = c.node(tr);
    if (otn.ints.size() != 4 || otn.ints[0] != 0 || otn.ints[1] != 2 || otn.ints[2] != 1 || otn.ints[3] != 3) continue;
    const int o5 = otn.outputs[0];
    if (!c.single_use(o5)) continue;
    const int r2 = c.only_consumer(o5);
    if (c.absorbed[r2] || c.node(r2).op != AC_OP_RESHAPE) continue;
    const int out = c.node(r2).outputs[0];
    const Value& ov = c.val(out);
    if (ov.rank != 3 || ov.dims[0] != f.q.B || ov.dims[1] != f.q.T || ov.dims[2] != f.q.H * f.q.hd) continue;
    nodes.push_back(r1); nodes.push_back(tr); nodes.push_back(r2);
    f.out = out;
    // Commit: absorb the chain. A Split is absorbed when every output of it feeds this core.
    std::map<int, int> split_uses;
    for (int id : nodes)
      if (id < 0) split_uses[-1 - id]++;
    bool ok = true;
    for (auto& kv : split_uses)
      if ((int)c.node(kv.first).outputs.size() != kv.second) ok = false;   // partly used Split: keep it simple
    if (!ok) continue;
    for (int id : nodes) c.absorbed[id < 0 ? -1 - id : id] = 1;
    plan.attention[nid] = f;
  }
}

void detect_epilogues(Ctx& c, Plan& plan) {
  AcSession& s = c.s;
  for (int nid : s.order) {
    Node& n = c.node(nid);
    if (c.absorbed[nid]) continue;
    if (n.op != AC_OP_MATMUL && n.op != AC_OP_GEMM && n.op != AC_OP_CONV2D) continue;
    Epilogue e;
    int cur = n.outputs[0];
    const Value& ov = c.val(cur);
    const bool conv = n.op == AC_OP_CONV2D;
    // rhs Transpose of the last two dims -> read the untransposed operand.
    if (n.op == AC_OP_MATMUL) {
      const int bv = n.inputs[1];
      const int tp = c.producer[bv];
      if (tp >= 0 && !c.absorbed[tp] && c.node(tp).op == AC_OP_TRANSPOSE && c.single_use(bv) &&
          !c.val(bv).is_const) {
        const Node& t = c.node(tp);
        const int r = (int)t.ints.size();
        bool swap_last = r >= 2 && t.ints[r - 1] == r - 2 && t.ints[r - 2] == r - 1;
        for (int i = 0; swap_last && i < r - 2; ++i) swap_last = t.ints[i] == i;
        if (swap_last) {
          e.trans_b_src = t.inputs[0];
          c.absorbed[tp] = 1;
        }
      }
    }
    // bias Add
    const bool has_bias_input = (n.op == AC_OP_GEMM || conv) && n.inputs.size() > 2 && n.inputs[2] >= 0;
    if (!has_bias_input && c.single_use(cur)) {
      const int an = c.only_consumer(cur);
      Node& a = c.node(an);
      if (!c.absorbed[an] && a.op == AC_OP_ADD) {
        const int other = a.inputs[0] == cur ? a.inputs[1] : a.inputs[0];
        const Value& bv = c.val(other);
        const bool ok = conv ? is_channel_vector(bv, ov.dims[1])
                             : is_last_axis_vector(bv, ov.dims[ov.rank - 1]);
        if (ok && other != cur && same_dims(c.val(a.outputs[0]), ov)) {
          e.bias = other;
          c.absorbed[an] = 1;
          cur = a.outputs[0];
        }
      }
    }
    // activation
    if (c.single_use(cur)) {
      const int un = c.only_consumer(cur);
      Node& u = c.node(un);
      if (!c.absorbed[un]) {
        if (u.op == AC_OP_RELU) e.act = ACT_RELU;
        else if (u.op == AC_OP_GELU) e.act = ACT_GELU;
        else if (u.op == AC_OP_HARDSIGMOID) {
          e.act = ACT_HARDSIGMOID;
          e.act_alpha = u.floats.size() > 0 ? u.floats[0] : 0.2f;
          e.act_beta = u.floats.size() > 1 ? u.floats[1] : 0.5f;
        }
        if (e.act != ACT_NONE) {
          c.absorbed[un] = 1;
          cur = u.outputs[0];
        }
      }
    } else {
      int hs = -1;
      const int mul = match_hardswish_pair(c, cur, &hs);
      if (mul >= 0) {
        e.act = ACT_HARDSWISH;
        e.act_alpha = c.node(hs).floats.size() > 0 ? c.node(hs).floats[0] : 0.2f;
        e.act_beta = c.node(hs).floats.size() > 1 ? c.node(hs).floats[1] : 0.5f;
        c.absorbed[hs] = 1;
        c.absorbed[mul] = 1;
        cur = c.node(mul).outputs[0];
      }
    }
    // residual Add (same shape, other operand produced outside this chain)
    if (c.single_use(cur)) {
      const int an = c.only_consumer(cur);
      Node& a = c.node(an);
      if (!c.absorbed[an] && a.op == AC_OP_ADD && a.inputs[0] != a.inputs[1]) {
        const int other = a.inputs[0] == cur ? a.inputs[1] : a.inputs[0];
        if (same_dims(c.val(other), c.val(cur)) && same_dims(c.val(a.outputs[0]), c.val(cur))) {
          e.residual = other;
          c.absorbed[an] = 1;
          cur = a.outputs[0];
        }
      }
    }
    e.out = cur;
    if (e.bias >= 0 || e.act != ACT_NONE || e.residual >= 0 || e.trans_b_src >= 0) plan.epi[nid] = e;
  }
}

// Softmax <- [Where(mask, ., c)] <- [Mul | Div by a scalar]: the masked, scaled softmax of an
// attention block in one kernel. The mask is a bool tensor over the trailing dims of the scores
// (broadcast over the leading ones: the interpreter's second Where pattern,
// session.rs:958-987), `c` a scalar.
void detect_softmax_scale(Ctx& c, Plan& plan) {
  for (int nid : c.s.order) {
    Node& n = c.node(nid);
    if (c.absorbed[nid] || n.op != AC_OP_SOFTMAX) continue;
    int x = n.inputs[0];
    const Value& sv = c.val(x);
    const int64_t axis = n.ints.empty() ? -1 : n.ints[0];
    if (!(axis == -1 || axis == sv.rank - 1)) continue;   // left to lower_node, which rejects it
    if (sv.elem_ty != AC_F32 || sv.rank < 1) continue;
    int p = c.producer[x];
    if (p >= 0 && !c.absorbed[p] && c.single_use(x) && c.node(p).op == AC_OP_WHERE) {
      const Node& w = c.node(p);
      const Value& cv = c.val(w.inputs[0]);
      const Value& xv = c.val(w.inputs[1]);
      const Value& yv = c.val(w.inputs[2]);
      bool ok = cv.elem_ty == AC_BOOL && same_dims(xv, sv) && yv.numel() == 1 && xv.elem_ty == AC_F32 &&
                yv.elem_ty == AC_F32 && cv.rank <= sv.rank && cv.rank >= 1;
      // The mask's dims, leading 1s aside, are the trailing dims of the scores.
      int lead = 0;
      while (ok && lead < cv.rank - 1 && cv.dims[lead] == 1) ++lead;
      for (int i = lead; ok && i < cv.rank; ++i) ok = cv.dims[i] == sv.dims[sv.rank - cv.rank + i];
      if (ok) {
        plan.softmax_mask[nid] = p;
        c.absorbed[p] = 1;
        x = w.inputs[1];
        p = c.producer[x];
      }
    }
    if (p < 0 || c.absorbed[p] || !c.single_use(x)) continue;
    Node& m = c.node(p);
    if (m.op != AC_OP_MUL && m.op != AC_OP_DIV) continue;
    const Value& a = c.val(m.inputs[0]);
    const Value& b = c.val(m.inputs[1]);
    const bool b_scalar = b.numel() == 1 && same_dims(a, c.val(x));
    const bool a_scalar = a.numel() == 1 && same_dims(b, c.val(x)) && m.op == AC_OP_MUL;
    if (!b_scalar && !a_scalar) continue;
    plan.softmax_scale[nid] = p;
    c.absorbed[p] = 1;
  }
}

void detect_layer_norm(Ctx& c, Plan& plan) {
  for (int nid : c.s.order) {
    Node& n = c.node(nid);
    if (c.absorbed[nid] || n.op != AC_OP_LAYERNORMALIZATION) continue;
    const Value& xv = c.val(n.inputs[0]);
    const int64_t len = xv.dims[xv.rank - 1];
    LnFusion f;
    int cur = n.inputs[0];
    // residual Add feeding the LayerNorm (its sum may have other users).
    {
      const int p = c.producer[cur];
      if (p >= 0 && !c.absorbed[p] && c.node(p).op == AC_OP_ADD && !c.val(cur).is_const) {
        Node& a = c.node(p);
        const int i0 = a.inputs[0], i1 = a.inputs[1];
        if (i0 != i1 && same_dims(c.val(i0), xv) && same_dims(c.val(i1), xv)) {
          // Prefer as the main chain the operand that itself continues into Gelu / bias Add.
          auto chain_like = [&](int v) {
            const int q = c.producer[v];
            if (q < 0 || c.absorbed[q] || !c.single_use(v)) return false;
            return c.node(q).op == AC_OP_GELU || c.node(q).op == AC_OP_ADD;
          };
          int main = i0, res = i1;
          if (!chain_like(i0) && chain_like(i1)) { main = i1; res = i0; }
          f.residual = res;
          if (!c.single_use(cur)) f.sum_val = cur;
          c.absorbed[p] = 1;
          cur = main;
        }
      }
    }
    if (f.residual >= 0) {
      const int p = c.producer[cur];
      if (p >= 0 && !c.absorbed[p] && c.node(p).op == AC_OP_GELU && c.single_use(cur)) {
        f.gelu = 1;
        c.absorbed[p] = 1;
        cur = c.node(p).inputs[0];
      }
      const int q = c.producer[cur];
      if (q >= 0 && !c.absorbed[q] && c.node(q).op == AC_OP_ADD && c.single_use(cur)) {
        Node& a = c.node(q);
        for (int k = 0; k < 2; ++k) {
          const int main = a.inputs[k], vec = a.inputs[1 - k];
          if (main != vec && same_dims(c.val(main), xv) && c.val(vec).rank == 1 &&
              c.val(vec).dims[0] == len) {
            f.pre_bias = vec;
            c.absorbed[q] = 1;
            cur = main;
            break;
          }
        }
      }
    }
    f.x = cur;
    if (f.residual >= 0) plan.ln[nid] = f;
  }
}

void detect_hardswish(Ctx& c, Plan& plan) {
  for (int nid : c.s.order) {
    Node& n = c.node(nid);
    if (c.absorbed[nid] || n.op != AC_OP_HARDSIGMOID) continue;
    const int t = n.inputs[0];
    const int hv = n.outputs[0];
    if (!c.single_use(hv)) continue;
    const int m = c.only_consumer(hv);
    Node& mul = c.node(m);
    if (c.absorbed[m] || mul.op != AC_OP_MUL) continue;
    const int other = mul.inputs[0] == hv ? mul.inputs[1] : mul.inputs[0];
    if (other != t || mul.inputs[0] == mul.inputs[1]) continue;
    plan.hardswish[m] = nid;
    c.absorbed[nid] = 1;
  }
}

// Squeeze-excite gate: Mul(x [N,C,H,W], g [N,C,1,1]) whose only user is a pointwise Conv2d that
// the tensor-core kernel runs with the planes as its [K, N] operand. The multiply moves into
// that kernel's operand split (one fp32 multiply per element, the bits of the separate Mul):
// the gated feature map is never written or re-read.
void detect_se_gate(Ctx& c, Plan& plan) {
  const int mode = c.s.opt.gemm_mode;
  if (mode == 1 || mode == 2) return;
  for (int nid : c.s.order) {
    const Node& m = c.node(nid);
    if (c.absorbed[nid] || m.op != AC_OP_MUL) continue;
    int x = -1, g = -1;
    for (int k = 0; k < 2; ++k) {
      const Value& a = c.val(m.inputs[k]);
      const Value& b = c.val(m.inputs[1 - k]);
      if (a.rank == 4 && b.rank == 4 && a.elem_ty == AC_F32 && b.elem_ty == AC_F32 && b.dims[0] == a.dims[0] &&
          b.dims[1] == a.dims[1] && b.dims[2] == 1 && b.dims[3] == 1 && a.dims[2] * a.dims[3] > 1) {
        x = m.inputs[k]; g = m.inputs[1 - k];
      }
    }
    if (x < 0 || c.val(x).is_const || c.val(g).is_const) continue;
    const int o = m.outputs[0];
    if (!c.single_use(o)) continue;
    const int cn = c.only_consumer(o);
    const Node& conv = c.node(cn);
    if (c.absorbed[cn] || conv.op != AC_OP_CONV2D || conv.inputs[0] != o) continue;
    const Value& xv = c.val(x);
    const Value& ov = c.val(conv.outputs[0]);
    const int64_t hw = xv.dims[2] * xv.dims[3], ch = xv.dims[1];
    const bool pointwise = conv.ints[0] == 1 && conv.ints[1] == 1 && conv.ints[2] == 1 && conv.ints[3] == 1 &&
                           conv.ints[6] == 1 && conv.ints[7] == 0;
    bool nopad = true;
    for (int64_t k = 0; k < conv.ints[9]; ++k) nopad = nopad && conv.ints[10 + k] == 0;
    const double flops = 2.0 * xv.dims[0] * ov.dims[1] * hw * ch;
    // The conditions under which lower_conv / emit_gemm take the [K, N] tensor-core path.
    if (!pointwise || !nopad || (hw % 4) != 0 || (ch % 4) != 0 || ch < 8 || flops < double(1 << 23) ||
        xv.dims[0] > 65535 || !c.val(conv.inputs[1]).is_const)
      continue;
    plan.se_gate[cn] = Plan::SeGate{x, g};
    c.absorbed[nid] = 1;
  }
}

// ReduceMean and ReduceMax over the last axis of the same value: one pass over the rows.
void detect_reduce_siblings(Ctx& c, Plan& plan) {
  auto last_axis_only = [&](const Node& n) {
    const Value& xv = c.val(n.inputs[0]);
    if (n.ints.size() != 2 || xv.elem_ty != AC_F32 || xv.rank < 1) return false;
    const int64_t ax = n.ints[1] < 0 ? n.ints[1] + xv.rank : n.ints[1];
    return ax == xv.rank - 1;
  };
  for (int nid : c.s.order) {
    const Node& n = c.node(nid);
    if (c.absorbed[nid] || n.op != AC_OP_REDUCEMEAN || !last_axis_only(n)) continue;
    for (int u : c.consumers[n.inputs[0]]) {
      const Node& m = c.node(u);
      if (u == nid || c.absorbed[u] || m.op != AC_OP_REDUCEMAX || m.inputs[0] != n.inputs[0] || !last_axis_only(m)) continue;
      plan.reduce_sibling[nid] = u;
      c.absorbed[u] = 1;
      break;
    }
  }
}

// ---- step construction ------------------------------------------------------------
struct Emit {
  Ctx& c;
  AcSession* s;
  explicit Emit(Ctx& c_) : c(c_), s(&c_.s) {}

  Step& add(const std::string& kind, int op, std::vector<int> read_vals, std::vector<int> write_vals,
            double bytes, double flops, std::function<cudaError_t(cudaStream_t)> fn, int launches = 1) {
    Step st;
    st.kind = kind;
    st.op = op;
    st.fn = std::move(fn);
    st.bytes = bytes;
    st.flops = flops;
    st.launches = launches;
    bool all_const = true;
    for (int v : read_vals) {
      if (v < 0) continue;
      st.reads.push_back(c.val(v).storage);
      all_const = all_const && c.val(v).is_const;
    }
    for (int v : write_vals) st.writes.push_back(c.val(v).storage);
    st.const_only = all_const;
    s->steps.push_back(std::move(st));
    return s->steps.back();
  }
};

void broadcast_strides(const Value& v, const Value& out, int64_t* str) {
  // crates/core/src/tensor.rs:369-406 `strides_for_broadcasting`
  int64_t st = 1;
  for (int i = 0; i < out.rank; ++i) str[i] = 0;
  for (int i = 0; i < v.rank; ++i) {
    const int vi = v.rank - 1 - i, oi = out.rank - 1 - i;
    str[oi] = (v.dims[vi] == 1 && out.dims[oi] != 1) ? 0 : (v.dims[vi] == 1 ? 0 : st);
    st *= v.dims[vi];
  }
}

BinaryParams make_binary(int op, const Value& a, const Value& b, const Value& out) {
  int64_t as[AC_MAX_RANK], bs[AC_MAX_RANK];
  broadcast_strides(a, out, as);
  broadcast_strides(b, out, bs);
  BinaryParams p{};
  p.op = op;
  p.n = out.numel();
  // Collapse: drop extent-1 dims, merge neighbours whose strides compose.
  int r = 0;
  for (int d = 0; d < out.rank; ++d) {
    const int64_t dim = out.dims[d];
    if (dim == 1) continue;
    if (r > 0 && p.a_str[r - 1] == as[d] * dim && p.b_str[r - 1] == bs[d] * dim) {
      p.dims[r - 1] *= dim;
      p.a_str[r - 1] = as[d];
      p.b_str[r - 1] = bs[d];
    } else {
      p.dims[r] = dim; p.a_str[r] = as[d]; p.b_str[r] = bs[d]; ++r;
    }
  }
  if (r == 0) { p.dims[0] = 1; p.a_str[0] = 0; p.b_str[0] = 0; r = 1; }
  p.rank = r;
  return p;
}

// Collapsed iteration space of three broadcast operands (condition, x, y) against `out`.
TernaryParams make_ternary(const Value& out, const Value& cnd, const Value& x, const Value& y) {
  int64_t cs[AC_MAX_RANK], xs[AC_MAX_RANK], ys[AC_MAX_RANK];
  broadcast_strides(cnd, out, cs);
  broadcast_strides(x, out, xs);
  broadcast_strides(y, out, ys);
  TernaryParams p{};
  p.n = out.numel();
  int r = 0;
  for (int d = 0; d < out.rank; ++d) {
    const int64_t dim = out.dims[d];
    if (dim == 1) continue;
    if (r > 0 && p.c_str[r - 1] == cs[d] * dim && p.x_str[r - 1] == xs[d] * dim && p.y_str[r - 1] == ys[d] * dim) {
      p.dims[r - 1] *= dim;
      p.c_str[r - 1] = cs[d]; p.x_str[r - 1] = xs[d]; p.y_str[r - 1] = ys[d];
    } else {
      p.dims[r] = dim; p.c_str[r] = cs[d]; p.x_str[r] = xs[d]; p.y_str[r] = ys[d]; ++r;
    }
  }
  if (r == 0) { p.dims[0] = 1; r = 1; }
  p.rank = r;
  return p;
}

void require_f32(const Value& v, const char* op) {
  if (v.elem_ty != AC_F32) fail(AC_ERR_UNSUPPORTED, std::string(op) + ": f32 tensors only");
}

void lower_binary(Emit& em, int nid, int binop) {
  Node& n = em.c.node(nid);
  const int a = n.inputs[0], b = n.inputs[1], o = n.outputs[0];
  require_f32(em.c.val(a), op_name(n.op));
  require_f32(em.c.val(b), op_name(n.op));
  const BinaryParams p = make_binary(binop, em.c.val(a), em.c.val(b), em.c.val(o));
  AcSession* s = em.s;
  const double bytes = f32_bytes(em.c.val(a)) + f32_bytes(em.c.val(b)) + f32_bytes(em.c.val(o));
  em.add("binary_" + std::string(op_name(n.op)), n.op, {a, b}, {o}, bytes, 0,
         [=](cudaStream_t st) { return launch_binary(p, s->fptr(a), s->fptr(b), s->fptr_mut(o), st); });
}

void lower_unary(Emit& em, int op, int x, int o, int un, float alpha, float beta) {
  require_f32(em.c.val(x), op_name(op));
  AcSession* s = em.s;
  const int64_t n = em.c.val(x).numel();
  static const char* names[] = {"relu", "sigmoid", "erf", "gelu", "hard_sigmoid", "leaky_relu",
                                "sqrt", "tanh", "hard_swish", "square", "copy"};
  em.add(std::string("unary_") + names[un], op, {x}, {o}, 8.0 * n, 0, [=](cudaStream_t st) {
    return launch_unary(un, alpha, beta, s->fptr(x), s->fptr_mut(o), n, st);
  });
}

struct GemmShape {
  int64_t m, n, k, batch, lda, ldb, ldc, sa, sb, sc;
  int ta, tb;
};

// Appends a scratch / derived value (not part of the caller's graph).
int new_value(Ctx& c, int64_t numel, bool is_const) {
  Value v;
  v.elem_ty = AC_F32;
  v.rank = 1;
  v.dims[0] = numel;
  v.is_const = is_const;
  v.storage = c.new_storage(v.bytes(), false, /*pinned=*/is_const);
  c.s.values.push_back(v);
  c.producer.push_back(-1);
  c.consumers.emplace_back();
  c.is_output.push_back(0);
  return (int)c.s.values.size() - 1;
}

int effective_pairs(const AcSession& s) {
  // AcOptions.gemm_pairs: 0 (default) and 2 -> CTA pairs with A pre-split for TMA where the
  // cost model prefers them, 1 -> pairs that stage A through registers, 3 -> no pairs.
  return s.opt.gemm_pairs == 0 ? 2 : (s.opt.gemm_pairs == 3 ? 0 : s.opt.gemm_pairs);
}

// The static part of emit_gemm's decision to run a GEMM with a constant rhs on the CTA-pair
// kernel that takes A pre-split (kept in one place: plan_presplit decides with it which
// producers write split results before the GEMMs themselves are lowered).
bool presplit_applies(const AcSession& s, const GemmShape& g, bool b_const, int64_t a_off, int64_t b_off) {
  const int mode = s.opt.gemm_mode;
  if (mode != 0 || effective_pairs(s) != 2 || !b_const || g.batch != 1 || g.ta || b_off != 0) return false;
  const double flops = 2.0 * g.batch * g.m * g.n * g.k;
  const double tc_floor = (g.batch == 1 && g.m <= 128 && g.k >= 64) ? double(1 << 19) : double(1 << 23);
  if ((g.lda % 4) || (a_off % 4) || flops < tc_floor || g.k < 8 || (g.k % 8)) return false;
  if (g.tb ? (g.ldb % 4) != 0 : (g.k % 4) != 0) return false;
  return gemm_tc_wants_presplit(g.m, g.n, g.k, g.batch);
}

GemmShape matmul_shape(Ctx& c, const Node& n, bool trans_b_folded) {
  const Value& av = c.val(n.inputs[0]);
  const Value& ov = c.val(n.outputs[0]);
  const Value& bv = c.val(n.inputs[1]);  // logical rhs [.., k, n]
  GemmShape g{};
  g.k = av.dims[av.rank - 1];
  g.n = ov.dims[ov.rank - 1];
  g.ta = 0;
  g.tb = trans_b_folded ? 1 : 0;
  g.lda = g.k;
  g.ldb = g.tb ? g.k : g.n;
  g.ldc = g.n;
  if (bv.rank == 2) {  // 2Dx2D and 3Dx2D: one GEMM over the flattened rows (session.rs:653-660)
    g.m = av.numel() / g.k;
    g.batch = 1;
  } else {             // 3Dx3D / 4Dx4D: a batch of GEMMs (session.rs:641-672)
    g.m = av.dims[av.rank - 2];
    g.batch = av.numel() / (g.m * g.k);
    g.sa = g.m * g.k; g.sb = g.k * g.n; g.sc = g.m * g.n;
  }
  return g;
}

// Which values will be consumed pre-split: the A operands of the MatMul nodes that
// presplit_applies to. Their scratch halves are created here.
void plan_presplit(Ctx& c, Plan& plan) {
  std::map<int, int> split_users;   // value -> MatMul nodes that take it pre-split
  for (int nid : c.s.order) {
    const Node& n = c.node(nid);
    if (c.absorbed[nid] || n.op != AC_OP_MATMUL) continue;
    const int a = n.inputs[0];
    if (c.val(a).is_const || c.val(a).elem_ty != AC_F32 || c.val(a).rank < 2) continue;
    auto it = plan.epi.find(nid);
    const bool folded_t = it != plan.epi.end() && it->second.trans_b_src >= 0;
    const int b = folded_t ? it->second.trans_b_src : n.inputs[1];
    const GemmShape g = matmul_shape(c, n, folded_t);
    if (!presplit_applies(c.s, g, c.val(b).is_const, 0, 0)) continue;
    split_users[a]++;
  }
  // The [B, T, 3D] projection in front of a fused attention core: its GEMM writes it on the fixed
  // scale and the TMA-fed attention kernel reads Q, K and V from there (the Split node between
  // them is the value's one consumer and is absorbed into the core).
  if (c.s.opt.gemm_mode == 0 && effective_pairs(c.s) == 2 && !std::getenv("ALTIUS_CUDA_NO_ATTENTION_TMA")) {
    for (auto& kv : plan.attention) {
      const AttentionFusion& f = kv.second;
      const int src = f.q.src;
      if (src != f.k.src || src != f.v.src || split_users.count(src) || c.val(src).is_const) continue;
      if (!attention_tc16_shape_ok((int)f.q.hd, (int)f.q.T, f.q.C, f.q.col, f.k.col, f.v.col, f.q.H * f.q.hd,
                                   f.q.T * f.q.H * f.q.hd))
        continue;
      split_users[src] = 1;
    }
  }
  for (auto& kv : split_users) {
    const int a = kv.first;
    const Value& av = c.val(a);
    const int64_t floats = av.numel() / 2;    // two halves per float of scratch; rows of k halves
    Ctx::Split sp;
    sp.hi = new_value(c, floats, false);
    sp.lo = new_value(c, floats, false);
    sp.fp32_needed = c.is_output[a] || (int)c.consumers[a].size() != kv.second;
    c.split[a] = sp;
  }
}

void emit_gemm(Emit& em, int op, const GemmShape& g_in, int a, int b, int out, int c_in, int bias_n,
               int bias_m, float alpha, float beta, float bias_scale, const Epilogue* e,
               int64_t a_off = 0, int64_t b_off = 0, int64_t c_off = 0, int b_row_scale = -1) {
  AcSession* s = em.s;
  GemmShape g = g_in;
  const int act = e ? e->act : ACT_NONE;
  const float aa = e ? e->act_alpha : 0.f, ab = e ? e->act_beta : 0.f;
  const int res = e ? e->residual : -1;
  double bytes = 4.0 * g.batch * (g.m * g.k + g.m * g.n) + 4.0 * (g.sb ? g.batch : 1) * g.k * g.n;
  if (res >= 0) bytes += 4.0 * g.batch * g.m * g.n;
  const double flops = 2.0 * g.batch * g.m * g.n * g.k;

  // ---- tensor-core eligibility (static part; alignment is re-checked at launch) ----
  const int mode = s->opt.gemm_mode;
  const int pairs = effective_pairs(*s);
  // Below about 8 MFLOP the CUDA-core kernel wins, except for few rows against a long K (the
  // squeeze-excite products, batch x channels): one or two of its blocks then walk K alone,
  // while the persistent kernel cuts K into slices over the idle SMs.
  const double tc_floor = (g.batch == 1 && g.m <= 128 && g.k >= 64) ? double(1 << 19) : double(1 << 23);
  bool tc = mode != 1 && !g.ta && (g.lda % 4) == 0 && (a_off % 4) == 0 && (g.sa % 4) == 0 &&
            flops >= tc_floor && g.k >= 8;
  int b_use = b, b_lo = -1;
  const bool b_const = em.c.val(b).is_const;
  if (tc) {
    if (g.tb) {
      tc = (g.ldb % 4) == 0 && (b_off % 4) == 0 && (g.sb % 4) == 0;
    } else if (b_const && g.batch == 1 && b_off == 0 && (g.k % 4) == 0) {
      // Constant rhs stored [K, N]: keep a [N, K] copy made once at load.
      const int bt = new_value(em.c, g.k * g.n, true);
      const int64_t kk = g.k, nn = g.n;
      em.add("weight_transpose", op, {b}, {bt}, 8.0 * kk * nn, 0, [=](cudaStream_t st) {
        return launch_transpose2d(s->fptr(b), s->fptr_mut(bt), 1, (int)kk, (int)nn, st);
      });
      b_use = bt;
      g.tb = 1;
      g.ldb = g.k;
    } else {
      // Activation rhs stored [K, N] (a convolution's input or column buffer, the value
      // operand of an unfused attention product): the 3xTF32 kernel reads it MN-major.
      tc = mode != 2 && (g.ldb % 4) == 0 && (b_off % 4) == 0 && (g.sb % 4) == 0;
    }
  }
  // mode 0 with a constant rhs: the fp16 split prepared once, [N, K8] halves: (hi, remainder * 2^11)
  // for the kernels with two accumulators, (hi, remainder) for the CTA-pair kernel that takes A
  // pre-split on the fixed scale and keeps one accumulator.
  int b16_hi = -1, b16_lo = -1, b16_scale = -1;
  int64_t ldb16 = 0;
  const bool b16_ok = tc && mode == 0 && em.c.val(b_use).is_const && g.tb && g.batch == 1 && b_off == 0;
  const bool pre = b16_ok && presplit_applies(*s, g, true, a_off, b_off);
  if (b16_ok) {
    ldb16 = (g.k + 7) / 8 * 8;
    const int64_t floats = g.n * ldb16 / 2;     // two halves per float of scratch
    b16_hi = new_value(em.c, floats, true);
    b16_lo = new_value(em.c, floats, true);
    // The weight is split after scaling by a power of two that brings its largest magnitude to
    // about 2^13 (weights of any magnitude then stay clear of the fp16 subnormals); the
    // epilogue multiplies by the inverse, kept in word 0 of this scratch (word 1: the maximum).
    b16_scale = new_value(em.c, 2, true);
    const int src = b_use, hi = b16_hi, lo = b16_lo, scv = b16_scale;
    const int64_t nn = g.n, kk = g.k, ld = g.ldb, k8 = ldb16;
    em.add("weight_f16_split", op, {src}, {hi, lo, scv}, 4.0 * nn * kk + 4.0 * nn * k8, 0, [=](cudaStream_t st) {
      return launch_f16_split(s->fptr(src), s->fptr_mut(hi), s->fptr_mut(lo), nn, kk, ld, k8, s->err_word,
                              s->fptr_mut(scv), reinterpret_cast<unsigned*>(s->fptr_mut(scv)) + 1, pre ? 1 : 0, st);
    }, 3);
  }
  const int b_plain = b_use;   // the operand before any TF32 rounding
  if (tc && b16_hi < 0 && mode != 2 && g.tb && em.c.val(b_use).is_const) {
    // TF32 hi / lo split of a constant rhs, prepared once.
    const int64_t cnt = em.c.val(b_use).numel();
    const int hi = new_value(em.c, cnt, true);
    b_lo = new_value(em.c, cnt, true);
    const int src = b_use, lo = b_lo;
    em.add("weight_tf32_split", op, {src}, {hi, lo}, 12.0 * cnt, 0, [=](cudaStream_t st) {
      return launch_tf32_split(s->fptr(src), s->fptr_mut(hi), s->fptr_mut(lo), cnt, st);
    });
    b_use = hi;
  }
  const int bsrc = b_use;
  // CTA pairs that take A by TMA want it already split into fp16 hi / lo halves (rows of K
  // halves): written by the kernel that produced A when plan_presplit arranged that, else by a
  // split kernel in front of the GEMM.
  int a16_hi = -1, a16_lo = -1;
  int64_t lda16 = 0;
  bool a_fp32_present = true;
  if (pre) {
    lda16 = g.k;
    auto sp = em.c.split.find(a);
    const bool planned = sp != em.c.split.end() && a_off == 0 && g.lda == g.k;
    if (planned) {
      a16_hi = sp->second.hi; a16_lo = sp->second.lo;
      a_fp32_present = sp->second.fp32_needed || !sp->second.produced;
    } else {
      const int64_t floats = g.m * lda16 / 2;
      a16_hi = new_value(em.c, floats, false);
      a16_lo = new_value(em.c, floats, false);
    }
    if (!planned || !sp->second.produced) {
      const int hi = a16_hi, lo = a16_lo;
      const int64_t mm = g.m, kk = g.k, ld = g.lda, off = a_off;
      em.add("act_f16_split", op, {a}, {hi, lo}, 8.0 * mm * kk, 0, [=](cudaStream_t st) {
        return launch_f16_split(s->fptr(a) + off, s->fptr_mut(hi), s->fptr_mut(lo), mm, kk, ld, kk, s->err_word,
                                nullptr, nullptr, 1, st);
      });
      if (planned) sp->second.produced = true;
    }
  }
  if (a16_hi < 0) {
    auto sp = em.c.split.find(a);
    if (sp != em.c.split.end() && sp->second.produced && !sp->second.fp32_needed)
      fail(AC_ERR_INVALID, "internal: a GEMM operand was planned pre-split but its GEMM does not take it so");
  }
  // This GEMM's own result, when a later GEMM takes it pre-split and this one runs on the pair
  // kernel with an epilogue that can write the halves.
  int c16_hi = -1, c16_lo = -1;
  bool c_fp32 = true, c16_fixed = false;
  {
    auto so = em.c.split.find(out);
    if (so != em.c.split.end() && !so->second.produced && a16_hi >= 0 && c_off == 0 && g.ldc == g.n && (g.n % 8) == 0 &&
        gemm_tc_can_split_output(act, bias_n >= 0, bias_m >= 0, c_in >= 0, alpha, bias_scale)) {
      c16_hi = so->second.hi; c16_lo = so->second.lo;
      c_fp32 = so->second.fp32_needed;
      c16_fixed = true;
      so->second.produced = true;
    }
  }
  // Scratch for the K-sliced tail tiles of the persistent kernel (lives for this step only).
  int ws = -1;
  size_t ws_bytes = 0;
  if (tc) {
    ws_bytes = gemm_tc_workspace_bytes(g.m, g.n, g.k, g.batch, b16_hi >= 0 ? 2 : (b_lo >= 0 ? 0 : 1), pairs);
    if (ws_bytes) ws = new_value(em.c, (int64_t)(ws_bytes / 4), false);
  }
  if (b_row_scale >= 0 && (!tc || g.tb || b16_hi >= 0 || b_lo >= 0))
    fail(AC_ERR_INVALID, "internal: a row scale was planned for a GEMM that does not read its rhs as [K, N] tiles");
  std::vector<int> reads = {a_fp32_present ? a : -1, bsrc, b_plain, b_lo, b16_hi, b16_lo, b16_scale, a16_hi, a16_lo,
                            c_in, bias_n, bias_m, res, b_row_scale};
  const char* kind = !tc ? "gemm_fp32_simt"
                     : (mode == 2 ? "gemm_tf32x1_tcgen05"
                                  : (b16_hi >= 0 ? (a16_hi >= 0 ? "gemm_f16x3_pair_tcgen05" : "gemm_f16x3_tcgen05")
                                                 : "gemm_tf32x3_tcgen05"));
  std::vector<int> writes;
  if (c_fp32) writes.push_back(out);
  if (c16_hi >= 0) { writes.push_back(c16_hi); writes.push_back(c16_lo); }
  if (ws >= 0) writes.push_back(ws);
  em.add(kind, op, reads, writes, bytes, flops, [=](cudaStream_t st) {
    GemmParams p{};
    p.workspace = ws >= 0 ? s->fptr_mut(ws) : nullptr;
    p.workspace_bytes = ws_bytes;
    p.allow_pairs = pairs;
    p.a16_hi = a16_hi >= 0 ? s->ptr(a16_hi) : nullptr;
    p.a16_lo = a16_lo >= 0 ? s->ptr(a16_lo) : nullptr;
    p.lda16 = lda16;
    p.a16_fixed = a16_hi >= 0 ? 1 : 0;
    p.b16_plain = pre ? 1 : 0;
    p.m = g.m; p.n = g.n; p.k = g.k; p.batch = g.batch;
    p.a = a_fp32_present ? s->fptr(a) + a_off : nullptr; p.lda = g.lda; p.stride_a = g.sa; p.trans_a = g.ta;
    p.b = s->fptr(bsrc) + b_off; p.ldb = g.ldb; p.stride_b = g.sb; p.trans_b = g.tb;
    p.b_lo = b_lo >= 0 ? s->fptr(b_lo) + b_off : nullptr;
    p.b16_hi = b16_hi >= 0 ? s->ptr(b16_hi) : nullptr;
    p.b16_lo = b16_lo >= 0 ? s->ptr(b16_lo) : nullptr;
    p.ldb16 = ldb16;
    p.c = c_fp32 ? s->fptr_mut(out) + c_off : nullptr; p.ldc = g.ldc; p.stride_c = g.sc;
    p.c16_hi = c16_hi >= 0 ? s->ptr(c16_hi) : nullptr;
    p.c16_lo = c16_lo >= 0 ? s->ptr(c16_lo) : nullptr;
    p.ldc16 = g.n;
    p.c16_fixed = c16_fixed ? 1 : 0;
    p.b16_inv_scale = b16_scale >= 0 ? s->fptr(b16_scale) : nullptr;
    p.b_row_scale = b_row_scale >= 0 ? s->fptr(b_row_scale) : nullptr;
    p.b_row_scale_stride = g.k;
    p.alpha = alpha; p.beta = c_in >= 0 ? beta : 0.f;
    p.c_in = c_in >= 0 ? s->fptr(c_in) + c_off : nullptr; p.ldc_in = g.ldc; p.stride_c_in = g.sc;
    p.bias_n = bias_n >= 0 ? s->fptr(bias_n) : nullptr;
    p.bias_m = bias_m >= 0 ? s->fptr(bias_m) : nullptr;
    p.bias_scale = bias_scale;
    p.act = act; p.act_alpha = aa; p.act_beta = ab;
    p.residual = res >= 0 ? s->fptr(res) + c_off : nullptr; p.ld_res = g.ldc; p.stride_res = g.sc;
    if (tc && gemm_tc_supported(p)) return launch_gemm_tc(p, mode, s->err_word, st);
    if (!p.a || !p.c || p.c16_hi || p.b_row_scale) return cudaErrorInvalidValue;   // operands exist for the tensor-core kernel only
    // The CUDA-core kernel multiplies the operand as given, not a TF32-rounded copy of it.
    if (b_lo >= 0) { p.b = s->fptr(b_plain) + b_off; p.b_lo = nullptr; }
    return launch_gemm_simt(p, st);
  }, ws >= 0 ? 2 : 1);
}

void lower_matmul(Emit& em, int nid, const Epilogue* e) {
  Node& n = em.c.node(nid);
  const int a = n.inputs[0];
  const int b = (e && e->trans_b_src >= 0) ? e->trans_b_src : n.inputs[1];
  const int out = e ? e->out : n.outputs[0];
  const Value& av = em.c.val(a);
  const Value& ov = em.c.val(n.outputs[0]);
  const Value& bv = em.c.val(n.inputs[1]);  // logical rhs [.., k, n]
  require_f32(av, "MatMul");
  (void)ov; (void)bv;
  const GemmShape g = matmul_shape(em.c, n, e && e->trans_b_src >= 0);
  emit_gemm(em, n.op, g, a, b, out, -1, e ? e->bias : -1, -1, 1.f, 0.f, 1.f, e);
}

void lower_gemm(Emit& em, int nid, const Epilogue* e) {
  // compute_gemm, session.rs:684-734: C pre-filled with the bias ([N] tiled or
  // [M,N]), then C = alpha * op(A) op(B) + beta * C.
  Node& n = em.c.node(nid);
  const int a = n.inputs[0], b = n.inputs[1];
  const int cin = n.inputs.size() > 2 ? n.inputs[2] : -1;
  const int out = e ? e->out : n.outputs[0];
  const Value& av = em.c.val(a);
  const Value& bv = em.c.val(b);
  require_f32(av, "Gemm");
  GemmShape g{};
  g.ta = n.ints[0] != 0; g.tb = n.ints[1] != 0;
  g.m = g.ta ? av.dims[1] : av.dims[0];
  g.k = g.ta ? av.dims[0] : av.dims[1];
  g.n = g.tb ? bv.dims[0] : bv.dims[1];
  g.lda = av.dims[1]; g.ldb = bv.dims[1]; g.ldc = g.n; g.batch = 1;
  const float alpha = n.floats.size() > 0 ? n.floats[0] : 1.f;
  const float beta = n.floats.size() > 1 ? n.floats[1] : 1.f;
  int bias_n = -1, c_in = -1;
  if (cin >= 0) {
    const Value& cv = em.c.val(cin);
    if (cv.rank == 1 && cv.dims[0] == g.n) bias_n = cin;
    else if (cv.rank == 2 && cv.dims[0] == g.m && cv.dims[1] == g.n) c_in = cin;
    else fail(AC_ERR_UNSUPPORTED, "Gemm: C must be [N] or [M,N]");
  }
  emit_gemm(em, n.op, g, a, b, out, c_in, bias_n, -1, alpha, beta, beta, e);
}

void lower_conv(Emit& em, int nid, const Epilogue* e, const Plan::SeGate* gate = nullptr) {
  Node& n = em.c.node(nid);
  AcSession* s = em.s;
  // With a folded squeeze-excite gate the convolution reads the un-gated planes.
  const int x = gate ? gate->x : n.inputs[0], w = n.inputs[1];
  int bias = n.inputs.size() > 2 ? n.inputs[2] : -1;
  if (e && e->bias >= 0) bias = e->bias;
  const int out = e ? e->out : n.outputs[0];
  const Value& xv = em.c.val(x);
  const Value& wv = em.c.val(w);
  const Value& ov = em.c.val(n.outputs[0]);
  require_f32(xv, "Conv2d");
  int64_t pads[4];
  resolve_pads(n, 7, xv.dims[2], xv.dims[3], pads);
  ConvParams p{};
  p.n = (int)xv.dims[0]; p.c = (int)xv.dims[1]; p.ih = (int)xv.dims[2]; p.iw = (int)xv.dims[3];
  p.oc = (int)ov.dims[1]; p.oh = (int)ov.dims[2]; p.ow = (int)ov.dims[3];
  p.kh = (int)n.ints[0]; p.kw = (int)n.ints[1]; p.sh = (int)n.ints[2]; p.sw = (int)n.ints[3];
  p.dh = (int)n.ints[4]; p.dw = (int)n.ints[5]; p.group = (int)n.ints[6];
  p.pad_t = (int)pads[0]; p.pad_l = (int)pads[1];
  // Conv2d.activation (crates/core/src/op.rs:68-75): applied when present, as
  // the clang backend does; merged with a folded consumer activation.
  Epilogue ep = e ? *e : Epilogue{};
  if (n.ints[8] != 0 && ep.act == ACT_NONE) {
    ep.act = n.ints[8] == 1 ? ACT_RELU : ACT_HARDSIGMOID;
    ep.act_alpha = n.floats.size() > 0 ? n.floats[0] : 0.2f;
    ep.act_beta = n.floats.size() > 1 ? n.floats[1] : 0.5f;
  } else if (n.ints[8] != 0) {
    fail(AC_ERR_UNSUPPORTED, "Conv2d: fused activation followed by another activation");
  }
  p.act = ep.act; p.act_alpha = ep.act_alpha; p.act_beta = ep.act_beta;
  if (p.group <= 0 || p.c % p.group || p.oc % p.group || wv.dims[1] != p.c / p.group)
    fail(AC_ERR_SHAPE, "Conv2d: group does not divide the channels");

  // Patch embedding: Conv2d with kernel == stride and no padding, followed by
  // Reshape [N, OC, P] -> Transpose [0, 2, 1]. One GEMM over patch rows writes the
  // [N, P, OC] token tensor directly (bias along N), no NCHW intermediate.
  if (!s->opt.disable_fusion && p.group == 1 && p.kh == p.sh && p.kw == p.sw && p.dh == 1 && p.dw == 1 &&
      pads[0] == 0 && pads[1] == 0 && pads[2] == 0 && pads[3] == 0 && p.ih == p.oh * p.kh &&
      p.iw == p.ow * p.kw && (p.kw % 4) == 0 && (p.iw % 4) == 0 && ep.act == ACT_NONE && ep.residual < 0 &&
      out == n.outputs[0] && em.c.single_use(out)) {
    const int rn = em.c.only_consumer(out);
    if (em.c.node(rn).op == AC_OP_RESHAPE) {
      const int rv = em.c.node(rn).outputs[0];
      const Value& rvv = em.c.val(rv);
      if (rvv.rank == 3 && rvv.dims[0] == p.n && rvv.dims[1] == p.oc && em.c.single_use(rv)) {
        const int tn = em.c.only_consumer(rv);
        const Node& tnode = em.c.node(tn);
        if (tnode.op == AC_OP_TRANSPOSE && tnode.ints.size() == 3 && tnode.ints[0] == 0 &&
            tnode.ints[1] == 2 && tnode.ints[2] == 1 && !em.c.absorbed[tn]) {
          const int tokens = tnode.outputs[0];
          em.c.absorbed[tn] = 1;
          const int64_t rows = (int64_t)p.n * p.oh * p.ow, kd = (int64_t)p.c * p.kh * p.kw;
          const int colv = new_value(em.c, rows * kd, false);
          em.add("patchify", n.op, {x}, {colv}, 2.0 * f32_bytes(xv), 0, [=](cudaStream_t st) {
            return launch_patchify(p, s->fptr(x), s->fptr_mut(colv), st);
          });
          GemmShape g{};
          g.m = rows; g.k = kd; g.n = p.oc; g.batch = 1;
          g.lda = kd; g.ldb = kd; g.ldc = p.oc; g.ta = 0; g.tb = 1;   // W is [OC, K]: already K-major
          emit_gemm(em, n.op, g, colv, w, tokens, -1, bias, -1, 1.f, 0.f, 1.f, nullptr);
          return;
        }
      }
    }
  }
  const int icg = p.c / p.group, ocg = p.oc / p.group;
  const int64_t ohw = (int64_t)p.oh * p.ow;
  const int64_t kdim = (int64_t)icg * p.kh * p.kw;
  const double flops = 2.0 * p.n * p.oc * ohw * kdim;

  if (p.group == p.c && icg == 1 && ocg == 1 && ep.residual < 0) {  // depthwise stencil
    const double bytes = f32_bytes(xv) + f32_bytes(wv) + f32_bytes(ov);
    em.add("conv_depthwise", n.op, {x, w, bias}, {out}, bytes, flops, [=](cudaStream_t st) {
      return launch_depthwise_conv(p, s->fptr(x), s->fptr(w), bias >= 0 ? s->fptr(bias) : nullptr,
                                   s->fptr_mut(out), st);
    });
    return;
  }
  // GEMM form: out[n] (ocg x ohw) = W_g (ocg x k) * col[n, g] (k x ohw), bias per row.
  const bool pointwise = p.kh == 1 && p.kw == 1 && p.sh == 1 && p.sw == 1 && p.pad_t == 0 &&
                         p.pad_l == 0 && pads[2] == 0 && pads[3] == 0;
  int bsrc = x;
  if (!pointwise) {
    // Scratch column buffer col[n, c, kh, kw, oh, ow] (conv2d.rs:81-143).
    Value colv;
    colv.elem_ty = AC_F32;
    colv.rank = 1;
    colv.dims[0] = (int64_t)p.n * p.c * p.kh * p.kw * ohw;
    colv.is_const = false;
    colv.storage = em.c.new_storage(colv.bytes());
    s->values.push_back(colv);
    const int col = (int)s->values.size() - 1;
    em.c.producer.push_back(-1);
    em.c.consumers.emplace_back();
    em.c.is_output.push_back(0);
    em.add("im2col", n.op, {x}, {col}, f32_bytes(xv) + (double)colv.bytes(), 0,
           [=](cudaStream_t st) { return launch_im2col(p, s->fptr(x), s->fptr_mut(col), st); });
    bsrc = col;
  }
  // A pointwise convolution of 1 x 1 planes (squeeze-and-excite) is one product over the whole
  // batch: out [n, oc] = x [n, c] * W^T, bias along the columns. As a batch of n matrix-vector
  // products it would leave every tile of either GEMM kernel almost empty.
  if (pointwise && p.group == 1 && ohw == 1 && ep.residual < 0) {
    GemmShape g{};
    g.m = p.n; g.k = p.c; g.n = p.oc; g.batch = 1;
    g.lda = p.c; g.ldb = p.c; g.ldc = p.oc;
    g.ta = 0; g.tb = 1;                       // W is [oc, c]: already K-major
    Epilogue eg = ep;
    emit_gemm(em, n.op, g, x, w, out, -1, bias, -1, 1.f, 0.f, 1.f, &eg);
    return;
  }
  // The tensor-core kernel reads the input planes as they are ([K, N] operand, MN-major tiles)
  // when the plane size is a multiple of four floats. Otherwise (7 x 7) the row stride is not a
  // multiple of 16 bytes and TMA cannot address the planes: pointwise convolutions of some size
  // then transpose them once to [n, hw, c], a K-contiguous rhs with row stride c.
  bool rhs_transposed = false;
  if (pointwise && p.group == 1 && (ohw % 4) != 0 && (p.c % 4) == 0 && flops >= double(1 << 23) &&
      s->opt.gemm_mode != 1 && s->opt.gemm_mode != 2 && p.n <= 65535) {
    const int xt = new_value(em.c, (int64_t)p.n * ohw * p.c, false);
    const int64_t nb = p.n;
    const int rows = p.c, cols = (int)ohw;
    em.add("transpose_copy", n.op, {x}, {xt}, 2.0 * f32_bytes(xv), 0, [=](cudaStream_t st) {
      return launch_transpose2d(s->fptr(x), s->fptr_mut(xt), nb, rows, cols, st);
    });
    bsrc = xt;
    rhs_transposed = true;
  }
  // A filter matrix whose row length is not a multiple of four floats (3 x 3 x 3 = 27 in the
  // first layer of the CNNs) gets a copy with padded rows, so that TMA can address it; K stays
  // what it is, the tensor-core kernel zero-fills past it.
  int a_src = w;
  int64_t lda_use = kdim;
  if (p.group == 1 && (kdim % 4) != 0 && !rhs_transposed && (ohw % 4) == 0 && flops >= double(1 << 23) &&
      s->opt.gemm_mode != 1 && s->opt.gemm_mode != 2) {
    const int64_t kpad = (kdim + 3) / 4 * 4, rows = p.oc, kd = kdim;
    const int wp = new_value(em.c, rows * kpad, em.c.val(w).is_const);
    em.add("weight_pad", n.op, {w}, {wp}, 4.0 * rows * (kd + kpad), 0, [=](cudaStream_t st) {
      cudaError_t e = cudaMemsetAsync(s->fptr_mut(wp), 0, (size_t)(rows * kpad) * sizeof(float), st);
      if (e != cudaSuccess) return e;
      return cudaMemcpy2DAsync(s->fptr_mut(wp), (size_t)kpad * sizeof(float), s->fptr(w), (size_t)kd * sizeof(float),
                               (size_t)kd * sizeof(float), (size_t)rows, cudaMemcpyDeviceToDevice, st);
    }, 2);
    a_src = wp;
    lda_use = kpad;
  }
  for (int gi = 0; gi < p.group; ++gi) {
    GemmShape g{};
    g.m = ocg; g.k = kdim; g.n = ohw; g.batch = p.n;
    g.lda = lda_use; g.ldb = ohw; g.ldc = ohw;
    g.sa = 0; g.sb = (int64_t)p.c * p.kh * p.kw * ohw; g.sc = (int64_t)p.oc * ohw;
    g.ta = 0; g.tb = 0;
    if (rhs_transposed) { g.tb = 1; g.ldb = kdim; }
    Epilogue eg = ep;
    // bias_m needs the group's slice of the bias: pass through an offset closure below.
    const int64_t a_off = (int64_t)gi * ocg * kdim, b_off = (int64_t)gi * kdim * ohw,
                  c_off = (int64_t)gi * ocg * ohw;
    if (p.group == 1) {
      if (gate && (bsrc != x || rhs_transposed))
        fail(AC_ERR_INVALID, "internal: a squeeze-excite gate was folded into a convolution that does not read its planes in place");
      emit_gemm(em, n.op, g, a_src, bsrc, out, -1, -1, bias, 1.f, 0.f, 1.f, &eg, a_off, b_off, c_off,
                gate ? gate->gate : -1);
    } else {
      if (bias >= 0 || eg.residual >= 0)
        fail(AC_ERR_UNSUPPORTED, "Conv2d: grouped (non-depthwise) convolution with bias");
      emit_gemm(em, n.op, g, w, bsrc, out, -1, -1, -1, 1.f, 0.f, 1.f, &eg, a_off, b_off, c_off);
    }
  }
}

void lower_copy(Emit& em, const std::string& kind, int op, int in, int out, const CopyParams& p) {
  AcSession* s = em.s;
  const double bytes = 2.0 * p.n * p.elem_bytes;
  em.add(kind, op, {in}, {out}, bytes, 0,
         [=](cudaStream_t st) { return launch_strided_copy(p, s->ptr(in), s->ptr(out), st); });
}

void contiguous_strides(const int64_t* dims, int rank, int64_t* str) {
  int64_t st = 1;
  for (int i = rank - 1; i >= 0; --i) { str[i] = st; st *= dims[i]; }
}

void lower_node(Emit& em, Plan& plan, int nid) {
  Ctx& c = em.c;
  AcSession* s = em.s;
  Node& n = c.node(nid);
  auto V = [&](int v) -> Value& { return c.val(v); };
  switch (n.op) {
    case AC_OP_IDENTITY: case AC_OP_RESHAPE: case AC_OP_FLATTEN: case AC_OP_SQUEEZE:
    case AC_OP_UNSQUEEZE:
      return;  // storage alias, no kernel
    case AC_OP_SHAPE:
      return;  // evaluated on the host during shape inference
    case AC_OP_ADD: return lower_binary(em, nid, BIN_ADD);
    case AC_OP_SUB: return lower_binary(em, nid, BIN_SUB);
    case AC_OP_DIV: return lower_binary(em, nid, BIN_DIV);
    case AC_OP_MUL: {
      auto it = plan.hardswish.find(nid);
      if (it != plan.hardswish.end()) {
        Node& hs = c.node(it->second);
        return lower_unary(em, n.op, hs.inputs[0], n.outputs[0], UN_HARDSWISH,
                           hs.floats.size() > 0 ? hs.floats[0] : 0.2f,
                           hs.floats.size() > 1 ? hs.floats[1] : 0.5f);
      }
      return lower_binary(em, nid, BIN_MUL);
    }
    case AC_OP_POW: {
      // compute_pow, session.rs:566-606: same shape, or a scalar exponent with
      // the b == 2 -> a * a special case.
      const Value& a = V(n.inputs[0]);
      const Value& b = V(n.inputs[1]);
      if (same_dims(a, b)) return lower_binary(em, nid, BIN_POW);
      if (b.numel() == 1 && b.rank <= 1) {
        if (b.host && *static_cast<const float*>(b.host) == 2.f)
          return lower_unary(em, n.op, n.inputs[0], n.outputs[0], UN_SQUARE, 0, 0);
        return lower_binary(em, nid, BIN_POW);
      }
      fail(AC_ERR_UNSUPPORTED, "Pow: only same-shape operands or a scalar exponent");
    }
    case AC_OP_SQRT: return lower_unary(em, n.op, n.inputs[0], n.outputs[0], UN_SQRT, 0, 0);
    case AC_OP_RELU: return lower_unary(em, n.op, n.inputs[0], n.outputs[0], UN_RELU, 0, 0);
    case AC_OP_GELU: return lower_unary(em, n.op, n.inputs[0], n.outputs[0], UN_GELU, 0, 0);
    case AC_OP_SIGMOID: return lower_unary(em, n.op, n.inputs[0], n.outputs[0], UN_SIGMOID, 0, 0);
    case AC_OP_ERF: return lower_unary(em, n.op, n.inputs[0], n.outputs[0], UN_ERF, 0, 0);
    case AC_OP_TANH: return lower_unary(em, n.op, n.inputs[0], n.outputs[0], UN_TANH, 0, 0);
    case AC_OP_LEAKYRELU:
      return lower_unary(em, n.op, n.inputs[0], n.outputs[0], UN_LEAKYRELU,
                         n.floats.size() > 0 ? n.floats[0] : 0.01f, 0);
    case AC_OP_HARDSIGMOID:
      return lower_unary(em, n.op, n.inputs[0], n.outputs[0], UN_HARDSIGMOID,
                         n.floats.size() > 0 ? n.floats[0] : 0.2f,
                         n.floats.size() > 1 ? n.floats[1] : 0.5f);
    case AC_OP_GREATER: {
      const int x = n.inputs[0], y = n.inputs[1], o = n.outputs[0];
      if (!(V(y).numel() == 1 && V(y).rank <= 1)) {
        // The reference stops here (session.rs:559); the general form broadcasts as ONNX defines.
        require_f32(V(x), "Greater");
        require_f32(V(y), "Greater");
        const TernaryParams tp = make_ternary(V(o), V(o), V(x), V(y));
        em.add("greater_bcast", n.op, {x, y}, {o}, f32_bytes(V(x)) + f32_bytes(V(y)) + (double)V(o).bytes(), 0,
               [=](cudaStream_t st) {
                 return launch_greater_bcast(tp, s->fptr(x), s->fptr(y), static_cast<uint8_t*>(s->ptr(o)), st);
               });
        return;
      }
      const int64_t cnt = V(x).numel();
      em.add("greater", n.op, {x, y}, {o}, 5.0 * cnt, 0, [=](cudaStream_t st) {
        return launch_greater_scalar(s->fptr(x), s->fptr(y), static_cast<uint8_t*>(s->ptr(o)), cnt, st);
      });
      return;
    }
    case AC_OP_WHERE: {
      const int cd = n.inputs[0], x = n.inputs[1], y = n.inputs[2], o = n.outputs[0];
      const Value& cv = V(cd);
      const Value& ov = V(o);
      int mode;
      int64_t inner = 1;
      if (same_dims(cv, V(y)) && V(x).numel() == 1 && V(x).rank <= 1) mode = 0;   // session.rs:947
      else if (V(y).numel() == 1 && V(y).rank <= 1 && V(x).rank == 4 && cv.rank == 4 &&
               cv.dims[0] == 1 && cv.dims[1] == 1 && cv.dims[2] == ov.dims[2] &&
               cv.dims[3] == ov.dims[3]) {                                          // session.rs:958-964
        mode = 1;
        inner = ov.dims[2] * ov.dims[3];
      } else {
        // Beyond the reference's two patterns: condition, x and y broadcast as ONNX defines.
        if (cv.elem_ty != AC_BOOL) fail(AC_ERR_UNSUPPORTED, "Where: the condition must be a bool tensor");
        require_f32(V(x), "Where");
        require_f32(V(y), "Where");
        const TernaryParams tp = make_ternary(ov, cv, V(x), V(y));
        em.add("where_bcast", n.op, {cd, x, y}, {o}, (double)cv.bytes() + f32_bytes(V(x)) + f32_bytes(V(y)) + f32_bytes(ov), 0,
               [=](cudaStream_t st) {
                 return launch_where_bcast(tp, static_cast<const uint8_t*>(s->ptr(cd)), s->fptr(x), s->fptr(y),
                                           s->fptr_mut(o), st);
               });
        return;
      }
      const int64_t cnt = ov.numel();
      em.add("where", n.op, {cd, x, y}, {o}, 9.0 * cnt, 0, [=](cudaStream_t st) {
        return launch_where(mode, static_cast<const uint8_t*>(s->ptr(cd)), s->fptr(x), s->fptr(y),
                            s->fptr_mut(o), cnt, inner, st);
      });
      return;
    }
    case AC_OP_EXPAND: {
      // compute_expand, session.rs:299-323, tiles an i64 [1,1,1,k] row; here any tensor
      // is broadcast to the requested shape (stride 0 along the expanded dims).
      const int x = n.inputs[0], o = n.outputs[0];
      const Value& xv = V(x);
      const Value& ov = V(o);
      if (xv.rank > ov.rank) fail(AC_ERR_SHAPE, "Expand: input rank above the requested shape's");
      CopyParams p{};
      p.rank = ov.rank;
      int64_t in_str[AC_MAX_RANK];
      contiguous_strides(xv.dims, xv.rank, in_str);
      for (int i = 0; i < ov.rank; ++i) {
        const int xi = i - (ov.rank - xv.rank);
        p.dims[i] = ov.dims[i];
        if (xi < 0 || xv.dims[xi] == 1) p.in_str[i] = 0;
        else if (xv.dims[xi] == ov.dims[i]) p.in_str[i] = in_str[xi];
        else fail(AC_ERR_SHAPE, "Expand: shapes cannot be broadcast");
      }
      contiguous_strides(p.dims, p.rank, p.out_str);
      p.n = ov.numel();
      p.elem_bytes = (int)xv.elem_bytes();
      lower_copy(em, "expand_copy", n.op, x, o, p);
      return;
    }
    case AC_OP_RESIZE: {
      const int x = n.inputs[0], o = n.outputs[0];
      const Value& xv = V(x);
      const Value& ov = V(o);
      require_f32(xv, "Resize");
      if (ov.dims[0] != xv.dims[0] || ov.dims[1] != xv.dims[1])
        fail(AC_ERR_UNSUPPORTED, "Resize: batch and channel extents must not change");
      const int64_t planes = xv.dims[0] * xv.dims[1];
      const int ih = (int)xv.dims[2], iw = (int)xv.dims[3], oh = (int)ov.dims[2], ow = (int)ov.dims[3];
      const int mode = (int)n.ints[0];
      em.add(mode == 0 ? "resize_nearest" : "resize_bilinear", n.op, {x}, {o}, (double)xv.bytes() + ov.bytes(), 0,
             [=](cudaStream_t st) {
               return launch_resize(s->fptr(x), s->fptr_mut(o), planes, ih, iw, oh, ow, mode, st);
             });
      return;
    }
    case AC_OP_CAST: {
      const int x = n.inputs[0], o = n.outputs[0];
      const int from = V(x).elem_ty, to = (int)n.ints[0];
      // session.rs:1350-1378 has i32->f32, i64->i32, i64->f32 and f32->bool; every other pair of
      // the four element types is converted as C does.
      if (from < AC_BOOL || from > AC_I64 || to < AC_BOOL || to > AC_I64) fail(AC_ERR_UNSUPPORTED, "Cast: unsupported type pair");
      const int64_t cnt = V(x).numel();
      em.add("cast", n.op, {x}, {o}, (double)V(x).bytes() + V(o).bytes(), 0, [=](cudaStream_t st) {
        return launch_cast(from, to, s->ptr(x), s->ptr(o), cnt, st);
      });
      return;
    }
    case AC_OP_BATCHNORMALIZATION: {
      const Value& xv = V(n.inputs[0]);
      if (xv.rank != 4) fail(AC_ERR_UNSUPPORTED, "Input data rank must be 4.");
      const int x = n.inputs[0], sc = n.inputs[1], b = n.inputs[2], mu = n.inputs[3], var = n.inputs[4],
                o = n.outputs[0];
      const float eps = n.floats.size() > 0 ? n.floats[0] : 1e-5f;
      const int64_t nb = xv.dims[0], ch = xv.dims[1], hw = xv.dims[2] * xv.dims[3];
      em.add("batch_norm", n.op, {x, sc, b, mu, var}, {o}, 8.0 * xv.numel(), 0, [=](cudaStream_t st) {
        return launch_batch_norm(s->fptr(x), s->fptr(sc), s->fptr(b), s->fptr(mu), s->fptr(var),
                                 s->fptr_mut(o), nb, ch, hw, eps, st);
      });
      return;
    }
    case AC_OP_SOFTMAX: {
      auto at = plan.attention.find(nid);
      if (at != plan.attention.end()) {
        const AttentionFusion f = at->second;
        const int64_t B = f.q.B, H = f.q.H, T = f.q.T, hd = f.q.hd, C = f.q.C;
        const double bytes = 4.0 * B * T * hd * H * 4;
        const double flops = 4.0 * B * H * T * T * hd;
        // gemm_mode 1 asks for exact fp32 FMA chains: it keeps the CUDA-core kernel.
        const bool tc_attn = s->opt.gemm_mode != 1 && hd == 64 && T > 64 && T <= 256;
        int o16_hi = -1, o16_lo = -1;
        bool o_fp32 = true;
        {
          auto so = c.split.find(f.out);
          if (so != c.split.end() && !so->second.produced && tc_attn) {
            o16_hi = so->second.hi; o16_lo = so->second.lo;
            o_fp32 = so->second.fp32_needed;
            so->second.produced = true;
          }
        }
        std::vector<int> awrites;
        if (o_fp32) awrites.push_back(f.out);
        if (o16_hi >= 0) { awrites.push_back(o16_hi); awrites.push_back(o16_lo); }
        // The projection was written on the fixed scale by its GEMM: the TMA-fed kernel.
        auto si = c.split.find(f.q.src);
        if (tc_attn && si != c.split.end() && si->second.produced && f.q.src == f.k.src && f.q.src == f.v.src &&
            attention_tc16_shape_ok((int)hd, (int)T, C, f.q.col, f.k.col, f.v.col, H * hd, T * H * hd)) {
          const int in_hi = si->second.hi, in_lo = si->second.lo;
          em.add("attention_tma_tcgen05", n.op, {in_hi, in_lo, f.scale}, awrites, bytes, flops, [=](cudaStream_t st) {
            Attention16Params p{};
            p.qkv16_hi = s->ptr(in_hi); p.qkv16_lo = s->ptr(in_lo);
            p.ld16 = C; p.q_col = f.q.col; p.k_col = f.k.col; p.v_col = f.v.col;
            p.out = o_fp32 ? s->fptr_mut(f.out) : nullptr; p.out_row_stride = H * hd; p.out_batch_stride = T * H * hd;
            p.out16_hi = o16_hi >= 0 ? s->ptr(o16_hi) : nullptr;
            p.out16_lo = o16_lo >= 0 ? s->ptr(o16_lo) : nullptr;
            p.batch = (int)B; p.heads = (int)H; p.tokens = (int)T; p.head_dim = (int)hd;
            p.scale = f.scale >= 0 ? s->fptr(f.scale) : nullptr; p.scale_mode = f.scale_mode;
            p.err_word = s->err_word;
            return launch_attention_tc16(p, st);
          });
          return;
        }
        em.add(tc_attn ? "attention_tcgen05" : "attention_fused", n.op, {f.q.src, f.k.src, f.v.src, f.scale}, awrites, bytes, flops,
               [=](cudaStream_t st) {
                 AttentionParams p{};
                 p.q = s->fptr(f.q.src) + f.q.col;
                 p.k = s->fptr(f.k.src) + f.k.col;
                 p.v = s->fptr(f.v.src) + f.v.col;
                 p.row_stride = C; p.batch_stride = T * C;
                 p.out = o_fp32 ? s->fptr_mut(f.out) : nullptr; p.out_row_stride = H * hd; p.out_batch_stride = T * H * hd;
                 p.out16_hi = o16_hi >= 0 ? s->ptr(o16_hi) : nullptr;
                 p.out16_lo = o16_lo >= 0 ? s->ptr(o16_lo) : nullptr;
                 p.batch = (int)B; p.heads = (int)H; p.tokens = (int)T; p.head_dim = (int)hd;
                 p.scale = f.scale >= 0 ? s->fptr(f.scale) : nullptr; p.scale_mode = f.scale_mode;
                 p.use_tc = tc_attn ? 1 : 0; p.err_word = s->err_word;
                 return launch_attention(p, st);
               });
        return;
      }
      const int o = n.outputs[0];
      int x = n.inputs[0];
      const Value& xv = V(x);
      require_f32(xv, "Softmax");
      const int64_t axis = n.ints.empty() ? -1 : n.ints[0];
      if (!(axis == -1 || axis == xv.rank - 1))
        fail(AC_ERR_UNSUPPORTED, "Softmax: last axis only");  // session.rs:999
      const int64_t len = xv.dims[xv.rank - 1], rows = xv.numel() / std::max<int64_t>(len, 1);
      int mode = 0, scale = -1, mask = -1, mask_else = -1;
      int64_t mask_rows = 1;
      auto mk = plan.softmax_mask.find(nid);
      if (mk != plan.softmax_mask.end()) {
        const Node& w = c.node(mk->second);
        mask = w.inputs[0]; x = w.inputs[1]; mask_else = w.inputs[2];
        mask_rows = V(mask).numel() / std::max<int64_t>(len, 1);
      }
      auto it = plan.softmax_scale.find(nid);
      if (it != plan.softmax_scale.end()) {
        Node& m = c.node(it->second);
        const bool b_scalar = V(m.inputs[1]).numel() == 1 && same_dims(V(m.inputs[0]), xv);
        scale = b_scalar ? m.inputs[1] : m.inputs[0];
        x = b_scalar ? m.inputs[0] : m.inputs[1];
        mode = m.op == AC_OP_MUL ? 1 : 2;
      }
      const char* kind = mask >= 0 ? (mode ? "softmax_scaled_masked" : "softmax_masked") : (mode ? "softmax_scaled" : "softmax");
      em.add(kind, n.op, {x, scale, mask, mask_else}, {o}, 8.0 * rows * len + (mask >= 0 ? (double)V(mask).bytes() : 0.0), 0,
             [=](cudaStream_t st) {
               return launch_softmax(s->fptr(x), s->fptr_mut(o), rows, len, mode,
                                     scale >= 0 ? s->fptr(scale) : nullptr,
                                     mask >= 0 ? static_cast<const uint8_t*>(s->ptr(mask)) : nullptr, mask_rows,
                                     mask_else >= 0 ? s->fptr(mask_else) : nullptr, st);
             });
      return;
    }
    case AC_OP_LAYERNORMALIZATION: {
      const int gamma = n.inputs[1], beta = n.inputs[2], o = n.outputs[0];
      const Value& xv = V(n.inputs[0]);
      require_f32(xv, "LayerNormalization");
      const int64_t axis = n.ints.size() > 0 ? n.ints[0] : -1;
      const int64_t stash = n.ints.size() > 1 ? n.ints[1] : 1;
      if (!(axis == -1 || axis == xv.rank - 1))
        fail(AC_ERR_UNSUPPORTED, "Axis must be the last dimension.");  // session.rs:1444-1447
      if (stash != 1) fail(AC_ERR_UNSUPPORTED, "Stash type must be 1.");
      const int64_t len = xv.dims[xv.rank - 1], rows = xv.numel() / std::max<int64_t>(len, 1);
      if (V(gamma).numel() != len || V(beta).numel() != len)
        fail(AC_ERR_SHAPE, "LayerNormalization: scale / bias length");
      const float eps = n.floats.size() > 0 ? n.floats[0] : 1e-5f;
      LnFusion f;
      f.x = n.inputs[0];
      auto it = plan.ln.find(nid);
      if (it != plan.ln.end()) f = it->second;
      const int x = f.x, pb = f.pre_bias, res = f.residual, sum = f.sum_val, gelu = f.gelu;
      // The GEMM(s) that consume the result may take it as fp16 hi / lo halves (vector path only).
      int o16_hi = -1, o16_lo = -1;
      bool o_fp32 = true;
      {
        auto so = c.split.find(o);
        if (so != c.split.end() && !so->second.produced && (len % 8) == 0 && len <= 1024) {
          o16_hi = so->second.hi; o16_lo = so->second.lo;
          o_fp32 = so->second.fp32_needed;
          so->second.produced = true;
        }
      }
      std::vector<int> writes;
      if (o_fp32) writes.push_back(o);
      if (o16_hi >= 0) { writes.push_back(o16_hi); writes.push_back(o16_lo); }
      if (sum >= 0) writes.push_back(sum);
      double bytes = 8.0 * rows * len + 8.0 * len;
      if (res >= 0 && res != x) bytes += 4.0 * rows * len;
      if (sum >= 0) bytes += 4.0 * rows * len;
      const char* kind = res >= 0 ? (gelu || pb >= 0 ? "layer_norm_bias_gelu_residual" : "layer_norm_residual")
                                  : "layer_norm";
      em.add(kind, n.op, {x, pb, res, gamma, beta}, writes, bytes, 0, [=](cudaStream_t st) {
        LayerNormParams p{};
        p.x = s->fptr(x);
        p.pre_bias = pb >= 0 ? s->fptr(pb) : nullptr;
        p.residual = res >= 0 ? s->fptr(res) : nullptr;
        p.gamma = s->fptr(gamma); p.beta = s->fptr(beta);
        p.sum_out = sum >= 0 ? s->fptr_mut(sum) : nullptr;
        p.out = o_fp32 ? s->fptr_mut(o) : nullptr;
        p.out16_hi = o16_hi >= 0 ? s->ptr(o16_hi) : nullptr;
        p.out16_lo = o16_lo >= 0 ? s->ptr(o16_lo) : nullptr;
        p.err_word = s->err_word;
        p.rows = rows; p.len = len; p.eps = eps; p.gelu = gelu;
        return launch_layer_norm(p, st);
      });
      return;
    }
    case AC_OP_REDUCEMEAN: case AC_OP_REDUCEMAX: {
      const int x = n.inputs[0], o = n.outputs[0];
      const Value& xv = V(x);
      require_f32(xv, op_name(n.op));
      std::vector<int64_t> axes;
      for (size_t i = 1; i < n.ints.size(); ++i) axes.push_back(n.ints[i] < 0 ? n.ints[i] + xv.rank : n.ints[i]);
      const bool last_only = axes.size() == 1 && axes[0] == xv.rank - 1;
      if (n.op == AC_OP_REDUCEMAX && (axes.empty() || (int)axes.size() == xv.rank)) {
        // compute_reduce_max, session.rs:1292-1305: all axes -> one scalar.
        Value sv;
        sv.elem_ty = AC_F32; sv.rank = 1;
        sv.dims[0] = reduce_max_all_scratch_elems(xv.numel());
        sv.storage = c.new_storage(sv.bytes());
        s->values.push_back(sv);
        const int scratch = (int)s->values.size() - 1;
        c.producer.push_back(-1); c.consumers.emplace_back(); c.is_output.push_back(0);
        const int64_t cnt = xv.numel();
        em.add("reduce_max_all", n.op, {x}, {o, scratch}, 4.0 * cnt, 0, [=](cudaStream_t st) {
          return launch_reduce_max_all(s->fptr(x), s->fptr_mut(o), cnt, s->fptr_mut(scratch), st);
        }, 2);
        return;
      }
      if (!last_only)
        fail(AC_ERR_UNSUPPORTED, std::string(op_name(n.op)) + ": only the last axis is supported");
      const int64_t len = xv.dims[xv.rank - 1], rows = xv.numel() / std::max<int64_t>(len, 1);
      const bool mean = n.op == AC_OP_REDUCEMEAN;
      auto sib = plan.reduce_sibling.find(nid);
      if (mean && sib != plan.reduce_sibling.end()) {
        const int o2 = c.node(sib->second).outputs[0];
        em.add("reduce_mean_max", n.op, {x}, {o, o2}, 4.0 * rows * len + 8.0 * rows, 0, [=](cudaStream_t st) {
          return launch_reduce_mean_max_last(s->fptr(x), s->fptr_mut(o), s->fptr_mut(o2), rows, len, st);
        });
        return;
      }
      em.add(mean ? "reduce_mean" : "reduce_max", n.op, {x}, {o}, 4.0 * rows * len + 4.0 * rows, 0,
             [=](cudaStream_t st) {
               return mean ? launch_reduce_mean_last(s->fptr(x), s->fptr_mut(o), rows, len, st)
                           : launch_reduce_max_last(s->fptr(x), s->fptr_mut(o), rows, len, st);
             });
      return;
    }
    case AC_OP_GLOBALAVERAGEPOOL: {
      const int x = n.inputs[0], o = n.outputs[0];
      const Value& xv = V(x);
      require_f32(xv, "GlobalAveragePool");
      const int64_t planes = xv.dims[0] * xv.dims[1], hw = xv.dims[2] * xv.dims[3];
      em.add("global_avg_pool", n.op, {x}, {o}, 4.0 * planes * hw + 4.0 * planes, 0,
             [=](cudaStream_t st) { return launch_gavg_pool(s->fptr(x), s->fptr_mut(o), planes, hw, st); });
      return;
    }
    case AC_OP_MAXPOOL: {
      const int x = n.inputs[0], o = n.outputs[0];
      const Value& xv = V(x);
      const Value& ov = V(o);
      require_f32(xv, "MaxPool");
      int64_t pads[4];
      resolve_pads(n, 4, xv.dims[2], xv.dims[3], pads);
      const int64_t planes = xv.dims[0] * xv.dims[1];
      const int ih = (int)xv.dims[2], iw = (int)xv.dims[3], oh = (int)ov.dims[2], ow = (int)ov.dims[3];
      const int kh = (int)n.ints[0], kw = (int)n.ints[1], sh = (int)n.ints[2], sw = (int)n.ints[3];
      const int pt = (int)pads[0], pl = (int)pads[1];
      em.add("max_pool", n.op, {x}, {o}, f32_bytes(xv) + f32_bytes(ov), 0, [=](cudaStream_t st) {
        return launch_max_pool(s->fptr(x), s->fptr_mut(o), planes, ih, iw, oh, ow, kh, kw, sh, sw, pt,
                               pl, st);
      });
      return;
    }
    case AC_OP_TRANSPOSE: {
      const int x = n.inputs[0], o = n.outputs[0];
      const Value& xv = V(x);
      const int r = xv.rank;
      // Batched swap of the last two dims -> tiled shared-memory transpose.
      bool swap_last = r >= 2 && n.ints[r - 1] == r - 2 && n.ints[r - 2] == r - 1 && xv.elem_ty == AC_F32;
      for (int i = 0; swap_last && i < r - 2; ++i) swap_last = n.ints[i] == i;
      const int64_t rows = r >= 2 ? xv.dims[r - 2] : 1, cols = r >= 1 ? xv.dims[r - 1] : 1;
      const int64_t batch = xv.numel() / std::max<int64_t>(rows * cols, 1);
      if (swap_last && batch <= 65535 && rows > 1 && cols > 1) {
        em.add("transpose_tiled", n.op, {x}, {o}, 2.0 * xv.bytes(), 0, [=](cudaStream_t st) {
          return launch_transpose2d(s->fptr(x), s->fptr_mut(o), batch, (int)rows, (int)cols, st);
        });
        return;
      }
      CopyParams p{};
      p.rank = r;
      int64_t in_str[AC_MAX_RANK];
      contiguous_strides(xv.dims, r, in_str);
      for (int i = 0; i < r; ++i) { p.dims[i] = xv.dims[n.ints[i]]; p.in_str[i] = in_str[n.ints[i]]; }
      contiguous_strides(p.dims, r, p.out_str);
      p.n = xv.numel();
      p.elem_bytes = (int)xv.elem_bytes();
      return lower_copy(em, "transpose_copy", n.op, x, o, p);
    }
    case AC_OP_CONCAT: {
      const int o = n.outputs[0];
      const Value& ov = V(o);
      int64_t axis = n.ints[0];
      if (axis < 0) axis += ov.rank;
      int64_t out_str[AC_MAX_RANK];
      contiguous_strides(ov.dims, ov.rank, out_str);
      int64_t off = 0;
      for (int x : n.inputs) {
        const Value& xv = V(x);
        CopyParams p{};
        p.rank = xv.rank;
        for (int i = 0; i < xv.rank; ++i) { p.dims[i] = xv.dims[i]; p.out_str[i] = out_str[i]; }
        contiguous_strides(xv.dims, xv.rank, p.in_str);
        p.out_off = off * out_str[axis];
        p.n = xv.numel();
        p.elem_bytes = (int)xv.elem_bytes();
        lower_copy(em, "concat_copy", n.op, x, o, p);
        off += xv.dims[axis];
      }
      return;
    }
    case AC_OP_SPLIT: {
      const int x = n.inputs[0];
      const Value& xv = V(x);
      int64_t axis = n.ints[0];
      if (axis < 0) axis += xv.rank;
      int64_t in_str[AC_MAX_RANK];
      contiguous_strides(xv.dims, xv.rank, in_str);
      int64_t off = 0;
      for (int o : n.outputs) {
        const Value& ov = V(o);
        CopyParams p{};
        p.rank = ov.rank;
        for (int i = 0; i < ov.rank; ++i) { p.dims[i] = ov.dims[i]; p.in_str[i] = in_str[i]; }
        contiguous_strides(ov.dims, ov.rank, p.out_str);
        p.in_off = off * in_str[axis];
        p.n = ov.numel();
        p.elem_bytes = (int)ov.elem_bytes();
        lower_copy(em, "split_copy", n.op, x, o, p);
        off += ov.dims[axis];
      }
      return;
    }
    case AC_OP_SLICE: {
      const int x = n.inputs[0], o = n.outputs[0];
      const Value& xv = V(x);
      const Value& ov = V(o);
      const int64_t* starts = static_cast<const int64_t*>(V(n.inputs[1]).host);
      const int64_t* axes = static_cast<const int64_t*>(V(n.inputs[3]).host);
      const int64_t na = V(n.inputs[3]).numel();
      const int64_t* steps = (n.inputs.size() > 4 && n.inputs[4] >= 0)
                                 ? static_cast<const int64_t*>(V(n.inputs[4]).host) : nullptr;
      CopyParams p{};
      p.rank = xv.rank;
      contiguous_strides(xv.dims, xv.rank, p.in_str);
      for (int i = 0; i < xv.rank; ++i) p.dims[i] = ov.dims[i];
      for (int64_t i = 0; i < na; ++i) {
        const int64_t ax = axes[i] < 0 ? axes[i] + xv.rank : axes[i];
        p.in_off += starts[i] * p.in_str[ax];
        p.in_str[ax] *= steps ? steps[i] : 1;
      }
      contiguous_strides(ov.dims, ov.rank, p.out_str);
      p.n = ov.numel();
      p.elem_bytes = (int)xv.elem_bytes();
      return lower_copy(em, "slice_copy", n.op, x, o, p);
    }
    case AC_OP_GATHER: {
      const int x = n.inputs[0], idx = n.inputs[1], o = n.outputs[0];
      const Value& xv = V(x);
      const Value& iv = V(idx);
      if (!iv.host || iv.elem_ty != AC_I64)
        fail(AC_ERR_UNSUPPORTED, "Gather: indices must be a constant i64 tensor");
      const int64_t* ind = static_cast<const int64_t*>(iv.host);
      const int64_t axis = n.ints[0];
      int64_t in_str[AC_MAX_RANK];
      contiguous_strides(xv.dims, xv.rank, in_str);
      const bool scalar = iv.rank == 0 || (iv.rank == 1 && iv.dims[0] <= 1);
      const int64_t cnt = scalar ? 1 : iv.dims[1];
      if (cnt > 256) fail(AC_ERR_UNSUPPORTED, "Gather: more than 256 indices");
      // One strided copy per index: out[.., j, ..] = x[.., ind[j], ..].
      const int64_t slab = xv.numel() / xv.dims[axis];
      for (int64_t j = 0; j < cnt; ++j) {
        if (ind[j] < 0 || ind[j] >= xv.dims[axis]) fail(AC_ERR_SHAPE, "Gather: index out of range");
        CopyParams p{};
        p.rank = 0;
        for (int i = 0; i < xv.rank; ++i) {
          if (i == axis) continue;
          p.dims[p.rank] = xv.dims[i];
          p.in_str[p.rank] = in_str[i];
          ++p.rank;
        }
        contiguous_strides(p.dims, p.rank, p.out_str);
        p.in_off = ind[j] * in_str[axis];
        p.out_off = j * slab;  // the [1, k] form gathers on axis 0: slabs are consecutive
        p.n = slab;
        p.elem_bytes = (int)xv.elem_bytes();
        lower_copy(em, "gather_copy", n.op, x, o, p);
      }
      return;
    }
    case AC_OP_MATMUL: {
      auto it = plan.epi.find(nid);
      return lower_matmul(em, nid, it == plan.epi.end() ? nullptr : &it->second);
    }
    case AC_OP_GEMM: {
      auto it = plan.epi.find(nid);
      return lower_gemm(em, nid, it == plan.epi.end() ? nullptr : &it->second);
    }
    case AC_OP_CONV2D: {
      auto it = plan.epi.find(nid);
      auto sg = plan.se_gate.find(nid);
      return lower_conv(em, nid, it == plan.epi.end() ? nullptr : &it->second,
                        sg == plan.se_gate.end() ? nullptr : &sg->second);
    }
    default:
      fail(AC_ERR_UNSUPPORTED, std::string(op_name(n.op)) + ": Kernel not implemented");
  }
}

// Orders the steps so that every storage is fully written before it is read;
// among ready steps the original (topological) order is kept.
bool order_steps(AcSession& s) {
  const int n = (int)s.steps.size();
  std::map<int, std::vector<int>> writers;
  for (int i = 0; i < n; ++i)
    for (int w : s.steps[i].writes) writers[w].push_back(i);
  std::vector<std::set<int>> deps(n);
  for (int i = 0; i < n; ++i)
    for (int r : s.steps[i].reads) {
      auto it = writers.find(r);
      if (it == writers.end()) continue;
      for (int w : it->second)
        if (w != i) deps[i].insert(w);
    }
  std::vector<int> done(n, 0), out;
  for (int placed = 0; placed < n;) {
    bool progress = false;
    for (int i = 0; i < n; ++i) {
      if (done[i]) continue;
      bool ready = true;
      for (int d : deps[i]) ready = ready && done[d];
      if (!ready) continue;
      done[i] = 1;
      out.push_back(i);
      ++placed;
      progress = true;
      break;  // restart from the lowest index to keep the original order
    }
    if (!progress) return false;
  }
  std::vector<Step> sorted;
  sorted.reserve(n);
  for (int i : out) sorted.push_back(std::move(s.steps[i]));
  s.steps.swap(sorted);
  return true;
}

}  // namespace

void lower_graph(AcSession& s) {
  Ctx c(s);
  const int nv = (int)s.values.size();
  c.producer.assign(nv, -1);
  c.consumers.assign(nv, {});
  c.is_output.assign(nv, 0);
  c.absorbed.assign(s.nodes.size(), 0);
  for (size_t i = 0; i < s.nodes.size(); ++i) {
    for (int v : s.nodes[i].inputs)
      if (v >= 0) c.consumers[v].push_back((int)i);
    for (int v : s.nodes[i].outputs) c.producer[v] = (int)i;
  }
  for (int o : s.outputs) c.is_output[o] = 1;

  // Storages: initializers in the weight blob, inputs and everything computed in the arena.
  for (int v = 0; v < nv; ++v) {
    Value& val = s.values[v];
    if (val.is_init) {
      val.is_const = true;
      val.storage = c.new_storage(val.bytes(), /*weight=*/true);
    }
  }
  for (int v : s.inputs) {
    if (s.values[v].is_init) fail(AC_ERR_INVALID, "a graph input is also an initializer");
    s.values[v].storage = c.new_storage(s.values[v].bytes(), false, /*pinned=*/true);
  }
  for (int nid : s.order) {
    Node& n = s.nodes[nid];
    bool all_const = true;
    for (int v : n.inputs)
      if (v >= 0) {
        if (s.values[v].storage < 0 && s.values[v].rank >= 0 && c.producer[v] < 0)
          fail(AC_ERR_INVALID, std::string(op_name(n.op)) + ": input is neither computed, an input nor an initializer");
        all_const = all_const && s.values[v].is_const;
      }
    const bool alias = n.op == AC_OP_IDENTITY || n.op == AC_OP_RESHAPE || n.op == AC_OP_FLATTEN ||
                       n.op == AC_OP_SQUEEZE || n.op == AC_OP_UNSQUEEZE;
    for (int o : n.outputs) {
      Value& ov = s.values[o];
      ov.is_const = all_const;
      if (alias) {
        const Value& iv = s.values[n.inputs[0]];
        ov.storage = iv.storage;
        if (iv.host && !ov.host) ov.host = iv.host;
      } else {
        ov.storage = c.new_storage(ov.bytes(), false, all_const);
      }
    }
  }
  for (int o : s.outputs) s.storages[s.values[o].storage].pinned_live = true;

  const size_t graph_values = s.values.size(), graph_storages = s.storages.size();
  for (int attempt = 0; attempt < 2; ++attempt) {
    const bool fuse = attempt == 0 && !s.opt.disable_fusion;
    Plan plan;
    std::fill(c.absorbed.begin(), c.absorbed.end(), 0);
    s.steps.clear();
    // Scratch values and storages of a first attempt do not survive into the second.
    s.values.resize(graph_values);
    s.storages.resize(graph_storages);
    c.producer.resize(graph_values);
    c.consumers.resize(graph_values);
    c.is_output.resize(graph_values);
    c.split.clear();
    if (fuse) {
      detect_attention(c, plan);
      detect_epilogues(c, plan);
      detect_softmax_scale(c, plan);
      detect_layer_norm(c, plan);
      detect_hardswish(c, plan);
      detect_se_gate(c, plan);
      detect_reduce_siblings(c, plan);
      // Debug toggle: ALTIUS_CUDA_NO_FUSED_SPLIT=1 keeps a split kernel in front of every pair GEMM.
      if (!std::getenv("ALTIUS_CUDA_NO_FUSED_SPLIT")) plan_presplit(c, plan);
    }
    Emit em(c);
    for (int nid : s.order)
      if (!c.absorbed[nid]) lower_node(em, plan, nid);
    if (order_steps(s)) break;
    if (!fuse) fail(AC_ERR_INVALID, "kernel schedule has a dependency cycle");
  }

  // Constant-only steps run once at create(); their results stay resident.
  std::vector<Step> run;
  for (Step& st : s.steps) {
    if (st.const_only) s.init_steps.push_back(std::move(st));
    else run.push_back(std::move(st));
  }
  s.steps.swap(run);
  s.launches_per_run = 0;
  for (const Step& st : s.steps) s.launches_per_run += st.launches;
}

}  // namespace ac
