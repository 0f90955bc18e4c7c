// Graph passes on raw exports: the four rewrites altius_py applies before it builds a session
// (crates/altius_py/src/lib.rs:54-62), restated over AcModel:
//   fuse_layer_norm     crates/core/src/optimize/layer_norm_fusion.rs:13-123
//   fuse_gelu           crates/core/src/optimize/gelu_fusion.rs:12-131
//   fuse_fast_gelu      crates/core/src/optimize/fast_gelu_fusion.rs:5-190
//   eliminate_identity  crates/core/src/optimize/identity_elim.rs:5-45
// Same patterns, same constants and tolerances, same rewiring. One deliberate difference:
// where the reference follows "the first user" of a value out of a hash set (an arbitrary one
// when the value has several users, so whether a pattern is found can depend on hash order),
// these passes look for a user with the operator the pattern wants next.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "model.h"

namespace ac {

std::map<int32_t, std::vector<int>> value_users(const AcModel& m) {
  std::map<int32_t, std::vector<int>> users;
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    if (m.nodes[i].deleted) continue;
    for (int32_t v : m.nodes[i].inputs) {
      if (v < 0) continue;
      std::vector<int>& u = users[v];
      if (std::find(u.begin(), u.end(), (int)i) == u.end()) u.push_back((int)i);
    }
  }
  return users;
}

std::map<int32_t, int> value_parents(const AcModel& m) {
  std::map<int32_t, int> parents;
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    if (m.nodes[i].deleted) continue;
    for (int32_t v : m.nodes[i].outputs) parents[v] = (int)i;
  }
  return parents;
}

// model.rs:62-102: a LIFO work list seeded, in arena order, with the nodes whose
// non-constant inputs are all available.
std::vector<int> topo_sort_nodes(const AcModel& m) {
  const auto users = value_users(m);
  const auto parents = value_parents(m);
  std::vector<char> is_const(m.values.size(), 0);
  for (int32_t v : m.inputs) is_const[v] = 1;
  for (const auto& kv : m.inits) is_const[kv.first] = 1;
  std::vector<int> pending(m.nodes.size(), 0), work, order;
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    if (m.nodes[i].deleted) continue;
    std::vector<int32_t> ins;
    for (int32_t v : m.nodes[i].inputs)
      if (v >= 0 && !is_const[v] && parents.count(v) && std::find(ins.begin(), ins.end(), v) == ins.end()) ins.push_back(v);
    pending[i] = (int)ins.size();
    if (ins.empty()) work.push_back((int)i);
  }
  while (!work.empty()) {
    const int id = work.back();
    work.pop_back();
    order.push_back(id);
    for (int32_t o : m.nodes[id].outputs) {
      auto it = users.find(o);
      if (it == users.end()) continue;
      for (int u : it->second)
        if (--pending[u] == 0) work.push_back(u);
    }
  }
  return order;
}

// model.rs:104-121: drop the deleted nodes, keep the rest in topological order.
void remove_unnecessary_nodes(AcModel& m) {
  const std::vector<int> order = topo_sort_nodes(m);
  std::vector<int> pos(m.nodes.size(), -1);
  for (size_t i = 0; i < order.size(); ++i) pos[order[i]] = (int)i;
  std::vector<int> keep;
  for (size_t i = 0; i < m.nodes.size(); ++i)
    if (!m.nodes[i].deleted) keep.push_back((int)i);
  std::stable_sort(keep.begin(), keep.end(), [&](int a, int b) { return pos[a] < pos[b]; });
  std::vector<MNode> nodes;
  nodes.reserve(keep.size());
  for (int i : keep) nodes.push_back(std::move(m.nodes[i]));
  m.nodes.swap(nodes);
}

namespace {

using Users = std::map<int32_t, std::vector<int>>;

// A user of `v` with operator `op`, or -1.
int user_with_op(const AcModel& m, const Users& users, int32_t v, int op) {
  auto it = users.find(v);
  if (it == users.end()) return -1;
  for (int u : it->second)
    if (m.nodes[u].op == op) return u;
  return -1;
}

bool single_user(const Users& users, int32_t v) {
  auto it = users.find(v);
  return it != users.end() && it->second.size() == 1;
}

// The first f32 element of an initializer (`inits.get(v)...data::<f32>()[0]`).
bool init_f32(const AcModel& m, int32_t v, float* out) {
  if (v < 0) return false;
  auto it = m.inits.find(v);
  if (it == m.inits.end() || m.values[v].elem_ty != AC_F32 || it->second.size() < 4) return false;
  std::memcpy(out, it->second.data(), 4);
  return true;
}

// Tensor::allclose(&[c]), tensor.rs:352-363, 518-523: a one-element f32 initializer within
// atol 1e-5 + rtol 1e-8 of c.
bool init_allclose(const AcModel& m, int32_t v, float c) {
  float x;
  if (!init_f32(m, v, &x)) return false;
  if (m.inits.at(v).size() != 4) return false;
  return std::fabs(x - c) <= 1e-5f + 1e-8f * std::fabs(c) || (std::isinf(x) && std::isinf(c) && (x > 0) == (c > 0));
}
bool init_equals(const AcModel& m, int32_t v, float c) {
  float x;
  return init_f32(m, v, &x) && x == c;
}

// Every use of `end` (node inputs, or the graph outputs when it has no user) becomes `fresh`.
void replace_value(AcModel& m, const Users& users, int32_t end, int32_t fresh) {
  auto it = users.find(end);
  if (it == users.end()) {
    for (int32_t& o : m.outputs)
      if (o == end) o = fresh;
    return;
  }
  for (int u : it->second)
    for (int32_t& in : m.nodes[u].inputs)
      if (in == end) in = fresh;
}

}  // namespace

int fuse_layer_norm(AcModel& m) {
  // X -> ReduceMean -> Sub -> Pow -> ReduceMean -> Add -> Sqrt -> Div -> Mul -> Add
  const std::vector<int> order = topo_sort_nodes(m);
  const Users users = value_users(m);
  struct Found { int32_t data, end, scale, bias, eps; };
  std::vector<Found> found;
  std::vector<int> dead;
  for (int mean_id : order) {
    const MNode& mean = m.nodes[mean_id];
    if (mean.op != AC_OP_REDUCEMEAN) continue;
    static const int chain[] = {AC_OP_SUB, AC_OP_POW, AC_OP_REDUCEMEAN, AC_OP_ADD, AC_OP_SQRT, AC_OP_DIV, AC_OP_MUL, AC_OP_ADD};
    int ids[9];
    ids[0] = mean_id;
    bool ok = true;
    for (int k = 0; k < 8 && ok; ++k) {
      ids[k + 1] = user_with_op(m, users, m.nodes[ids[k]].outputs[0], chain[k]);
      ok = ids[k + 1] >= 0;
    }
    if (!ok) continue;
    const MNode& add = m.nodes[ids[4]];
    const MNode& mul = m.nodes[ids[7]];
    const MNode& add2 = m.nodes[ids[8]];
    if (add.inputs.size() < 2 || mul.inputs.size() < 2 || add2.inputs.size() < 2) continue;
    float eps;
    if (!init_f32(m, add.inputs[1], &eps)) continue;       // the reference unwraps here
    found.push_back({mean.inputs[0], add2.outputs[0], mul.inputs[1], add2.inputs[1], add.inputs[1]});
    dead.insert(dead.end(), ids, ids + 9);
  }
  for (const Found& f : found) {
    float eps = 0;
    init_f32(m, f.eps, &eps);
    const int32_t out = m.new_value();
    MNode ln;
    ln.op = AC_OP_LAYERNORMALIZATION;
    ln.inputs = {f.data, f.scale, f.bias};
    ln.outputs = {out};
    ln.ints = {-1, 1};          // axis, stash_type
    ln.floats = {eps};
    m.nodes.push_back(ln);
    replace_value(m, users, f.end, out);
  }
  for (int id : dead) m.nodes[id].deleted = true;
  remove_unnecessary_nodes(m);
  return (int)found.size();
}

int fuse_gelu(AcModel& m) {
  // x -> Div(1.41421) -> Erf -> Add(1) -> Mul(x) -> Mul(0.5)
  const std::vector<int> order = topo_sort_nodes(m);
  const Users users = value_users(m);
  std::vector<std::pair<int32_t, int32_t>> found;
  std::vector<int> dead;
  for (int div_id : order) {
    const MNode& div = m.nodes[div_id];
    if (div.op != AC_OP_DIV || div.inputs.size() < 2 || !init_allclose(m, div.inputs[1], 1.4142099618911743f)) continue;
    const int erf_id = user_with_op(m, users, div.outputs[0], AC_OP_ERF);
    if (erf_id < 0) continue;
    const int add_id = user_with_op(m, users, m.nodes[erf_id].outputs[0], AC_OP_ADD);
    if (add_id < 0) continue;
    const MNode& add = m.nodes[add_id];
    const bool erf_lhs = add.inputs[0] == m.nodes[erf_id].outputs[0];
    if (!init_equals(m, add.inputs[erf_lhs ? 1 : 0], 1.f)) continue;
    const int mul1_id = user_with_op(m, users, add.outputs[0], AC_OP_MUL);
    if (mul1_id < 0) continue;
    const MNode& mul1 = m.nodes[mul1_id];
    const bool add_lhs = mul1.inputs[0] == add.outputs[0];
    if (mul1.inputs[add_lhs ? 1 : 0] != div.inputs[0]) continue;
    const int mul2_id = user_with_op(m, users, mul1.outputs[0], AC_OP_MUL);
    if (mul2_id < 0) continue;
    const MNode& mul2 = m.nodes[mul2_id];
    const bool mul1_lhs = mul2.inputs[0] == mul1.outputs[0];
    if (!init_equals(m, mul2.inputs[mul1_lhs ? 1 : 0], 0.5f)) continue;
    found.push_back({div.inputs[0], mul2.outputs[0]});
    for (int id : {div_id, erf_id, add_id, mul1_id, mul2_id}) dead.push_back(id);
  }
  for (const auto& se : found) {
    const int32_t out = m.new_value();
    MNode g;
    g.op = AC_OP_GELU;
    g.inputs = {se.first};
    g.outputs = {out};
    m.nodes.push_back(g);
    replace_value(m, users, se.second, out);
  }
  for (int id : dead) m.nodes[id].deleted = true;
  remove_unnecessary_nodes(m);
  return (int)found.size();
}

int fuse_fast_gelu(AcModel& m) {
  // x -> Pow(3) -> Mul(0.044715) -> Add(x, .) -> Mul(0.79788) -> Tanh -> Add(1) -> Mul(Mul(x, 0.5), .)
  const std::vector<int> order = topo_sort_nodes(m);
  const Users users = value_users(m);
  const auto parents = value_parents(m);
  std::vector<std::pair<int32_t, int32_t>> found;
  std::vector<int> dead;
  for (int nid : order) {
    const MNode& src = m.nodes[nid];
    if (src.outputs.size() != 1) continue;
    const int32_t x = src.outputs[0];
    const int pow_id = user_with_op(m, users, x, AC_OP_POW);
    if (pow_id < 0) continue;
    const MNode& pow = m.nodes[pow_id];
    if (pow.inputs.size() < 2 || !init_equals(m, pow.inputs[1], 3.f) || !single_user(users, pow.outputs[0])) continue;
    const int mul1_id = user_with_op(m, users, pow.outputs[0], AC_OP_MUL);
    if (mul1_id < 0) continue;
    const MNode& mul1 = m.nodes[mul1_id];
    if (!init_allclose(m, mul1.inputs[1], 0.044714998453855515f) || !single_user(users, mul1.outputs[0])) continue;
    const int add1_id = user_with_op(m, users, mul1.outputs[0], AC_OP_ADD);
    if (add1_id < 0) continue;
    const MNode& add1 = m.nodes[add1_id];
    if (add1.inputs[0] != x || !single_user(users, add1.outputs[0])) continue;
    const int mul2_id = user_with_op(m, users, add1.outputs[0], AC_OP_MUL);
    if (mul2_id < 0) continue;
    const MNode& mul2 = m.nodes[mul2_id];
    if (!init_allclose(m, mul2.inputs[1], 0.7978845834732056f) || !single_user(users, mul2.outputs[0])) continue;
    const int tanh_id = user_with_op(m, users, mul2.outputs[0], AC_OP_TANH);
    if (tanh_id < 0 || !single_user(users, m.nodes[tanh_id].outputs[0])) continue;
    const int add2_id = user_with_op(m, users, m.nodes[tanh_id].outputs[0], AC_OP_ADD);
    if (add2_id < 0) continue;
    const MNode& add2 = m.nodes[add2_id];
    if (!init_equals(m, add2.inputs[1], 1.f) || !single_user(users, add2.outputs[0])) continue;
    const int mul3_id = user_with_op(m, users, add2.outputs[0], AC_OP_MUL);
    if (mul3_id < 0) continue;
    const MNode& mul3 = m.nodes[mul3_id];
    if (mul3.inputs[1] != add2.outputs[0]) continue;        // the reference asserts this
    auto pit = parents.find(mul3.inputs[0]);
    if (pit == parents.end()) continue;
    const int mul4_id = pit->second;
    const MNode& mul4 = m.nodes[mul4_id];
    if (mul4.op != AC_OP_MUL || mul4.inputs[0] != x || !init_equals(m, mul4.inputs[1], 0.5f) ||
        !single_user(users, mul4.outputs[0]))
      continue;
    found.push_back({x, mul3.outputs[0]});
    for (int id : {pow_id, mul1_id, add1_id, mul2_id, tanh_id, add2_id, mul3_id, mul4_id}) dead.push_back(id);
  }
  for (const auto& se : found) {
    const int32_t out = m.new_value();
    MNode g;
    g.op = AC_OP_GELU;
    g.inputs = {se.first};
    g.outputs = {out};
    m.nodes.push_back(g);
    replace_value(m, users, se.second, out);
  }
  for (int id : dead) m.nodes[id].deleted = true;
  remove_unnecessary_nodes(m);
  return (int)found.size();
}

int eliminate_identity(AcModel& m) {
  const Users users = value_users(m);
  const std::vector<int> order = topo_sort_nodes(m);
  int count = 0;
  for (int nid : order) {
    MNode& n = m.nodes[nid];
    if (n.op != AC_OP_IDENTITY) continue;
    if (n.inputs.size() != 1 || n.outputs.size() != 1) throw ModelError{AC_ERR_INVALID, "Identity: one input and one output expected"};
    const int32_t in = n.inputs[0], out = n.outputs[0];
    auto it = users.find(out);
    if (it == users.end()) continue;       // feeds a graph output: kept, so that input and output stay distinct values
    for (int u : it->second)
      for (int32_t& v : m.nodes[u].inputs)
        if (v == out) v = in;
    n.deleted = true;
    ++count;
  }
  remove_unnecessary_nodes(m);
  return count;
}

}  // namespace ac
