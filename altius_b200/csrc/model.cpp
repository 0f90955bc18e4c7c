// C ABI of the model object: load an .onnx file (or buffer), take a graph description, run
// the graph passes, and hand the graph out as the AcGraphDesc that altius_cuda_create takes.
// Host code only; no CUDA call is made here.
#include <cstdio>
#include <cstring>
#include <fstream>

#include "model.h"

namespace ac {
void set_thread_error(const std::string& msg);   // session.cu: read back by altius_cuda_last_error(NULL)
}

using namespace ac;

namespace {

template <typename Fn>
int guarded(Fn&& fn) {
  try {
    fn();
    return AC_OK;
  } catch (const ModelError& e) {
    set_thread_error(e.msg);
    return e.status;
  } catch (const std::exception& e) {
    set_thread_error(e.what());
    return AC_ERR_INVALID;
  }
}

void from_graph(const AcGraphDesc& g, AcModel& m) {
  if (g.n_values < 0 || g.n_nodes < 0 || (g.n_values && !g.values) || (g.n_nodes && !g.nodes))
    throw ModelError{AC_ERR_INVALID, "malformed graph description"};
  m.opset = g.opset_version;
  m.values.resize(g.n_values);
  for (int i = 0; i < g.n_values; ++i) {
    m.values[i].elem_ty = g.values[i].elem_ty;
    m.values[i].rank = g.values[i].rank < 0 ? -1 : g.values[i].rank;
    if (g.values[i].rank > AC_MAX_RANK) throw ModelError{AC_ERR_SHAPE, "rank above 8 is not supported"};
    for (int k = 0; k < m.values[i].rank; ++k) m.values[i].dims[k] = g.values[i].dims[k];
  }
  auto check = [&](int32_t v, bool allow_missing) {
    if (v == -1 && allow_missing) return;
    if (v < 0 || v >= g.n_values) throw ModelError{AC_ERR_INVALID, "value id out of range"};
  };
  m.nodes.resize(g.n_nodes);
  for (int i = 0; i < g.n_nodes; ++i) {
    const AcNodeDesc& d = g.nodes[i];
    MNode& n = m.nodes[i];
    if (d.op < 0 || d.op >= AC_OP_COUNT) throw ModelError{AC_ERR_INVALID, "bad operator code"};
    n.op = d.op;
    for (int k = 0; k < d.n_inputs; ++k) { check(d.inputs[k], true); n.inputs.push_back(d.inputs[k]); }
    for (int k = 0; k < d.n_outputs; ++k) { check(d.outputs[k], false); n.outputs.push_back(d.outputs[k]); }
    if (d.n_ints > 0) n.ints.assign(d.ints, d.ints + d.n_ints);
    if (d.n_floats > 0) n.floats.assign(d.floats, d.floats + d.n_floats);
    if (d.name) n.name = d.name;
  }
  for (int i = 0; i < g.n_inits; ++i) {
    const AcInitDesc& d = g.inits[i];
    check(d.value, false);
    if (d.location != 0) throw ModelError{AC_ERR_INVALID, "a model is built from host initializers"};
    const char* p = static_cast<const char*>(d.data);
    m.inits[d.value].assign(p, p + d.bytes);
  }
  for (int i = 0; i < g.n_inputs; ++i) { check(g.inputs[i], false); m.inputs.push_back(g.inputs[i]); }
  for (int i = 0; i < g.n_outputs; ++i) { check(g.outputs[i], false); m.outputs.push_back(g.outputs[i]); }
}

}  // namespace

extern "C" {

int altius_model_load_onnx_buffer(const void* buf, size_t len, AcModel** out) {
  if (!buf || !out) { set_thread_error("null argument"); return AC_ERR_INVALID; }
  *out = nullptr;
  AcModel* m = new AcModel();
  const int rc = guarded([&] { load_onnx_buffer(static_cast<const uint8_t*>(buf), len, *m); });
  if (rc != AC_OK) { delete m; return rc; }
  *out = m;
  return AC_OK;
}

int altius_model_load_onnx(const char* path, AcModel** out) {
  if (!path || !out) { set_thread_error("null argument"); return AC_ERR_INVALID; }
  *out = nullptr;
  std::ifstream f(path, std::ios::binary);
  if (!f) { set_thread_error(std::string("cannot open ") + path); return AC_ERR_INVALID; }   // ModelLoadError::Io
  std::vector<char> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  return altius_model_load_onnx_buffer(bytes.data(), bytes.size(), out);
}

int altius_model_from_graph(const AcGraphDesc* graph, AcModel** out) {
  if (!graph || !out) { set_thread_error("null argument"); return AC_ERR_INVALID; }
  *out = nullptr;
  AcModel* m = new AcModel();
  const int rc = guarded([&] { from_graph(*graph, *m); });
  if (rc != AC_OK) { delete m; return rc; }
  *out = m;
  return AC_OK;
}

int altius_model_run_pass(AcModel* m, int32_t pass, int32_t* n_rewrites) {
  if (!m) { set_thread_error("null argument"); return AC_ERR_INVALID; }
  int count = 0;
  const int rc = guarded([&] {
    switch (pass) {
      case 0: count = fuse_layer_norm(*m); break;
      case 1: count = fuse_gelu(*m); break;
      case 2: count = fuse_fast_gelu(*m); break;
      case 3: count = eliminate_identity(*m); break;
      default: throw ModelError{AC_ERR_INVALID, "unknown pass"};
    }
  });
  if (n_rewrites) *n_rewrites = count;
  return rc;
}

int altius_model_optimize(AcModel* m) {
  for (int pass = 0; pass < 4; ++pass) {
    const int rc = altius_model_run_pass(m, pass, nullptr);
    if (rc != AC_OK) return rc;
  }
  return AC_OK;
}

int altius_model_graph(AcModel* m, AcGraphDesc* out) {
  if (!m || !out) { set_thread_error("null argument"); return AC_ERR_INVALID; }
  m->v_values.resize(m->values.size());
  for (size_t i = 0; i < m->values.size(); ++i) {
    AcValueDesc& d = m->v_values[i];
    std::memset(&d, 0, sizeof(d));
    d.elem_ty = m->values[i].elem_ty;
    d.rank = m->values[i].rank;
    for (int k = 0; k < m->values[i].rank && k < AC_MAX_RANK; ++k) d.dims[k] = m->values[i].dims[k];
  }
  m->v_nodes.resize(m->nodes.size());
  for (size_t i = 0; i < m->nodes.size(); ++i) {
    const MNode& n = m->nodes[i];
    AcNodeDesc& d = m->v_nodes[i];
    d.op = n.op;
    d.n_inputs = (int32_t)n.inputs.size(); d.inputs = n.inputs.data();
    d.n_outputs = (int32_t)n.outputs.size(); d.outputs = n.outputs.data();
    d.n_ints = (int32_t)n.ints.size(); d.ints = n.ints.data();
    d.n_floats = (int32_t)n.floats.size(); d.floats = n.floats.data();
    d.name = n.name.empty() ? nullptr : n.name.c_str();
  }
  m->v_inits.clear();
  for (const auto& kv : m->inits) {
    AcInitDesc d;
    d.value = kv.first;
    d.location = 0;
    d.data = kv.second.data();
    d.bytes = kv.second.size();
    m->v_inits.push_back(d);
  }
  out->opset_version = m->opset;
  out->n_values = (int32_t)m->v_values.size(); out->values = m->v_values.data();
  out->n_nodes = (int32_t)m->v_nodes.size(); out->nodes = m->v_nodes.data();
  out->n_inits = (int32_t)m->v_inits.size(); out->inits = m->v_inits.data();
  out->n_inputs = (int32_t)m->inputs.size(); out->inputs = m->inputs.data();
  out->n_outputs = (int32_t)m->outputs.size(); out->outputs = m->outputs.data();
  return AC_OK;
}

const char* altius_model_value_name(const AcModel* m, int32_t value) {
  if (!m || value < 0 || value >= (int32_t)m->values.size() || m->values[value].name.empty()) return nullptr;
  return m->values[value].name.c_str();
}

int32_t altius_model_lookup_named_value(const AcModel* m, const char* name) {
  if (!m || !name) return -1;
  for (size_t i = 0; i < m->values.size(); ++i)
    if (m->values[i].name == name) return (int32_t)i;
  return -1;
}

void altius_model_destroy(AcModel* m) { delete m; }

int altius_cuda_create_from_onnx(const char* path, const AcOptions* options, AcSession** out) {
  if (!out) { set_thread_error("null argument"); return AC_ERR_INVALID; }
  *out = nullptr;
  AcModel* m = nullptr;
  int rc = altius_model_load_onnx(path, &m);
  if (rc != AC_OK) return rc;
  rc = altius_model_optimize(m);
  AcGraphDesc g;
  if (rc == AC_OK) rc = altius_model_graph(m, &g);
  if (rc == AC_OK) rc = altius_cuda_create(&g, options, out);
  altius_model_destroy(m);
  return rc;
}

}  // extern "C"
