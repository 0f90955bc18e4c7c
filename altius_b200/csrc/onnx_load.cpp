// ONNX loader: protobuf wire format -> AcModel, with the reference loader's operator
// table, attribute defaults and initializer handling
// (crates/core/src/onnx/load.rs:55-445; field numbers from crates/core/src/onnx/onnx.proto).
//
// Only the two wire types the ONNX messages need are decoded in depth (varint and
// length-delimited; fixed32 / fixed64 for floats and for skipping). No protobuf library.
// Differences from the reference, both additions: a `Constant` node becomes an initializer of
// its output value (the reference keeps the node and its interpreter cannot run it), and a
// Conv / MaxPool auto_pad other than NOTSET / SAME_UPPER is refused here rather than at run time.
#include <cstring>
#include <map>

#include "model.h"

namespace ac {
namespace {

[[noreturn]] void bad(const std::string& msg, int status = AC_ERR_INVALID) { throw ModelError{status, msg}; }

// ---- wire format -------------------------------------------------------------------------
struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool done() const { return p >= end; }
  uint64_t varint() {
    uint64_t v = 0;
    for (int shift = 0; shift < 64; shift += 7) {
      if (p >= end) bad("Model is invalid: truncated varint");
      const uint8_t b = *p++;
      v |= (uint64_t)(b & 0x7F) << shift;
      if (!(b & 0x80)) return v;
    }
    bad("Model is invalid: varint too long");
  }
  // Reads a field key; returns false at the end of the message.
  bool key(uint32_t* field, uint32_t* wire) {
    if (done()) return false;
    const uint64_t k = varint();
    *field = (uint32_t)(k >> 3);
    *wire = (uint32_t)(k & 7);
    return true;
  }
  Reader sub() {
    const uint64_t n = varint();
    if (n > (uint64_t)(end - p)) bad("Model is invalid: length-delimited field past the end");
    Reader r{p, p + n};
    p += n;
    return r;
  }
  std::string str() {
    Reader r = sub();
    return std::string(reinterpret_cast<const char*>(r.p), r.end - r.p);
  }
  uint32_t fixed32() {
    if (end - p < 4) bad("Model is invalid: truncated fixed32");
    uint32_t v;
    std::memcpy(&v, p, 4);
    p += 4;
    return v;
  }
  void skip(uint32_t wire) {
    switch (wire) {
      case 0: (void)varint(); break;
      case 1: if (end - p < 8) bad("Model is invalid: truncated fixed64"); p += 8; break;
      case 2: (void)sub(); break;
      case 5: (void)fixed32(); break;
      default: bad("Model is invalid: unsupported wire type");
    }
  }
};

float as_float(uint32_t bits) {
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// repeated scalar fields arrive packed (one length-delimited run) or one key per element
void read_ints(Reader& r, uint32_t wire, std::vector<int64_t>* out) {
  if (wire == 2) {
    Reader s = r.sub();
    while (!s.done()) out->push_back((int64_t)s.varint());
  } else if (wire == 0) {
    out->push_back((int64_t)r.varint());
  } else {
    bad("Model is invalid: repeated integer field with an unexpected wire type");
  }
}
void read_floats(Reader& r, uint32_t wire, std::vector<float>* out) {
  if (wire == 2) {
    Reader s = r.sub();
    while (!s.done()) out->push_back(as_float(s.fixed32()));
  } else if (wire == 5) {
    out->push_back(as_float(r.fixed32()));
  } else {
    bad("Model is invalid: repeated float field with an unexpected wire type");
  }
}

// ---- messages ---------------------------------------------------------------------------
// TensorProto.DataType values the reference accepts (load.rs:389-447)
enum { DT_FLOAT = 1, DT_INT32 = 6, DT_INT64 = 7, DT_BOOL = 9 };

int elem_type_of(int64_t data_type) {
  switch (data_type) {
    case DT_BOOL: return AC_BOOL;
    case DT_INT32: return AC_I32;
    case DT_INT64: return AC_I64;
    case DT_FLOAT: return AC_F32;
    default: bad("Something went wrong: Unsupported tensor element type: " + std::to_string(data_type), AC_ERR_UNSUPPORTED);
  }
}

struct TensorP {
  std::string name;
  std::vector<int64_t> dims;
  int64_t data_type = 0;
  std::vector<float> float_data;
  std::vector<int64_t> int32_data, int64_data;
  std::string raw;
  bool has_raw = false;
};

TensorP read_tensor(Reader r) {
  TensorP t;
  uint32_t f, w;
  while (r.key(&f, &w)) {
    switch (f) {
      case 1: read_ints(r, w, &t.dims); break;
      case 2: t.data_type = (int64_t)r.varint(); break;
      case 4: read_floats(r, w, &t.float_data); break;
      case 5: read_ints(r, w, &t.int32_data); break;
      case 7: read_ints(r, w, &t.int64_data); break;
      case 8: t.name = r.str(); break;
      case 9: t.raw = r.str(); t.has_raw = true; break;
      default: r.skip(w);
    }
  }
  return t;
}

// get_tensor, load.rs:389-432: typed arrays when raw_data is empty, raw bytes otherwise.
std::vector<char> tensor_bytes(const TensorP& t, int* elem_ty) {
  *elem_ty = elem_type_of(t.data_type);
  int64_t n = 1;
  for (int64_t d : t.dims) n *= d;
  const size_t es = *elem_ty == AC_BOOL ? 1 : (*elem_ty == AC_I64 ? 8 : 4);
  std::vector<char> out;
  if (!t.raw.empty() || *elem_ty == AC_BOOL) {
    out.assign(t.raw.begin(), t.raw.end());
  } else if (*elem_ty == AC_F32) {
    out.resize(t.float_data.size() * 4);
    std::memcpy(out.data(), t.float_data.data(), out.size());
  } else if (*elem_ty == AC_I64) {
    out.resize(t.int64_data.size() * 8);
    std::memcpy(out.data(), t.int64_data.data(), out.size());
  } else {
    out.resize(t.int32_data.size() * 4);
    for (size_t i = 0; i < t.int32_data.size(); ++i) {
      const int32_t v = (int32_t)t.int32_data[i];
      std::memcpy(out.data() + 4 * i, &v, 4);
    }
  }
  if (out.size() != (size_t)n * es) bad("Model is invalid: tensor '" + t.name + "' holds " + std::to_string(out.size()) +
                                        " bytes for " + std::to_string(n) + " elements");   // Tensor::verify, tensor.rs:365-367
  return out;
}

struct AttrP {
  std::string name;
  bool has_f = false, has_i = false;
  float f = 0;
  int64_t i = 0;
  std::string s;
  std::vector<float> floats;
  std::vector<int64_t> ints;
  bool has_t = false;
  TensorP t;
  bool has_g = false;
};

AttrP read_attr(Reader r) {
  AttrP a;
  uint32_t f, w;
  while (r.key(&f, &w)) {
    switch (f) {
      case 1: a.name = r.str(); break;
      case 2: a.f = as_float(r.fixed32()); a.has_f = true; break;
      case 3: a.i = (int64_t)r.varint(); a.has_i = true; break;
      case 4: a.s = r.str(); break;
      case 5: a.t = read_tensor(r.sub()); a.has_t = true; break;
      case 6: (void)r.sub(); a.has_g = true; break;
      case 7: read_floats(r, w, &a.floats); break;
      case 8: read_ints(r, w, &a.ints); break;
      default: r.skip(w);
    }
  }
  return a;
}

struct NodeP {
  std::vector<std::string> inputs, outputs;
  std::string name, op_type;
  std::vector<AttrP> attrs;
  const AttrP* find(const char* n) const {
    for (const AttrP& a : attrs)
      if (a.name == n) return &a;
    return nullptr;
  }
  const AttrP& need(const char* n) const {       // ModelLoadError::NoAttribute
    const AttrP* a = find(n);
    if (!a) bad(std::string("Attribute '") + n + "' is not specified");
    return *a;
  }
  int64_t i_or(const char* n, int64_t d) const { const AttrP* a = find(n); return a ? a->i : d; }
  float f_or(const char* n, float d) const { const AttrP* a = find(n); return a ? a->f : d; }
  std::string s_or(const char* n, const char* d) const { const AttrP* a = find(n); return a ? a->s : std::string(d); }
};

NodeP read_node(Reader r) {
  NodeP n;
  uint32_t f, w;
  while (r.key(&f, &w)) {
    switch (f) {
      case 1: n.inputs.push_back(r.str()); break;
      case 2: n.outputs.push_back(r.str()); break;
      case 3: n.name = r.str(); break;
      case 4: n.op_type = r.str(); break;
      case 5: n.attrs.push_back(read_attr(r.sub())); break;
      default: r.skip(w);
    }
  }
  return n;
}

struct ValueInfoP {
  std::string name;
  bool has_type = false, is_tensor = false, has_shape = false;
  int64_t elem_type = 0;
  std::vector<int64_t> dims;   // -1: a named (dynamic) dimension
};

ValueInfoP read_value_info(Reader r) {
  ValueInfoP v;
  uint32_t f, w;
  while (r.key(&f, &w)) {
    if (f == 1) v.name = r.str();
    else if (f == 2) {
      v.has_type = true;
      Reader ty = r.sub();
      uint32_t tf, tw;
      while (ty.key(&tf, &tw)) {
        if (tf != 1) { ty.skip(tw); continue; }     // TypeProto.tensor_type
        v.is_tensor = true;
        Reader tt = ty.sub();
        uint32_t f2, w2;
        while (tt.key(&f2, &w2)) {
          if (f2 == 1) v.elem_type = (int64_t)tt.varint();
          else if (f2 == 2) {
            v.has_shape = true;
            Reader sh = tt.sub();
            uint32_t f3, w3;
            while (sh.key(&f3, &w3)) {
              if (f3 != 1) { sh.skip(w3); continue; }
              Reader dim = sh.sub();
              int64_t val = -1;
              uint32_t f4, w4;
              while (dim.key(&f4, &w4)) {
                if (f4 == 1) val = (int64_t)dim.varint();
                else dim.skip(w4);              // dim_param: Dimension::Dynamic
              }
              v.dims.push_back(val);
            }
          } else tt.skip(w2);
        }
      }
    } else r.skip(w);
  }
  return v;
}

int pads_code(const std::string& auto_pad, const char* op) {
  if (auto_pad.empty() || auto_pad == "NOTSET") return 0;
  if (auto_pad == "SAME_UPPER") return 1;
  bad(std::string(op) + ": auto_pad " + auto_pad + " is not supported", AC_ERR_UNSUPPORTED);
}

void push_ints(std::vector<int64_t>* dst, const std::vector<int64_t>& v) { dst->insert(dst->end(), v.begin(), v.end()); }

// Operator name and attributes -> AcOp + flattened attributes (load.rs:170-361).
void convert_op(const NodeP& n, int64_t opset, MNode* out) {
  static const std::map<std::string, int> plain = {
      {"Identity", AC_OP_IDENTITY}, {"Add", AC_OP_ADD}, {"Sub", AC_OP_SUB}, {"Mul", AC_OP_MUL}, {"Div", AC_OP_DIV},
      {"Greater", AC_OP_GREATER}, {"Pow", AC_OP_POW}, {"Sqrt", AC_OP_SQRT}, {"Relu", AC_OP_RELU},
      {"Sigmoid", AC_OP_SIGMOID}, {"Erf", AC_OP_ERF}, {"Tanh", AC_OP_TANH}, {"Where", AC_OP_WHERE},
      {"Round", AC_OP_ROUND}, {"Exp", AC_OP_EXP}, {"Expand", AC_OP_EXPAND}, {"Range", AC_OP_RANGE},
      {"Tile", AC_OP_TILE}, {"Slice", AC_OP_SLICE}, {"NonMaxSuppression", AC_OP_NONMAXSUPPRESSION},
      {"Reshape", AC_OP_RESHAPE}, {"MatMul", AC_OP_MATMUL}, {"GlobalAveragePool", AC_OP_GLOBALAVERAGEPOOL},
      {"Clip", AC_OP_CLIP}};
  const std::string& t = n.op_type;
  auto it = plain.find(t);
  if (it != plain.end()) { out->op = it->second; return; }
  std::vector<int64_t>& I = out->ints;
  std::vector<float>& F = out->floats;
  if (t == "Softmax") { out->op = AC_OP_SOFTMAX; I = {n.i_or("axis", -1)}; }
  else if (t == "Split") {
    out->op = AC_OP_SPLIT;
    I = {n.i_or("axis", 0)};
    if (const AttrP* a = n.find("split")) push_ints(&I, a->ints);
  }
  else if (t == "Gather") { out->op = AC_OP_GATHER; I = {n.i_or("axis", 0)}; }
  else if (t == "Conv") {
    out->op = AC_OP_CONV2D;
    const int auto_pad = pads_code(n.s_or("auto_pad", "NOTSET"), "Conv2d");
    const std::vector<int64_t>& k = n.need("kernel_shape").ints;
    if (k.size() != 2) bad("Conv2d: kernel_shape must have two entries", AC_ERR_UNSUPPORTED);
    const AttrP* st = n.find("strides");
    const AttrP* pd = n.find("pads");
    const AttrP* dl = n.find("dilations");
    const std::vector<int64_t> strides = st ? st->ints : std::vector<int64_t>{1, 1};
    const std::vector<int64_t> pads = pd ? pd->ints : std::vector<int64_t>{0, 0};
    const std::vector<int64_t> dil = dl ? dl->ints : std::vector<int64_t>{1, 1};
    if (strides.size() != 2 || dil.size() != 2) bad("Conv2d: strides and dilations must have two entries", AC_ERR_UNSUPPORTED);
    I = {k[0], k[1], strides[0], strides[1], dil[0], dil[1], n.i_or("group", 1), auto_pad, 0, (int64_t)pads.size()};
    push_ints(&I, pads);
    F = {0.2f, 0.5f};
  }
  else if (t == "LeakyRelu") { out->op = AC_OP_LEAKYRELU; F = {n.f_or("alpha", 0.01f)}; }
  else if (t == "Resize") {
    out->op = AC_OP_RESIZE;
    I = {n.s_or("mode", "nearest") == "nearest" ? 0 : 1,
         n.s_or("coordinate_transformation_mode", "half_pixel") == "asymmetric" ? 0 : 1,
         n.s_or("nearest_mode", "round_prefer_floor") == "floor" ? 0 : 1};
  }
  else if (t == "Concat") { out->op = AC_OP_CONCAT; I = {n.need("axis").i}; }
  else if (t == "Transpose") { out->op = AC_OP_TRANSPOSE; I = n.need("perm").ints; }
  else if (t == "Squeeze") {
    out->op = AC_OP_SQUEEZE;
    if (opset < 12) I = n.need("axes").ints;
  }
  else if (t == "Unsqueeze") {
    out->op = AC_OP_UNSQUEEZE;
    if (const AttrP* a = n.find("axes")) I = a->ints;
  }
  else if (t == "ReduceMin" || t == "ReduceMax" || t == "ReduceMean") {
    out->op = t == "ReduceMin" ? AC_OP_REDUCEMIN : (t == "ReduceMax" ? AC_OP_REDUCEMAX : AC_OP_REDUCEMEAN);
    I = {n.i_or("keepdims", 1) != 0 ? 1 : 0};
    if (t == "ReduceMax") { if (const AttrP* a = n.find("axes")) push_ints(&I, a->ints); }
    else push_ints(&I, n.need("axes").ints);
  }
  else if (t == "Loop") { (void)n.need("body"); out->op = AC_OP_LOOP; }
  else if (t == "Cast") { out->op = AC_OP_CAST; I = {elem_type_of(n.need("to").i)}; }
  else if (t == "MaxPool") {
    out->op = AC_OP_MAXPOOL;
    const int auto_pad = pads_code(n.s_or("auto_pad", "NOTSET"), "MaxPool");
    const std::vector<int64_t>& k = n.need("kernel_shape").ints;
    const std::vector<int64_t>& st = n.need("strides").ints;
    const AttrP* pd = n.find("pads");
    const std::vector<int64_t> pads = pd ? pd->ints : std::vector<int64_t>{0, 0};
    if (k.size() != 2 || st.size() != 2) bad("MaxPool: kernel_shape and strides must have two entries", AC_ERR_UNSUPPORTED);
    I = {k[0], k[1], st[0], st[1], auto_pad, (int64_t)pads.size()};
    push_ints(&I, pads);
  }
  else if (t == "HardSigmoid") { out->op = AC_OP_HARDSIGMOID; F = {n.f_or("alpha", 0.2f), n.f_or("beta", 0.5f)}; }
  else if (t == "Flatten") { out->op = AC_OP_FLATTEN; I = {n.i_or("axis", 1)}; }
  else if (t == "Gemm") {
    out->op = AC_OP_GEMM;
    I = {n.i_or("transA", 0) == 1 ? 1 : 0, n.i_or("transB", 0) == 1 ? 1 : 0};
    F = {n.f_or("alpha", 1.0f), n.f_or("beta", 1.0f)};
  }
  else if (t == "BatchNormalization") { out->op = AC_OP_BATCHNORMALIZATION; F = {n.f_or("epsilon", 1e-5f)}; }
  else if (t == "LayerNormalization") {
    out->op = AC_OP_LAYERNORMALIZATION;
    I = {n.i_or("axis", -1), n.i_or("stash_type", 1)};
    F = {n.f_or("epsilon", 1e-5f)};
  }
  else if (t == "Shape") {
    out->op = AC_OP_SHAPE;
    const AttrP* e = n.find("end");
    I = {n.i_or("start", 0), e ? 1 : 0, e ? e->i : 0};
  }
  else bad("Something went wrong: Unsupported op: " + t, AC_ERR_UNSUPPORTED);
}

}  // namespace

void load_onnx_buffer(const uint8_t* buf, size_t len, AcModel& model) {
  Reader top{buf, buf + len};
  bool has_graph = false;
  Reader graph{nullptr, nullptr};
  bool have_opset = false;
  uint32_t f, w;
  while (top.key(&f, &w)) {
    if (f == 7 && w == 2) { graph = top.sub(); has_graph = true; }
    else if (f == 8 && w == 2) {                 // opset_import (load.rs:71-85)
      Reader o = top.sub();
      std::string domain;
      int64_t version = 0;
      uint32_t f2, w2;
      while (o.key(&f2, &w2)) {
        if (f2 == 1) domain = o.str();
        else if (f2 == 2) version = (int64_t)o.varint();
        else o.skip(w2);
      }
      if (domain.empty() || domain == "ai.onnx") {
        if (have_opset) bad("Model contains duplicated opsets");
        have_opset = true;
        model.opset = version;
      } else {
        bad("Something went wrong: Custom domain ('" + domain + "') not supported yet", AC_ERR_UNSUPPORTED);
      }
    } else top.skip(w);
  }
  if (!has_graph) bad("Model does not contain any graph");
  if (!have_opset) bad("Model contains duplicated opsets");   // the reference reports a missing opset this way (load.rs:86)

  std::vector<TensorP> initializers;
  std::vector<NodeP> nodes;
  std::vector<ValueInfoP> g_inputs, g_outputs;
  while (graph.key(&f, &w)) {
    if (w != 2) { graph.skip(w); continue; }
    switch (f) {
      case 1: nodes.push_back(read_node(graph.sub())); break;
      case 5: initializers.push_back(read_tensor(graph.sub())); break;
      case 11: g_inputs.push_back(read_value_info(graph.sub())); break;
      case 12: g_outputs.push_back(read_value_info(graph.sub())); break;
      default: graph.skip(w);
    }
  }

  std::map<std::string, int32_t> name_to_val;
  auto set_tensor = [&](int32_t v, const TensorP& t) {
    int ety = AC_F32;
    std::vector<char> bytes = tensor_bytes(t, &ety);
    MValue& mv = model.values[v];
    if (t.dims.size() > AC_MAX_RANK) bad("rank above 8 is not supported", AC_ERR_SHAPE);
    mv.elem_ty = ety;
    mv.rank = (int)t.dims.size();
    for (size_t i = 0; i < t.dims.size(); ++i) mv.dims[i] = t.dims[i];
    model.inits[v] = std::move(bytes);
  };
  // Initializers (load.rs:88-99)
  for (const TensorP& t : initializers) {
    auto it = name_to_val.find(t.name);
    const int32_t v = it != name_to_val.end() ? it->second : (name_to_val[t.name] = model.new_value(t.name));
    set_tensor(v, t);
  }
  // Graph inputs and outputs (load.rs:101-141)
  auto load_infos = [&](const std::vector<ValueInfoP>& infos, std::vector<int32_t>* dst) {
    for (const ValueInfoP& vi : infos) {
      if (!vi.has_type) bad("Value type is not specified");
      if (!vi.is_tensor) bad("Something went wrong: Graph input must be tensor type", AC_ERR_UNSUPPORTED);
      if (!vi.has_shape) bad("Value shape is not specified");
      auto it = name_to_val.find(vi.name);
      int32_t v;
      if (it != name_to_val.end()) v = it->second;
      else {
        v = name_to_val[vi.name] = model.new_value(vi.name);
        MValue& mv = model.values[v];
        if (vi.dims.size() > AC_MAX_RANK) bad("rank above 8 is not supported", AC_ERR_SHAPE);
        mv.elem_ty = elem_type_of(vi.elem_type);
        mv.rank = (int)vi.dims.size();
        for (size_t i = 0; i < vi.dims.size(); ++i) mv.dims[i] = vi.dims[i];
      }
      dst->push_back(v);
    }
  };
  load_infos(g_inputs, &model.inputs);
  load_infos(g_outputs, &model.outputs);
  // Initializers are not run-time inputs (load.rs:143-148)
  {
    std::vector<int32_t> kept;
    for (int32_t v : model.inputs)
      if (!model.inits.count(v)) kept.push_back(v);
    model.inputs.swap(kept);
  }
  // Nodes (load.rs:150-378)
  auto value_of = [&](const std::string& name) {
    auto it = name_to_val.find(name);
    if (it != name_to_val.end()) return it->second;
    return name_to_val[name] = model.new_value(name);
  };
  for (const NodeP& np : nodes) {
    if (np.op_type == "Constant") {
      const AttrP* a = np.find("value");
      if (!a || !a->has_t) bad("Something went wrong: Constant.value must be specified for now", AC_ERR_UNSUPPORTED);
      if (np.outputs.size() != 1) bad("Constant: one output expected");
      set_tensor(value_of(np.outputs[0]), a->t);
      continue;
    }
    MNode mn;
    mn.name = np.name;
    // An empty name is an omitted optional input; it maps to one unnamed value like any other
    // name in the reference (load.rs:152-160) and is value id -1 here.
    for (const std::string& s : np.inputs) mn.inputs.push_back(s.empty() ? -1 : value_of(s));
    for (const std::string& s : np.outputs) mn.outputs.push_back(value_of(s));
    convert_op(np, model.opset, &mn);
    model.nodes.push_back(std::move(mn));
  }
}

}  // namespace ac
