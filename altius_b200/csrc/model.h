// The graph a session is built from, as a mutable host-side object: what the ONNX loader
// produces and the graph passes rewrite. Mirrors `Model { graph, opset_version }` and
// `Graph { nodes, values, inits, inputs, outputs }` of the reference
// (crates/core/src/model.rs:13-17, crates/core/src/graph.rs:10-16); operators and
// attributes are kept in the flattened form of AcNodeDesc (include/altius_session_cuda.h).
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "../../include/altius_session_cuda.h"

namespace ac {

struct MValue {
  std::string name;          // empty: unnamed
  int elem_ty = AC_F32;
  int rank = -1;             // -1: shape unknown; a dim of -1: dynamic (crates/core/src/dim.rs)
  int64_t dims[AC_MAX_RANK] = {0};
};

struct MNode {
  int op = 0;
  std::string name;
  std::vector<int32_t> inputs, outputs;   // value ids; -1: absent optional input
  std::vector<int64_t> ints;
  std::vector<float> floats;
  bool deleted = false;
};

}  // namespace ac

struct AcModel {
  int64_t opset = 0;
  std::vector<ac::MValue> values;
  std::vector<ac::MNode> nodes;
  std::map<int32_t, std::vector<char>> inits;     // value id -> bytes
  std::vector<int32_t> inputs, outputs;

  // Storage behind the AcGraphDesc view handed out by altius_model_graph().
  std::vector<AcValueDesc> v_values;
  std::vector<AcNodeDesc> v_nodes;
  std::vector<AcInitDesc> v_inits;

  int32_t new_value(const std::string& name = std::string()) {
    ac::MValue v;
    v.name = name;
    values.push_back(v);
    return (int32_t)values.size() - 1;
  }
};

namespace ac {

struct ModelError {
  int status;
  std::string msg;
};

// crates/core/src/model.rs:30-102
std::map<int32_t, std::vector<int>> value_users(const AcModel& m);
std::map<int32_t, int> value_parents(const AcModel& m);
std::vector<int> topo_sort_nodes(const AcModel& m);
void remove_unnecessary_nodes(AcModel& m);

// crates/core/src/onnx/load.rs:55-445
void load_onnx_buffer(const uint8_t* buf, size_t len, AcModel& out);

// crates/core/src/optimize/{layer_norm_fusion,gelu_fusion,fast_gelu_fusion,identity_elim}.rs;
// each returns the number of rewrites.
int fuse_layer_norm(AcModel& m);
int fuse_gelu(AcModel& m);
int fuse_fast_gelu(AcModel& m);
int eliminate_identity(AcModel& m);

}  // namespace ac
