// Host side of the CUDA session: graph description -> shapes -> static kernel
// schedule -> device arena -> replay. Internal header shared by the scheduler
// translation units; the public surface is include/altius_session_cuda.h.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/altius_session_cuda.h"
#include "kernels.h"

namespace ac {

struct Value {
  int elem_ty = AC_F32;
  int rank = -1;                 // -1: unknown
  int64_t dims[AC_MAX_RANK] = {0};
  bool is_init = false;
  bool is_const = false;         // initializer or computed from initializers only
  const void* host = nullptr;    // host copy (initializers and host-evaluated shape tensors)
  std::vector<char> host_owned;  // backing store when the session made the host copy
  int storage = -1;              // index into Session::storages
  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= dims[i];
    return n;
  }
  size_t elem_bytes() const { return elem_ty == AC_BOOL ? 1 : (elem_ty == AC_I64 ? 8 : 4); }
  size_t bytes() const { return (size_t)numel() * elem_bytes(); }
};

struct Node {
  int op = 0;
  std::vector<int> inputs, outputs;
  std::vector<int64_t> ints;
  std::vector<float> floats;
  std::string name;
};

struct Storage {
  size_t bytes = 0;
  int first = 1 << 30;   // first step touching it
  int last = -1;         // last step touching it
  bool weight = false;   // lives in the weight blob, not the arena
  bool pinned_live = false;  // graph input/output or constant: live for the whole run
  size_t offset = 0;     // byte offset inside its region
};

struct Step {
  std::string kind;      // kernel kind, the key of the profile
  int op = 0;            // AcOp of the anchoring node (for messages)
  std::function<cudaError_t(cudaStream_t)> fn;
  std::vector<int> reads, writes;  // storage ids
  double bytes = 0, flops = 0;     // algorithmic work
  int launches = 1;
  bool const_only = false;         // all inputs constant: executed once at create()
};

struct ProfileAcc {
  uint64_t launches = 0;
  double ms = 0, bytes = 0, flops = 0;
};

}  // namespace ac

namespace ac {
// What create() keeps of the caller's graph description (everything but the initializer
// payloads) so that the session can be lowered a second time with other options.
struct GraphCopy {
  struct NodeCopy {
    int32_t op;
    std::vector<int32_t> inputs, outputs;
    std::vector<int64_t> ints;
    std::vector<float> floats;
    std::string name;
    bool has_name;
  };
  int64_t opset;
  std::vector<AcValueDesc> values;
  std::vector<NodeCopy> nodes;
  std::vector<AcInitDesc> inits;      // data pointers are filled in when the copy is used
  std::vector<int32_t> inputs, outputs;
};
}  // namespace ac

struct AcSession {
  int device = 0;
  AcOptions opt{};
  int64_t opset = 13;
  std::deque<ac::Value> values;        // a deque: lowering appends scratch values while it holds references
  std::vector<ac::Node> nodes;
  std::vector<int> inputs, outputs;
  std::vector<int> order;              // topological order of node ids
  std::vector<ac::Storage> storages;
  std::vector<ac::Step> steps;         // per-run schedule
  std::vector<ac::Step> init_steps;    // constant-only steps, run once
  char* arena = nullptr;
  size_t arena_bytes = 0;
  char* weights = nullptr;
  size_t weight_bytes = 0;
  int* err_word = nullptr;             // device word written by kernels whose bounded waits expire
  int* err_host = nullptr;             // page-locked mirror
  cudaStream_t stream = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  std::vector<cudaEvent_t> events;     // profiling: a start and a stop event per step
  char* sweep_buf = nullptr;           // enable_profiling 2: buffer read before each step to clear L2
  std::map<std::string, ac::ProfileAcc> profile;
  int64_t launches_per_run = 0;
  std::string err;
  // gemm_mode 0 only: when an operand of an fp16-split GEMM turns out not to fit fp16,
  // a second session lowered with gemm_mode 3 (3xTF32) takes over for good.
  // run_batches: second stream, two sets of device staging buffers for the inputs, events
  cudaStream_t copy_stream = nullptr;
  std::vector<void*> staging[2];
  cudaEvent_t staged[2] = {nullptr, nullptr};    // H2D of a staging set has landed
  cudaEvent_t consumed[2] = {nullptr, nullptr};  // the set has been copied into the arena
  std::unique_ptr<ac::GraphCopy> desc;
  AcSession* fallback = nullptr;
  bool use_fallback = false;
  // run / run_device / run_batches / time_device_runs share the arena, the staging buffers, the
  // error word and the fallback switch: one caller at a time per session (recursive: a run
  // re-enters itself once when it switches to the fallback plan).
  std::recursive_mutex run_mutex;

  void* ptr(int value) const {
    const ac::Storage& st = storages[values[value].storage];
    return (st.weight ? weights : arena) + st.offset;
  }
  const float* fptr(int value) const { return static_cast<const float*>(ptr(value)); }
  float* fptr_mut(int value) const { return static_cast<float*>(ptr(value)); }
};

namespace ac {
// Thrown inside create(); turned into a status + message at the ABI.
struct BuildError {
  int status;
  std::string msg;
};
[[noreturn]] void fail(int status, const std::string& msg);

const char* op_name(int op);       // shapes.cpp
// Resolves the four pads (top, left, bottom, right) of a Conv2d / MaxPool node.
void resolve_pads(Node& n, int auto_pad_pos, int64_t ih, int64_t iw, int64_t pads[4]);
void infer_shapes(AcSession& s);   // shapes.cpp
void lower_graph(AcSession& s);    // lower.cpp
}  // namespace ac
