// C ABI of the CUDA session (include/altius_session_cuda.h): parse the graph
// description, infer shapes, lower to the kernel schedule, plan one device
// arena from value lifetimes, upload the weights once, capture the schedule in
// a CUDA graph and replay it per run.
//
// Replaces InterpreterSessionBuilder::build
// (crates/session_interpreter/src/builder.rs:37-65) and InterpreterSession::run
// (crates/session_interpreter/src/session.rs:66-134). Where the reference
// allocates every node output per run (`Tensor::uninit_of_type`, :159-162) and
// frees by last use (crates/session/src/plan.rs:14-58), the same last-use
// analysis here assigns fixed arena offsets at build time.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "session.h"

using namespace ac;

namespace {

thread_local std::string g_create_error;

#define AC_CUDA(expr)                                                                     \
  do {                                                                                    \
    cudaError_t e__ = (expr);                                                             \
    if (e__ != cudaSuccess)                                                               \
      fail(AC_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e__));             \
  } while (0)

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Reads a buffer twice the size of L2: afterwards L2 holds clean lines of that buffer only,
// so the next kernel's reads miss and its evictions cost no write-back.
constexpr size_t kSweepBytes = size_t(256) << 20;
__global__ void l2_sweep_kernel(const float4* __restrict__ p, size_t n4, float* sink) {
  float acc = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = __ldg(p + i);
    acc += v.x + v.y + v.z + v.w;
  }
  if (acc == 123.25f) *sink = acc;   // never true for a zeroed buffer; keeps the loads alive
}

void parse_graph(AcSession& s, const AcGraphDesc& g) {
  if (g.n_values < 0 || g.n_nodes < 0 || (g.n_values && !g.values) || (g.n_nodes && !g.nodes))
    fail(AC_ERR_INVALID, "malformed graph description");
  s.opset = g.opset_version;
  s.values.resize(g.n_values);
  for (int i = 0; i < g.n_values; ++i) {
    const AcValueDesc& d = g.values[i];
    Value& v = s.values[i];
    if (d.elem_ty < 0 || d.elem_ty > AC_I64) fail(AC_ERR_INVALID, "bad element type");
    v.elem_ty = d.elem_ty;
    v.rank = d.rank < 0 ? -1 : d.rank;
    if (d.rank > AC_MAX_RANK) fail(AC_ERR_SHAPE, "rank above 8 is not supported");
    for (int k = 0; k < v.rank; ++k) {
      if (d.dims[k] < 0) fail(AC_ERR_SHAPE, "Must be fixed dimension");  // shape.rs:675
      v.dims[k] = d.dims[k];
    }
  }
  auto check_val = [&](int v, bool allow_missing) {
    if (v == -1 && allow_missing) return;
    if (v < 0 || v >= g.n_values) fail(AC_ERR_INVALID, "value id out of range");
  };
  s.nodes.resize(g.n_nodes);
  for (int i = 0; i < g.n_nodes; ++i) {
    const AcNodeDesc& d = g.nodes[i];
    Node& n = s.nodes[i];
    if (d.op < 0 || d.op >= AC_OP_COUNT) fail(AC_ERR_INVALID, "bad operator code");
    n.op = d.op;
    for (int k = 0; k < d.n_inputs; ++k) { check_val(d.inputs[k], true); n.inputs.push_back(d.inputs[k]); }
    for (int k = 0; k < d.n_outputs; ++k) { check_val(d.outputs[k], false); n.outputs.push_back(d.outputs[k]); }
    if (n.outputs.empty()) fail(AC_ERR_INVALID, "node without outputs");
    if (d.n_ints > 0) n.ints.assign(d.ints, d.ints + d.n_ints);
    if (d.n_floats > 0) n.floats.assign(d.floats, d.floats + d.n_floats);
    if (d.name) n.name = d.name;
  }
  for (int i = 0; i < g.n_inits; ++i) {
    const AcInitDesc& d = g.inits[i];
    check_val(d.value, false);
    Value& v = s.values[d.value];
    if (v.rank < 0) fail(AC_ERR_SHAPE, "initializer without a static shape");
    if (d.bytes != v.bytes() || (!d.data && d.bytes)) fail(AC_ERR_INVALID, "initializer size mismatch");
    v.is_init = true;
    if (d.location == 0) {
      v.host = d.data;  // valid during create(); small shape tensors are kept below
      if (v.elem_ty == AC_I64 || v.numel() <= 16) {
        v.host_owned.assign(static_cast<const char*>(d.data), static_cast<const char*>(d.data) + d.bytes);
      }
    }
  }
  for (int i = 0; i < g.n_inputs; ++i) {
    check_val(g.inputs[i], false);
    if (s.values[g.inputs[i]].rank < 0) fail(AC_ERR_SHAPE, "graph input without a static shape");
    s.inputs.push_back(g.inputs[i]);
  }
  for (int i = 0; i < g.n_outputs; ++i) { check_val(g.outputs[i], false); s.outputs.push_back(g.outputs[i]); }
  if (s.outputs.empty()) fail(AC_ERR_INVALID, "graph without outputs");
}

// Lifetimes by step index, then first-fit placement of the largest buffers
// first: two storages may share bytes only if their live ranges are disjoint.
void plan_arena(AcSession& s) {
  const int nsteps = (int)s.steps.size();
  for (Storage& st : s.storages) { st.first = 1 << 30; st.last = -1; }
  auto touch = [&](int sid, int step) {
    Storage& st = s.storages[sid];
    st.first = std::min(st.first, step);
    st.last = std::max(st.last, step);
  };
  for (int i = 0; i < nsteps; ++i) {
    for (int r : s.steps[i].reads) touch(r, i);
    for (int w : s.steps[i].writes) touch(w, i);
  }
  for (const Step& st : s.init_steps) {
    for (int r : st.reads) s.storages[r].pinned_live = s.storages[r].pinned_live || !s.storages[r].weight;
    for (int w : st.writes) s.storages[w].pinned_live = true;
  }
  size_t woff = 0;
  std::vector<int> live;
  for (int i = 0; i < (int)s.storages.size(); ++i) {
    Storage& st = s.storages[i];
    if (st.weight) {
      st.offset = woff;
      woff += align_up(st.bytes, 256);
      continue;
    }
    if (st.pinned_live) { st.first = -1; st.last = nsteps; }
    if (st.last < 0) continue;  // never touched
    live.push_back(i);
  }
  s.weight_bytes = woff;
  std::sort(live.begin(), live.end(), [&](int a, int b) {
    if (s.storages[a].bytes != s.storages[b].bytes) return s.storages[a].bytes > s.storages[b].bytes;
    return a < b;
  });
  std::vector<int> placed;
  size_t top = 0;
  for (int id : live) {
    Storage& st = s.storages[id];
    const size_t need = align_up(st.bytes, 256);
    std::vector<std::pair<size_t, size_t>> busy;
    for (int o : placed) {
      const Storage& q = s.storages[o];
      if (q.first <= st.last && st.first <= q.last) busy.push_back({q.offset, q.offset + align_up(q.bytes, 256)});
    }
    std::sort(busy.begin(), busy.end());
    size_t off = 0;
    for (auto& b : busy) {
      if (off + need <= b.first) break;
      off = std::max(off, b.second);
    }
    st.offset = off;
    top = std::max(top, off + need);
    placed.push_back(id);
  }
  s.arena_bytes = std::max<size_t>(top, 256);
}

void upload_weights(AcSession& s, const AcGraphDesc& g) {
  AC_CUDA(cudaMalloc(&s.weights, std::max<size_t>(s.weight_bytes, 256)));
  for (int i = 0; i < g.n_inits; ++i) {
    const AcInitDesc& d = g.inits[i];
    if (!d.bytes) continue;
    void* dst = s.weights + s.storages[s.values[d.value].storage].offset;
    AC_CUDA(cudaMemcpyAsync(dst, d.data, d.bytes,
                            d.location == 1 ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice,
                            s.stream));
  }
  AC_CUDA(cudaStreamSynchronize(s.stream));
  // Host pointers of large initializers belong to the caller: forget them.
  for (Value& v : s.values)
    if (v.is_init) v.host = v.host_owned.empty() ? nullptr : v.host_owned.data();
}

cudaError_t replay(AcSession* s, cudaStream_t st) {
  for (Step& step : s->steps) {
    cudaError_t e = step.fn(st);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace

namespace ac {
// Lets other translation units of the library report through altius_cuda_last_error(NULL).
void set_thread_error(const std::string& msg) { g_create_error = msg; }
}  // namespace ac

namespace {

int set_err(AcSession* s, int status, const std::string& msg) {
  if (s) s->err = msg;
  else g_create_error = msg;
  return status;
}

std::unique_ptr<GraphCopy> copy_graph(const AcGraphDesc& g) {
  std::unique_ptr<GraphCopy> c(new GraphCopy());
  c->opset = g.opset_version;
  c->values.assign(g.values, g.values + g.n_values);
  c->nodes.resize(g.n_nodes);
  for (int i = 0; i < g.n_nodes; ++i) {
    const AcNodeDesc& d = g.nodes[i];
    GraphCopy::NodeCopy& n = c->nodes[i];
    n.op = d.op;
    if (d.n_inputs > 0) n.inputs.assign(d.inputs, d.inputs + d.n_inputs);
    if (d.n_outputs > 0) n.outputs.assign(d.outputs, d.outputs + d.n_outputs);
    if (d.n_ints > 0) n.ints.assign(d.ints, d.ints + d.n_ints);
    if (d.n_floats > 0) n.floats.assign(d.floats, d.floats + d.n_floats);
    n.has_name = d.name != nullptr;
    if (d.name) n.name = d.name;
  }
  if (g.n_inits > 0) c->inits.assign(g.inits, g.inits + g.n_inits);
  for (AcInitDesc& d : c->inits) d.data = nullptr;
  if (g.n_inputs > 0) c->inputs.assign(g.inputs, g.inputs + g.n_inputs);
  if (g.n_outputs > 0) c->outputs.assign(g.outputs, g.outputs + g.n_outputs);
  return c;
}

int create_session(const AcGraphDesc* graph, const AcOptions* options, AcSession** out);

// Second session on the 3xTF32 path, built from the kept description; its initializers
// are read from this session's weight blob (or the host copies of the small ones).
int create_fallback(AcSession* s) {
  if (s->fallback) return AC_OK;
  if (!s->desc) return set_err(s, AC_ERR_CUDA, "an operand exceeds the fp16 range and no fallback description was kept");
  GraphCopy& c = *s->desc;
  std::vector<AcNodeDesc> nodes(c.nodes.size());
  for (size_t i = 0; i < c.nodes.size(); ++i) {
    GraphCopy::NodeCopy& n = c.nodes[i];
    nodes[i] = AcNodeDesc{n.op, (int32_t)n.inputs.size(), n.inputs.data(), (int32_t)n.outputs.size(), n.outputs.data(),
                          (int32_t)n.ints.size(), n.ints.data(), (int32_t)n.floats.size(), n.floats.data(),
                          n.has_name ? n.name.c_str() : nullptr};
  }
  std::vector<AcInitDesc> inits = c.inits;
  for (AcInitDesc& d : inits) {
    const Value& v = s->values[d.value];
    if (!v.host_owned.empty()) { d.location = 0; d.data = v.host_owned.data(); }
    else { d.location = 1; d.data = s->ptr(d.value); }
  }
  AcGraphDesc g{};
  g.opset_version = c.opset;
  g.n_values = (int32_t)c.values.size(); g.values = c.values.data();
  g.n_nodes = (int32_t)nodes.size(); g.nodes = nodes.data();
  g.n_inits = (int32_t)inits.size(); g.inits = inits.data();
  g.n_inputs = (int32_t)c.inputs.size(); g.inputs = c.inputs.data();
  g.n_outputs = (int32_t)c.outputs.size(); g.outputs = c.outputs.data();
  AcOptions o = s->opt;
  o.gemm_mode = 3;
  const int rc = create_session(&g, &o, &s->fallback);
  if (rc != AC_OK) return set_err(s, rc, "building the 3xTF32 fallback failed: " + g_create_error);
  return AC_OK;
}

// The error word after a run: 0 fine; the range code switches to the fallback session
// (returns 1: the caller re-runs there); anything else is a kernel that gave up a wait.
int check_err_word(AcSession* s) {
  const int code = *s->err_host;
  if (code == 0) return AC_OK;
  cudaMemsetAsync(s->err_word, 0, sizeof(int), s->stream);
  cudaStreamSynchronize(s->stream);
  *s->err_host = 0;
  if (code == kGemmRangeCode && s->opt.gemm_mode == 0) {
    const int rc = create_fallback(s);
    if (rc != AC_OK) return rc;
    s->use_fallback = true;
    return 1;
  }
  return set_err(s, AC_ERR_CUDA, "a kernel gave up a bounded wait (code " + std::to_string(code) + ")");
}

int run_common(AcSession* s, const void* const* ins, void* const* outs, bool device_io) {
  if (!s) return set_err(s, AC_ERR_INVALID, "null argument");
  std::lock_guard<std::recursive_mutex> lock(s->run_mutex);
  if ((!ins && !s->inputs.empty()) || !outs) return set_err(s, AC_ERR_INVALID, "null argument");
  if (s->opt.plan_only) return set_err(s, AC_ERR_NO_DEVICE, "session was created with plan_only");
  // Every buffer is checked before anything is enqueued: an error return leaves no copy or
  // kernel in flight that could still write into the caller's memory.
  for (size_t i = 0; i < s->inputs.size(); ++i)
    if (!ins[i]) return set_err(s, AC_ERR_INVALID, "null input buffer");
  for (size_t i = 0; i < s->outputs.size(); ++i)
    if (!outs[i]) return set_err(s, AC_ERR_INVALID, "null output buffer");
  if (s->use_fallback) {
    const int rc = run_common(s->fallback, ins, outs, device_io);
    if (rc != AC_OK) s->err = s->fallback->err;
    return rc;
  }
  cudaError_t e = cudaSetDevice(s->device);
  if (e != cudaSuccess) return set_err(s, AC_ERR_CUDA, cudaGetErrorString(e));
  const cudaMemcpyKind in_kind = device_io ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
  const cudaMemcpyKind out_kind = device_io ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost;
  // An error after this point drains the stream before returning, for the same reason.
  auto fail_cuda = [&](const std::string& what, cudaError_t err) {
    cudaStreamSynchronize(s->stream);
    return set_err(s, AC_ERR_CUDA, what + cudaGetErrorString(err));
  };
  for (size_t i = 0; i < s->inputs.size(); ++i) {
    const Value& v = s->values[s->inputs[i]];
    e = cudaMemcpyAsync(s->ptr(s->inputs[i]), ins[i], v.bytes(), in_kind, s->stream);
    if (e != cudaSuccess) return fail_cuda("input copy: ", e);
  }
  if (s->opt.enable_profiling) {
    const size_t n = s->steps.size();
    for (size_t i = 0; i < n; ++i) {
      // enable_profiling 2: every step starts on a cold L2 that holds no dirty lines.
      if (s->sweep_buf) l2_sweep_kernel<<<device_sm_count() * 8, 256, 0, s->stream>>>(
          reinterpret_cast<const float4*>(s->sweep_buf), kSweepBytes / 16, reinterpret_cast<float*>(s->sweep_buf));
      cudaEventRecord(s->events[2 * i], s->stream);
      e = s->steps[i].fn(s->stream);
      if (e != cudaSuccess) return fail_cuda(s->steps[i].kind + ": ", e);
      cudaEventRecord(s->events[2 * i + 1], s->stream);
    }
  } else if (s->graph_exec) {
    e = cudaGraphLaunch(s->graph_exec, s->stream);
    if (e != cudaSuccess) return fail_cuda("graph launch: ", e);
  } else {
    e = replay(s, s->stream);
    if (e != cudaSuccess) return fail_cuda("kernel launch: ", e);
  }
  for (size_t i = 0; i < s->outputs.size(); ++i) {
    const Value& v = s->values[s->outputs[i]];
    e = cudaMemcpyAsync(outs[i], s->ptr(s->outputs[i]), v.bytes(), out_kind, s->stream);
    if (e != cudaSuccess) return fail_cuda("output copy: ", e);
  }
  cudaMemcpyAsync(s->err_host, s->err_word, sizeof(int), cudaMemcpyDeviceToHost, s->stream);
  e = cudaStreamSynchronize(s->stream);
  if (e != cudaSuccess) return set_err(s, AC_ERR_CUDA, std::string("run: ") + cudaGetErrorString(e));
  if (const int rc = check_err_word(s)) return rc == 1 ? run_common(s, ins, outs, device_io) : rc;
  if (s->opt.enable_profiling) {
    for (size_t i = 0; i < s->steps.size(); ++i) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, s->events[2 * i], s->events[2 * i + 1]);
      ProfileAcc& acc = s->profile[s->steps[i].kind];
      acc.launches += s->steps[i].launches;
      acc.ms += ms;
      acc.bytes += s->steps[i].bytes;
      acc.flops += s->steps[i].flops;
    }
  }
  return AC_OK;
}

}  // namespace

extern "C" {

int altius_cuda_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return -AC_ERR_NO_DEVICE;
  return n;
}

}  // extern "C"

namespace {
int create_session(const AcGraphDesc* graph, const AcOptions* options, AcSession** out) {
  if (!graph || !out) return set_err(nullptr, AC_ERR_INVALID, "null argument");
  *out = nullptr;
  AcSession* s = new AcSession();
  try {
    if (options) s->opt = *options;
    s->device = s->opt.device;
    if (s->opt.plan_only) {
      parse_graph(*s, *graph);
      infer_shapes(*s);
      lower_graph(*s);
      plan_arena(*s);
      *out = s;
      return AC_OK;
    }
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
      fail(AC_ERR_NO_DEVICE, "no CUDA device is visible: this backend has no CPU fallback");
    if (s->device < 0 || s->device >= ndev) fail(AC_ERR_NO_DEVICE, "device ordinal out of range");
    cudaDeviceProp prop;
    AC_CUDA(cudaGetDeviceProperties(&prop, s->device));
    if (prop.major != 10)
      fail(AC_ERR_NO_DEVICE, "device is not sm_100 (the kernels are built for sm_100a only)");
    AC_CUDA(cudaSetDevice(s->device));
    AC_CUDA(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
    AC_CUDA(cudaMalloc(&s->err_word, sizeof(int)));
    AC_CUDA(cudaMemset(s->err_word, 0, sizeof(int)));
    AC_CUDA(cudaHostAlloc(&s->err_host, sizeof(int), cudaHostAllocDefault));
    *s->err_host = 0;
    parse_graph(*s, *graph);
    infer_shapes(*s);
    lower_graph(*s);
    plan_arena(*s);
    AC_CUDA(cudaMalloc(&s->arena, s->arena_bytes));
    upload_weights(*s, *graph);
    for (Step& st : s->init_steps) AC_CUDA(st.fn(s->stream));
    AC_CUDA(cudaStreamSynchronize(s->stream));
    AC_CUDA(cudaMemcpy(s->err_host, s->err_word, sizeof(int), cudaMemcpyDeviceToHost));
    if (*s->err_host == kGemmRangeCode) fail(-kGemmRangeCode, "a constant operand exceeds the fp16 range");
    if (*s->err_host != 0) fail(AC_ERR_CUDA, "a kernel gave up a bounded wait while preparing constants");
    if (s->opt.gemm_mode == 0) s->desc = copy_graph(*graph);
    if (s->opt.enable_profiling) {
      s->events.resize(2 * s->steps.size());
      for (cudaEvent_t& ev : s->events) AC_CUDA(cudaEventCreate(&ev));
      if (s->opt.enable_profiling == 2) {
        AC_CUDA(cudaMalloc(&s->sweep_buf, kSweepBytes));
        AC_CUDA(cudaMemset(s->sweep_buf, 0, kSweepBytes));
      }
    } else if (!s->opt.disable_cuda_graph && !s->steps.empty()) {
      AC_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
      cudaError_t e = replay(s, s->stream);
      cudaError_t e2 = cudaStreamEndCapture(s->stream, &s->graph);
      if (e != cudaSuccess) fail(AC_ERR_CUDA, std::string("capture: ") + cudaGetErrorString(e));
      AC_CUDA(e2);
      AC_CUDA(cudaGraphInstantiate(&s->graph_exec, s->graph, 0));
    }
  } catch (const BuildError& e) {
    set_err(nullptr, e.status, e.msg);
    altius_cuda_destroy(s);
    return e.status;
  } catch (const std::exception& e) {
    set_err(nullptr, AC_ERR_INVALID, e.what());
    altius_cuda_destroy(s);
    return AC_ERR_INVALID;
  }
  *out = s;
  return AC_OK;
}
}  // namespace

extern "C" {

int altius_cuda_create(const AcGraphDesc* graph, const AcOptions* options, AcSession** out) {
  int rc = create_session(graph, options, out);
  if (rc == -kGemmRangeCode) {
    // A weight does not fit the fp16 split: lower everything on the 3xTF32 path instead.
    AcOptions o{};
    if (options) o = *options;
    o.gemm_mode = 3;
    rc = create_session(graph, &o, out);
  }
  return rc;
}

int altius_cuda_run(AcSession* s, const void* const* ins, void* const* outs) {
  return run_common(s, ins, outs, false);
}

int altius_cuda_run_device(AcSession* s, const void* const* d_ins, void* const* d_outs) {
  return run_common(s, d_ins, d_outs, true);
}

int altius_cuda_run_batches(AcSession* s, int32_t n_batches, const void* const* ins, void* const* outs) {
  if (!s) return set_err(s, AC_ERR_INVALID, "bad argument");
  std::lock_guard<std::recursive_mutex> lock(s->run_mutex);
  if (n_batches < 0 || (!ins && !s->inputs.empty() && n_batches) || (!outs && n_batches))
    return set_err(s, AC_ERR_INVALID, "bad argument");
  if (s->opt.plan_only) return set_err(s, AC_ERR_NO_DEVICE, "session was created with plan_only");
  const size_t ni = s->inputs.size(), no = s->outputs.size();
  // All buffers of all batches are checked before the first copy is enqueued.
  for (size_t i = 0; i < (size_t)n_batches * ni; ++i)
    if (!ins[i]) return set_err(s, AC_ERR_INVALID, "null input buffer");
  for (size_t i = 0; i < (size_t)n_batches * no; ++i)
    if (!outs[i]) return set_err(s, AC_ERR_INVALID, "null output buffer");
  // Sessions that profile, or that have switched to their fallback plan, take the plain path.
  if (s->opt.enable_profiling || s->use_fallback || n_batches < 2) {
    for (int b = 0; b < n_batches; ++b) {
      const int rc = run_common(s, ins + (size_t)b * ni, outs + (size_t)b * no, false);
      if (rc != AC_OK) return rc;
    }
    return AC_OK;
  }
  cudaError_t e = cudaSetDevice(s->device);
  if (e == cudaSuccess && !s->copy_stream) {
    e = cudaStreamCreateWithFlags(&s->copy_stream, cudaStreamNonBlocking);
    for (int k = 0; k < 2 && e == cudaSuccess; ++k) {
      s->staging[k].assign(ni, nullptr);
      for (size_t i = 0; i < ni && e == cudaSuccess; ++i)
        e = cudaMalloc(&s->staging[k][i], std::max<size_t>(s->values[s->inputs[i]].bytes(), 16));
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->staged[k], cudaEventDisableTiming);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->consumed[k], cudaEventDisableTiming);
    }
  }
  for (int b = 0; b < n_batches && e == cudaSuccess; ++b) {
    const int k = b & 1;
    // copy stream: inputs of batch b into staging set k (free again once batch b-2 has left it)
    if (b >= 2) e = cudaStreamWaitEvent(s->copy_stream, s->consumed[k], 0);
    for (size_t i = 0; i < ni && e == cudaSuccess; ++i) {
      const void* src = ins[(size_t)b * ni + i];
      e = cudaMemcpyAsync(s->staging[k][i], src, s->values[s->inputs[i]].bytes(), cudaMemcpyHostToDevice, s->copy_stream);
    }
    if (e == cudaSuccess) e = cudaEventRecord(s->staged[k], s->copy_stream);
    // compute stream: staging -> arena (device copy), schedule, outputs to the host
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s->stream, s->staged[k], 0);
    for (size_t i = 0; i < ni && e == cudaSuccess; ++i)
      e = cudaMemcpyAsync(s->ptr(s->inputs[i]), s->staging[k][i], s->values[s->inputs[i]].bytes(),
                          cudaMemcpyDeviceToDevice, s->stream);
    if (e == cudaSuccess) e = cudaEventRecord(s->consumed[k], s->stream);
    if (e == cudaSuccess) e = s->graph_exec ? cudaGraphLaunch(s->graph_exec, s->stream) : replay(s, s->stream);
    for (size_t i = 0; i < no && e == cudaSuccess; ++i) {
      void* dst = outs[(size_t)b * no + i];
      e = cudaMemcpyAsync(dst, s->ptr(s->outputs[i]), s->values[s->outputs[i]].bytes(), cudaMemcpyDeviceToHost, s->stream);
    }
  }
  if (e == cudaSuccess) e = cudaMemcpyAsync(s->err_host, s->err_word, sizeof(int), cudaMemcpyDeviceToHost, s->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s->stream);
  if (e != cudaSuccess) {
    // Whatever was enqueued before the failure finishes before the caller gets its buffers back.
    if (s->copy_stream) cudaStreamSynchronize(s->copy_stream);
    cudaStreamSynchronize(s->stream);
    return set_err(s, AC_ERR_CUDA, std::string("run_batches: ") + cudaGetErrorString(e));
  }
  if (const int rc = check_err_word(s))   // out of fp16 range somewhere: all batches again on the fallback plan
    return rc == 1 ? altius_cuda_run_batches(s, n_batches, ins, outs) : rc;
  return AC_OK;
}

int altius_cuda_time_device_runs(AcSession* s, const void* const* d_ins, void* const* d_outs,
                                 int32_t iters, float* elapsed_ms) {
  if (!s) return set_err(s, AC_ERR_INVALID, "bad argument");
  std::lock_guard<std::recursive_mutex> lock(s->run_mutex);
  if (!elapsed_ms || iters <= 0 || !d_outs || (!d_ins && !s->inputs.empty()))
    return set_err(s, AC_ERR_INVALID, "bad argument");
  if (s->opt.plan_only) return set_err(s, AC_ERR_NO_DEVICE, "session was created with plan_only");
  if (s->opt.enable_profiling) return set_err(s, AC_ERR_INVALID, "not available on a profiling session");
  for (size_t i = 0; i < s->inputs.size(); ++i)
    if (!d_ins[i]) return set_err(s, AC_ERR_INVALID, "null input buffer");
  for (size_t i = 0; i < s->outputs.size(); ++i)
    if (!d_outs[i]) return set_err(s, AC_ERR_INVALID, "null output buffer");
  if (s->use_fallback) {
    const int rc = altius_cuda_time_device_runs(s->fallback, d_ins, d_outs, iters, elapsed_ms);
    if (rc != AC_OK) s->err = s->fallback->err;
    return rc;
  }
  cudaError_t e = cudaSetDevice(s->device);
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  if (e == cudaSuccess) e = cudaEventCreate(&t0);
  if (e == cudaSuccess) e = cudaEventCreate(&t1);
  if (e == cudaSuccess) e = cudaEventRecord(t0, s->stream);
  for (int it = 0; it < iters && e == cudaSuccess; ++it) {
    for (size_t i = 0; i < s->inputs.size() && e == cudaSuccess; ++i)
      e = cudaMemcpyAsync(s->ptr(s->inputs[i]), d_ins[i], s->values[s->inputs[i]].bytes(),
                          cudaMemcpyDeviceToDevice, s->stream);
    if (e == cudaSuccess) e = s->graph_exec ? cudaGraphLaunch(s->graph_exec, s->stream) : replay(s, s->stream);
    for (size_t i = 0; i < s->outputs.size() && e == cudaSuccess; ++i)
      e = cudaMemcpyAsync(d_outs[i], s->ptr(s->outputs[i]), s->values[s->outputs[i]].bytes(),
                          cudaMemcpyDeviceToDevice, s->stream);
  }
  if (e == cudaSuccess) e = cudaEventRecord(t1, s->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(s->err_host, s->err_word, sizeof(int), cudaMemcpyDeviceToHost, s->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s->stream);
  if (e == cudaSuccess && *s->err_host != 0) {
    if (t0) cudaEventDestroy(t0);
    if (t1) cudaEventDestroy(t1);
    const int rc = check_err_word(s);
    return rc == 1 ? altius_cuda_time_device_runs(s, d_ins, d_outs, iters, elapsed_ms) : rc;
  }
  if (e == cudaSuccess) e = cudaEventElapsedTime(elapsed_ms, t0, t1);
  if (t0) cudaEventDestroy(t0);
  if (t1) cudaEventDestroy(t1);
  if (e != cudaSuccess) return set_err(s, AC_ERR_CUDA, std::string("timed runs: ") + cudaGetErrorString(e));
  return AC_OK;
}

int altius_cuda_num_inputs(const AcSession* s) { return s ? (int)s->inputs.size() : -AC_ERR_INVALID; }
int altius_cuda_num_outputs(const AcSession* s) { return s ? (int)s->outputs.size() : -AC_ERR_INVALID; }
int altius_cuda_input_value(const AcSession* s, int32_t i) {
  return (s && i >= 0 && i < (int)s->inputs.size()) ? s->inputs[i] : -AC_ERR_INVALID;
}
int altius_cuda_output_value(const AcSession* s, int32_t i) {
  return (s && i >= 0 && i < (int)s->outputs.size()) ? s->outputs[i] : -AC_ERR_INVALID;
}

int altius_cuda_value_info(const AcSession* s, int32_t value, AcValueDesc* out) {
  if (!s || !out || value < 0 || value >= (int)s->values.size()) return AC_ERR_INVALID;
  const Value& v = s->values[value];
  out->elem_ty = v.elem_ty;
  out->rank = v.rank;
  for (int i = 0; i < AC_MAX_RANK; ++i) out->dims[i] = i < v.rank ? v.dims[i] : 0;
  return AC_OK;
}

int64_t altius_cuda_launches_per_run(const AcSession* s) {
  if (s && s->use_fallback) s = s->fallback;
  return s ? s->launches_per_run : -1;
}
uint64_t altius_cuda_arena_bytes(const AcSession* s) {
  if (s && s->use_fallback) s = s->fallback;
  return s ? s->arena_bytes : 0;
}

int altius_cuda_profile(AcSession* s, AcProfileEntry* entries, size_t* n) {
  if (s && s->use_fallback) s = s->fallback;
  if (!s || !n) return AC_ERR_INVALID;
  const size_t cap = *n;
  size_t i = 0;
  for (auto& kv : s->profile) {
    if (entries && i < cap) {
      AcProfileEntry& e = entries[i];
      std::memset(&e, 0, sizeof(e));
      std::snprintf(e.name, sizeof(e.name), "%s", kv.first.c_str());
      e.launches = kv.second.launches;
      e.total_ms = kv.second.ms;
      e.bytes = kv.second.bytes;
      e.flops = kv.second.flops;
    }
    ++i;
  }
  *n = i;
  return AC_OK;
}

int altius_cuda_schedule(const AcSession* s, AcProfileEntry* entries, size_t* n) {
  if (s && s->use_fallback) s = s->fallback;
  if (!s || !n) return AC_ERR_INVALID;
  const size_t cap = *n;
  for (size_t i = 0; i < s->steps.size() && entries && i < cap; ++i) {
    AcProfileEntry& e = entries[i];
    std::memset(&e, 0, sizeof(e));
    std::snprintf(e.name, sizeof(e.name), "%s", s->steps[i].kind.c_str());
    e.launches = s->steps[i].launches;
    e.bytes = s->steps[i].bytes;
    e.flops = s->steps[i].flops;
  }
  *n = s->steps.size();
  return AC_OK;
}

int altius_cuda_profile_reset(AcSession* s) {
  if (s && s->use_fallback) s = s->fallback;
  if (!s) return AC_ERR_INVALID;
  s->profile.clear();
  return AC_OK;
}

const char* altius_cuda_last_error(const AcSession* s) {
  return s ? s->err.c_str() : g_create_error.c_str();
}

void altius_cuda_destroy(AcSession* s) {
  if (!s) return;
  if (s->fallback) altius_cuda_destroy(s->fallback);
  if (s->stream) cudaSetDevice(s->device);
  if (s->graph_exec) cudaGraphExecDestroy(s->graph_exec);
  if (s->graph) cudaGraphDestroy(s->graph);
  for (cudaEvent_t ev : s->events)
    if (ev) cudaEventDestroy(ev);
  if (s->err_word) cudaFree(s->err_word);
  if (s->sweep_buf) cudaFree(s->sweep_buf);
  for (int k = 0; k < 2; ++k) {
    for (void* p : s->staging[k])
      if (p) cudaFree(p);
    if (s->staged[k]) cudaEventDestroy(s->staged[k]);
    if (s->consumed[k]) cudaEventDestroy(s->consumed[k]);
  }
  if (s->copy_stream) cudaStreamDestroy(s->copy_stream);
  if (s->err_host) cudaFreeHost(s->err_host);
  if (s->arena) cudaFree(s->arena);
  if (s->weights) cudaFree(s->weights);
  if (s->stream) cudaStreamDestroy(s->stream);
  delete s;
}

int altius_cuda_host_alloc(size_t bytes, void** out) {
  if (!out) return AC_ERR_INVALID;
  cudaError_t e = cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault);
  if (e != cudaSuccess) return set_err(nullptr, AC_ERR_CUDA, cudaGetErrorString(e));
  return AC_OK;
}

int altius_cuda_host_free(void* p) {
  if (!p) return AC_OK;
  return cudaFreeHost(p) == cudaSuccess ? AC_OK : AC_ERR_CUDA;
}

}  // extern "C"
