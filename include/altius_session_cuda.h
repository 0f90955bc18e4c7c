/*
 * altius_session_cuda -- C ABI of the B200 (sm_100a) execution backend.
 *
 * This is the boundary a Rust `crates/session_cuda` (or any FFI caller) binds.
 * It replaces, for the CUDA backend, what the reference's backends expose as
 *
 *   XSessionBuilder::new(model).with_profiling_enabled(b).build()
 *       crates/session_interpreter/src/builder.rs:18-65
 *   XSession::run(&self, Vec<Tensor>) -> Result<Vec<Tensor>, SessionError>
 *       crates/session_interpreter/src/session.rs:66-134
 *       trait Session, crates/session/src/lib.rs:43-45
 *
 * and follows the shape of the one C ABI the reference already has, the
 * generated `model.so` of session_clang: `initialize()` once, then
 * `trampoline(const void **ins, const void **outs)` per inference with
 * caller-owned, shape-fixed buffers
 * (crates/session_clang/src/translator.rs:441-444, :499-503;
 *  crates/session_clang/src/session.rs:32-56).
 *
 * All types are plain C; no CUDA or C++ types cross the boundary. Every
 * function returns 0 on success and a non-zero AcStatus otherwise; the message
 * is available from altius_cuda_last_error(). Nothing aborts or throws across
 * the ABI. Unsupported operators or shapes are rejected by
 * altius_cuda_create(), never in the middle of a run.
 */
#ifndef ALTIUS_SESSION_CUDA_H
#define ALTIUS_SESSION_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define AC_MAX_RANK 8

typedef enum AcStatus {
  AC_OK = 0,
  AC_ERR_INVALID = 1,     /* null pointer, bad id, malformed description        */
  AC_ERR_SHAPE = 2,       /* shape inference failed (SessionError::Shape)        */
  AC_ERR_UNSUPPORTED = 3, /* operator / pattern without a kernel                 */
  AC_ERR_CUDA = 4,        /* a CUDA runtime call failed                          */
  AC_ERR_NO_DEVICE = 5    /* no usable sm_100 device                             */
} AcStatus;

/* Element types: TensorElemType, crates/core/src/tensor.rs:47-53 */
typedef enum AcElemType { AC_BOOL = 0, AC_F32 = 1, AC_I32 = 2, AC_I64 = 3 } AcElemType;

/* Operator codes, in the order of `enum Op`, crates/core/src/op.rs:8-58 */
typedef enum AcOp {
  AC_OP_IDENTITY = 0, AC_OP_CONV2D, AC_OP_ADD, AC_OP_SUB, AC_OP_MUL, AC_OP_DIV, AC_OP_POW,
  AC_OP_GREATER, AC_OP_SQRT, AC_OP_RELU, AC_OP_GELU, AC_OP_LEAKYRELU, AC_OP_SIGMOID, AC_OP_ERF,
  AC_OP_TANH, AC_OP_CLIP, AC_OP_WHERE, AC_OP_SOFTMAX, AC_OP_CAST, AC_OP_MAXPOOL,
  AC_OP_GLOBALAVERAGEPOOL, AC_OP_RESHAPE, AC_OP_FLATTEN, AC_OP_RESIZE, AC_OP_CONCAT,
  AC_OP_TRANSPOSE, AC_OP_SQUEEZE, AC_OP_UNSQUEEZE, AC_OP_REDUCEMIN, AC_OP_REDUCEMAX,
  AC_OP_REDUCEMEAN, AC_OP_ROUND, AC_OP_EXP, AC_OP_EXPAND, AC_OP_RANGE, AC_OP_LOOP, AC_OP_TILE,
  AC_OP_SPLIT, AC_OP_SLICE, AC_OP_GATHER, AC_OP_SHAPE, AC_OP_NONMAXSUPPRESSION, AC_OP_MATMUL,
  AC_OP_GEMM, AC_OP_BATCHNORMALIZATION, AC_OP_LAYERNORMALIZATION, AC_OP_HARDSIGMOID,
  AC_OP_CONSTANT, AC_OP_FUSEDELEMWISE, AC_OP_COUNT
} AcOp;

/* A value of the graph (crates/core/src/value.rs). rank < 0: shape unknown, to
 * be inferred. Graph inputs and initializers must carry static shapes. */
typedef struct AcValueDesc {
  int32_t elem_ty;            /* AcElemType */
  int32_t rank;
  int64_t dims[AC_MAX_RANK];
} AcValueDesc;

/* A node (crates/core/src/node.rs:8-14). Attributes are flattened into an
 * integer and a float array, laid out per operator as follows
 * (fields of the structs in crates/core/src/op.rs:60-211):
 *
 *   CONV2D   ints  = kh, kw, sh, sw, dh, dw, group, auto_pad (0 none / NOTSET,
 *                    1 SAME_UPPER), activation (0 none, 1 Relu, 2 HardSigmoid),
 *                    npads (0, 2 or 4), pads[npads] (top, left[, bottom, right])
 *            floats = activation alpha, activation beta
 *   MAXPOOL  ints  = kh, kw, sh, sw, auto_pad, npads, pads[npads]
 *   HARDSIGMOID floats = alpha, beta      LEAKYRELU floats = alpha
 *   RESIZE   ints = mode (0 nearest, 1 anything else: bilinear, as the interpreter),
 *                   coordinate_transformation_mode (0 asymmetric, 1 other),
 *                   nearest_mode (0 floor, 1 other)
 *   SOFTMAX  ints = axis                  FLATTEN ints = axis
 *   CAST     ints = to (AcElemType)       CONCAT  ints = axis
 *   TRANSPOSE ints = perm[rank]           GATHER  ints = axis
 *   SQUEEZE / UNSQUEEZE ints = axes[]     (opset >= 13: taken from input 1)
 *   REDUCEMAX / REDUCEMEAN ints = keep_dims, axes[]
 *   SPLIT    ints = axis, split[]         (opset >= 13: sizes from input 1)
 *   GEMM     ints = trans_a, trans_b;  floats = alpha, beta
 *   BATCHNORMALIZATION floats = epsilon
 *   LAYERNORMALIZATION ints = axis, stash_type;  floats = epsilon
 *   SHAPE    ints = start, has_end, end   (may be absent: start 0, no end)
 *
 * An absent optional input is value id -1. */
typedef struct AcNodeDesc {
  int32_t op;                /* AcOp */
  int32_t n_inputs;
  const int32_t *inputs;
  int32_t n_outputs;
  const int32_t *outputs;
  int32_t n_ints;
  const int64_t *ints;
  int32_t n_floats;
  const float *floats;
  const char *name;          /* may be NULL */
} AcNodeDesc;

/* An initializer (Graph::inits, crates/core/src/graph.rs:13). `location` 0:
 * `data` is host memory, copied to the device once by create(). 1: `data` is
 * already memory of the session's device (e.g. the landing buffer of an NCCL
 * broadcast); it is copied device-to-device and not referenced afterwards.
 * Shape-like initializers (Reshape shapes, Slice starts, Split sizes, Gather
 * indices) are read on the host and must use location 0. */
typedef struct AcInitDesc {
  int32_t value;
  int32_t location;
  const void *data;
  uint64_t bytes;
} AcInitDesc;

/* A direct serialisation of `Model` (crates/core/src/model.rs:13-17) after
 * altius's fusion passes. `inputs` are the run-time inputs in positional order
 * (initializers are not listed, as after crates/core/src/onnx/load.rs:144-148). */
typedef struct AcGraphDesc {
  int64_t opset_version;
  int32_t n_values;
  const AcValueDesc *values;
  int32_t n_nodes;
  const AcNodeDesc *nodes;
  int32_t n_inits;
  const AcInitDesc *inits;
  int32_t n_inputs;
  const int32_t *inputs;
  int32_t n_outputs;
  const int32_t *outputs;
} AcGraphDesc;

/* Builder options (InterpreterSessionBuilder fields,
 * crates/session_interpreter/src/builder.rs:12-16; intra_op_num_threads has no
 * meaning on a GPU and is not carried). Zero-initialise for defaults. */
typedef struct AcOptions {
  int32_t device;            /* CUDA device ordinal                               */
  int32_t enable_profiling;  /* 1: time every kernel with CUDA events; 2: same, and
                                sweep L2 before each kernel (cold, clean cache)    */
  int32_t disable_cuda_graph;/* 1: launch kernels one by one instead of a graph   */
  int32_t disable_fusion;    /* 1: one kernel per node, no producer/consumer folds*/
  int32_t gemm_mode;         /* 0 auto (tcgen05: fp16-split products for constant
                                weights, 3xTF32 otherwise, where shapes allow),
                                1 CUDA-core fp32 FMA only, 2 tcgen05 1xTF32,
                                3 tcgen05 3xTF32 only                             */
  int32_t plan_only;         /* 1: infer shapes, lower and plan the arena without
                                touching a GPU; run() then fails. For inspecting
                                the schedule on a machine without a device.      */
  int32_t gemm_pairs;        /* fp16-split GEMMs of 256 x 256 tiles on clusters of two CTAs
                                (tcgen05 .cta_group::2, each SM stages its rows of A and half
                                of the weight tile). 0 (default) and 2: where the cost model
                                prefers them, with A arriving already split into fp16 halves
                                (written by the kernel that produced it, or by a split kernel
                                in front) so that every tile comes by TMA; 1: pairs that split
                                A in registers; 3: never (the one-CTA kernel). Same results. */
  int32_t reserved;
} AcOptions;

typedef struct AcSession AcSession;

/* One line of the per-kernel profile: what `enable_profiling` logs per op name
 * in the reference (crates/session_interpreter/src/session.rs:118-125,251-255),
 * here per kernel kind, with the algorithmic work used for roofline figures. */
typedef struct AcProfileEntry {
  char name[48];             /* kernel kind, e.g. "layer_norm", "gemm_tf32x3"    */
  uint64_t launches;         /* launches accumulated since the last reset        */
  double total_ms;           /* device time, CUDA events on the session's stream */
  double bytes;              /* algorithmic bytes moved by those launches        */
  double flops;              /* algorithmic FLOPs (2*MACs) of those launches     */
} AcProfileEntry;

/* builder.build(): shape inference, lowering to a static kernel schedule, one
 * device arena sized from the inferred shapes, weights copied to the device.
 * Replaces InterpreterSessionBuilder::build, builder.rs:37-65. */
int altius_cuda_create(const AcGraphDesc *graph, const AcOptions *options, AcSession **out);

/* session.run(inputs): `ins[i]` / `outs[i]` are caller-owned HOST buffers of
 * the i-th graph input / output, sized by their (inferred) shapes. Copies
 * inputs to the device, replays the schedule, copies outputs back, and returns
 * after the outputs are complete. The run calls of one session (run, run_device,
 * run_batches, time_device_runs) are serialised by a lock inside the session. Replaces
 * InterpreterSession::run, session.rs:66-134, in the calling convention of
 * session_clang's trampoline, translator.rs:499-503. */
int altius_cuda_run(AcSession *s, const void *const *ins, void *const *outs);

/* Same, with DEVICE buffers on the session's device (inputs already resident
 * in HBM); returns after the work is complete. */
int altius_cuda_run_device(AcSession *s, const void *const *d_ins, void *const *d_outs);

/* `n_batches` independent runs from HOST buffers, pipelined: `ins` holds n_batches *
 * num_inputs pointers (batch-major), `outs` n_batches * num_outputs. The inputs of batch
 * b+1 travel to the device (second stream, double-buffered staging) while batch b
 * computes; outputs are complete on return. The buffers should be page-locked
 * (altius_cuda_host_alloc), otherwise the copies do not overlap. Results are those of
 * n_batches calls of altius_cuda_run. The reference has no counterpart (its run() is
 * synchronous CPU code, session.rs:66-134); a caller with a queue of batches uses this
 * to keep the copy engines and the SMs busy at the same time. */
int altius_cuda_run_batches(AcSession *s, int32_t n_batches, const void *const *ins, void *const *outs);

/* `iters` back-to-back runs with device buffers, timed on the device: CUDA
 * events recorded on the session's stream before the first and after the last
 * run; *elapsed_ms receives the time between them. For measurement harnesses
 * (the reference's counterpart is the `Instant` pair around run(),
 * session.rs:68,123). */
int altius_cuda_time_device_runs(AcSession *s, const void *const *d_ins, void *const *d_outs,
                                 int32_t iters, float *elapsed_ms);

/* session.model() surrogate (session.rs:62-64): static facts of the built
 * session. altius_cuda_value_info fills the inferred type and shape of any
 * value id of the graph description (crates/core/src/analysis/shape.rs:659-692). */
int altius_cuda_num_inputs(const AcSession *s);
int altius_cuda_num_outputs(const AcSession *s);
int altius_cuda_input_value(const AcSession *s, int32_t i);
int altius_cuda_output_value(const AcSession *s, int32_t i);
int altius_cuda_value_info(const AcSession *s, int32_t value, AcValueDesc *out);

/* Kernel launches one run() issues, and the bytes of the device arena. */
int64_t altius_cuda_launches_per_run(const AcSession *s);
uint64_t altius_cuda_arena_bytes(const AcSession *s);

/* The static kernel schedule, one entry per step in launch order (total_ms is
 * 0). On entry *n is the capacity of `entries`; on return the number of steps. */
int altius_cuda_schedule(const AcSession *s, AcProfileEntry *entries, size_t *n);

/* Profile accumulated by runs of a session created with enable_profiling.
 * On entry *n is the capacity of `entries`; on return the number of kinds.
 * Replaces the `Profile: {...}` log of session.rs:118-125. */
int altius_cuda_profile(AcSession *s, AcProfileEntry *entries, size_t *n);
int altius_cuda_profile_reset(AcSession *s);

/* Message of the last failure on this session (or, with s == NULL, of the last
 * failed altius_cuda_create on this thread). Stands in for SessionError's
 * Display, crates/session/src/lib.rs:14-34. */
const char *altius_cuda_last_error(const AcSession *s);

void altius_cuda_destroy(AcSession *s);

/* Page-locked host buffers for callers that want run()'s copies to overlap and
 * run at full PCIe rate. (The reference has no counterpart: its tensors never
 * leave host memory.) */
int altius_cuda_host_alloc(size_t bytes, void **out);
int altius_cuda_host_free(void *p);

/* Maximum of `n` f32 values at device address `d_x`, written to the device float
 * `d_out`, enqueued on `stream` (a cudaStream_t passed as void*, NULL = the
 * default stream) of the current device. It has no counterpart in the reference
 * (whose reductions run inside a session on host memory). It exists for callers
 * that must not allocate device memory when they need the value -- real-time or
 * callback code that cannot take cudaMalloc's synchronisation, plug-ins without a
 * pool of their own, code between allocation-free checkpoints: unlike a session
 * it calls no cudaMalloc / cudaFree or other allocating routine. Its partial
 * results live in a fixed 64 KB array inside the library's device image, which
 * limits `n` to 67,108,864 elements (larger `n`: AC_ERR_INVALID with a message
 * from altius_cuda_last_error(NULL)) and is shared by every call on that GPU, so
 * calls that can overlap on one GPU must be serialised by the caller. The first
 * call on each device also looks up the array's device address; make that call
 * before starting any stream capture. */
int altius_cuda_reduce_max_noalloc(const float *d_x, int64_t n, float *d_out, void *stream);

/* Number of visible CUDA devices, or a negative AcStatus. */
int altius_cuda_device_count(void);

/* ---- the model object: loader and graph passes (host only) ------------------------------
 * `Model` of the reference (crates/core/src/model.rs:13-17) as an opaque handle. */
typedef struct AcModel AcModel;

/* altius_core::onnx::load_onnx / load_onnx_from_buffer (crates/core/src/onnx/load.rs:55-64):
 * operator table, attribute defaults and initializer types (f32 / i32 / i64 / bool, raw_data
 * or typed arrays) as there (:170-361, :389-432); initializers are removed from the graph
 * inputs (:143-148). A dynamic dimension of a graph input is loaded as -1 (and refused by
 * altius_cuda_create, as shape inference refuses it in the reference). Additions: a Constant
 * node becomes an initializer of its output value. Errors: AC_ERR_INVALID / AC_ERR_UNSUPPORTED
 * with ModelLoadError's message from altius_cuda_last_error(NULL). */
int altius_model_load_onnx(const char *path, AcModel **out);
int altius_model_load_onnx_buffer(const void *buf, size_t len, AcModel **out);

/* A model from a graph description (initializers are copied; they must be host memory). */
int altius_model_from_graph(const AcGraphDesc *graph, AcModel **out);

/* One graph pass; *n_rewrites (may be NULL) receives the number of patterns rewritten.
 * pass 0 fuse_layer_norm     crates/core/src/optimize/layer_norm_fusion.rs:13-123
 *      1 fuse_gelu           crates/core/src/optimize/gelu_fusion.rs:12-131
 *      2 fuse_fast_gelu      crates/core/src/optimize/fast_gelu_fusion.rs:5-190
 *      3 eliminate_identity  crates/core/src/optimize/identity_elim.rs:5-45 */
int altius_model_run_pass(AcModel *m, int32_t pass, int32_t *n_rewrites);
/* The four passes in the order altius_py runs them before it builds a session
 * (crates/altius_py/src/lib.rs:54-62). */
int altius_model_optimize(AcModel *m);

/* The model as a graph description for altius_cuda_create. The pointers in *out belong to
 * the model and stay valid until it is modified or destroyed. */
int altius_model_graph(AcModel *m, AcGraphDesc *out);
/* Name of a value (NULL: unnamed), and Model::lookup_named_value (-1: not found). */
const char *altius_model_value_name(const AcModel *m, int32_t value);
int32_t altius_model_lookup_named_value(const AcModel *m, const char *name);
void altius_model_destroy(AcModel *m);

/* load_onnx + the passes + builder.build() in one call: what
 * `altius_py.InferenceSession(path, backend=...)` does (crates/altius_py/src/lib.rs:32-88). */
int altius_cuda_create_from_onnx(const char *path, const AcOptions *options, AcSession **out);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* ALTIUS_SESSION_CUDA_H */
