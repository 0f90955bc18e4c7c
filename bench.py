"""Benchmark of the session hot path: ViT-B/16 forward passes, 32 images per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE for N > 1).
A step is one forward pass of ViT-B/16 (f32, batch 32 per GPU) over a synthetic
~N(0,1) input with seeded ~N(0,0.02) weights. Rank 0 prints one JSON line:

  value   images/s, whole job, inputs already resident in HBM, timed with CUDA
          events on the session's stream (max over ranks);
  e2e     images/s through the public API with page-locked HOST buffers: the H2D
          copy of every step's images and the D2H copy of its logits are inside the
          timed region. `CudaSession.run_batches` (a queue of batches: the copy of
          step i+1 overlaps the kernels of step i); `e2e.sync_run` is the same with
          one synchronous `CudaSession.run` per step;
  roofline  the dominant kernel (the GEMM) from a per-kernel CUDA-event profile
          taken in the same process, against the measured tensor peak;
  hbm_kernels  the tensor-op micrograph (B=64) kernels' achieved GB/s against
          the measured copy bandwidth -- the second half of the metric;
  cpu_baseline  the CPU oracle (a port of the reference interpreter) timed on
          the host cores on a bounded sample of the same workload.

`--impl reference` times that CPU port instead (the reference itself is Rust
and cannot be built offline), all host threads, same metric and config.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PER_GPU_BATCH = 32
WORKLOAD = "ViT-B/16 224x224 f32 forward, batch 32 per GPU (197 tokens, dim 768, 12 layers, 12 heads)"
VIT_GFLOP_PER_IMAGE = 35.13


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "50"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def host_threads():
    """All host cores this process may use (torchrun presets OMP_NUM_THREADS=1, so the
    OpenMP default cannot be trusted); also lifts numpy's BLAS pool to that count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=n)
    except Exception:
        pass
    return n


def time_cpu_port(target_seconds=12.0, batch=2, max_runs=50):
    """The CPU oracle on a bounded sample: forward passes of ViT-B/16 at a small
    batch, repeated for about `target_seconds`; all host threads; OpenBLAS sgemm
    (numpy's) standing in for the reference's BLIS."""
    from altius_b200 import configs
    from oracle import InterpreterSessionBuilder
    threads = host_threads()
    model, feeds = configs.vit_base_16(batch=batch)
    sess = (InterpreterSessionBuilder(model).with_intra_op_num_threads(threads)
            .with_sgemm("openblas").build())
    x = list(feeds.values())
    sess.run(x)  # warm-up
    t0 = time.perf_counter()
    runs = 0
    while runs < max_runs:
        sess.run(x)
        runs += 1
        if time.perf_counter() - t0 >= target_seconds:
            break
    dt = time.perf_counter() - t0
    return dict(value=batch * runs / dt, unit="images/s", cores=threads, kind="port",
                sample=f"{runs} forward passes of ViT-B/16 at batch {batch} in {dt:.1f} s; "
                       f"oracle port of the interpreter, OpenBLAS sgemm, {threads} threads"), dt / runs


def reference_arm(args, rank):
    if rank != 0:
        return
    batch = 2
    from altius_b200 import configs
    from oracle import InterpreterSessionBuilder
    threads = host_threads()
    model, feeds = configs.vit_base_16(batch=batch)
    sess = (InterpreterSessionBuilder(model).with_intra_op_num_threads(threads)
            .with_sgemm("openblas").build())
    x = list(feeds.values())
    for _ in range(args.warmup):
        sess.run(x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sess.run(x)
    dt = time.perf_counter() - t0
    value = batch * args.steps / dt
    line = {
        "impl": "reference", "metric": "ViT-B/16 images/s", "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample_per_step": f"{batch} images on the host CPU"},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": threads, "kind": "port",
                         "sample": f"each step = ViT-B/16 forward at batch {batch}; CPU oracle port of "
                                   f"the reference interpreter (the Rust reference cannot be built "
                                   f"offline), OpenBLAS sgemm, {threads} threads"},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def micrograph_hbm(device, peaks):
    """Per-kernel achieved HBM GB/s on the tensor-op micrograph at B=64. L2 is swept before
    every kernel (a 256 MB read), so each is timed cold and without another kernel's dirty
    lines to write back."""
    from altius_b200 import configs
    from altius_b200.session import CudaSessionBuilder
    import torch
    model, feeds = configs.micrograph(batch=64)
    out = {}
    for fuse in (True, False):
        sess = (CudaSessionBuilder(model).with_device(device).with_fusion(fuse)
                .with_profiling_enabled(True, cold_l2=True).build())
        ins = [torch.from_numpy(v).to(f"cuda:{device}") for v in feeds.values()]
        outs = [torch.empty(tuple(shape), dtype=torch.float32, device=f"cuda:{device}")
                for shape, _ in sess.output_info]
        torch.cuda.synchronize(device)
        for it in range(8):
            if it == 3:
                sess.profile_reset()
            sess.run_device([t.data_ptr() for t in ins], [t.data_ptr() for t in outs])
        for kind, p in sess.profile().items():
            n = p["launches"]
            gbs = p["bytes"] / (p["total_ms"] * 1e-3) / 1e9
            out[("fused:" if fuse else "unfused:") + kind] = {
                "us": round(1e3 * p["total_ms"] / max(n, 1), 2), "MB": round(p["bytes"] / max(n, 1) / 1e6, 2),
                "GBps": round(gbs, 1), "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 3)}
        sess.close()
        del ins, outs
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gemm-mode", type=int, default=0)
    ap.add_argument("--gemm-pairs", type=int, default=0, help="AcOptions.gemm_pairs (0 default, 3: the one-CTA GEMM kernel only)")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-micrograph", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist
    from altius_b200 import configs, replicas
    from altius_b200.session import CudaSessionBuilder, alloc_pinned

    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(dev))

    peaks = measured_peaks()

    # Every rank builds the same graph; rank 0's weights are broadcast once.
    model, _ = configs.vit_base_16(batch=PER_GPU_BATCH, seed=0)
    builder = CudaSessionBuilder(model).with_device(local_rank).with_gemm_mode(args.gemm_mode).with_gemm_pairs(args.gemm_pairs)
    blob = None
    if distributed:
        blob, ptrs = replicas.broadcast_weights(model, dev, src=0)
        builder = builder.with_device_initializers(ptrs)
    sess = builder.build()
    del blob

    # This rank's shard of the global batch (seeded per rank).
    rng = np.random.default_rng(1000 + rank)
    x_host = alloc_pinned((PER_GPU_BATCH, 3, 224, 224))
    x_host[...] = rng.standard_normal(x_host.shape, dtype=np.float32)
    y_host = alloc_pinned((PER_GPU_BATCH, 1000))
    x_dev = torch.from_numpy(np.ascontiguousarray(x_host)).to(dev)
    y_dev = torch.empty((PER_GPU_BATCH, 1000), dtype=torch.float32, device=dev)
    in_ptrs, out_ptrs = [x_dev.data_ptr()], [y_dev.data_ptr()]

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v):
        if not distributed:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident throughput ("value") -------------------------------------
    for _ in range(args.warmup):
        sess.run_device(in_ptrs, out_ptrs)
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.4)                      # let nvidia-smi start sampling
    sess.run_device(in_ptrs, out_ptrs)   # and put the GPU under load before the first sample counts
    barrier()
    n_before = len(sampler.lines)
    ms = sess.time_device_runs(in_ptrs, out_ptrs, args.steps)
    barrier()
    sampler.lines = sampler.lines[max(n_before - 1, 0):] if len(sampler.lines) > n_before else sampler.lines[-2:]
    clocks = sampler.stop()
    ms = max_over_ranks(ms)
    value = world * PER_GPU_BATCH * args.steps / (ms * 1e-3)

    # ---- end to end through the public API with host buffers ("e2e") ----------------
    # `run_batches` is the call for a queue of batches: the host->device copy of step i+1
    # overlaps the kernels of step i (every step's 19.3 MB H2D and 128 KB D2H are inside the
    # timed region); the one-batch-at-a-time `run` is timed beside it.
    for _ in range(3):
        sess.run([x_host], outputs=[y_host])
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sess.run([x_host], outputs=[y_host])
    sync_s = time.perf_counter() - t0
    barrier()
    e2e_sync = world * PER_GPU_BATCH * args.steps / max_over_ranks(sync_s)
    queue_in = [[x_host]] * args.steps
    queue_out = [[y_host]] * args.steps
    sess.run_batches(queue_in[:3], outputs=queue_out[:3])
    barrier()
    t0 = time.perf_counter()
    sess.run_batches(queue_in, outputs=queue_out)
    e2e_s = time.perf_counter() - t0
    barrier()
    e2e_s = max_over_ranks(e2e_s)
    e2e = world * PER_GPU_BATCH * args.steps / e2e_s
    logits = np.array(y_host)
    launches = sess.launches_per_run * args.steps * world
    sess.close()

    if rank != 0:
        if distributed:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- per-kernel profile of the same workload (rank 0) ---------------------------
    prof_sess = (CudaSessionBuilder(model).with_device(local_rank).with_gemm_mode(args.gemm_mode).with_gemm_pairs(args.gemm_pairs)
                 .with_profiling_enabled(True).build())
    for it in range(6):
        if it == 2:
            prof_sess.profile_reset()
        prof_sess.run_device(in_ptrs, out_ptrs)
    prof = prof_sess.profile()
    prof_sess.close()
    total_ms = sum(p["total_ms"] for p in prof.values())
    kernels = {k: {"share": round(p["total_ms"] / total_ms, 4),
                   "ms_per_step": round(p["total_ms"] / 4, 4),
                   "launches_per_step": p["launches"] // 4}
               for k, p in sorted(prof.items(), key=lambda kv: -kv[1]["total_ms"])}
    top = max(prof.items(), key=lambda kv: kv[1]["total_ms"])
    top_kind, tp = top
    if tp["flops"] > 0:
        achieved = tp["flops"] / (tp["total_ms"] * 1e-3) / 1e12
        # The fp16-split kernel issues fp16 MMAs (the rate of the measured bf16 GEMM), the TF32
        # kernels run at half of it; both spend three MMAs per product, so `frac` tops out at 1/3.
        f16 = "f16" in top_kind
        peak = peaks["bf16_tflops_sustained"] / (1.0 if f16 else 2.0)
        roofline = {"kernel": top_kind, "bound": "tensor", "achieved": round(achieved, 2),
                    "peak": round(peak, 1), "unit": "TFLOP/s", "frac": round(achieved / peak, 4),
                    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at the
                    # QKV shape (M 6304, K 768, N 2304; algorithmic operand + result bytes 84.6 MB, of
                    # which A, B and most of C stay in L2), from the ncu capture summarised in
                    # profiles/gemm_f16x3_6304x768x2304.md
                    "traffic": 50155264 if f16 else None,
                    "tensor_pipe_frac": round(3.0 * achieved / peak, 4),
                    "peak_note": f"{peaks['source']} sustained bf16 cuBLAS TFLOP/s"
                                 + ("" if f16 else " / 2 (no TF32 peak is measured)")
                                 + "; achieved = algorithmic 2*M*N*K FLOPs / CUDA-event time; the kernel "
                                   "issues three MMAs per product for fp32 fidelity, so frac tops out at "
                                   "1/3 and tensor_pipe_frac = 3 * frac is the share of the tensor peak in use"}
    else:
        achieved = tp["bytes"] / (tp["total_ms"] * 1e-3) / 1e9
        roofline = {"kernel": top_kind, "bound": "hbm", "achieved": round(achieved, 1),
                    "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                    "traffic": None, "peak_note": f"{peaks['source']} copy bandwidth"}

    line = {
        "metric": "ViT-B/16 images/s", "value": round(value, 2), "unit": "images/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": world * PER_GPU_BATCH,
                   "parallelism": f"{world} batch-sharded replica(s), no per-inference collective",
                   "l2": "working set per step (346 MB of weights + activations) is larger than the 126 MB L2",
                   "gemm_mode": args.gemm_mode},
        "e2e": {"value": round(e2e, 2), "unit": "images/s",
                "h2d_bytes_per_step": int(x_host.nbytes), "d2h_bytes_per_step": int(y_host.nbytes),
                "api": "CudaSession.run_batches (pipelined queue of batches)", "sync_run": round(e2e_sync, 2)},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
        "algorithmic_tflops_whole_step": round(VIT_GFLOP_PER_IMAGE * value / 1e3, 2),
        "kernels": kernels,
        "logits_checksum": float(np.abs(logits).sum()),
    }
    if not args.skip_micrograph:
        line["hbm_kernels"] = micrograph_hbm(local_rank, peaks)
    if world == 1 and not args.skip_cpu_baseline:
        line["cpu_baseline"], _ = time_cpu_port()
    print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
