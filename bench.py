"""Benchmark of the data-parallel MLP training step and of the kernels under it.

    python bench.py --gpus N --steps K --warmup W            # the CUDA backend, one rank per GPU
    python bench.py --impl reference --gpus N --steps K ...  # the reference-shaped CPU path
    python bench.py --case gemm --m 65536 --k 4096 --n 4096  # one kernel case alone (also the ncu workloads)

Workload of the headline line: 784 -> 4096 -> 4096 -> 4096 -> 10 Linear/ReLU classifier, softmax
cross-entropy, Adam (1e-3, 0.9, 0.999, 1e-8), global batch 65536 split evenly over the ranks,
gradients sum-allreduced with NCCL over NVLink overlapped with the backward pass, FP32 (GEMMs in 3xTF32
on tcgen05).  Synthetic seeded data: x ~ U(0,1), labels ~ U{0..9}, Glorot-uniform weights, zero biases.
The batch is a function of the global row index alone, so every number of ranks trains on the same
65536 rows; `config.final_loss` and `config.parameter_checksums` are therefore comparable across N.

One JSON line is printed by rank 0.  `value` times K steps with the batch already resident in HBM;
`e2e` times K steps through the same C-ABI calls with the batch uploaded from pinned host memory
and the loss read back every step.  Further records on the same line: `inference` (the same network,
forward and row arg-max, 8192 rows per GPU, weights replicated, no collective), `kernels` (the
standalone dense layer and classifier-head cases, one GPU only), `tf32_peak` (a cuBLAS TF32 GEMM timed
in this run, the direct denominator of the 3xTF32 roofline), `cpu_baseline`.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DIMS = [784, 4096, 4096, 4096, 10]
GLOBAL_BATCH = 65536
INFERENCE_ROWS_PER_GPU = 8192
ADAM = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)
METRIC = "mlp_train_samples_per_s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
DATA_BLOCK = 1024       # rows per independently seeded block of the synthetic batch

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch of the two-SM 3xTF32 kernel, mean over
# the eight launches of one training step, from two ncu captures of exactly these launches: at 8192 rows per
# GPU (this build) and at 65536 rows (the same main loop and tile order).  The weight planes are read once per
# group of row bands whatever the batch, so traffic does not grow in proportion to the rows; other row counts
# are interpolated between the two captures.
NCU_GEMM_TRAFFIC = {8192: 9.912e9 / 8, 65536: (66.31e9 + 14.58e9) / 8}
# FP32 operands read once, results written once and the hi / lo planes that four of the launches write for the
# products that read their results, per launch (mean over the same eight launches)
ALGORITHMIC_GEMM_BYTES = {8192: (2.628e9 + 1.074e9) / 8, 65536: (28.7e9 + 8.59e9) / 8}
TENSOR_FLOP_PER_CLOCK_PER_SM = 4096.0       # dense TF32 multiply-add throughput of one SM's tensor pipe (2048 FMA per clock)
SM_COUNT = 148


def interpolate_rows(table, rows):
    (r0, v0), (r1, v1) = sorted(table.items())
    return v0 + (rows - r0) * (v1 - v0) / (r1 - r0)


def step_flops(batch: int) -> float:
    """Algorithmic FLOPs of one training step: forward 2*B*P, backward 4*B*P minus the input gradient."""
    weights = sum(DIMS[i] * DIMS[i + 1] for i in range(len(DIMS) - 1))
    return 6.0 * batch * weights - 2.0 * batch * DIMS[0] * DIMS[1]


def forward_flops(batch: int) -> float:
    return 2.0 * batch * sum(DIMS[i] * DIMS[i + 1] for i in range(len(DIMS) - 1))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def synthetic_rows(first_row: int, rows: int, seed: int = 1234):
    """Rows [first_row, first_row + rows) of the synthetic batch.  Each block of DATA_BLOCK rows has its
    own generator keyed by (seed, block index), so a row's values depend on its global index only and
    not on how the batch is cut into ranks."""
    if first_row % DATA_BLOCK or rows % DATA_BLOCK:
        raise ValueError(f"rank slices must be multiples of {DATA_BLOCK} rows")
    x = np.empty((rows, DIMS[0]), dtype=np.float32)
    labels = np.empty(rows, dtype=np.int32)
    for i in range(rows // DATA_BLOCK):
        rng = np.random.default_rng([seed, first_row // DATA_BLOCK + i])
        x[i * DATA_BLOCK:(i + 1) * DATA_BLOCK] = rng.random((DATA_BLOCK, DIMS[0]), dtype=np.float32)
        labels[i * DATA_BLOCK:(i + 1) * DATA_BLOCK] = rng.integers(0, DIMS[-1], DATA_BLOCK)
    return x, labels


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int, period_ms: int = 200):
        self.device_index = device_index
        self.period_ms = period_ms
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)], stdout=subprocess.PIPE, text=True)
        except OSError:
            self.proc = None
            return self
        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        return self

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxes, powers, reasons = [], [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1])); maxes.append(float(parts[2])); powers.append(float(parts[3]))
            except ValueError:
                continue
            for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        loaded = [c for c, p in zip(clocks, powers) if p >= 0.5 * max(powers)] or clocks
        return {"sm_mhz": float(np.median(loaded)), "sm_max_mhz": max(maxes), "power_w_max": max(powers),
                "samples": len(clocks), "reasons": sorted(reasons)}


def at_equal_clock(ms: float, clocks) -> float | None:
    """Duration x median SM MHz: a clock-independent figure (kilo-cycles) for comparing runs whose boxes
    settled at different clocks."""
    if not clocks or not clocks.get("sm_mhz"):
        return None
    return ms * clocks["sm_mhz"]


def cpu_baseline(threads: int, rows: int, steps: int = 1, warmup: int = 0):
    """Times the reference-shaped CPU training step on `rows` samples of the same workload: `warmup`
    untimed steps, then the median of `steps` timed ones."""
    from oracle import oracle
    blas = oracle.baseline_bind_openblas()
    rng = np.random.default_rng(7)
    weights = [rng.uniform(-1, 1, (DIMS[i + 1], DIMS[i])).astype(np.float32) * np.float32(np.sqrt(6.0 / (DIMS[i] + DIMS[i + 1])))
               for i in range(len(DIMS) - 1)]
    biases = [np.zeros(DIMS[i + 1], dtype=np.float32) for i in range(len(DIMS) - 1)]
    m1 = [np.zeros(a.size, dtype=np.float32) for pair in zip(weights, biases) for a in pair]
    m2 = [np.zeros(a.size, dtype=np.float32) for pair in zip(weights, biases) for a in pair]
    x, labels = synthetic_rows(0, rows)
    seconds = []
    for step in range(warmup + steps):
        s, _, _ = oracle.baseline_mlp_step(DIMS, x, labels, weights, biases, m1, m2, train=True, count_total=GLOBAL_BATCH,
                                           adam_step=step + 1, threads=threads, **{"lr": ADAM["lr"], "beta1": ADAM["beta1"],
                                                                                    "beta2": ADAM["beta2"], "eps": ADAM["eps"]})
        if step >= warmup:
            seconds.append(s)
    return rows / float(np.median(seconds)), blas, float(np.median(seconds))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    rows = 2048
    value, blas, seconds = cpu_baseline(threads, rows, steps=max(args.steps, 1), warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": seconds * 1e3 * GLOBAL_BATCH / rows, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "mlp_784_4096x3_10_softmax_ce_adam_train", "global_batch": GLOBAL_BATCH,
                   "note": "reference-shaped CPU step (OpenBLAS sgemm as the reference calls it + scalar loops) on a row sample; ms_per_step scaled to the global batch"},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": threads, "kind": "port",
                         "sample": f"{rows} of {GLOBAL_BATCH} rows per step, median of {max(args.steps, 1)} timed steps after {args.warmup} warm-up, BLAS: {os.path.basename(blas)}"},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def measure_tf32_peak(device_index: int):
    """A cuBLAS TF32 GEMM (torch.matmul on FP32 operands with TF32 allowed, 8192^3) timed here: best of
    ten single launches (burst) and back to back for about four seconds (sustained, under the power cap),
    with the clocks seen during the sustained run.  A library GEMM as the yardstick of the tensor-core
    roofline; nothing in the product path calls it."""
    import torch
    n = 8192
    before = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(n, n, device="cuda", dtype=torch.float32)
        b = torch.randn(n, n, device="cuda", dtype=torch.float32)
        c = torch.empty(n, n, device="cuda", dtype=torch.float32)
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        flops = 2.0 * n ** 3
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch.matmul(a, b, out=c); e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        sampler = ClockSampler(device_index).start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches = 0
        wall = time.perf_counter()
        e0.record()
        while time.perf_counter() - wall < 4.0:
            for _ in range(50):
                torch.matmul(a, b, out=c)
            launches += 50
            torch.cuda.synchronize()
        e1.record(); torch.cuda.synchronize()
        sustained_ms = e0.elapsed_time(e1) / launches
        clocks = sampler.stop()
        del a, b, c
        torch.cuda.empty_cache()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = before
    return {"burst_tflops": flops / (best * 1e-3) / 1e12, "sustained_tflops": flops / (sustained_ms * 1e-3) / 1e12,
            "how": "torch.matmul FP32 operands, TF32 allowed, 8192^3: best of 10 (burst), back to back for 4 s (sustained)", "clocks": clocks}


def run_cuda(args):
    import torch
    import torch.distributed as dist
    from synaptik_b200 import native, nn

    global_batch = args.global_batch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    ctx = native.Context(local_rank)
    # experiment hook: SYNAPTIK_BENCH_OPTIONS="gemm_dynamic=0,gemm_slices=0" sets context options before the
    # executable is created (the defaults are what the numbers in the repository were measured with)
    for item in filter(None, os.environ.get("SYNAPTIK_BENCH_OPTIONS", "").split(",")):
        name, _, value = item.partition("=")
        ctx.set_option(name.strip(), int(value))
    comm = None
    if distributed:
        holder = [native.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(holder, src=0)
        comm = native.Comm(ctx, world, rank, holder[0])
    rows = global_batch // world
    model = nn.Model(DIMS, ctx, seed=42, comm=comm, world_size=world)       # same seed: replicas start identical
    model.configure_training("ce", nn.Adam(ADAM["lr"], ADAM["beta1"], ADAM["beta2"], ADAM["eps"]))
    exe, xbuf, tbuf, seed, loss, grads = model.training_state(rows)
    inputs, outputs = [xbuf, tbuf, seed] + model.param_buffers, [loss] + grads
    x_host = native.PinnedArray((rows, DIMS[0]), np.float32)
    t_host = native.PinnedArray((rows,), np.int32)
    loss_host = native.PinnedArray((1,), np.float32)
    x, labels = synthetic_rows(rank * rows, rows)           # this rank's slice of the one global batch
    x_host.array[...] = x
    t_host.array[...] = labels
    xbuf.upload(x)
    tbuf.upload(labels)
    optimizer = model._optimizer

    def barrier():
        ctx.synchronize()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    # experiment hook: SYNAPTIK_BENCH_OCCUPY="blocks,microseconds" puts a co-tenant on the communication stream
    # at the start of every resident step (blocks that each hold one SM for that long, as a collective's do)
    cotenant = [int(v) for v in os.environ.get("SYNAPTIK_BENCH_OCCUPY", "0,0").split(",")]

    def resident_step():
        if cotenant[0] > 0:
            ctx.occupy(cotenant[0], cotenant[1])
        exe.enqueue(inputs, outputs)
        optimizer.step_enqueue(grads)

    # end to end: two sets of input buffers; while step i computes, the batch of step i + 1 is copied
    # from pinned host memory on the context's copy stream.  Every step's batch is copied inside the
    # timed region and every step ends with the loss read back on the host.
    input_sets = [(xbuf, tbuf), (ctx.buffer(x_host.nbytes), ctx.buffer(t_host.nbytes))]

    def prefetch(step_index: int):
        xb, tb = input_sets[step_index & 1]
        xb.prefetch(x_host.pointer, x_host.nbytes)
        tb.prefetch(t_host.pointer, t_host.nbytes)

    def e2e_steps(count: int):
        prefetch(0)
        for i in range(count):
            if i + 1 < count:
                prefetch(i + 1)
            xb, tb = input_sets[i & 1]
            exe.enqueue([xb, tb, seed] + model.param_buffers, outputs)
            optimizer.step_enqueue(grads)
            loss.download_async(loss_host.pointer, 4)
            optimizer.finish()                  # one wait per step: the objective and the context's error word (run and update)

    def reduce_max(value: float) -> float:
        if not distributed:
            return value
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_mean(value: float) -> float:
        if not distributed:
            return value
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item()) / world

    for _ in range(max(args.warmup, 3)):
        resident_step()
    exe.finish(); optimizer.finish()

    # ---- device-resident timing ----------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    ctx.timer_start()
    for _ in range(args.steps):
        resident_step()
    resident_ms = ctx.timer_stop()
    barrier()
    exe.finish(); optimizer.finish()
    # per-kernel times: two more steps with a CUDA-event pair around every plan step (outside the timed
    # region, whose steps run without them)
    ctx.set_option("time_steps", 1)
    for _ in range(2):
        resident_step()
    exe.finish(); optimizer.finish()
    step_ms = exe.step_timings_ms()
    plan = exe.describe().strip().split("\n")
    ctx.set_option("time_steps", 0)
    launches_per_step = exe.launch_count() + 1
    resident_ms = reduce_max(resident_ms)

    # ---- end to end ------------------------------------------------------------------------------
    e2e_steps(2)
    barrier()
    ctx.timer_start()
    wall = time.perf_counter()
    e2e_steps(args.steps)
    e2e_ms = ctx.timer_stop()
    wall = (time.perf_counter() - wall) * 1e3
    barrier()
    exe.finish(); optimizer.finish()
    clocks = sampler.stop() if rank == 0 else None
    e2e_ms = reduce_max(max(e2e_ms, wall))
    total_steps = max(args.warmup, 3) + 2 * args.steps + 4
    # the objective of the last step over the WHOLE batch (mean of the ranks' equal-sized means), and a
    # checksum of every parameter tensor after the last step: the same for every N up to the rounding of
    # the gradient sums
    final_loss = reduce_mean(float(loss_host.array[0]))
    parameters = model.parameters()
    checksums = [[float(np.sum(p, dtype=np.float64)), float(np.sum(np.square(p, dtype=np.float64)))] for p in parameters]
    replicas_identical = True
    if distributed:
        mine = torch.tensor(checksums, dtype=torch.float64, device="cuda")
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        replicas_identical = all(bool(torch.equal(everyone[0], other)) for other in everyone)
    del parameters

    # ---- inference: the same network, forward + row arg-max, 8192 rows per GPU, no collective --------
    inference = None
    if not args.no_inference:
        inference = measure_inference(ctx, model, rank, world, local_rank, max(200, 20 * args.steps), barrier, reduce_max)

    tf32 = None
    if rank == 0 and not args.no_peak:
        tf32 = measure_tf32_peak(local_rank)
    barrier()

    if rank == 0:
        peak_data, peak_kind = peaks()
        # dominant kernel: the tcgen05 3xTF32 GEMM; algorithmic FLOPs 2*m*n*k per launch
        flops, ms = 0.0, 0.0
        gemm_launches = 0
        shares = {}
        for text, t in zip(plan, step_ms):
            kind = text.split()[0] + (":" + re.search(r"engine=(\w+)", text).group(1) if text.startswith("gemm") else "")
            shares[kind] = shares.get(kind, 0.0) + t
            if "engine=tcgen05_3xtf32" in text:
                m, n, k = (int(re.search(rf" {d}=(\d+)", text).group(1)) for d in "mnk")
                flops += 2.0 * m * n * k
                ms += t
                gemm_launches += 1
        emulated_peak = peak_data["bf16_tflops_sustained"] / 2.0 / 3.0       # TF32 dense = BF16 / 2; three MMAs per FP32 product
        achieved = flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
        total_step = sum(step_ms) or 1.0
        traffic = interpolate_rows(NCU_GEMM_TRAFFIC, rows)
        roofline = {"bound": "tensor", "kernel": "gemm_tf32x3_pair_kernel", "achieved": achieved, "peak": emulated_peak, "unit": "TFLOP/s",
                    "frac": achieved / emulated_peak if emulated_peak else None,
                    "peak_source": f"{peak_kind} cuBLAS BF16 sustained / 2 (TF32) / 3 (three MMAs per FP32 product)",
                    "traffic": traffic,
                    "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, mean over the step's eight launches of this kernel, "
                                      "captured at 8192 and at 65536 rows per GPU and interpolated to this run's rows",
                    "algorithmic_bytes_per_launch": interpolate_rows(ALGORITHMIC_GEMM_BYTES, rows),
                    "launches_per_step": gemm_launches, "ms_per_step_in_kernel": ms,
                    "kilocycles_in_kernel": at_equal_clock(ms, clocks),
                    "step_time_shares": {k: v / total_step for k, v in sorted(shares.items())},
                    "steps_ms": [[text.split(" nodes=")[0], round(t, 4)] for text, t in zip(plan, step_ms)]}
        if clocks and clocks.get("sm_mhz"):
            # the tensor pipe's own ceiling at the clock this run held: 148 SMs x 4096 dense TF32 FLOP per clock,
            # three MMAs per FP32 product (ncu: the pipe is active 96 % of the cycles of a 4096-deep product)
            ceiling = SM_COUNT * TENSOR_FLOP_PER_CLOCK_PER_SM * clocks["sm_mhz"] * 1e6 / 3.0 / 1e12
            roofline["peak_tensor_pipe_at_sampled_clock"] = ceiling
            roofline["frac_of_tensor_pipe_at_sampled_clock"] = achieved / ceiling
        if tf32:
            direct = tf32["sustained_tflops"] / 3.0
            roofline["peak_tf32_measured"] = direct
            roofline["frac_of_tf32_measured"] = achieved / direct
            roofline["frac_of_tf32_burst"] = achieved / (tf32["burst_tflops"] / 3.0)
            roofline["peak_tf32_source"] = "cuBLAS TF32 GEMM timed in this run (tf32_peak.sustained_tflops) / 3"
        line = {
            "metric": METRIC, "value": global_batch * args.steps / (resident_ms * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": resident_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "mlp_784_4096x3_10_softmax_ce_adam_train", "global_batch": global_batch, "rows_per_gpu": rows,
                       "parallelism": f"dp{world}", "gemm": "3xTF32 on tcgen05", "l2": "inputs_exceed_l2 (per-step working set > 1 GB)",
                       "data_seed": "one global batch, row blocks seeded by global index: identical rows for every number of ranks",
                       "optimizer_steps_taken": total_steps, "final_loss": final_loss,
                       "parameter_checksums": checksums, "replicas_identical": replicas_identical},
            "e2e": {"value": global_batch * args.steps / (e2e_ms * 1e-3), "unit": "samples/s",
                    "h2d_bytes_per_step": x_host.nbytes + t_host.nbytes, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": roofline,
            "model_tflops": step_flops(global_batch) * args.steps / (resident_ms * 1e-3) / 1e12,
            "inference": inference,
        }
        if tf32:
            line["tf32_peak"] = tf32
    model.close()
    for xb, tb in input_sets[1:]:
        xb.close(); tb.close()
    if rank == 0:
        if world == 1 and not args.no_kernels and global_batch == GLOBAL_BATCH:
            line["kernels"] = kernel_cases(ctx, local_rank)
        if world == 1 and not args.no_cpu_baseline and global_batch == GLOBAL_BATCH:
            threads = os.cpu_count() or 1
            value, blas, seconds = cpu_baseline(threads, 4096, steps=3, warmup=1)     # about 10 s of CPU work
            line["cpu_baseline"] = {"value": value, "unit": "samples/s", "cores": threads, "kind": "port",
                                    "sample": f"4096 of {GLOBAL_BATCH} rows per step, median of 3 timed steps after 1 warm-up, {seconds:.2f} s/step, BLAS: {os.path.basename(blas)}"}
        print(json.dumps(line))
    if comm is not None:
        comm.close()
    if distributed:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def measure_inference(ctx, model, rank, world, local_rank, steps, barrier, reduce_max):
    """Model.compute with the row arg-max at INFERENCE_ROWS_PER_GPU rows per GPU: every rank holds the
    weights and runs its own rows, nothing is exchanged (weak scaling).  Resident: the batch already in
    HBM.  End to end: per batch the input is copied from pinned host memory (on the copy stream, under
    the previous batch) and logits and arg-max are copied back, all inside the timed region."""
    from synaptik_b200 import native
    rows = INFERENCE_ROWS_PER_GPU
    exe, xbuf, outs = model._inference_state((rows,), True)
    x, _ = synthetic_rows(rank * rows, rows, seed=4321)
    x_host = native.PinnedArray((rows, DIMS[0]), np.float32)
    x_host.array[...] = x
    logits_host = native.PinnedArray((rows, DIMS[-1]), np.float32)
    index_host = native.PinnedArray((rows,), np.int64)
    xbuf.upload(x)
    feeds = [xbuf] + model.param_buffers
    for _ in range(5):
        exe.enqueue(feeds, outs)
    exe.finish()
    sampler = ClockSampler(local_rank, 100)
    barrier()
    if rank == 0:
        sampler.start()
    ctx.timer_start()
    for _ in range(steps):
        exe.enqueue(feeds, outs)
    resident_ms = reduce_max(ctx.timer_stop())
    exe.finish()
    ctx.set_option("time_steps", 1)
    exe.run(feeds, outs)
    ctx.set_option("time_steps", 0)
    plan, step_ms = exe.describe().strip().split("\n"), exe.step_timings_ms()
    launches = exe.launch_count()
    second = ctx.buffer(x_host.nbytes)
    sets = [xbuf, second]

    def batches(count):
        sets[0].prefetch(x_host.pointer, x_host.nbytes)
        for i in range(count):
            if i + 1 < count:
                sets[(i + 1) & 1].prefetch(x_host.pointer, x_host.nbytes)
            exe.enqueue([sets[i & 1]] + model.param_buffers, outs)
            outs[0].download_async(logits_host.pointer, logits_host.nbytes)
            outs[1].download_async(index_host.pointer, index_host.nbytes)
            exe.finish()

    batches(2)
    barrier()
    ctx.timer_start()
    wall = time.perf_counter()
    batches(steps)
    e2e_ms = ctx.timer_stop()
    wall = (time.perf_counter() - wall) * 1e3
    e2e_ms = reduce_max(max(e2e_ms, wall))
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    checksum = int(np.sum(index_host.array))
    second.close(); x_host.close(); logits_host.close(); index_host.close()
    if rank != 0:
        return None
    peak_data, peak_kind = peaks()
    flops = gemm_ms = 0.0
    for text, t in zip(plan, step_ms):
        if "engine=tcgen05_3xtf32" in text:
            m, n, k = (int(re.search(rf" {d}=(\d+)", text).group(1)) for d in "mnk")
            flops += 2.0 * m * n * k
            gemm_ms += t
    achieved = flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms else 0.0
    peak = peak_data["bf16_tflops_sustained"] / 6.0
    return {"metric": "mlp_inference_samples_per_s", "value": world * rows * steps / (resident_ms * 1e-3), "unit": "samples/s",
            "scaling": "weak", "n_gpus": world, "rows_per_gpu": rows, "steps": steps, "ms_per_batch": resident_ms / steps,
            "workload": "mlp_784_4096x3_10_forward_argmax", "collective": "none (weights replicated, rows split)",
            "e2e": {"value": world * rows * steps / (e2e_ms * 1e-3), "unit": "samples/s", "ms_per_batch": e2e_ms / steps,
                    "h2d_bytes_per_step": rows * DIMS[0] * 4, "d2h_bytes_per_step": rows * DIMS[-1] * 4 + rows * 8},
            "model_tflops_per_gpu": forward_flops(rows) * steps / (resident_ms * 1e-3) / 1e12,
            "gpu_launches": launches * steps,
            "roofline": {"bound": "tensor", "kernel": "gemm_tf32x3_pair_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak if peak else None, "peak_source": f"{peak_kind} cuBLAS BF16 sustained / 2 / 3",
                         "ms_per_batch_in_kernel": gemm_ms,
                         "steps_ms": [[text.split(" nodes=")[0], round(t, 4)] for text, t in zip(plan, step_ms)]},
            "arg_max_checksum": checksum, "clocks": clocks, "kilocycles_per_batch": at_equal_clock(resident_ms / steps, clocks)}


def measure_kernel_case(ctx, device_index, case, m, k, n, forward_only=False, steps=10, warmup=3, blocks=31, warm_seconds=1.0, dtype="f32"):
    """One kernel case through the C ABI on context `ctx`: the standalone fused dense layer (forward and
    backward) or a piece of the classifier head.  Times `steps` back-to-back launches between two CUDA
    events on the context's stream, then follows the reference's own protocol (warm-up of at least
    `warm_seconds`, then `blocks` timed blocks of at least 30 ms, median reported), samples the clocks
    during all of it, and brackets every plan step with events once for the per-kernel times."""
    from synaptik_b200 import native
    from synaptik_b200.program import F32, I32, GraphBuilder
    rng = np.random.default_rng(3)
    g = GraphBuilder()
    peak_data, peak_kind = peaks()
    if case == "gemm" and dtype != "f32":
        # the dense layer on 16-bit storage (BFLOAT16 / FLOAT16 values, FLOAT32 accumulation): forward only,
        # operands read by TMA straight from the tensors, one tcgen05 kind::f16 MMA per 16 contraction steps
        from synaptik_b200 import program
        storage = program.STORAGE_DTYPES[dtype]
        x, w, b = g.feed(storage, (m, k)), g.feed(storage, (n, k)), g.feed(storage, (n,))
        _, z = g.linear(x, w, b)
        g.publish(g.relu(z))
        bound = np.sqrt(6.0 / (k + n))
        feeds = [program.to_storage(dtype, rng.random((m, k), dtype=np.float32) * 2 - 1),
                 program.to_storage(dtype, (rng.random((n, k), dtype=np.float32) * 2 - 1) * np.float32(bound)),
                 program.to_storage(dtype, (rng.random(n, dtype=np.float32) * 2 - 1) * np.float32(0.1))]
        forward_only = True
        work = 2.0 * m * k * n
        unit, denom, bound_kind = "TFLOP/s", peak_data["bf16_tflops"], "tensor"
        name = f"dense_layer_fwd_{dtype}_m{m}_k{k}_n{n}"
    elif case == "gemm":
        x, w, b, dy = g.feed(F32, (m, k)), g.feed(F32, (n, k)), g.feed(F32, (n,)), g.feed(F32, (m, n))
        wt, z = g.linear(x, w, b)
        g.publish(g.relu(z))
        if not forward_only:
            dz = g.relu_backward(z, dy)
            dx, dw, db = g.linear_backward(x, wt, dz, need_dx=True)
            for v in (dx, dw, db):
                g.publish(v)
        bound = np.sqrt(6.0 / (k + n))
        feeds = [rng.random((m, k), dtype=np.float32) * 2 - 1, (rng.random((n, k), dtype=np.float32) * 2 - 1) * np.float32(bound),
                 (rng.random(n, dtype=np.float32) * 2 - 1) * np.float32(0.1), rng.standard_normal((m, n), dtype=np.float32)]
        work = (2.0 if forward_only else 6.0) * m * k * n
        unit, denom, bound_kind = "TFLOP/s", peak_data["bf16_tflops"] / 6.0, "tensor"
        name = f"dense_layer_{'fwd' if forward_only else 'fwd_bwd'}_m{m}_k{k}_n{n}"
    elif case == "dense_ce":
        rows, classes = m, n
        logits, target = g.feed(F32, (rows, classes)), g.feed(F32, (rows, classes))
        g.publish(g.dense_cross_entropy(logits, target, "mean"))
        weights = rng.random((rows, classes), dtype=np.float32)
        feeds = [rng.standard_normal((rows, classes), dtype=np.float32) * 2, weights / weights.sum(axis=1, keepdims=True)]
        work = 8.0 * rows * classes + 4.0 * rows + 4.0           # read logits and target weights, row losses, the mean
        unit, denom, bound_kind = "GB/s", peak_data["hbm_gbs"], "hbm"
        name = f"dense_cross_entropy_rows{rows}_classes{classes}"
    elif case == "argmax":
        rows, classes = m, n
        logits = g.feed(F32, (rows, classes))
        g.publish(g.arg_max(logits, 1))
        feeds = [rng.standard_normal((rows, classes), dtype=np.float32) * 2]
        work = 4.0 * rows * classes + 8.0 * rows                 # read the logits, write one INT64 index per row
        unit, denom, bound_kind = "GB/s", peak_data["hbm_gbs"], "hbm"
        name = f"argmax_rows{rows}_classes{classes}"
    elif case in ("softmax", "log_softmax"):
        rows, classes = m, n
        logits = g.feed(F32, (rows, classes))
        g.publish(g.softmax(logits, 1) if case == "softmax" else g.log_softmax(logits, 1))
        feeds = [rng.standard_normal((rows, classes), dtype=np.float32) * 2]
        work = 8.0 * rows * classes                              # one pass: read the logits, write the result
        unit, denom, bound_kind = "GB/s", peak_data["hbm_gbs"], "hbm"
        name = f"{case}_rows{rows}_classes{classes}"
    else:
        rows, classes = m, n
        logits, labels, seed = g.feed(F32, (rows, classes)), g.feed(I32, (rows,)), g.feed(F32, ())
        g.publish(g.index_cross_entropy(logits, labels))
        g.publish(g.index_cross_entropy_backward(logits, labels, seed))
        g.publish(g.arg_max(logits, 1))
        feeds = [rng.standard_normal((rows, classes), dtype=np.float32) * 2, rng.integers(0, classes, rows).astype(np.int32),
                 np.array(1.0, dtype=np.float32)]
        work = 8.0 * rows * classes + 12.0 * rows + 4.0          # one pass: read logits, write gradient, labels, arg-max, loss
        unit, denom, bound_kind = "GB/s", peak_data["hbm_gbs"], "hbm"
        name = f"classifier_head_rows{rows}_classes{classes}"
    exe = native.Executable(ctx, g.build())
    inputs = [ctx.upload(a) for a in feeds]
    del feeds
    outputs = [ctx.buffer(max(g.values[i].nbytes, 4)) for i in g.publications]
    resident_bytes = sum(b.nbytes for b in inputs + outputs)
    # Inputs and results smaller than twice the 126 MB L2 would be timed warm: such a case is timed one run
    # at a time (the run's own start / stop events), with a 524 MB streaming pass in front of every timed run.
    flush = None
    if resident_bytes < 2 * 126e6:
        fg = GraphBuilder()
        fg.publish(fg.softmax(fg.feed(F32, (65536, 1000)), 1))
        flush = (native.Executable(ctx, fg.build()), [ctx.buffer(65536 * 1000 * 4)], [ctx.buffer(65536 * 1000 * 4)])
    for _ in range(max(warmup, 3)):
        exe.run(inputs, outputs)
    sampler = ClockSampler(device_index, 100).start()
    if flush is None:
        # timed region: the launches back to back between two CUDA events on the context's stream
        ctx.timer_start()
        for _ in range(steps):
            exe.enqueue(inputs, outputs)
        ms = ctx.timer_stop()
        exe.finish()
        per_step = max(ms / steps, 1e-3)
        block_steps = max(1, int(np.ceil(30.0 / per_step)))
        for _ in range(max(20, int(np.ceil(1000.0 * warm_seconds / per_step))) if warm_seconds > 0 else 0):
            exe.enqueue(inputs, outputs)
        exe.finish()
        timed = []
        for _ in range(blocks):
            ctx.timer_start()
            for _ in range(block_steps):
                exe.enqueue(inputs, outputs)
            timed.append(ctx.timer_stop() / block_steps)
        exe.finish()
        protocol = f"median of {blocks} blocks of {block_steps} back-to-back launches after a warm-up of at least {warm_seconds} s"
        l2 = "inputs_exceed_l2"
    else:
        timed = []
        for _ in range(max(steps, 40 * blocks)):
            flush[0].enqueue(flush[1], flush[2])
            exe.enqueue(inputs, outputs)
            exe.finish()
            timed.append(exe.last_timing_ms())
        ms = float(np.sum(timed[:steps]))
        protocol = f"median of {len(timed)} single runs, each behind a streaming pass over 524 MB"
        l2 = f"flushed before every timed run (inputs and results are {resident_bytes / 1e6:.0f} MB)"
    clocks = sampler.stop()
    median_ms = float(np.median(timed))
    # one more run with an event pair around every plan step, for the per-kernel times
    ctx.set_option("time_steps", 1)
    if flush is not None:
        flush[0].enqueue(flush[1], flush[2])
    exe.run(inputs, outputs)
    ctx.set_option("time_steps", 0)
    plan = exe.describe().strip().split("\n")
    step_times = exe.step_timings_ms()
    per_unit = 1e12 if unit == "TFLOP/s" else 1e9
    # roofline of the dominant kernel: its algorithmic work over its own event-bracketed time (the
    # per-step CUDA events of the last run) for the dense layer, whose step has other launches too; for
    # the one-launch cases the median block time over the launches
    if case == "gemm":
        kernel, kernel_work, kernel_ms = "gemm_tf32x3_pair_kernel", 0.0, 0.0
        for text, t in zip(plan, step_times):
            if "engine=tcgen05_3xtf32" in text or "engine=tcgen05_f16" in text:
                mm, nn_, kk = (int(re.search(rf" {d}=(\d+)", text).group(1)) for d in "mnk")
                kernel_work += 2.0 * mm * nn_ * kk
                kernel_ms += t
        if dtype != "f32":
            kernel = "gemm_low_pair_kernel (gemm_low_kernel where the product has few tiles)"
    else:
        kernel = {"ce": "ce_rows_vec_kernel", "argmax": "argmax_vec_kernel", "dense_ce": "dense_ce_rows_vec_kernel"}.get(case, "softmax_rows_vec_kernel")
        kernel_work, kernel_ms = work, median_ms
    achieved = kernel_work / (kernel_ms * 1e-3) / per_unit if kernel_ms > 0 else 0.0
    record = {"metric": f"{case}_{unit}", "value": work / (median_ms * 1e-3) / per_unit, "unit": unit, "n_gpus": 1, "steps": steps,
              "warmup": max(warmup, 3), "ms_per_step": ms / steps, "median_ms_per_step": median_ms,
              "protocol": protocol,
              "higher_is_better": True, "dtype": dtype, "data": "synthetic",
              "config": {"workload": name, "l2": l2},
              "gpu_launches": exe.launch_count() * steps, "clocks": clocks, "kilocycles_per_step": at_equal_clock(median_ms, clocks),
              "roofline": {"bound": bound_kind, "kernel": kernel, "achieved": achieved, "peak": denom, "unit": unit, "frac": achieved / denom,
                           "ms_in_kernel": kernel_ms,
                           "peak_source": peak_kind + ((" cuBLAS BF16 burst" if dtype != "f32" else " cuBLAS BF16 burst / 2 / 3") if unit == "TFLOP/s" else " copy bandwidth"), "traffic": None},
              "steps_ms": {text.split(" nodes=")[0]: t for text, t in zip(plan, step_times)}}
    exe.close()
    if flush is not None:
        flush[0].close()
        inputs = inputs + flush[1] + flush[2]
    for b in inputs + outputs:
        b.close()
    return record


def kernel_cases(ctx, device_index):
    """The standalone cases the headline names beside the training step, each for a second or so: the six
    fused dense layer shapes (forward + dX + dW + db) and the 1000-class classifier head."""
    records = []
    for m in (4096, 16384, 65536):
        for kn in (1024, 4096):
            r = measure_kernel_case(ctx, device_index, "gemm", m, kn, kn, steps=5, blocks=9, warm_seconds=0.3)
            records.append({"workload": r["config"]["workload"], "unit": r["unit"], "whole_layer": r["value"], "median_ms": r["median_ms_per_step"],
                            "kernel": r["roofline"]["kernel"], "in_kernel": r["roofline"]["achieved"], "ms_in_kernel": r["roofline"]["ms_in_kernel"],
                            "peak": r["roofline"]["peak"], "frac": r["roofline"]["frac"], "algorithmic_flop": 6.0 * m * kn * kn,
                            "clocks": r["clocks"], "kilocycles": r["kilocycles_per_step"]})
    for low in ("bf16", "f16"):
        r = measure_kernel_case(ctx, device_index, "gemm", 65536, 4096, 4096, steps=5, blocks=9, warm_seconds=0.3, dtype=low)
        records.append({"workload": r["config"]["workload"], "unit": r["unit"], "whole_layer": r["value"], "median_ms": r["median_ms_per_step"],
                        "kernel": r["roofline"]["kernel"], "in_kernel": r["roofline"]["achieved"], "ms_in_kernel": r["roofline"]["ms_in_kernel"],
                        "peak": r["roofline"]["peak"], "frac": r["roofline"]["frac"], "algorithmic_flop": 2.0 * 65536 * 4096 * 4096,
                        "clocks": r["clocks"], "kilocycles": r["kilocycles_per_step"]})
    for case in ("ce", "softmax", "argmax"):
        r = measure_kernel_case(ctx, device_index, case, 65536, 0, 1000, steps=20, blocks=9, warm_seconds=0.3)
        records.append({"workload": r["config"]["workload"], "unit": r["unit"], "value": r["value"], "median_ms": r["median_ms_per_step"],
                        "kernel": r["roofline"]["kernel"], "peak": r["roofline"]["peak"], "frac": r["roofline"]["frac"],
                        "clocks": r["clocks"], "kilocycles": r["kilocycles_per_step"]})
    return records


def run_kernel_case(args):
    from synaptik_b200 import native
    ctx = native.Context(0)
    for item in filter(None, os.environ.get("SYNAPTIK_BENCH_OPTIONS", "").split(",")):      # experiment hook, as in run_cuda
        name, _, value = item.partition("=")
        ctx.set_option(name.strip(), int(value))
    if args.quick:
        record = measure_kernel_case(ctx, 0, args.case, args.m, args.k, args.n, args.forward_only, args.steps, args.warmup, blocks=1, warm_seconds=0.0, dtype=args.dtype)
    else:
        record = measure_kernel_case(ctx, 0, args.case, args.m, args.k, args.n, args.forward_only, args.steps, args.warmup, dtype=args.dtype)
    print(json.dumps(record))
    ctx.close()
    return 0


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--case", default="train", choices=["train", "gemm", "ce", "softmax", "log_softmax", "argmax", "dense_ce"])
    parser.add_argument("--m", type=int, default=16384)
    parser.add_argument("--k", type=int, default=4096)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--forward-only", action="store_true")
    parser.add_argument("--dtype", default="f32", choices=["f32", "bf16", "f16"], help="storage type of the dense-layer case (16-bit: forward only)")
    parser.add_argument("--quick", action="store_true", help="kernel cases: only the plain timed region (few launches: the workload of a profiler capture)")
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-kernels", action="store_true")
    parser.add_argument("--no-peak", action="store_true")
    parser.add_argument("--no-inference", action="store_true")
    parser.add_argument("--global-batch", type=int, default=GLOBAL_BATCH,
                        help="rows of the training batch; anything but the default is a reduced workload for profiler captures, not a benchmark")
    args = parser.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.case != "train":
        return run_kernel_case(args)
    return run_cuda(args)


if __name__ == "__main__":
    sys.exit(main())
