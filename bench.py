"""Benchmark of the data-parallel MLP training step (BASELINE.json configs[4]).

    python bench.py --gpus N --steps K --warmup W            # the CUDA backend, one rank per GPU
    python bench.py --impl reference --gpus N --steps K ...  # the reference-shaped CPU path

Workload: 784 -> 4096 -> 4096 -> 4096 -> 10 Linear/ReLU classifier, softmax cross-entropy, Adam
(1e-3, 0.9, 0.999, 1e-8), global batch 65536 split evenly over the ranks, gradients sum-allreduced
with NCCL over NVLink overlapped with the backward pass, FP32 (GEMMs in 3xTF32 on tcgen05).
Synthetic seeded data: x ~ U(0,1), labels ~ U{0..9}, Glorot-uniform weights, zero biases.

One JSON line is printed by rank 0.  `value` times K steps with the batch already resident in HBM;
`e2e` times K steps through the same C-ABI calls with the batch uploaded from pinned host memory
and the loss read back every step.
"""
from __future__ import annotations

import argparse
import json
import os
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
ADAM = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)
METRIC = "mlp_train_samples_per_s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def step_flops(batch: int) -> float:
    """Algorithmic FLOPs of one training step: forward 2*B*P, backward 4*B*P minus the input gradient."""
    weights = sum(DIMS[i] * DIMS[i + 1] for i in range(len(DIMS) - 1))
    return 6.0 * batch * weights - 2.0 * batch * DIMS[0] * DIMS[1]


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        data = json.load(open(path))
        return data, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def synthetic_batch(rank: int, rows: int):
    rng = np.random.default_rng(1234 + rank)
    x = rng.random((rows, DIMS[0]), dtype=np.float32)
    labels = rng.integers(0, DIMS[-1], rows).astype(np.int32)
    return x, labels


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE, text=True)
        except OSError:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

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
    x, labels = synthetic_batch(0, rows)
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


def run_cuda(args):
    import torch
    import torch.distributed as dist
    from synaptik_b200 import native, nn

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
    rows = GLOBAL_BATCH // world
    model = nn.Model(DIMS, ctx, seed=42, comm=comm, world_size=world)       # same seed: replicas start identical
    model.configure_training("ce", nn.Adam(ADAM["lr"], ADAM["beta1"], ADAM["beta2"], ADAM["eps"]))
    exe, xbuf, tbuf, seed, loss, grads = model.training_state(rows)
    inputs, outputs = [xbuf, tbuf, seed] + model.param_buffers, [loss] + grads
    x_host = native.PinnedArray((rows, DIMS[0]), np.float32)
    t_host = native.PinnedArray((rows,), np.int32)
    loss_host = native.PinnedArray((1,), np.float32)
    x, labels = synthetic_batch(rank, rows)
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

    def resident_step():
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
    final_loss = float(loss_host.array[0])

    if rank == 0:
        peak_data, peak_kind = peaks()
        # dominant kernel: the tcgen05 3xTF32 GEMM; algorithmic FLOPs 2*m*n*k per launch
        import re
        flops, ms = 0.0, 0.0
        gemm_launches = 0
        shares = {}
        for line, t in zip(plan, step_ms):
            kind = line.split()[0] + (":" + re.search(r"engine=(\w+)", line).group(1) if line.startswith("gemm") else "")
            shares[kind] = shares.get(kind, 0.0) + t
            if "engine=tcgen05_3xtf32" in line:
                m, n, k = (int(re.search(rf" {d}=(\d+)", line).group(1)) for d in "mnk")
                flops += 2.0 * m * n * k
                ms += t
                gemm_launches += 1
        tf32_peak = peak_data["bf16_tflops_sustained"] / 2.0          # TF32 dense = BF16 / 2 on B200
        emulated_peak = tf32_peak / 3.0                                 # three MMAs per FP32 product
        achieved = flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
        total_step = sum(step_ms) or 1.0
        line = {
            "metric": METRIC, "value": GLOBAL_BATCH * args.steps / (resident_ms * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": resident_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "mlp_784_4096x3_10_softmax_ce_adam_train", "global_batch": GLOBAL_BATCH, "rows_per_gpu": rows,
                       "parallelism": f"dp{world}", "gemm": "3xTF32 on tcgen05", "l2": "inputs_exceed_l2 (per-step working set > 1 GB)",
                       "final_loss": final_loss},
            "e2e": {"value": GLOBAL_BATCH * args.steps / (e2e_ms * 1e-3), "unit": "samples/s",
                    "h2d_bytes_per_step": x_host.nbytes + t_host.nbytes, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "gemm_tf32x3_pair_kernel", "achieved": achieved, "peak": emulated_peak, "unit": "TFLOP/s",
                         "frac": achieved / emulated_peak if emulated_peak else None,
                         # DRAM bytes per launch (read + written, mean over the step's 8 GEMM launches) from the
                         # committed ncu capture of exactly these launches; other shapes were not captured
                         "traffic": 8.67e9 if rows == GLOBAL_BATCH else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, profiles/train_step_launch_list.md" if rows == GLOBAL_BATCH else None,
                         "algorithmic_bytes_per_launch": 28.7e9 / 8 if rows == GLOBAL_BATCH else None,
                         "peak_source": f"{peak_kind} bf16_tflops_sustained / 2 (TF32) / 3 (3xTF32)",
                         "launches_per_step": gemm_launches, "ms_per_step_in_kernel": ms,
                         "step_time_shares": {k: v / total_step for k, v in sorted(shares.items())},
                         "steps_ms": [[line.split(" nodes=")[0], round(t, 4)] for line, t in zip(plan, step_ms)]},
            "model_tflops": step_flops(GLOBAL_BATCH) * args.steps / (resident_ms * 1e-3) / 1e12,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            value, blas, seconds = cpu_baseline(threads, 4096, steps=3, warmup=1)     # about 10 s of CPU work
            line["cpu_baseline"] = {"value": value, "unit": "samples/s", "cores": threads, "kind": "port",
                                    "sample": f"4096 of {GLOBAL_BATCH} rows per step, median of 3 timed steps after 1 warm-up, {seconds:.2f} s/step, BLAS: {os.path.basename(blas)}"}
        print(json.dumps(line))
    model.close()
    if comm is not None:
        comm.close()
    if distributed:
        dist.destroy_process_group()
    return 0


def run_kernel_case(args):
    """Single-GPU kernel cases behind the same C ABI: BASELINE.json configs[1] (fused dense layer,
    forward and backward) and configs[2] (classifier head).  Used for the roofline lines and as the
    small workloads of the ncu captures."""
    from synaptik_b200 import native, program
    from synaptik_b200.program import F32, I32, GraphBuilder
    ctx = native.Context(0)
    for item in filter(None, os.environ.get("SYNAPTIK_BENCH_OPTIONS", "").split(",")):      # experiment hook, as in run_cuda
        name, _, value = item.partition("=")
        ctx.set_option(name.strip(), int(value))
    rng = np.random.default_rng(3)
    g = GraphBuilder()
    peak_data, peak_kind = peaks()
    if args.case == "gemm":
        m, k, n = args.m, args.k, args.n
        x, w, b, dy = g.feed(F32, (m, k)), g.feed(F32, (n, k)), g.feed(F32, (n,)), g.feed(F32, (m, n))
        wt, z = g.linear(x, w, b)
        g.publish(g.relu(z))
        if not args.forward_only:
            dz = g.relu_backward(z, dy)
            dx, dw, db = g.linear_backward(x, wt, dz, need_dx=True)
            for v in (dx, dw, db):
                g.publish(v)
        bound = np.sqrt(6.0 / (k + n))
        feeds = [rng.uniform(-1, 1, (m, k)).astype(np.float32), rng.uniform(-bound, bound, (n, k)).astype(np.float32),
                 rng.uniform(-0.1, 0.1, n).astype(np.float32), rng.standard_normal((m, n)).astype(np.float32)]
        work = (2.0 if args.forward_only else 6.0) * m * k * n
        unit, denom, bound_kind = "TFLOP/s", peak_data["bf16_tflops"] / 6.0, "tensor"
        name = f"dense_layer_{'fwd' if args.forward_only else 'fwd_bwd'}_m{m}_k{k}_n{n}"
    elif args.case == "dense_ce":
        rows, classes = args.m, args.n
        logits, target = g.feed(F32, (rows, classes)), g.feed(F32, (rows, classes))
        g.publish(g.dense_cross_entropy(logits, target, "mean"))
        weights = rng.random((rows, classes)).astype(np.float32)
        feeds = [(rng.standard_normal((rows, classes)) * 2).astype(np.float32), weights / weights.sum(axis=1, keepdims=True)]
        work = 8.0 * rows * classes + 4.0 * rows + 4.0           # read logits and target weights, row losses, the mean
        unit, denom, bound_kind = "GB/s", peak_data["hbm_gbs"], "hbm"
        name = f"dense_cross_entropy_rows{rows}_classes{classes}"
    elif args.case == "argmax":
        rows, classes = args.m, args.n
        logits = g.feed(F32, (rows, classes))
        g.publish(g.arg_max(logits, 1))
        feeds = [(rng.standard_normal((rows, classes)) * 2).astype(np.float32)]
        work = 4.0 * rows * classes + 8.0 * rows                 # read the logits, write one INT64 index per row
        unit, denom, bound_kind = "GB/s", peak_data["hbm_gbs"], "hbm"
        name = f"argmax_rows{rows}_classes{classes}"
    elif args.case in ("softmax", "log_softmax"):
        rows, classes = args.m, args.n
        logits = g.feed(F32, (rows, classes))
        g.publish(g.softmax(logits, 1) if args.case == "softmax" else g.log_softmax(logits, 1))
        feeds = [(rng.standard_normal((rows, classes)) * 2).astype(np.float32)]
        work = 8.0 * rows * classes                              # one pass: read the logits, write the result
        unit, denom, bound_kind = "GB/s", peak_data["hbm_gbs"], "hbm"
        name = f"{args.case}_rows{rows}_classes{classes}"
    else:
        rows, classes = args.m, args.n
        logits, labels, seed = g.feed(F32, (rows, classes)), g.feed(I32, (rows,)), g.feed(F32, ())
        g.publish(g.index_cross_entropy(logits, labels))
        g.publish(g.index_cross_entropy_backward(logits, labels, seed))
        g.publish(g.arg_max(logits, 1))
        feeds = [(rng.standard_normal((rows, classes)) * 2).astype(np.float32), rng.integers(0, classes, rows).astype(np.int32),
                 np.array(1.0, dtype=np.float32)]
        work = 8.0 * rows * classes + 12.0 * rows + 4.0          # one pass: read logits, write gradient, labels, arg-max, loss
        unit, denom, bound_kind = "GB/s", peak_data["hbm_gbs"], "hbm"
        name = f"classifier_head_rows{rows}_classes{classes}"
    exe = native.Executable(ctx, g.build())
    inputs = [ctx.upload(a) for a in feeds]
    outputs = [ctx.buffer(max(g.values[i].nbytes, 4)) for i in g.publications]
    for _ in range(max(args.warmup, 1)):
        exe.run(inputs, outputs)
    # timed region: the launches back to back between two CUDA events on the context's stream
    ctx.timer_start()
    for _ in range(args.steps):
        exe.enqueue(inputs, outputs)
    ms = ctx.timer_stop()
    exe.finish()
    # the reference's own timing protocol (warm-up of at least 20 calls and 1 s, then 31 timed blocks of
    # at least 30 ms each, median reported): blocks of back-to-back launches between two CUDA events
    per_step = max(ms / args.steps, 1e-3)
    block_steps = max(1, int(np.ceil(30.0 / per_step)))
    for _ in range(max(20, int(np.ceil(1000.0 / per_step)))):
        exe.enqueue(inputs, outputs)
    exe.finish()
    blocks = []
    for _ in range(31):
        ctx.timer_start()
        for _ in range(block_steps):
            exe.enqueue(inputs, outputs)
        blocks.append(ctx.timer_stop() / block_steps)
    exe.finish()
    median_ms = float(np.median(blocks))
    # one more run with an event pair around every plan step, for the per-kernel times
    ctx.set_option("time_steps", 1)
    exe.run(inputs, outputs)
    ctx.set_option("time_steps", 0)
    plan = exe.describe().strip().split("\n")
    steps = exe.step_timings_ms()
    rate = work * args.steps / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
    # roofline of the dominant kernel: its algorithmic work over its own event-bracketed time (the
    # per-step CUDA events of the last timed run), not over the whole run with its other launches
    import re
    if args.case == "gemm":
        kernel, kernel_work, kernel_ms = "gemm_tf32x3_pair_kernel", 0.0, 0.0
        for text, t in zip(plan, steps):
            if "engine=tcgen05_3xtf32" in text:
                mm, nn, kk = (int(re.search(rf" {d}=(\d+)", text).group(1)) for d in "mnk")
                kernel_work += 2.0 * mm * nn * kk
                kernel_ms += t
    else:
        # the whole step is this one launch: its average duration is the timed region over the launches
        kernel = {"ce": "ce_rows_vec_kernel", "argmax": "argmax_vec_kernel", "dense_ce": "dense_ce_rows_vec_kernel"}.get(args.case, "softmax_rows_vec_kernel")
        kernel_work, kernel_ms = work, ms / args.steps
    achieved = kernel_work / (kernel_ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9) if kernel_ms > 0 else 0.0
    line = {"metric": f"{args.case}_{unit}", "value": rate, "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 1),
            "ms_per_step": ms / args.steps, "median_ms_per_step": median_ms,
            "protocol": f"median of 31 blocks of {block_steps} launches after a warm-up of at least 1 s",
            "higher_is_better": True, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name}, "gpu_launches": exe.launch_count() * args.steps,
            "roofline": {"bound": bound_kind, "kernel": kernel, "achieved": achieved, "peak": denom, "unit": unit, "frac": achieved / denom,
                         "ms_in_kernel": kernel_ms,
                         "peak_source": peak_kind + (" bf16_tflops / 2 / 3" if unit == "TFLOP/s" else " hbm_gbs"), "traffic": None},
            "steps_ms": {line.split(" nodes=")[0]: t for line, t in zip(plan, steps)}}
    print(json.dumps(line))
    exe.close()
    ctx.close()
    return 0


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--case", default="train", choices=["train", "gemm", "ce", "softmax", "log_softmax", "argmax", "dense_ce"])
    parser.add_argument("--m", type=int, default=16384)
    parser.add_argument("--k", type=int, default=4096)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--forward-only", action="store_true")
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    args = parser.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.case != "train":
        return run_kernel_case(args)
    return run_cuda(args)


if __name__ == "__main__":
    sys.exit(main())
