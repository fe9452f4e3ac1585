"""Benchmark of the compiled-graph hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one execution of a compiled graph (`mc_enqueue`) on inputs already resident in HBM.
The default workload is the batch-sharded 8-layer MLP stack in FP16 tensor-core arithmetic
(x[65536,2048], eight 2048x2048 layers with a folded BatchNorm affine and relu in each GEMM's
epilogue: 8 launches, 4.4 TFLOP per step), reported as graph TFLOP/s. With N > 1 (launched by
torchrun, one rank per GPU) its batch dim is sharded over the ranks (strong scaling), and so are
c3/c1; c2/c4 run one replica per GPU on rank-specific data (weak scaling).
At N = 1 the same JSON line carries an `also` list with brief measurements of the other configs
(`--also none` turns it off): c2 (tanh-GELU chain, fused-eltwise HBM GB/s), c4 shapes of the
tensor-core sweep, c3 in TF32 and FP32, c1.
Other workloads (`--workload`): c1, c2, c3_fp32, c3_tf32, c4_bf16, c4_f16, c4_tf32, c4_fp32, c5_f16,
c5_bf16, the rest of the c4 sweep (c4_<fmt>_<size>|m16|m128|tallk); x1_softmax and x2_layernorm
(extension graphs) report GB/s of read-x-plus-write-y bytes.

Rank 0 prints ONE JSON line. `value` is device-timed with CUDA events on the launching stream,
max over ranks; `e2e` is the same metric through `mc_run` on pinned host buffers (copies inside
the timed region); `roofline` relates the dominant kernel to the measured peak in
MEASURED_PEAKS.json; `cpu_baseline` times the CPU oracle on a bounded sample, on all host threads
and on one thread (the reference's own CPU configuration, bench/harness.hpp:254).
Inputs are seeded synthetic tensors with the configs' shapes and distributions (numpy's PCG64
generator: the bench never compares values, the parity tests do, on the oracle's own stream).

`--impl reference` times the reference's CPU path instead: the Eigen backend cannot be built
here (Eigen 3.4.0 is not vendored and not installed), so it is the oracle port, on host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

# workload -> (graph, dims, matmul kernel, batch dim, metric kind, input distribution)
WORKLOADS = {
    "c2": ("c2_gelu_chain", {"M": 8192, "N": 8192}, "auto", None, "bytes", "normal"),
    "c1": ("c1_mlp_block", {"B": 256}, "auto", "B", "flops", "uniform"),
    "c3_fp32": ("c3_ffn", {"T": 8192, "D": 1024, "H": 4096}, "auto", "T", "flops", "normal"),
    "c3_tf32": ("c3_ffn", {"T": 8192, "D": 1024, "H": 4096}, "tensor_core_tf32", "T", "flops", "normal"),
    "c4_bf16": ("c4_matmul", {"M": 8192, "N": 8192, "K": 8192}, "tensor_core_bf16", None, "flops", "uniform"),
    "c4_f16": ("c4_matmul", {"M": 8192, "N": 8192, "K": 8192}, "tensor_core_f16", None, "flops", "uniform"),
    "c4_tf32": ("c4_matmul", {"M": 8192, "N": 8192, "K": 8192}, "tensor_core_tf32", None, "flops", "uniform"),
    "c4_fp32": ("c4_matmul", {"M": 4096, "N": 4096, "K": 4096}, "auto", None, "flops", "uniform"),
    "c5_f16": ("c5_mlp_stack", {"B": 65536, "D": 2048}, "tensor_core_f16", "B", "flops", "normal"),
    "c5_bf16": ("c5_mlp_stack", {"B": 65536, "D": 2048}, "tensor_core_bf16", "B", "flops", "normal"),
    # Extension graphs built from the row reductions; bytes = read x + write y, what a single fused kernel would move.
    "x1_softmax": ("x1_softmax", {"M": 8192, "N": 8192}, "auto", "M", "bytes", "normal"),
    "x2_layernorm": ("x2_layernorm", {"M": 16384, "N": 4096}, "auto", "M", "bytes", "normal"),
}
# The rest of the C4 sweep: squares, skinny-M and tall-K shapes, per 16-bit format.
for _fmt in ("bf16", "f16"):
    for _s in (1024, 2048, 4096, 16384):
        WORKLOADS[f"c4_{_fmt}_{_s}"] = ("c4_matmul", {"M": _s, "N": _s, "K": _s}, f"tensor_core_{_fmt}", None, "flops", "uniform")
    WORKLOADS[f"c4_{_fmt}_m16"] = ("c4_matmul", {"M": 16, "N": 8192, "K": 8192}, f"tensor_core_{_fmt}", None, "flops", "uniform")
    WORKLOADS[f"c4_{_fmt}_m128"] = ("c4_matmul", {"M": 128, "N": 8192, "K": 8192}, f"tensor_core_{_fmt}", None, "flops", "uniform")
    WORKLOADS[f"c4_{_fmt}_tallk"] = ("c4_matmul", {"M": 1024, "N": 1024, "K": 65536}, f"tensor_core_{_fmt}", None, "flops", "uniform")
DTYPES = {"auto": "f32", "tensor_core_tf32": "tf32", "tensor_core_bf16": "bf16", "tensor_core_f16": "f16"}


def algorithmic_work(oracle, graph, kind):
    """Bytes: every compute node's output once plus each distinct non-scalar operand once, on the graph as
    executed (the reference's bytes_moved convention, bench/bench_cuda.cpp:76-95); for the fused GELU chain that
    is read x + write y. FLOPs: 2 m n k per matmul (bench/bench_cuda.cpp:634)."""
    if kind == "bytes":
        x = graph.node(graph.inputs[0])
        return 2 * 4 * int(np.prod(x.shape))
    flops = 0
    for n in graph.nodes:
        if n.op == "matmul":
            a, b = graph.node(n.operands[0]), graph.node(n.operands[1])
            flops += 2 * a.shape[0] * a.shape[1] * b.shape[1]
    return flops


def matmul_operand_bytes(graph, elem_bytes):
    """Bytes a matmul graph must move at least: each matmul's two operands once in the arithmetic's operand width and
    its FP32 result once (2(mk + kn) + 4mn for 16-bit operands). Used to tell whether HBM or the math bounds a shape."""
    total = 0
    for n in graph.nodes:
        if n.op == "matmul":
            a, b = graph.node(n.operands[0]), graph.node(n.operands[1])
            m, k, nn = a.shape[0], a.shape[1], b.shape[1]
            total += elem_bytes * (m * k + k * nn) + 4 * m * nn
    return total


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples for one GPU, every 20 ms, each with nvidia-smi's own time stamp.
    It is started before the warm-up steps (nvidia-smi needs a moment to come up); the caller marks the wall-clock
    window of the load, and only samples taken inside that window are summarised."""

    QUERY = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    MIN_LOAD_S = 0.5  # a timed region shorter than this is followed by more of the same steps until it has lasted this long

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None
        self.window = None        # (begin, end of the timed region, end of the load) in time.time() seconds
        self.timed_steps_only = True

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def wait_for_first_sample(self, limit_s: float = 3.0):
        """Blocks until nvidia-smi has printed a sample (or the limit passes), so that the load is sampled from its start."""
        t0 = time.time()
        while self.proc is not None and not self.lines and time.time() - t0 < limit_s:
            time.sleep(0.01)

    @staticmethod
    def _stamp(text):
        import datetime
        try:
            return datetime.datetime.strptime(text, "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        sm, smax, power, reasons, in_timed, sm_timed = [], [], [], set(), 0, []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [t.strip() for t in line.split(",")]
            if len(f) < 10:
                continue
            stamp = self._stamp(f[0])
            if self.window is not None:
                if stamp is None or not (self.window[0] <= stamp <= self.window[2]):
                    continue
            try:
                sm.append(float(f[2]))
                smax.append(float(f[3]))
            except ValueError:
                continue
            if self.window is not None and stamp <= self.window[1]:
                in_timed += 1
                sm_timed.append(sm[-1])
            try:
                power.append(float(f[4]))
            except ValueError:
                pass
            for name, val in zip(names, f[6:10]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        out = {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
               "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(power) if power else None}
        if self.window is not None:
            out["samples_in_timed_region"] = in_timed
            out["sm_mhz_timed_region"] = float(np.median(sm_timed)) if sm_timed else None
            out["window"] = ("the timed region" if self.timed_steps_only else
                             f"the timed region ({(self.window[1] - self.window[0]) * 1e3:.0f} ms) and the same steps repeated "
                             f"right behind it, untimed, until {self.MIN_LOAD_S} s of load had passed")
        return out


def make_inputs(graph, dist, seed):
    """Seeded synthetic inputs of the workload's shapes and distribution (N(0,1) or uniform(-1,1)), float32.
    numpy's PCG64 generator: a 65536 x 2048 tensor takes about a second, where the oracle's scalar splitmix64
    stream (the one the parity tests feed to GPU and oracle alike) takes most of a minute."""
    ins = []
    for k, name in enumerate(graph.inputs):
        shape = graph.node(name).shape
        n = int(np.prod(shape))
        rng = np.random.default_rng(seed + k)
        if dist == "normal":
            v = rng.standard_normal(n, dtype=np.float32)
        else:
            v = rng.random(n, dtype=np.float32)
            v *= 2.0
            v -= 1.0
        ins.append(v.reshape(shape))
    return ins


def workload_config(workload, dims):
    """The `config` object both arms print for a workload."""
    name, _, matmul, batch_dim, kind, dist = WORKLOADS[workload]
    return {"workload": workload, "graph": name, "dims": dims, "matmul": matmul, "sharded_dim": batch_dim,
            "inputs": f"{dist}, seeded (numpy PCG64, seed 1 + 1000*rank)",
            "l2": "a step whose arena is below 256 MiB is timed on its own after a 256 MiB overwrite that flushes L2; "
                  "larger steps stream more than the 126 MB L2 holds and run back to back"}


def cpu_sample(oracle, path, dims, batch_dim, kind, dist, rows_cap, threads=None):
    """The CPU port (oracle/cpu_baseline.py over oracle_kernels.c) prepared on a row sample of the workload."""
    from oracle import cpu_baseline

    sample_dims = dict(dims)
    lead = batch_dim or ("M" if "M" in dims else None)
    rows_full = dims[lead] if lead else 1
    rows = min(rows_full, rows_cap)
    if lead:
        sample_dims[lead] = rows
    g = oracle.parse_mcg_file(path, sample_dims)
    plan = cpu_baseline.CpuPlan(g, threads or cpu_baseline.max_threads())
    ins = make_inputs(g, dist, 1)
    return plan, ins, algorithmic_work(oracle, g, kind), plan.threads, f"{rows} of {rows_full} rows of '{lead}'"


def cpu_sample_rate(oracle, path, dims, batch_dim, kind, dist, seconds_target=10.0, threads=None, rows_cap=None):
    """Times the CPU port on a bounded sample; returns (rate, threads, description)."""
    cap = rows_cap or (2048 if kind == "bytes" else 1024)
    plan, ins, work, threads, what = cpu_sample(oracle, path, dims, batch_dim, kind, dist, cap, threads)
    plan.run(ins)  # warm
    t0, reps = time.perf_counter(), 0
    while True:
        plan.run(ins)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > seconds_target or reps >= 200:
            break
    rate = work * reps / dt / (1e9 if kind == "bytes" else 1e12)
    return rate, threads, f"{what}, {reps} runs in {dt:.1f} s, {plan.how}"


def run_reference_arm(args):
    """The reference's CPU path, timed on host cores (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import reference_cpu as oracle
    import minicompiler_b200 as mc

    name, dims, matmul, batch_dim, kind, dist = WORKLOADS[args.workload]
    path = mc.graph_path(name)
    plan, ins, work, threads, what = cpu_sample(oracle, path, dims, batch_dim, kind, dist, 2048 if kind == "bytes" else 1024)
    for _ in range(max(1, min(args.warmup, 3))):
        plan.run(ins)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        plan.run(ins)
    dt = time.perf_counter() - t0
    unit = "GB/s" if kind == "bytes" else "TFLOP/s"
    value = work * args.steps / dt / (1e9 if kind == "bytes" else 1e12)
    line = {
        "impl": "reference", "metric": "fused-eltwise HBM GB/s" if kind == "bytes" else "graph TFLOP/s", "value": value, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong" if batch_dim is not None and args.gpus > 1 else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, dims),
        "note": "reference CPU path = C port of its CPU kernels in FP32 (Eigen 3.4.0 is absent, so the reference's own CPU "
                f"backend cannot be built); each step runs {what}",
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": f"{what} per step"},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


DEFAULT_ALSO = "c2,c4_bf16,c4_bf16_16384,c4_bf16_m128,c3_tf32,c3_fp32,c1"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c5_f16", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--also", default=None,
                    help="comma-separated extra workloads measured briefly (N=1 only); default: "
                         f"{DEFAULT_ALSO} beside the default workload, nothing beside any other; 'none' turns it off")
    ap.add_argument("--options", default="", help="extra compile options, e.g. gemm_variant=2,fuse_epilogue=0 (for A/B measurements)")
    ap.add_argument("--dims", default="", help="override dims of the workload, e.g. M=4096,N=8192 (for small profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.also is None:
        args.also = DEFAULT_ALSO if (args.workload == "c5_f16" and not args.dims and not args.options) else ""
    if args.also == "none":
        args.also = ""

    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        # Started by hand for several GPUs: one rank per GPU is what torch.distributed.run sets up.
        os.execvp(sys.executable, [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
                                   "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29500"),
                                   str(Path(__file__).resolve()), *sys.argv[1:]])

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    import minicompiler_b200 as mc
    from oracle import reference_cpu as oracle  # checker / CPU baseline only; never on the measured path

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: no CUDA device is visible and there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    comm_box = []

    def library_comm():
        """The library's own NCCL communicator (mcd_nccl_*): rank 0 makes the unique id, torch.distributed carries
        its 128 bytes to the others."""
        if not comm_box:
            uid = [mc.Communicator.unique_id() if rank == 0 else None]
            dist.broadcast_object_list(uid, src=0)
            comm_box.append(mc.Communicator(world, rank, uid[0], local_rank, timeout_s=120.0))
        return comm_box[0]

    def measure(workload, steps, warmup, with_e2e, with_cpu):
        name, dims, matmul, batch_dim, kind, dist_name = WORKLOADS[workload]
        if args.dims and workload == args.workload:
            dims = dict(dims) | {k: int(v) for k, v in (kv.split("=") for kv in args.dims.split(","))}
        path = mc.graph_path(name)
        my_dims, scaling = dict(dims), "weak"
        if world > 1 and batch_dim is not None:
            dims_str, row_offset, rows = mc.shard_dims(path, dims, batch_dim, rank, world)
            my_dims = {k: int(v) for k, v in (kv.split("=") for kv in dims_str.split(","))}
            scaling = "strong"
        compile_options = {"device": local_rank, "matmul": matmul}
        if args.options:
            compile_options |= dict(kv.split("=") for kv in args.options.split(","))
        exe = mc.CompiledGraph(path, dims=my_dims, options=compile_options)
        if world > 1:
            # Constants are generated identically on every rank; one NCCL broadcast over NVLink, issued by the
            # library on its own communicator, makes rank 0's copy the one everybody uses. It is the only
            # collective on this path (an output is gathered only where a caller wants it assembled).
            exe.replicate_constants(library_comm(), root=0)
        g = oracle.parse_mcg_file(path, my_dims)
        work_rank = algorithmic_work(oracle, g, kind)
        ins = make_inputs(g, dist_name, 1 + 1000 * rank)
        pinned_in = [torch.from_numpy(a.reshape(-1)).pin_memory() for a in ins]
        del ins
        pinned_out = [torch.empty(n, dtype=torch.float32).pin_memory() for n in exe.output_elements]
        exe.upload([t.numpy() for t in pinned_in])
        # A stream of our own: torch's default stream has handle 0, which mc_enqueue reads as "the executable's
        # own stream", and CUDA events only see the stream they are recorded on.
        stream = torch.cuda.Stream()
        launches_per_step = exe.kernel_launches

        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        for _ in range(warmup):
            exe.enqueue(stream.cuda_stream)
        torch.cuda.synchronize()
        if rank == 0:
            sampler.wait_for_first_sample()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        load_begin = time.time()
        # A working set that fits the 126 MB L2 would be served from it on every repeat: then each step is
        # timed on its own and a 256 MiB buffer is overwritten between steps to flush the cache.
        flush_l2 = exe.arena_bytes < (256 << 20)
        count0 = mc.lib().mcd_launch_count()
        if flush_l2:
            scrub = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
            starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
            stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
            with torch.cuda.stream(stream):
                for i in range(steps):
                    scrub.fill_(i & 0xFF)
                    starts[i].record(stream)
                    exe.enqueue(stream.cuda_stream)
                    stops[i].record(stream)
            torch.cuda.synchronize()
            step_ms = [starts[i].elapsed_time(stops[i]) for i in range(steps)]
        else:
            events = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
            events[0].record(stream)
            for i in range(steps):
                exe.enqueue(stream.cuda_stream)
                events[i + 1].record(stream)
            torch.cuda.synchronize()
            step_ms = [events[i].elapsed_time(events[i + 1]) for i in range(steps)]
        count1 = mc.lib().mcd_launch_count()
        timed_end = time.time()
        # nvidia-smi samples every 20 ms at best: a timed region of a few tens of milliseconds is followed, without a
        # gap, by the same steps (untimed) so that the clocks under this load are seen by more than a sample or two.
        while time.time() - load_begin < ClockSampler.MIN_LOAD_S:
            sampler.timed_steps_only = False
            for _ in range(max(1, steps // 4)):
                exe.enqueue(stream.cuda_stream)
            torch.cuda.synchronize()
        sampler.window = (load_begin, timed_end, time.time())
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
        exe.synchronize()  # also surfaces a kernel that gave up a bounded wait
        total_ms = float(sum(step_ms)) if flush_l2 else events[0].elapsed_time(events[-1])
        per_step = sorted(step_ms)
        t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
        w = torch.tensor([float(work_rank)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(w, op=dist.ReduceOp.SUM)
        total_ms, work_all = float(t.item()), float(w.item())
        denom = 1e9 if kind == "bytes" else 1e12
        value = work_all * steps / (total_ms * 1e-3) / denom

        e2e = None
        if with_e2e:
            in_ptrs = [t_.data_ptr() for t_ in pinned_in]
            out_ptrs = [t_.data_ptr() for t_ in pinned_out]
            e2e_steps = max(3, min(steps, 10))
            exe.run_ptrs(in_ptrs, out_ptrs)
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                exe.run_ptrs(in_ptrs, out_ptrs)  # H2D from pinned memory, kernels, D2H into pinned memory, synchronized
            dt = time.perf_counter() - t0
            tt = torch.tensor([dt], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e2e = {"value": work_all * e2e_steps / float(tt.item()) / denom, "unit": "GB/s" if kind == "bytes" else "TFLOP/s",
                   "h2d_bytes_per_step": int(sum(a.numel() * 4 for a in pinned_in)),
                   "d2h_bytes_per_step": int(sum(a.numel() * 4 for a in pinned_out)), "steps": e2e_steps,
                   "ms_per_step": float(tt.item()) / e2e_steps * 1e3,
                   "timing": "host wall clock around mc_run (it synchronizes), max over ranks",
                   "path": "mc_run on pinned host buffers: a graph whose rows are independent is cut into row slices whose "
                           "H2D copy, kernels and D2H copy overlap on three streams; any other graph is copied in, run and "
                           "copied out"}

        peaks = measured_peaks()
        median_ms = per_step[len(per_step) // 2]
        avg_ms = total_ms / steps
        min_bytes = 0
        if kind == "bytes":
            achieved = work_rank / (avg_ms * 1e-3) / 1e9
            peak, unit, bound = peaks["hbm_gbs"], "GB/s", "hbm"
            peak_kind = "copy bandwidth"
        else:
            achieved = work_rank / (avg_ms * 1e-3) / 1e12
            sustained = total_ms > 1000.0
            base = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
            peak = {"f32": 2 * 148 * 128 * 1.965e9 / 1e12, "tf32": base / 2.0}.get(DTYPES[matmul], base)
            unit, bound = "TFLOP/s", "tensor" if matmul != "auto" else "fp32-fma"
            peak_kind = ("FP32 FMA peak at the maximum SM clock (2 x 148 SMs x 128 lanes x 1965 MHz)" if matmul == "auto" else
                         ("sustained" if sustained else "burst") + " cuBLAS bf16 GEMM" + (", halved for TF32" if DTYPES[matmul] == "tf32" else ""))
            # A shape whose arithmetic intensity lies below the ridge of the two peaks is bound by streaming its
            # operands, not by the math: its roofline is the HBM one (skinny matmuls: 16 or 128 rows against 8192^2).
            min_bytes = matmul_operand_bytes(g, 4 if DTYPES[matmul] in ("f32", "tf32") else 2)
            if min_bytes > 0 and work_rank / min_bytes < peak * 1e12 / (peaks["hbm_gbs"] * 1e9):
                achieved = min_bytes / (avg_ms * 1e-3) / 1e9
                peak, unit, bound = peaks["hbm_gbs"], "GB/s", "hbm"
                peak_kind = "copy bandwidth (operands once + FP32 result once; intensity below the ridge)"
        traffic = None
        tfile = ROOT / "profiles" / "ncu_traffic.json"
        if tfile.exists():
            try:
                traffic = json.loads(tfile.read_text()).get(workload, {}).get("dram_bytes_per_launch")
            except Exception:
                traffic = None
        roofline = {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                    "traffic": traffic, "peak_source": f"of {peaks['source']}: {peak_kind}",
                    "kernel_ms_avg": avg_ms / max(1, launches_per_step), "step_ms_median": median_ms,
                    "launches_per_step": launches_per_step,
                    "algorithmic_per_launch": (min_bytes if (kind == "flops" and bound == "hbm") else work_rank) / max(1, launches_per_step),
                    "kernels": exe.matmul_kernels if kind == "flops" else ["mc_elementwise (generated)"]}

        cpu = None
        if with_cpu and rank == 0:
            rate, threads, sample = cpu_sample_rate(oracle, path, dims, batch_dim, kind, dist_name)
            one_rate, _, one_sample = cpu_sample_rate(oracle, path, dims, batch_dim, kind, dist_name, seconds_target=6.0, threads=1,
                                                      rows_cap=512 if kind == "bytes" else 128)
            cpu = {"value": rate, "unit": "GB/s" if kind == "bytes" else "TFLOP/s", "cores": threads, "kind": "port", "sample": sample,
                   "one_thread": {"value": one_rate, "cores": 1, "sample": one_sample,
                                  "note": "the reference's own CPU configuration is single-threaded (bench/harness.hpp:254)"}}

        result = {
            "metric": "fused-eltwise HBM GB/s" if kind == "bytes" else "graph TFLOP/s", "value": value,
            "unit": "GB/s" if kind == "bytes" else "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": avg_ms, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": DTYPES[matmul], "data": "synthetic",
            "config": workload_config(workload, dims),
            "per_rank_dims": my_dims, "matmul_kernels": exe.matmul_kernels, "kernel_launches_per_step": launches_per_step,
            "l2_flushed_between_steps": flush_l2,
            "e2e": e2e, "gpu_launches": int(count1 - count0), "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks,
            "jit_compile_ms": exe.jit_compile_ms, "arena_bytes": exe.arena_bytes,
        }
        exe.release()
        del pinned_in, pinned_out
        return result

    line = measure(args.workload, args.steps, args.warmup, not args.no_e2e, not args.no_cpu_baseline)
    if args.also and world == 1:
        extra = []
        for wl in [w for w in args.also.split(",") if w]:
            try:
                r = measure(wl, max(5, min(args.steps, 20)), 3, False, False)
                extra.append({k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "dtype", "roofline", "gpu_launches",
                                                "matmul_kernels", "clocks")} | {"workload": wl, "dims": r["config"]["dims"]})
            except Exception as e:  # an extra must never lose the headline line
                extra.append({"workload": wl, "error": str(e)[:300]})
        line["also"] = extra
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        if comm_box:
            comm_box[0].destroy()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
