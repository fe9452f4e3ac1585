"""The reference's GPU benchmark suites, re-hosted on this backend (needs a B200).

    python -m minicompiler_b200.bench_suites --suite elementwise|matmul|tensor_core|rows|profile|all [--out FILE]

They follow bench/bench_cuda.cpp of the reference:
  elementwise   the GELU chain at M in {1,16,256,1024,4096,16384}, N=4096, unfused (passes
                dne,fold,dne) against fused (default): time, bandwidth from the bytes the executed graph
                moves, speed-up (run_elementwise, bench_cuda.cpp:182-288).
  matmul        the FP32 kernel against cuBLAS SGEMM on square and split-K shapes (run_matmul, :543-673).
  tensor_core   the tcgen05 kernels against cuBLAS in the same format (run_tensor_core, :700-851).
  rows          (no counterpart in the reference) softmax and LayerNorm graphs built from the row reductions
                against torch's kernels.
  profile       one launch of every kernel, each inside its own NVTX range "<workload>.<kernel>", nothing timed,
                for `ncu --nvtx --nvtx-include "<label>/"` (run_profile, :860-928; `--list` prints the labels,
                `--only LABEL` runs one).
Every variant is checked before it is timed: 1000 sampled outputs against float64 dot products
(the method of run_and_check, :386-436). cuBLAS is reached through torch.matmul and is a comparison
column only, never part of the product.
Matmul rows are timed the way the reference times them (time_graphs, :445-493): the launch is captured in a CUDA
graph between two event-record nodes and the graph is replayed, so the time between the events leaves out the
host's cost of launching, which differs between cuBLAS and these kernels. The elementwise and rows suites time
CUDA events around `mc_enqueue` on a side stream. Median of `--rounds` rounds, L2 flushed between rounds for
working sets that fit it.
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _median_ms(fn, stream, rounds, flush):
    import torch

    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    times = []
    with torch.cuda.stream(stream):
        for i in range(rounds):
            if scrub is not None:
                scrub.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            times.append((e0, e1))
    torch.cuda.synchronize()
    return float(np.median([a.elapsed_time(b) for a, b in times]))


def _graph_median_ms(mc, fn, stream, rounds, flush):
    """Median time of `fn` (which enqueues on `stream`) inside a replayed CUDA graph, between two event nodes."""
    import torch

    lib = mc.lib()
    start, stop = C.c_void_p(), C.c_void_p()
    assert lib.mcd_event_create(C.byref(start)) == 0 and lib.mcd_event_create(C.byref(stop)) == 0
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
        assert lib.mcd_event_record_external(start, C.c_void_p(stream.cuda_stream)) == 0
        fn()
        assert lib.mcd_event_record_external(stop, C.c_void_p(stream.cuda_stream)) == 0
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    times, ms = [], C.c_float()
    with torch.cuda.stream(stream):
        for i in range(rounds + 3):
            if scrub is not None:
                scrub.fill_(i & 0xFF)
            graph.replay()
            assert lib.mcd_event_elapsed_ms(start, stop, C.byref(ms)) == 0  # waits for the stop event
            if i >= 3:
                times.append(ms.value)
    torch.cuda.synchronize()
    del graph
    lib.mcd_event_destroy(start)
    lib.mcd_event_destroy(stop)
    return float(np.median(times))


def _bytes_moved(mc, path, dims, passes):
    """Every compute node's output once plus each distinct non-scalar operand once, on the graph as executed
    (bytes_moved, bench_cuda.cpp:76-95), read off the printed graph."""
    import re

    total = 0
    text = mc.HostGraph(path, dims=dims, passes=passes).print()
    shapes = {}
    for line in text.splitlines():
        m = re.match(r"\s+%(\d+) \S+ = (\S+)(.*) : f32\[(.*?)\]", line)
        if not m:
            continue
        idx, op, rest, shape = int(m.group(1)), m.group(2), m.group(3), m.group(4)
        n = int(np.prod([int(t) for t in shape.split(",") if t])) if shape else 1
        shapes[idx] = n
        if op in ("input", "const"):
            continue
        total += 4 * n
        for operand in sorted(set(int(t) for t in re.findall(r"%(\d+)", rest))):
            if shapes[operand] > 1:
                total += 4 * shapes[operand]
    return total


def _sampled_matmul_f64(a, b, rows, cols):
    a64 = a[rows, :].astype(np.float64)
    b64 = b[:, cols].astype(np.float64).T
    return np.einsum("ik,ik->i", a64, b64), np.einsum("ik,ik->i", np.abs(a64), np.abs(b64))


def suite_elementwise(mc, rounds):
    import torch

    path = mc.graph_path("c2_gelu_chain")
    stream = torch.cuda.Stream()
    rows = []
    for m in (1, 16, 256, 1024, 4096, 16384):
        dims = {"M": m, "N": 4096}
        x = np.random.default_rng(1).standard_normal(m * 4096, dtype=np.float32)
        entry = {"M": m, "N": 4096}
        outs = {}
        for label, passes in (("unfused", "dne,fold,dne"), ("fused", "default")):
            with mc.CompiledGraph(path, dims=dims, passes=passes) as exe:
                exe.upload([x])
                ms = _median_ms(lambda: exe.enqueue(stream.cuda_stream), stream, rounds, flush=m * 4096 * 8 < (200 << 20))
                outs[label] = exe.download()[0]
                moved = _bytes_moved(mc, path, dims, passes)
                entry[label] = {"ms": ms, "launches": exe.kernel_launches, "bytes_moved": moved, "gbs": moved / ms / 1e6}
        assert np.allclose(outs["fused"], outs["unfused"], rtol=1e-6, atol=1e-7)
        entry["speedup"] = entry["unfused"]["ms"] / entry["fused"]["ms"]
        rows.append(entry)
    return rows


def _check_sampled(got, a, b, u_in, k):
    rng = np.random.default_rng(0)
    rows, cols = rng.integers(0, a.shape[0], 1000), rng.integers(0, b.shape[1], 1000)
    exact, abs_dot = _sampled_matmul_f64(a, b, rows, cols)
    u32 = 2.0 ** -24
    gamma = k * u32 / (1 - k * u32)
    bound = (2 * u_in + u_in * u_in + 2 * gamma) * abs_dot + 2 * u32 * np.abs(exact) + (2 * k * 2.0 ** -25 if u_in else 0)
    err = np.abs(got[rows, cols].astype(np.float64) - exact)
    assert np.all(err <= bound), f"sampled check failed: worst {float(np.max(err / bound)):.2f}x the bound"
    return float(np.max(err / np.maximum(abs_dot, 1e-30)))


def _gemm_rows(mc, rounds, shapes, kernels):
    import torch

    text = "dim M = 8\ndim N = 8\ndim K = 8\ninput a : f32[M, K]\ninput b : f32[K, N]\nc = matmul a, b\noutput c"
    stream = torch.cuda.Stream()
    rows = []
    for m, n, k in shapes:
        a = mc.uniform_values(m * k, 1, -1, 1).reshape(m, k)
        b = mc.uniform_values(k * n, 2, -1, 1).reshape(k, n)
        ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        flops = 2.0 * m * n * k
        small = (m * k + k * n + m * n) * 4 < (200 << 20)
        entry = {"m": m, "n": n, "k": k}
        for name, torch_dtype, tf32, u_in in kernels:
            with mc.CompiledGraph(text=text, dims={"M": m, "N": n, "K": k}, options={"matmul": name}) as exe:
                exe.upload([a, b])
                exe.enqueue(stream.cuda_stream)
                got = exe.download()[0].reshape(m, n)
                rel = _check_sampled(got, a, b, u_in, k)
                ms = _graph_median_ms(mc, lambda: exe.enqueue(stream.cuda_stream), stream, rounds, small)
                ran = exe.matmul_kernels
            torch.backends.cuda.matmul.allow_tf32 = tf32
            xa, xb = ta.to(torch_dtype), tb.to(torch_dtype)
            out = torch.empty((m, n), dtype=torch_dtype, device="cuda")
            lib_ms = _graph_median_ms(mc, lambda: torch.matmul(xa, xb, out=out), stream, rounds, small)
            torch.backends.cuda.matmul.allow_tf32 = False
            entry[name] = {"ms": ms, "tflops": flops / ms / 1e9, "cublas_ms": lib_ms, "cublas_tflops": flops / lib_ms / 1e9,
                           "pct_of_cublas": 100.0 * lib_ms / ms, "ran": ran, "max_err_over_abs_dot": rel}
        rows.append(entry)
    return rows


def suite_matmul(mc, rounds, shapes=None):
    import torch

    shapes = shapes or [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (256, 2048, 512), (128, 512, 2048), (256, 1024, 1024),
              (8192, 4096, 1024)]
    return _gemm_rows(mc, rounds, shapes, [("auto", torch.float32, False, 0.0)])


def suite_tensor_core(mc, rounds, shapes=None):
    import torch

    shapes = shapes or [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (16, 8192, 8192), (128, 8192, 8192),
              (1024, 1024, 65536), (65536, 2048, 2048)]
    kernels = [("tensor_core_tf32", torch.float32, True, 2.0 ** -11), ("tensor_core_bf16", torch.bfloat16, False, 2.0 ** -8),
               ("tensor_core_f16", torch.float16, False, 2.0 ** -11)]
    return _gemm_rows(mc, rounds, shapes, kernels)


def suite_rows(mc, rounds):
    """The extension graphs built from row reductions (softmax, LayerNorm over the last dimension) against
    torch.softmax / torch.nn.functional.layer_norm: time, and bandwidth from read x + write y. Each result is
    checked against a float64 computation of the same rows first."""
    import torch

    stream = torch.cuda.Stream()
    rows = []
    for name, m, n in [("x1_softmax", 8192, 128), ("x1_softmax", 8192, 1024), ("x1_softmax", 8192, 4096), ("x1_softmax", 8192, 8192),
                       ("x1_softmax", 4096, 16384), ("x1_softmax", 2048, 32768), ("x2_layernorm", 16384, 4096), ("x2_layernorm", 65536, 4096)]:
        x = np.random.default_rng(2).standard_normal(m * n, dtype=np.float32)
        t = torch.from_numpy(x).cuda().reshape(m, n)
        with mc.CompiledGraph(mc.graph_path(name), dims={"M": m, "N": n}) as exe:
            exe.upload([x])
            exe.enqueue(stream.cuda_stream)
            got = exe.download()[0].reshape(m, n)
            launches = exe.kernel_launches
            sample = got[:: max(1, m // 64)].astype(np.float64)
            x64 = x.reshape(m, n)[:: max(1, m // 64)].astype(np.float64)
            if name == "x1_softmax":
                e = np.exp(x64 - x64.max(axis=1, keepdims=True))
                want = e / e.sum(axis=1, keepdims=True)
                lib = lambda: torch.softmax(t, dim=-1)  # noqa: E731
            else:
                gamma = mc.HostGraph(mc.graph_path(name), dims={"M": 1, "N": n}, passes="none").constant("gamma").astype(np.float64)
                beta = mc.HostGraph(mc.graph_path(name), dims={"M": 1, "N": n}, passes="none").constant("beta").astype(np.float64)
                mean = x64.sum(axis=1, keepdims=True) / 4096.0  # the graph's constant 1/4096, whatever N is
                c = x64 - mean
                want = c / np.sqrt((c * c).sum(axis=1, keepdims=True) / 4096.0 + 1e-5) * gamma + beta
                lib = lambda: torch.nn.functional.layer_norm(t, (n,))  # noqa: E731
            assert np.allclose(sample, want, rtol=2e-5, atol=1e-6), f"{name} {m}x{n}"
            small = m * n * 8 < (200 << 20)
            ms = _median_ms(lambda: exe.enqueue(stream.cuda_stream), stream, rounds, small)
        with torch.cuda.stream(stream):
            lib_ms = _median_ms(lib, stream, rounds, small)
        moved = 2 * 4 * m * n
        rows.append({"graph": name, "M": m, "N": n, "launches": launches, "ms": ms, "gbs": moved / ms / 1e6, "torch_ms": lib_ms,
                     "torch_gbs": moved / lib_ms / 1e6, "pct_of_torch": 100.0 * lib_ms / ms})
    return rows


PROFILE_SHAPES = [(2048, 2048, 2048), (512, 512, 512), (128, 2048, 512)]  # m, k, n: the reference's three
PROFILE_KERNELS = ["auto", "tensor_core_tf32", "tensor_core_bf16", "tensor_core_f16"]


def profile_labels():
    labels = ["gelu_64MB.unfused", "gelu_64MB.fused"]
    for m, k, n in PROFILE_SHAPES:
        base = f"matmul_{m}x{k}x{n}"
        labels += [f"{base}.{kernel}" for kernel in PROFILE_KERNELS]
        labels += [f"{base}.cublas", f"{base}.cublas_tf32", f"{base}.cublas_bf16", f"{base}.cublas_f16"]
    return labels


def suite_profile(mc, only=""):
    """One launch of every kernel inside its own NVTX range; each runs once outside the ranges first, so module
    loading and first-call set-up stay out of the profile. Returns the labels that ran."""
    import torch

    lib = mc.lib()
    stream = torch.cuda.Stream()
    ran = []

    def profiled(label, launch):
        if only and label != only:
            return
        with torch.cuda.stream(stream):
            launch()
            torch.cuda.synchronize()
            lib.mcd_range_push(label.encode())
            launch()
            torch.cuda.synchronize()
            lib.mcd_range_pop()
        ran.append(label)
        print(label)

    if not only or only.startswith("gelu_64MB."):
        x = np.random.default_rng(1).standard_normal(4096 * 4096, dtype=np.float32)
        for name, passes in (("unfused", "dne,fold,dne"), ("fused", "default")):
            with mc.CompiledGraph(mc.graph_path("c2_gelu_chain"), dims={"M": 4096, "N": 4096}, passes=passes) as exe:
                exe.upload([x])
                profiled(f"gelu_64MB.{name}", lambda: exe.enqueue(stream.cuda_stream))
    text = "dim M = 8\ndim N = 8\ndim K = 8\ninput a : f32[M, K]\ninput b : f32[K, N]\nc = matmul a, b\noutput c"
    for m, k, n in PROFILE_SHAPES:
        base = f"matmul_{m}x{k}x{n}"
        if only and not only.startswith(base + "."):
            continue
        a = mc.uniform_values(m * k, 1, -1, 1).reshape(m, k)
        b = mc.uniform_values(k * n, 2, -1, 1).reshape(k, n)
        for kernel in PROFILE_KERNELS:
            with mc.CompiledGraph(text=text, dims={"M": m, "N": n, "K": k}, options={"matmul": kernel}) as exe:
                exe.upload([a, b])
                profiled(f"{base}.{kernel}", lambda: exe.enqueue(stream.cuda_stream))
        ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        for suffix, dtype, tf32 in (("cublas", torch.float32, False), ("cublas_tf32", torch.float32, True),
                                    ("cublas_bf16", torch.bfloat16, False), ("cublas_f16", torch.float16, False)):
            xa, xb = ta.to(dtype), tb.to(dtype)
            torch.backends.cuda.matmul.allow_tf32 = tf32
            profiled(f"{base}.{suffix}", lambda: torch.matmul(xa, xb))
            torch.backends.cuda.matmul.allow_tf32 = False
    return ran


def _parse_shapes(text):
    return [tuple(int(t) for t in item.split("x")) for item in text.split(",") if item]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--suite", default="all", choices=["elementwise", "matmul", "tensor_core", "rows", "profile", "all"])
    ap.add_argument("--rounds", type=int, default=30)
    ap.add_argument("--out", default="")
    ap.add_argument("--shapes", default="", help="matmul / tensor_core: MxNxK,MxNxK,... instead of the suite's own shapes")
    ap.add_argument("--only", default="", help="profile: run this label only")
    ap.add_argument("--list", action="store_true", help="profile: print the labels and exit (needs no GPU)")
    args = ap.parse_args()
    if args.suite == "profile" and args.list:
        print("\n".join(profile_labels()))
        return
    import torch

    import minicompiler_b200 as mc

    if not torch.cuda.is_available():
        raise SystemExit("the suites need a B200")
    if args.suite == "profile":
        ran = suite_profile(mc, args.only)
        print(f"profiled {len(ran)} launch(es) on {torch.cuda.get_device_name(0)}")
        return
    result = {"device": torch.cuda.get_device_name(0)}
    if args.suite in ("elementwise", "all"):
        result["elementwise"] = suite_elementwise(mc, args.rounds)
    if args.suite in ("matmul", "all"):
        result["matmul"] = suite_matmul(mc, args.rounds, _parse_shapes(args.shapes) if args.suite == "matmul" else None)
    if args.suite in ("tensor_core", "all"):
        result["tensor_core"] = suite_tensor_core(mc, args.rounds, _parse_shapes(args.shapes) if args.suite == "tensor_core" else None)
    if args.suite in ("rows", "all"):
        result["rows"] = suite_rows(mc, args.rounds)
    text = json.dumps(result, indent=1)
    if args.out:
        Path(args.out).write_text(text)
    print(text)


if __name__ == "__main__":
    main()
