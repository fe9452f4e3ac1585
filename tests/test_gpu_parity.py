"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a B200.

Tolerances are the reference's own between its CUDA and CPU backends
(tests/test_cuda_backend.cpp:66-72, :119-162, :164-219, :395-437) and the per-precision bars of
the build target: 1e-5 relative for elementwise FP32 graphs, 1e-4 for FP32 GEMM graphs, 5e-3
(TF32) and 2e-2 (BF16/FP16) against a norm-scaled FP32 reference.
"""

import ctypes as C
import json

import numpy as np
import pytest

from conftest import GOLDEN

pytestmark = pytest.mark.gpu

U32 = 2.0 ** -24


def all_close(actual, expected, rtol, atol):
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    assert a.shape == e.shape
    both_nan = np.isnan(a) & np.isnan(e)
    err = np.abs(a - e)
    bad = ~(err <= atol + rtol * np.abs(e)) & ~both_nan & ~(a == e)
    if bad.any():
        i = int(np.argmax(np.where(bad, err, 0)))
        return False, f"{int(bad.sum())} of {a.size} elements differ; worst at [{i}]: actual {a[i]!r}, expected {e[i]!r}"
    return True, ""


def run_graph(mc, text=None, path=None, dims=None, passes="default", options=None, inputs=None):
    with mc.CompiledGraph(path, text=text, dims=dims, passes=passes, options=options or {}) as exe:
        return exe.run(inputs)


def oracle_inputs(oracle, text=None, path=None, dims=None, seed=1, lo=-1.0, hi=1.0):
    d = None
    if dims:
        d = dims if isinstance(dims, dict) else {k: int(v) for k, v in (kv.split("=") for kv in dims.split(","))}
    g = oracle.parse_mcg(text, d) if text is not None else oracle.parse_mcg_file(path, d)
    return g, oracle.make_random_inputs(g, seed, lo, hi)


# ------------------------------------------------------------- device layer


def test_device_is_a_b200_and_reports_sane_peaks(mc):
    buf = C.create_string_buffer(4096)
    assert mc.lib().mc_gpu_device_json(None, 0, buf, len(buf)) == 0
    info = json.loads(buf.value.decode())
    assert info["compute_capability"].startswith("10.")
    assert info["sm_count"] >= 100 and info["peak_bandwidth_gbs"] > 1000 and info["peak_fp32_gflops"] > 10000


# -------------------------------------------------------------- elementwise


@pytest.mark.parametrize("shape", ["[37, 29]", "[64, 64]", "[3, 1000]"])
def test_unary_ops_match_the_oracle(mc, oracle, shape):
    # tests/test_cuda_backend.cpp:85-101: exact for neg/relu, rtol 1e-6 + atol 1.2e-7 otherwise
    for op in ["neg", "exp", "log", "sqrt", "relu", "sigmoid", "tanh"]:
        text = f"input x : f32{shape}\ny = {op} x\noutput y"
        positive = op in ("log", "sqrt")
        g, ins = oracle_inputs(oracle, text, seed=11, lo=0.01 if positive else -6.0, hi=6.0)
        got = run_graph(mc, text=text, passes="none", inputs=ins)[0]
        if op in ("neg", "relu", "sqrt"):
            want = oracle.evaluate_f32(g, ins)[0]
            assert np.array_equal(got, want), op  # IEEE-exact on both sides (sqrtf is correctly rounded)
        else:
            ok, msg = all_close(got, oracle.evaluate_f64(g, ins)[0], 1e-6, 1.2e-7)
            assert ok, f"{op} {shape}: {msg}"


BROADCASTS = [("[17, 33]", "[17, 33]"), ("[17, 32]", "[]"), ("[]", "[17, 33]"), ("[17, 32]", "[32]"), ("[17, 33]", "[17, 1]"),
              ("[17, 1]", "[1, 33]"), ("[2, 3, 4]", "[3, 1]"), ("[5, 1, 6]", "[1, 4, 1]"), ("[16, 64]", "[16, 1]"),
              ("[4, 8, 16]", "[8, 1]"), ("[4, 8, 16]", "[4, 1, 16]")]


@pytest.mark.parametrize("sa,sb", BROADCASTS)
def test_binary_ops_are_bit_exact_for_every_broadcast_pattern(mc, oracle, sa, sb):
    # tests/test_cuda_backend.cpp:103-117
    for op in ["add", "sub", "mul", "div"]:
        text = f"input a : f32{sa}\ninput b : f32{sb}\ny = {op} a, b\noutput y"
        g, ins = oracle_inputs(oracle, text, seed=5, lo=0.5, hi=2.0)
        for options in ({}, {"vectorize": 0}, {"unroll": 1}):
            got = run_graph(mc, text=text, passes="none", options=options, inputs=ins)[0]
            assert np.array_equal(got, oracle.evaluate_f32(g, ins)[0]), (op, sa, sb, options)


def test_fused_arithmetic_is_bit_exact_and_tails_are_covered(mc, oracle):
    # A fused group of IEEE-exact ops must equal the oracle bit for bit (no FMA contraction), at sizes that
    # end inside a trip, inside a vector and inside a block.
    for n in [1, 3, 4, 1023, 1024, 1025, 4096 + 4, 256 * 4 * 4 * 3 + 8]:
        text = (f"input x : f32[{n}]\ninput y : f32[{n}]\nconst c : f32[] = 0.3\n"
                "a = mul x, y\nb = add a, x\nd = mul b, c\ne = sub d, y\nf = div e, b\noutput f")
        g, ins = oracle_inputs(oracle, text, seed=2, lo=0.5, hi=2.0)
        got = run_graph(mc, text=text, inputs=ins)[0]
        assert np.array_equal(got, oracle.evaluate_f32(g, ins)[0]), n


def test_benchmark_graphs_fused_and_unfused_match_the_oracle(mc, oracle):
    # tests/test_cuda_backend.cpp:395-416: rtol 1e-5, atol 1e-5 * max|expected|
    cases = [("ref_gelu_chain", "M=64,N=256", 1e-5), ("ref_matmul_bias_relu", "M=64,K=256,N=128", 1e-4),
             ("ref_mlp_block", "B=32,D=128,H=256", 1e-4)]
    for name, dims, rtol in cases:
        path = str(GOLDEN / "graphs" / f"{name}.mcg")
        g, ins = oracle_inputs(oracle, path=path, dims=dims)
        want = oracle.evaluate_f64(g, ins)[0]
        scale = float(np.max(np.abs(want)))
        for passes in ["none", "default"]:
            for options in ({}, {"fuse_epilogue": 0}):
                got = run_graph(mc, path=path, dims=dims, passes=passes, options=options, inputs=ins)[0]
                ok, msg = all_close(got, want, rtol, rtol * scale)
                assert ok, f"{name} {passes} {options}: {msg}"


def test_random_graphs_match_the_reference_evaluator(mc, oracle):
    # tests/test_cuda_backend.cpp:418-437: 1e-4 * scale, optimized and unoptimized; the expected values are the
    # reference's own evaluator outputs (tests/golden/evaluator.npz).
    gold = json.loads((GOLDEN / "host_logic.json").read_text())["random"]
    expected = np.load(GOLDEN / "evaluator.npz")
    for seed, entry in gold.items():
        g = oracle.parse_mcg(entry["mcg"])
        ins = oracle.make_random_inputs(g, 1)
        for passes in ["none", "default"]:
            outs = run_graph(mc, text=entry["mcg"], passes=passes, inputs=ins)
            for k, got in enumerate(outs):
                want = expected[f"random/{seed}/out{k}"]
                scale = max(1.0, float(np.max(np.abs(want))))
                ok, msg = all_close(got, want, 1e-4, 1e-4 * scale)
                assert ok, f"random graph {seed}, passes {passes}, output {k}: {msg}"


def test_buffer_reuse_launch_counts_and_repeatability(mc, oracle):
    # tests/test_cuda_backend.cpp:439-482
    chain = "input x : f32[1024]\n" + "".join(f"t{i} = tanh {'x' if i == 0 else 't' + str(i - 1)}\n" for i in range(8)) + "output t7"
    with mc.CompiledGraph(text=chain, passes="none") as exe:
        assert exe.intermediate_bytes == 2 * 4096 and exe.kernel_launches == 8
    path = str(GOLDEN / "graphs" / "ref_gelu_chain.mcg")
    for passes, launches in [("none", 11), ("dne,fold,dne", 9), ("default", 1)]:
        with mc.CompiledGraph(path, dims="M=16,N=64", passes=passes) as exe:
            assert exe.kernel_launches == launches
    path = str(GOLDEN / "graphs" / "ref_mlp_block.mcg")
    g, ins = oracle_inputs(oracle, path=path, dims="B=64,D=128,H=256")
    with mc.CompiledGraph(path, dims="B=64,D=128,H=256") as exe:
        first = exe.run(ins)[0].copy()
        exe.upload(ins)
        exe.enqueue()
        exe.enqueue()
        again = exe.download()[0]
        assert np.array_equal(first, again)
        with pytest.raises(mc.McError, match="expected 1 inputs, got 2"):
            exe.run([ins[0], ins[0]])


def test_outputs_that_are_inputs_or_constants(mc, oracle):
    text = "input x : f32[8]\nconst c : f32[4] = [1, 2, 3, 4]\ny = exp x\noutput x, c, y"
    g, ins = oracle_inputs(oracle, text)
    outs = run_graph(mc, text=text, inputs=ins)
    assert np.array_equal(outs[0], ins[0]) and list(outs[1]) == [1, 2, 3, 4]


# ------------------------------------------------------------------ matmuls

FP32_SHAPES = [(1, 1, 1), (3, 5, 7), (1, 1000, 1), (33, 257, 65), (65, 9, 63), (127, 129, 131), (128, 128, 128),
               (129, 13, 129), (256, 256, 256), (16, 4099, 16), (513, 77, 259), (129, 132, 260), (300, 1004, 36), (2, 12, 4)]
TC_SHAPES = [(1, 1, 1), (3, 5, 7), (33, 257, 65), (127, 129, 131), (128, 128, 128), (129, 33, 129), (16, 4099, 16),
             (300, 1004, 36), (2, 12, 4), (256, 256, 256), (384, 512, 640)]


def matmul_text(m, k, n):
    return f"input a : f32[{m}, {k}]\ninput w : f32[{k}, {n}]\nc = matmul a, w\noutput c"


def exact_and_abs(a, b):
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    return a64 @ b64, np.abs(a64) @ np.abs(b64)


def check_bound(got, exact, abs_dot, k, u_in, subnormals, label):
    gamma = k * U32 / (1.0 - k * U32)
    if u_in == 0.0:
        bound = 2.0 * gamma * abs_dot + 2.0 * U32 * np.abs(exact)
    else:
        tiny = 2.0 * k * 2.0 ** -25 if subnormals else 0.0
        bound = (2.0 * u_in + u_in * u_in + 2.0 * gamma) * abs_dot + 2.0 * U32 * np.abs(exact) + tiny
    err = np.abs(got.astype(np.float64).reshape(exact.shape) - exact)
    bad = ~(err <= bound)
    assert not bad.any(), (f"{label}: {int(bad.sum())} of {bad.size} outside the bound; first at {np.argwhere(bad)[0].tolist()} "
                           f"got {got.reshape(exact.shape)[tuple(np.argwhere(bad)[0])]!r} exact {exact[tuple(np.argwhere(bad)[0])]!r}")


@pytest.mark.parametrize("kernel", ["auto", "split_k", "double_buffered", "naive"])
def test_fp32_matmul_within_the_dot_product_bound(mc, oracle, kernel):
    # tests/test_cuda_backend.cpp:119-162
    for m, k, n in FP32_SHAPES:
        text = matmul_text(m, k, n)
        g, ins = oracle_inputs(oracle, text, seed=3)
        got = run_graph(mc, text=text, options={"matmul": kernel}, inputs=ins)[0]
        exact, abs_dot = exact_and_abs(ins[0], ins[1])
        check_bound(got, exact, abs_dot, k, 0.0, False, f"{kernel} {m}x{k}x{n}")


def _torch():
    import torch

    return torch


def _device_gemm(mc, arith, a, b, splits, b_transposed=False, half=None, variant=0, tile_n=0):
    """Calls mcd_gemm directly with device buffers held by torch; C is pre-filled with NaN."""
    torch = _torch()
    lib = mc.lib()

    class GemmArgs(C.Structure):
        _fields_ = [("arith", C.c_int), ("m", C.c_int), ("n", C.c_int), ("k", C.c_int), ("a", C.c_void_p), ("b", C.c_void_p),
                    ("lda", C.c_longlong), ("ldb", C.c_longlong), ("b_transposed", C.c_int), ("c", C.c_void_p),
                    ("ldc", C.c_longlong), ("c16", C.c_void_p), ("c16_kind", C.c_int), ("ldc16", C.c_longlong),
                    ("splits", C.c_int), ("workspace", C.c_void_p), ("function", C.c_void_p), ("reduce_function", C.c_void_p),
                    ("epilogue_inputs", C.c_void_p * 6), ("num_epilogue_inputs", C.c_int), ("status", C.c_void_p),
                    ("variant", C.c_int), ("tile_n", C.c_int), ("has_epilogue", C.c_int)]

    m, k = a.shape
    n = b.shape[1]
    dev = torch.device("cuda:0")
    ta = torch.from_numpy(a).to(dev)
    tb = torch.from_numpy(b).to(dev)
    if half is not None:
        dt = torch.bfloat16 if half == "bf16" else torch.float16
        kp, np_ = (k + 7) // 8 * 8, (n + 7) // 8 * 8
        pa = torch.zeros((m, kp), dtype=dt, device=dev)
        pa[:, :k] = ta.to(dt)
        if b_transposed:
            pb = torch.zeros((n, kp), dtype=dt, device=dev)
            pb[:, :k] = tb.t().to(dt)
            ldb = kp
        else:
            pb = torch.zeros((k, np_), dtype=dt, device=dev)
            pb[:, :n] = tb.to(dt)
            ldb = np_
        ta, tb, lda = pa, pb, kp
    else:
        lda = k
        if b_transposed:
            tb = tb.t().contiguous()
            ldb = k
        else:
            ldb = n
    tc = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
    ws = torch.full((max(1, splits) * m * n,), float("nan"), dtype=torch.float32, device=dev)
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    args = GemmArgs()
    args.arith, args.m, args.n, args.k = arith, m, n, k
    args.a, args.b, args.lda, args.ldb, args.b_transposed = ta.data_ptr(), tb.data_ptr(), lda, ldb, int(b_transposed)
    args.c, args.ldc, args.splits, args.workspace = tc.data_ptr(), n, splits, ws.data_ptr()
    args.status = status.data_ptr()
    args.variant = variant
    args.tile_n = tile_n
    lib.mcd_gemm.restype = C.c_int
    lib.mcd_last_error.restype = C.c_char_p
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.mcd_gemm(C.byref(args), C.c_void_p(stream))
    assert rc == 0, lib.mcd_last_error().decode()
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0, f"kernel gave up a wait: status {int(status[0].item()):#x}"
    return tc.cpu().numpy()


def test_forced_split_counts_fp32(mc, oracle):
    # tests/test_cuda_backend.cpp:241-313: any split count, C pre-filled with NaN
    for m, k, n in [(33, 1000, 65), (128, 2048, 512), (16, 4099, 16), (2, 12, 4), (129, 260, 132), (64, 5, 8)]:
        a = oracle.uniform_values(m * k, 1, -1, 1).reshape(m, k)
        b = oracle.uniform_values(k * n, 2, -1, 1).reshape(k, n)
        exact, abs_dot = exact_and_abs(a, b)
        for splits in [1, 2, 3, 7, 16, 64]:
            got = _device_gemm(mc, 0, a, b, splits)
            check_bound(got, exact, abs_dot, k, 0.0, False, f"fp32 {m}x{k}x{n} splits={splits}")


def test_fp32_tma_fed_kernel_gives_the_bits_of_the_register_staged_one(mc, oracle):
    """The FP32 kernel whose operands arrive through TMA (tensor maps, a 4-stage mbarrier ring; taken whenever A and B
    are 16-byte aligned with row pitches that are multiples of 4 and a block has at least 512 of K; forced here with
    variant bit 1024) accumulates every output over K in the order of the register-staged kernel (variant bit 512):
    identical bits, ragged M, N and K edges and K splits included."""
    for m, k, n in [(128, 128, 128), (1, 4, 4), (33, 260, 68), (127, 132, 132), (129, 16, 260), (513, 76, 260), (300, 1004, 36),
                    (256, 2048, 512), (1024, 1024, 1024)]:
        a = oracle.uniform_values(m * k, 1, -1, 1).reshape(m, k)
        b = oracle.uniform_values(k * n, 2, -1, 1).reshape(k, n)
        for splits in [1, 3, 8]:
            through_tma = _device_gemm(mc, 0, a, b, splits, variant=1024)
            staged = _device_gemm(mc, 0, a, b, splits, variant=512)
            assert np.array_equal(through_tma, staged), f"fp32 {m}x{k}x{n} splits={splits}"
        exact, abs_dot = exact_and_abs(a, b)
        check_bound(through_tma, exact, abs_dot, k, 0.0, False, f"fp32 tma {m}x{k}x{n}")


TC_KINDS = [("tensor_core_bf16", 2, "bf16", 2.0 ** -8, False), ("tensor_core_f16", 3, "f16", 2.0 ** -11, True),
            ("tensor_core_tf32", 1, None, 2.0 ** -11, False)]


@pytest.mark.parametrize("layout", [False, True])
@pytest.mark.parametrize("name,arith,half,u,sub", TC_KINDS)
def test_tensor_core_kernel_direct(mc, oracle, name, arith, half, u, sub, layout):
    """The tcgen05 kernels through the device layer, both layouts of B, with and without a K split."""
    if half is None and not layout:
        pytest.skip("TF32 reads B as a [n,k] copy only")
    for m, k, n in [(128, 64, 256), (128, 256, 256), (256, 512, 512), (300, 1004, 36), (33, 264, 72), (1024, 1024, 1024)]:
        if half is None and (k % 4 or n % 4):
            continue
        a = oracle.uniform_values(m * k, 1, -1, 1).reshape(m, k)
        b = oracle.uniform_values(k * n, 2, -1, 1).reshape(k, n)
        exact, abs_dot = exact_and_abs(a, b)
        for splits in [1, 3]:
            got = _device_gemm(mc, arith, a, b, splits, b_transposed=layout, half=half)
            check_bound(got, exact, abs_dot, k, u, sub, f"{name} {m}x{k}x{n} splits={splits} transposed={layout}")


@pytest.mark.parametrize("layout", [False, True])
@pytest.mark.parametrize("name,arith,half,u,sub", TC_KINDS)
def test_tensor_core_cluster_reduction_direct(mc, oracle, name, arith, half, u, sub, layout):
    """K split 2, 4 or 8 ways with the partial tiles added inside thread-block clusters (through distributed shared
    memory, one launch; variant bit 64) gives the bits of the default workspace-and-second-launch form: both add the
    slices in index order. C is pre-filled with NaN; ragged M, N and K, a single row block, several tiles."""
    if half is None and not layout:
        pytest.skip("TF32 reads B as a [n,k] copy only")
    for m, k, n in [(128, 512, 256), (16, 2048, 512), (300, 1004, 36), (33, 264, 72), (130, 4096, 1000), (256, 8192, 768)]:
        if half is None and (k % 4 or n % 4):
            continue
        a = oracle.uniform_values(m * k, 1, -1, 1).reshape(m, k)
        b = oracle.uniform_values(k * n, 2, -1, 1).reshape(k, n)
        exact, abs_dot = exact_and_abs(a, b)
        for splits in [2, 4, 8]:
            if (k + (31 if half is None else 63)) // (32 if half is None else 64) < splits:
                continue
            in_cluster = _device_gemm(mc, arith, a, b, splits, b_transposed=layout, half=half, variant=64)
            through_workspace = _device_gemm(mc, arith, a, b, splits, b_transposed=layout, half=half)
            assert np.array_equal(in_cluster, through_workspace), f"{name} {m}x{k}x{n} splits={splits} transposed={layout}"
            check_bound(in_cluster, exact, abs_dot, k, u, sub, f"{name} {m}x{k}x{n} splits={splits} transposed={layout}")


@pytest.mark.parametrize("layout", [False, True])
@pytest.mark.parametrize("name,arith,half,u,sub", TC_KINDS)
def test_tensor_core_narrow_tiles_direct(mc, oracle, name, arith, half, u, sub, layout):
    """128 x 128 and 128 x 64 tiles of the one-CTA kernel give the bits of its 128 x 256 tiles."""
    if half is None and not layout:
        pytest.skip("TF32 reads B as a [n,k] copy only")
    for m, k, n in [(128, 64, 64), (256, 512, 512), (300, 1004, 36), (33, 264, 72), (1024, 1024, 1024), (130, 200, 1000)]:
        if half is None and (k % 4 or n % 4):
            continue
        a = oracle.uniform_values(m * k, 1, -1, 1).reshape(m, k)
        b = oracle.uniform_values(k * n, 2, -1, 1).reshape(k, n)
        whole = _device_gemm(mc, arith, a, b, 1, b_transposed=layout, half=half, variant=4)
        for tile_n in (128, 64):
            got = _device_gemm(mc, arith, a, b, 1, b_transposed=layout, half=half, variant=4, tile_n=tile_n)
            assert np.array_equal(got, whole), f"{name} {m}x{k}x{n} transposed={layout} tile_n={tile_n}"
        exact, abs_dot = exact_and_abs(a, b)
        check_bound(whole, exact, abs_dot, k, u, sub, f"{name} {m}x{k}x{n} transposed={layout}")


@pytest.mark.parametrize("layout", [False, True])
@pytest.mark.parametrize("name,arith,half,u,sub", TC_KINDS)
def test_tensor_core_pair_kernel_direct(mc, oracle, name, arith, half, u, sub, layout):
    """The SM-pair (cta_group::2) kernel, forced with variant bit 8 (bit 16: two tiles per work item), against the
    one-CTA kernel (bit 4): they accumulate every output in the same order, so they agree bit for bit; and against
    the float64 bound."""
    if half is None and not layout:
        pytest.skip("TF32 reads B as a [n,k] copy only")
    for m, k, n in [(256, 64, 256), (256, 512, 512), (128, 256, 256), (300, 1004, 36), (33, 264, 72), (1024, 1024, 1024),
                    (1300, 520, 2000), (5000, 256, 4200), (1024, 136, 2048), (4096, 256, 4096)]:
        if half is None and (k % 4 or n % 4):
            continue
        a = oracle.uniform_values(m * k, 1, -1, 1).reshape(m, k)
        b = oracle.uniform_values(k * n, 2, -1, 1).reshape(k, n)
        pair = _device_gemm(mc, arith, a, b, 1, b_transposed=layout, half=half, variant=8)
        wide = _device_gemm(mc, arith, a, b, 1, b_transposed=layout, half=half, variant=8 | 16)
        single = _device_gemm(mc, arith, a, b, 1, b_transposed=layout, half=half, variant=4)
        assert np.array_equal(pair, single), f"{name} {m}x{k}x{n} transposed={layout}: pair and one-CTA kernels differ"
        assert np.array_equal(wide, single), f"{name} {m}x{k}x{n} transposed={layout}: wide pair and one-CTA kernels differ"
        if m * n <= 1 << 21:
            exact, abs_dot = exact_and_abs(a, b)
            check_bound(pair, exact, abs_dot, k, u, sub, f"{name} pair {m}x{k}x{n} transposed={layout}")


@pytest.mark.parametrize("name,arith,half,u,sub", TC_KINDS)
def test_tensor_core_matmuls_within_their_precision_bounds(mc, oracle, name, arith, half, u, sub):
    # tests/test_cuda_backend.cpp:164-219
    for m, k, n in TC_SHAPES:
        text = matmul_text(m, k, n)
        g, ins = oracle_inputs(oracle, text, seed=3)
        exact, abs_dot = exact_and_abs(ins[0], ins[1])
        for layout in ["kn", "transposed"]:
            with mc.CompiledGraph(text=text, options={"matmul": name, "b_layout": layout}) as exe:
                got = exe.run(ins)[0]
                kernels = exe.matmul_kernels
            check_bound(got, exact, abs_dot, k, u, sub, f"{name} {m}x{k}x{n} {layout} ran {kernels}")


@pytest.mark.parametrize("name,u", [("tensor_core_bf16", 2.0 ** -8), ("tensor_core_f16", 2.0 ** -11), ("tensor_core_tf32", 2.0 ** -11)])
def test_pair_kernel_writes_fp32_and_16_bit_copies_of_ragged_results_through_tma(mc, oracle, name, u):
    """A matmul large enough for the SM-pair kernel whose result is both a graph output (FP32) and the left operand of a
    second tensor-core matmul (16-bit copy): both forms leave the kernel as TMA stores of 32 x 32 boxes. Rows and
    columns are no multiples of 32 (nor of the 128 x 256 tile), so boxes are clipped at both edges of both tensors; a
    bias and relu ride in the first matmul's epilogue. Checked against the float64 bound per matmul, the second one
    from the 16-bit rounding of the first one's GPU result."""
    m, k, n, n2 = 2000, 520, 2296, 264
    text = (f"input x : f32[{m}, {k}]\nconst w1 : f32[{k}, {n}] = uniform(seed=5, lo=-0.1, hi=0.1)\n"
            f"const b1 : f32[{n}] = uniform(seed=6, lo=-0.5, hi=0.5)\nconst w2 : f32[{n}, {n2}] = uniform(seed=7, lo=-0.1, hi=0.1)\n"
            "h0 = matmul x, w1\nh1 = add h0, b1\nh = relu h1\ny = matmul h, w2\noutput h\noutput y")
    g, ins = oracle_inputs(oracle, text, seed=9)
    consts = {node.name: np.asarray(node.value, dtype=np.float32).reshape(node.shape) for node in g.nodes if node.value is not None}
    x = ins[0]
    with mc.CompiledGraph(text=text, options={"matmul": name}) as exe:
        plan = exe.matmul_kernels
        h, y = exe.run(ins)
        again = exe.run(ins)
    assert np.array_equal(h, again[0]) and np.array_equal(y, again[1])
    h, y = h.reshape(m, n), y.reshape(m, n2)
    exact, abs_dot = exact_and_abs(x, consts["w1"])
    pre = exact + consts["b1"].astype(np.float64)
    want_h = np.maximum(pre, 0.0)
    gamma = k * U32 / (1.0 - k * U32)
    bound = (2.0 * u + u * u + 2.0 * gamma) * abs_dot + 4.0 * U32 * (np.abs(exact) + np.abs(consts["b1"])) + 2.0 * k * 2.0 ** -25
    err = np.abs(h.astype(np.float64) - want_h)
    assert (err <= bound).all(), f"{name} first matmul ({plan}): {int((err > bound).sum())} outside the bound, worst {err.max():.3e}"
    exact2, abs2 = exact_and_abs(h, consts["w2"])  # from the GPU's own h: isolates the second matmul and its 16-bit operand
    check_bound(y, exact2, abs2, n, u, True, f"{name} second matmul ({plan})")


# -------------------------------------------------- the benchmark configs, small


def norm_scaled_error(got, want):
    want = want.astype(np.float64)
    return float(np.max(np.abs(got.astype(np.float64) - want)) / max(1e-30, np.sqrt(np.mean(want ** 2))))


def test_config_graphs_small(mc, oracle):
    cases = [("c1_mlp_block", "B=64", "uniform"), ("c3_ffn", "T=256,D=128,H=512", "normal"),
             ("c5_mlp_stack", "B=256,D=256", "normal")]
    for name, dims, dist in cases:
        path = mc.graph_path(name)
        d = {k: int(v) for k, v in (kv.split("=") for kv in dims.split(","))}
        g = oracle.parse_mcg_file(path, d)
        shape = g.node(g.inputs[0]).shape
        n = int(np.prod(shape))
        x = oracle.uniform_values(n, 1, -1, 1) if dist == "uniform" else oracle.normal_values(n, 1)
        ins = [x.reshape(shape)]
        want = oracle.evaluate_f64(g, ins)[0]
        scale = float(np.max(np.abs(want)))
        for matmul, tol in [("auto", 1e-4), ("tensor_core_tf32", 5e-3), ("tensor_core_bf16", 2e-2), ("tensor_core_f16", 2e-2)]:
            for fuse in (1, 0):
                got = run_graph(mc, path=path, dims=dims, options={"matmul": matmul, "fuse_epilogue": fuse}, inputs=ins)[0]
                if matmul == "auto":
                    ok, msg = all_close(got, want, tol, tol * scale)
                    assert ok, f"{name} {matmul} fuse={fuse}: {msg}"
                else:
                    err = norm_scaled_error(got, want)  # end to end, at the bar itself, whatever the depth
                    assert err <= tol, f"{name} {matmul} fuse={fuse}: norm-scaled error {err:.3e}"


def test_c2_gelu_full_size_properties(mc, oracle):
    """At the full 8192 x 8192 size: gelu(x) - gelu(-x) == x (odd-part identity), and sampled rows equal the oracle."""
    path = mc.graph_path("c2_gelu_chain")
    n = 8192 * 8192
    x = oracle.normal_values(n, 7)
    with mc.CompiledGraph(path) as exe:
        y_pos = exe.run([x])[0]
        y_neg = exe.run([-x])[0]
    resid = np.abs((y_pos.astype(np.float64) - y_neg.astype(np.float64)) - x)
    assert float(resid.max()) <= 1e-5 * max(1.0, float(np.abs(x).max()))
    rows = [0, 1, 4095, 8191]
    g = oracle.parse_mcg_file(path, {"M": len(rows), "N": 8192})
    sample = np.stack([x.reshape(8192, 8192)[r] for r in rows])
    want = oracle.evaluate_f64(g, [sample])[0]
    got = np.stack([y_pos.reshape(8192, 8192)[r] for r in rows]).reshape(-1)
    ok, msg = all_close(got, want, 1e-5, 1e-7)
    assert ok, msg


def test_large_matmul_sampled_and_checksum(mc, oracle):
    """4096^3 in every arithmetic: 1000 sampled dot products in float64 (bench/bench_cuda.cpp:386-436) and the
    row-sum identity C 1 = A (B 1)."""
    m = k = n = 4096
    a = oracle.uniform_values(m * k, 1, -1, 1).reshape(m, k)
    b = oracle.uniform_values(k * n, 2, -1, 1).reshape(k, n)
    rng = np.random.default_rng(0)
    rows, cols = rng.integers(0, m, 1000), rng.integers(0, n, 1000)
    exact, abs_dot = oracle.sampled_matmul_f64(a, b, rows, cols)
    rowsum = a.astype(np.float64) @ b.astype(np.float64).sum(axis=1)
    text = matmul_text(m, k, n)
    for name, u, sub in [("auto", 0.0, False), ("tensor_core_tf32", 2.0 ** -11, False), ("tensor_core_bf16", 2.0 ** -8, False),
                         ("tensor_core_f16", 2.0 ** -11, True)]:
        got = run_graph(mc, text=text, options={"matmul": name}, inputs=[a, b])[0].reshape(m, n)
        check_bound(got[rows, cols], exact, abs_dot, k, u, sub, f"{name} 4096^3 sampled")
        scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64).sum(axis=1)
        rel = np.max(np.abs(got.astype(np.float64).sum(axis=1) - rowsum) / scale)
        assert rel <= (2 * u + 4096 * U32 * 2), f"{name}: row-sum identity off by {rel:.3e}"


def test_run_on_pinned_host_memory_equals_run_with_copies(mc, oracle):
    """mc_run on pinned buffers lets a streaming graph read and write caller memory in place (no staging
    copies); the results must be the ones the copying path gives, bit for bit."""
    torch = _torch()
    path = mc.graph_path("c2_gelu_chain")
    dims = {"M": 1000, "N": 1028}
    x = oracle.normal_values(1000 * 1028, 3)
    with mc.CompiledGraph(path, dims=dims, options={"host_io": 0}) as exe:
        want = exe.run([x])[0]
    pin_in = torch.from_numpy(x.copy()).pin_memory()
    pin_out = torch.full((x.size,), float("nan"), dtype=torch.float32).pin_memory()
    with mc.CompiledGraph(path, dims=dims) as exe:
        exe.run_ptrs([pin_in.data_ptr()], [pin_out.data_ptr()])
        assert np.array_equal(pin_out.numpy(), want)
        assert np.array_equal(exe.run([x])[0], want)  # pageable memory: falls back to copies
    # two chained kernels (no fusion): the intermediate stays on the device, the ends stream from/to the host
    text = "input a : f32[512, 64]\ninput b : f32[512, 64]\ninput c : f32[512, 64]\nt = mul a, b\nu = exp t\ny = add u, c\noutput y"
    g, ins = oracle_inputs(oracle, text, seed=4)
    with mc.CompiledGraph(text=text, passes="none", options={"host_io": 0}) as exe:
        want = exe.run(ins)[0]
    pins = [torch.from_numpy(a.reshape(-1).copy()).pin_memory() for a in ins]
    out = torch.empty(512 * 64, dtype=torch.float32).pin_memory()
    with mc.CompiledGraph(text=text, passes="none") as exe:
        exe.run_ptrs([p.data_ptr() for p in pins], [out.data_ptr()])
    assert np.array_equal(out.numpy(), want)


# ------------------------------------------------ row reductions (extension)


@pytest.mark.parametrize("shape", ["[5, 1]", "[7, 33]", "[64, 1000]", "[3, 1024]", "[2, 5, 5000]", "[300, 7]", "[4097]"])
def test_row_reductions_match_the_oracle(mc, oracle, shape):
    """row_max is exact; row_sum (FP32 partial sums in a fixed order) stays within n * 2^-24 * sum|x| of the
    double-precision sum that defines the op, and two runs give the same bits."""
    text = f"input x : f32{shape}\ns = row_sum x\nm = row_max x\noutput s, m"
    g, ins = oracle_inputs(oracle, text, seed=5, lo=-3.0, hi=3.0)
    width = int(shape.strip("[]").split(",")[-1])
    want_s, want_m = oracle.evaluate_f64(g, ins)
    with mc.CompiledGraph(text=text, passes="none") as exe:
        got_s, got_m = exe.run(ins)
        again_s, _ = exe.run(ins)
    assert np.array_equal(got_m, want_m)
    assert np.array_equal(got_s, again_s)
    abs_sum = np.abs(ins[0].astype(np.float64)).reshape(-1, width).sum(axis=1)
    err = np.abs(got_s.astype(np.float64) - want_s.astype(np.float64))
    assert np.all(err <= width * U32 * abs_sum + U32 * np.abs(want_s)), f"{shape}: worst {float(np.max(err / abs_sum)):.2e} of sum|x|"


def test_row_reduction_with_an_absorbed_broadcasting_producer(mc, oracle):
    text = ("input x : f32[6, 3, 700]\ninput b : f32[3, 1]\ninput r : f32[700]\nt = mul x, b\nu = add t, r\nv = exp u\n"
            "s = row_sum v\nm = row_max v\noutput s, m")
    g, ins = oracle_inputs(oracle, text, seed=9, lo=-1.0, hi=1.0)
    want_s, want_m = oracle.evaluate_f64(g, ins)
    # The [3,1] operand keeps exp(...) out of a row kernel. Its two readers are one row kernel by default; as separate
    # reductions each recomputes it, unless that is turned off too and it is written once and read twice.
    for options, launches in [({}, 2), ({"fuse_rows": 0}, 2), ({"fuse_rows": 0, "rematerialize": 0}, 3)]:
        with mc.CompiledGraph(text=text, options=options) as exe:
            got_s, got_m = exe.run(ins)
            assert exe.kernel_launches == launches
        ok, msg = all_close(got_m, want_m, 1e-6, 1.2e-7)
        assert ok, msg
        ok, msg = all_close(got_s, want_s, 1e-5, 0.0)
        assert ok, msg
    single = "input x : f32[6, 3, 700]\ninput b : f32[3, 1]\nt = mul x, b\nq = mul t, t\ns = row_sum q\noutput s"
    g, ins = oracle_inputs(oracle, single, seed=9, lo=-1.0, hi=1.0)
    with mc.CompiledGraph(text=single) as exe:
        got = exe.run(ins)[0]
        assert exe.kernel_launches == 1  # the whole producer chain is evaluated inside the reduction
    ok, msg = all_close(got, oracle.evaluate_f64(g, ins)[0], 1e-5, 0.0)
    assert ok, msg


def test_softmax_and_layernorm_graphs(mc, oracle):
    for name, dims in [("x1_softmax", "M=128,N=1000"), ("x1_softmax", "M=64,N=4096"), ("x2_layernorm", "M=96,N=4096"),
                       ("x1_softmax", "M=300,N=5000"), ("x1_softmax", "M=7,N=8192"), ("x1_softmax", "M=33,N=16384"),
                       ("x1_softmax", "M=1000,N=33"), ("x1_softmax", "M=5,N=1023"), ("x1_softmax", "M=9,N=20000"),
                       ("x1_softmax", "M=6,N=32768"), ("x2_layernorm", "M=4,N=32768"), ("x1_softmax", "M=3,N=40000"),
                       ("x1_softmax", "M=300,N=16384"), ("x2_layernorm", "M=5,N=65536"), ("x1_softmax", "M=3,N=70000")]:
        path = mc.graph_path(name)
        g, _ = oracle_inputs(oracle, path=path, dims=dims)
        x = oracle.normal_values(int(np.prod(g.node(g.inputs[0]).shape)), 7)
        want = oracle.evaluate_f64(g, [x])[0]
        with mc.CompiledGraph(path, dims=dims) as exe:
            got = exe.run([x])[0]
            fused_launches = exe.kernel_launches
        width = int(dims.split("N=")[1])
        assert fused_launches == (1 if width <= 65536 else 3)  # whole rows in one kernel while they fit in registers  # whole rows in one kernel when they fit in registers
        for options in ({"fuse_rows": 0}, {"fuse_rows": 0, "rematerialize": 0}):
            with mc.CompiledGraph(path, dims=dims, options=options) as exe:
                separate = exe.run([x])[0]
            # the row kernel and the recomputing form perform the same operations per element in the same order
            assert np.array_equal(got, separate), f"{name} {dims} {options}"
        assert norm_scaled_error(got, want) <= 1e-5, f"{name} {dims}: {norm_scaled_error(got, want):.2e}"
        if name == "x1_softmax":
            assert np.allclose(got.reshape(-1, width).sum(axis=1), 1.0, atol=1e-5)


def test_row_kernel_with_several_outputs_and_operand_kinds(mc, oracle):
    """One row-fused kernel reading a full tensor, a per-row column, a row vector and a scalar, and writing a
    full-shaped and two per-row values; against the oracle and, bit for bit, against the separate kernels."""
    text = ("input x : f32[5, 6, 1500]\ninput col : f32[5, 6, 1]\ninput vec : f32[1500]\nconst k : f32[] = 0.5\n"
            "a = mul x, vec\nb = add a, col\nm = row_max b\nd = sub b, m\ne = exp d\ns = row_sum e\nh = mul s, k\n"
            "y = div e, h\noutput y, m, h")
    g, ins = oracle_inputs(oracle, text, seed=4, lo=-1.0, hi=1.0)
    want = oracle.evaluate_f64(g, ins)
    with mc.CompiledGraph(text=text) as exe:
        got = exe.run(ins)
        assert exe.kernel_launches == 1
    with mc.CompiledGraph(text=text, options={"fuse_rows": 0}) as exe:
        separate = exe.run(ins)
        assert exe.kernel_launches > 1
    for g_, s_, w_ in zip(got, separate, want):
        assert np.array_equal(g_, s_)
        ok, msg = all_close(g_, w_, 2e-5, 1e-7)
        assert ok, msg


def _random_row_graph(rng, rows_shape):
    """A random graph of elementwise steps on `rows_shape`, row reductions and per-row steps, with full-shaped,
    per-row, row-vector and scalar operands; every value stays bounded so that tolerances mean something."""
    dims = ", ".join(str(d) for d in rows_shape)
    reduced = ", ".join(str(d) for d in rows_shape[:-1] + (1,))
    lines = [f"input x : f32[{dims}]", f"input col : f32[{reduced}]", f"input vec : f32[{rows_shape[-1]}]", "const k : f32[] = 0.75"]
    full, per_row = ["x"], ["col"]
    count = 0

    def fresh():
        nonlocal count
        count += 1
        return f"t{count}"

    for _ in range(int(rng.integers(4, 10))):
        kind = rng.choice(["unary", "binary", "reduce", "per_row"], p=[0.25, 0.35, 0.25, 0.15])
        name = fresh()
        if kind == "unary":
            lines.append(f"{name} = {rng.choice(['tanh', 'sigmoid', 'relu', 'neg'])} {rng.choice(full)}")
            full.append(name)
        elif kind == "binary":
            other = rng.choice(full + per_row + ["vec", "k"])
            a, b = (rng.choice(full), other) if rng.random() < 0.5 else (other, rng.choice(full))
            lines.append(f"{name} = {rng.choice(['add', 'sub', 'mul'])} {a}, {b}")
            full.append(name)
        elif kind == "reduce":
            lines.append(f"{name} = {rng.choice(['row_sum', 'row_max'])} {rng.choice(full)}")
            if lines[-1].split()[2] == "row_sum":  # keep magnitudes bounded: scale the sum by 1 / width
                scaled = fresh()
                lines.append(f"const inv{scaled} : f32[] = {1.0 / rows_shape[-1]!r}")
                lines.append(f"{scaled} = mul {name}, inv{scaled}")
                name = scaled
            per_row.append(name)
        else:
            lines.append(f"{name} = {rng.choice(['add', 'mul', 'sub'])} {rng.choice(per_row)}, {rng.choice(per_row + ['k'])}")
            per_row.append(name)
    outputs = [full[-1]] + ([per_row[-1]] if len(per_row) > 1 else [])
    if len(full) > 3 and rng.random() < 0.5:
        outputs.append(full[len(full) // 2])
    lines.append("output " + ", ".join(dict.fromkeys(outputs)))
    return "\n".join(lines)


def test_random_row_graphs_fused_and_separate_agree(mc, oracle):
    """40 random row graphs: the default lowering (row kernels, recomputation) gives the bits of the plain per-step
    lowering, and both are within the elementwise tolerance of the double-precision oracle."""
    rng = np.random.default_rng(2024)
    fused_seen = 0
    for case in range(40):
        shape = [(7, 1536), (3, 5, 1100), (64, 96), (5, 9000), (2, 3, 33), (16, 1024)][case % 6]
        text = _random_row_graph(rng, shape)
        g, ins = oracle_inputs(oracle, text, seed=case + 1, lo=-1.0, hi=1.0)
        want = oracle.evaluate_f64(g, ins)
        with mc.CompiledGraph(text=text) as exe:
            got = exe.run(ins)
            fused_seen += "mc_row_fused" in exe.kernel_sources
        with mc.CompiledGraph(text=text, options={"fuse_rows": 0, "rematerialize": 0}) as exe:
            plain = exe.run(ins)
        for a, b, w in zip(got, plain, want):
            assert np.array_equal(a, b), f"case {case}:\n{text}"
            ok, msg = all_close(a, w, 2e-5, 2e-6)
            assert ok, f"case {case}: {msg}\n{text}"
    assert fused_seen >= 20


@pytest.mark.parametrize("matmul,tol", [("auto", 1e-4), ("tensor_core_bf16", 2e-2), ("tensor_core_tf32", 5e-3)])
def test_attention_like_graph_mixes_matmuls_and_a_row_kernel(mc, oracle, matmul, tol):
    """scores = q k^T (given as k_t), softmax over rows in one row kernel, out = p v: the row kernel reads a matmul
    result and feeds the next matmul, which for the 16-bit kernel needs its operand recast after the row kernel."""
    text = ("input q : f32[192, 64]\ninput kt : f32[64, 1280]\ninput v : f32[1280, 96]\nconst scale : f32[] = 0.125\n"
            "s = matmul q, kt\nt = mul s, scale\nm = row_max t\nd = sub t, m\ne = exp d\nz = row_sum e\np = div e, z\n"
            "o = matmul p, v\noutput o, z")
    g, ins = oracle_inputs(oracle, text, seed=21, lo=-1.0, hi=1.0)
    want = oracle.evaluate_f64(g, ins)
    with mc.CompiledGraph(text=text, options={"matmul": matmul}) as exe:
        got = exe.run(ins)
        assert "mc_row_fused" in exe.kernel_sources
    with mc.CompiledGraph(text=text, options={"matmul": matmul, "fuse_rows": 0, "rematerialize": 0}) as exe:
        plain = exe.run(ins)
    for a, b, w in zip(got, plain, want):
        assert np.array_equal(a, b)
        assert norm_scaled_error(a, w) <= tol, f"{matmul}: {norm_scaled_error(a, w):.2e}"
