"""The benchmark configurations at their stated sizes, the sharded path on the device, and the status-word
error path - all through the C ABI on a B200.

Bars (per element, against a float64 evaluation, error divided by the root-mean-square of the expected
tensor): 1e-5 elementwise FP32 graphs, 1e-4 FP32 GEMM graphs, 5e-3 TF32, 2e-2 BF16/FP16 - with no allowance
for depth: a multi-layer graph is held to the same bar end to end, and every layer is also checked on its own
from the GPU's own input of that layer.

Large shapes are checked the way the reference checks its large matmuls (bench/bench_cuda.cpp:386-436):
sampled outputs recomputed in float64, the output buffer pre-filled with NaN. Graphs whose rows are
independent are checked on sampled rows: the oracle evaluates the same graph on just those rows.
Inputs at these sizes come from numpy's PCG64 generator (the same buffer goes to the GPU and to the checker).
"""

import ctypes as C
import re

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

U32 = 2.0 ** -24
TOL = {"auto": 1e-4, "tensor_core_tf32": 5e-3, "tensor_core_bf16": 2e-2, "tensor_core_f16": 2e-2}
UNIT = {"auto": 0.0, "tensor_core_tf32": 2.0 ** -11, "tensor_core_bf16": 2.0 ** -8, "tensor_core_f16": 2.0 ** -11}


def nse(got, want):
    """Largest element error over the root-mean-square of the expected values."""
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    return float(np.max(np.abs(got - want)) / max(1e-30, np.sqrt(np.mean(want ** 2))))


def fast_normal(n, seed):
    return np.random.default_rng(seed).standard_normal(n, dtype=np.float32)


def fast_uniform(n, seed):
    v = np.random.default_rng(seed).random(n, dtype=np.float32)
    v *= 2.0
    v -= 1.0
    return v


def graph_text(mc, name):
    with open(mc.graph_path(name)) as f:
        return f.read()


def with_outputs(text, names):
    """The same graph with another output list."""
    lines = [ln for ln in text.splitlines() if not ln.strip().startswith("output ")]
    return "\n".join(lines) + "\noutput " + ", ".join(names) + "\n"


def dot_bound(exact, abs_dot, k, u_in, subnormals=False):
    gamma = k * U32 / (1.0 - k * U32)
    if u_in == 0.0:
        return 2.0 * gamma * abs_dot + 2.0 * U32 * np.abs(exact)
    tiny = 2.0 * k * 2.0 ** -25 if subnormals else 0.0
    return (2.0 * u_in + u_in * u_in + 2.0 * gamma) * abs_dot + 2.0 * U32 * np.abs(exact) + tiny


# ------------------------------------------------------- per-layer and end-to-end


def c5_layer_text(text, layer):
    """Layer `layer` of the MLP stack as a graph of its own: the same constants, its input fed as x."""
    keep = []
    for ln in text.splitlines():
        s = ln.strip()
        if s.startswith(("graph ", "dim ", "input ", "const eps")):
            keep.append(ln)
            continue
        m = re.match(r"(?:const\s+)?([a-z]+)(\d+)\b", s)
        if m and int(m.group(2)) == layer and not s.startswith("output"):
            keep.append(re.sub(rf"matmul a{layer - 1}\b", "matmul x", ln))
    return "\n".join(keep) + f"\noutput a{layer}\n"


@pytest.mark.parametrize("matmul", ["auto", "tensor_core_tf32", "tensor_core_bf16", "tensor_core_f16"])
def test_c5_every_layer_and_end_to_end_at_the_stated_bar(mc, oracle, matmul):
    """The 8-layer stack with every activation as an output: each layer against float64 from the GPU's own
    input of that layer, and the last against float64 of the whole graph - both at the bar itself."""
    dims = {"B": 384, "D": 256}
    text = graph_text(mc, "c5_mlp_stack")
    all_text = with_outputs(text, [f"a{i}" for i in range(8)])
    x = oracle.normal_values(dims["B"] * dims["D"], 1).reshape(dims["B"], dims["D"])
    with mc.CompiledGraph(text=all_text, dims=dims, options={"matmul": matmul}) as exe:
        acts = [a.reshape(dims["B"], dims["D"]) for a in exe.run([x])]
    with mc.CompiledGraph(text=text, dims=dims, options={"matmul": matmul}) as exe:
        last_only = exe.run([x])[0].reshape(dims["B"], dims["D"])
    # activations kept in FP32 for output do not change what the next layer reads
    assert np.array_equal(last_only, acts[7])
    worst = 0.0
    for layer in range(8):
        g = oracle.parse_mcg(c5_layer_text(text, layer), dims)
        fed = x if layer == 0 else acts[layer - 1]
        want = oracle.evaluate_f64(g, [fed])[0]
        err = nse(acts[layer], want)
        worst = max(worst, err)
        assert err <= TOL[matmul], f"{matmul} layer {layer}: {err:.3e} > {TOL[matmul]:.0e}"
    g = oracle.parse_mcg(text, dims)
    e2e = nse(acts[7], oracle.evaluate_f64(g, [x])[0])
    print(f"\nC5 {matmul} B=384 D=256: worst single layer {worst:.3e}, end to end over 8 layers {e2e:.3e} (bar {TOL[matmul]:.0e})")
    assert e2e <= TOL[matmul], f"{matmul}: end-to-end error {e2e:.3e} > {TOL[matmul]:.0e}"


@pytest.mark.parametrize("matmul", ["auto", "tensor_core_tf32", "tensor_core_bf16", "tensor_core_f16"])
def test_c3_both_layers_and_end_to_end_at_the_stated_bar(mc, oracle, matmul):
    dims = {"T": 256, "D": 128, "H": 512}
    text = graph_text(mc, "c3_ffn")
    x = oracle.normal_values(dims["T"] * dims["D"], 1).reshape(dims["T"], dims["D"])
    with mc.CompiledGraph(text=with_outputs(text, ["h", "y"]), dims=dims, options={"matmul": matmul}) as exe:
        h, y = exe.run([x])
    g_h = oracle.parse_mcg(with_outputs(text, ["h"]), dims)
    err_h = nse(h, oracle.evaluate_f64(g_h, [x])[0])
    # second layer from the GPU's own h: y = h w2 + b2 + x
    second = ("dim T = 256\ndim D = 128\ndim H = 512\ninput h : f32[T, H]\ninput x : f32[T, D]\n"
              "const w2 : f32[H, D] = uniform(seed=23, lo=-0.015625, hi=0.015625)\n"
              "const b2 : f32[D] = uniform(seed=24, lo=-0.01, hi=0.01)\no = matmul h, w2\nob = add o, b2\ny = add ob, x\noutput y\n")
    g_y = oracle.parse_mcg(second, dims)
    err_y = nse(y, oracle.evaluate_f64(g_y, [h.reshape(dims["T"], dims["H"]), x])[0])
    g = oracle.parse_mcg(text, dims)
    e2e = nse(y, oracle.evaluate_f64(g, [x])[0])
    print(f"\nC3 {matmul}: layer 1 {err_h:.3e}, layer 2 {err_y:.3e}, end to end {e2e:.3e} (bar {TOL[matmul]:.0e})")
    assert max(err_h, err_y, e2e) <= TOL[matmul]


# ----------------------------------------------------------- the configs at full size


def run_into_nan(exe, inputs):
    outs = [np.full(n, np.nan, dtype=np.float32) for n in exe.output_elements]
    exe.run(inputs, outs)
    return outs


def sampled_rows_check(mc, oracle, name, dims, lead, matmul, rows, tol, x, label):
    """Runs the full-size graph; the oracle evaluates the same graph on `rows` only."""
    path = mc.graph_path(name)
    with mc.CompiledGraph(path, dims=dims, options={"matmul": matmul}) as exe:
        got = run_into_nan(exe, [x])[0]
        kernels = exe.matmul_kernels
    width = got.size // dims[lead]
    got = got.reshape(dims[lead], width)
    assert not np.isnan(got).any(), f"{label}: output elements were never written"
    g = oracle.parse_mcg_file(path, dims | {lead: len(rows)})
    want = oracle.evaluate_f64(g, [x.reshape(dims[lead], -1)[rows]])[0].reshape(len(rows), width)
    err = nse(got[rows], want)
    print(f"\n{label} ({','.join(sorted(set(kernels)))}): {len(rows) * width} sampled outputs, norm-scaled error {err:.3e} (bar {tol:.0e})")
    assert err <= tol, f"{label}: {err:.3e} > {tol:.0e}"
    return got


def test_c1_at_b256(mc, oracle):
    x = oracle.uniform_values(256 * 512, 1, -1, 1)
    rows = np.arange(256)
    sampled_rows_check(mc, oracle, "c1_mlp_block", {"B": 256}, "B", "auto", rows, 1e-4, x, "C1 B=256 FP32")


@pytest.mark.parametrize("matmul", ["auto", "tensor_core_tf32"])
def test_c3_at_full_size(mc, oracle, matmul):
    dims = {"T": 8192, "D": 1024, "H": 4096}
    x = fast_normal(8192 * 1024, 3)
    rows = np.array([0, 1, 127, 128, 255, 256, 4095, 4096, 5000, 8063, 8064, 8191])
    sampled_rows_check(mc, oracle, "c3_ffn", dims, "T", matmul, rows, TOL[matmul], x, f"C3 full size {matmul}")


@pytest.mark.parametrize("matmul,batch", [("tensor_core_bf16", 8192), ("tensor_core_f16", 8192), ("tensor_core_f16", 65536)])
def test_c5_at_d2048(mc, oracle, matmul, batch):
    dims = {"B": batch, "D": 2048}
    x = fast_normal(batch * 2048, 5)
    rows = np.unique(np.concatenate([np.array([0, 1, 127, 128, 255, 256, batch // 2 - 1, batch // 2, batch - 129, batch - 1]),
                                     np.random.default_rng(1).integers(0, batch, 6)]))
    sampled_rows_check(mc, oracle, "c5_mlp_stack", dims, "B", matmul, rows, TOL[matmul], x, f"C5 B={batch} D=2048 {matmul}")


C4_SHAPES = [(8192, 8192, 8192), (16384, 16384, 16384), (16, 8192, 8192), (128, 8192, 8192), (1024, 1024, 65536)]


@pytest.mark.parametrize("m,n,k", C4_SHAPES)
def test_c4_sweep_shapes_sampled_in_float64(mc, oracle, m, n, k):
    """The large, skinny and tall-K shapes of the tensor-core sweep in BF16 and FP16: 1000 sampled outputs against
    float64 dot products within the rounding bound of the format, a NaN-filled C fully overwritten, and the
    norm-scaled error at the 2e-2 bar."""
    a = fast_uniform(m * k, 11).reshape(m, k)
    b = fast_uniform(k * n, 12).reshape(k, n)
    rng = np.random.default_rng(0)
    rows, cols = rng.integers(0, m, 1000), rng.integers(0, n, 1000)
    # corners and tile seams
    rows[:8] = [0, m - 1, 0, m - 1, min(m - 1, 127), min(m - 1, 128), m // 2, m - 1]
    cols[:8] = [0, 0, n - 1, n - 1, 255, 256, n // 2, n - 129]
    exact, abs_dot = oracle.sampled_matmul_f64(a, b, rows, cols)
    rms = float(np.sqrt(k / 9.0))  # uniform(-1,1) operands: each product has variance 1/9
    text = f"input a : f32[{m}, {k}]\ninput w : f32[{k}, {n}]\nc = matmul a, w\noutput c"
    for name, sub in [("tensor_core_bf16", False), ("tensor_core_f16", True)]:
        with mc.CompiledGraph(text=text, options={"matmul": name}) as exe:
            got = run_into_nan(exe, [a, b])[0].reshape(m, n)
            kernels, launches = exe.matmul_kernels, exe.kernel_launches
        assert not np.isnan(got).any(), f"{name} {m}x{n}x{k}: output elements were never written"
        err = np.abs(got[rows, cols].astype(np.float64) - exact)
        bad = ~(err <= dot_bound(exact, abs_dot, k, UNIT[name], sub))
        assert not bad.any(), f"{name} {m}x{n}x{k}: {int(bad.sum())} of 1000 samples outside the rounding bound"
        scaled = float(err.max()) / rms
        print(f"\nC4 {name} {m}x{n}x{k} ({','.join(kernels)}, {launches} launch(es)): sampled norm-scaled error {scaled:.3e}")
        assert scaled <= 2e-2
        del got


# ----------------------------------------------------- sharded == unsharded, on the device


@pytest.mark.parametrize("name,dims,lead,matmul", [
    ("c5_mlp_stack", {"B": 4096, "D": 512}, "B", "tensor_core_f16"),
    ("c5_mlp_stack", {"B": 1024, "D": 256}, "B", "auto"),
    ("c3_ffn", {"T": 2048, "D": 256, "H": 1024}, "T", "tensor_core_tf32"),
    ("c3_ffn", {"T": 512, "D": 128, "H": 512}, "T", "auto"),
    ("c1_mlp_block", {"B": 256}, "B", "auto"),
])
def test_two_shards_on_the_device_reproduce_the_unsharded_rows(mc, oracle, name, dims, lead, matmul):
    """What rank 0 and rank 1 of a 2-GPU run would compute (the graph compiled at B/2 through mc_shard_dims, each on
    its row slice), run here on one GPU, against the graph compiled at B. Tile shape, split rule and the choice between
    the one-CTA and the SM-pair kernel all change with the row count; every output element is still the same dot
    product, accumulated over K in the same order unless K is split differently - so the halves must equal the whole
    bit for bit when both plans split K the same way, and stay within the config's bar otherwise."""
    path = mc.graph_path(name)
    g = oracle.parse_mcg_file(path, dims)
    shape = g.node(g.inputs[0]).shape
    x = oracle.normal_values(int(np.prod(shape)), 9).reshape(shape)
    def k_splits(d):
        plan = mc.HostGraph(path, dims=d).launch_plan({"matmul": matmul})
        return re.findall(r"splits=(\d+)", plan)

    with mc.CompiledGraph(path, dims=dims, options={"matmul": matmul}) as exe:
        whole = exe.run([x])[0].reshape(shape[0], -1)
    parts, same_splits = [], True
    for rank in range(2):
        shard, first, rows = mc.shard_dims(path, dims, lead, rank, 2)
        assert (first, rows) == (rank * shape[0] // 2, shape[0] // 2)
        same_splits = same_splits and k_splits(shard) == k_splits(dims)
        with mc.CompiledGraph(path, dims=shard, options={"matmul": matmul}) as exe:
            parts.append(exe.run([x[first:first + rows]])[0].reshape(rows, -1))
    halves = np.concatenate(parts)
    if same_splits:
        assert np.array_equal(halves, whole), f"{name} {matmul}: shards differ from the unsharded run"
    else:  # a different K split adds the same FP32 products in another order
        err = nse(halves, whole)
        print(f"\n{name} {matmul}: the shards split K differently; they differ from the unsharded run by {err:.3e}")
        assert err <= TOL[matmul] * 0.1, f"{name} {matmul}: shards differ from the unsharded run by {err:.3e}"


# --------------------------------------------------------------- the status-word path


def test_a_set_status_word_fails_synchronize_and_download_then_clears(mc, oracle):
    """A tensor-core kernel that gives up a bounded wait ORs a code into the executable's status word. No kernel
    is made to wait here: the word is written from the host, and mc_synchronize / mc_download must report it, name
    the code, and clear it so that the next run is clean."""
    text = "input a : f32[128, 64]\ninput w : f32[64, 256]\nc = matmul a, w\noutput c"
    g = oracle.parse_mcg(text)
    ins = oracle.make_random_inputs(g, 1)
    lib = mc.lib()
    with mc.CompiledGraph(text=text, options={"matmul": "tensor_core_bf16"}) as exe:
        want = exe.run(ins)[0]
        word = exe.status_word_ptr()
        assert word != 0
        for call in ("synchronize", "download"):
            code = C.c_uint(0x21)
            assert lib.mcd_copy_h2d(C.c_void_p(word), C.byref(code), 4, None) == 0
            assert lib.mcd_device_synchronize() == 0
            with pytest.raises(mc.McError, match=r"gave up a bounded wait \(status 0x21\)"):
                getattr(exe, call)()
            back = C.c_uint(0xFFFFFFFF)
            assert lib.mcd_copy_d2h(C.byref(back), C.c_void_p(word), 4, None) == 0
            assert lib.mcd_device_synchronize() == 0
            assert back.value == 0, "the status word is cleared once it has been reported"
            exe.synchronize()  # clean again
        assert np.array_equal(exe.run(ins)[0], want)
    with mc.CompiledGraph(text="input x : f32[8]\ny = exp x\noutput y") as exe:
        assert exe.status_word_ptr() == 0  # nothing in this graph can wait


def test_kernel_cache_gives_modules_back(mc):
    """Compiling and releasing executables must not grow the set of held kernels: references are returned on
    release, and idle modules are bounded."""
    lib = mc.lib()
    held = lambda: (lambda m, i: (lib.mcd_jit_cache_stats(C.byref(m), C.byref(i)), m.value - i.value)[1])(C.c_longlong(), C.c_longlong())
    before = held()
    for n in (1000, 1001, 1002):
        with mc.CompiledGraph(text=f"input x : f32[{n}]\ny = exp x\nz = tanh y\noutput z", passes="none") as exe:
            assert held() >= before + 2
            exe.run([np.zeros(n, dtype=np.float32)])
    assert held() == before


# ------------------------------------------------ row reductions against torch in float64


def test_softmax_and_layernorm_against_torch_float64(mc, oracle):
    """The row-reduction extension has no reference behaviour to pin against, so its values are compared with an
    implementation this project did not write: torch.softmax and torch.nn.functional.layer_norm evaluated in float64
    on the CPU, at 1e-5 norm-scaled."""
    import torch

    for name, dims in [("x1_softmax", {"M": 64, "N": 1000}), ("x1_softmax", {"M": 16, "N": 8192}), ("x1_softmax", {"M": 9, "N": 20000}),
                       ("x1_softmax", {"M": 3, "N": 40000}), ("x2_layernorm", {"M": 32, "N": 4096}), ("x2_layernorm", {"M": 7, "N": 1023}),
                       ("x2_layernorm", {"M": 5, "N": 33000}), ("x1_softmax", {"M": 200, "N": 16384}), ("x2_layernorm", {"M": 3, "N": 70000})]:
        # the shipped LayerNorm graph spells 1/N for its default width: write the one of this width
        text = re.sub(r"const inv_n : f32\[\] = \S+", f"const inv_n : f32[] = {1.0 / dims['N']!r}", graph_text(mc, name))
        x = oracle.normal_values(dims["M"] * dims["N"], 7).reshape(dims["M"], dims["N"])
        with mc.CompiledGraph(text=text, dims=dims) as exe:
            got = exe.run([x])[0].reshape(dims["M"], dims["N"])
        t = torch.from_numpy(x).to(torch.float64)
        if name == "x1_softmax":
            want = torch.softmax(t, dim=-1).numpy()
        else:
            g = oracle.parse_mcg(text, dims)
            gamma, beta = (np.asarray(g.node(c).value, dtype=np.float64).reshape(-1) for c in ("gamma", "beta"))
            eps = float(np.asarray(g.node("eps").value).reshape(-1)[0])
            want = torch.nn.functional.layer_norm(t, (dims["N"],), torch.from_numpy(gamma), torch.from_numpy(beta), eps).numpy()
        err = nse(got, want)
        assert err <= 1e-5, f"{name} {dims}: {err:.2e} against torch float64"


# ------------------------------------------ mc_run on pinned memory in overlapping row slices


@pytest.mark.parametrize("name,dims,matmul", [
    ("c5_mlp_stack", {"B": 8192, "D": 1024}, "tensor_core_f16"),
    ("c5_mlp_stack", {"B": 4096, "D": 1024}, "tensor_core_bf16"),
    ("c3_ffn", {"T": 4096, "D": 1024, "H": 4096}, "tensor_core_tf32"),
    ("c3_ffn", {"T": 4096, "D": 1024, "H": 2048}, "auto"),
    ("c1_mlp_block", {"B": 16384}, "auto"),
    ("c4_matmul", {"M": 8192, "N": 2048, "K": 512}, "tensor_core_bf16"),
    ("x1_softmax", {"M": 4096, "N": 4096}, "auto"),
])
def test_run_in_row_slices_on_pinned_memory_is_bit_identical(mc, oracle, name, dims, matmul):
    """On pinned buffers mc_run cuts a row-independent graph into slices whose copy-in, kernels and copy-out overlap.
    The result must be, bit for bit, what the plain copy-in / run / copy-out path gives (host_io=0), twice in a row
    (the second call reuses buffers the first one left dirty), and the pageable-memory path must agree too."""
    import torch

    path = mc.graph_path(name)
    g = oracle.parse_mcg_file(path, dims)
    ins = [fast_normal(int(np.prod(g.node(n).shape)), 40 + k) for k, n in enumerate(g.inputs)]
    with mc.CompiledGraph(path, dims=dims, options={"matmul": matmul, "host_io": 0}) as exe:
        assert exe.row_slices == 0
        want = exe.run(ins)[0]
    pins = [torch.from_numpy(a).pin_memory() for a in ins]
    out = torch.full((want.size,), float("nan"), dtype=torch.float32).pin_memory()
    with mc.CompiledGraph(path, dims=dims, options={"matmul": matmul}) as exe:
        assert exe.row_slices >= 2, "this graph should run in row slices"
        for _ in range(2):
            exe.run_ptrs([p.data_ptr() for p in pins], [out.data_ptr()])
            assert np.array_equal(out.numpy(), want), f"{name} {matmul}: sliced run differs from the plain run"
            out.fill_(float("nan"))
        assert np.array_equal(exe.run(ins)[0], want)  # pageable buffers: plain path of the same executable
        exe.upload(ins)
        exe.enqueue()
        assert np.array_equal(exe.download()[0], want)  # and the unsliced launch list still works beside it
    with mc.CompiledGraph(path, dims=dims, options={"matmul": matmul, "host_io_row_slices": 5}) as exe:
        # a slice count that does not divide the rows into whole tiles is lowered to one that does
        assert exe.row_slices in (0, 2, 4)
        exe.run_ptrs([p.data_ptr() for p in pins], [out.data_ptr()])
        assert np.array_equal(out.numpy(), want)


def test_row_slices_move_per_row_columns_and_epilogue_operands_with_their_rows(mc, oracle):
    """A graph whose cut values include a per-row column that a matmul epilogue reads, a second full-size input added
    as a residual, an input that is not cut (a row vector) and a row kernel after the matmul: every pointer into a cut
    tensor has to move with the slice, whatever role the tensor plays in its launch."""
    import torch

    text = ("input x : f32[8192, 512]\ninput s : f32[8192, 1]\ninput r : f32[8192, 1024]\ninput v : f32[1024]\n"
            "const w : f32[512, 1024] = uniform(seed=3, lo=-0.05, hi=0.05)\n"
            "z = matmul x, w\nzs = mul z, s\nzr = add zs, r\nzv = add zr, v\nm = row_max zv\nd = sub zv, m\ny = exp d\noutput y, m")
    g = oracle.parse_mcg(text)
    ins = [fast_normal(int(np.prod(g.node(n).shape)), 60 + k) for k, n in enumerate(g.inputs)]
    for matmul in ("auto", "tensor_core_bf16"):
        with mc.CompiledGraph(text=text, options={"matmul": matmul, "host_io": 0}) as exe:
            want = exe.run(ins)
        pins = [torch.from_numpy(a).pin_memory() for a in ins]
        outs = [torch.full((w.size,), float("nan"), dtype=torch.float32).pin_memory() for w in want]
        with mc.CompiledGraph(text=text, options={"matmul": matmul}) as exe:
            assert exe.row_slices >= 2
            exe.run_ptrs([p.data_ptr() for p in pins], [o.data_ptr() for o in outs])
        for got, expect in zip(outs, want):
            assert np.array_equal(got.numpy(), expect), matmul
    rows = np.array([0, 511, 512, 4095, 8191])
    sub = oracle.parse_mcg(text.replace("8192", str(len(rows))))
    expect = oracle.evaluate_f64(sub, [ins[0].reshape(8192, 512)[rows], ins[1].reshape(8192, 1)[rows], ins[2].reshape(8192, 1024)[rows], ins[3]])
    with mc.CompiledGraph(text=text) as exe:
        got = exe.run(ins)
    assert nse(got[0].reshape(8192, 1024)[rows], expect[0]) <= 1e-4 and nse(got[1].reshape(8192, 1)[rows], expect[1]) <= 1e-4


def test_row_slices_with_an_output_that_later_layers_also_read(mc, oracle):
    """The MLP stack with a middle activation as a second output: that value is written in FP32 (for the caller, outside
    the buffer pool) and in 16 bits (for the next layer, inside it) by the same launch; both forms move with the slice."""
    import torch

    dims = {"B": 8192, "D": 1024}
    text = with_outputs(graph_text(mc, "c5_mlp_stack"), ["a3", "a7"])
    x = fast_normal(8192 * 1024, 77)
    with mc.CompiledGraph(text=text, dims=dims, options={"matmul": "tensor_core_f16", "host_io": 0}) as exe:
        want = exe.run([x])
    pin = torch.from_numpy(x).pin_memory()
    outs = [torch.full((w.size,), float("nan"), dtype=torch.float32).pin_memory() for w in want]
    with mc.CompiledGraph(text=text, dims=dims, options={"matmul": "tensor_core_f16"}) as exe:
        assert exe.row_slices >= 2
        exe.run_ptrs([pin.data_ptr()], [o.data_ptr() for o in outs])
    for got, expect in zip(outs, want):
        assert np.array_equal(got.numpy(), expect)


def test_small_or_row_dependent_graphs_are_not_sliced(mc):
    with mc.CompiledGraph(mc.graph_path("c5_mlp_stack"), dims={"B": 256, "D": 256}, options={"matmul": "tensor_core_f16"}) as exe:
        assert exe.row_slices == 0  # moves too little for the overlap to pay
    with mc.CompiledGraph(mc.graph_path("c2_gelu_chain"), dims={"M": 4096, "N": 4096}) as exe:
        assert exe.row_slices == 0  # one streaming kernel: it has its own pipeline
    text = "input x : f32[4096, 4096]\nz = matmul x, x\noutput z"
    with mc.CompiledGraph(text=text, options={"matmul": "tensor_core_bf16"}) as exe:
        assert exe.row_slices == 0


# ------------------------------------------------------- collectives through the library


def test_replicate_constants_and_gather_output_on_a_one_rank_communicator(mc, oracle):
    """The library's own NCCL calls on real NCCL with a world of one (all a single GPU offers): the broadcast leaves
    the constants as they were and rebuilds their 16-bit forms, the all-gather delivers the output."""
    import torch

    if not mc.lib().mcd_nccl_available():
        pytest.skip("libnccl.so.2 cannot be loaded on this machine")
    dims = {"B": 256, "D": 256}
    path = mc.graph_path("c5_mlp_stack")
    x = oracle.normal_values(256 * 256, 1)
    comm = mc.Communicator(1, 0, mc.Communicator.unique_id(), device=0, timeout_s=60.0)
    try:
        with mc.CompiledGraph(path, dims=dims, options={"matmul": "tensor_core_f16"}) as exe:
            want = exe.run([x])[0]
            exe.replicate_constants(comm, root=0)
            assert np.array_equal(exe.run([x])[0], want)
            dst = torch.full((want.size,), float("nan"), dtype=torch.float32, device="cuda")
            exe.gather_output(0, comm, dst.data_ptr())
            assert np.array_equal(dst.cpu().numpy(), want)
            with pytest.raises(mc.McError, match="no output 3"):
                exe.gather_output(3, comm, dst.data_ptr())
    finally:
        comm.destroy()


# --------------------------------------------------------- the re-hosted benchmark suites


def test_bench_suites_tensor_core_rows_and_profile_labels(mc):
    """The tensor_core suite on two small shapes: every row was checked against float64 samples before it was timed
    (the suite asserts the rounding bound itself), the sampled-error column stays inside each format's unit
    roundoff, and the times come from a replayed CUDA graph. The profile suite runs one labelled launch."""
    from minicompiler_b200 import bench_suites

    rows = bench_suites.suite_tensor_core(mc, rounds=5, shapes=[(256, 256, 256), (1024, 512, 2048)])
    assert [(r["m"], r["n"], r["k"]) for r in rows] == [(256, 256, 256), (1024, 512, 2048)]
    for r in rows:
        for name, unit in (("tensor_core_tf32", 2.0 ** -11), ("tensor_core_bf16", 2.0 ** -8), ("tensor_core_f16", 2.0 ** -11)):
            col = r[name]
            assert 0.0 < col["max_err_over_abs_dot"] <= 2.0 * unit + 1e-6, (name, col)
            assert col["ms"] > 0 and col["cublas_ms"] > 0 and col["ran"] == [name]
    fp32 = bench_suites.suite_matmul(mc, rounds=5, shapes=[(256, 2048, 512)])[0]["auto"]
    assert fp32["max_err_over_abs_dot"] <= 1e-6 and fp32["ran"] == ["split_k"]
    assert "matmul_512x512x512.tensor_core_bf16" in bench_suites.profile_labels()
    assert bench_suites.suite_profile(mc, only="matmul_512x512x512.tensor_core_bf16") == ["matmul_512x512x512.tensor_core_bf16"]
