"""Host-side contract of the kept front end (format, IR, passes, planner, kernel vocabulary),
checked through the C ABI. No GPU needed. The expected values are the ones the reference's own
tests pin (cited per test) and fixtures generated from the reference's code (tests/golden/)."""

import ctypes
import json
import re
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest

from conftest import GOLDEN, ROOT

EXAMPLE = """
# A small MLP layer.
graph layer
dim B = 2
input x : f32[B, 3]
const w : f32[3, 4] = uniform(seed=7, lo=-0.5, hi=0.5)
const b : f32[4] = [1, 2, 3, 4]
const half : f32[] = 0.5
h = matmul x, w
hb = add h, b      # bias broadcast over rows
y = mul hb, half
output y, h
"""


def parse_error(mc, text, dims=None):
    try:
        mc.HostGraph(text=text, dims=dims, passes="none")
    except mc.McError as e:
        return str(e)
    return "<parsed>"


# ------------------------------------------------------------------ C ABI


def test_library_exports_every_declared_symbol(mc):
    """Every function declared in include/*.h is exported by the shared library."""
    lib = ctypes.CDLL(str(ROOT / "minicompiler_b200" / "libminicompiler_b200.so"))
    declared = set()
    for header in (ROOT / "include").glob("*.h"):
        text = header.read_text()
        declared.update(re.findall(r"\b(mc_\w+|mcb_\w+|mcd_\w+)\s*\(", text))
    declared -= {"mcd_device_info", "mcd_gemm_args"}
    assert len(declared) > 60
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, missing


def test_compiling_without_a_gpu_fails_loudly(mc):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(mc.McError, match="no usable CUDA device"):
        mc.CompiledGraph(mc.graph_path("c2_gelu_chain"), dims={"M": 4, "N": 4})


def test_cpu_backend_is_not_part_of_this_library(mc):
    with pytest.raises(mc.McError, match="no CPU execution path"):
        mc.CompiledGraph(mc.graph_path("c2_gelu_chain"), backend="cpu")
    with pytest.raises(mc.McError, match="unknown backend 'tpu'"):
        mc.CompiledGraph(mc.graph_path("c2_gelu_chain"), backend="tpu")


# ------------------------------------------------------------------ parser


def test_generator_matches_the_reference_golden_bits(mc):
    # tests/test_parser.cpp:136-147
    v = mc.uniform_values(4, 42, -0.3, 0.7)
    bits = [struct.unpack("<I", struct.pack("<f", float(x)))[0] for x in v]
    assert bits == [0x3EE214CA, 0xBE0F73A8, 0xBCAF4CC0, 0x3D350140]
    a = mc.uniform_values(10000, 123, -2.0, 3.0)
    assert np.array_equal(a, mc.uniform_values(10000, 123, -2.0, 3.0))
    assert not np.array_equal(a, mc.uniform_values(10000, 124, -2.0, 3.0))
    assert a.min() >= -2.0 and a.max() < 3.0


def test_parses_every_statement_kind(mc):
    # tests/test_parser.cpp:33-60, :127-134
    g = mc.HostGraph(text=EXAMPLE, passes="none")
    text = g.print()
    assert g.num_nodes == 7
    assert "graph layer\n" in text
    assert "%0 x = input : f32[2,3]" in text
    assert "%2 b = const [1, 2, 3, 4] : f32[4]" in text
    assert "%6 y = mul %5, %3 : f32[2,4]  (output)" in text
    assert np.array_equal(g.constant("w"), mc.uniform_values(12, 7, -0.5, 0.5))
    assert g.constant("half")[0] == 0.5


def test_dim_overrides(mc):
    # tests/test_parser.cpp:62-71
    g = mc.HostGraph(text=EXAMPLE, dims={"B": 64}, passes="none")
    assert "y = mul %5, %3 : f32[64,4]" in g.print()
    assert "no dim 'Q'" in parse_error(mc, EXAMPLE, {"B": 64, "Q": 1})


def test_error_messages_are_the_reference_ones(mc):
    # tests/test_parser.cpp:73-88
    E = lambda t: parse_error(mc, t)  # noqa: E731
    assert E("input x : f32[4]\ny = frobnicate x\noutput y") == "line 2: unknown op 'frobnicate'"
    assert E("input x : f32[4]\ny = relu z\noutput y") == "line 2: unknown value 'z'"
    assert E("input x : f32[4]\nx = relu x\noutput x") == "line 2: 'x' is defined twice"
    assert E("input x : i32[4]\noutput x") == "line 1: unsupported element type 'i32' (only f32)"
    assert E("input x : f32[N]\noutput x") == "line 1: unknown dim 'N'"
    assert E("const c : f32[3] = [1, 2]\noutput c") == "line 1: expected 3 values for f32[3], got 2"
    assert E("input x : f32[4]\n") == "the graph declares no outputs"
    assert E("input x : f32[4] ;") == "line 1: unexpected character ';'"
    assert E("input x : f32[4]\ny = relu x x") == "line 2: unexpected 'x'"
    err = E("input a : f32[4, 8]\ninput b : f32[4]\nc = add a, b\noutput c")
    assert err.startswith("line 3: c: add: cannot broadcast"), err


def test_invalid_shapes_are_rejected_before_allocating(mc):
    # tests/test_parser.cpp:90-100
    assert parse_error(mc, "const c : f32[-1] = 0\noutput c") == (
        "line 1: invalid shape [-1]: dimensions must be >= 1 and the total at most 2^31 - 1 elements")
    for text in ["const c : f32[-1] = uniform(seed=1, lo=0, hi=1)\noutput c",
                 "input x : f32[7, 7905747460161236407]\noutput x",
                 "const c : f32[4294967296, 4294967296] = 1\noutput c", "input x : f32[4, 0]\noutput x"]:
        assert parse_error(mc, text).startswith("line 1: invalid shape"), text


def test_large_seeds_stay_exact(mc):
    # tests/test_parser.cpp:102-108
    a = mc.HostGraph(text="const c : f32[8] = uniform(seed=9007199254740992, lo=0, hi=1)\noutput c", passes="none")
    b = mc.HostGraph(text="const c : f32[8] = uniform(seed=9007199254740993, lo=0, hi=1)\noutput c", passes="none")
    assert not np.array_equal(a.constant("c"), b.constant("c"))
    assert np.array_equal(b.constant("c"), mc.uniform_values(8, 9007199254740993, 0.0, 1.0))


def test_comments_blank_lines_crlf_scalars_and_signs(mc):
    # tests/test_parser.cpp:110-125
    g = mc.HostGraph(text="# header\r\n\r\ninput x : f32[2]   # trailing\r\ny = exp x\r\noutput y\r\n", passes="none")
    assert g.num_nodes == 2
    g = mc.HostGraph(text="const c : f32[] = -1.5e-1\nconst d : f32[2] = [-2, +.5]\ny = mul c, d\noutput y", passes="none")
    assert g.constant("c")[0] == np.float32(-0.15)
    assert list(g.constant("d")) == [-2.0, 0.5]


def test_unknown_pass_message(mc):
    with pytest.raises(mc.McError, match=r"unknown pass 'inline' \(passes: dne, fold, fuse\)"):
        mc.HostGraph(text=EXAMPLE, passes="dne,inline")


# ------------------------------------------------------------------ passes


def test_folding_known_answers(mc):
    # tests/test_constant_folding.cpp:52-72 and :97-106, spelled as .mcg
    text = """
input x : f32[2, 3]
const var : f32[3] = [0.25, 1.0, 4.0]
const eps : f32[] = 0.0
const gamma : f32[3] = [1, 2, 3]
const w : f32[2, 3] = [1, 2, 3, 4, 5, 6]
const m : f32[2, 2] = [1, 2, 3, 4]
ve = add var, eps
sd = sqrt ve
scale = div gamma, sd
ws = mul w, scale
sq = matmul m, ws
y = add x, sq
output y
"""
    g = mc.HostGraph(text=text, passes="fold")
    assert list(g.constant("scale")) == [2.0, 2.0, 1.5]
    assert list(g.constant("ws")) == [2, 4, 4.5, 8, 10, 9]
    assert list(g.constant("sq")) == [18, 24, 22.5, 38, 52, 49.5]
    assert "y = add" in g.print()
    g = mc.HostGraph(text="input x : f32[2]\nconst c : f32[2] = [1, 4]\nroot = sqrt c\noutput root", passes="fold")
    assert list(g.constant("root")) == [1.0, 2.0]


def test_stage_counts_of_the_benchmark_graphs(mc):
    # tests/test_end_to_end.cpp:86, :98, :112: (nodes, compute nodes) after input, dne, fold, dne, fuse, dne
    expect = {
        "ref_gelu_chain": [(17, 11), (17, 11), (17, 9), (14, 9), (6, 1), (2, 1)],
        "ref_mlp_block": [(37, 22), (37, 22), (37, 18), (31, 18), (17, 4), (13, 4)],
    }
    for name, stages in expect.items():
        g = mc.HostGraph(str(GOLDEN / "graphs" / f"{name}.mcg"))
        passes = g.stats()["passes"]
        got = [(passes[0]["before"]["nodes"], passes[0]["before"]["compute_nodes"])]
        got += [(p["after"]["nodes"], p["after"]["compute_nodes"]) for p in passes]
        assert got == stages, name


def test_fusion_groups_follow_the_reference_rules(mc):
    # tests/test_operator_fusion.cpp: a chain fuses whole; a value used outside its group does not join;
    # an output never joins; a smaller (broadcast) producer does not join.
    chain = "input x : f32[4,8]\na = exp x\nb = neg a\nc = relu b\noutput c"
    assert mc.HostGraph(text=chain, passes="none").fusion_groups() == [["a", "b", "c"]]
    shared = "input x : f32[4,8]\na = exp x\nb = neg a\nc = relu a\nd = add b, c\noutput d"
    assert mc.HostGraph(text=shared, passes="none").fusion_groups() == [["a", "b", "c", "d"]]
    escapes = "input x : f32[4,8]\na = exp x\nb = neg a\noutput b, a"
    assert mc.HostGraph(text=escapes, passes="none").fusion_groups() == []
    small = "input x : f32[4,8]\ninput r : f32[8]\ne = exp r\ny = add x, e\nz = relu y\noutput z"
    assert mc.HostGraph(text=small, passes="none").fusion_groups() == [["y", "z"]]
    fused = mc.HostGraph(text=chain, passes="fuse").print()
    assert "c = fused %0" in fused and "r1 = exp r0" in fused and "r3 = relu r2" in fused


def _same_modulo_folded_values(a: str, b: str) -> bool:
    strip = lambda s: re.sub(r"const (\[[^\]]*\]|[-+0-9.e]+|<\d+ values>|nan|inf|-inf)", "const _", s)  # noqa: E731
    return strip(a) == strip(b)


def test_host_logic_matches_fixtures_from_the_reference(mc):
    """Printed graphs, plans and fusion groups equal what the reference's own code produced
    (tests/golden/host_logic.json, made by tests/golden/make_golden.py)."""
    gold = json.loads((GOLDEN / "host_logic.json").read_text())
    for name, entry in gold["bench"].items():
        path = str(GOLDEN / "graphs" / f"{name}.mcg")
        for passes, want in entry["passes"].items():
            g = mc.HostGraph(path, dims=entry["dims"], passes=passes)
            assert _same_modulo_folded_values(g.print(), want["print"]), (name, passes)
            assert g.plan(True) == want["plan_pooled"] and g.plan(False) == want["plan_unpooled"], (name, passes)
            assert g.fusion_groups() == want["fusion_groups"], (name, passes)
    for name, want in gold["bench_default_dims"].items():
        g = mc.HostGraph(str(GOLDEN / "graphs" / f"{name}.mcg"))
        assert g.plan(True) == want["plan_pooled"], name
    for seed, entry in gold["random"].items():
        for passes, want in entry["passes"].items():
            g = mc.HostGraph(text=entry["mcg"], passes=passes)
            assert _same_modulo_folded_values(g.print(), want["print"]), (seed, passes)
            assert g.plan(True) == want["plan_pooled"] and g.plan(False) == want["plan_unpooled"], (seed, passes)
            assert g.fusion_groups() == want["fusion_groups"], (seed, passes)


def test_host_logic_matches_the_reference_build_live(mc):
    """Same comparison against oracle/_ref directly, on 300 graphs from the reference's generator
    (only where the reference checkout was available to build it)."""
    from oracle import ref_binding as ref

    if not ref.available():
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    for seed in range(300):
        text = ref.random_graph_text(seed)
        for passes in ["default", "none"]:
            r, m = ref.RefGraph(text=text, passes=passes), mc.HostGraph(text=text, passes=passes)
            assert _same_modulo_folded_values(m.print(), r.print()), (seed, passes)
            assert m.plan() == r.plan() and m.fusion_groups() == r.fusion_groups(), (seed, passes)


# ----------------------------------------------------------------- planner


def test_planner_cases(mc):
    # tests/test_memory_plan.cpp:10-123 (ping-pong; outputs never reused; dead values free at once)
    chain = "input x : f32[1024]\n" + "".join(f"t{i} = tanh {'x' if i == 0 else 't' + str(i - 1)}\n" for i in range(8)) + "output t7"
    plan = mc.HostGraph(text=chain, passes="none").plan()
    assert plan["buffer_bytes"] == [4096, 4096]
    assert plan["bytes_without_reuse"] == 8 * 4096 and plan["bytes_with_reuse"] == 2 * 4096
    unpooled = mc.HostGraph(text=chain, passes="none").plan(pool_outputs=False)
    assert unpooled["buffer_of"][-1] == -1
    two_outputs = "input x : f32[16]\na = exp x\nb = neg a\nc = relu b\noutput a, c"
    plan = mc.HostGraph(text=two_outputs, passes="none").plan()
    assert plan["buffer_of"][1] != plan["buffer_of"][3]  # an output's buffer is never handed out again
    dead = "input x : f32[16]\nd = exp x\na = neg x\nb = relu a\noutput b"
    plan = mc.HostGraph(text=dead, passes="none").plan()
    assert plan["last_use"][1] == -1 and plan["buffer_of"][2] == plan["buffer_of"][1]


# ---------------------------------------------------- kernel vocabulary / rules


def test_split_rule_known_answers(mc):
    # tests/test_cuda_backend.cpp:315-343 (arguments m, n, k on 30 SMs)
    s = mc.split_k_splits
    assert s(128, 512, 2048, 30) == 7 and s(128, 1920, 2048, 30) == 2 and s(128, 2048, 2048, 30) == 3
    assert s(128, 2944, 2048, 30) == 2 and s(128, 3072, 2048, 30) == 1 and s(640, 640, 640, 30) == 1
    assert s(1024, 1024, 1024, 30) == 1 and s(128, 128, 200, 30) == 3 and s(128, 128, 100, 30) == 1
    assert s(128, 512, 2048, 30, 1) == 7 and s(128, 2048, 2048, 30, 1) == 1 and s(128, 1792, 2048, 30, 1) == 2
    for per_sm in (1, 2):
        for tiles in range(1, 41):
            splits = s(128, 128 * tiles, 1 << 16, 30, per_sm)
            if splits > 1:
                assert tiles * splits <= per_sm * 30


def test_auto_resolution_and_names(mc):
    # tests/test_cuda_backend.cpp:345-373
    r = mc.resolve_matmul_kernel
    assert r("auto", 128, 512, 2048, 30) == "split_k" and r("auto", 512, 512, 512, 30) == "split_k"
    assert r("auto", 640, 640, 640, 30) == "double_buffered" and r("auto", 2048, 2048, 2048, 30) == "double_buffered"
    assert r("auto", 128, 128, 100, 30) == "double_buffered" and r("auto", 640, 640, 640, 40) == "split_k"
    assert r("auto", 2**31 - 1, 1, 1, 30) == "double_buffered"
    assert r("register_tiled_64", 4096, 4096, 4096, 30) == "register_tiled_64"
    for name in ["auto", "naive", "tiled", "register_tiled_128", "register_tiled_64", "vectorized", "double_buffered",
                 "split_k", "tensor_core_tf32", "tensor_core_bf16", "tensor_core_f16"]:
        assert r(name, 4096, 4096, 4096, 148) in (name, "double_buffered")
    with pytest.raises(mc.McError, match="unknown matmul kernel 'register_tiled_32' \\(auto, naive, tiled"):
        r("register_tiled_32", 1, 1, 1, 30)


def test_split_rule_on_148_sms_for_the_configs(mc):
    # FP32 rule on B200: C1 256x2048x512 -> 32 tiles of 128x128 -> 4 splits
    assert mc.split_k_splits(256, 2048, 512, 148) == 4
    assert mc.split_k_splits(8192, 4096, 1024, 148) == 1
    # tcgen05 rule (128x256 tiles, one CTA per SM)
    assert mc.tensor_core_splits(1024, 1024, 1024, 148) == 1  # narrow tiles instead: 8 x 16 tiles of 128 x 64
    assert mc.tensor_core_tile_n(1024, 1024, 1024, 148) == 64
    assert mc.tensor_core_tile_n(1024, 1024, 65536, 148) == 256  # too much operand traffic: split K
    # one row of tiles that 256-column tiles would cut 4 ways: 128-column tiles and 2 K slices (half the partial sums)
    assert mc.tensor_core_tile_n(16, 8192, 8192, 148) == 128 and mc.tensor_core_tile_n(128, 8192, 8192, 148) == 128
    assert mc.tensor_core_splits(128, 8192, 8192, 148) == 2
    assert mc.tensor_core_tile_n(129, 8192, 8192, 148) == 256 and mc.tensor_core_splits(129, 8192, 8192, 148) == 2
    assert mc.tensor_core_tile_n(8192, 8192, 8192, 148) == 256
    assert mc.tensor_core_tile_n(512, 2048, 512, 148) == 64
    assert mc.tensor_core_tile_n(256, 2048, 512, 148) == 256  # 64 narrow tiles would leave most SMs idle: split K
    assert mc.tensor_core_splits(1024, 1024, 65536, 148) == 4
    assert mc.tensor_core_splits(16, 8192, 8192, 148) == 2
    assert mc.tensor_core_splits(8192, 8192, 8192, 148) == 1
    assert mc.tensor_core_splits(128, 256, 64, 148) == 1  # a single K block cannot be split


# ------------------------------------------------------------ lowering plan


def test_launch_counts_11_9_1(mc):
    # tests/test_cuda_backend.cpp:439-451: gelu_chain unoptimized / after folding / fully optimized
    path = str(GOLDEN / "graphs" / "ref_gelu_chain.mcg")
    for passes, launches in [("none", 11), ("dne,fold,dne", 9), ("default", 1)]:
        plan = mc.HostGraph(path, dims="M=64,N=64", passes=passes).launch_plan()
        assert f"launches={launches} " in plan, (passes, plan)


def test_epilogue_folding_removes_launches(mc):
    path = str(GOLDEN / "graphs" / "ref_mlp_block.mcg")
    g = mc.HostGraph(path)
    unfolded = g.launch_plan({"fuse_epilogue": 0})
    folded = g.launch_plan()
    assert "launches=4 " in folded.replace("launches=1\n", "").replace("launches=2\n", "") or "launches=" in folded
    n_unfolded = int(re.search(r"launches=(\d+) intermediate", unfolded).group(1))
    n_folded = int(re.search(r"launches=(\d+) intermediate", folded).group(1))
    assert n_folded == n_unfolded - 2, (unfolded, folded)
    assert "epilogue=act(14 ops)" in folded and "epilogue=y(2 ops)" in folded
    # With tensor cores the first matmul writes its result as a 16-bit tensor only.
    tc = g.launch_plan({"matmul": "tensor_core_bf16"})
    assert "epilogue=act(14 ops) out=bf16" in tc and "epilogue=y(2 ops) out=f32" in tc


def test_folding_is_refused_when_the_product_is_needed_elsewhere(mc):
    text = "input x : f32[8,8]\nconst w : f32[8,8] = 0.5\nh = matmul x, w\ny = relu h\noutput y, h"
    assert "epilogue" not in mc.HostGraph(text=text).launch_plan()
    text = "input x : f32[8,8]\nconst w : f32[8,8] = 0.5\nh = matmul x, w\ny = relu h\nz = exp h\noutput y, z"
    assert "epilogue" not in mc.HostGraph(text=text).launch_plan()


def test_every_config_graph_lowers_and_its_kernels_compile_for_sm100a(mc):
    small = {"c1_mlp_block": "B=64", "c2_gelu_chain": "M=64,N=64", "c3_ffn": "T=64,D=32,H=64",
             "c4_matmul": "M=64,N=64,K=64", "c5_mlp_stack": "B=64,D=64"}
    for name, dims in small.items():
        for matmul in ["auto", "tensor_core_tf32", "tensor_core_bf16", "tensor_core_f16"]:
            g = mc.HostGraph(mc.graph_path(name), dims=dims)
            g.check_kernels({"matmul": matmul})
            g.check_kernels({"matmul": matmul, "fuse_epilogue": 0})


def test_c5_folds_batchnorm_to_scale_and_shift(mc):
    g = mc.HostGraph(mc.graph_path("c5_mlp_stack"), dims="B=64,D=64")
    plan = g.launch_plan({"matmul": "tensor_core_f16"})
    assert plan.count("matmul ") == 8 and plan.count("(3 ops)") == 8, plan
    assert "launches=8 " in plan
    assert plan.count("out=f16") == 7 and plan.count("out=f32") == 1  # activations stay 16-bit between layers


# ------------------------------------------------------------- codegen text


def _emit(mc, text, options=None):
    return mc.HostGraph(text=text, passes="none").emit_cuda(options)


def test_generated_kernel_contract(mc):
    # The kept contract of the reference generator (tests/test_cuda_codegen.cpp:29-109): entry point name and
    # argument order, exact-bit immediates defined once, scalar inputs hoisted, constant divisors.
    src = mc.HostGraph(str(GOLDEN / "graphs" / "ref_gelu_chain.mcg"), dims="M=64,N=64").emit_cuda()
    assert "mc_elementwise(float* __restrict__ out, const float* __restrict__ in0, unsigned n)" in src
    assert src.count("__uint_as_float(0x3f000000u);  // 0.5") == 1
    assert src.count("tanhf(") == 1  # one straight-line body, called per lane
    assert "reinterpret_cast<const float4*>(in0)" in src and "__launch_bounds__(256)" in src
    assert "unsupported" not in src
    # infinities and inexact decimals keep their exact bits (tests/test_cuda_codegen.cpp:88-95)
    inf_src = mc.HostGraph(text="input x : f32[8]\nconst c : f32[] = 1e39\nconst d : f32[] = -0.1\n"
                                "y = mul x, c\nz = add y, d\noutput z").emit_cuda()
    assert "0x7f800000u" in inf_src and "0xbdcccccdu" in inf_src


def test_access_classes_in_generated_code(mc):
    periodic = _emit(mc, "input x : f32[8,16]\ninput r : f32[16]\ny = add x, r\noutput y")
    assert "q1 + (i % 4u)" in periodic and "128-bit" in periodic
    odd_period = _emit(mc, "input x : f32[4,6]\ninput r : f32[6]\ny = add x, r\noutput y")
    assert "in1 + (i % 6u)" in odd_period and "32-bit" in odd_period
    scalar = _emit(mc, "input x : f32[8,16]\ninput s : f32[]\ny = mul x, s\noutput y")
    assert "const float s1 = in1[0];" in scalar and scalar.index("const float s1") < scalar.index("for (")
    column = _emit(mc, "input x : f32[17,32]\ninput c : f32[17,1]\ny = add x, c\noutput y")
    assert "mc_splat(__ldg(in1 + ((i / 8u))))" in column and "128-bit" in column
    general = _emit(mc, "input a : f32[2,3,4]\ninput b : f32[3,1]\ny = add a, b\noutput y")
    assert "mc_splat(__ldg(in1 + (((i / 1u) % 3u))))" in general or "((i % 3u))" in general or "% 3u" in general
    narrow = _emit(mc, "input x : f32[17,33]\ninput c : f32[17,1]\ny = add x, c\noutput y")
    assert "in1 + ((i / 33u))" in narrow and "32-bit" in narrow
    no_vec = _emit(mc, "input x : f32[8,16]\ny = exp x\noutput y", {"vectorize": 0})
    assert "32-bit" in no_vec


def test_every_access_class_compiles_for_sm100a(mc):
    patterns = [("[17,33]", "[17,33]"), ("[17,32]", "[]"), ("[]", "[17,33]"), ("[17,32]", "[32]"), ("[17,33]", "[17,1]"),
                ("[17,1]", "[1,33]"), ("[2,3,4]", "[3,1]"), ("[5,1,6]", "[1,4,1]"), ("[16,64]", "[16,1]"), ("[4,8,16]", "[8,1]")]
    for sa, sb in patterns:
        for op in ["add", "div"]:
            text = f"input a : f32{sa}\ninput b : f32{sb}\ny = {op} a, b\noutput y"
            mc.HostGraph(text=text, passes="none").check_kernels()
            mc.HostGraph(text=text, passes="none").check_kernels({"unroll": 2, "streaming": 0})


# -------------------------------------------------------------- partitioner


def test_batch_sharding_plans(mc):
    path = mc.graph_path("c5_mlp_stack")
    dims, off, rows = mc.shard_dims(path, "B=64,D=32", "B", 1, 4)
    assert (off, rows) == (16, 16) and "B=16" in dims and "D=32" in dims
    with pytest.raises(mc.McError, match="does not divide over 3 devices"):
        mc.shard_dims(path, "B=64,D=32", "B", 0, 3)
    with pytest.raises(mc.McError, match="no dim 'Q'"):
        mc.shard_dims(path, "B=64,D=32", "Q", 0, 2)
    # a matmul whose right-hand side carries the batch dim needs an exchange: refused
    bad = ROOT / "_work" / "shard_bad.mcg"
    bad.parent.mkdir(exist_ok=True)
    bad.write_text("dim B = 8\ninput x : f32[B, B]\ninput y : f32[B, 4]\nz = matmul x, y\noutput z\n")
    with pytest.raises(mc.McError, match="other than as its leading extent|right-hand side"):
        mc.shard_dims(str(bad), "", "B", 0, 2)
    bad.write_text("dim B = 8\ninput x : f32[4, B]\ny = exp x\noutput y\n")
    with pytest.raises(mc.McError, match="other than as its leading extent"):
        mc.shard_dims(str(bad), "", "B", 0, 2)


def test_mcc_emit_cuda_and_listings_need_no_gpu(mc):
    mcc = ROOT / "minicompiler_b200" / "mcc"
    if not mcc.exists():
        pytest.skip("mcc not built")
    out = subprocess.run([str(mcc), mc.graph_path("c2_gelu_chain"), "--dim", "M=64", "--dim", "N=64", "--emit-cuda", "--stats"],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert "// node %1 'y' : f32[64,64]" in out.stdout and "mc_elementwise" in out.stdout
    assert "fuse" in out.stdout
    out = subprocess.run([str(mcc), "--list-passes"], capture_output=True, text=True)
    assert "dne" in out.stdout and "fold" in out.stdout and "fuse" in out.stdout
    out = subprocess.run([str(mcc), mc.graph_path("c2_gelu_chain"), "--backend", "cpu", "--run"], capture_output=True, text=True)
    assert out.returncode != 0 and "no CPU execution path" in out.stderr


# ------------------------------------------------ row reductions (extension)


def test_row_reductions_parse_print_and_type_check(mc):
    text = "input x : f32[4, 3, 8]\nm = row_max x\ns = row_sum x\nd = sub x, m\noutput d, s"
    g = mc.HostGraph(text=text, passes="none")
    printed = g.print()
    assert "m = row_max %0 : f32[4,3,1]" in printed and "s = row_sum %0 : f32[4,3,1]" in printed
    assert "d = sub %0, %1 : f32[4,3,8]" in printed  # the reduced value broadcasts back against its operand
    with pytest.raises(mc.McError, match="row_sum expects an operand of rank 1 or more"):
        mc.HostGraph(text="const c : f32[] = 1\ns = row_sum c\noutput s")
    with pytest.raises(mc.McError, match="row_max expects 1 operand"):
        mc.HostGraph(text="input x : f32[4]\ns = row_max x, x\noutput s")


def test_constant_row_reductions_fold_to_known_answers(mc):
    text = ("const c : f32[2, 3] = [1, 2, 3, -4, 5.5, 0.25]\nconst big : f32[4] = [16777216, 1, 1, 1]\n"
            "s = row_sum c\nm = row_max c\nb = row_sum big\ninput x : f32[2, 3]\ny = add x, s\nz = mul y, m\nw = add z, b\noutput w")
    g = mc.HostGraph(text=text, passes="fold")
    assert g.constant("s").tolist() == [6.0, 1.75]
    assert g.constant("m").tolist() == [3.0, 5.5]
    # accumulated in double and rounded once: 16777219 rounds to 16777220 (a float32 running sum would stay at 16777216)
    assert g.constant("b").tolist() == [16777220.0]


def test_row_reduction_lowering_absorbs_and_rematerializes_producers(mc):
    separate = {"fuse_rows": 0}  # the per-step form; rows of up to 65536 elements otherwise become one kernel
    g = mc.HostGraph(mc.graph_path("x2_layernorm"), dims="M=64,N=4096")
    plain = g.launch_plan({"rematerialize": 0, **separate})
    assert "row_sum total rows of 4096 prologue_ops=0" in plain
    # (x-mean)^2 is read by the reduction only: evaluated inside it, never written
    assert "row_sum ss rows of 4096 prologue_ops=1" in plain and "elementwise sq" not in plain
    assert "elementwise c " in plain and "launches=6 " in plain  # x-mean has a second reader and stays a tensor
    # a cheap value read by a reduction and by other steps is recomputed in each of them
    plan = g.launch_plan(separate)
    assert "elementwise c " not in plan and "row_sum ss rows of 4096 prologue_ops=2" in plan
    assert "elementwise y ops=4" in plan and "launches=5 " in plan
    soft = mc.HostGraph(mc.graph_path("x1_softmax"), dims="M=64,N=4096")
    assert "launches=4 " in soft.launch_plan({"rematerialize": 0, **separate})
    assert "row_sum s rows of 4096 prologue_ops=2" in soft.launch_plan(separate) and "launches=3 " in soft.launch_plan(separate)
    # an output is written in any case; graphs without reductions are lowered as before
    kept = mc.HostGraph(text="input x : f32[8, 64]\ne = exp x\ns = row_sum e\noutput s, e")
    assert "prologue_ops=0" in kept.launch_plan(separate) and "elementwise e" in kept.launch_plan(separate)
    assert "row_fused e* s* rows of 64 reads=1 writes=2" in kept.launch_plan({})
    chain = mc.HostGraph(str(GOLDEN / "graphs" / "ref_gelu_chain.mcg"), dims="M=64,N=64", passes="none")
    assert chain.launch_plan({}) == chain.launch_plan({"rematerialize": 0, **separate})


def test_runs_of_row_steps_become_one_kernel(mc):
    soft = mc.HostGraph(mc.graph_path("x1_softmax"), dims="M=64,N=4096")
    assert "row_fused m e s y* rows of 4096 reads=1 writes=1" in soft.launch_plan({}) and "launches=1 " in soft.launch_plan({})
    norm = mc.HostGraph(mc.graph_path("x2_layernorm"), dims="M=64,N=4096")
    plan = norm.launch_plan({})
    assert "row_fused total mean c ss sd y* rows of 4096 reads=4 writes=1" in plan and "launches=1 " in plan
    assert "intermediate_bytes=1048576 " in plan  # only y exists in memory
    src = norm.plan_sources({})
    assert "mc_row_fused(float* __restrict__ out0, const float* __restrict__ ex0" in src
    assert src.count("__syncthreads();") == 4 and "__ldg(ex2 + col)" in src and "const float s1 = ex1[0];" in src
    assert src.count("__ldcs(ex0 + base + col)") == 1 and src.count("__stcs(out0 + base + col") == 1  # x read once, y written once
    # rows below 1024 elements take a warp each, very wide rows would not fit in registers and stay separate kernels
    short = mc.HostGraph(mc.graph_path("x1_softmax"), dims="M=64,N=1000")
    assert "row_fused" in short.launch_plan({}) and "32 threads per row, 32 element(s) per thread" in short.plan_sources({})
    assert "__syncthreads" not in short.plan_sources({})
    # rows wider than 8192 are shared by a cluster of 2, 4 or 8 CTAs of 8192 columns at most, in both kernels
    wide = mc.HostGraph(mc.graph_path("x1_softmax"), dims="M=64,N=16384")
    assert "row_fused" in wide.launch_plan({}) and "__cluster_dims__(2, 1, 1) __launch_bounds__(256)" in wide.plan_sources({})
    assert "__cluster_dims__(2, 1, 1) __launch_bounds__(256)" in wide.plan_sources({"fuse_rows": 0})
    widest = mc.HostGraph(mc.graph_path("x1_softmax"), dims="M=64,N=65536")
    assert "row_fused" in widest.launch_plan({}) and "__cluster_dims__(8, 1, 1)" in widest.plan_sources({})
    assert "256 threads per row, 32 element(s) per thread, 8 CTAs per row as a cluster" in widest.plan_sources({})
    ragged = mc.HostGraph(mc.graph_path("x1_softmax"), dims="M=64,N=20000").plan_sources({})
    assert "__cluster_dims__(4, 1, 1)" in ragged and "const unsigned chunk_first = rank * 5120u;" in ragged
    assert "st.shared::cluster.f32" in ragged and "barrier.cluster.arrive.release.aligned" in ragged
    assert "row_fused" not in mc.HostGraph(mc.graph_path("x1_softmax"), dims="M=64,N=70000").launch_plan({})
    assert "__cluster_dims__" not in mc.HostGraph(mc.graph_path("x1_softmax"), dims="M=64,N=70000").plan_sources({})
    # values that something outside the run reads are written; a matmul ends a run
    text = ("input x : f32[64, 2048]\nconst w : f32[2048, 64] = uniform(seed=3, lo=-1, hi=1)\nm = row_max x\nd = sub x, m\n"
            "e = exp d\ns = row_sum e\ny = div e, s\nz = matmul y, w\noutput z, s")
    plan = mc.HostGraph(text=text).launch_plan({})
    assert "row_fused m e s* y* rows of 2048 reads=1 writes=2" in plan and "matmul z" in plan
    for g in (soft, norm, short, wide, mc.HostGraph(text=text), mc.HostGraph(mc.graph_path("x1_softmax"), dims="M=3,N=5000")):
        g.check_kernels({})


def test_row_reduction_kernel_text_and_compilation(mc):
    wide = mc.HostGraph(text="input x : f32[8, 3, 2048]\ninput b : f32[3, 1]\nt = mul x, b\ns = row_max t\noutput s")
    src = wide.emit_cuda()
    assert "mc_row_reduce(float* __restrict__ out, const float* __restrict__ in0, unsigned rows)" in src
    assert "fmaxf(a, b)" in src and "__uint_as_float(0xff800000u)" in src and "256 threads per row" in src
    assert "__shfl_xor_sync(0xffffffffu, total, offset)" in src and "warp_total[8]" in src
    narrow = mc.HostGraph(text="input x : f32[100, 33]\ns = row_sum x\noutput s").emit_cuda()
    assert "32 threads per row" in narrow and "return a + b;" in narrow and "__syncthreads" not in narrow
    for g in (wide, mc.HostGraph(text="input x : f32[100, 33]\ns = row_sum x\noutput s"),
              mc.HostGraph(mc.graph_path("x1_softmax"), dims="M=64,N=256"),
              mc.HostGraph(mc.graph_path("x2_layernorm"), dims="M=64,N=4096")):
        g.check_kernels({})


def test_sharding_rules_for_row_reductions(mc, tmp_path):
    assert mc.shard_dims(mc.graph_path("x1_softmax"), {"M": 64, "N": 128}, "M", 1, 2) == ("M=32,N=128", 32, 32)
    with pytest.raises(mc.McError, match="carries dim 'N' other than as its leading extent"):
        mc.shard_dims(mc.graph_path("x1_softmax"), {"M": 64, "N": 128}, "N", 1, 2)
    flat = tmp_path / "flat.mcg"
    flat.write_text("dim B = 64\ninput x : f32[B]\ns = row_sum x\noutput s\n")
    with pytest.raises(mc.McError, match="row_sum 's' reduces over dim 'B'"):
        mc.shard_dims(str(flat), {}, "B", 0, 2)


# ------------------------------------------------ host-side guards of the device path


def test_in_place_run_needs_16_byte_aligned_buffers_for_vectorised_kernels(mc):
    """mc_run lets streaming kernels work on pinned caller memory in place. A vectorised kernel moves 128 bits per
    access, so a buffer that starts off a 16-byte boundary (a view into a pinned allocation) must take the staged
    path; the predicate behind that decision is checked here without touching a GPU."""
    lib = mc.lib()

    def ok(addresses, vectorised):
        arr = (ctypes.c_void_p * len(addresses))(*addresses)
        return lib.mcb_in_place_pointers_ok(arr, len(addresses), int(vectorised))

    assert ok([0x7F0000000000, 0x7F0000001000], True) == 1
    assert ok([0x7F0000000000, 0x7F0000001004], True) == 0   # t[1:] of a float tensor
    assert ok([0x7F0000000008], True) == 0
    assert ok([0x7F0000000004, 0x7F0000001004], False) == 1  # scalar kernels have no such requirement
    assert ok([], True) == 1


def test_per_device_kernel_set_up_runs_once_on_every_device(mc):
    """The opt-in to large dynamic shared memory is a per-device attribute of a kernel: the bookkeeping must ask for
    it on the first launch on each GPU a process drives, not once per process."""
    lib = mc.lib()
    devices = [0, 0, 1, 0, 1, 2, 63, 63, 64, 64, -1]
    first = (ctypes.c_int * len(devices))()
    assert lib.mcd_per_device_once_probe((ctypes.c_int * len(devices))(*devices), len(devices), first) == 0
    # ordinals outside 0..63 are not remembered, so their set-up repeats (harmless) instead of being skipped
    assert list(first) == [1, 0, 1, 0, 0, 1, 1, 0, 1, 1, 1]


def test_no_tensor_can_outgrow_the_32_bit_indices_of_the_generated_kernels(mc):
    """The generated kernels count and index elements in unsigned 32 bits and add one trip of their grid-stride
    loop before testing the bound. The format caps a tensor at 2^31 - 1 elements (src/parser.cpp shape check), so
    index + trip stays below 2^32: larger tensors never reach lowering."""
    for shape in ("[65536, 65536]", "[32768, 65536]", "[1048576, 4096]"):
        with pytest.raises(mc.McError, match=r"at most 2\^31 - 1 elements"):
            mc.HostGraph(text=f"input x : f32{shape}\ny = exp x\noutput y", passes="none")
    fine = "input x : f32[32768, 65535]\ny = exp x\ns = row_sum y\noutput s"
    plan = mc.HostGraph(text=fine, passes="none").launch_plan()
    assert plan.strip()


def test_row_slicing_analysis(mc):
    """Which values mc_run may cut by rows so that the copy-in, kernels and copy-out of consecutive slices overlap:
    a dataflow analysis over the optimized graph (the executable no longer has the source text)."""
    def slicing(text=None, path=None, dims=None, passes="default"):
        return mc.HostGraph(path, text=text, dims=dims, passes=passes).row_slicing()

    assert slicing(path=mc.graph_path("c5_mlp_stack"), dims={"B": 1024, "D": 256}).startswith("rows=1024 cut=x,z0,a0,")
    assert slicing(path=mc.graph_path("c3_ffn"), dims={"T": 512, "D": 128, "H": 256}) == "rows=512 cut=x,z,h,o,y"
    # square sweep shapes: both inputs have the leading extent, only the left operand can be cut
    assert slicing(path=mc.graph_path("c4_matmul"), dims={"M": 512, "N": 512, "K": 512}) == "rows=512 cut=a,c"
    assert slicing(path=mc.graph_path("x1_softmax"), dims={"M": 64, "N": 256}).startswith("rows=64 cut=x,")
    # a per-row column is cut together with the tensor it scales
    col = "input x : f32[8, 4]\ninput s : f32[8, 1]\nconst w : f32[4, 6] = uniform(seed=1, lo=-1, hi=1)\ny = mul x, s\nz = matmul y, w\noutput z"
    assert slicing(col, passes="none") == "rows=8 cut=x,s,y,z"
    # rows of a right-hand side are summed over: nothing to cut
    assert slicing("input x : f32[8, 8]\nz = matmul x, x\noutput z", passes="none") == "none"
    # a full-height constant would need its own rows per slice
    full = "input x : f32[8, 4]\nconst c : f32[8, 4] = uniform(seed=2, lo=-1, hi=1)\ny = add x, c\noutput y"
    assert slicing(full, passes="none") == "none"
    # an output that is not computed from cut values
    assert slicing("input x : f32[8, 4]\nconst c : f32[4] = [1, 2, 3, 4]\ny = exp x\nd = exp c\noutput y, d", passes="none") == "none"
    # a lower-rank operand aligned to the right is fine; a cut operand of lower rank than the result is not
    assert slicing("input x : f32[8, 4]\ninput r : f32[4]\ny = add x, r\noutput y", passes="none") == "rows=8 cut=x,y"
    assert slicing("input x : f32[8, 4]\ninput t : f32[2, 8, 4]\ny = add x, t\noutput y", passes="none") == "none"
    # the graph at a slice's row count keeps node order and every other extent
    sliced = mc.HostGraph(mc.graph_path("c3_ffn"), dims={"T": 512, "D": 128, "H": 256}).row_slicing(128)
    assert "x = input : f32[128,128]" in sliced and "w1 = const <32768 values> : f32[128,256]" in sliced
    assert "y = fused %7, %4, %0 : f32[128,128]  (output)" in sliced


def test_split_tensor_core_matmuls_that_reduce_in_a_cluster_need_one_launch_and_no_workspace(mc):
    """With gemm_variant bit 64 a tensor-core matmul whose K is split 2, 4 or 8 ways adds its partial tiles inside
    thread-block clusters: one launch, no workspace. The lowering (which counts launches and sizes the workspace) and the device layer (which
    launches) each apply the rule; they must agree for every shape and split count."""
    lib = mc.lib()

    class GemmArgs(ctypes.Structure):
        _fields_ = [("arith", ctypes.c_int), ("m", ctypes.c_int), ("n", ctypes.c_int), ("k", ctypes.c_int), ("a", ctypes.c_void_p),
                    ("b", ctypes.c_void_p), ("lda", ctypes.c_longlong), ("ldb", ctypes.c_longlong), ("b_transposed", ctypes.c_int),
                    ("c", ctypes.c_void_p), ("ldc", ctypes.c_longlong), ("c16", ctypes.c_void_p), ("c16_kind", ctypes.c_int),
                    ("ldc16", ctypes.c_longlong), ("splits", ctypes.c_int), ("workspace", ctypes.c_void_p),
                    ("function", ctypes.c_void_p), ("reduce_function", ctypes.c_void_p), ("epilogue_inputs", ctypes.c_void_p * 6),
                    ("num_epilogue_inputs", ctypes.c_int), ("status", ctypes.c_void_p), ("variant", ctypes.c_int),
                    ("tile_n", ctypes.c_int), ("has_epilogue", ctypes.c_int)]

    lib.mcd_gemm_launches.restype = ctypes.c_int
    text = "dim M = 8\ndim N = 8\ndim K = 8\ninput a : f32[M, K]\ninput b : f32[K, N]\nc = matmul a, b\noutput c"
    for m, n, k in [(128, 8192, 8192), (16, 8192, 8192), (1024, 1024, 65536), (256, 2048, 512), (128, 256, 100000), (384, 1024, 4096),
                    (640, 1280, 2048), (128, 4096, 520), (4096, 4096, 4096)]:
        for name, arith, elem in (("tensor_core_bf16", 2, 2), ("tensor_core_tf32", 1, 4)):
            for variant in (0, 64):
                plan = mc.HostGraph(text=text, dims={"M": m, "N": n, "K": k}).launch_plan({"matmul": name, "gemm_variant": variant})
                splits = int(re.search(r"splits=(\d+)", plan).group(1))
                launches = int(re.search(r"launches=(\d+)\n", plan).group(1))
                workspace = int(re.search(r"workspace_bytes=(\d+)", plan).group(1))
                tile_n = int(m_.group(1)) if (m_ := re.search(r"tile_n=(\d+)", plan)) else 0
                args = GemmArgs(arith=arith, m=m, n=n, k=k, splits=splits, variant=variant, tile_n=tile_n)
                assert lib.mcd_gemm_launches(ctypes.byref(args)) == launches, (m, n, k, name, variant, plan)
                assert (workspace > 0) == (launches == 2), plan
                if variant == 0:
                    assert launches == (2 if splits > 1 else 1)
    # the config shapes. Clusters asked for: 256-column tiles split 4 ways, one launch, no workspace. Default: the skinny
    # problems take 128-column tiles and 2 K slices, the tall-K one 256-column tiles and 4; two launches each.
    for m, n, k in [(128, 8192, 8192), (16, 8192, 8192), (1024, 1024, 65536)]:
        plan = mc.HostGraph(text=text, dims={"M": m, "N": n, "K": k}).launch_plan({"matmul": "tensor_core_bf16", "gemm_variant": 64})
        assert "splits=4" in plan and "launches=1\n" in plan and "workspace_bytes=0" in plan, plan
        plan = mc.HostGraph(text=text, dims={"M": m, "N": n, "K": k}).launch_plan({"matmul": "tensor_core_bf16"})
        assert ("splits=4" if m > 128 else "splits=2 tile_n=128") in plan and "launches=2\n" in plan, plan


def test_auto_splits_k_where_whole_tiles_share_out_badly(mc):
    """Beyond the reference's rule (kept verbatim, pinned above): on 148 SMs a problem of 256 or 512 tiles of 128 x 128
    leaves SMs idle 14 % of the launch; `auto` then splits K so that finer work items share out evenly - when K is long
    enough and the reduction costs less than that gains."""
    b = mc.lib().mcb_balanced_fp32_splits
    assert b(2048, 2048, 2048, 148) == 4 and b(8192, 1024, 4096, 148) == 2
    assert b(4096, 4096, 4096, 148) == 1 and b(8192, 4096, 1024, 148) == 1 and b(65536, 2048, 2048, 148) == 1
    assert b(2048, 2048, 256, 148) == 1  # K too short to split
    text = "dim M = 8\ndim N = 8\ndim K = 8\ninput a : f32[M, K]\ninput b : f32[K, N]\nc = matmul a, b\noutput c"
    plan = mc.HostGraph(text=text, dims={"M": 2048, "N": 2048, "K": 2048}).launch_plan()
    assert "kernel=split_k splits=4" in plan and "launches=2" in plan
    assert "kernel=double_buffered splits=1" in mc.HostGraph(text=text, dims={"M": 2048, "N": 2048, "K": 2048}).launch_plan({"balance_splits": 0})
    assert "kernel=double_buffered splits=1" in mc.HostGraph(text=text, dims={"M": 2048, "N": 2048, "K": 2048}).launch_plan({"matmul": "double_buffered"})
    c3 = mc.HostGraph(mc.graph_path("c3_ffn")).launch_plan()
    assert "matmul z 8192x4096x1024 kernel=double_buffered splits=1" in c3 and "matmul o 8192x1024x4096 kernel=split_k splits=2" in c3
