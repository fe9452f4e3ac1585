"""The CPU oracle is pinned before anything is checked against it: against the reference's golden
bits, against fixtures produced by the reference's own evaluator, and (where the reference checkout
was available to build oracle/_ref) against that evaluator live. No GPU needed."""

import json
import struct

import numpy as np
import pytest

from conftest import GOLDEN


def test_generator_golden_bits(oracle):
    # tests/test_parser.cpp:136-147 (the same bits bench/mcgraph.py:32-36 checks its NumPy port against)
    v = oracle.uniform_values(4, 42, -0.3, 0.7)
    assert [struct.unpack("<I", struct.pack("<f", float(x)))[0] for x in v] == [0x3EE214CA, 0xBE0F73A8, 0xBCAF4CC0, 0x3D350140]


def test_generator_equals_the_library_one(oracle, mc):
    for seed, lo, hi, n in [(1, -1.0, 1.0, 4097), (11, -0.044, 0.044, 1000), (9007199254740993, 0.0, 1.0, 64)]:
        assert np.array_equal(oracle.uniform_values(n, seed, lo, hi), mc.uniform_values(n, seed, lo, hi))


def test_reader_agrees_with_the_library_reader(oracle, mc):
    for name, dims in [("c1_mlp_block", {"B": 4}), ("c3_ffn", {"T": 4, "D": 8, "H": 16}), ("c5_mlp_stack", {"B": 4, "D": 8})]:
        g = oracle.parse_mcg_file(mc.graph_path(name), dims)
        h = mc.HostGraph(mc.graph_path(name), dims=dims, passes="none")
        assert h.num_nodes == len(g.nodes)
        for n in g.nodes:
            if n.op == "const":
                assert np.array_equal(n.value.reshape(-1), h.constant(n.name)), n.name


def test_f64_evaluator_equals_the_reference_fixtures(oracle):
    """Bit-for-bit against outputs of the reference's evaluator (tests/test_util.cpp:87-159)."""
    gold = json.loads((GOLDEN / "host_logic.json").read_text())
    expected = np.load(GOLDEN / "evaluator.npz")
    checked = 0
    for seed, entry in gold["random"].items():
        g = oracle.parse_mcg(entry["mcg"])
        outs = oracle.evaluate_f64(g, oracle.make_random_inputs(g, 1))
        for k, got in enumerate(outs):
            want = expected[f"random/{seed}/out{k}"]
            # identical up to the last bit of libm's double-precision exp/log/tanh (numpy vs glibc)
            assert np.allclose(got, want, rtol=2.4e-7, atol=0, equal_nan=True), (seed, k)
            checked += 1
    for name, entry in gold["bench"].items():
        dims = {k: int(v) for k, v in (kv.split("=") for kv in entry["dims"].split(","))}
        g = oracle.parse_mcg_file(str(GOLDEN / "graphs" / f"{name}.mcg"), dims)
        got = oracle.evaluate_f64(g, oracle.make_random_inputs(g, 1))[0]
        assert np.allclose(got, expected[f"bench/{name}/out0"], rtol=2.4e-7, atol=0), name
        checked += 1
    assert checked >= 27


def test_f64_evaluator_equals_the_reference_build_live(oracle):
    from oracle import ref_binding as ref

    if not ref.available():
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    exact = 0
    for seed in range(100, 160):
        text = ref.random_graph_text(seed)
        g = oracle.parse_mcg(text)
        ins = oracle.make_random_inputs(g, 1)
        for got, want in zip(oracle.evaluate_f64(g, ins), ref.RefGraph(text=text, passes="none").evaluate(ins)):
            assert np.allclose(got, want, rtol=2.4e-7, atol=0, equal_nan=True), seed
            exact += int(np.array_equal(got, want))
    assert exact > 50


def test_f32_evaluator_is_within_the_reference_cpu_tolerances_of_f64(oracle):
    # tests/test_cpu_backend.cpp:56-58, :176-191: CPU backend vs the double evaluator: 1e-4 * scale on random graphs
    gold = json.loads((GOLDEN / "host_logic.json").read_text())
    for seed, entry in gold["random"].items():
        g = oracle.parse_mcg(entry["mcg"])
        ins = oracle.make_random_inputs(g, 1)
        for a, b in zip(oracle.evaluate_f32(g, ins), oracle.evaluate_f64(g, ins)):
            scale = max(1.0, float(np.max(np.abs(b))))
            assert np.all(np.abs(a.astype(np.float64) - b) <= 1e-4 * scale), seed


def test_unary_and_binary_semantics(oracle):
    # tests/test_cpu_backend.cpp:60-101: neg/relu exact; binary ops bit-exact over broadcast patterns
    g = oracle.parse_mcg("input x : f32[5]\na = neg x\nb = relu x\noutput a, b")
    x = np.array([-2.0, -0.0, 0.0, 3.5, -1e-30], dtype=np.float32)
    a, b = oracle.evaluate_f32(g, [x])
    assert np.array_equal(a, -x) and np.array_equal(b, np.maximum(x, 0))
    g = oracle.parse_mcg("input a : f32[2, 3, 4]\ninput b : f32[3, 1]\ny = div a, b\noutput y")
    ins = oracle.make_random_inputs(g, 5, 0.5, 2.0)
    want = (ins[0] / ins[1].reshape(1, 3, 1)).reshape(-1)
    assert np.array_equal(oracle.evaluate_f32(g, ins)[0], want)


def test_folding_known_answers_hold_in_the_oracle(oracle):
    # tests/test_constant_folding.cpp:52-72
    g = oracle.parse_mcg("""
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
output scale, ws, sq
""")
    scale, ws, sq = oracle.evaluate_f32(g, [np.zeros((2, 3), np.float32)])
    assert list(scale) == [2.0, 2.0, 1.5] and list(ws) == [2, 4, 4.5, 8, 10, 9] and list(sq) == [18, 24, 22.5, 38, 52, 49.5]


def test_rounding_helpers(oracle):
    x = np.array([1.0, 1.00390625, 1.001953125, -3.14159, 65504.0, 1e-8], dtype=np.float32)
    import torch

    t = torch.from_numpy(x)
    assert np.array_equal(oracle.round_to_bf16(x), t.to(torch.bfloat16).to(torch.float32).numpy())
    assert np.array_equal(oracle.round_to_f16(x), t.to(torch.float16).to(torch.float32).numpy())
    tf = oracle.round_to_tf32(x)
    assert np.all(np.abs(tf - x) <= np.abs(x) * 2.0 ** -11) and np.all((tf.view(np.uint32) & 0x1FFF) == 0)


def test_normal_generator_is_seeded_and_standard(oracle):
    a = oracle.normal_values(200000, 7)
    assert np.array_equal(a, oracle.normal_values(200000, 7)) and not np.array_equal(a, oracle.normal_values(200000, 8))
    assert abs(float(a.mean())) < 0.01 and abs(float(a.std()) - 1.0) < 0.01


def test_row_reductions_of_the_oracle_known_answers(oracle):
    """The extension ops as the oracle defines them: last dimension to extent 1, sums in double rounded once."""
    g = oracle.parse_mcg("input x : f32[2, 4]\ns = row_sum x\nm = row_max x\nd = sub x, m\noutput s, m, d")
    x = np.array([[16777216, 1, 1, 1], [-1, -2, -0.5, -8]], dtype=np.float32)
    s, m, d = oracle.evaluate_f32(g, [x])
    assert s.tolist() == [16777220.0, -11.5] and m.tolist() == [16777216.0, -0.5]
    assert d.reshape(2, 4)[1].tolist() == [-0.5, -1.5, 0.0, -7.5]
    s64, m64, _ = oracle.evaluate_f64(g, [x])
    assert np.array_equal(s64, s) and np.array_equal(m64, m)
    assert g.node("s").shape == (2, 1)
