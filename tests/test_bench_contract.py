"""The parts of bench.py's contract that need no GPU: the reference arm's JSON line, the config both arms print,
the work model behind the roofline, and the parsing of the clock samples."""

import importlib.util
import json
import subprocess
import sys

from conftest import ROOT


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "c1", "--steps", "2", "--warmup", "1"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in line, key
    assert line["impl"] == "reference" and line["metric"] == "graph TFLOP/s" and line["unit"] == "TFLOP/s" and line["steps"] == 2
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1 and line["value"] > 0
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["vs_baseline"] is None and line["gpu_launches"] == 0
    # the same config object the GPU arm prints for this workload
    assert line["config"] == _bench().workload_config("c1", {"B": 256})


def test_default_workload_and_the_also_list():
    bench = _bench()
    assert "c5_f16" in bench.WORKLOADS and bench.WORKLOADS["c5_f16"][1] == {"B": 65536, "D": 2048} and bench.WORKLOADS["c5_f16"][3] == "B"
    for name in bench.DEFAULT_ALSO.split(","):
        assert name in bench.WORKLOADS
    assert {"c2", "c4_bf16", "c4_bf16_16384", "c4_bf16_m128", "c3_tf32", "c3_fp32", "c1"} == set(bench.DEFAULT_ALSO.split(","))


def test_work_model(oracle, mc):
    bench = _bench()
    g = oracle.parse_mcg_file(mc.graph_path("c5_mlp_stack"), {"B": 64, "D": 32})
    assert bench.algorithmic_work(oracle, g, "flops") == 8 * 2 * 64 * 32 * 32
    g = oracle.parse_mcg_file(mc.graph_path("c2_gelu_chain"), {"M": 8, "N": 16})
    assert bench.algorithmic_work(oracle, g, "bytes") == 2 * 4 * 8 * 16
    g = oracle.parse_mcg_file(mc.graph_path("c4_matmul"), {"M": 128, "N": 8192, "K": 8192})
    # 2(mk + kn) + 4mn with 16-bit operands: what a skinny matmul must stream at least
    assert bench.matmul_operand_bytes(g, 2) == 2 * (128 * 8192 + 8192 * 8192) + 4 * 128 * 8192


def test_clock_samples_are_summarised():
    bench = _bench()

    class Finished:
        def terminate(self):
            pass

    sampler = bench.ClockSampler(0)
    sampler.proc = Finished()
    sampler.lines = ["2026/01/02 03:04:05.100, 0, 1665, 1965, 998.21, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
                     "2026/01/02 03:04:05.120, 0, 1700, 1965, [N/A], 0x0, Not Active, Not Active, Not Active, Not Active", "not a sample"]
    assert sampler.stop() == {"sm_mhz": 1682.5, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 2, "power_w_max": 998.21}
    # with the load's window marked, only the samples taken inside it count; those of the timed region are counted apart
    import datetime
    at = lambda text: datetime.datetime.strptime(text, "%Y/%m/%d %H:%M:%S.%f").timestamp()
    windowed = bench.ClockSampler(0)
    windowed.proc = Finished()
    windowed.lines = ["2026/01/02 03:04:04.900, 0, 1965, 1965, 150.0, 0x0, Not Active, Not Active, Not Active, Not Active"] + sampler.lines + [
        "2026/01/02 03:04:05.300, 0, 1500, 1965, 990.0, 0x4, Not Active, Not Active, Not Active, Active",
        "2026/01/02 03:04:06.000, 0, 1965, 1965, 140.0, 0x0, Not Active, Not Active, Not Active, Not Active"]
    windowed.window = (at("2026/01/02 03:04:05.000"), at("2026/01/02 03:04:05.200"), at("2026/01/02 03:04:05.500"))
    windowed.timed_steps_only = False
    got = windowed.stop()
    assert got["samples"] == 3 and got["samples_in_timed_region"] == 2 and got["sm_mhz"] == 1665.0 and got["power_w_max"] == 998.21
    assert got["sm_mhz_timed_region"] == 1682.5
    assert got["reasons"] == ["sw_power_cap"] and "repeated" in got["window"]
    idle = bench.ClockSampler(0)
    assert idle.stop()["reasons"] == ["nvidia-smi unavailable"]
