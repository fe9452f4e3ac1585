"""Generates the committed fixtures from the reference's own code.

    python tests/golden/make_golden.py

Needs oracle/_ref/libmcref.so (oracle/build_ref.sh; requires the reference checkout). Writes:

  host_logic.json   what the reference's parser + passes + planner produce for its three benchmark
                    graphs and for graphs from its random-graph generator: the printed graph, the
                    memory plans, the fusion groups and the per-stage node counts.
  evaluator.npz     outputs of the reference's double-precision evaluator
                    (tests/test_util.cpp:87-159) on seeded inputs, for the same random graphs and
                    for small instances of the benchmark graphs.

Folded constants in host_logic.json come from the Eigen-free stand-in for the reference's CPU
kernels (oracle/ref_shim/execute_node.cpp), so tests compare them to within 2 ulp, not bitwise.
"""

import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import ref_binding as ref  # noqa: E402
from oracle import reference_cpu as orc  # noqa: E402

BENCH = [("ref_gelu_chain", "M=8,N=64"), ("ref_mlp_block", "B=8,D=32,H=64"), ("ref_matmul_bias_relu", "M=8,K=32,N=16")]
PASSES = ["default", "none", "dne,fold,dne"]
RANDOM_SEEDS = list(range(24))


def describe(graph: "ref.RefGraph") -> dict:
    return {
        "print": graph.print(),
        "plan_pooled": graph.plan(True),
        "plan_unpooled": graph.plan(False),
        "fusion_groups": graph.fusion_groups(),
        "stage_counts": graph.stage_counts(),
    }


def main() -> None:
    if not ref.available():
        raise SystemExit("oracle/_ref/libmcref.so is missing: run oracle/build_ref.sh first")
    logic = {"bench": {}, "bench_default_dims": {}, "random": {}}
    arrays = {}
    for name, dims in BENCH:
        path = str(HERE / "graphs" / f"{name}.mcg")
        logic["bench"][name] = {"dims": dims, "passes": {p: describe(ref.RefGraph(path, dims=dims, passes=p)) for p in PASSES}}
        full = ref.RefGraph(path, passes="default")
        logic["bench_default_dims"][name] = {"stage_counts": full.stage_counts(), "plan_pooled": full.plan(True),
                                             "fusion_groups": full.fusion_groups()}
        g = orc.parse_mcg_file(path, {k: int(v) for k, v in (kv.split("=") for kv in dims.split(","))})
        ins = orc.make_random_inputs(g, 1)
        outs = ref.RefGraph(path, dims=dims, passes="none").evaluate(ins)
        for k, o in enumerate(outs):
            arrays[f"bench/{name}/out{k}"] = o
    for seed in RANDOM_SEEDS:
        text = ref.random_graph_text(seed)
        logic["random"][str(seed)] = {"mcg": text, "passes": {p: describe(ref.RefGraph(text=text, passes=p)) for p in ["default", "none"]}}
        g = orc.parse_mcg(text)
        ins = orc.make_random_inputs(g, 1)
        for k, o in enumerate(ref.RefGraph(text=text, passes="none").evaluate(ins)):
            arrays[f"random/{seed}/out{k}"] = o
    (HERE / "host_logic.json").write_text(json.dumps(logic, indent=0, sort_keys=True))
    np.savez_compressed(HERE / "evaluator.npz", **arrays)
    print("wrote", HERE / "host_logic.json", (HERE / "host_logic.json").stat().st_size, "bytes;",
          HERE / "evaluator.npz", (HERE / "evaluator.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
