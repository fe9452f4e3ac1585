#!/bin/sh
# Builds oracle/_ref/libmcref.so from the reference's own sources where they lie
# (read-only checkout, default /root/reference) plus the two shim files in
# oracle/ref_shim. Only the reference's Eigen-dependent translation unit
# (src/cpu/kernels.cpp) is replaced, by ref_shim/execute_node.cpp.
# Nothing is copied out of the reference; the output is git-ignored.
set -e
REF="${MINICOMPILER_REFERENCE:-/root/reference}"
HERE="$(cd "$(dirname "$0")" && pwd)"
[ -d "$REF/src" ] || { echo "no reference checkout at $REF" >&2; exit 3; }
mkdir -p "$HERE/_ref"
g++ -std=c++17 -O2 -fPIC -shared -ffp-contract=off -fvisibility=hidden \
    -I "$HERE/ref_shim" -I "$REF/include" -I "$REF/src" -I "$REF/tests" \
    "$REF/src/graph.cpp" "$REF/src/ops.cpp" "$REF/src/fused_program.cpp" "$REF/src/parser.cpp" "$REF/src/random.cpp" \
    "$REF/src/graph_builder.cpp" "$REF/src/passes/dead_node_elimination.cpp" "$REF/src/passes/constant_folding.cpp" \
    "$REF/src/passes/operator_fusion.cpp" "$REF/src/passes/pipeline.cpp" "$REF/src/runtime/memory_plan.cpp" \
    "$REF/src/runtime/host_tensor.cpp" "$REF/src/cuda/codegen.cpp" "$REF/tests/test_util.cpp" \
    "$HERE/ref_shim/execute_node.cpp" "$HERE/ref_shim/ref_driver.cpp" \
    -o "$HERE/_ref/libmcref.so"
echo "$HERE/_ref/libmcref.so"
