#!/bin/sh
# One Nsight Compute report per labelled launch of the profile suite, as the reference collects its per-kernel
# evidence (scripts/profile_kernels_ncu.sh:30-60 over bench_cuda --suite profile):
#
#     sh minicompiler_b200/profile_kernels_ncu.sh OUT_DIR [LABEL ...]
#
# Without labels every label of `python -m minicompiler_b200.bench_suites --suite profile --list` is captured.
# Each label runs once without the profiler first and is captured only if that run exits 0; the capture is one
# NVTX range holding one launch of a small problem (64 MB of GELU, or a matmul of at most 2048^3), taken with
# --clock-control none so that the GPU's clocks are left alone. Raw CSV pages are written beside the reports.
set -eu
OUT="${1:?usage: profile_kernels_ncu.sh OUT_DIR [LABEL ...]}"
shift
mkdir -p "$OUT"
if [ "$#" -eq 0 ]; then
    set -- $(python -m minicompiler_b200.bench_suites --suite profile --list)
fi
for label in "$@"; do
    echo "profiling $label"
    if ! python -m minicompiler_b200.bench_suites --suite profile --only "$label" > "$OUT/$label.plain.log" 2>&1; then
        echo "  skipped: the plain run failed, see $OUT/$label.plain.log"
        continue
    fi
    ncu --set full --clock-control none --nvtx --nvtx-include "$label/" --force-overwrite --export "$OUT/$label" \
        python -m minicompiler_b200.bench_suites --suite profile --only "$label" > "$OUT/$label.log" 2>&1
    ncu --import "$OUT/$label.ncu-rep" --page raw --csv --print-units base > "$OUT/$label.csv"
done
echo "wrote $OUT"
