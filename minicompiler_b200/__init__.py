"""minicompiler-b200: a B200-native (sm_100a) execution backend for minicompiler graphs.

The product is the shared library `libminicompiler_b200.so` (C++17 host code + hand-written
CUDA kernels) and its C ABI (`include/minicompiler_b200.h`). This package is the thin
Python binding over that ABI, mirroring how the reference is driven from Python
(bench/torch_compare.py:187-211 binds the same `mc_*` calls with ctypes).

There is no CPU execution path in here: compiling or running needs a B200 and raises
otherwise. Host-only calls (parsing, passes, memory plan, kernel generation) work anywhere.
"""

from .api import (  # noqa: F401
    Communicator,
    CompiledGraph,
    HostGraph,
    McError,
    compile_graph,
    graph_path,
    lib,
    resolve_matmul_kernel,
    shard_dims,
    split_k_splits,
    tensor_core_splits,
    tensor_core_tile_n,
    uniform_values,
)

__all__ = [
    "Communicator",
    "CompiledGraph",
    "HostGraph",
    "McError",
    "compile_graph",
    "graph_path",
    "lib",
    "resolve_matmul_kernel",
    "shard_dims",
    "split_k_splits",
    "tensor_core_splits",
    "tensor_core_tile_n",
    "uniform_values",
]
