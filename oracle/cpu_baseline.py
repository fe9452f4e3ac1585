"""The timed CPU baseline: the oracle's graph executor driven through oracle_kernels.c.

TEST / BENCH INFRASTRUCTURE, NOT PRODUCT (see oracle/reference_cpu.py).

It executes a graph the way the reference's CPU backend does after its pass pipeline: nodes in
order (src/cpu/cpu_backend.cpp:86-114); runs of same-shape elementwise nodes are evaluated as one
fused program, block by block (src/cpu/kernels.cpp:199-262), which is what the `fuse` pass gives
the reference; matmuls go to a row-major float32 GEMM (:192-197). Constant-only subexpressions
are evaluated once ahead of time, as the `fold` pass would. The kernels take a thread count; the
reference itself is single-threaded (bench/harness.hpp:254).

build() compiles oracle_kernels.c with gcc into oracle/liboracle_kernels.so (git-ignored).
"""

from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import reference_cpu as orc

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "oracle_kernels.c"
_LIB = _HERE / "liboracle_kernels.so"
_lib: Optional[C.CDLL] = None

_OPS = {"neg": 0, "exp": 1, "log": 2, "sqrt": 3, "relu": 4, "sigmoid": 5, "tanh": 6, "add": 7, "sub": 8, "mul": 9, "div": 10}


class _Instr(C.Structure):
    _fields_ = [("kind", C.c_int), ("op", C.c_int), ("a", C.c_int), ("b", C.c_int), ("imm", C.c_float)]


def build(force: bool = False) -> Path:
    if force or not _LIB.exists() or _LIB.stat().st_mtime < _SRC.stat().st_mtime:
        # x86-64-v3 (AVX2 + FMA units, no contraction) runs on every host this is used on.
        subprocess.run(["gcc", "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
                        "-fvisibility=hidden", str(_SRC), "-o", str(_LIB), "-lm"], check=True)
    return _LIB


def _load() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_LIB))
        L.oracle_fused.restype = C.c_int
        L.oracle_sgemm.restype = None
        L.oracle_max_threads.restype = C.c_int
        _lib = L
    return _lib


def max_threads() -> int:
    """Host threads the port may use: the cores this process may run on. The OpenMP default is not used because
    launchers such as torchrun export OMP_NUM_THREADS=1 to every rank; the kernels take the count explicitly."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    return max(1, min(cores, 64))


def _fptr(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _classify(shape: Sequence[int], out: Sequence[int]):
    n_in = int(np.prod(shape)) if len(shape) else 1
    n_out = int(np.prod(out)) if len(out) else 1
    if n_in == 1:
        return 1, 0
    if n_in == n_out:
        return 0, 0
    core = list(shape)
    while core and core[0] == 1:
        core.pop(0)
    if len(core) <= len(out) and list(out[len(out) - len(core):]) == core:
        return 2, n_in
    return None, 0


class CpuPlan:
    """A graph prepared for repeated timed runs."""

    def __init__(self, graph: orc.McgGraph, threads: int = 1):
        self.g, self.threads = graph, max(1, threads)
        # Graphs with row reductions (an extension without a C port) run through the numpy restatement, one thread.
        self.numpy_only = any(n.op in orc.REDUCE for n in graph.nodes)
        if self.numpy_only:
            self.threads = 1
        self.how = ("numpy restatement of the CPU path, 1 thread" if self.numpy_only
                    else f"C port of the reference CPU kernels with {self.threads} OpenMP threads")
        self.users: Dict[str, List[str]] = {n.name: [] for n in graph.nodes}
        for n in graph.nodes:
            for o in n.operands:
                self.users[o].append(n.name)
        # fold: values that depend on constants only
        self.values: Dict[str, np.ndarray] = {}
        const = set()
        for n in graph.nodes:
            if n.op == "const":
                self.values[n.name] = np.ascontiguousarray(n.value, dtype=np.float32)
                const.add(n.name)
            elif n.op != "input" and all(o in const for o in n.operands):
                sub = orc.McgGraph("fold", [graph.node(o) for o in self._closure(n.name)], [], [n.name], {})
                self.values[n.name] = np.ascontiguousarray(orc.evaluate_f32(sub, [])[0].reshape(n.shape))
                const.add(n.name)
        self.const = const
        self.segments = [] if self.numpy_only else self._segment()

    def _closure(self, name: str) -> List[str]:
        need, order = set(), []

        def visit(v):
            if v in need:
                return
            need.add(v)
            for o in self.g.node(v).operands:
                visit(o)
            order.append(v)

        visit(name)
        pos = {n.name: i for i, n in enumerate(self.g.nodes)}
        return sorted(order, key=lambda v: pos[v])

    def _segment(self):
        segs, cur = [], []
        for n in self.g.nodes:
            if n.op in ("input", "const") or n.name in self.const:
                continue
            if n.op == "matmul":
                if cur:
                    segs.append(("fused", cur))
                    cur = []
                segs.append(("matmul", [n]))
                continue
            ok = not cur or tuple(cur[0].shape) == tuple(n.shape)
            if ok:
                inside = {c.name for c in cur}
                for o in n.operands:
                    if o not in inside and _classify(self.g.node(o).shape, n.shape)[0] is None:
                        ok = False
            if not ok and cur:
                segs.append(("fused", cur))
                cur = []
            cur.append(n)
        if cur:
            segs.append(("fused", cur))
        return segs

    def run(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        if self.numpy_only:
            return orc.evaluate_f32(self.g, inputs)
        L = _load()
        vals = dict(self.values)
        for name, a in zip(self.g.inputs, inputs):
            vals[name] = np.ascontiguousarray(a, dtype=np.float32).reshape(self.g.node(name).shape)
        outputs = set(self.g.outputs)
        for kind, nodes in self.segments:
            if kind == "matmul":
                n = nodes[0]
                a, b = vals[n.operands[0]], vals[n.operands[1]]
                c = np.empty(n.shape, dtype=np.float32)
                L.oracle_sgemm(_fptr(a), _fptr(b), _fptr(c), C.c_longlong(a.shape[0]), C.c_longlong(a.shape[1]),
                               C.c_longlong(b.shape[1]), C.c_int(self.threads))
                vals[n.name] = c
                continue
            shape = nodes[0].shape
            count = int(np.prod(shape)) if len(shape) else 1
            inside = {n.name for n in nodes}
            ext, prog, reg = [], [], {}
            for n in nodes:
                for o in n.operands:
                    if o not in reg:
                        if o in inside:
                            raise AssertionError("operand order")
                        v = vals[o]
                        if v.size == 1 and o in self.const:
                            prog.append((1, 0, -1, -1, float(v.reshape(-1)[0])))
                        else:
                            k, period = _classify(self.g.node(o).shape, shape)
                            ext.append((v, k, period))
                            prog.append((0, 0, len(ext) - 1, -1, 0.0))
                        reg[o] = len(prog) - 1
                if n.op in orc.UNARY:
                    prog.append((2, _OPS[n.op], reg[n.operands[0]], -1, 0.0))
                else:
                    prog.append((3, _OPS[n.op], reg[n.operands[0]], reg[n.operands[1]], 0.0))
                reg[n.name] = len(prog) - 1
            instrs = (_Instr * len(prog))(*[_Instr(*p) for p in prog])
            outs = (C.POINTER(C.c_float) * len(prog))()
            for n in nodes:
                needed = n.name in outputs or any(u not in inside for u in self.users[n.name]) or n is nodes[-1]
                if needed:
                    buf = np.empty(count, dtype=np.float32)
                    vals[n.name] = buf.reshape(shape)
                    outs[reg[n.name]] = _fptr(buf)
            in_ptrs = (C.POINTER(C.c_float) * max(1, len(ext)))(*[_fptr(e[0]) for e in ext])
            kinds = (C.c_int * max(1, len(ext)))(*[e[1] for e in ext])
            periods = (C.c_longlong * max(1, len(ext)))(*[e[2] for e in ext])
            rc = L.oracle_fused(instrs, C.c_int(len(prog)), in_ptrs, kinds, periods, C.c_int(len(ext)), outs,
                                C.c_longlong(count), C.c_int(self.threads))
            if rc != 0:
                raise RuntimeError("oracle_fused rejected the program")
        return [np.ascontiguousarray(vals[o]).reshape(-1) for o in self.g.outputs]
