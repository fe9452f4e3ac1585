"""ctypes binding of oracle/_ref/libmcref.so: the reference's own host code (parser, passes,
planner, elementwise generator, double-precision evaluator, random-graph generator) compiled
from its sources by oracle/build_ref.sh.

TEST INFRASTRUCTURE, NOT PRODUCT. The library exists only where the reference checkout was
available at build time; `available()` says whether it does, and tests that need it skip
otherwise (fixtures generated from it are committed under tests/golden/).
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import List, Optional, Sequence

import numpy as np

_PATH = Path(__file__).resolve().parent / "_ref" / "libmcref.so"
_lib: Optional[C.CDLL] = None


def available() -> bool:
    return _PATH.exists()


def _load() -> C.CDLL:
    global _lib
    if _lib is None:
        L = C.CDLL(str(_PATH))
        vp, cp, i32, i64 = C.c_void_p, C.c_char_p, C.c_int, C.c_longlong
        fpp = C.POINTER(C.POINTER(C.c_float))
        for name, res, args in [
            ("ref_open_file", vp, [cp, cp, cp, cp, i32]),
            ("ref_open_text", vp, [cp, cp, cp, cp, i32]),
            ("ref_close", None, [vp]),
            ("ref_print", i32, [vp, cp, i32]),
            ("ref_stage_counts", i32, [vp, cp, i32]),
            ("ref_plan", i32, [vp, i32, cp, i32]),
            ("ref_fusion_groups", i32, [vp, cp, i32]),
            ("ref_emit_cuda", i32, [vp, cp, i32]),
            ("ref_num_inputs", i32, [vp]),
            ("ref_num_outputs", i32, [vp]),
            ("ref_input_elements", i64, [vp, i32]),
            ("ref_output_elements", i64, [vp, i32]),
            ("ref_evaluate", i32, [vp, fpp, fpp]),
            ("ref_random_graph", i32, [C.c_ulonglong, i32, i32, cp, i32]),
            ("ref_uniform_values", None, [C.POINTER(C.c_float), i64, C.c_ulonglong, C.c_float, C.c_float]),
        ]:
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _text(fn, *args) -> str:
    need = fn(*args, None, 0)
    buf = C.create_string_buffer(need + 1)
    fn(*args, buf, need + 1)
    return buf.value.decode()


class RefGraph:
    """A graph parsed and optimized by the reference's own code."""

    def __init__(self, path: Optional[str] = None, *, text: Optional[str] = None, dims: str = "", passes: str = "default"):
        L = _load()
        err = C.create_string_buffer(1 << 14)
        if text is not None:
            self._g = L.ref_open_text(text.encode(), dims.encode(), passes.encode(), err, len(err))
        else:
            self._g = L.ref_open_file(path.encode(), dims.encode(), passes.encode(), err, len(err))
        if not self._g:
            raise RuntimeError(err.value.decode())

    def __del__(self):
        if getattr(self, "_g", None):
            _load().ref_close(self._g)
            self._g = None

    def print(self) -> str:
        return _text(_load().ref_print, self._g)

    def stage_counts(self) -> List[tuple]:
        return [tuple(int(v) for v in pair.split(",")) for pair in _text(_load().ref_stage_counts, self._g).split()]

    def plan(self, pool_outputs: bool = True) -> dict:
        import json
        return json.loads(_text(_load().ref_plan, self._g, 1 if pool_outputs else 0))

    def fusion_groups(self) -> List[List[str]]:
        return [line.split() for line in _text(_load().ref_fusion_groups, self._g).splitlines() if line]

    def emit_cuda(self) -> str:
        return _text(_load().ref_emit_cuda, self._g)

    def input_elements(self) -> List[int]:
        L = _load()
        return [L.ref_input_elements(self._g, k) for k in range(L.ref_num_inputs(self._g))]

    def output_elements(self) -> List[int]:
        L = _load()
        return [L.ref_output_elements(self._g, k) for k in range(L.ref_num_outputs(self._g))]

    def evaluate(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        """The reference's double-precision evaluator (tests/test_util.cpp:87-159)."""
        ins = [np.ascontiguousarray(a, dtype=np.float32).reshape(-1) for a in inputs]
        outs = [np.empty(n, dtype=np.float32) for n in self.output_elements()]
        in_arr = (C.POINTER(C.c_float) * max(1, len(ins)))(*[a.ctypes.data_as(C.POINTER(C.c_float)) for a in ins])
        out_arr = (C.POINTER(C.c_float) * max(1, len(outs)))(*[a.ctypes.data_as(C.POINTER(C.c_float)) for a in outs])
        _load().ref_evaluate(self._g, in_arr, out_arr)
        return outs


def random_graph_text(seed: int, num_ops: int = 16, allow_matmul: bool = True) -> str:
    """The reference's random-graph generator (tests/test_util.cpp:177-341) as .mcg text."""
    return _text(_load().ref_random_graph, seed, num_ops, 1 if allow_matmul else 0)


def uniform_values(count: int, seed: int, lo: float, hi: float) -> np.ndarray:
    out = np.empty(count, dtype=np.float32)
    _load().ref_uniform_values(out.ctypes.data_as(C.POINTER(C.c_float)), count, seed, lo, hi)
    return out
