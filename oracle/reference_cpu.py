"""CPU restatement of the reference's graph-execution path.

TEST INFRASTRUCTURE, NOT PRODUCT: only tests/, __graft_entry__.smoke() and the CPU-baseline /
reference legs of bench.py may import this. The product (minicompiler_b200/) never does.

What it restates, with the reference file:line each part follows:

* `uniform_values`      the seeded generator: splitmix64, top 24 bits as an exact float in [0,1),
                        `lo + (hi-lo)*u` with the product rounded to float before the add
                        (src/random.cpp:6-26); input k of a graph uses seed S+k
                        (src/runtime/host_tensor.cpp:7-14).
* `parse_mcg`           an independent reader of the .mcg text format (grammar of
                        include/minicompiler/parser.hpp:13-25): graph / dim (with overrides) /
                        input / const (splat, literal list, uniform(...)) / `name = op a, b` / output.
* `evaluate_f32`        the CPU backend's semantics: nodes run in order (src/cpu/cpu_backend.cpp:86-114),
                        every op is one float32 operation per element with NumPy-style broadcasting
                        (src/cpu/kernels.cpp:143-190), sigmoid is 1/(1+exp(-x)) (:27), relu is max(x,0)
                        (:26), matmul is a row-major float32 GEMM (:192-197). The reference evaluates
                        fused programs instruction by instruction in float registers (:199-262), which
                        is the same arithmetic as running the unfused ops, so this evaluator runs the
                        graph as written, without passes.
* `evaluate_f64`        the reference's own test oracle (tests/test_util.cpp:87-159): every node is
                        computed in double from float operands and rounded to float once.

Parity status: PINNED. The generator is checked against the reference's golden bits
(tests/test_parser.cpp:136-147); `evaluate_f64` is checked against the reference's own evaluator
compiled from its sources (oracle/_ref, built by oracle/build_ref.sh) and against fixtures
generated from it (tests/golden/); `evaluate_f32` is held to `evaluate_f64` within the tolerances
the reference uses between its CPU backend and that evaluator (tests/test_cpu_backend.cpp:56-58).
The arithmetic of the reference's CPU backend itself lives in Eigen 3.4.0 (pinned in
cmake/Dependencies.cmake:12-28, not vendored, absent here), so there are no bit-level golden
outputs of its transcendental functions to pin against; the reference's tests do not have any either.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

_MASK = (1 << 64) - 1


def _splitmix64_stream(seed: int, count: int) -> np.ndarray:
    """count draws of splitmix64 started at `seed` (src/random.cpp:6-12), vectorised."""
    with np.errstate(over="ignore"):
        idx = np.arange(1, count + 1, dtype=np.uint64)
        z = np.uint64(seed & _MASK) + idx * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform_values(count: int, seed: int, lo: float, hi: float) -> np.ndarray:
    """src/random.cpp:14-26: u = (draw >> 40) * 2^-24; lo + (hi - lo) * u, each step rounded to float."""
    draws = _splitmix64_stream(seed, count)
    u = (draws >> np.uint64(40)).astype(np.float32) * np.float32(2.0 ** -24)
    lo32, hi32 = np.float32(lo), np.float32(hi)
    scaled = (hi32 - lo32) * u  # float32 product, rounded
    return (lo32 + scaled).astype(np.float32)


def normal_values(count: int, seed: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    """N(mean, std) floats by Box-Muller over the same splitmix64 stream. The reference has no normal
    generator (its .mcg only knows uniform, src/parser.cpp:336-345); configs that ask for N(0,1) inputs
    get this one, fed identically to the GPU and to this oracle."""
    pairs = (count + 1) // 2
    draws = _splitmix64_stream(seed, 2 * pairs)
    u = ((draws >> np.uint64(11)).astype(np.float64) + 1.0) * (2.0 ** -53)  # (0, 1]
    r = np.sqrt(-2.0 * np.log(u[:pairs]))
    theta = 2.0 * np.pi * u[pairs:]
    z = np.concatenate([r * np.cos(theta), r * np.sin(theta)])[:count]
    return (mean + std * z).astype(np.float32)


# ------------------------------------------------------------------ reader

UNARY = ("neg", "exp", "log", "sqrt", "relu", "sigmoid", "tanh")
BINARY = ("add", "sub", "mul", "div")
# Row reductions: an extension of this build with no counterpart in the reference (its README.md:561-562 lists
# reductions as future work), so their parity is unpinned. Definition: the last dimension collapses to extent 1;
# row_sum is the double-precision sum rounded to float32 once, row_max the largest element (no NaN expected).
REDUCE = ("row_sum", "row_max")


def _reduce(op: str, x: np.ndarray) -> np.ndarray:
    if op == "row_sum":
        return np.sum(x.astype(np.float64), axis=-1, keepdims=True).astype(np.float32)
    return np.max(x, axis=-1, keepdims=True)


@dataclass
class McgNode:
    name: str
    op: str  # "input", "const", one of UNARY / BINARY, "matmul"
    shape: Tuple[int, ...]
    operands: List[str] = field(default_factory=list)
    value: Optional[np.ndarray] = None  # constants


@dataclass
class McgGraph:
    name: str
    nodes: List[McgNode]
    inputs: List[str]
    outputs: List[str]
    dims: Dict[str, int]

    def node(self, name: str) -> McgNode:
        for n in self.nodes:
            if n.name == name:
                return n
        raise KeyError(name)


_NUM = r"[-+]?(?:\d+\.?\d*|\.\d+)(?:[eE][-+]?\d+)?"


def _broadcast(a: Sequence[int], b: Sequence[int]) -> Tuple[int, ...]:
    return tuple(np.broadcast_shapes(tuple(a), tuple(b)))


def parse_mcg(text: str, dims: Optional[Dict[str, int]] = None) -> McgGraph:
    dims = dict(dims or {})
    declared: Dict[str, int] = {}
    nodes: List[McgNode] = []
    by_name: Dict[str, McgNode] = {}
    g = McgGraph("graph", nodes, [], [], declared)

    def shape_of(spec: str) -> Tuple[int, ...]:
        spec = spec.strip()
        if not spec:
            return ()
        return tuple(declared[t.strip()] if not re.fullmatch(r"[-+]?\d+", t.strip()) else int(t) for t in spec.split(","))

    def add(node: McgNode) -> None:
        if node.name in by_name:
            raise ValueError(f"'{node.name}' is defined twice")
        nodes.append(node)
        by_name[node.name] = node

    for raw in text.splitlines():
        line = raw.split("#", 1)[0].strip()
        if not line:
            continue
        m = re.fullmatch(r"graph\s+(\w+)", line)
        if m:
            g.name = m.group(1)
            continue
        m = re.fullmatch(r"dim\s+(\w+)\s*=\s*([-+]?\d+)", line)
        if m:
            declared[m.group(1)] = int(dims.get(m.group(1), int(m.group(2))))
            continue
        m = re.fullmatch(r"input\s+(\w+)\s*:\s*f32\s*\[(.*?)\]", line)
        if m:
            add(McgNode(m.group(1), "input", shape_of(m.group(2))))
            g.inputs.append(m.group(1))
            continue
        m = re.fullmatch(r"const\s+(\w+)\s*:\s*f32\s*\[(.*?)\]\s*=\s*(.+)", line)
        if m:
            shape = shape_of(m.group(2))
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            init = m.group(3).strip()
            if init.startswith("uniform"):
                args = dict((k, v) for k, v in re.findall(r"(\w+)\s*=\s*(" + _NUM + ")", init))
                value = uniform_values(count, int(args["seed"]), float(args["lo"]), float(args["hi"]))
            elif init.startswith("["):
                value = np.array([float(v) for v in re.findall(_NUM, init)], dtype=np.float64).astype(np.float32)
                if value.size != count:
                    raise ValueError(f"expected {count} values, got {value.size}")
            else:
                value = np.full(count, np.float32(float(init)), dtype=np.float32)
            add(McgNode(m.group(1), "const", shape, value=value.reshape(shape)))
            continue
        m = re.fullmatch(r"output\s+(.+)", line)
        if m:
            g.outputs.extend(t.strip() for t in m.group(1).split(","))
            continue
        m = re.fullmatch(r"(\w+)\s*=\s*(\w+)\s+(.+)", line)
        if m:
            name, op, rest = m.group(1), m.group(2), [t.strip() for t in m.group(3).split(",")]
            ops = [by_name[t] for t in rest]
            if op in UNARY:
                shape = ops[0].shape
            elif op in BINARY:
                shape = _broadcast(ops[0].shape, ops[1].shape)
            elif op in REDUCE:
                if len(ops[0].shape) < 1:
                    raise ValueError(f"{name}: {op} expects an operand of rank 1 or more")
                shape = tuple(ops[0].shape[:-1]) + (1,)
            elif op == "matmul":
                if len(ops[0].shape) != 2 or len(ops[1].shape) != 2 or ops[0].shape[1] != ops[1].shape[0]:
                    raise ValueError(f"{name}: bad matmul shapes {ops[0].shape} x {ops[1].shape}")
                shape = (ops[0].shape[0], ops[1].shape[1])
            else:
                raise ValueError(f"unknown op '{op}'")
            add(McgNode(name, op, shape, rest))
            continue
        raise ValueError(f"cannot read line: {raw!r}")
    for k in dims:
        if k not in declared:
            raise ValueError(f"the graph declares no dim '{k}'")
    if not g.outputs:
        raise ValueError("the graph declares no outputs")
    return g


def parse_mcg_file(path: str, dims: Optional[Dict[str, int]] = None) -> McgGraph:
    with open(path, "r") as f:
        return parse_mcg(f.read(), dims)


def make_random_inputs(graph: McgGraph, seed: int = 1, lo: float = -1.0, hi: float = 1.0) -> List[np.ndarray]:
    """Input k ~ uniform_values(n, seed + k, lo, hi) (src/runtime/host_tensor.cpp:7-14)."""
    out = []
    for k, name in enumerate(graph.inputs):
        shape = graph.node(name).shape
        n = int(np.prod(shape, dtype=np.int64)) if shape else 1
        out.append(uniform_values(n, seed + k, lo, hi).reshape(shape))
    return out


# -------------------------------------------------------------- evaluators


def _unary32(op: str, x: np.ndarray) -> np.ndarray:
    one = np.float32(1.0)
    if op == "neg":
        return -x
    if op == "exp":
        return np.exp(x)
    if op == "log":
        return np.log(x)
    if op == "sqrt":
        return np.sqrt(x)
    if op == "relu":
        return np.maximum(x, np.float32(0.0))
    if op == "sigmoid":
        return one / (one + np.exp(-x))
    if op == "tanh":
        return np.tanh(x)
    raise ValueError(op)


def _binary(op: str, a, b):
    if op == "add":
        return a + b
    if op == "sub":
        return a - b
    if op == "mul":
        return a * b
    if op == "div":
        return a / b
    raise ValueError(op)


def evaluate_f32(graph: McgGraph, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
    """Float32 execution with the CPU backend's semantics (see the module docstring)."""
    values: Dict[str, np.ndarray] = {}
    for name, a in zip(graph.inputs, inputs):
        values[name] = np.asarray(a, dtype=np.float32).reshape(graph.node(name).shape)
    with np.errstate(all="ignore"):
        for n in graph.nodes:
            if n.op == "input":
                continue
            if n.op == "const":
                values[n.name] = n.value
            elif n.op in UNARY:
                values[n.name] = _unary32(n.op, values[n.operands[0]]).astype(np.float32, copy=False)
            elif n.op in BINARY:
                r = _binary(n.op, values[n.operands[0]], values[n.operands[1]])
                values[n.name] = np.broadcast_to(r, n.shape).astype(np.float32, copy=False)
            elif n.op in REDUCE:
                values[n.name] = _reduce(n.op, values[n.operands[0]])
            else:
                values[n.name] = np.matmul(values[n.operands[0]], values[n.operands[1]]).astype(np.float32, copy=False)
    return [np.ascontiguousarray(values[o]).reshape(-1) for o in graph.outputs]


def _unary64(op: str, x: np.ndarray) -> np.ndarray:
    if op == "neg":
        return -x
    if op == "exp":
        return np.exp(x)
    if op == "log":
        return np.log(x)
    if op == "sqrt":
        return np.sqrt(x)
    if op == "relu":
        return np.where(x > 0.0, x, 0.0)
    if op == "sigmoid":
        return 1.0 / (1.0 + np.exp(-x))
    if op == "tanh":
        return np.tanh(x)
    raise ValueError(op)


def evaluate_f64(graph: McgGraph, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
    """tests/test_util.cpp:87-159: each node in double from float operands, rounded to float once."""
    values: Dict[str, np.ndarray] = {}
    for name, a in zip(graph.inputs, inputs):
        values[name] = np.asarray(a, dtype=np.float32).reshape(graph.node(name).shape)
    with np.errstate(all="ignore"):
        for n in graph.nodes:
            if n.op == "input":
                continue
            if n.op == "const":
                values[n.name] = n.value
                continue
            if n.op in REDUCE:
                values[n.name] = _reduce(n.op, values[n.operands[0]])
                continue
            ops = [values[o].astype(np.float64) for o in n.operands]
            if n.op in UNARY:
                r = _unary64(n.op, ops[0])
            elif n.op in BINARY:
                r = np.broadcast_to(_binary(n.op, ops[0], ops[1]), n.shape)
            else:
                r = np.matmul(ops[0], ops[1])
            values[n.name] = r.astype(np.float32)
    return [np.ascontiguousarray(values[o]).reshape(-1) for o in graph.outputs]


def sampled_matmul_f64(a: np.ndarray, b: np.ndarray, rows: np.ndarray, cols: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Exact dot products (float64) and sum|a*b| for sampled (row, col) pairs: the reference's check for
    shapes too large to evaluate in full (bench/bench_cuda.cpp:386-436)."""
    a64 = a[rows, :].astype(np.float64)
    b64 = b[:, cols].astype(np.float64).T
    return np.einsum("ik,ik->i", a64, b64), np.einsum("ik,ik->i", np.abs(a64), np.abs(b64))


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bfloat16, returned as float32 (what `__float2bfloat16_rn` does,
    src/cuda/matmul_tensor_core.cu:49)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return rounded.view(np.float32)


def round_to_f16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to IEEE half, returned as float32 (src/cuda/matmul_tensor_core.cu:56)."""
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def round_to_tf32(x: np.ndarray) -> np.ndarray:
    """Round to TF32 (10 explicit mantissa bits), nearest with ties away from zero as cvt.rna does
    (`__float_to_tf32`, src/cuda/matmul_tensor_core.cu:36); returned as float32."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (bits + np.uint32(0x1000)) & np.uint32(0xFFFFE000)
    return rounded.view(np.float32)
