"""ctypes binding of the minicompiler-b200 C ABI (include/minicompiler_b200.h).

The class and method names follow the C entry points one to one, so a test written against
this module reads like the reference's own driver code (bench/torch_compare.py:187-272):
compile -> upload -> enqueue (on the caller's stream) -> download.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Iterable, Optional, Sequence

import numpy as np

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "libminicompiler_b200.so"


class McError(RuntimeError):
    """A failing mc_* / mcb_* call; the message is the library's own."""


_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """The loaded shared library. Fails loudly when it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise McError(
            f"{_LIB_PATH} is missing: build it with `python -m minicompiler_b200.build` "
            "(or __graft_entry__.build()). There is no Python or CPU fallback."
        )
    L = C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)
    vp, cp, i32, i64, f64 = C.c_void_p, C.c_char_p, C.c_int, C.c_longlong, C.c_double
    fpp = C.POINTER(C.POINTER(C.c_float))
    sigs = {
        "mc_compile": (vp, [cp, cp, cp, cp, cp, i32]),
        "mc_compile_ex": (vp, [cp, cp, cp, cp, cp, cp, i32]),
        "mc_num_inputs": (i32, [vp]),
        "mc_num_outputs": (i32, [vp]),
        "mc_output_elements": (i64, [vp, i32]),
        "mc_input_elements": (i64, [vp, i32]),
        "mc_run": (i32, [vp, fpp, fpp]),
        "mc_upload": (i32, [vp, fpp]),
        "mc_enqueue": (i32, [vp, vp]),
        "mc_download": (i32, [vp, fpp]),
        "mc_synchronize": (i32, [vp]),
        "mc_kernel_launches": (i32, [vp]),
        "mc_matmul_kernels": (i32, [vp, cp, i32]),
        "mc_gpu_sm_clock_mhz": (f64, []),
        "mc_gpu_device_json": (i32, [C.POINTER(C.c_double), i32, cp, i32]),
        "mc_release": (None, [vp]),
        "mc_last_error": (cp, []),
        "mc_constants_region": (i32, [vp, C.POINTER(vp), C.POINTER(C.c_size_t)]),
        "mc_refresh_constants": (i32, [vp]),
        "mc_status_word_ptr": (i32, [vp, C.POINTER(vp)]),
        "mc_row_slices": (i32, [vp]),
        "mc_replicate_constants": (i32, [vp, vp, i32]),
        "mc_gather_output": (i32, [vp, i32, vp, vp]),
        "mcd_nccl_available": (i32, []),
        "mcd_nccl_unique_id": (i32, [cp]),
        "mcd_nccl_init": (i32, [C.POINTER(vp), i32, i32, cp, i32, f64]),
        "mcd_nccl_broadcast": (i32, [vp, vp, C.c_size_t, i32, vp]),
        "mcd_nccl_all_gather": (i32, [vp, vp, vp, C.c_size_t, vp]),
        "mcd_nccl_wait": (i32, [vp, vp]),
        "mcd_nccl_abort": (i32, [vp]),
        "mcd_nccl_destroy": (i32, [vp]),
        "mcd_nccl_install_fake": (i32, [cp, i32, i32]),
        "mcd_nccl_remove_fake": (i32, []),
        "mcd_nccl_fake_aborts": (i32, []),
        "mcd_last_error": (cp, []),
        "mcb_in_place_pointers_ok": (i32, [C.POINTER(vp), i32, i32]),
        "mcd_copy_h2d": (i32, [vp, vp, C.c_size_t, vp]),
        "mcd_copy_d2h": (i32, [vp, vp, C.c_size_t, vp]),
        "mcd_copy_d2d": (i32, [vp, vp, C.c_size_t, vp]),
        "mcd_device_synchronize": (i32, []),
        "mcd_event_create": (i32, [C.POINTER(vp)]),
        "mcd_event_destroy": (i32, [vp]),
        "mcd_event_record_external": (i32, [vp, vp]),
        "mcd_event_elapsed_ms": (i32, [vp, vp, C.POINTER(C.c_float)]),
        "mcd_range_push": (i32, [cp]),
        "mcd_range_pop": (i32, []),
        "mcd_jit_cache_stats": (i32, [C.POINTER(i64), C.POINTER(i64)]),
        "mcd_per_device_once_probe": (i32, [C.POINTER(i32), i32, C.POINTER(i32)]),
        "mc_input_device_ptr": (i32, [vp, i32, C.POINTER(vp), C.POINTER(C.c_size_t)]),
        "mc_output_device_ptr": (i32, [vp, i32, C.POINTER(vp), C.POINTER(C.c_size_t)]),
        "mc_intermediate_bytes": (i64, [vp]),
        "mc_arena_bytes": (i64, [vp]),
        "mc_jit_compile_ms": (f64, [vp]),
        "mc_kernel_sources": (i32, [vp, cp, i32]),
        "mc_shard_dims": (i32, [cp, cp, cp, i32, i32, cp, i32, C.POINTER(i64), C.POINTER(i64)]),
        "mcb_graph_open": (vp, [cp, cp, cp, cp, cp, i32]),
        "mcb_graph_close": (None, [vp]),
        "mcb_graph_print": (i32, [vp, cp, i32]),
        "mcb_graph_stats_json": (i32, [vp, cp, i32]),
        "mcb_graph_plan_json": (i32, [vp, i32, cp, i32]),
        "mcb_graph_fusion_groups": (i32, [vp, cp, i32]),
        "mcb_graph_emit_cuda": (i32, [vp, cp, cp, i32]),
        "mcb_graph_launch_plan": (i32, [vp, cp, i32, cp, i32]),
        "mcb_graph_plan_sources": (i32, [vp, cp, i32, cp, i32]),
        "mcb_graph_num_nodes": (i32, [vp]),
        "mcb_graph_row_slicing": (i32, [vp, i64, cp, i32]),
        "mcb_graph_constant": (i64, [vp, cp, C.POINTER(C.c_float), i64]),
        "mcb_graph_check_kernels": (i32, [vp, cp, i32]),
        "mcb_uniform_values": (None, [C.POINTER(C.c_float), i64, C.c_ulonglong, C.c_float, C.c_float]),
        "mcb_split_k_splits": (i32, [i32, i32, i32, i32, i32]),
        "mcb_tensor_core_splits": (i32, [i32, i32, i32, i32, i32]),
        "mcb_balanced_fp32_splits": (i32, [i32, i32, i32, i32]),
        "mcb_tensor_core_tile_n": (i32, [i32, i32, i32, i32, i32]),
        "mcb_resolve_matmul_kernel": (cp, [cp, i32, i32, i32, i32]),
        "mcd_launch_count": (C.c_ulonglong, []),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def _last_error() -> str:
    msg = lib().mc_last_error()
    return msg.decode() if msg else ""


def _enc(s: Optional[str]) -> Optional[bytes]:
    return None if s is None else s.encode()


def graph_path(name: str) -> str:
    """Path of a graph shipped with the package, e.g. graph_path('c2_gelu_chain')."""
    p = _PKG / "graphs" / (name if name.endswith(".mcg") else name + ".mcg")
    if not p.exists():
        raise FileNotFoundError(p)
    return str(p)


def _dims_str(dims) -> str:
    if dims is None:
        return ""
    if isinstance(dims, str):
        return dims
    return ",".join(f"{k}={int(v)}" for k, v in dims.items())


def _opts_str(options) -> str:
    if options is None:
        return ""
    if isinstance(options, str):
        return options
    return ",".join(f"{k}={v}" for k, v in options.items())


def _float_ptr_array(arrays: Sequence[np.ndarray]):
    arr = (C.POINTER(C.c_float) * max(1, len(arrays)))()
    for i, a in enumerate(arrays):
        arr[i] = a.ctypes.data_as(C.POINTER(C.c_float))
    return arr


def _read_string(fn, *args) -> str:
    """Calls a `(…, char* out, int size) -> needed length` style function."""
    need = fn(*args, None, 0)
    if need < 0:
        raise McError(_last_error())
    buf = C.create_string_buffer(need + 1)
    fn(*args, buf, need + 1)
    return buf.value.decode()


class CompiledGraph:
    """A graph compiled for the GPU: the handle returned by mc_compile / mc_compile_ex."""

    def __init__(self, path: Optional[str] = None, *, text: Optional[str] = None, dims=None, passes: str = "default",
                 options=None, backend: str = "cuda"):
        L = lib()
        err = C.create_string_buffer(1 << 16)
        if options is None and text is None:
            self._h = L.mc_compile(_enc(path), _enc(_dims_str(dims)), _enc(passes), _enc(backend), err, len(err))
        else:
            if backend != "cuda":
                raise McError("mc_compile_ex compiles for the CUDA backend only")
            self._h = L.mc_compile_ex(_enc(path), _enc(text), _enc(_dims_str(dims)), _enc(passes), _enc(_opts_str(options)),
                                      err, len(err))
        if not self._h:
            raise McError(err.value.decode())
        self.num_inputs = L.mc_num_inputs(self._h)
        self.num_outputs = L.mc_num_outputs(self._h)
        self.input_elements = [L.mc_input_elements(self._h, k) for k in range(self.num_inputs)]
        self.output_elements = [L.mc_output_elements(self._h, k) for k in range(self.num_outputs)]

    # -- lifetime
    def release(self) -> None:
        if getattr(self, "_h", None):
            lib().mc_release(self._h)
            self._h = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()

    # -- running
    def _check_inputs(self, inputs: Sequence[np.ndarray]) -> list:
        if len(inputs) != self.num_inputs:
            raise McError(f"expected {self.num_inputs} inputs, got {len(inputs)}")
        out = []
        for k, a in enumerate(inputs):
            a = np.ascontiguousarray(a, dtype=np.float32)
            if a.size != self.input_elements[k]:
                raise McError(f"input {k} should have {self.input_elements[k]} elements, got {a.size}")
            out.append(a)
        return out

    def new_outputs(self) -> list:
        return [np.empty(n, dtype=np.float32) for n in self.output_elements]

    def run(self, inputs: Sequence[np.ndarray], outputs: Optional[Sequence[np.ndarray]] = None) -> list:
        """mc_run: host buffers in, host buffers out, copies included."""
        ins = self._check_inputs(inputs)
        outs = list(outputs) if outputs is not None else self.new_outputs()
        if lib().mc_run(self._h, _float_ptr_array(ins), _float_ptr_array(outs)) != 0:
            raise McError(_last_error())
        return outs

    def run_ptrs(self, in_ptrs: Sequence[int], out_ptrs: Sequence[int]) -> None:
        """mc_run on raw host addresses (e.g. pinned torch tensors' data_ptr())."""
        ins = (C.POINTER(C.c_float) * max(1, len(in_ptrs)))(*[C.cast(p, C.POINTER(C.c_float)) for p in in_ptrs])
        outs = (C.POINTER(C.c_float) * max(1, len(out_ptrs)))(*[C.cast(p, C.POINTER(C.c_float)) for p in out_ptrs])
        if lib().mc_run(self._h, ins, outs) != 0:
            raise McError(_last_error())

    def upload(self, inputs: Sequence[np.ndarray]) -> None:
        ins = self._check_inputs(inputs)
        if lib().mc_upload(self._h, _float_ptr_array(ins)) != 0:
            raise McError(_last_error())

    def enqueue(self, stream: int = 0) -> None:
        """mc_enqueue: launch on `stream` (a cudaStream_t as an int; 0 = the executable's own)."""
        if lib().mc_enqueue(self._h, C.c_void_p(stream or None)) != 0:
            raise McError(_last_error())

    def download(self, outputs: Optional[Sequence[np.ndarray]] = None) -> list:
        outs = list(outputs) if outputs is not None else self.new_outputs()
        if lib().mc_download(self._h, _float_ptr_array(outs)) != 0:
            raise McError(_last_error())
        return outs

    def synchronize(self) -> None:
        if lib().mc_synchronize(self._h) != 0:
            raise McError(_last_error())

    # -- introspection
    @property
    def kernel_launches(self) -> int:
        return lib().mc_kernel_launches(self._h)

    @property
    def matmul_kernels(self) -> list:
        buf = C.create_string_buffer(1 << 14)
        if lib().mc_matmul_kernels(self._h, buf, len(buf)) != 0:
            raise McError(_last_error())
        text = buf.value.decode()
        return text.split(",") if text else []

    @property
    def intermediate_bytes(self) -> int:
        return lib().mc_intermediate_bytes(self._h)

    @property
    def arena_bytes(self) -> int:
        return lib().mc_arena_bytes(self._h)

    @property
    def jit_compile_ms(self) -> float:
        return lib().mc_jit_compile_ms(self._h)

    @property
    def kernel_sources(self) -> str:
        return _read_string(lib().mc_kernel_sources, self._h)

    def constants_region(self):
        ptr, size = C.c_void_p(), C.c_size_t()
        if lib().mc_constants_region(self._h, C.byref(ptr), C.byref(size)) != 0:
            raise McError(_last_error())
        return (ptr.value or 0), size.value

    def refresh_constants(self) -> None:
        if lib().mc_refresh_constants(self._h) != 0:
            raise McError(_last_error())

    @property
    def row_slices(self) -> int:
        """Slices mc_run cuts a call on pinned host buffers into (0: not sliced)."""
        return lib().mc_row_slices(self._h)

    def replicate_constants(self, comm: "Communicator", root: int = 0) -> None:
        """mc_replicate_constants: rank `root`'s constants become every rank's (one NCCL broadcast)."""
        if lib().mc_replicate_constants(self._h, comm.handle, root) != 0:
            raise McError(_last_error())

    def gather_output(self, k: int, comm: "Communicator", device_dst: int) -> None:
        """mc_gather_output: all ranks' rows of output k, in rank order, into device memory at `device_dst`."""
        if lib().mc_gather_output(self._h, k, comm.handle, C.c_void_p(device_dst)) != 0:
            raise McError(_last_error())

    def status_word_ptr(self) -> int:
        """Device address of the status word (0 when no kernel of this graph can wait)."""
        ptr = C.c_void_p()
        if lib().mc_status_word_ptr(self._h, C.byref(ptr)) != 0:
            raise McError("not a GPU executable")
        return ptr.value or 0

    def input_device_ptr(self, k: int):
        ptr, n = C.c_void_p(), C.c_size_t()
        if lib().mc_input_device_ptr(self._h, k, C.byref(ptr), C.byref(n)) != 0:
            raise McError("no such input")
        return (ptr.value or 0), n.value

    def output_device_ptr(self, k: int):
        ptr, n = C.c_void_p(), C.c_size_t()
        if lib().mc_output_device_ptr(self._h, k, C.byref(ptr), C.byref(n)) != 0:
            raise McError("no such output")
        return (ptr.value or 0), n.value


class Communicator:
    """An NCCL communicator of the device layer (mcd_nccl_*): one rank per process, one GPU per rank.

    `unique_id()` is called on one rank and its 128 bytes are handed to the others by whatever means the
    launcher offers (a torch.distributed store, MPI, a file); every rank then constructs the communicator.
    Calls are bounded by `timeout_s`: a peer that never joins makes the call fail and aborts the communicator."""

    def __init__(self, world_size: int, rank: int, unique_id: bytes, device: int, timeout_s: float = 60.0):
        h = C.c_void_p()
        if lib().mcd_nccl_init(C.byref(h), world_size, rank, unique_id, device, timeout_s) != 0:
            raise McError(_device_error())
        self.handle, self.world_size, self.rank = h, world_size, rank

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        if lib().mcd_nccl_unique_id(buf) != 0:
            raise McError(_device_error())
        return buf.raw

    def broadcast(self, device_ptr: int, nbytes: int, root: int = 0, stream: int = 0) -> None:
        if lib().mcd_nccl_broadcast(self.handle, C.c_void_p(device_ptr), nbytes, root, C.c_void_p(stream or None)) != 0:
            raise McError(_device_error())

    def all_gather(self, send_ptr: int, recv_ptr: int, bytes_per_rank: int, stream: int = 0) -> None:
        if lib().mcd_nccl_all_gather(self.handle, C.c_void_p(send_ptr), C.c_void_p(recv_ptr), bytes_per_rank,
                                     C.c_void_p(stream or None)) != 0:
            raise McError(_device_error())

    def wait(self, stream: int = 0) -> None:
        if lib().mcd_nccl_wait(self.handle, C.c_void_p(stream or None)) != 0:
            raise McError(_device_error())

    def abort(self) -> None:
        lib().mcd_nccl_abort(self.handle)

    def destroy(self) -> None:
        if getattr(self, "handle", None):
            lib().mcd_nccl_destroy(self.handle)
            self.handle = None


def _device_error() -> str:
    msg = lib().mcd_last_error()
    return msg.decode() if msg else ""


def compile_graph(path: Optional[str] = None, **kw) -> CompiledGraph:
    return CompiledGraph(path, **kw)


class HostGraph:
    """A parsed and optimized graph, for host-only inspection (no GPU needed)."""

    def __init__(self, path: Optional[str] = None, *, text: Optional[str] = None, dims=None, passes: str = "default"):
        err = C.create_string_buffer(1 << 16)
        self._g = lib().mcb_graph_open(_enc(path), _enc(text), _enc(_dims_str(dims)), _enc(passes), err, len(err))
        if not self._g:
            raise McError(err.value.decode())

    def close(self) -> None:
        if getattr(self, "_g", None):
            lib().mcb_graph_close(self._g)
            self._g = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def num_nodes(self) -> int:
        return lib().mcb_graph_num_nodes(self._g)

    def print(self) -> str:
        return _read_string(lib().mcb_graph_print, self._g)

    def stats(self) -> dict:
        import json
        return json.loads(_read_string(lib().mcb_graph_stats_json, self._g))

    def plan(self, pool_outputs: bool = True) -> dict:
        import json
        return json.loads(_read_string(lib().mcb_graph_plan_json, self._g, 1 if pool_outputs else 0))

    def fusion_groups(self) -> list:
        text = _read_string(lib().mcb_graph_fusion_groups, self._g)
        return [line.split() for line in text.splitlines() if line]

    def emit_cuda(self, options=None) -> str:
        return _read_string(lib().mcb_graph_emit_cuda, self._g, _enc(_opts_str(options)))

    def launch_plan(self, options=None, sm_count: int = 148) -> str:
        return _read_string(lib().mcb_graph_launch_plan, self._g, _enc(_opts_str(options)), sm_count)

    def plan_sources(self, options=None, sm_count: int = 148) -> str:
        """The CUDA text the launch plan generates, step by step (no GPU needed)."""
        return _read_string(lib().mcb_graph_plan_sources, self._g, _enc(_opts_str(options)), sm_count)

    def row_slicing(self, slice_rows: int = 0) -> str:
        """Which values mc_run may cut by rows ("none" or "rows=N cut=a,b,..."), optionally with the graph at
        `slice_rows` rows printed after it."""
        return _read_string(lib().mcb_graph_row_slicing, self._g, slice_rows)

    def constant(self, name: str) -> np.ndarray:
        n = lib().mcb_graph_constant(self._g, name.encode(), None, 0)
        if n < 0:
            raise McError(f"no constant named '{name}'")
        out = np.empty(n, dtype=np.float32)
        lib().mcb_graph_constant(self._g, name.encode(), out.ctypes.data_as(C.POINTER(C.c_float)), n)
        return out

    def check_kernels(self, options=None, sm_count: int = 148) -> None:
        """NVRTC-compiles every generated kernel for sm_100a (works without a GPU)."""
        if lib().mcb_graph_check_kernels(self._g, _enc(_opts_str(options)), sm_count) != 0:
            raise McError(_last_error())


def uniform_values(count: int, seed: int, lo: float, hi: float) -> np.ndarray:
    out = np.empty(count, dtype=np.float32)
    lib().mcb_uniform_values(out.ctypes.data_as(C.POINTER(C.c_float)), count, seed, lo, hi)
    return out


def split_k_splits(m: int, n: int, k: int, sm_count: int, blocks_per_sm: int = 2) -> int:
    return lib().mcb_split_k_splits(m, n, k, sm_count, blocks_per_sm)


def tensor_core_splits(m: int, n: int, k: int, sm_count: int, elem_bytes: int = 2) -> int:
    return lib().mcb_tensor_core_splits(m, n, k, sm_count, elem_bytes)


def tensor_core_tile_n(m: int, n: int, k: int, sm_count: int, elem_bytes: int = 2) -> int:
    return lib().mcb_tensor_core_tile_n(m, n, k, sm_count, elem_bytes)


def resolve_matmul_kernel(name: str, m: int, n: int, k: int, sm_count: int) -> str:
    res = lib().mcb_resolve_matmul_kernel(name.encode(), m, n, k, sm_count)
    if res is None:
        raise McError(_last_error())
    return res.decode()


def shard_dims(path: str, dims, batch_dim: str, rank: int, world_size: int):
    """(dims string for this rank, first row, rows) or McError when the graph cannot be row-sharded."""
    out = C.create_string_buffer(4096)
    off, rows = C.c_longlong(), C.c_longlong()
    rc = lib().mc_shard_dims(path.encode(), _enc(_dims_str(dims)), batch_dim.encode(), rank, world_size, out, len(out),
                             C.byref(off), C.byref(rows))
    if rc != 0:
        raise McError(_last_error())
    return out.value.decode(), off.value, rows.value
