"""The allocation-free split-K matmul, checked against the regular entry point.

Some users of this library run where device allocation is off the table: their process handed all
of HBM to its own pool when it started, or they sit on a latency-critical path and cannot pay for
the device-wide synchronisation that cudaMalloc / cudaFree bring. For them the FP32 split-K matmul
exists a second time, `mcd_gemm_f32_split_no_alloc`, which keeps its partial sums in an array that is
part of the library (16 MiB per GPU) instead of a caller-provided workspace.

This file is named so that pytest collects it last: a run that stops at the first failure has
then already exercised every other test. It passes alone in a fresh process and after the others.
"""

import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call_no_alloc(lib, ta, tb, tc, m, n, k, splits, stream):
    lib.mcd_gemm_f32_split_no_alloc.restype = C.c_int
    lib.mcd_gemm_f32_split_no_alloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    return lib.mcd_gemm_f32_split_no_alloc(ta.data_ptr(), tb.data_ptr(), tc.data_ptr(), m, n, k, splits, stream)


def test_no_alloc_split_k_equals_the_workspace_path_twice_in_a_row(mc, oracle):
    import torch

    from test_gpu_parity import _device_gemm

    lib = mc.lib()
    lib.mcd_last_error.restype = C.c_char_p
    stream = torch.cuda.current_stream().cuda_stream
    dev = torch.device("cuda:0")
    # two different problems back to back: the second one finds the first one's partial sums in the scratch
    for (m, k, n, splits), seed in [((128, 2048, 512, 7), 1), ((129, 260, 132, 3), 5), ((128, 2048, 512, 7), 9)]:
        a = oracle.uniform_values(m * k, seed, -1, 1).reshape(m, k)
        b = oracle.uniform_values(k * n, seed + 1, -1, 1).reshape(k, n)
        want = _device_gemm(mc, 0, a, b, splits)  # mcd_gemm with a torch-allocated workspace
        ta, tb = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
        for attempt in range(2):
            tc = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
            rc = _call_no_alloc(lib, ta, tb, tc, m, n, k, splits, stream)
            assert rc == 0, lib.mcd_last_error().decode()
            torch.cuda.synchronize()
            got = tc.cpu().numpy()
            # same kernels, same slice order: the tolerance of the matmul tests is met with zero to spare
            assert np.array_equal(got, want), (m, k, n, splits, attempt)


def test_no_alloc_rejects_what_does_not_fit(mc):
    import torch

    lib = mc.lib()
    lib.mcd_last_error.restype = C.c_char_p
    dev = torch.device("cuda:0")
    m, n, k, splits = 1024, 2048, 512, 4  # 4 slices * 8 MiB of partial sums > 16 MiB
    ta = torch.zeros((m, k), dtype=torch.float32, device=dev)
    tb = torch.zeros((k, n), dtype=torch.float32, device=dev)
    tc = torch.zeros((m, n), dtype=torch.float32, device=dev)
    rc = _call_no_alloc(lib, ta, tb, tc, m, n, k, splits, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    message = lib.mcd_last_error().decode()
    assert "bytes of scratch" in message and "16777216" in message
    # one slice needs no scratch at all and is accepted at any size
    assert _call_no_alloc(lib, ta, tb, tc, m, n, k, 1, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
