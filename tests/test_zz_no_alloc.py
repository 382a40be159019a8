"""hb200_nvfp4_gemv_bf16in_tc_builtin_scratch: the tensor-core GEMV on the library's own scratch array.

Called through the C ABI and compared with hb200_nvfp4_gemv_bf16in_tc (caller workspace) on the same inputs,
twice in a row; device memory in use must not move across the calls.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from helion_b200 import _lib
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(n, k, batch, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(batch, k, generator=g).to(torch.bfloat16)
    packed, scales, gs = O.nvfp4_quantize(w)
    return packed.to(DEV), scales.to(DEV).view(torch.uint8), float(gs), x.to(DEV)


def _with_workspace(lib, w, x, s, out, n, k, batch, alpha, ws):
    ptrs = (ctypes.c_void_p * 1)(out.data_ptr())
    return lib.hb200_nvfp4_gemv_bf16in_tc(w.data_ptr(), x.data_ptr(), s.data_ptr(), ptrs, 1, n, k, batch, n, 0, alpha,
                                          ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)


def _builtin(lib, w, x, s, out, n, k, batch, alpha):
    return lib.hb200_nvfp4_gemv_bf16in_tc_builtin_scratch(w.data_ptr(), x.data_ptr(), s.data_ptr(),
                                                          None if out is None else out.data_ptr(), n, k,
                                                          batch, alpha, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("n,k,batch", [(8192, 8192, 1), (4096, 4096, 8), (1000, 2080, 3)])
def test_matches_the_workspace_entry_point_twice_in_a_row(n, k, batch):
    lib = _lib.load()
    w, s, alpha, x = _inputs(n, k, batch, seed=n + batch)
    need = lib.hb200_nvfp4_gemv_tc_workspace_bytes(n, k, batch, 4)
    assert 0 < need <= 8 << 20
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    want = torch.empty(batch, n, dtype=torch.bfloat16, device=DEV)
    assert _with_workspace(lib, w, x, s, want, n, k, batch, alpha, ws) == 0
    # the first call on the device does the one-time set-up; take the memory reading after it
    got = [torch.full((batch, n), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    warm = torch.empty_like(want)
    assert _builtin(lib, w, x, s, warm, n, k, batch, alpha) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    allocated_before = torch.cuda.memory_allocated()
    for out in got:
        assert _builtin(lib, w, x, s, out, n, k, batch, alpha) == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == allocated_before
    assert torch.cuda.mem_get_info()[0] == free_before
    assert lib.hb200_device_status(1) == 0
    for out in (warm, *got):
        assert torch.equal(out, want)


def test_shape_beyond_the_builtin_scratch_is_refused():
    lib = _lib.load()
    n, k, batch = 2048, 4096, 16  # 16 rows x 4 terms = 64 columns: the partial sums alone need 9.7 MB
    w, s, alpha, x = _inputs(n, k, batch, seed=1)
    out = torch.full((batch, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    rc = _builtin(lib, w, x, s, out, n, k, batch, alpha)
    assert rc == _lib.HB200_ERR_SCRATCH_LIMIT
    assert b"8 MiB" in lib.hb200_error_string(rc)
    torch.cuda.synchronize()
    assert torch.isnan(out).all()  # nothing ran
    assert _builtin(lib, w, x, s, None, n, k, batch, alpha) == _lib.HB200_ERR_INVALID_ARGUMENT
