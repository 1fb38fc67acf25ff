"""The entry point that allocates nothing (ksana_gemm_smallm_noalloc, see csrc/kernels/ksana_noalloc.h).

Some hosts of the kernel library may not allocate device memory when they call it - a serving loop that
handed out all of its memory up front, or a plugin running where cudaMalloc is forbidden. For them the
skinny GEMM has a variant whose split-K scratch is a fixed array inside the library. This test calls that
variant through its exported C symbol, twice in a row (the scratch is shared and keeps the previous call's
contents), and checks the result against the regular entry point, which takes caller-provided scratch.
The file sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

from ksanallm_b200.ops import native, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _noalloc_fn():
    lib = native.lib()
    fn = lib.ksana_gemm_smallm_noalloc
    vp, i32 = C.c_void_p, C.c_int
    fn.argtypes = [i32, vp, i32, vp, i32, vp, i32, vp, vp, i32, vp, vp, i32, i32, i32, i32, vp, vp]
    fn.restype = C.c_int
    lib.ksana_noalloc_last_error.restype = C.c_char_p
    return lib, fn


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


@pytest.mark.parametrize("kind", ["bf16", "fp8"])
@pytest.mark.parametrize("M,N,K", [(8, 8192, 8192), (3, 1280, 4096), (16, 4096, 14336)])
def test_noalloc_matches_regular_entry_point(kind, M, N, K):
    lib, fn = _noalloc_fn()
    torch.manual_seed(21)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    err = native.err_flag(DEV)
    st = torch.cuda.current_stream().cuda_stream
    if kind == "bf16":
        w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
        want = native.gemm_bf16(x, w, bias=bias, residual=res, splits=-1)
        oracle = ref.gemm(x, w, bias, res, out_dtype=torch.float32)
        args = (0, x.data_ptr(), x.stride(0), None, 0, w.data_ptr(), w.stride(0), None)
    else:
        wq, ws = ref.quant_weight_fp8_block(torch.randn(N, K, device=DEV) * 0.05)
        xq, xs = native.quant_fp8(x)
        want = native.gemm_fp8(xq, xs, wq, ws, bias=bias, residual=res, splits=-1)
        oracle = ref.gemm_fp8(xq, xs, wq, ws, bias, res, out_dtype=torch.float32)
        args = (1, xq.data_ptr(), xq.stride(0), xs.data_ptr(), xs.stride(0), wq.data_ptr(), wq.stride(0), ws.data_ptr())
    outs = [torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    free_seen = []
    for out in outs:                         # two calls in a row share the built-in scratch
        torch.cuda.synchronize()
        held = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(*args, out.data_ptr(), out.stride(0), bias.data_ptr(), res.data_ptr(), res.stride(0), M, N, K,
                err.data_ptr(), st)
        assert rc == 0, lib.ksana_noalloc_last_error().decode()
        torch.cuda.synchronize()
        free_seen.append((free_before, torch.cuda.mem_get_info()[0]))
        assert torch.cuda.memory_allocated() == held       # nothing came from torch's allocator ...
    # ... and the driver's own count of free device memory did not move across the second call either (a cudaMalloc
    # inside the library would show there; the first call on a device may load the kernel image)
    assert free_seen[1][0] == free_seen[1][1], free_seen
    native.check_err_flag(DEV)
    for out in outs:
        assert rel_err(out, want) < 1e-2, rel_err(out, want)
        assert rel_err(out, oracle) < 1e-2
    assert torch.equal(outs[0], outs[1])


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    lib, fn = _noalloc_fn()
    x = torch.zeros(128, 256, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(8, 256, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros(8, 8, device=DEV, dtype=torch.bfloat16)
    st = torch.cuda.current_stream().cuda_stream
    # 200 rows: above the 128-row limit
    rc = fn(0, x.data_ptr(), 256, None, 0, w.data_ptr(), 256, None, out.data_ptr(), 8, None, None, 0, 200, 8, 256, None, st)
    assert rc == -30 and b"exceed" in lib.ksana_noalloc_last_error()
    # 128 rows x 20000 columns needs more partial-tile scratch than the library carries
    rc = fn(0, x.data_ptr(), 256, None, 0, w.data_ptr(), 256, None, out.data_ptr(), 8, None, None, 0, 128, 20000, 256, None, st)
    assert rc == -30 and b"scratch" in lib.ksana_noalloc_last_error()
    # a kind the entry point does not serve is refused before anything is launched
    rc = fn(7, x.data_ptr(), 256, None, 0, w.data_ptr(), 256, None, out.data_ptr(), 8, None, None, 0, 8, 8, 256, None, st)
    assert rc == -32 and b"kind 7" in lib.ksana_noalloc_last_error()
    torch.cuda.synchronize()
