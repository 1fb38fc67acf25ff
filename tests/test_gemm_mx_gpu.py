"""Hardware block-scaled FP8 GEMM (tcgen05 block_scale MMA, power-of-two scales) against the fp32 statement."""
import pytest
import torch

from ksanallm_b200.ops import native, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def _operands(M, N, K, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    # rows, weight blocks and K groups of very different magnitude: a scale applied to the wrong row, block
    # or K group shows up as a gross error
    x = torch.randn(M, K, generator=g) * torch.exp2(torch.randint(-6, 7, (M, 1), generator=g).float())
    x = x * torch.exp2(torch.randint(-3, 4, (1, K // 128), generator=g).float()).repeat_interleave(128, 1)
    w = torch.randn(N, K, generator=g) * 0.05
    nb, kb = (N + 127) // 128, K // 128
    blk = torch.exp2(torch.randint(-5, 6, (nb, kb), generator=g).float())
    w = w * blk.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)
    return x.to(DEV, torch.bfloat16), w.to(DEV)


@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 128, 256), (128, 128, 512, 128), (300, 1000, 640, 256),
                                      (300, 1000, 640, 128), (77, 264, 1024, 0), (1000, 7168, 3584, 0),
                                      (4096, 10240, 8192, 256), (2500, 57344, 1024, 0), (64, 8192, 8192, 0)])
def test_gemm_mxfp8(M, N, K, bn):
    x, w = _operands(M, N, K, seed=M + N + K)
    wq, ws = ref.quant_weight_fp8_block(w)
    assert ref.is_pow2(ws)
    xq, xs = native.quant_fp8(x)
    assert ref.is_pow2(xs[:, :M])
    xq_r, xs_r = ref.quant_fp8(x)
    assert torch.equal(xs[:, :M], xs_r) and torch.equal(xq.float(), xq_r.float())
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        y = native.gemm_mxfp8(xq, xs, wq, ws, torch.empty(M, N, device=DEV, dtype=torch.bfloat16), bias, res, bn=bn)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = ref.gemm_fp8(xq, xs, wq, ws, bias, res, out_dtype=torch.float32)
    assert rel_err(y, want) < 1e-2, rel_err(y, want)
    yf = torch.empty(M, N, device=DEV, dtype=torch.float32)
    native.gemm_mxfp8(xq, xs, wq, ws, None, out_f32=yf, bn=bn)
    assert rel_err(yf, ref.gemm_fp8(xq, xs, wq, ws, out_dtype=torch.float32)) < 2e-3


@pytest.mark.parametrize("M,N,K,bn,ranks", [(1024, 512, 512, 256, 4), (1000, 264, 256, 128, 3), (2048, 8192, 1024, 0, 8),
                                            (1024, 1000, 512, "tall", 4), (3000, 8192, 256, "tall", 8)])
def test_gemm_mxfp8_push_epilogue(M, N, K, bn, ranks):
    """Push mode: rows leave for the receive slot of the rank that reduces them (here every slot is local memory),
    64 contiguous bytes per row and store; bits must equal the plain epilogue's."""
    import ctypes as C
    x, w = _operands(M, N, K, seed=M + N + K + ranks)
    wq, ws = ref.quant_weight_fp8_block(w)
    xq, xs = native.quant_fp8(x)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    if bn == "tall":
        def gemm(*a, **kw):
            kw.pop("bn")
            return native.gemm_mxfp8_tall(*a, **kw)
    else:
        gemm = native.gemm_mxfp8
    plain = gemm(xq, xs, wq, ws, torch.empty(M, N, device=DEV, dtype=torch.bfloat16), bias, bn=bn)
    rows_per = (M + ranks - 1) // ranks
    slots = torch.full((ranks, rows_per, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    ptrs = (C.c_ulonglong * 8)(*([slots[r].data_ptr() for r in range(ranks)] + [0] * (8 - ranks)))
    gemm(xq, xs, wq, ws, bias=bias, bn=bn, push=ptrs, push_n=ranks, push_rows=rows_per, ldd=N)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    got = slots.reshape(ranks * rows_per, N)[:M]
    assert torch.equal(got, plain)
    assert torch.isnan(slots.reshape(ranks * rows_per, N)[M:].float()).all()      # nothing written past the last row
    if bn != "tall" and M <= 1024:
        # broadcast form (push_rows = 0): every rank's slot receives every row
        every = torch.full((ranks, M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        ptrs = (C.c_ulonglong * 8)(*([every[r].data_ptr() for r in range(ranks)] + [0] * (8 - ranks)))
        gemm(xq, xs, wq, ws, bias=bias, bn=bn, push=ptrs, push_n=ranks, push_rows=0, ldd=N)
        torch.cuda.synchronize()
        native.check_err_flag(DEV)
        for r in range(ranks):
            assert torch.equal(every[r], plain)


def test_gemm_fp8_exact_scales_still_served():
    """Weights whose scales are not powers of two (a checkpoint's own) stay on the exact-fp32-scale kernel."""
    from ksanallm_b200.ops.dispatch import LinearWeight, linear
    x, w = _operands(300, 1024, 1024, seed=3)
    wq, ws = ref.quant_weight_fp8_block(w, pow2=False)
    W = LinearWeight(wq=wq, ws=ws)
    assert not W.ue8m0
    y = linear(x, W)
    xq, xs = native.quant_fp8(x)
    assert rel_err(y, ref.gemm_fp8(xq, xs, wq, ws, out_dtype=torch.float32)) < 1e-2
    W2 = LinearWeight(w=w.to(torch.bfloat16)).quantize_fp8_block()
    assert W2.ue8m0
    y2 = linear(x, W2)
    assert rel_err(y2, ref.gemm_fp8(xq, xs, W2.wq, W2.ws, out_dtype=torch.float32)) < 1e-2


@pytest.mark.parametrize("M,N,K,splits", [(1, 512, 1024, 0), (8, 8192, 8192, 0), (16, 1280, 8192, 37), (17, 4096, 4096, 7),
                                          (64, 57344, 8192, -1), (64, 8192, 28672, -1), (128, 1000, 2048, 3),
                                          (100, 10240, 1024, -1), (32, 57344, 8192, 0), (3, 8192, 28672, 0),
                                          (8, 7168, 640, 1), (33, 8192, 8192, 0)])
def test_gemm_smallm_hw_scaled(M, N, K, splits):
    """Skinny stream-K kernel with tensor-core-applied scales (kind 2), through the public routing."""
    x, w = _operands(M, N, K, seed=M * 7 + N + K)
    wq, ws = ref.quant_weight_fp8_block(w)
    xq, xs = native.quant_fp8(x)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):   # twice: the tile counters must come back to zero
        y = native.gemm_fp8(xq, xs, wq, ws, bias=bias, residual=res, splits=splits, hw_scale=True)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = ref.gemm_fp8(xq, xs, wq, ws, bias, res, out_dtype=torch.float32)
    assert rel_err(y, want) < 1e-2, rel_err(y, want)


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (256, 256, 1024), (300, 1000, 640), (1000, 7168, 3584),
                                   (4096, 10240, 8192), (2500, 57344, 1024)])
def test_gemm_mxfp8_pair(M, N, K):
    """CTA-pair variant (cta_group::2): both CTAs' rows and both weight halves carry their own scales."""
    x, w = _operands(M, N, K, seed=M + N + K + 1)
    wq, ws = ref.quant_weight_fp8_block(w)
    xq, xs = native.quant_fp8(x)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        y = native.gemm_mxfp8_pair(xq, xs, wq, ws, torch.empty(M, N, device=DEV, dtype=torch.bfloat16), bias, res)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = ref.gemm_fp8(xq, xs, wq, ws, bias, res, out_dtype=torch.float32)
    assert rel_err(y, want) < 1e-2, rel_err(y, want)
    yf = torch.empty(M, N, device=DEV, dtype=torch.float32)
    native.gemm_mxfp8_pair(xq, xs, wq, ws, None, out_f32=yf)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    assert rel_err(yf, ref.gemm_fp8(xq, xs, wq, ws, out_dtype=torch.float32)) < 2e-3


@pytest.mark.parametrize("M,N,K", [(256, 224, 128), (256, 448, 1024), (300, 1000, 640), (1000, 7168, 3584),
                                   (4096, 10240, 8192), (2500, 57344, 1024), (77, 264, 1024)])
def test_gemm_mxfp8_tall(M, N, K):
    """256 x 224 tiles: 224-wide tiles straddle the 128 x 128 weight blocks, so every 32-column run picks its block."""
    x, w = _operands(M, N, K, seed=M + N + K + 2)
    wq, ws = ref.quant_weight_fp8_block(w)
    xq, xs = native.quant_fp8(x)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        y = native.gemm_mxfp8_tall(xq, xs, wq, ws, torch.empty(M, N, device=DEV, dtype=torch.bfloat16), bias, res)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    want = ref.gemm_fp8(xq, xs, wq, ws, bias, res, out_dtype=torch.float32)
    assert rel_err(y, want) < 1e-2, rel_err(y, want)
    yf = torch.empty(M, N, device=DEV, dtype=torch.float32)
    native.gemm_mxfp8_tall(xq, xs, wq, ws, None, out_f32=yf)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    assert rel_err(yf, ref.gemm_fp8(xq, xs, wq, ws, out_dtype=torch.float32)) < 2e-3
