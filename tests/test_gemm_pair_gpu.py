"""CTA-pair (tcgen05 cta_group::2) GEMM against fp32 PyTorch references."""
import pytest
import torch

from ksanallm_b200.ops import native, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (300, 264, 192), (1024, 512, 1024), (2047, 4104, 4096),
                                   (4096, 10240, 8192)])
def test_pair_bf16(M, N, K):
    torch.manual_seed(0)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    native.gemm_pair(0, x, None, w, None, out, bias, res)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    assert rel_err(out, ref.gemm(x, w, bias, res, out_dtype=torch.float32)) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (300, 1000, 1024), (1000, 7168, 3584), (4096, 10240, 8192),
                                   (2500, 57344, 1024)])
def test_pair_fp8(M, N, K):
    torch.manual_seed(2)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.float32) * 0.05
    wq, ws = ref.quant_weight_fp8_block(w)
    xq, xs = native.quant_fp8(x)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    native.gemm_pair(1, xq, xs, wq, ws, out, None, res)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    assert rel_err(out, ref.gemm_fp8(xq, xs, wq, ws, None, res, out_dtype=torch.float32)) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (300, 264, 200), (1024, 512, 1024), (2047, 4104, 4096),
                                   (4096, 10240, 8192)])
def test_tall_bf16(M, N, K):
    """256 x 256 tiles per CTA: two 128-row accumulators over one weight tile, ragged M / N / K."""
    torch.manual_seed(1)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        native.gemm_bf16_tall(x, w, out, bias, res)
    torch.cuda.synchronize()
    native.check_err_flag(DEV)
    assert rel_err(out, ref.gemm(x, w, bias, res, out_dtype=torch.float32)) < 1e-2
    of = torch.empty(M, N, device=DEV, dtype=torch.float32)
    native.gemm_bf16_tall(x, w, None, out_f32=of)
    torch.cuda.synchronize()
    assert rel_err(of, ref.gemm(x, w, out_dtype=torch.float32)) < 2e-3
