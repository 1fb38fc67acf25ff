"""4-bit weight-only linear layers on the GPU: streaming GEMV (small batches) and expand + tcgen05 GEMM (large)."""
import pytest
import torch

from ksanallm_b200.ops import native, reference as ref
from ksanallm_b200.ops.dispatch import LinearWeight, linear

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _layer(N, K, g, seed=0):
    gen = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=gen) * 0.05
    packed, scale, zs = ref.quant_w4(w, g)
    dense = ref.dequant_w4(packed, scale, zs)
    return packed.to(DEV), scale.to(DEV), zs.to(DEV), dense.to(DEV)


@pytest.mark.parametrize("M,N,K,g", [(1, 256, 512, 128), (3, 1000, 1024, 64), (8, 4096, 4096, 128), (13, 520, 2048, 32),
                                     (32, 1024, 1024, 128)])
def test_w4_gemv_matches_reference(M, N, K, g):
    packed, scale, zs, dense = _layer(N, K, g, seed=M)
    gen = torch.Generator().manual_seed(100 + M)
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16).to(DEV)
    bias = torch.randn(N, generator=gen).to(torch.bfloat16).to(DEV)
    res = torch.randn(M, N, generator=gen).to(torch.bfloat16).to(DEV)
    y = native.linear_w4(x, packed, scale, zs, bias=bias, residual=res)
    want = x.float() @ dense.t() + bias.float() + res.float()
    assert float((y.float() - want).abs().max()) < 0.06
    assert float((y.float() - want).norm() / want.norm()) < 1e-2
    y2 = native.linear_w4(x, packed, scale, zs)
    want2 = x.float() @ dense.t()
    assert float((y2.float() - want2).norm() / want2.norm()) < 1e-2


def test_w4_large_batch_expands_and_uses_the_gemm():
    packed, scale, zs, dense = _layer(1024, 2048, 128, seed=7)
    x = torch.randn(300, 2048, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    y = native.linear_w4(x, packed, scale, zs)
    want = x.float() @ dense.t()
    assert float((y.float() - want).norm() / want.norm()) < 1e-2
    # the expansion alone
    w = torch.empty(1024, 2048, dtype=torch.bfloat16, device=DEV)
    native._check(native.lib().ksana_w4_dequant(packed.data_ptr(), scale.data_ptr(), zs.data_ptr(), w.data_ptr(), 2048, 1024,
                                                2048, 128, native._st()), "ksana_w4_dequant")
    assert float((w.float() - dense).abs().max()) < 2e-3


def test_linear_dispatch_w4():
    W = LinearWeight(w=torch.randn(512, 1024, device=DEV) * 0.05).quantize_w4(128)
    assert W.w4a16 and W.in_features == 1024 and W.out_features == 512
    x = torch.randn(4, 1024, device=DEV, dtype=torch.bfloat16)
    y = linear(x, W)
    want = x.float() @ W.dense().t()
    assert float((y.float() - want).norm() / want.norm()) < 1e-2


def test_w4_model_through_the_engine_matches_cpu():
    """A small Llama with 4-bit weight-only projections: greedy decoding on the GPU (GEMV kernel for decode steps,
    expansion + tcgen05 GEMM for the prefill) follows the CPU engine running the same quantised weights."""
    from ksanallm_b200.config import EngineConfig, ModelConfig
    from ksanallm_b200.models.weights import RandomSource, build_model
    from ksanallm_b200.runtime.engine import LLMEngine
    from ksanallm_b200.utils import native_engine as ne
    cfg = ModelConfig(model_type="llama", hidden_size=512, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=1000, max_position_embeddings=256, max_token_len=256)
    outs = {}
    for dev, dt in (("cpu", torch.float32), ("cuda", torch.bfloat16)):
        model = build_model(cfg, RandomSource(seed=4, std=0.05), device=dev, dtype=dt, quant="w4a16:128")
        assert model.layers[0].qkv.w4a16 and model.layers[1].down.w4a16
        ec = EngineConfig()
        ec.batch_scheduler.max_token_len = 200
        ec.global_.enable_cuda_graph = dev == "cuda"
        eng = LLMEngine(model, cfg, ec, num_blocks=64)
        s = ne.SamplingConfig()
        s.max_new_tokens, s.ignore_eos = 5, True
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (50, 9)]
        logits = []
        eng.step_hook = lambda plan, lg: logits.append(lg.float().cpu().clone())
        eng.generate(prompts, s)
        outs[dev] = logits
        if dev == "cuda":
            native.check_err_flag(torch.device("cuda"))
            eng.runner.release_graphs()
    a = next(x for x in outs["cpu"] if x.numel())
    b = next(x for x in outs["cuda"] if x.numel())
    assert a.shape == b.shape and float((a - b).norm() / a.norm()) < 0.05
