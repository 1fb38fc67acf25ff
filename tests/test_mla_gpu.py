"""tcgen05 latent-attention kernel (DeepSeek MLA, absorbed form) and its rope/append companion vs fp32 PyTorch."""
import math

import pytest
import torch

from ksanallm_b200.ops import native, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _setup(q_lens, kv_lens, G, bt, layers=2, layer=1, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    B = len(q_lens)
    T = sum(q_lens)
    nblk_seq = [(k + bt - 1) // bt for k in kv_lens]
    nblocks = sum(nblk_seq) + 3
    cache = (torch.randn(nblocks, layers, bt, 576, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    perm = torch.randperm(nblocks, generator=g).tolist()
    table = torch.full((B, max(nblk_seq) + 1), -1, dtype=torch.int32)
    o = 0
    for s in range(B):
        for j in range(nblk_seq[s]):
            table[s, j] = perm[o]
            o += 1
    q = (torch.randn(T, G, 576, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device=DEV)
    return q, cache, cache[:, layer], table.to(DEV), cu, kvl


@pytest.mark.parametrize("G,bt,q_lens,kv_lens,nsplit", [
    (16, 16, [70, 9], [70, 200], 1),          # prefill from scratch + chunk with a cached prefix
    (128, 16, [3, 1], [35, 97], 1),           # all heads of one token fill a CTA
    (4, 64, [130], [130], 1),                 # blocks larger than a tile, several query tiles
    (16, 16, [1, 1, 1], [1, 333, 1024], 4),   # decode with split KV (one split range empty for the short rows)
    (128, 32, [1, 1], [700, 64], 3),
])
def test_mla_attention_matches_reference(G, bt, q_lens, kv_lens, nsplit):
    q, cache, layer, table, cu, kvl = _setup(q_lens, kv_lens, G, bt)
    T = q.shape[0]
    out = torch.zeros(T, G, 512, dtype=torch.bfloat16, device=DEV)
    scale = 1.0 / math.sqrt(192)
    ok = native.mla_attention(q, out, layer, layer.stride(0), bt, table, cu, kvl, len(q_lens), max(q_lens), G, scale, nsplit)
    assert ok
    torch.cuda.synchronize()
    native.check_err_flag(q.device)
    want = ref.mla_attention(q, layer, table, cu, kvl, scale)
    err = float((out.float() - want).abs().max())
    rel = float((out.float() - want).norm() / want.norm())
    assert rel < 2e-2 and err < 5e-2, (rel, err)


def test_mla_rope_append_matches_reference():
    T, G, nope, bt = 37, 16, 128, 16
    g = torch.Generator().manual_seed(3)
    q = torch.randn(T, G * (nope + 64), generator=g).to(torch.bfloat16).to(DEV)
    kv = torch.randn(T, 576, generator=g).to(torch.bfloat16).to(DEV)
    w = (1 + 0.1 * torch.randn(512, generator=g)).to(torch.bfloat16).to(DEV)
    pos = torch.randint(0, 500, (T,), generator=g).to(torch.int32).to(DEV)
    slots = torch.randperm(10 * bt, generator=g)[:T].to(torch.int32)
    slots[5] = -1
    slots = slots.to(DEV)
    cos_sin = ref.build_cos_sin_cache(64, 512, 10000.0, None, DEV)
    cache = torch.zeros(10, 3, bt, 576, dtype=torch.bfloat16, device=DEV)
    layer = cache[:, 2]
    qfull = torch.zeros(T, G, 576, dtype=torch.bfloat16, device=DEV)
    native.mla_rope_append(q, nope, kv, w, 1e-6, pos, slots, cos_sin, qfull, layer, layer.stride(0), bt, G)
    torch.cuda.synchronize()
    c = ref.norm(kv[:, :512].float(), w.float(), 1e-6)[0]
    kpe = ref.apply_rope(kv[:, 512:].float().reshape(T, 1, 64), pos, cos_sin, 64, neox=False).reshape(T, 64)
    qpe = ref.apply_rope(q.view(T, G, nope + 64)[..., nope:].float(), pos, cos_sin, 64, neox=False)
    assert float((qfull[..., 512:].float() - qpe).abs().max()) < 3e-2
    assert float(qfull[..., :512].abs().max()) == 0.0
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        row = layer[s // bt, s % bt].float()
        assert float((row[:512] - c[t]).abs().max()) < 4e-2
        assert float((row[512:] - kpe[t]).abs().max()) < 3e-2
    assert float(cache[:, :2].abs().max()) == 0.0          # other layers untouched


def test_deepseek_engine_gpu_uses_latent_kernel():
    """A small DeepSeek-V3-shaped model (latent 512 / rotary 64) through the engine on the GPU: greedy tokens equal
    the CPU engine's (which uses the plain matmul statement of the same attention)."""
    from ksanallm_b200.config import EngineConfig, ModelConfig
    from ksanallm_b200.models.weights import RandomSource, build_model
    from ksanallm_b200.runtime.engine import LLMEngine
    from ksanallm_b200.utils import native_engine as ne

    cfg = ModelConfig(model_type="deepseek_v3", hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=4, head_dim=192,
                      intermediate_size=512, vocab_size=512, rms_norm_eps=1e-6, rope_theta=10000.0, rope_neox=False,
                      max_position_embeddings=512, max_token_len=512, num_experts=8, num_experts_per_tok=2,
                      moe_intermediate_size=128, shared_expert_intermediate_size=128, num_shared_experts=1,
                      moe_scoring="sigmoid", routed_scaling_factor=2.5, n_group=4, topk_group=2, first_k_dense_replace=1,
                      q_lora_rank=128, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128)
    outs = {}
    calls = {"n": 0}
    real = native.mla_attention

    def counted(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    native.mla_attention = counted
    try:
        for dev, dt in (("cpu", torch.float32), ("cuda", torch.bfloat16)):
            model = build_model(cfg, RandomSource(seed=5, std=0.05), device=dev, dtype=dt)
            ec = EngineConfig()
            ec.batch_scheduler.max_token_len = 256
            ec.batch_scheduler.split_fuse_token_num = 48
            ec.global_.enable_cuda_graph = dev == "cuda"
            eng = LLMEngine(model, cfg, ec, num_blocks=64)
            s = ne.SamplingConfig()
            s.max_new_tokens, s.ignore_eos = 6, True
            g = torch.Generator().manual_seed(0)
            prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (61, 7, 130)]
            logits = []
            eng.step_hook = lambda plan, lg: logits.append(lg.float().cpu().clone())
            eng.generate(prompts, s)
            outs[dev] = logits
            if dev == "cuda":
                native.check_err_flag(torch.device("cuda"))
                # the latent-attention kernel reads cu_q in decode graphs too: every captured graph must own its step
                assert eng.runner.graphs and all(g[4].cu_q is not None for g in eng.runner.graphs.values())
                eng.runner.release_graphs()
    finally:
        native.mla_attention = real
    assert calls["n"] > 0
    a = next(x for x in outs["cpu"] if x.numel())             # first step that produced logits rows
    b = next(x for x in outs["cuda"] if x.numel())
    assert a.shape == b.shape
    assert float((a - b).norm() / a.norm()) < 0.06
