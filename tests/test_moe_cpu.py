"""MoE architectures end-to-end on CPU (Mixtral-style, Qwen2-MoE-style with shared expert) vs a dense restatement."""
import torch

from ksanallm_b200.config import EngineConfig, ModelConfig
from ksanallm_b200.models.moe import route_reference
from ksanallm_b200.models.weights import RandomSource, build_model
from ksanallm_b200.runtime.engine import LLMEngine
from ksanallm_b200.utils import native_engine as ne


def moe_cfg(kind):
    c = ModelConfig(model_type=kind, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
                    intermediate_size=256, vocab_size=1000, max_position_embeddings=256, max_token_len=256,
                    num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128)
    if kind == "qwen2_moe":
        c.qkv_bias, c.shared_expert_intermediate_size, c.shared_expert_gate, c.norm_topk_prob = True, 256, True, False
    return c


def test_moe_models_generate():
    for kind in ("mixtral", "qwen2_moe"):
        cfg = moe_cfg(kind)
        src = RandomSource(seed=5, std=0.05)
        model = build_model(cfg, src, device="cpu", dtype=torch.float32)
        assert all(l.moe is not None for l in model.layers)
        ec = EngineConfig()
        ec.batch_scheduler.max_token_len = 128
        eng = LLMEngine(model, cfg, ec, num_blocks=64)
        s = ne.SamplingConfig()
        s.max_new_tokens, s.ignore_eos = 4, True
        reqs = eng.generate([[1, 2, 3, 4, 5], [7, 8, 9]], s)
        assert all(len(r.outputs[0].tokens) == 4 for r in reqs)
        # batch composition must not change results: rerun the second prompt alone
        eng2 = LLMEngine(build_model(cfg, src, device="cpu", dtype=torch.float32), cfg, ec, num_blocks=64)
        alone = eng2.generate([[7, 8, 9]], s)[0]
        assert alone.outputs[0].tokens == reqs[1].outputs[0].tokens


def test_route_reference_group_limited():
    cfg = ModelConfig(num_experts=16, num_experts_per_tok=4, moe_scoring="sigmoid", n_group=4, topk_group=2,
                      routed_scaling_factor=2.5)
    logits = torch.randn(9, 16)
    ids, w = route_reference(logits, cfg, torch.zeros(16))
    groups = ids // 4
    assert all(len(set(g.tolist())) <= 2 for g in groups)
    assert torch.allclose(w.sum(-1), torch.full((9,), 2.5), atol=1e-5)


def test_expert_parallel_partials_sum_to_full():
    """Expert parallelism over a 2-rank tensor-parallel group: each rank holds whole experts and the
    tensor-parallel slice of the shared expert; the sum of the ranks' block outputs (the all-reduce) equals
    the single-rank block."""
    from types import SimpleNamespace
    from ksanallm_b200.models.moe import load_moe, moe_forward
    for kind in ("mixtral", "qwen2_moe"):
        cfg = moe_cfg(kind)
        src = RandomSource(seed=9, std=0.05)
        stub = SimpleNamespace(cfg=cfg, tp_size=1, comm=None)
        x = torch.randn(11, cfg.hidden_size)
        zero = torch.zeros(11, cfg.hidden_size)
        full = moe_forward(stub, load_moe(cfg, src, "model.layers.0.", 0, 1, "cpu", torch.float32, None), x, zero)
        parts = []
        for r in range(2):
            mw = load_moe(cfg, src, "model.layers.0.", r, 2, "cpu", torch.float32, None, ep_rank=r, ep_size=2)
            assert (mw.expert_lo, mw.expert_hi) == (4 * r, 4 * r + 4) and mw.inter == cfg.moe_intermediate_size
            parts.append(moe_forward(stub, mw, x, zero))
        assert torch.allclose(parts[0] + parts[1], full, atol=1e-5, rtol=1e-4)
