"""FP8 checkpoints (float8_e4m3fn weights with 128 x 128 block scales in ``weight_scale_inv``, or one per-tensor
``weight_scale``): the loader hands the checkpoint's own values and scales to the GEMMs - sliced for tensor
parallelism and packed (QKV, gate|up, expert stacks) on block boundaries - instead of expanding and re-quantising."""
import pytest
import torch

from ksanallm_b200.config import ModelConfig
from ksanallm_b200.models.common import StepInput
from ksanallm_b200.models.weights import DictSource, Fp8Pair, build_model

FP8 = torch.float8_e4m3fn


def _quant_blocks(w: torch.Tensor, gen):
    """A checkpoint-style quantisation: arbitrary (not power-of-two) block scales."""
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    pad = torch.zeros(nb * 128, kb * 128)
    pad[:N, :K] = w
    blocks = pad.view(nb, 128, kb, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-6)
    s = amax / 448.0 * (1.0 + 0.3 * torch.rand(nb, kb, generator=gen))
    q = (blocks / s[:, None, :, None]).view(nb * 128, kb * 128)[:N, :K].to(FP8)
    return q, s


def _step(tokens):
    T = len(tokens)
    ar = torch.arange(T, dtype=torch.int32)
    return StepInput(torch.tensor(tokens, dtype=torch.int32), ar, ar.clone(), torch.tensor([0, T], dtype=torch.int32),
                     torch.tensor([T], dtype=torch.int32), torch.arange(8, dtype=torch.int32).view(1, 8),
                     num_multi=1, num_single=0, num_tokens=T, num_multi_tokens=T, max_q_len=T, max_kv_len=T)


def _llama_cfg():
    return ModelConfig(model_type="llama", hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                       intermediate_size=512, vocab_size=300, rms_norm_eps=1e-5, max_position_embeddings=128, max_token_len=128)


def _llama_checkpoint(cfg, gen, per_tensor=False):
    H, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    sd, dense = {}, {}
    rnd = lambda *s: torch.randn(*s, generator=gen) * 0.05
    for name, shape in [("model.embed_tokens.weight", (cfg.vocab_size, H)), ("lm_head.weight", (cfg.vocab_size, H))]:
        sd[name] = dense[name] = rnd(*shape)
    sd["model.norm.weight"] = dense["model.norm.weight"] = torch.ones(H)
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        for n in ("input_layernorm.weight", "post_attention_layernorm.weight"):
            sd[p + n] = dense[p + n] = 1 + rnd(H)
        for n, shape in [("self_attn.q_proj", (cfg.num_heads * D, H)), ("self_attn.k_proj", (cfg.num_kv_heads * D, H)),
                         ("self_attn.v_proj", (cfg.num_kv_heads * D, H)), ("self_attn.o_proj", (H, cfg.num_heads * D)),
                         ("mlp.gate_proj", (I, H)), ("mlp.up_proj", (I, H)), ("mlp.down_proj", (H, I))]:
            w = rnd(*shape)
            if per_tensor:
                s = w.abs().max() / 448.0 * 1.17
                q = (w / s).to(FP8)
                sd[p + n + ".weight"], sd[p + n + ".weight_scale"] = q, s.reshape(())
                dense[p + n + ".weight"] = q.float() * s
            else:
                q, s = _quant_blocks(w, gen)
                sd[p + n + ".weight"], sd[p + n + ".weight_scale_inv"] = q, s
                dense[p + n + ".weight"] = Fp8Pair(q, s).dense()
    return sd, dense


@pytest.mark.parametrize("per_tensor", [False, True])
def test_dense_model_keeps_the_checkpoint_quantisation(per_tensor):
    gen = torch.Generator().manual_seed(7)
    cfg = _llama_cfg()
    sd, dense = _llama_checkpoint(cfg, gen, per_tensor)
    m = build_model(cfg, DictSource(sd, "llama"), device="cpu", dtype=torch.float32)
    lw = m.layers[0]
    q_cat = torch.cat([sd[f"model.layers.0.self_attn.{n}_proj.weight"] for n in "qkv"], 0)
    assert lw.qkv.wq is not None and torch.equal(lw.qkv.wq.view(torch.uint8), q_cat.view(torch.uint8))
    if not per_tensor:
        s_cat = torch.cat([sd[f"model.layers.0.self_attn.{n}_proj.weight_scale_inv"] for n in "qkv"], 0)
        assert torch.equal(lw.qkv.ws, s_cat) and not lw.qkv.ue8m0
    assert torch.equal(lw.down.wq.view(torch.uint8), sd["model.layers.0.mlp.down_proj.weight"].view(torch.uint8))
    # tensor parallel rank 1 of 2: rows of q / k / v / gate / up, columns of o_proj / down with their block scales
    m1 = build_model(cfg, DictSource(sd, "llama"), tp_rank=1, tp_size=2, device="cpu", dtype=torch.float32)
    o = sd["model.layers.1.self_attn.o_proj.weight"]
    assert torch.equal(m1.layers[1].o_proj.wq.view(torch.uint8), o[:, 128:].contiguous().view(torch.uint8))
    g = sd["model.layers.1.mlp.gate_proj.weight"]
    assert torch.equal(m1.layers[1].gate_up.wq[:256].view(torch.uint8), g[256:].contiguous().view(torch.uint8))
    if not per_tensor:
        assert torch.equal(m1.layers[1].o_proj.ws, sd["model.layers.1.self_attn.o_proj.weight_scale_inv"][:, 1:])
    # same function as the expanded weights up to the e4m3 rounding of the activations on the FP8 path (3 mantissa bits
    # at each of the eight GEMMs of this tiny random model; a misplaced scale block would be off by far more)
    ref = build_model(cfg, DictSource(dense, "llama"), device="cpu", dtype=torch.float32)
    tokens = torch.randint(3, cfg.vocab_size, (17,), generator=gen).tolist()
    for mod in (m, ref):
        mod.allocate_kv_cache(8, 16)
    got, want = m.forward(_step(tokens)), ref.forward(_step(tokens))
    assert float((got - want).norm() / want.norm()) < 0.15


def test_expert_stacks_keep_the_checkpoint_quantisation():
    gen = torch.Generator().manual_seed(9)
    cfg = ModelConfig(model_type="qwen2_moe", hidden_size=128, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=64,
                      intermediate_size=256, vocab_size=200, rms_norm_eps=1e-5, max_position_embeddings=64, max_token_len=64,
                      num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128, shared_expert_intermediate_size=128,
                      shared_expert_gate=True, norm_topk_prob=False, qkv_bias=False)
    H, I = 128, 128
    rnd = lambda *s: torch.randn(*s, generator=gen) * 0.05
    sd = {"model.embed_tokens.weight": rnd(200, H), "lm_head.weight": rnd(200, H), "model.norm.weight": torch.ones(H)}
    p = "model.layers.0."
    sd[p + "input_layernorm.weight"] = sd[p + "post_attention_layernorm.weight"] = torch.ones(H)
    for n in ("q", "k", "v", "o"):
        sd[p + f"self_attn.{n}_proj.weight"] = rnd(H, H)
    sd[p + "mlp.gate.weight"] = rnd(4, H)
    sd[p + "mlp.shared_expert_gate.weight"] = rnd(1, H)
    parts = {}
    for e in list(range(4)) + ["shared"]:
        ep = p + (f"mlp.experts.{e}." if e != "shared" else "mlp.shared_expert.")
        for n, shape in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
            q, s = _quant_blocks(rnd(*shape), gen)
            sd[ep + n + ".weight"], sd[ep + n + ".weight_scale_inv"] = q, s
            parts[(e, n)] = (q, s)
    m = build_model(cfg, DictSource(sd, "qwen2_moe"), device="cpu", dtype=torch.float32)
    moe = m.layers[0].moe
    w13 = torch.cat([torch.cat([parts[(e, "gate_proj")][0], parts[(e, "up_proj")][0]], 0) for e in range(4)], 0)
    assert moe.w13.dtype == FP8 and torch.equal(moe.w13.view(torch.uint8).reshape(w13.shape), w13.view(torch.uint8))
    s13 = torch.cat([torch.cat([parts[(e, "gate_proj")][1], parts[(e, "up_proj")][1]], 0) for e in range(4)], 0)
    assert torch.equal(moe.w13_scale.reshape(s13.shape), s13)
    assert torch.equal(moe.shared_down.wq.view(torch.uint8), parts[("shared", "down_proj")][0].view(torch.uint8))


def test_deepseek_fp8_checkpoint_layout():
    """DeepSeek-V3's published layout (every projection and expert in e4m3 with weight_scale_inv): the latent
    attention projections and expert stacks keep the checkpoint's values; kv_b_proj is expanded (it is folded into
    the absorbed attention matrices)."""
    gen = torch.Generator().manual_seed(11)
    cfg = ModelConfig(model_type="deepseek_v3", hidden_size=128, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=128,
                      intermediate_size=256, vocab_size=200, rms_norm_eps=1e-6, max_position_embeddings=64, max_token_len=64,
                      rope_neox=False, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128,
                      shared_expert_intermediate_size=128, num_shared_experts=1, moe_scoring="sigmoid", routed_scaling_factor=2.5,
                      n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=128, kv_lora_rank=128, qk_nope_head_dim=64,
                      qk_rope_head_dim=64, v_head_dim=64)
    H = 128
    rnd = lambda *s: torch.randn(*s, generator=gen) * 0.05
    sd = {"model.embed_tokens.weight": rnd(200, H), "lm_head.weight": rnd(200, H), "model.norm.weight": torch.ones(H)}
    fp8_names = []

    def put(name, shape):
        q, s = _quant_blocks(rnd(*shape), gen)
        sd[name + ".weight"], sd[name + ".weight_scale_inv"] = q, s
        fp8_names.append(name)

    for i in range(2):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = sd[p + "post_attention_layernorm.weight"] = torch.ones(H)
        a = p + "self_attn."
        put(a + "q_a_proj", (128, H)); put(a + "q_b_proj", (2 * 128, 128)); put(a + "kv_a_proj_with_mqa", (128 + 64, H))
        put(a + "kv_b_proj", (2 * (64 + 64), 128)); put(a + "o_proj", (H, 2 * 64))
        sd[a + "q_a_layernorm.weight"], sd[a + "kv_a_layernorm.weight"] = torch.ones(128), torch.ones(128)
        if i == 0:
            for n, shape in (("gate_proj", (256, H)), ("up_proj", (256, H)), ("down_proj", (H, 256))):
                put(p + "mlp." + n, shape)
        else:
            sd[p + "mlp.gate.weight"] = rnd(4, H)
            sd[p + "mlp.gate.e_score_correction_bias"] = torch.zeros(4)
            for e in list(range(4)) + ["s"]:
                ep = p + (f"mlp.experts.{e}." if e != "s" else "mlp.shared_experts.")
                for n, shape in (("gate_proj", (128, H)), ("up_proj", (128, H)), ("down_proj", (H, 128))):
                    put(ep + n, shape)
    m = build_model(cfg, DictSource(sd, "deepseek_v3"), device="cpu", dtype=torch.float32)
    l0, l1 = m.layers[0], m.layers[1]
    assert torch.equal(l0.o_proj.wq.view(torch.uint8), sd["model.layers.0.self_attn.o_proj.weight"].view(torch.uint8))
    assert torch.equal(l0.qkv.wq.view(torch.uint8), sd["model.layers.0.self_attn.kv_a_proj_with_mqa.weight"].view(torch.uint8))
    assert torch.equal(l0.qkv.ws, sd["model.layers.0.self_attn.kv_a_proj_with_mqa.weight_scale_inv"])
    assert l1.moe.w13.dtype == FP8 and l1.moe.w2.dtype == FP8
    m.allocate_kv_cache(8, 16)
    out = m.forward(_step(torch.randint(3, 200, (9,), generator=gen).tolist()))
    assert out.shape == (9, 200) and bool(torch.isfinite(out).all())
