"""Architecture parity with the Hugging Face implementations: tiny randomly initialised HF models, their state
dicts loaded through the weight maps, logits compared on CPU in fp32 (prefill of one sequence)."""
import os
import re

import pytest
import torch

from ksanallm_b200.config import model_config_from_hf
from ksanallm_b200.models.common import StepInput
from ksanallm_b200.models.weights import DictSource, build_model

transformers = pytest.importorskip("transformers")


def _ours(hf_cfg: dict, state_dict, tokens):
    cfg = model_config_from_hf(hf_cfg)
    cfg.max_token_len = min(cfg.max_token_len, 256)
    sd = {k: v.detach().clone() for k, v in state_dict.items()}
    model = build_model(cfg, DictSource(sd, cfg.model_type), device="cpu", dtype=torch.float32)
    T = len(tokens)
    model.allocate_kv_cache(8, 16)
    ar = torch.arange(T, dtype=torch.int32)
    step = StepInput(torch.tensor(tokens, dtype=torch.int32), ar, ar.clone(), torch.tensor([0, T], dtype=torch.int32),
                     torch.tensor([T], dtype=torch.int32), torch.arange(8, dtype=torch.int32).view(1, 8),
                     num_multi=1, num_single=0, num_tokens=T, num_multi_tokens=T, max_q_len=T, max_kv_len=T)
    return model.forward(step)


def _check(hf_model, hf_cfg, tol=2e-4):
    torch.manual_seed(0)
    tokens = torch.randint(3, hf_cfg["vocab_size"], (23,)).tolist()
    hf_model.eval()
    with torch.no_grad():
        want = hf_model(torch.tensor([tokens])).logits[0].float()
        got = _ours(hf_cfg, hf_model.state_dict(), tokens)
    assert got.shape == want.shape
    err = float((got - want).abs().max())
    assert err < tol * max(1.0, float(want.abs().max())), err


def _init(model, std=0.05):
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * std)
            elif "norm" in n or "ln_" in n:
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g) if n.endswith("weight") else 0.1 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(torch.randn(p.shape, generator=g) * std)
    return model


def test_llama_gqa_with_llama3_rope_scaling():
    from transformers import LlamaConfig, LlamaForCausalLM
    c = LlamaConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                    vocab_size=200, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=10000.0,
                    rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                  "original_max_position_embeddings": 64}, tie_word_embeddings=False)
    _check(_init(LlamaForCausalLM(c)), c.to_dict())


def test_qwen2_qkv_bias_and_tied_embeddings():
    from transformers import Qwen2Config, Qwen2ForCausalLM
    c = Qwen2Config(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                    vocab_size=200, max_position_embeddings=256, rms_norm_eps=1e-6, tie_word_embeddings=True)
    _check(_init(Qwen2ForCausalLM(c)), c.to_dict())


def test_gpt2_learned_positions_layernorm_gelu_conv1d():
    from transformers import GPT2Config, GPT2LMHeadModel
    c = GPT2Config(n_embd=64, n_layer=2, n_head=4, vocab_size=200, n_positions=128, activation_function="gelu_new")
    _check(_init(GPT2LMHeadModel(c)), c.to_dict(), tol=5e-4)


def test_gpt1_post_norm_blocks():
    """GPT-1 (`openai-gpt`): learned positions, blocks that normalise after the residual add, Conv1D weights, tied head."""
    from transformers import OpenAIGPTConfig, OpenAIGPTLMHeadModel
    c = OpenAIGPTConfig(n_embd=64, n_layer=2, n_head=4, vocab_size=200, n_positions=128, afn="gelu",
                        resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    _check(_init(OpenAIGPTLMHeadModel(c)), c.to_dict(), tol=5e-4)


def test_fairseq_style_decoder_sinusoidal_positions_scaled_embeddings():
    """A fairseq-style decoder (XGLM is the Hugging Face export of that family): sinusoidal positions offset by the
    padding index, embeddings scaled by sqrt(d), pre-norm blocks with self_attn_layer_norm / fc1 / fc2 /
    final_layer_norm names and a closing layer_norm, through the `fairseq-transformer` model type and the
    GPT-family weight map."""
    from transformers import XGLMConfig, XGLMForCausalLM
    c = XGLMConfig(vocab_size=200, max_position_embeddings=128, d_model=64, ffn_dim=160, num_layers=2, attention_heads=4,
                   activation_function="gelu", dropout=0.0, attention_dropout=0.0, activation_dropout=0.0, layerdrop=0.0,
                   scale_embedding=True, pad_token_id=1, bos_token_id=0, eos_token_id=2)
    m = _init(XGLMForCausalLM(c))
    hf_cfg = {"model_type": "fairseq-transformer", "decoder_embed_dim": 64, "decoder_layers": 2, "decoder_attention_heads": 4,
              "decoder_ffn_embed_dim": 160, "vocab_size": 200, "max_target_positions": 128, "activation_function": "gelu",
              "decoder_normalize_before": True, "no_scale_embedding": False, "pad_token_id": 1,
              "tie_word_embeddings": True}
    torch.manual_seed(0)
    tokens = torch.randint(3, 200, (23,)).tolist()
    m.eval()
    with torch.no_grad():
        want = m(torch.tensor([tokens])).logits[0].float()
        got = _ours(hf_cfg, m.state_dict(), tokens)
    err = float((got - want).abs().max())
    assert err < 5e-4 * max(1.0, float(want.abs().max())), err


def test_mixtral_softmax_top2_experts():
    from transformers import MixtralConfig, MixtralForCausalLM
    c = MixtralConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=96,
                      vocab_size=200, max_position_embeddings=256, num_local_experts=4, num_experts_per_tok=2,
                      rms_norm_eps=1e-5, sliding_window=None, tie_word_embeddings=False)
    _check(_init(MixtralForCausalLM(c)), c.to_dict())


def test_qwen2_moe_shared_expert_gate():
    from transformers import Qwen2MoeConfig, Qwen2MoeForCausalLM
    c = Qwen2MoeConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=128, moe_intermediate_size=48, shared_expert_intermediate_size=80, num_experts=4,
                       num_experts_per_tok=2, norm_topk_prob=False, vocab_size=200, max_position_embeddings=256,
                       decoder_sparse_step=1, mlp_only_layers=[], tie_word_embeddings=False)
    _check(_init(Qwen2MoeForCausalLM(c)), c.to_dict())


def test_deepseek_v3_mla_and_grouped_sigmoid_routing():
    try:
        from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
    except ImportError:
        pytest.skip("this transformers build has no DeepseekV3")
    c = DeepseekV3Config(hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
                         intermediate_size=128, moe_intermediate_size=32, n_routed_experts=8, n_shared_experts=1,
                         num_experts_per_tok=2, n_group=4, topk_group=2, routed_scaling_factor=2.5, norm_topk_prob=True,
                         first_k_dense_replace=1, q_lora_rank=24, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8,
                         v_head_dim=16, vocab_size=200, max_position_embeddings=256, rms_norm_eps=1e-6, rope_scaling=None,
                         tie_word_embeddings=False)
    m = _init(DeepseekV3ForCausalLM(c))
    with torch.no_grad():
        for n, b in m.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.copy_(0.1 * torch.randn(b.shape, generator=torch.Generator().manual_seed(5)))
    _check(m, c.to_dict(), tol=5e-4)


def test_glm4_partial_interleaved_rope_fused_gate_up():
    """GLM-4 in the Hugging Face layout runs on the ChatGLM flags: interleaved rotary pairs over half of the
    head, QKV bias, one fused gate|up matrix."""
    from transformers import GlmConfig, GlmForCausalLM
    c = GlmConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                  vocab_size=200, max_position_embeddings=256, rms_norm_eps=1e-5, head_dim=16, partial_rotary_factor=0.5,
                  attention_bias=True, tie_word_embeddings=False, pad_token_id=0)
    _check(_init(GlmForCausalLM(c)), c.to_dict())


def test_mistral_runs_as_llama():
    from transformers import MistralConfig, MistralForCausalLM
    c = MistralConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                      vocab_size=200, max_position_embeddings=256, rms_norm_eps=1e-5, sliding_window=None,
                      tie_word_embeddings=False)
    _check(_init(MistralForCausalLM(c)), c.to_dict())


def test_qwen2_vl_image_tokens_mrope_and_vision_tower():
    """Whole Qwen2-VL forward: the plug-in's vision tower (loaded from the checkpoint's visual.* tensors) feeds the
    image tokens' embeddings, its mrope positions drive the 3-axis rotary, and the language model's weights arrive
    through the ``model.language_model.*`` names of newer exports with their fields under ``text_config``."""
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration
    from ksanallm_b200.ksana_plugin.qwen2_vl.ksana_plugin import VisionTower, mrope_positions
    pad = 290
    cfg = Qwen2VLConfig(
        text_config=dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                         vocab_size=400, max_position_embeddings=256, rms_norm_eps=1e-6,
                         rope_parameters={"rope_type": "default", "mrope_section": [2, 3, 3], "rope_theta": 10000.0}),
        vision_config=dict(depth=1, embed_dim=32, hidden_size=64, num_heads=2, patch_size=14, spatial_merge_size=2,
                           temporal_patch_size=2),
        image_token_id=pad, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293, tie_word_embeddings=False)
    hf = _init(Qwen2VLForConditionalGeneration(cfg)).eval()
    mc = model_config_from_hf(cfg.to_dict())
    assert mc.model_type == "qwen2_vl" and mc.position_embedding == "mrope" and mc.mrope_section == [2, 3, 3] and mc.qkv_bias
    mc.max_token_len = 256
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    model = build_model(mc, DictSource(sd, mc.model_type), device="cpu", dtype=torch.float32)
    tower = VisionTower(hidden_out=64, dim=32, depth=1, heads=2, patch=14, merge=2, temporal=2).eval()
    missing, unexpected = tower.load_state_dict({k.split("visual.", 1)[1]: v for k, v in sd.items() if "visual." in k}, strict=False)
    assert not missing and not unexpected
    img = torch.rand(3, 56, 84, generator=torch.Generator().manual_seed(5))
    flat, grids = tower.patchify([img])
    n_img = grids[0][0] * (grids[0][1] // 2) * (grids[0][2] // 2)
    toks = [5, 6, 292] + [pad] * n_img + [293, 7, 8, 9, 10]
    kinds = torch.tensor([[1 if t == pad else 0 for t in toks]], dtype=torch.int32)
    with torch.no_grad():
        try:
            want = hf(input_ids=torch.tensor([toks]), pixel_values=flat, image_grid_thw=torch.tensor(grids),
                      mm_token_type_ids=kinds).logits[0].float()
        except TypeError:
            pytest.skip("this transformers version has another multimodal forward signature")
        emb = tower.forward_patches(flat, grids)
    T = len(toks)
    model.allocate_kv_cache(8, 16)
    ar = torch.arange(T, dtype=torch.int32)
    step = StepInput(torch.tensor(toks, dtype=torch.int32), ar, ar.clone(), torch.tensor([0, T], dtype=torch.int32),
                     torch.tensor([T], dtype=torch.int32), torch.arange(8, dtype=torch.int32).view(1, 8),
                     num_multi=1, num_single=0, num_tokens=T, num_multi_tokens=T, max_q_len=T, max_kv_len=T)
    step.mrope_positions = mrope_positions(toks, pad, grids, 2)
    step.refit_positions = torch.arange(3, 3 + n_img, dtype=torch.int32)
    step.refit_embeddings = emb.float()
    got = model.forward(step)
    assert float((got - want).abs().max()) < 2e-4 * max(1.0, float(want.abs().max()))


def test_baichuan_13b_style_alibi_wpack_normhead():
    """Baichuan has no implementation inside transformers; this restates its published modeling code (13B class):
    packed W_pack projection, ALiBi bias slope_h * key_position on the attention scores, RMSNorm, SwiGLU, and
    Baichuan2's NormHead (rows of lm_head normalised). The slopes are also checked against BLOOM's builder."""
    import math
    import torch.nn.functional as F
    from transformers.models.bloom.modeling_bloom import build_alibi_tensor
    from ksanallm_b200.models.common import alibi_slopes
    for heads in (8, 32, 40):
        want = build_alibi_tensor(torch.ones(1, 5), heads, torch.float32).view(heads, 5)[:, 1]     # slope * position 1
        assert torch.allclose(alibi_slopes(heads), want, rtol=1e-6)

    H, L, heads, inter, V, T = 80, 2, 5, 96, 125696 // 512, 19          # hidden != 4096 -> ALiBi
    hf_cfg = {"model_type": "baichuan", "hidden_size": H, "num_hidden_layers": L, "num_attention_heads": heads,
              "intermediate_size": inter, "vocab_size": 125696, "rms_norm_eps": 1e-6, "max_position_embeddings": 128}
    g = torch.Generator().manual_seed(2)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.08
    sd = {"model.embed_tokens.weight": rnd(125696, H) * 0, "model.norm.weight": 1 + rnd(H), "lm_head.weight": rnd(125696, H) * 0}
    # only the first V rows of the big vocabulary are exercised; the rest stays zero (the size selects Baichuan2's NormHead)
    sd["model.embed_tokens.weight"][:V] = rnd(V, H)
    sd["lm_head.weight"][:V] = rnd(V, H)
    for i in range(L):
        p = f"model.layers.{i}."
        sd[p + "self_attn.W_pack.weight"] = rnd(3 * H, H)
        sd[p + "self_attn.o_proj.weight"] = rnd(H, H)
        sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"] = rnd(inter, H), rnd(inter, H)
        sd[p + "mlp.down_proj.weight"] = rnd(H, inter)
        sd[p + "input_layernorm.weight"], sd[p + "post_attention_layernorm.weight"] = 1 + rnd(H), 1 + rnd(H)
    tokens = torch.randint(3, V, (T,), generator=g).tolist()

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w

    h = sd["model.embed_tokens.weight"][tokens]
    slopes = alibi_slopes(heads)
    D = H // heads
    bias = slopes.view(heads, 1, 1) * torch.arange(T).view(1, 1, T).float()
    causal = torch.full((T, T), float("-inf")).triu(1)
    for i in range(L):
        p = f"model.layers.{i}."
        x = rms(h, sd[p + "input_layernorm.weight"])
        q, k, v = (x @ sd[p + "self_attn.W_pack.weight"].t()).view(T, 3, heads, D).unbind(1)
        s = torch.einsum("thd,shd->hts", q, k) / math.sqrt(D) + bias + causal
        a = torch.einsum("hts,shd->thd", s.softmax(-1), v).reshape(T, H)
        h = h + a @ sd[p + "self_attn.o_proj.weight"].t()
        x = rms(h, sd[p + "post_attention_layernorm.weight"])
        h = h + (F.silu(x @ sd[p + "mlp.gate_proj.weight"].t()) * (x @ sd[p + "mlp.up_proj.weight"].t())) @ sd[p + "mlp.down_proj.weight"].t()
    want = rms(h, sd["model.norm.weight"]) @ F.normalize(sd["lm_head.weight"][:V], dim=-1).t()
    got = _ours(hf_cfg, sd, tokens)[:, :V]
    assert float((got - want).abs().max()) < 2e-4 * max(1.0, float(want.abs().max()))


def test_chatglm3_checkpoint_names_and_config_keys():
    """The original ChatGLM2/3 layout (fused query_key_value with bias, dense_h_to_4h = gate|up, THUDM config keys)
    arrives through the weight map: the tensors of a tiny GLM-4 model renamed that way give GLM-4's logits."""
    from transformers import GlmConfig, GlmForCausalLM
    c = GlmConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                  vocab_size=200, max_position_embeddings=256, rms_norm_eps=1e-5, head_dim=16, partial_rotary_factor=0.5,
                  attention_bias=True, tie_word_embeddings=False, pad_token_id=0)
    hf = _init(GlmForCausalLM(c)).eval()
    src = hf.state_dict()
    sd = {"transformer.embedding.word_embeddings.weight": src["model.embed_tokens.weight"],
          "transformer.encoder.final_layernorm.weight": src["model.norm.weight"],
          "transformer.output_layer.weight": src["lm_head.weight"],
          "transformer.rotary_pos_emb.inv_freq": torch.zeros(4)}
    for i in range(2):
        p, q = f"model.layers.{i}.", f"transformer.encoder.layers.{i}."
        sd[q + "input_layernorm.weight"] = src[p + "input_layernorm.weight"]
        sd[q + "post_attention_layernorm.weight"] = src[p + "post_attention_layernorm.weight"]
        for kind in ("weight", "bias"):
            sd[q + f"self_attention.query_key_value.{kind}"] = torch.cat(
                [src[p + f"self_attn.{n}_proj.{kind}"] for n in ("q", "k", "v")], 0)
        sd[q + "self_attention.dense.weight"] = src[p + "self_attn.o_proj.weight"]
        sd[q + "mlp.dense_h_to_4h.weight"] = src[p + "mlp.gate_up_proj.weight"]
        sd[q + "mlp.dense_4h_to_h.weight"] = src[p + "mlp.down_proj.weight"]
    thudm = {"model_type": "chatglm", "hidden_size": 64, "num_layers": 2, "num_attention_heads": 4, "kv_channels": 16,
             "multi_query_attention": True, "multi_query_group_num": 2, "ffn_hidden_size": 128, "padded_vocab_size": 200,
             "layernorm_epsilon": 1e-5, "add_qkv_bias": True, "seq_length": 256, "rmsnorm": True}
    torch.manual_seed(0)
    tokens = torch.randint(3, 200, (23,)).tolist()
    with torch.no_grad():
        want = hf(torch.tensor([tokens])).logits[0].float()
    got = _ours(thudm, sd, tokens)
    assert float((got - want).abs().max()) < 2e-4 * max(1.0, float(want.abs().max()))


def test_qwen_first_generation_checkpoint_names():
    """Qwen-7B/14B (first generation) layout through its weight map: fused c_attn with bias, w2 = gate, w1 = up,
    intermediate_size counting both. The tensors of a tiny Qwen2 model (no grouped KV heads) renamed that way give
    Qwen2's logits."""
    from transformers import Qwen2Config, Qwen2ForCausalLM
    c = Qwen2Config(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, intermediate_size=96,
                    vocab_size=200, max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=10000.0,
                    tie_word_embeddings=False, use_sliding_window=False)
    hf = _init(Qwen2ForCausalLM(c)).eval()
    src = hf.state_dict()
    sd = {"transformer.wte.weight": src["model.embed_tokens.weight"], "transformer.ln_f.weight": src["model.norm.weight"],
          "lm_head.weight": src["lm_head.weight"]}
    for i in range(2):
        p, q = f"model.layers.{i}.", f"transformer.h.{i}."
        sd[q + "ln_1.weight"], sd[q + "ln_2.weight"] = src[p + "input_layernorm.weight"], src[p + "post_attention_layernorm.weight"]
        for kind in ("weight", "bias"):
            sd[q + f"attn.c_attn.{kind}"] = torch.cat([src[p + f"self_attn.{n}_proj.{kind}"] for n in ("q", "k", "v")], 0)
        sd[q + "attn.c_proj.weight"] = src[p + "self_attn.o_proj.weight"]
        sd[q + "mlp.w2.weight"], sd[q + "mlp.w1.weight"] = src[p + "mlp.gate_proj.weight"], src[p + "mlp.up_proj.weight"]
        sd[q + "mlp.c_proj.weight"] = src[p + "mlp.down_proj.weight"]
    v1 = {"model_type": "qwen", "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "kv_channels": 16,
          "intermediate_size": 192, "vocab_size": 200, "layer_norm_epsilon": 1e-6, "rotary_emb_base": 10000, "seq_length": 256}
    torch.manual_seed(0)
    tokens = torch.randint(3, 200, (23,)).tolist()
    with torch.no_grad():
        want = hf(torch.tensor([tokens])).logits[0].float()
    got = _ours(v1, sd, tokens)
    assert float((got - want).abs().max()) < 2e-4 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("scaling", [{"rope_type": "linear", "factor": 4.0},
                                     {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 16,
                                      "beta_fast": 32.0, "beta_slow": 1.0}])
def test_llama_rope_scaling_variants(scaling):
    from transformers import LlamaConfig, LlamaForCausalLM
    c = LlamaConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                    vocab_size=200, max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=10000.0,
                    rope_scaling=dict(scaling), tie_word_embeddings=False)
    _check(_init(LlamaForCausalLM(c)), c.to_dict())


@pytest.mark.parametrize("layout", ["sharded-safetensors", "pytorch-bin"])
def test_checkpoint_directories_on_disk(tmp_path, layout):
    """A checkpoint directory as users have it (config.json + sharded safetensors with an index, or a pickled
    pytorch_model.bin; tied embeddings) loads through CheckpointSource and reproduces Hugging Face's logits."""
    import os
    from transformers import Qwen2Config, Qwen2ForCausalLM
    from ksanallm_b200.config import load_model_config
    from ksanallm_b200.models.weights import CheckpointSource
    c = Qwen2Config(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                    vocab_size=200, max_position_embeddings=128, rms_norm_eps=1e-6, tie_word_embeddings=True, dtype="float32")
    hf = _init(Qwen2ForCausalLM(c)).eval()
    hf.tie_weights()
    d = str(tmp_path)
    if layout == "sharded-safetensors":
        hf.save_pretrained(d, safe_serialization=True, max_shard_size="60KB")
        assert len([f for f in os.listdir(d) if f.endswith(".safetensors")]) > 1
    else:
        hf.config.save_pretrained(d)
        torch.save(dict(hf.state_dict()), os.path.join(d, "pytorch_model.bin"))
    mc = load_model_config(d)
    assert mc.tie_word_embeddings and mc.qkv_bias and mc.dtype == "float32"
    mc.max_token_len = 128
    model = build_model(mc, CheckpointSource(d, mc.model_type), device="cpu", dtype=torch.float32)
    torch.manual_seed(0)
    tokens = torch.randint(3, 200, (19,)).tolist()
    T = len(tokens)
    model.allocate_kv_cache(8, 16)
    ar = torch.arange(T, dtype=torch.int32)
    step = StepInput(torch.tensor(tokens, dtype=torch.int32), ar, ar.clone(), torch.tensor([0, T], dtype=torch.int32),
                     torch.tensor([T], dtype=torch.int32), torch.arange(8, dtype=torch.int32).view(1, 8),
                     num_multi=1, num_single=0, num_tokens=T, num_multi_tokens=T, max_q_len=T, max_kv_len=T)
    with torch.no_grad():
        want = hf(torch.tensor([tokens])).logits[0].float()
    got = model.forward(step)
    assert float((got - want).abs().max()) < 2e-4 * max(1.0, float(want.abs().max()))


def test_unknown_model_type_with_its_own_weight_map(tmp_path):
    """A Llama-shaped checkpoint under a model_type nobody knows, with its tensors under other names and a
    ``<model_type>_weight_map.json`` (``$N`` groups, as written for the reference) next to it: served as Llama with
    Hugging Face Llama's logits. Without the map the type is refused; a map next to the checkpoint wins over the
    package's map of the same name."""
    import json
    from transformers import LlamaConfig, LlamaForCausalLM
    from ksanallm_b200.config import find_weight_map, load_model_config, resolve_architecture
    from ksanallm_b200.models.weights import CheckpointSource, load_weight_map
    c = LlamaConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                    vocab_size=200, max_position_embeddings=128, rms_norm_eps=1e-5, tie_word_embeddings=False)
    hf = _init(LlamaForCausalLM(c)).eval()
    d = str(tmp_path)
    cfg = c.to_dict()
    cfg["model_type"] = "my_house_model"
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    renamed = {}
    for k, v in hf.state_dict().items():
        k = k.replace("model.embed_tokens.", "backbone.tok.").replace("model.norm.", "backbone.final_norm.")
        k = re.sub(r"^model\.layers\.(\d+)\.", r"backbone.blocks.\1.", k)
        renamed[k] = v.clone()
    torch.save(renamed, os.path.join(d, "pytorch_model.bin"))
    with pytest.raises(ValueError, match="not supported"):
        load_model_config(d)
    with open(os.path.join(d, "my_house_model_weight_map.json"), "w") as f:
        json.dump({r"^backbone\.tok\.(.*)$": "model.embed_tokens.$1", r"^backbone\.final_norm\.(.*)$": "model.norm.$1",
                   r"^backbone\.blocks\.(\d+)\.(.*)$": "model.layers.$1.$2"}, f)
    mc = load_model_config(d)
    assert mc.model_type == "llama" and mc.hf_model_type == "my_house_model"
    mc.max_token_len = 128
    model = build_model(mc, CheckpointSource(d, mc.model_type, mc.hf_model_type), device="cpu", dtype=torch.float32)
    torch.manual_seed(0)
    tokens = torch.randint(3, 200, (17,)).tolist()
    T = len(tokens)
    model.allocate_kv_cache(8, 16)
    ar = torch.arange(T, dtype=torch.int32)
    step = StepInput(torch.tensor(tokens, dtype=torch.int32), ar, ar.clone(), torch.tensor([0, T], dtype=torch.int32),
                     torch.tensor([T], dtype=torch.int32), torch.arange(8, dtype=torch.int32).view(1, 8),
                     num_multi=1, num_single=0, num_tokens=T, num_multi_tokens=T, max_q_len=T, max_kv_len=T)
    with torch.no_grad():
        want = hf(torch.tensor([tokens])).logits[0].float()
    assert float((model.forward(step) - want).abs().max()) < 2e-4 * max(1.0, float(want.abs().max()))
    # family by containment, and the search order of the map file
    assert resolve_architecture("CodeLlama") == "llama" and resolve_architecture("gpt_bigcode") == "gpt"
    assert find_weight_map("qwen").endswith(os.path.join("weight_map", "qwen_weight_map.json"))
    with open(os.path.join(d, "qwen_weight_map.json"), "w") as f:
        json.dump({"^a$": "b"}, f)
    assert find_weight_map("qwen", d) == os.path.join(d, "qwen_weight_map.json")
    assert len(load_weight_map("qwen", model_dir=d)) == 1 and len(load_weight_map("qwen")) > 1
    # config.json's own spelling names the file before the family does
    with open(os.path.join(d, "gpt2_weight_map.json"), "w") as f:
        json.dump({"^x$": "y", "^z$": "w"}, f)
    assert len(load_weight_map("gpt", model_dir=d, hf_model_type="gpt2")) == 2


@pytest.mark.parametrize("world", [2, 4])
def test_families_under_tensor_parallelism(tmp_path, world):
    """Every model family as tensor-parallel CPU ranks (gloo, library collectives): each rank loads its shard of the
    same tiny Hugging Face model - with four ranks there are more ranks than KV heads, and the vocabulary of 203 never
    divides - and every rank's logits equal Hugging Face's."""
    import json
    import socket
    import subprocess
    import sys
    try:
        from transformers import DeepseekV3Config  # noqa: F401
        names = "llama,qwen2,gpt2,mixtral,qwen2_moe,glm,deepseek_v3"
    except ImportError:
        names = "llama,qwen2,gpt2,mixtral,qwen2_moe,glm"
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "result.json"
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(here, "tp_families_worker.py"),
                        str(out), names], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    per_rank = json.loads(out.read_text())
    assert len(per_rank) == world
    for rank, res in enumerate(per_rank):
        assert set(res) == set(names.split(","))
        for name, v in res.items():
            assert v["ok"], (rank, name, v)


@pytest.mark.parametrize("name", ["llama", "qwen2", "gpt2", "mixtral", "qwen2_moe", "glm", "deepseek_v3"])
def test_engine_features_across_families(name):
    """Chunked prefill (16-token pieces), the prefix cache and swap preemption in a small block pool, for every family:
    five prompts that share a 35-token head, generated in two waves through the engine, continue exactly as Hugging
    Face's greedy generation does (learned positions, latent-attention caches and routed layers all see prompts in
    pieces and cached heads)."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from tp_families_worker import family
    from ksanallm_b200.config import EngineConfig
    from ksanallm_b200.runtime.engine import LLMEngine
    from ksanallm_b200.utils import native_engine as ne
    try:
        hf, c, _ = family(name)
    except AttributeError:
        pytest.skip(f"this transformers build has no {name}")
    hf = _init(hf, std=0.2).eval()
    cfg = model_config_from_hf(c.to_dict())
    cfg.max_token_len = 128
    cfg.eos_token_ids = []
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    model = build_model(cfg, DictSource(sd, cfg.model_type), device="cpu", dtype=torch.float32)
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size = 8
    ec.batch_scheduler.max_token_len = 128
    ec.batch_scheduler.max_step_tokens = 64
    ec.batch_scheduler.split_fuse_token_num = 16
    ec.batch_scheduler.enable_auto_prefix_cache = True
    ec.batch_scheduler.preempt_mode = 0            # swap
    eng = LLMEngine(model, cfg, ec, num_blocks=9, num_host_blocks=32)      # nine blocks: one sequence gets swapped out
    g = torch.Generator().manual_seed(2)
    head = torch.randint(3, 203, (35,), generator=g).tolist()
    prompts = [head + torch.randint(3, 203, (4 + 3 * i,), generator=g).tolist() for i in range(5)]
    s = ne.SamplingConfig()
    s.max_new_tokens, s.ignore_eos, s.topk = 10, True, 1
    reqs = eng.generate(prompts[:1], s) + eng.generate(prompts[1:], s)
    for r, p in zip(reqs, prompts):
        assert r.status_code == 0, r.status_message
        with torch.no_grad():
            want = hf.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, eos_token_id=None, pad_token_id=0)
        assert list(r.outputs[0].tokens) == want[0, len(p):].tolist()
    st = eng.scheduler.stats()
    assert st["prefix_hit_tokens"] >= 4 * 32 and st["preempt_swap"] >= 1 and st["swapped_in_blocks"] >= 1
    assert eng.scheduler.check_invariants()[0]
