"""Worker of the tensor-parallel family test (launched by torchrun on CPU ranks, gloo): every rank builds the same tiny
Hugging Face model of each family (seeded), loads its own tensor-parallel shard of it through the weight maps, runs one
prefill through the library-collective path and compares the logits with Hugging Face's on that rank.
argv: out_path family[,family...]"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from ksanallm_b200.config import model_config_from_hf  # noqa: E402
from ksanallm_b200.models.common import StepInput  # noqa: E402
from ksanallm_b200.models.weights import DictSource, build_model  # noqa: E402
from ksanallm_b200.parallel.comm import TPComm  # noqa: E402
from test_hf_parity_cpu import _init  # noqa: E402


def family(name):
    import transformers as tf
    common = dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=203,
                  max_position_embeddings=256)
    if name == "llama":
        c = tf.LlamaConfig(intermediate_size=128, rms_norm_eps=1e-5, tie_word_embeddings=False, **common)
        return tf.LlamaForCausalLM(c), c, 2e-4
    if name == "qwen2":
        c = tf.Qwen2Config(intermediate_size=128, rms_norm_eps=1e-6, tie_word_embeddings=True, **common)
        return tf.Qwen2ForCausalLM(c), c, 2e-4
    if name == "gpt2":
        c = tf.GPT2Config(n_embd=64, n_layer=2, n_head=4, vocab_size=203, n_positions=128, activation_function="gelu_new")
        return tf.GPT2LMHeadModel(c), c, 5e-4
    if name == "mixtral":
        c = tf.MixtralConfig(intermediate_size=96, num_local_experts=4, num_experts_per_tok=2, rms_norm_eps=1e-5,
                             sliding_window=None, tie_word_embeddings=False, **common)
        return tf.MixtralForCausalLM(c), c, 2e-4
    if name == "qwen2_moe":
        c = tf.Qwen2MoeConfig(intermediate_size=128, moe_intermediate_size=48, shared_expert_intermediate_size=80,
                              num_experts=4, num_experts_per_tok=2, norm_topk_prob=False, decoder_sparse_step=1,
                              mlp_only_layers=[], tie_word_embeddings=False, **common)
        return tf.Qwen2MoeForCausalLM(c), c, 2e-4
    if name == "glm":
        c = tf.GlmConfig(intermediate_size=128, rms_norm_eps=1e-5, head_dim=16, partial_rotary_factor=0.5,
                         attention_bias=True, tie_word_embeddings=False, pad_token_id=0, **common)
        return tf.GlmForCausalLM(c), c, 2e-4
    if name == "deepseek_v3":
        c = tf.DeepseekV3Config(hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
                                intermediate_size=128, moe_intermediate_size=32, n_routed_experts=8, n_shared_experts=1,
                                num_experts_per_tok=2, n_group=4, topk_group=2, routed_scaling_factor=2.5,
                                norm_topk_prob=True, first_k_dense_replace=1, q_lora_rank=24, kv_lora_rank=32,
                                qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, vocab_size=203,
                                max_position_embeddings=256, rms_norm_eps=1e-6, rope_scaling=None, tie_word_embeddings=False)
        m = tf.DeepseekV3ForCausalLM(c)
        return m, c, 5e-4
    raise ValueError(name)


def main():
    out_path, names = sys.argv[1], sys.argv[2].split(",")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    results = {}
    for name in names:
        hf, c, tol = family(name)
        hf = _init(hf).eval()
        if name == "deepseek_v3":
            with torch.no_grad():
                for n, b in hf.named_buffers():
                    if n.endswith("e_score_correction_bias"):
                        b.copy_(0.1 * torch.randn(b.shape, generator=torch.Generator().manual_seed(5)))
        cfg = model_config_from_hf(c.to_dict())
        cfg.max_token_len = min(cfg.max_token_len, 256)
        sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
        comm = TPComm(dist.group.WORLD, rank, world, "nccl", "cpu")
        model = build_model(cfg, DictSource(sd, cfg.model_type), rank, world, comm, device="cpu", dtype=torch.float32)
        torch.manual_seed(0)
        tokens = torch.randint(3, 203, (23,)).tolist()
        T = len(tokens)
        model.allocate_kv_cache(8, 16)
        ar = torch.arange(T, dtype=torch.int32)
        step = StepInput(torch.tensor(tokens, dtype=torch.int32), ar, ar.clone(), torch.tensor([0, T], dtype=torch.int32),
                         torch.tensor([T], dtype=torch.int32), torch.arange(8, dtype=torch.int32).view(1, 8),
                         num_multi=1, num_single=0, num_tokens=T, num_multi_tokens=T, max_q_len=T, max_kv_len=T)
        with torch.no_grad():
            want = hf(torch.tensor([tokens])).logits[0].float()
            got = model.forward(step)
        err = float((got[:, :want.shape[1]] - want).abs().max())
        bound = tol * max(1.0, float(want.abs().max()))
        results[name] = {"err": err, "bound": bound, "shape": list(got.shape), "ok": bool(got.shape[0] == T and err < bound)}
        dist.barrier()
    gathered = [None] * world
    dist.all_gather_object(gathered, results)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(gathered, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
