"""GGUF single-file checkpoints: parser, block-format dequantisation, llama.cpp name map and rotary un-permutation."""
import torch

from ksanallm_b200.config import ModelConfig
from ksanallm_b200.models import gguf
from ksanallm_b200.models.weights import RandomSource, build_model


def tiny_cfg():
    return ModelConfig(model_type="llama", hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                       intermediate_size=128, vocab_size=320, max_position_embeddings=128, max_token_len=128)


def _export(cfg, src, path, gtype):
    """Write the model the way llama.cpp's converter does: its tensor names, q/k rows permuted per head."""
    H, D = cfg.hidden_size, cfg.head_dim
    t, kinds = {}, {}
    def put(name, x, quant=True):
        t[name] = x
        kinds[name] = gtype if (quant and x.dim() == 2) else gguf.GGML_F32
    put("token_embd.weight", src.get("model.embed_tokens.weight", (cfg.vocab_size, H)))
    put("output_norm.weight", src.get("model.norm.weight", (H,), kind="ones"))
    put("output.weight", src.get("lm_head.weight", (cfg.vocab_size, H)))
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        put(f"blk.{i}.attn_norm.weight", src.get(p + "input_layernorm.weight", (H,), kind="ones"))
        put(f"blk.{i}.ffn_norm.weight", src.get(p + "post_attention_layernorm.weight", (H,), kind="ones"))
        put(f"blk.{i}.attn_q.weight", gguf._permute_rope(src.get(p + "self_attn.q_proj.weight", (cfg.num_heads * D, H)), cfg.num_heads))
        put(f"blk.{i}.attn_k.weight", gguf._permute_rope(src.get(p + "self_attn.k_proj.weight", (cfg.num_kv_heads * D, H)), cfg.num_kv_heads))
        put(f"blk.{i}.attn_v.weight", src.get(p + "self_attn.v_proj.weight", (cfg.num_kv_heads * D, H)))
        put(f"blk.{i}.attn_output.weight", src.get(p + "self_attn.o_proj.weight", (H, cfg.num_heads * D)))
        put(f"blk.{i}.ffn_gate.weight", src.get(p + "mlp.gate_proj.weight", (cfg.intermediate_size, H)))
        put(f"blk.{i}.ffn_up.weight", src.get(p + "mlp.up_proj.weight", (cfg.intermediate_size, H)))
        put(f"blk.{i}.ffn_down.weight", src.get(p + "mlp.down_proj.weight", (H, cfg.intermediate_size)))
    meta = {"general.architecture": "llama", "llama.embedding_length": H, "llama.block_count": cfg.num_layers,
            "llama.attention.head_count": cfg.num_heads, "llama.attention.head_count_kv": cfg.num_kv_heads,
            "llama.feed_forward_length": cfg.intermediate_size, "llama.context_length": 128,
            "llama.attention.layer_norm_rms_epsilon": 1e-5, "llama.rope.freq_base": 10000.0,
            "llama.vocab_size": cfg.vocab_size, "tokenizer.ggml.tokens": ["a", "b"]}
    gguf.write_gguf(path, meta, t, kinds)


def _logits(model, cfg):
    from ksanallm_b200.config import EngineConfig
    from ksanallm_b200.runtime.engine import LLMEngine
    from ksanallm_b200.utils import native_engine as ne
    ec = EngineConfig()
    ec.batch_scheduler.max_token_len = 64
    eng = LLMEngine(model, cfg, ec, num_blocks=32)
    s = ne.SamplingConfig()
    s.max_new_tokens, s.ignore_eos = 3, True
    return [r.outputs[0].tokens for r in eng.generate([[5, 6, 7, 8], [9, 10]], s)]


def test_gguf_roundtrip_f32_and_f16(tmp_path):
    cfg, src = tiny_cfg(), RandomSource(seed=3, std=0.05)
    want = _logits(build_model(cfg, src, device="cpu", dtype=torch.float32), cfg)
    for gtype in (gguf.GGML_F32, gguf.GGML_F16):
        path = str(tmp_path / f"m{gtype}.gguf")
        _export(cfg, src, path, gtype)
        gs = gguf.GGUFSource(path)
        assert gs.has("model.layers.1.self_attn.q_proj.weight") and gs.has("lm_head.weight")
        q = gs.get("model.layers.0.self_attn.q_proj.weight")
        ref_q = src.get("model.layers.0.self_attn.q_proj.weight", (cfg.num_heads * cfg.head_dim, cfg.hidden_size))
        assert torch.allclose(q, ref_q, atol=1e-3 if gtype == gguf.GGML_F16 else 0)
        c2 = gguf.model_config_from_gguf(gs.file.meta)
        assert (c2.hidden_size, c2.num_layers, c2.num_heads, c2.num_kv_heads, c2.intermediate_size, c2.vocab_size) == \
               (cfg.hidden_size, cfg.num_layers, cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size, cfg.vocab_size)
        if gtype == gguf.GGML_F32:
            assert _logits(build_model(cfg, gs, device="cpu", dtype=torch.float32), cfg) == want


def test_gguf_block_formats(tmp_path):
    torch.manual_seed(0)
    w = torch.randn(8, 64)
    path = str(tmp_path / "q.gguf")
    gguf.write_gguf(path, {"general.architecture": "llama"}, {"a.weight": w, "b.weight": w}, {"a.weight": gguf.GGML_Q8_0, "b.weight": gguf.GGML_BF16})
    f = gguf.GGUFFile(path)
    assert f.tensors["a.weight"][0] == (8, 64)
    assert (f.get("a.weight") - w).abs().max() < w.abs().max() / 127 + 1e-3
    assert torch.equal(f.get("b.weight"), w.to(torch.bfloat16).float())
    # Q4_0 decoding against a hand-built block: d = 0.5, nibbles 0..15 twice -> (n - 8) * 0.5
    import numpy as np, struct
    blk = np.frombuffer(np.float16(0.5).tobytes() + bytes((i | ((15 - i) << 4)) for i in range(16)), dtype=np.uint8)
    head = struct.pack("<IIQQ", gguf.GGUF_MAGIC, 3, 1, 0)
    info = gguf._w_string("q4") + struct.pack("<I", 1) + struct.pack("<Q", 32) + struct.pack("<IQ", gguf.GGML_Q4_0, 0)
    pre = head + info
    pre += b"\0" * ((-len(pre)) % 32)
    p2 = str(tmp_path / "q4.gguf")
    open(p2, "wb").write(pre + blk.tobytes())
    got = gguf.GGUFFile(p2).get("q4")
    want = torch.tensor([(i - 8) * 0.5 for i in range(16)] + [((15 - i) - 8) * 0.5 for i in range(16)])
    assert torch.equal(got, want)
