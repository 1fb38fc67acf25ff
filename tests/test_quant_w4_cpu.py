"""GPTQ / AWQ checkpoint unpacking, the native 4-bit group format, and a 4-bit model end to end on CPU."""
import torch

from ksanallm_b200.config import ModelConfig
from ksanallm_b200.models import quant_w4 as q4
from ksanallm_b200.models.weights import DictSource, RandomSource, build_model
from ksanallm_b200.ops import reference as ref
from ksanallm_b200.ops.dispatch import LinearWeight, linear


def _lattice(w, group, perm=None):
    """What a 4-bit asymmetric group quantiser makes of w (groups over the given feature order)."""
    N, K = w.shape
    wp = w if perm is None else w[:, perm]
    q, zero, scale = q4.quantize_levels(wp, group)
    gi = torch.arange(K) // group
    d = ((q.float() - zero.float()[gi]) * scale.float()[gi]).t()
    if perm is not None:
        d = d[:, torch.argsort(perm)]
    return d


def test_gptq_roundtrip_plain_and_act_order():
    torch.manual_seed(0)
    w = torch.randn(48, 256) * 0.1
    t = q4.pack_gptq(w, 64)
    assert t["qweight"].shape == (32, 48) and t["qzeros"].shape == (4, 6) and t["qweight"].dtype == torch.int32
    got = q4.unpack_gptq(t["qweight"], t["qzeros"], t["scales"], t["g_idx"])
    assert torch.allclose(got, _lattice(w, 64), atol=1e-6)
    assert float((got - w).abs().max()) < 0.05
    t = q4.pack_gptq(w, 64, act_order=True)
    perm = torch.randperm(256, generator=torch.Generator().manual_seed(256))
    got = q4.unpack_auto(t["qweight"], t["qzeros"], t["scales"], t["g_idx"])
    assert torch.allclose(got, _lattice(w, 64, perm), atol=1e-6)


def test_awq_roundtrip_and_layout_detection():
    torch.manual_seed(1)
    w = torch.randn(64, 128) * 0.1
    t = q4.pack_awq(w, 32)
    assert t["qweight"].shape == (128, 8) and t["qzeros"].shape == (4, 8)
    got = q4.unpack_auto(t["qweight"], t["qzeros"], t["scales"])
    assert torch.allclose(got, _lattice(w, 32), atol=1e-6)
    # nibble order: nibble 1 of the first word holds column 2
    qk, _, _ = q4.quantize_levels(w, 32)
    assert int((t["qweight"][0, 0] >> 4) & 15) == int(qk[0, 2])


def test_native_format_reproduces_a_checkpoint_lattice():
    torch.manual_seed(2)
    w = torch.randn(32, 256) * 0.1
    dense = _lattice(w, 128)                               # what a GPTQ / AWQ checkpoint holds
    packed, scale, zs = ref.quant_w4(dense, 128)
    assert packed.dtype == torch.uint8 and packed.shape == (32, 128) and scale.shape == (32, 2)
    back = ref.dequant_w4(packed, scale, zs)
    assert float((back - dense).abs().max()) < 2e-3         # only the bf16 rounding of scale / zero*scale
    x = torch.randn(5, 256)
    y = linear(x, LinearWeight(w=dense.clone()).quantize_w4(128))
    assert float((y - x @ dense.t()).abs().max()) < 2e-2


def test_gptq_checkpoint_runs_end_to_end():
    """A tiny Llama whose projections are stored GPTQ-style: logits match the model built from the dequantised
    weights, in 4-bit mode (the default for such checkpoints) and when the weights are served as dense."""
    cfg = ModelConfig(model_type="llama", hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
                      intermediate_size=256, vocab_size=300, max_position_embeddings=128, max_token_len=128)
    rnd = RandomSource(seed=3, std=0.08)
    dense, packed = {}, {}
    H, D = 128, 32
    shapes = {"self_attn.q_proj": (4 * D, H), "self_attn.k_proj": (2 * D, H), "self_attn.v_proj": (2 * D, H),
              "self_attn.o_proj": (H, 4 * D), "mlp.gate_proj": (256, H), "mlp.up_proj": (256, H), "mlp.down_proj": (H, 256)}
    for l in range(2):
        for n, shp in shapes.items():
            name = f"model.layers.{l}.{n}"
            w = rnd.get(name + ".weight", shp)
            t = q4.pack_gptq(w, 64) if l == 0 else q4.pack_awq(w, 64)
            for k, v in t.items():
                packed[f"{name}.{k}"] = v
            dense[name + ".weight"] = q4.unpack_auto(t["qweight"], t["qzeros"], t["scales"], t.get("g_idx"))
        for n in ("input_layernorm", "post_attention_layernorm"):
            dense[f"model.layers.{l}.{n}.weight"] = packed[f"model.layers.{l}.{n}.weight"] = torch.ones(H)
    for n, shp in (("model.embed_tokens.weight", (300, H)), ("lm_head.weight", (300, H))):
        dense[n] = packed[n] = rnd.get(n, shp)
    dense["model.norm.weight"] = packed["model.norm.weight"] = torch.ones(H)
    src = DictSource(packed)
    assert src.has("model.layers.0.self_attn.q_proj.weight") and not src._has_raw("model.layers.0.self_attn.q_proj.weight")
    from ksanallm_b200.models.common import StepInput
    m_ref = build_model(cfg, DictSource(dense), device="cpu", dtype=torch.float32)
    m_4 = build_model(cfg, src, device="cpu", dtype=torch.float32, quant="w4a16:64")
    m_d = build_model(cfg, src, device="cpu", dtype=torch.float32)
    assert m_4.layers[0].qkv.w4a16 and m_4.layers[1].down.w4a16 and not m_d.layers[0].qkv.w4a16
    T = 9
    outs = []
    for m in (m_ref, m_4, m_d):
        m.allocate_kv_cache(4, 16)
        step = StepInput(torch.arange(T, dtype=torch.int32) + 5, torch.arange(T, dtype=torch.int32),
                         torch.arange(T, dtype=torch.int32), torch.tensor([0, T], dtype=torch.int32),
                         torch.tensor([T], dtype=torch.int32), torch.tensor([[0, 1, 2, 3]], dtype=torch.int32),
                         num_multi=1, num_single=0, num_tokens=T, num_multi_tokens=T, max_q_len=T)
        outs.append(m.forward(step))
    assert float((outs[2] - outs[0]).abs().max()) < 1e-4
    assert float((outs[1] - outs[0]).norm() / outs[0].norm()) < 2e-2
