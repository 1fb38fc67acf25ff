"""The CPU end-to-end slice: a tiny Llama through the real engine (C++ scheduler, paged KV, model
definition, sampler) on fp32 reference ops, checked against a plain PyTorch forward."""
import math

import pytest
import torch

from ksanallm_b200.config import EngineConfig, ModelConfig
from ksanallm_b200.models.weights import RandomSource, build_model
from ksanallm_b200.runtime.engine import LLMEngine
from ksanallm_b200.utils import native_engine as ne


def tiny_cfg(**kw):
    c = ModelConfig(model_type="llama", hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                    intermediate_size=688, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0,
                    max_position_embeddings=512, max_token_len=512)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def plain_forward(cfg, src, tokens):
    """Independent restatement: dense causal attention over the full sequence, fp32."""
    H, D, Hq, Hkv = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    g = lambda n, s: src.get(n, s).float()
    x = g("model.embed_tokens.weight", (cfg.vocab_size, H))[tokens]
    T = len(tokens)
    pos = torch.arange(T)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2).float() / D))
    ang = torch.outer(pos.float(), inv)
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rope(t):
        a, b = t[..., : D // 2], t[..., D // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    def rms(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    for l in range(cfg.num_layers):
        p = f"model.layers.{l}."
        hn = rms(x, g(p + "input_layernorm.weight", (H,)) * 0 + 1)
        q = (hn @ g(p + "self_attn.q_proj.weight", (Hq * D, H)).t()).view(T, Hq, D)
        k = (hn @ g(p + "self_attn.k_proj.weight", (Hkv * D, H)).t()).view(T, Hkv, D)
        v = (hn @ g(p + "self_attn.v_proj.weight", (Hkv * D, H)).t()).view(T, Hkv, D)
        q, k = rope(q), rope(k)
        k = k.repeat_interleave(Hq // Hkv, 1)
        v = v.repeat_interleave(Hq // Hkv, 1)
        att = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        att = att.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hqk,khd->qhd", att.softmax(-1), v).reshape(T, Hq * D)
        x = x + o @ g(p + "self_attn.o_proj.weight", (H, Hq * D)).t()
        hn = rms(x, torch.ones(H))
        gate = hn @ g(p + "mlp.gate_proj.weight", (cfg.intermediate_size, H)).t()
        up = hn @ g(p + "mlp.up_proj.weight", (cfg.intermediate_size, H)).t()
        x = x + (torch.nn.functional.silu(gate) * up) @ g(p + "mlp.down_proj.weight", (H, cfg.intermediate_size)).t()
    x = rms(x, torch.ones(H))
    return x @ g("lm_head.weight", (cfg.vocab_size, H)).t()


def make_engine(cfg, src, num_blocks=64, **sched):
    model = build_model(cfg, src, device="cpu", dtype=torch.float32)
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size = 8
    ec.batch_scheduler.max_token_len = 256
    for k, v in sched.items():
        setattr(ec.batch_scheduler, k, v)
    return LLMEngine(model, cfg, ec, num_blocks=num_blocks, num_host_blocks=32)


def greedy(max_new):
    s = ne.SamplingConfig()
    s.max_new_tokens = max_new
    s.ignore_eos = True
    return s


def test_tiny_llama_matches_plain_pytorch():
    cfg, src = tiny_cfg(), RandomSource(seed=0)
    eng = make_engine(cfg, src)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 32000, (16,), generator=g).tolist() for _ in range(4)]
    captured = []
    eng.step_hook = lambda plan, logits: captured.append(logits.clone())
    reqs = eng.generate(prompts, greedy(8))
    for r, p in zip(reqs, prompts):
        assert r.status_code == 0 and len(r.outputs[0].tokens) == 8
        toks = list(p)
        for t in r.outputs[0].tokens:
            want = plain_forward(cfg, src, toks)[-1]
            assert int(want.argmax()) == t
            toks.append(t)
    # first step = prefill of all four prompts: logits of the last prompt tokens match
    want0 = torch.stack([plain_forward(cfg, src, p)[-1] for p in prompts])
    assert torch.allclose(captured[0], want0, atol=2e-4, rtol=1e-3)


@pytest.mark.parametrize("split_fuse,prefix", [(0, False), (32, False), (0, True), (16, True)])
def test_chunked_prefill_and_prefix_cache_equal_plain(split_fuse, prefix):
    cfg, src = tiny_cfg(), RandomSource(seed=1)
    eng = make_engine(cfg, src, split_fuse_token_num=split_fuse, enable_auto_prefix_cache=prefix)
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 32000, (40,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 32000, (7 + i,), generator=g).tolist() for i in range(3)]
    first = eng.generate(prompts[:1], greedy(4))[0]
    rest = eng.generate(prompts[1:], greedy(4))
    for r, p in zip([first] + rest, prompts):
        toks = list(p)
        for t in r.outputs[0].tokens:
            assert int(plain_forward(cfg, src, toks)[-1].argmax()) == t
            toks.append(t)
    st = eng.scheduler.stats()
    if prefix:
        assert st["prefix_hit_tokens"] >= 2 * 32
    assert eng.scheduler.check_invariants()[0]


def test_nvfp4_weights_cpu():
    """NVFP4 weight mode end to end on the CPU statement: runs, and stays close to the bf16 model's logits."""
    import torch
    from ksanallm_b200.config import ModelConfig
    from ksanallm_b200.models.weights import RandomSource, build_model
    from ksanallm_b200.ops.dispatch import LinearWeight, linear
    cfg = ModelConfig(model_type="llama", hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                      intermediate_size=512, vocab_size=500, max_position_embeddings=128, max_token_len=128)
    src = RandomSource(seed=0, std=0.05)
    m4 = build_model(cfg, src, device="cpu", dtype=torch.float32, quant="nvfp4")
    assert m4.layers[0].qkv.nvfp4 and m4.layers[0].down.nvfp4
    x = torch.randn(5, 256)
    W = LinearWeight(w=torch.randn(64, 256) * 0.05)
    want = x @ W.w.t()
    got = linear(x, LinearWeight(w=W.w.clone()).quantize_nvfp4())
    assert float((got - want).norm() / want.norm()) < 0.2


def test_embedding_table_on_the_host_gives_the_same_tokens():
    """embed_tokens_use_cpu keeps the table in host memory; only the looked-up rows reach the model's device."""
    import torch
    from helpers import tiny_model_cfg
    from ksanallm_b200.config import EngineConfig
    from ksanallm_b200.llm import LLM
    from ksanallm_b200.utils import native_engine as ne
    outs = []
    for on_host in (False, True):
        ec = EngineConfig()
        ec.global_.embed_tokens_use_cpu = on_host
        ec.batch_scheduler.max_token_len = 64
        ec.block_manager.device_blocks_num = 32
        llm = LLM(ec, tiny_model_cfg(), weights="random", device="cpu", dtype=torch.float32)
        s = ne.SamplingConfig()
        s.max_new_tokens, s.ignore_eos = 5, True
        outs.append([r.outputs[0].tokens for r in llm.generate([[5, 6, 7, 8], [9, 10]], s)])
    assert outs[0] == outs[1]


def test_offline_example_script_runs():
    """examples/offline_generate.py (random weights, public API) runs on a machine without a GPU and prints two
    continuations of sixteen tokens."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "offline_generate.py")], capture_output=True, text=True,
                       timeout=300, env=dict(os.environ, PYTHONPATH=root, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    lines = [l for l in r.stdout.splitlines() if "->" in l]
    assert len(lines) == 2 and all(len(l.split("->")[1].split(",")) == 16 for l in lines)
