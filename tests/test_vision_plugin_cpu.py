"""Qwen2-VL style vision plug-in: tower shapes, multimodal rotary positions, and a request with an image through
the serving model (embeddings spliced at the image tokens, mrope positions used by the model)."""
import torch

from helpers import ByteTokenizer, tiny_model_cfg
from ksanallm_b200.ksana_plugin.qwen2_vl.ksana_plugin import KsanaPlugin, VisionTower, mrope_positions

PAD = 290


def test_tower_and_positions():
    tower = VisionTower(hidden_out=64, dim=32, depth=1, heads=2, patch=14, merge=2)
    emb, grids = tower([torch.rand(3, 56, 84), torch.rand(2, 3, 28, 28)])
    assert grids == [(1, 4, 6), (2, 2, 2)] and emb.shape == (1 * 2 * 3 + 2 * 1 * 1, 64)
    # frames do not attend to each other: the second image's embeddings do not depend on the first image
    emb2, _ = tower([torch.rand(3, 56, 84), torch.rand(2, 3, 28, 28)])
    assert emb2.shape == emb.shape
    toks = [5, 6] + [PAD] * 6 + [7, 8]
    pos = mrope_positions(toks, PAD, [(1, 4, 6)], 2)
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6                        # one frame
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8].tolist() == [5, 5, 5] and pos[:, 9].tolist() == [6, 6, 6]   # text resumes after max(f, h, w) = 3


def test_image_request_through_serving_model(tmp_path):
    from ksanallm_b200.config import EngineConfig
    from ksanallm_b200.llm import LLM
    from ksanallm_b200.serving.plugin import KsanaPlugin as PluginHost, PluginConfig
    from ksanallm_b200.serving.serving_model import ServingModel
    tok = ByteTokenizer()
    cfg = tiny_model_cfg(vocab=300, model_type="qwen2_vl", position_embedding="mrope", mrope_section=[2, 3, 3], qkv_bias=True)
    ec = EngineConfig()
    ec.batch_scheduler.max_token_len = 128
    ec.block_manager.device_blocks_num = 64
    llm = LLM(ec, cfg, weights="random", device="cpu", dtype=torch.float32, tokenizer=tok)
    model = ServingModel("", llm=llm, tokenizer=tok)
    model.init_serving()
    host = PluginHost(PluginConfig(model_dir=str(tmp_path), plugin_name="qwen2_vl"))
    assert host.loaded
    host._plugin.init_plugin(model_path="", hidden_size=cfg.hidden_size, image_token_id=PAD)
    model.plugin = host
    img = torch.rand(3, 28, 56, generator=torch.Generator().manual_seed(1))
    prompt = [1, 20, PAD, 21, 22]
    gen = {"max_new_tokens": 4, "ignore_eos": True}
    st, out = model.generate(inputs=list(prompt), generation_config=gen, additional_params={"images": [img]})
    assert st.OK()
    assert out.input_tokens == [1, 20, PAD, PAD, 21, 22] and len(out.output_tokens[0]) == 4     # 1x2 merged patches
    # the picture matters: another image changes the continuation's logits path (same tokens, other embeddings)
    seen = []
    # prefill steps only: the hook of a request's last decode step may still run after generate() has returned
    llm.engine.step_hook = lambda plan, lg: seen.append(lg.float().clone()) if plan.num_multi else None
    model.generate(inputs=list(prompt), generation_config=gen, additional_params={"images": [img]})
    a = seen[0]
    seen.clear()
    model.generate(inputs=list(prompt), generation_config=gen, additional_params={"images": [1.0 - img]})
    assert float((seen[0] - a).abs().max()) > 1e-4
    seen.clear()
    model.generate(inputs=list(prompt), generation_config=gen, additional_params={"images": [img]})
    assert torch.allclose(seen[0], a, atol=1e-5)
    model.shutdown()
