"""Qwen2-VL style vision plug-in: tower shapes, multimodal rotary positions, and a request with an image through
the serving model (embeddings spliced at the image tokens, mrope positions used by the model)."""
import torch

from helpers import ByteTokenizer, tiny_model_cfg
from ksanallm_b200.ksana_plugin.qwen2_vl.ksana_plugin import KsanaPlugin, VisionTower, mrope_positions

PAD = 290


def test_tower_and_positions():
    tower = VisionTower(hidden_out=64, dim=32, depth=1, heads=2, patch=14, merge=2)
    clip = torch.rand(4, 3, 28, 28)
    emb, grids = tower([torch.rand(3, 56, 84), clip])
    # a still image is one temporal patch (its own second frame); four frames are two temporal patches
    assert grids == [(1, 4, 6), (2, 2, 2)] and emb.shape == (1 * 2 * 3 + 2 * 1 * 1, 64)
    # images do not attend to each other: the clip's embeddings do not depend on the first image
    emb2, _ = tower([torch.rand(3, 56, 84), clip])
    assert emb2.shape == emb.shape and torch.allclose(emb2[6:], emb[6:], atol=1e-5)
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


def test_tower_matches_hugging_face_visual():
    """The tower loads the checkpoint's ``visual.*`` tensors by name and reproduces the Hugging Face Qwen2-VL vision
    transformer: same flattened patches in, same merged embeddings out."""
    import pytest
    transformers = pytest.importorskip("transformers")
    from transformers.models.qwen2_vl import modeling_qwen2_vl as hf
    from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig
    vc = Qwen2VLVisionConfig(depth=2, embed_dim=32, hidden_size=48, num_heads=4, mlp_ratio=4, patch_size=14,
                             spatial_merge_size=2, temporal_patch_size=2, in_channels=3)
    ref = hf.Qwen2VisionTransformerPretrainedModel(vc).eval()
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.05 if p.dim() > 1 else 0.1) + (1.0 if p.dim() == 1 and p.shape[0] == 32 else 0.0))
    tower = VisionTower(hidden_out=48, dim=32, depth=2, heads=4, patch=14, merge=2, temporal=2, mlp_ratio=4).eval()
    missing, unexpected = tower.load_state_dict(ref.state_dict(), strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    images = [torch.rand(3, 56, 84, generator=g), torch.rand(4, 3, 28, 56, generator=g)]
    flat, grids = tower.patchify(images)
    with torch.no_grad():
        got = tower.forward_patches(flat, grids)
        want = ref(flat, grid_thw=torch.tensor(grids)).pooler_output
    assert got.shape == want.shape
    assert float((got - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max()))


def test_mrope_positions_match_hugging_face_rope_index():
    import pytest
    pytest.importorskip("transformers")
    from transformers import Qwen2VLConfig
    from transformers.models.qwen2_vl import modeling_qwen2_vl as hf
    cfg = Qwen2VLConfig(
        text_config=dict(hidden_size=32, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2, intermediate_size=64,
                         vocab_size=400, rope_parameters={"rope_type": "default", "mrope_section": [2, 3, 3], "rope_theta": 10000.0}),
        vision_config=dict(depth=1, embed_dim=16, hidden_size=32, num_heads=2, patch_size=14, spatial_merge_size=2,
                           temporal_patch_size=2),
        image_token_id=PAD, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    model = hf.Qwen2VLModel(cfg)
    toks = [5, 6, 292] + [PAD] * 6 + [293, 7, 8, 292] + [PAD] * 4 + [293, 9]
    ids = torch.tensor([toks])
    kinds = torch.tensor([[1 if t == PAD else 0 for t in toks]], dtype=torch.int32)
    try:
        want, _ = model.get_rope_index(ids, kinds, image_grid_thw=torch.tensor([[1, 4, 6], [1, 4, 4]]),
                                       attention_mask=torch.ones_like(ids))
    except TypeError:
        pytest.skip("this transformers version has another get_rope_index signature")
    got = mrope_positions(toks, PAD, [(1, 4, 6), (1, 4, 4)], 2)
    assert torch.equal(want[:, 0].to(torch.int32), got)


def test_qwen_vl_first_generation_tower_and_spans():
    """First-generation Qwen-VL: the tower's parameters carry the checkpoint's names, a picture of any size becomes a
    fixed number of embeddings, and the <img>path</img> spans of the token stream are found and filled."""
    from ksanallm_b200.ksana_plugin.qwen_vl.ksana_plugin import KsanaPlugin as QwenVLPlugin, VisionTower as Tower1, image_spans
    from ksanallm_b200.ksana_plugin.qwen_vl.ksana_plugin import resize_positions, sincos_2d
    tower = Tower1(image_size=56, patch=14, width=32, depth=1, heads=2, mlp_ratio=2.0, queries=4, out_dim=128, trained_grid=2).eval()
    names = set(tower.state_dict().keys())
    expected = {"conv1.weight", "positional_embedding", "ln_pre.weight", "ln_pre.bias", "proj", "ln_post.weight", "ln_post.bias",
                "attn_pool.pos_embed", "attn_pool.query", "attn_pool.kv_proj.weight", "attn_pool.attn.in_proj_weight",
                "attn_pool.attn.in_proj_bias", "attn_pool.attn.out_proj.weight", "attn_pool.attn.out_proj.bias",
                "attn_pool.ln_q.weight", "attn_pool.ln_q.bias", "attn_pool.ln_kv.weight", "attn_pool.ln_kv.bias"}
    expected |= {f"transformer.resblocks.0.{n}" for n in (
        "ln_1.weight", "ln_1.bias", "ln_2.weight", "ln_2.bias", "attn.in_proj.weight", "attn.in_proj.bias",
        "attn.out_proj.weight", "attn.out_proj.bias", "mlp.c_fc.weight", "mlp.c_fc.bias", "mlp.c_proj.weight", "mlp.c_proj.bias")}
    assert names == expected
    g = torch.Generator().manual_seed(0)
    img = torch.rand(3, 40, 70, generator=g)
    px = tower.preprocess(img)
    assert px.shape == (3, 56, 56)
    out = tower(torch.stack([px, tower.preprocess(1.0 - img)]))
    assert out.shape == (2, 4, 128) and float((out[0] - out[1]).abs().max()) > 1e-6
    # position tables: identity when the grid matches, smooth resize otherwise; sine/cosine table is bounded
    t = torch.arange(8.0).view(4, 2)
    assert torch.equal(resize_positions(t, 4), t) and resize_positions(t, 16).shape == (16, 2)
    assert sincos_2d(16, 3).shape == (9, 16) and float(sincos_2d(16, 3).abs().max()) <= 1.0
    # spans: <img> = 500, </img> = 501, pad = 502; the path is spelled in bytes
    path = "a/b.pt"
    toks = [1, 2, 500] + list(path.encode()) + [502] * (6 - len(path)) + [501, 9, 500] + list(b"zz") + [502, 502, 502, 502] + [501]
    spans = image_spans(toks, 500)
    assert [(p, n, s) for p, n, s in spans] == [(3, 6, path), (12, 6, "zz")]
    plugin = QwenVLPlugin()
    plugin.init_plugin(model_path="", visual={"image_start_id": 500, "image_size": 56, "width": 32, "layers": 1, "heads": 2,
                                              "mlp_ratio": 2.0, "n_queries": 4, "output_dim": 128})
    plugin.tower.float().cpu()
    inp = {"input_tokens": toks}
    plugin.preprocess(ksana_python_input=inp, additional_params={"images": [img, 1.0 - img]})
    assert inp["input_refit_embedding"]["pos"] == [3, 12]
    assert [tuple(e.shape) for e in inp["input_refit_embedding"]["embeddings"]] == [(4, 128), (4, 128)]


def test_plugin_written_for_the_reference_loads_unchanged(tmp_path):
    """A plug-in in the reference's style: it imports ``plugin_utils`` as a top-level module, a neighbour module by its
    folder name, expects ``config_file`` among the arguments of ``init_plugin`` and raises the reserved memory share in
    that YAML, and rewrites the request through attributes of the input object (tokens, spliced embeddings as
    tensors). The host loads it, runs pre- and post-processing on its pool, and a broken plug-in only costs a warning."""
    from ksanallm_b200.serving.plugin import KsanaPlugin as PluginHost, PluginConfig
    pkg = tmp_path / "plugins" / "my_vl"
    pkg.mkdir(parents=True)
    (pkg / "tower_model.py").write_text("SCALE = 3\n")
    (pkg / "ksana_plugin.py").write_text('''
import os, sys
from my_vl.tower_model import SCALE
from plugin_utils import adjust_device_memory_ratio, check_file_dir, free_cache


class KsanaPlugin:
    def init_plugin(self, **kwargs):
        self.seen = dict(kwargs)
        free_cache()
        adjust_device_memory_ratio(kwargs["config_file"], 0.04)

    def preprocess(self, **kwargs):
        import torch
        ksana_python_input = kwargs["ksana_python_input"]
        assert "messages" in kwargs and "additional_params" in kwargs and "prompt" in kwargs
        ksana_python_input.input_tokens = [t * SCALE for t in ksana_python_input.input_tokens]
        ksana_python_input.input_refit_embedding.pos = [1]
        ksana_python_input.input_refit_embedding.embedding_tensors = torch.unbind(torch.full((1, 2, 64), 0.25))

    def postprocess(self, **kwargs):
        kwargs["ksana_python_output"].output_tokens[0].append(4242)
''')
    yaml_path = tmp_path / "ksana_llm.yaml"
    yaml_path.write_text("setting:\n  block_manager:\n    # room for the tower\n    reserved_device_memory_ratio: 0.01   # share\n    block_token_num: 16\n")
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    (model_dir / "ksana_plugin.py").write_text((pkg / "ksana_plugin.py").read_text())
    import sys
    sys.path.append(str(tmp_path / "plugins"))            # where "my_vl" lives, as an installed plug-in package would
    try:
        host = PluginHost(PluginConfig(model_dir=str(model_dir), config_file=str(yaml_path), plugin_name="my_vl",
                                       thread_pool_size=2))
        assert host.loaded and host._plugin.seen["config_file"] == str(yaml_path) and host._plugin.seen["enable_trt"] is True
        text = yaml_path.read_text()
        assert "reserved_device_memory_ratio: 0.04   # share" in text and "# room for the tower" in text
        # through the serving model: the rewritten tokens and the spliced embeddings reach the engine, the answer
        # passes through the post-processing
        from ksanallm_b200.config import EngineConfig
        from ksanallm_b200.llm import LLM
        from ksanallm_b200.serving.serving_model import KsanaPythonInput, ServingModel
        from ksanallm_b200.utils import native_engine as ne
        inp = KsanaPythonInput([1, 2, 3])
        host.preprocess(ksana_python_input=inp, messages=None, additional_params={}, prompt="")
        assert inp.input_tokens == [3, 6, 9] and inp["input_tokens"] == [3, 6, 9] and inp.input_refit_embedding.pos == [1]
        ec = EngineConfig()
        ec.batch_scheduler.max_token_len = 64
        ec.block_manager.device_blocks_num = 32
        llm = LLM(ec, tiny_model_cfg(), weights="random", device="cpu", dtype=torch.float32, tokenizer=ByteTokenizer())
        model = ServingModel("", llm=llm, tokenizer=ByteTokenizer())
        model.init_serving()
        model.plugin = host
        try:
            st, out = model.generate(inputs=[1, 2, 3], generation_config={"max_new_tokens": 3, "ignore_eos": True})
            assert st.OK() and out.input_tokens == [3, 6, 9] and out.output_tokens[0][-1] == 4242
            s = ne.SamplingConfig()
            s.max_new_tokens, s.ignore_eos = 3, True
            want = llm.engine.add_request([3, 6, 9], s, refit=([1], [torch.full((2, 64), 0.25)]))
            assert want.done.wait(30) and out.output_tokens[0][:-1] == want.outputs[0].tokens
            plain = llm.engine.add_request([3, 6, 9], s)
            assert plain.done.wait(30)
            # a request that brings its own embeddings is not pre-processed again
            st, own = model.generate(inputs=[3, 6, 9], generation_config={"max_new_tokens": 3, "ignore_eos": True},
                                     input_refit_embedding={"pos": [1], "embeddings": [torch.full((2, 64), 0.25).tolist()]})
            assert st.OK() and own.input_tokens == [3, 6, 9] and own.output_tokens[0][:-1] == want.outputs[0].tokens
        finally:
            model.shutdown()
        # a larger value in the file is left alone; a plug-in that fails to import is skipped with a warning
        from ksanallm_b200.ksana_plugin.plugin_utils import adjust_device_memory_ratio
        assert adjust_device_memory_ratio(str(yaml_path), 0.02) is False
        (model_dir / "ksana_plugin.py").write_text("import module_that_does_not_exist\n")
        assert not PluginHost(PluginConfig(model_dir=str(model_dir), config_file=str(yaml_path))).loaded
    finally:
        sys.path.remove(str(tmp_path / "plugins"))
