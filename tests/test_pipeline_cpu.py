"""Pipeline parallelism on CPU ranks (gloo): stage layer ranges, micro-batch splitting, and the whole engine over
2 and 3 stages (and 2 stages x 2 tensor-parallel ranks) against a single-process run."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from ksanallm_b200.parallel.pipeline import split_sequences, stage_layers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_stage_layers_quotient_remainder():
    assert [stage_layers(80, 4, r) for r in range(4)] == [(0, 19), (20, 39), (40, 59), (60, 79)]
    assert [stage_layers(5, 3, r) for r in range(3)] == [(0, 1), (2, 3), (4, 4)]
    with pytest.raises(ValueError):
        stage_layers(2, 3, 2)


def test_split_sequences_balances_tokens():
    q = np.array([70, 5, 33, 128, 1, 1])
    parts = split_sequences(q, 2)
    assert parts[0][0] == 0 and parts[-1][1] == 6 and all(a < b for a, b in parts)
    assert [b for _, b in parts[:-1]] == [a for a, _ in parts[1:]]
    assert split_sequences(np.array([4]), 3) == [(0, 1)]
    assert split_sequences(np.array([], dtype=np.int64), 2) == []
    assert len(split_sequences(np.ones(8, dtype=np.int64), 4)) == 4


def _launch(nproc, out, pp, mb, port, **env):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "pp_worker.py"), out, "cpu", str(pp), str(mb)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="1", **env))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return torch.load(out)


def _single():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from pp_worker import model_cfg, prompts_for
    from ksanallm_b200.config import EngineConfig
    from ksanallm_b200.models.weights import RandomSource, build_model
    from ksanallm_b200.runtime.engine import LLMEngine
    from ksanallm_b200.utils import native_engine as ne
    mc = model_cfg("cpu")
    model = build_model(mc, RandomSource(seed=11, std=0.2), device="cpu", dtype=torch.float32)
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size = 8
    ec.batch_scheduler.max_token_len = 300
    ec.batch_scheduler.max_step_tokens = 512
    eng = LLMEngine(model, mc, ec, num_blocks=128)
    first = {}

    def hook(plan, lg):
        for i, sid in enumerate(plan.sample_seq_ids.tolist()):
            first.setdefault(sid, lg[i].float().clone())

    eng.step_hook = hook
    s = ne.SamplingConfig()
    s.max_new_tokens, s.ignore_eos = 5, True
    reqs = eng.generate(prompts_for(mc.vocab_size), s)
    return [r.outputs[0].tokens for r in reqs], torch.stack([first[k] for k in sorted(first)])


@pytest.mark.parametrize("nproc,pp,mb,port", [(2, 2, 2, 29711), (3, 3, 3, 29712), (4, 2, 1, 29713)])
def test_pipeline_matches_single_process(tmp_path, nproc, pp, mb, port):
    want_tokens, want_first = _single()
    got = _launch(nproc, str(tmp_path / "pp.pt"), pp, mb, port)
    assert got["layers"][0] == 0 and got["layers"][1] < 4            # rank 0 holds only the first layers
    assert got["sent_bytes"] > 0
    assert float((got["first"] - want_first).abs().max()) < 1e-3
    assert got["tokens"] == want_tokens


@pytest.mark.parametrize("nproc,pp,mb,port", [(2, 2, 2, 29714), (4, 2, 2, 29715)])
def test_request_targets_over_pipeline_stages(tmp_path, nproc, pp, mb, port):
    """/forward style targets under pipeline (and pipeline x tensor) parallelism: the last stage owns the final
    hidden states and the lm_head, rank 0 answers the request - same tensors as one process."""
    import copy
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from pp_worker import TARGETS, model_cfg, prompts_for, refit_for
    from ksanallm_b200.config import EngineConfig
    from ksanallm_b200.models.weights import RandomSource, build_model
    from ksanallm_b200.runtime.engine import LLMEngine
    from ksanallm_b200.utils import native_engine as ne
    mc = model_cfg("cpu")
    model = build_model(mc, RandomSource(seed=11, std=0.2), device="cpu", dtype=torch.float32)
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size, ec.batch_scheduler.max_token_len, ec.batch_scheduler.max_step_tokens = 8, 300, 512
    eng = LLMEngine(model, mc, ec, num_blocks=128)
    s = ne.SamplingConfig()
    s.max_new_tokens = 1
    want = [eng.add_request(p, s, request_target=copy.deepcopy(TARGETS)) for p in prompts_for(mc.vocab_size)[2:]]
    want.append(eng.add_request(prompts_for(mc.vocab_size)[2], s, request_target=copy.deepcopy(TARGETS), refit=refit_for(mc)))
    while not all(r.done.is_set() for r in want):
        eng.step()
    got = _launch(nproc, str(tmp_path / "pp.pt"), pp, mb, port, PP_TARGETS="1")["targets"]
    assert len(got) == len(want) == 3
    # the spliced embeddings change the states of the third request (same prompt as the first)
    assert float((want[2].response["transformer"] - want[0].response["transformer"]).abs().max()) > 1e-2
    for g, w in zip(got, want):
        assert set(g) == set(w.response) == set(TARGETS)
        assert g["transformer"].shape == (4, mc.hidden_size) and g["logits"].shape == (11,)
        for k in TARGETS:
            assert float((g[k] - w.response[k]).abs().max()) < 1e-3, k



def test_families_over_pipeline_stages(tmp_path):
    """Every model family split into two pipeline stages (CPU ranks, gloo) through the public API: the greedy
    continuations equal Hugging Face's own generation from the same tiny models (embedding kinds, final norms, dense
    and routed layers, latent attention each land on the stage that needs them)."""
    import json
    import socket
    pytest.importorskip("transformers")
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
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(here, "pp_families_worker.py"), str(out), "2",
                        names], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = json.loads(out.read_text())
    assert set(res) == set(names.split(","))
    for name, v in res.items():
        assert v["ok"], (name, v)
