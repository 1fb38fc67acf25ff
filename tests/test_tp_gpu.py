"""Tensor parallelism on 2+ GPUs: fused peer-memory path vs the NCCL path vs a single-GPU run."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(nproc, out, backend, quant, port, graphs=None, arch=None, **extra_env):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py"),
           out, backend, quant]
    if graphs is not None or arch is not None:
        cmd.append("graphs" if (graphs or graphs is None and backend == "fused") else "eager")
    if arch is not None:
        cmd.append(arch)
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=150)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return torch.load(out)


@pytest.mark.parametrize("push", ["0", "1"], ids=["pull", "epilogue-push"])
def test_peer_memory_primitives(tmp_path, push):
    """The peer-memory collectives and the fused row-parallel linear against NCCL / fp32 references; once with the
    reduce kernel pulling the partial rows from the peers and once with the GEMM epilogue pushing them (small batches:
    the default from four ranks on; large batches: KSANA_PUSH_PREFILL). One rank per visible GPU; on a one-GPU box
    the same kernels run as a group of one (flags raised to and awaited from the rank itself)."""
    out_dir = os.environ.get("KSANA_TP_LOG_DIR", str(tmp_path))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", KSANA_PUSH=push, KSANA_PUSH_PREFILL=push)
    n = min(torch.cuda.device_count(), 8)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", "29621", os.path.join(ROOT, "tests", "tp_comm_worker.py"), out_dir]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    logs = "".join(open(os.path.join(out_dir, f)).read() for f in sorted(os.listdir(out_dir)) if f.startswith("tp_comm_rank"))
    assert r.returncode == 0, logs + r.stdout[-2000:] + r.stderr[-3000:]
    assert "done" in logs


def rel(a, b):
    return float((a - b).norm() / b.norm())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("quant,tol", [("auto", 3e-2), ("fp8_block", 0.15)])
def test_tp2_fused_matches_nccl_and_single(tmp_path, quant, tol):
    n = 2
    single = _launch(1, str(tmp_path / "single.pt"), "nccl", quant, 29631)
    nccl = _launch(n, str(tmp_path / "nccl.pt"), "nccl", quant, 29632)
    eager = _launch(n, str(tmp_path / "fused_eager.pt"), "fused", quant, 29634, graphs=False)
    assert rel(nccl["first"], single["first"]) < tol
    assert rel(eager["first"], single["first"]) < tol      # (later logits depend on the tokens each run sampled)
    fused = _launch(n, str(tmp_path / "fused.pt"), "fused", quant, 29633)
    assert rel(fused["first"], single["first"]) < tol
    assert rel(fused["first"], nccl["first"]) < tol
    assert fused["graph_replays"] > 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("sampling", ["greedy", "topk"])
def test_tp2_shard_sampling_matches_whole_logits(tmp_path, sampling):
    """Vocabulary-sharded sampling: when nothing needs whole logits rows the ranks exchange each shard's top-k
    (value, token id) pairs and sample from the merged lists. The tokens (and top-N log-probs) are those of the run
    that gathers whole rows: same kernels up to the lm_head, exact merge, counter-based random draws."""
    n = 2
    env = {"KSANA_TP_SAMPLING": sampling}
    whole = _launch(n, str(tmp_path / "whole.pt"), "fused", "auto", 29681, **env)                      # the hook reads logits
    cand = _launch(n, str(tmp_path / "cand.pt"), "fused", "auto", 29682, KSANA_TP_TEST_NOHOOK="1", **env)
    assert cand["tokens"] == whole["tokens"]
    assert cand["graph_replays"] > 0
    if sampling == "topk":
        for a, b in zip(cand["logprobs"], whole["logprobs"]):
            assert [[t for t, _ in step] for step in a] == [[t for t, _ in step] for step in b]
            assert all(abs(x[1] - y[1]) < 1e-4 for sa, sb in zip(a, b) for x, y in zip(sa, sb))


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp4_fused(tmp_path):
    single = _launch(1, str(tmp_path / "single.pt"), "nccl", "auto", 29641)
    fused = _launch(4, str(tmp_path / "fused4.pt"), "fused", "auto", 29642)
    assert rel(fused["first"], single["first"]) < 3e-2


@pytest.fixture(scope="module")
def moe_single(tmp_path_factory):
    return _launch(1, str(tmp_path_factory.mktemp("moe") / "single.pt"), "nccl", "auto", 29651, arch="moe")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("arch", ["moe", "moe_ep"])
def test_tp2_moe_fused_combine(tmp_path, moe_single, arch):
    """MoE layers on the fused path: each rank's expert outputs are combined into its peer-visible slot and the
    cross-rank sum + residual + norm is the reduce kernel (experts sliced by tensor parallelism, or whole experts
    per rank with expert parallelism). Checked against a single-GPU run; the library-collective path of the same
    layouts is covered by the CPU (gloo) tests."""
    fused = _launch(2, str(tmp_path / "fused.pt"), "fused", "auto", 29653, arch=arch)
    rows = [rel(fused["first"][i], moe_single["first"][i]) for i in range(fused["first"].shape[0])]
    # bf16 partial sums of the sliced / distributed experts are rounded before the cross-rank reduction, and the
    # sharpened router amplifies small differences: measured 2 % (short prompts) to 6 % (long prompts) per row
    assert rel(fused["first"], moe_single["first"]) < 6e-2 and max(rows) < 0.1, rows
    assert fused["graph_replays"] > 0


def _launch_worker(script, nproc, out, port, *args):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", script), out, "cuda", *map(str, args)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return torch.load(out)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pipeline_two_stages_over_nccl_p2p(tmp_path):
    """Two pipeline stages on two GPUs (hidden states by NCCL send / recv, two micro-batches in flight)."""
    single = _launch_worker("pp_worker.py", 1, str(tmp_path / "single.pt"), 29661, 1, 1)
    pp = _launch_worker("pp_worker.py", 2, str(tmp_path / "pp.pt"), 29662, 2, 2)
    assert pp["layers"] == (0, 1) and pp["sent_bytes"] > 0
    assert rel(pp["first"], single["first"]) < 3e-2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_attention_dp_with_expert_parallel_over_nccl(tmp_path):
    """Sequences split over two GPUs, routed experts split over the same two (all-gather dispatch, reduce-scatter
    combine)."""
    single = _launch_worker("dp_worker.py", 1, str(tmp_path / "single.pt"), 29671)
    dp = _launch_worker("dp_worker.py", 2, str(tmp_path / "dp.pt"), 29672)
    assert dp["experts"] == (0, 4) and dp["gathered_bytes"] > 0 and not dp["peer_memory"]
    # bf16 activations: another batch split picks other GEMM tile shapes, and a router logit that moves by one bf16
    # step can flip a token's expert choice (measured 3-6 % over runs of the same layout)
    assert rel(dp["first"], single["first"]) < 8e-2
    # the same layout with dispatch and combine over peer memory (row pull + fused reduce / residual kernel)
    fused = _launch_worker("dp_worker.py", 2, str(tmp_path / "dpf.pt"), 29673, "fused")
    assert fused["peer_memory"] and fused["gathered_bytes"] > 0
    assert rel(fused["first"], single["first"]) < 8e-2
    assert rel(fused["first"], dp["first"]) < 8e-2
