"""Attention data parallelism + expert parallelism on CPU ranks (gloo) against a single-process run."""
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from ksanallm_b200.parallel.data_parallel import AttentionDP

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sub_plan_selects_own_sequences():
    plan = SimpleNamespace(seq_ids=np.array([4, 7, 9, 10, 12]), cu_q=np.array([0, 3, 8, 9, 10, 11]),
                           kv_lens=np.array([3, 20, 31, 5, 8]), input_ids=np.arange(11) + 100, positions=np.arange(11),
                           slots=np.arange(11) + 50, block_table=np.arange(10), max_blocks=2,
                           sample_rows=np.array([2, 7, 8, 9, 10]), sample_seq_ids=np.array([4, 7, 9, 10, 12]),
                           num_multi=2, num_single=3, num_tokens=11, num_multi_tokens=8, max_q_len=5,
                           swap_out=np.zeros(0), swap_in=np.zeros(0), copies=np.zeros(0))
    dp = AttentionDP(rank=0, size=2)
    sub = dp.sub_plan(plan)                      # even sequence ids: 4, 10, 12
    assert dp.counts == [5, 6]
    assert sub.seq_ids.tolist() == [4, 10, 12] and sub.cu_q.tolist() == [0, 3, 4, 5]
    assert sub.input_ids.tolist() == [100, 101, 102, 109, 110] and sub.kv_lens.tolist() == [3, 5, 8]
    assert sub.block_table.tolist() == [0, 1, 6, 7, 8, 9]
    assert (sub.num_multi, sub.num_single, sub.num_multi_tokens, sub.max_q_len) == (1, 2, 3, 3)
    assert sub.sample_rows.tolist() == [2, 3, 4]
    sub1 = AttentionDP(rank=1, size=2).sub_plan(plan)
    assert sub1.seq_ids.tolist() == [7, 9] and sub1.sample_rows.tolist() == [4, 5] and sub1.num_multi == 1


def _single(new_tokens=5, n=0):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from dp_worker import engine_cfg, model_cfg, prompts_for
    from ksanallm_b200.models.weights import RandomSource, build_model
    from ksanallm_b200.runtime.engine import LLMEngine
    from ksanallm_b200.utils import native_engine as ne
    mc = model_cfg("cpu")
    model = build_model(mc, RandomSource(seed=11, std=0.2), device="cpu", dtype=torch.float32)
    eng = LLMEngine(model, mc, engine_cfg(), num_blocks=128)
    first = {}

    def hook(plan, lg):
        for i, sid in enumerate(plan.sample_seq_ids.tolist()):
            first.setdefault(sid, lg[i].float().clone())

    eng.step_hook = hook
    s = ne.SamplingConfig()
    s.max_new_tokens, s.ignore_eos = new_tokens, True
    if n:
        s.num_return_sequences, s.topk, s.temperature, s.seed = n, 20, 1.0, 1234
    reqs = eng.generate(prompts_for(mc.vocab_size), s)
    if n:
        return [[o.tokens for o in r.outputs] for r in reqs], None
    return [r.outputs[0].tokens for r in reqs], torch.stack([first[k] for k in sorted(first)])


@pytest.mark.parametrize("nproc,port,dispatch", [(2, 29721, "allgather"), (4, 29722, "allgather"),
                                                 (2, 29723, "alltoall"), (4, 29724, "alltoall")])
def test_attention_dp_matches_single_process(tmp_path, nproc, port, dispatch):
    """Attention data parallelism + expert parallelism on CPU ranks against one process, with both forms of the
    expert dispatch: all-gather of every rank's rows, and the all-to-all that sends a row only to the ranks holding
    one of its experts (fewer bytes received than with the all-gather)."""
    want_tokens, want_first = _single()
    out = str(tmp_path / "dp.pt")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "dp_worker.py"), out, "cpu"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, OMP_NUM_THREADS="1", KSANA_EP_DISPATCH=dispatch))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    assert got["experts"] == (0, 8 // nproc)                    # rank 0 holds whole experts, a 1/nproc share
    assert got["gathered_bytes"] > 0
    if dispatch == "alltoall":
        assert got["dispatched_rows"] > 0

    assert float((got["first"] - want_first).abs().max()) < 1e-3
    assert got["tokens"] == want_tokens


@pytest.mark.parametrize("blocks,host", [(12, 0), (8, 32)])
def test_attention_dp_ranks_pool_their_caches(tmp_path, blocks, host):
    """Two ranks with `blocks` KV blocks each: together they hold what one pool of that size cannot (12 blocks: no
    preemption although the five sequences need 14); the results stay those of the single process. With 8 blocks per
    rank and a host pool the ranks swap: every rank executes only its own pool's entries of the plan's swap lists
    (device blocks are written as rank * blocks_per_rank + block there), and the tokens still match."""
    new_tokens = 40 if host else 5
    want_tokens, want_first = _single(new_tokens)
    out = str(tmp_path / "dp.pt")
    env = dict(os.environ, OMP_NUM_THREADS="1", KSANA_TEST_DP_BLOCKS=str(blocks), KSANA_TEST_DP_NEW=str(new_tokens))
    if host:
        env["KSANA_TEST_DP_HOST_BLOCKS"] = str(host)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29671 + blocks), os.path.join(ROOT, "tests", "dp_worker.py"), out, "cpu"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    assert got["tokens"] == want_tokens
    assert got["refused"] == (1, True)
    st = got["stats"]
    if host:
        assert st["preempt_swap"] > 0 and st["swap_in"] > 0
    else:
        assert st["preempt_swap"] == 0 and st["preempt_recompute"] == 0


def test_alltoall_dispatch_moves_fewer_rows_than_allgather(tmp_path):
    """Four CPU ranks, top-2 of 8 experts (two experts per rank): with the all-to-all a row reaches at most two
    ranks, with the all-gather every rank receives every row; same tokens either way."""
    res = {}
    for i, dispatch in enumerate(("allgather", "alltoall")):
        out = str(tmp_path / f"dp_{dispatch}.pt")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
               "127.0.0.1", "--master-port", str(29731 + i), os.path.join(ROOT, "tests", "dp_worker.py"), out, "cpu"]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=300,
                           env=dict(os.environ, OMP_NUM_THREADS="1", KSANA_EP_DISPATCH=dispatch))
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        res[dispatch] = torch.load(out)
    assert res["alltoall"]["tokens"] == res["allgather"]["tokens"]
    assert 0 < res["alltoall"]["gathered_bytes"] < 0.75 * res["allgather"]["gathered_bytes"]


def test_attention_dp_with_sampled_siblings(tmp_path):
    """Three sampled sequences per request (fixed seed) under attention data parallelism: siblings fork from their
    request's prompt blocks by copy-on-write inside one rank's pool, every rank runs only its own pool's copies, and
    all fifteen continuations equal those of the single process."""
    want, _ = _single(12, n=3)
    assert all(len(w) == 3 and len(set(map(tuple, w))) > 1 for w in want)          # siblings do differ
    out = str(tmp_path / "dp.pt")
    env = dict(os.environ, OMP_NUM_THREADS="1", KSANA_TEST_DP_NEW="12", KSANA_TEST_DP_N="3")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29731", os.path.join(ROOT, "tests", "dp_worker.py"), out, "cpu"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    got = torch.load(out)
    assert got["all_tokens"] == want
