"""Scheduler + cache manager simulation without any model: a fake token generator drives the real C++
scheduler (the idea of the reference's BlockManagerSimulator / BatchSchedulerEnvironmentSimulator tests,
src/ksana_llm/batch_scheduler/batch_scheduler_test.cpp:86-188)."""
import threading

import numpy as np
import pytest

from ksanallm_b200.utils import native_engine as ne


def make(num_blocks=100, host_blocks=100, **kw):
    c = ne.SchedulerConfig()
    c.block_token_num = 6
    c.max_batch_size = 16
    c.max_token_len = 1024
    c.max_step_tokens = 4096
    for k, v in kw.items():
        setattr(c, k, v)
    return ne.Scheduler(c, num_blocks, host_blocks)


def fake_token(seq_tokens_len, seed):
    return (seed * 7919 + seq_tokens_len * 104729) % 29989 + 10


def run_to_completion(s, seeds, max_steps=5000, kv_check=None):
    """Drives the scheduler; every sampled token is a deterministic function of (request seed, position)."""
    outputs = {}
    lens = {}
    finished = {}
    steps = 0
    while not s.idle() and steps < max_steps:
        plan = s.schedule()
        for ev in plan.events:
            if ev[4]:
                finished[ev[0]] = ev[5]
        if plan.empty():
            continue
        steps += 1
        if kv_check is not None:
            kv_check(plan)
        toks = []
        for sid in plan.sample_seq_ids.tolist():
            n = len(s.get_tokens(sid))
            toks.append(fake_token(n, seeds[sid]))
        for ev in s.post_step(plan, toks):
            sid, _, _, tok, fin, code, _ = ev
            if tok >= 0:
                outputs.setdefault(sid, []).append(tok)
            if fin:
                finished[sid] = code
        ok, why = s.check_invariants()
        assert ok, why
    return outputs, finished, steps


def cfg(max_new, **kw):
    c = ne.SamplingConfig()
    c.max_new_tokens = max_new
    c.ignore_eos = True
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def expected(prompt_len, seed, n):
    out, L = [], prompt_len
    for _ in range(n):
        out.append(fake_token(L, seed))
        L += 1
    return out


def test_no_swap_all_requests_complete_with_expected_tokens():
    s = make()
    seeds, prompts = {}, {}
    for r in range(8):
        p = list(range(100 + r, 100 + r + 10 + r))
        code, msg, ids = s.add_request(r, p, cfg(12))
        assert code == 0
        seeds[ids[0]], prompts[ids[0]] = r + 1, len(p)
    outs, fin, steps = run_to_completion(s, seeds)
    assert all(fin[sid] == 0 for sid in seeds)
    for sid in seeds:
        assert outs[sid] == expected(prompts[sid], seeds[sid], 12)
    st = s.stats()
    assert st["preempt_swap"] == 0 and st["preempt_recompute"] == 0
    assert st["free_blocks"] + st["usable_blocks"] - st["free_blocks"] == st["usable_blocks"] == 100


@pytest.mark.parametrize("mode", [0, 1])
def test_memory_pressure_preempts_and_still_matches(mode):
    # 20 blocks of 6 tokens cannot hold 6 requests growing to 40 tokens: swap (mode 0) or recompute (mode 1)
    s = make(num_blocks=20, host_blocks=64, preempt_mode=mode)
    seeds, prompts = {}, {}
    for r in range(6):
        p = list(range(50 + r * 3, 50 + r * 3 + 8))
        code, _, ids = s.add_request(r, p, cfg(32))
        seeds[ids[0]], prompts[ids[0]] = r + 11, len(p)
    outs, fin, _ = run_to_completion(s, seeds)
    for sid in seeds:
        assert fin[sid] == 0
        assert outs[sid] == expected(prompts[sid], seeds[sid], 32)
    st = s.stats()
    if mode == 0:
        assert st["preempt_swap"] > 0 and st["swap_in"] > 0 and st["swapped_out_blocks"] == st["swapped_in_blocks"]
    else:
        assert st["preempt_recompute"] > 0
    assert st["usable_blocks"] == 20 and st["free_host_blocks"] == 64


def test_slots_never_collide_and_positions_are_contiguous():
    s = make(num_blocks=40, enable_prefix_cache=True, split_fuse_token_num=24)
    seeds = {}
    for r in range(5):
        code, _, ids = s.add_request(r, list(range(10, 10 + 30 + r)), cfg(10))
        seeds[ids[0]] = r + 3
    seen_pos = {}

    def check(plan):
        slots = plan.slots
        assert len(set(slots.tolist())) == len(slots), "two tokens of one step write the same KV slot"
        row = 0
        for k, sid in enumerate(plan.seq_ids.tolist()):
            q = int(plan.q_lens[k]); kv = int(plan.kv_lens[k])
            pos = plan.positions[row:row + q].tolist()
            assert pos == list(range(kv - q, kv))
            start = seen_pos.get(sid)
            if start is not None:
                assert pos[0] <= start, "a sequence skipped positions"
            seen_pos[sid] = kv
            row += q

    outs, fin, _ = run_to_completion(s, seeds, kv_check=check)
    assert all(v == 0 for v in fin.values())


def test_prefix_cache_hits_and_dedup():
    s = make(num_blocks=60, enable_prefix_cache=True)
    shared = list(range(1000, 1036))              # 6 full blocks
    seeds = {}
    code, _, ids = s.add_request(0, shared + [7, 8, 9], cfg(4))
    seeds[ids[0]] = 1
    run_to_completion(s, seeds)
    assert s.stats()["prefix_hit_tokens"] == 0
    for r in (1, 2):
        code, _, ids = s.add_request(r, shared + [20 + r, 30 + r], cfg(4))
        seeds[ids[0]] = r + 1
    run_to_completion(s, seeds)
    st = s.stats()
    assert st["prefix_hit_requests"] == 2 and st["prefix_hit_tokens"] == 2 * 36
    # the same prompt again: everything but the last token is reused
    code, _, ids = s.add_request(5, shared + [7, 8, 9], cfg(2))
    seeds[ids[0]] = 9
    run_to_completion(s, seeds)
    assert s.stats()["prefix_hit_tokens"] >= 3 * 36


def test_admission_limits_timeouts_and_abort():
    s = make(max_waiting_queue_len=2, max_token_len=32, waiting_timeout_in_ms=0)
    code, msg, _ = s.add_request(0, list(range(40)), cfg(4))
    assert code == int(ne.RET_EXCEED_LENGTH)
    assert s.add_request(1, [1, 2, 3], cfg(4))[0] == 0
    assert s.add_request(2, [1, 2, 3], cfg(4))[0] == 0
    assert s.add_request(3, [1, 2, 3], cfg(4))[0] == int(ne.RET_EXCEED_CAPACITY)
    plan = s.schedule()          # timeout 0 ms: everything still waiting expires
    codes = sorted(ev[5] for ev in plan.events)
    assert codes == [int(ne.RET_TIMEOUT)] * 2 and plan.empty()
    s2 = make()
    _, _, ids = s2.add_request(7, [1, 2, 3, 4], cfg(50))
    seeds = {ids[0]: 1}
    plan = s2.schedule(); s2.post_step(plan, [11])
    s2.abort(7)
    plan = s2.schedule()
    assert [ev[5] for ev in plan.events] == [int(ne.RET_TERMINATED)] and s2.idle()
    bad = cfg(4, topk=2000)
    assert s2.add_request(8, [1], bad)[0] == int(ne.RET_INVALID_ARGUMENT)


def test_stop_tokens_and_eos():
    c = ne.SchedulerConfig(); c.eos_token_ids = [99]; c.block_token_num = 4
    s = ne.Scheduler(c, 32, 0)
    sc = ne.SamplingConfig(); sc.max_new_tokens = 10; sc.stop_token_ids = [55]
    _, _, a = s.add_request(1, [1, 2, 3], sc)
    sc2 = ne.SamplingConfig(); sc2.max_new_tokens = 3; sc2.ignore_eos = True
    _, _, b = s.add_request(2, [4, 5], sc2)
    plan = s.schedule()
    ev = s.post_step(plan, [99, 99])          # EOS finishes the first, is ignored by the second
    fin = {e[0]: e[4] for e in ev}
    assert fin[a[0]] is True and fin[b[0]] is False
    plan = s.schedule(); s.post_step(plan, [5])
    plan = s.schedule(); ev = s.post_step(plan, [6])
    assert ev[0][4] is True and s.idle()      # max_new_tokens reached


def test_parallel_sampling_shares_prefill_and_forks():
    s = make(num_blocks=50, enable_prefix_cache=True)
    sc = cfg(5, num_return_sequences=3, topk=5)
    _, _, ids = s.add_request(1, list(range(20)), sc)      # 3 full blocks + 2 tokens
    assert len(ids) == 3
    plan = s.schedule()
    assert len(plan.seq_ids) == 1 and plan.num_tokens == 20          # one prefill for the whole group
    assert plan.sample_seq_ids.tolist() == ids and plan.sample_rows.tolist() == [19, 19, 19]
    s.post_step(plan, [100, 101, 102])
    plan = s.schedule()
    assert sorted(plan.seq_ids.tolist()) == ids and plan.num_tokens == 3
    assert plan.pre_copies.size == 2 * 3 and plan.copies.size == 0   # two siblings copy the partial tail block, before
                                                                     # anything else this plan does to the cache
    tbl = plan.block_table.reshape(3, plan.max_blocks)
    assert (tbl[:, :3] == tbl[0, :3]).all() and len(set(tbl[:, 3].tolist())) == 3   # shared full blocks, private tails
    toks = {sid: s.get_tokens(sid) for sid in ids}
    assert [toks[i][-1] for i in ids] == [100, 101, 102]


def test_beam_reparenting_shares_history():
    s = make(num_blocks=50)
    sc = cfg(6, num_beams=2, logprobs_num=2)
    _, _, ids = s.add_request(1, list(range(13)), sc)
    plan = s.schedule(); s.post_step(plan, [7, 8])
    plan = s.schedule()
    # both beams continue from beam 1's history
    s.post_step(plan, [20, 21], [ids[1], -1])
    assert s.get_tokens(ids[0])[-3:] == [12, 8, 20] and s.get_tokens(ids[1])[-3:] == [12, 8, 21]
    plan = s.schedule()
    assert plan.pre_copies.size == 3
    assert s.check_invariants()[0]


def test_plan_pack_roundtrip_and_threaded_clients():
    s = make(num_blocks=200, max_batch_size=32)
    seeds, lock = {}, threading.Lock()

    def client(base):
        for r in range(10):
            _, _, ids = s.add_request(base * 100 + r, list(range(base, base + 9 + r)), cfg(6))
            with lock:
                seeds[ids[0]] = base + r

    ts = [threading.Thread(target=client, args=(b,)) for b in range(1, 5)]
    [t.start() for t in ts]; [t.join() for t in ts]
    plan = s.schedule()
    img = plan.pack()
    back = ne.StepPlan.unpack(img)
    for f in ("seq_ids", "q_lens", "kv_lens", "input_ids", "positions", "slots", "cu_q", "block_table", "sample_rows"):
        assert np.array_equal(getattr(plan, f), getattr(back, f)), f
    toks = [fake_token(len(s.get_tokens(sid)), seeds[sid]) for sid in plan.sample_seq_ids.tolist()]
    s.post_step(plan, toks)
    outs, fin, _ = run_to_completion(s, seeds)
    assert len(fin) == 40 and all(v == 0 for v in fin.values())


def test_static_batching_runs_batches_to_completion():
    s = make(schedule_strategy=1, auto_batch_wait_ms=0)
    seeds = {}
    for r in range(3):
        _, _, ids = s.add_request(r, [1, 2, 3, 4], cfg(4)); seeds[ids[0]] = r + 1
    plan = s.schedule()
    assert len(plan.seq_ids) == 3
    _, _, late = s.add_request(9, [5, 6], cfg(2)); seeds[late[0]] = 5
    s.post_step(plan, [11, 12, 13])
    plan = s.schedule()
    assert late[0] not in plan.seq_ids.tolist()      # no admission while the batch is running
    s.post_step(plan, [11, 12, 13])
    outs, fin, _ = run_to_completion(s, seeds)
    assert fin[late[0]] == 0


def test_data_parallel_ranks_have_block_pools_of_their_own():
    """dp_size ranks: a sequence's blocks come from the pool of rank seq_id % dp_size, so two ranks hold twice the
    sequences; slots may repeat across ranks but never inside one; siblings stay on their leader's rank; memory
    pressure on one rank preempts only that rank's sequences."""
    B, blocks = 6, 12
    one = make(num_blocks=blocks, host_blocks=0, preempt_mode=1)
    two = make(num_blocks=blocks, host_blocks=0, preempt_mode=1, dp_size=2)
    results = []
    for s, dp in ((one, 1), (two, 2)):
        seeds, prompts = {}, {}
        for r in range(8):
            p = list(range(40 + r, 40 + r + 10))
            code, _, ids = s.add_request(r, p, cfg(20))
            assert code == 0
            seeds[ids[0]], prompts[ids[0]] = r + 5, len(p)

        def check(plan, dp=dp):
            per_rank = {}
            row = 0
            for k, sid in enumerate(plan.seq_ids.tolist()):
                q = int(plan.q_lens[k])
                rank = sid % dp
                for slot in plan.slots[row:row + q].tolist():
                    assert slot not in per_rank.setdefault(rank, set()), "two tokens of one rank write the same KV slot"
                    per_rank[rank].add(slot)
                    assert 0 <= slot < blocks * B
                row += q

        outs, fin, steps = run_to_completion(s, seeds, kv_check=check)
        for sid in seeds:
            assert fin[sid] == 0 and outs[sid] == expected(prompts[sid], seeds[sid], 20)
        results.append((steps, s.stats()["preempt_recompute"]))
    # 8 sequences x 5 blocks at the end do not fit 12 blocks, but fit 2 x 12 better: fewer preemptions and steps
    assert results[1][1] < results[0][1] and results[1][0] <= results[0][0]
    # parallel sampling: the siblings share the leader's blocks, hence its rank
    s = make(num_blocks=40, dp_size=4)
    code, _, ids = s.add_request(1, list(range(10, 30)), cfg(6, num_return_sequences=3, topk=4))
    code, _, ids2 = s.add_request(2, list(range(50, 70)), cfg(6))
    assert len({i % 4 for i in ids}) == 1 and len(set(ids + ids2)) == 4
    seeds = {i: 3 + k for k, i in enumerate(ids + ids2)}
    outs, fin, _ = run_to_completion(s, seeds)
    assert all(fin[i] == 0 and len(outs[i]) == 6 for i in ids + ids2)


def test_data_parallel_swap_lists_name_the_owning_pool():
    """Swap mode under data parallelism: a device block in the swap lists is rank * blocks_per_rank + block, the rank
    being the owner of the swapped sequence; what goes out comes back; tokens are unaffected."""
    blocks = 10
    s = make(num_blocks=blocks, host_blocks=40, preempt_mode=0, dp_size=2)
    seeds, prompts = {}, {}
    for r in range(8):
        p = list(range(60 + r, 60 + r + 9))
        code, _, ids = s.add_request(r, p, cfg(30))
        seeds[ids[0]], prompts[ids[0]] = r + 2, len(p)
    seen = {"out": set(), "in": set()}

    def check(plan):
        for key, arr in (("out", plan.swap_out), ("in", plan.swap_in)):
            a = np.asarray(arr).reshape(-1, 2)
            for dev, host in a.tolist():
                assert 0 <= dev < 2 * blocks and 0 <= host < 40
                seen[key].add(dev // blocks)

    outs, fin, _ = run_to_completion(s, seeds, kv_check=check)
    for sid in seeds:
        assert fin[sid] == 0 and outs[sid] == expected(prompts[sid], seeds[sid], 30)
    st = s.stats()
    assert st["preempt_swap"] > 0 and st["swapped_out_blocks"] == st["swapped_in_blocks"]
    assert seen["out"] == {0, 1} and seen["in"] == {0, 1}
