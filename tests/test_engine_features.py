"""Request-level features through the real engine on CPU: parallel sampling, beam search, log-probs,
penalties, n-gram bans, stop strings, structured output, streaming + abort, /forward targets, swap."""
import math
import pytest
import threading

import torch

from helpers import ByteTokenizer, sampling, tiny_engine, tiny_model_cfg
from ksanallm_b200.runtime.sampler import banned_encoder_ngram_tokens, banned_ngram_tokens, beam_final_order
from ksanallm_b200.serving.forward_api import verify_request_target


def test_parallel_sampling_returns_distinct_sequences():
    eng = tiny_engine()
    req = eng.generate([[5, 6, 7, 8, 9]], sampling(max_new_tokens=6, ignore_eos=True, topk=50, temperature=1.5,
                                                   num_return_sequences=4, seed=7))[0]
    assert req.status_code == 0 and len(req.outputs) == 4
    assert all(len(o.tokens) == 6 for o in req.outputs)
    assert len({tuple(o.tokens) for o in req.outputs}) > 1
    again = tiny_engine().generate([[5, 6, 7, 8, 9]], sampling(max_new_tokens=6, ignore_eos=True, topk=50, temperature=1.5,
                                                               num_return_sequences=4, seed=7))[0]
    assert [o.tokens for o in again.outputs] == [o.tokens for o in req.outputs]      # per-request seed


def test_greedy_is_argmax_and_logprobs_are_topn_logsoftmax():
    eng = tiny_engine()
    captured = []
    eng.step_hook = lambda plan, logits: captured.append(logits.clone())
    req = eng.generate([[11, 12, 13]], sampling(max_new_tokens=3, ignore_eos=True, logprobs_num=4))[0]
    out = req.outputs[0]
    assert len(out.logprobs) == 3
    for step, (tok, lps) in enumerate(zip(out.tokens, out.logprobs)):
        row = captured[step][0]
        assert tok == int(row.argmax())
        top = torch.topk(row, 4)
        want = torch.log_softmax(top.values, -1)
        assert [i for i, _ in lps] == top.indices.tolist()
        assert all(abs(a - float(b)) < 1e-4 for (_, a), b in zip(lps, want))


def test_repetition_penalty_and_ngram_bans_change_choices():
    base = tiny_engine().generate([[20, 21, 22, 23]], sampling(max_new_tokens=12, ignore_eos=True))[0].outputs[0].tokens
    pen = tiny_engine().generate([[20, 21, 22, 23]], sampling(max_new_tokens=12, ignore_eos=True,
                                                              no_repeat_ngram_size=1))[0].outputs[0].tokens
    assert len(set(pen + [20, 21, 22, 23])) == len(pen) + 4      # 1-gram ban: no token is ever repeated
    assert banned_ngram_tokens([1, 2, 3, 1, 2], 3) == [3]
    assert banned_encoder_ngram_tokens([5, 6, 7], [9, 5], 2) == [6]
    assert isinstance(base, list)


def test_beam_search_orders_by_score_and_beats_greedy():
    prompt = [30, 31, 32, 33, 34]
    eng = tiny_engine()
    req = eng.generate([prompt], sampling(max_new_tokens=5, ignore_eos=True, num_beams=3, num_return_sequences=3))[0]
    assert req.status_code == 0 and all(len(o.tokens) == 5 for o in req.outputs)
    order = beam_final_order(req.outputs, 1.0)
    scores = [req.outputs[i].cum_logprob for i in order]
    assert scores == sorted(scores, reverse=True)
    assert len({tuple(o.tokens) for o in req.outputs}) == 3
    assert eng.scheduler.check_invariants()[0]


def test_stop_strings_truncate_output():
    tok = ByteTokenizer()
    eng = tiny_engine(tokenizer=tok)
    free = eng.generate([tok.encode("hello")], sampling(max_new_tokens=12, ignore_eos=True))[0].outputs[0].tokens
    text = tok.decode(free)
    stop = text[4:6]
    eng2 = tiny_engine(tokenizer=tok)
    req = eng2.generate([tok.encode("hello")], sampling(max_new_tokens=12, ignore_eos=True, stop_strings=[stop]))[0]
    got = tok.decode(req.outputs[0].tokens)
    assert stop not in got and text.startswith(got) and len(got) <= text.find(stop)
    assert eng2.scheduler.idle()


def test_structured_output_injects_constants_and_finishes():
    tok = ByteTokenizer()
    eng = tiny_engine(tokenizer=tok)
    regex = r'\{"a": "[a-z]*", "n": [0-9]+\}'
    req = eng.add_request(tok.encode("x"), sampling(max_new_tokens=60, ignore_eos=True, topk=40, temperature=2.0, seed=3),
                          structured_regex=regex)
    while not req.done.is_set():
        if not eng.step() and eng.scheduler.idle():
            break
    text = tok.decode(req.outputs[0].tokens)
    assert text.startswith('{"a": "')
    if '", "n": ' in text:              # the free segment ended: the injected constant follows verbatim
        assert text.count('{"a": "') == 1


def test_streaming_queue_and_abort():
    eng = tiny_engine()
    eng.start()
    try:
        req = eng.add_request([40, 41, 42], sampling(max_new_tokens=200, ignore_eos=True), stream=True)
        first = req.stream_queue.get(timeout=30)
        assert first[0] == "step" and len(first[1][0]) >= 1
        eng.abort(req)
        assert req.done.wait(30)
        assert req.status_code == 4 and len(req.outputs[0].tokens) < 200
    finally:
        eng.stop()


def test_forward_targets_validation_and_values():
    assert verify_request_target({"logits": {"slice_pos": [[0, 3]], "token_reduce_mode": "GATHER_TOKEN_ID"}}, 6)[0] == 0
    assert verify_request_target({"logits": {"slice_pos": [[0, 5]], "token_reduce_mode": "GATHER_TOKEN_ID"}}, 6)[0] == 1
    assert verify_request_target({"logits": {"slice_pos": [[0, 2]], "token_reduce_mode": "GATHER_ALL"}}, 6)[0] == 1
    assert verify_request_target({"transformer": {"token_id": [3], "slice_pos": [[0, 1]]}}, 6)[0] == 1
    assert verify_request_target({"bogus": {}}, 6)[0] == 1
    assert verify_request_target({"layernorm": {"slice_pos": [[-2, -1]]}}, 6) == (0, "")
    eng = tiny_engine()
    prompt = [50, 51, 52, 53, 54, 55]
    target = {"logits": {"slice_pos": [[0, 4]], "token_reduce_mode": "GATHER_TOKEN_ID", "token_id": []},
              "transformer": {"slice_pos": [[5, 5]], "token_reduce_mode": "GATHER_ALL", "token_id": []},
              "layernorm": {"slice_pos": [], "token_reduce_mode": "GATHER_ALL", "token_id": []}}
    req = eng.add_request(prompt, sampling(max_new_tokens=1), request_target=target)
    while not req.done.is_set():
        eng.step()
    probs = req.response["logits"]
    assert probs.shape == (5,) and bool(((probs > 0) & (probs <= 1)).all())
    assert req.response["transformer"].shape == (1, 64) and req.response["layernorm"].shape == (1, 64)
    ppl = math.exp(-float(probs.log().mean()))
    assert ppl > 1.0


def test_swap_under_pressure_keeps_results():
    prompts = [[60 + i, 61 + i, 62 + i, 63 + i] for i in range(6)]
    s = sampling(max_new_tokens=40, ignore_eos=True)
    calm = tiny_engine(num_blocks=128, max_token_len=64).generate(prompts, s)
    tight = tiny_engine(num_blocks=10, host_blocks=64, max_token_len=64)
    pressed = tight.generate(prompts, s)
    assert [r.outputs[0].tokens for r in pressed] == [r.outputs[0].tokens for r in calm]
    st = tight.scheduler.stats()
    assert st["preempt_swap"] > 0 and st["swap_in"] > 0


def test_debug_input_checks_catch_bad_indices(monkeypatch):
    """KSANA_CHECK_INPUTS=1: every step of a normal run passes the host-side validation; corrupted metadata is
    reported before any kernel would consume it."""
    import torch
    from ksanallm_b200.ops import checks
    monkeypatch.setenv("KSANA_CHECK_INPUTS", "1")
    eng = tiny_engine(enable_auto_prefix_cache=True, split_fuse_token_num=16)
    steps = []
    real = eng.runner.build_step

    def spy(plan, extra=None, patch=None):
        st = real(plan, extra, patch)
        steps.append(st)
        return st

    eng.runner.build_step = spy
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 300, (n,), generator=g).tolist() for n in (40, 7, 23)]
    reqs = eng.generate(prompts, sampling(max_new_tokens=5, ignore_eos=True))
    assert all(len(r.outputs[0].tokens) == 5 for r in reqs) and len(steps) > 3
    model = eng.runner.model
    nb, bt = model.kv_cache.shape[0], model.block_tokens
    good = steps[0]
    assert checks.step_violations(good, nb, bt, 300, 512) == []
    import dataclasses
    bad_table = dataclasses.replace(good, block_table=good.block_table.clone())
    bad_table.block_table[0, 0] = nb + 5
    assert any("block id outside" in v for v in checks.step_violations(bad_table, nb, bt, 300, 512))
    bad_ids = dataclasses.replace(good, input_ids=good.input_ids.clone())
    bad_ids.input_ids[0] = 300
    assert any("token id outside" in v for v in checks.step_violations(bad_ids, nb, bt, 300, 512))
    bad_slots = dataclasses.replace(good, slots=good.slots.clone())
    bad_slots.slots[1] = bad_slots.slots[0]
    assert any("same cache slot" in v or "says otherwise" in v for v in checks.step_violations(bad_slots, nb, bt, 300, 512))


def test_fp8_tile_choice_rule():
    """The dispatch rule between 256 x 224 and 128 x 256 FP8 tiles reproduces the measured winners."""
    from ksanallm_b200.ops.native import _tall_wins
    tall = [(16384, 10240, 8192), (16384, 57344, 8192), (16384, 8192, 28672), (16384, 4096, 14336), (2048, 10240, 8192),
            (512, 57344, 8192), (16384, 28672, 4096)]
    std = [(4096, 7168, 2048), (16384, 4096, 1024), (16384, 2048, 7168), (8192, 1280, 8192), (256, 1024, 8192)]
    assert all(_tall_wins(*s) for s in tall) and not any(_tall_wins(*s) for s in std)


def test_kv_scale_calibration_writes_the_reference_file_format(tmp_path):
    """The calibration tool's file is read back by the config loader, and its scales are the cache's largest
    magnitudes over the e4m3 range."""
    from ksanallm_b200.config import EngineConfig, load_kv_scales
    from ksanallm_b200.llm import LLM
    from ksanallm_b200.utils.kv_scale_calibration import calibrate_kv_scales, layer_amax, write_kv_scales
    cfg = tiny_model_cfg()
    ec = EngineConfig()
    ec.batch_scheduler.max_token_len = 128
    ec.block_manager.device_blocks_num = 64
    llm = LLM(ec, cfg, weights="random", device="cpu", dtype=torch.float32)
    prompts = [[5 + i, 9, 11, 13 + i, 17, 19] for i in range(5)]
    scales = calibrate_kv_scales(llm, prompts, max_new_tokens=3, batch=2)
    assert len(scales) == cfg.num_layers and all(s > 0 for s in scales)
    want = layer_amax(llm.model.kv_cache).amax(dim=1) / 448.0
    assert all(s >= float(w) - 1e-9 for s, w in zip(scales, want))        # the running maximum covers the last batch
    out = tmp_path / "kv_cache_scales.json"
    write_kv_scales(str(out), scales)
    back = load_kv_scales(str(out), cfg.num_layers)
    assert [b[0] for b in back] == pytest.approx(scales) and all(b[0] == b[1] for b in back)
    llm.shutdown()


def test_step_extras_survive_the_wire_format():
    """The optional inputs of a step (spliced embeddings, multimodal positions, /forward flags and row ranges)
    reach worker ranks as a byte image: tensors keep dtype and values, plain values stay plain."""
    from ksanallm_b200.parallel.control import pack_extras, unpack_extras
    assert pack_extras(None) is None and pack_extras({}) is None and unpack_extras(None) is None
    extra = {"refit_positions": torch.tensor([3, 4], dtype=torch.int32), "refit_embeddings": torch.randn(2, 8),
             "mrope_positions": torch.arange(12, dtype=torch.int32).view(3, 4), "want_hidden": True,
             "full_logits": [[0, 5], [9, 2]]}
    back = unpack_extras(pack_extras(extra))
    assert set(back) == set(extra) and back["want_hidden"] is True and back["full_logits"] == [[0, 5], [9, 2]]
    for k in ("refit_positions", "refit_embeddings", "mrope_positions"):
        assert back[k].dtype == extra[k].dtype and torch.equal(back[k], extra[k])


def test_device_error_word_fails_requests_in_flight():
    """A non-zero device error word read back with the sampled tokens ends the step's requests with RET_RUNTIME
    instead of returning tokens sampled from invalid logits; a peer wait that ran out also stops admission."""
    from ksanallm_b200.ops import native
    eng = tiny_engine(num_blocks=64, max_token_len=64)
    s = sampling(max_new_tokens=8, ignore_eos=True)
    req = eng.add_request(list(range(5, 25)), s)
    assert eng.step()                                   # prefill step, fine
    with torch.inference_mode():
        native.err_flag(eng.model.device).fill_(3)
    for _ in range(3):                                  # the word is read back with a step's tokens; with pipelined
        if req.done.is_set():                           # stepping that is one step after the step that set it
            break
        assert eng.step()
    assert req.done.is_set() and req.status_code == 12 and "peer" in req.status_message
    assert int(native.err_flag(eng.model.device).item()) == 0
    r2 = eng.add_request(list(range(5, 25)), s)         # the group's collective epochs are out of step: refuse
    assert r2.done.is_set() and r2.status_code == 12
    eng.fatal = None
    r3 = eng.generate([list(range(5, 25))], s)[0]
    assert r3.status_code == 0 and len(r3.outputs[0].tokens) == 8


def test_forked_siblings_survive_swap_preemption():
    """Parallel sampling forks the partly filled tail block of the shared prompt, and under memory pressure the
    freshly forked (youngest) sibling is the first to be swapped out: the fork's copy has to land before the swap
    reads its destination. Greedy siblings under pressure produce the tokens of the unconstrained run."""
    prompts = [[40 + i, 41 + i, 42 + i, 43 + i, 44 + i] for i in range(3)]
    s = sampling(max_new_tokens=40, ignore_eos=True, num_return_sequences=3)
    calm = tiny_engine(num_blocks=256, max_token_len=64).generate(prompts, s)
    tight = tiny_engine(num_blocks=14, host_blocks=128, max_token_len=64)
    pressed = tight.generate(prompts, s)
    for a, b in zip(pressed, calm):
        assert a.status_code == 0 and b.status_code == 0
        assert [o.tokens for o in a.outputs] == [o.tokens for o in b.outputs]
        assert a.outputs[0].tokens == a.outputs[1].tokens == a.outputs[2].tokens
    st = tight.scheduler.stats()
    assert st["preempt_swap"] > 0 and st["swap_in"] > 0


def test_warmup_request_runs_at_start_unless_disabled(monkeypatch):
    """The engine answers one short request from its constructor (kernels, workspaces and collectives set up before
    the first user request); DISABLE_WARMUP=1 skips it."""
    from ksanallm_b200.config import EngineConfig
    from ksanallm_b200.llm import LLM
    from ksanallm_b200.models.weights import RandomSource

    def build():
        ec = EngineConfig()
        ec.batch_scheduler.max_token_len = 64
        ec.block_manager.device_blocks_num = 32
        return LLM(ec, tiny_model_cfg(), weights=RandomSource(seed=0, std=0.2), device="cpu", dtype=torch.float32)

    monkeypatch.setenv("DISABLE_WARMUP", "1")
    assert build().engine.steps == 0
    monkeypatch.delenv("DISABLE_WARMUP")
    llm = build()
    assert llm.engine.steps == 2 and llm.engine.scheduler.idle()
    st = llm.engine.scheduler.stats()
    assert st["total_requests"] == 1 and st["finished"] == 1


def test_pipelined_steps_give_the_tokens_of_synchronous_steps():
    """Pipelined stepping (next step planned and launched before the current step's tokens reach the host) against
    synchronous stepping: same tokens for every request, with sequences that stop on EOS while their next row is
    already in flight, a length limit that is known in advance, chunked prefill, the prefix cache and preemption."""
    from ksanallm_b200.utils import native_engine as ne
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 300, (n,), generator=g).tolist() for n in (40, 7, 23, 61, 5, 33)]
    prompts.append(list(prompts[0][:32]) + [9, 8, 7])                 # shares two cache blocks with the first prompt
    probe = tiny_engine(max_token_len=120)
    probe.pipelined = False
    seqs = [set(r.outputs[0].tokens) for r in probe.generate(prompts, sampling(max_new_tokens=30, ignore_eos=True))]
    # a token that some sequences produce and others do not serves as EOS: some stop early, some run to their limit
    eos = next(t for t in sorted(set().union(*seqs)) if 2 <= sum(t in q for q in seqs) <= len(seqs) - 2)
    for pressure in (dict(num_blocks=128, host_blocks=0), dict(num_blocks=14, host_blocks=0, preempt_mode=1)):
        outs = []
        for pipelined in (False, True):
            eng = tiny_engine(enable_auto_prefix_cache=True, split_fuse_token_num=32, max_token_len=120, **pressure)
            eng.pipelined = pipelined
            eng.sched_cfg.eos_token_ids = [int(eos)]
            eng.scheduler = ne.Scheduler(eng.sched_cfg, pressure["num_blocks"], pressure["host_blocks"])
            reqs = eng.generate(prompts, sampling(max_new_tokens=30))
            outs.append([(r.outputs[0].tokens, r.status_code) for r in reqs])
            assert eng.scheduler.idle() and eng.scheduler.check_invariants()[0]
            assert eng._flight is None
        assert outs[0] == outs[1]
        assert any(len(t) < 30 for t, _ in outs[1]) and any(len(t) == 30 for t, _ in outs[1])


def test_abort_while_a_pipelined_step_is_in_flight():
    """A request is aborted after its next token has been launched but before that step's tokens reached the host: the
    request ends with the abort status, the other request's tokens equal a run without the abort, nothing leaks."""
    prompts = [[40, 41, 42, 43], [7, 8, 9]]
    ref = tiny_engine()
    ref.pipelined = True
    want = ref.generate([prompts[1]], sampling(max_new_tokens=12, ignore_eos=True))[0].outputs[0].tokens
    eng = tiny_engine()
    eng.pipelined = True
    a = eng.add_request(prompts[0], sampling(max_new_tokens=50, ignore_eos=True))
    b = eng.add_request(prompts[1], sampling(max_new_tokens=12, ignore_eos=True))
    for _ in range(4):
        assert eng.step()
    assert eng._flight is not None                      # a step is in flight: its tokens are still on the device
    eng.abort(a)
    for _ in range(200):
        if a.done.is_set() and b.done.is_set():
            break
        eng.step()
    assert a.done.is_set() and a.status_code == 4 and 0 < len(a.outputs[0].tokens) < 50
    assert b.done.is_set() and b.status_code == 0 and b.outputs[0].tokens == want
    while eng.step():
        pass
    assert eng._flight is None and eng.scheduler.idle() and eng.scheduler.check_invariants()[0]


def test_request_that_needs_the_host_joins_pipelined_requests():
    """A request with log-probabilities (the host looks at every step's logits) arrives while plain requests are being
    stepped in pipelined mode: the step in flight is drained, stepping goes synchronous while that request lives and
    pipelined again afterwards; every request's tokens equal a fully synchronous run."""
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(3, 300, (n,), generator=g).tolist() for n in (9, 21, 5)]

    def run(pipelined):
        eng = tiny_engine()
        eng.pipelined = pipelined
        plain = [eng.add_request(p, sampling(max_new_tokens=24, ignore_eos=True)) for p in prompts[:2]]
        modes = []
        for _ in range(5):
            eng.step()
            modes.append(eng._flight is not None)
        probe = eng.add_request(prompts[2], sampling(max_new_tokens=6, ignore_eos=True, logprobs_num=2))
        for _ in range(300):
            if all(r.done.is_set() for r in plain + [probe]):
                break
            eng.step()
            modes.append(eng._flight is not None)
        while eng.step():
            pass
        assert eng._flight is None and eng.scheduler.idle()
        assert len(probe.outputs[0].logprobs) == 6
        return [r.outputs[0].tokens for r in plain + [probe]], modes

    want, sync_modes = run(False)
    got, modes = run(True)
    assert got == want
    assert not any(sync_modes)
    assert modes[0] or modes[1]                       # pipelined before the probe arrives ...
    assert not all(modes[5:11])                       # ... synchronous while it lives ...
    assert modes[-1] or any(modes[11:])               # ... and pipelined again for the rest of the plain requests


def test_streaming_under_pipelined_steps_delivers_every_token_in_order():
    """Streamed pieces of a pipelined run (tokens reach the host one step late) add up to the tokens of a blocking,
    synchronous run, in order, and the stream ends with its end marker."""
    prompt = [5, 6, 7, 8, 9]
    base = tiny_engine()
    base.pipelined = False
    want = base.generate([prompt], sampling(max_new_tokens=15, ignore_eos=True))[0].outputs[0].tokens
    eng = tiny_engine()
    eng.pipelined = True
    eng.start()
    try:
        req = eng.add_request(prompt, sampling(max_new_tokens=15, ignore_eos=True), stream=True)
        seen = []
        while True:
            item = req.stream_queue.get(timeout=30)
            if item is None:
                break
            assert item[0] == "step"
            seen.append(list(item[1][0]))
        assert req.done.wait(30) and req.status_code == 0
    finally:
        eng.stop()
    # every piece carries the tokens so far (or the new ones): the last piece, or their concatenation, is the answer
    flat = seen[-1] if len(seen[-1]) == len(want) else [t for piece in seen for t in piece]
    assert flat == want and req.outputs[0].tokens == want


@pytest.mark.parametrize("native_loop", ["1", "0"])
def test_generate_on_a_started_engine_waits_for_the_loop(monkeypatch, native_loop):
    """``generate`` on an engine whose background loop runs (native thread or Python thread) hands its requests to that
    loop instead of stepping on the calling thread beside it; tokens equal those of an engine stepped by the caller."""
    monkeypatch.setenv("KSANA_NATIVE_LOOP", native_loop)
    prompts = [[5, 6, 7, 8, 9], [3, 1, 4, 1, 5, 9, 2, 6]]
    want = [r.outputs[0].tokens for r in tiny_engine().generate(prompts, sampling(max_new_tokens=12, ignore_eos=True))]
    eng = tiny_engine()
    eng.start()
    try:
        assert (eng._native_loop is not None) == (native_loop == "1")
        stepped_by = set()
        real_step = eng.step

        def step():
            stepped_by.add(threading.get_ident())
            return real_step()
        eng.step = step
        got = [r.outputs[0].tokens for r in eng.generate(prompts, sampling(max_new_tokens=12, ignore_eos=True), timeout=60)]
    finally:
        eng.stop()
    assert got == want
    assert threading.get_ident() not in stepped_by and len(stepped_by) == 1


@pytest.mark.parametrize("quant", ["fp8_block", "nvfp4", "w4a16"])
def test_quantised_weights_keep_the_perplexity(quant):
    """Perplexity-style check of the quantised paths (CPU restatements of block FP8, NVFP4 and 4-bit weight-only):
    the mean next-token loss of a two-layer model over 95 positions stays within 8 % (as a perplexity ratio) of the
    same model with unquantised weights."""
    from ksanallm_b200.config import ModelConfig
    from ksanallm_b200.models.common import StepInput
    from ksanallm_b200.models.weights import RandomSource, build_model
    cfg = ModelConfig(model_type="llama", hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                      intermediate_size=512, vocab_size=300, max_position_embeddings=256, max_token_len=256)
    torch.manual_seed(1)
    T = 96
    toks = torch.randint(3, cfg.vocab_size, (T,))

    def loss(q):
        m = build_model(cfg, RandomSource(seed=3, std=0.05), device="cpu", dtype=torch.float32, quant=q)
        m.allocate_kv_cache(16, 16)
        ar = torch.arange(T, dtype=torch.int32)
        step = StepInput(toks.to(torch.int32), ar, ar.clone(), torch.tensor([0, T], dtype=torch.int32),
                         torch.tensor([T], dtype=torch.int32), torch.arange(16, dtype=torch.int32).view(1, 16),
                         num_multi=1, num_single=0, num_tokens=T, num_multi_tokens=T, max_q_len=T, max_kv_len=T)
        logits = m.forward(step).float()
        assert logits.shape == (T, cfg.vocab_size)
        return float(-torch.log_softmax(logits[:-1], -1).gather(1, toks[1:].view(-1, 1)).mean())

    ratio = math.exp(loss(quant) - loss(None))
    assert 0.92 < ratio < 1.08, ratio
