"""Host runtime components: cache manager, control plane over localhost TCP (incl. host-side failure
injection), structured-output FSM, profiler / trace recorder, config parsing."""
import json
import os
import threading
import time

import pytest
import yaml

from ksanallm_b200 import config as cfgmod
from ksanallm_b200.utils import native_engine as ne


# ----------------------------------------------------------------------------------- cache manager
def test_cache_manager_prefix_share_evict_and_swap():
    c = ne.CacheManager(16, 8, 4, True)
    toks = list(range(100, 119))                       # 4 full blocks + 3 tokens
    n, blocks = c.acquire_prefix(toks)
    assert n == 0 and blocks == []
    ok, blocks = c.allocate(5)
    assert ok and c.free_blocks == 11
    promoted, blocks = c.promote(toks, blocks, 19, 0)
    assert promoted == 4 and all(c.in_tree(b) for b in blocks[:4]) and not c.in_tree(blocks[4])
    # a second sequence with the same prefix shares the four full blocks
    n, shared = c.acquire_prefix(toks[:16] + [1, 2])
    assert n == 16 and shared == blocks[:4] and all(c.ref_count(b) == 2 for b in shared)
    # identical content computed privately is deduplicated on promotion
    ok, own = c.allocate(2)
    p2, merged = c.promote(toks[:8], own, 8, 0)
    assert p2 == 2 and merged == blocks[:2] and c.ref_count(blocks[0]) == 3
    c.release(merged); c.release(shared)
    # swap-out moves only exclusively owned blocks; shared ones stay
    n, other = c.acquire_prefix(toks[:8] + [9])
    ok, kept, host, pairs = c.swap_out(list(blocks))
    assert ok and kept == blocks[:2] and len(host) == 3 and [p[0] for p in pairs] == blocks[2:]
    assert c.free_host_blocks == 5
    ok, back, pairs_in = c.swap_in(kept, host)
    assert ok and len(back) == 5 and c.free_host_blocks == 8
    c.release(back); c.release(other)
    assert c.check_invariants()[0] and c.usable_blocks == 16
    # eviction: filling the pool reclaims cached blocks, oldest first
    ok, big = c.allocate(16)
    assert ok and c.free_blocks == 0 and c.evictable_blocks == 0
    assert c.acquire_prefix(toks)[0] == 0
    c.release(big)
    assert c.check_invariants()[0]


def test_cache_manager_fork_and_flexible():
    c = ne.CacheManager(32, 0, 4, True)
    toks = list(range(50, 64))                         # 3 full + 2
    ok, blocks = c.allocate(4)
    _, blocks = c.promote(toks, blocks, 14, 0)
    ok, dst, copies = c.fork(blocks, 14)
    assert ok and dst[:3] == blocks[:3] and dst[3] != blocks[3] and copies == [(blocks[3], dst[3])]
    assert all(c.ref_count(b) == 2 for b in blocks[:3])
    # flexible cache: the same 8 tokens appear at another position of a new prompt
    new = [1, 2, 3, 4] + toks[4:12] + [9]
    n, pre = c.acquire_prefix(new)
    assert n == 0
    got, fb, tasks = c.acquire_flexible([7, 7, 7, 7] + toks[4:12] + [9, 9], 4, 8)
    assert got == 8 and len(fb) == 2 and [t[0] for t in tasks] == blocks[1:3] and all(t[2] == 0 for t in tasks)
    got2, fb2, tasks2 = c.acquire_flexible(toks[4:12] + [9, 9], 0, 8)
    assert got2 == 8 and all(t[2] == -4 for t in tasks2)     # one block earlier than where it was computed
    assert c.check_invariants()[0]


# ----------------------------------------------------------------------------------- control plane
def test_control_plane_barrier_layers_blocknum_broadcast():
    master = ne.ControlMaster("127.0.0.1", 0, 3, 50, 2000)
    workers = [ne.ControlWorker("127.0.0.1", master.port, r, 50, 2000) for r in (1, 2)]
    assert all(w.connect(3000) for w in workers)
    assert master.wait_for_nodes(3000)
    res = {}

    def wk(i, w):
        res[("bar", i)] = w.barrier(3000)
        res[("layers", i)] = w.get_layers(3000)
        res[("blocks", i)] = w.sync_block_num(10 - i * 3, 3000)
        res[("bc", i)] = w.recv_broadcast(3000)

    ts = [threading.Thread(target=wk, args=(i, w)) for i, w in enumerate(workers, 1)]
    [t.start() for t in ts]
    assert master.barrier(3000)
    ranges = master.assign_layers(32, 3000)
    assert ranges == [(0, 10), (11, 21), (22, 31)]
    assert master.sync_block_num(6, 3000) == 4
    assert master.broadcast(b"plan-bytes")
    [t.join() for t in ts]
    assert res[("bar", 1)] and res[("bar", 2)]
    assert res[("layers", 1)] == (11, 21) and res[("layers", 2)] == (22, 31)
    assert res[("blocks", 1)] == 4 and res[("blocks", 2)] == 4
    assert res[("bc", 1)] == b"plan-bytes" and res[("bc", 2)] == b"plan-bytes"
    assert ne.split_layers(32, 2) == [(0, 15), (16, 31)]
    master.shutdown_cluster()
    time.sleep(0.2)
    assert all(w.shutdown_requested() for w in workers)
    [w.stop() for w in workers]; master.stop()


def test_failure_detection_by_eof_and_missed_heartbeats():
    """Host-side fault injection only: a worker that closes its socket, and one that stops heart-beating."""
    master = ne.ControlMaster("127.0.0.1", 0, 2, 30, 300)
    w = ne.ControlWorker("127.0.0.1", master.port, 1, 30, 300)
    assert w.connect(3000) and master.wait_for_nodes(3000) and master.alive()
    w.stop()                                            # peer exits between steps
    for _ in range(100):
        if not master.alive():
            break
        time.sleep(0.02)
    assert not master.alive() and master.failed_nodes() == [1]
    assert master.barrier(200) is False                 # collectives fail fast instead of hanging
    master.stop()
    # silent worker: registers, then never heart-beats (huge interval) -> the master times it out
    master = ne.ControlMaster("127.0.0.1", 0, 2, 30, 200)
    silent = ne.ControlWorker("127.0.0.1", master.port, 1, 10_000_000, 10_000_000)
    assert silent.connect(3000) and master.wait_for_nodes(3000)
    for _ in range(150):
        if not master.alive():
            break
        time.sleep(0.02)
    assert not master.alive()
    # and the other direction: the master disappears, the worker notices
    m2 = ne.ControlMaster("127.0.0.1", 0, 2, 30, 300)
    w2 = ne.ControlWorker("127.0.0.1", m2.port, 1, 30, 300)
    assert w2.connect(3000) and m2.wait_for_nodes(3000)
    m2.stop()
    for _ in range(100):
        if not w2.alive():
            break
        time.sleep(0.02)
    assert not w2.alive() and w2.barrier(200) is False
    w2.stop(); silent.stop(); master.stop()


# ----------------------------------------------------------------------------------- FSM
def test_fsm_segments_and_steps():
    f = ne.FiniteStateMachine(r'\{"name": "[\w\d\s]*", "age": [\d]+\}')
    segs = f.segments()
    assert [t for t, _ in segs] == [0, 1, 0, 1, 0]
    assert segs[0][1] == '{"name": "' and segs[2][1] == '", "age": ' and segs[4][1] == '}'
    changed, final, text, seg, start = f.step("", 0, 0)
    assert changed and not final and text == '{"name": "' and seg == 1
    # free generation continues until the next constant's first character shows up
    assert f.step(text + "Bob Sm", seg, start)[:3] == (False, False, text + "Bob Sm")
    changed, final, text2, seg2, start2 = f.step(text + 'Bob Smith"xyz', seg, start)
    assert changed and text2 == '{"name": "Bob Smith", "age": ' and seg2 == 3
    changed, final, text3, seg3, _ = f.step(text2 + "42}", seg2, start2)
    assert final and text3 == '{"name": "Bob Smith", "age": 42}'
    ctl = ne.FsmController()
    assert ctl.get_or_create("a[0-9]+b") is ctl.get_or_create("a[0-9]+b") and ctl.size() == 1
    assert [t for t, _ in ne.FiniteStateMachine(r"yes|no").segments()] == [1]
    assert ne.FiniteStateMachine(r"a\.b\n").segments() == [(0, "a.b\n")]


# ----------------------------------------------------------------------------------- profiler
def test_metrics_spans_and_chrome_trace(tmp_path):
    ne.metrics_reset()
    names = ne.metric_names()
    assert len(names) == 25 and "time_to_first_token_ms" in names and "block_num_free" in names
    ne.report_metric("time_to_first_token_ms", 12.5)
    ne.report_metric("time_to_first_token_ms", 7.5)
    ne.report_counter("forward_req_total_num", 3)
    snap = ne.metrics_snapshot()
    assert snap["time_to_first_token_ms"]["count"] == 2 and snap["time_to_first_token_ms"]["sum"] == 20.0
    assert snap["forward_req_total_num"]["sum"] == 3
    text = ne.metrics_prometheus()
    assert "ksana_time_to_first_token_ms_count 2" in text and "ksana_block_num_used_count 0" in text
    assert json.loads(ne.metrics_json())["metrics"]["forward_req_total_num"]["sum"] == 3
    tp = "00-0af7651916cd43dd8448eb211c80319c-b7ad6b7169203331-01"
    sid = ne.span_start("generate", tp)
    ne.span_end(sid, {"code": "0"})
    span = json.loads(ne.spans_finished()[-1])
    assert span["trace_id"] == "0af7651916cd43dd8448eb211c80319c" and span["parent_id"] == "b7ad6b7169203331"
    path = str(tmp_path / "trace.json")
    assert set(ne.trace_event_names()) >= {"SchedBegin", "Prefill", "Decode", "SwapOut", "SwapIn", "FinishReq"}
    ne.trace_enable(path)
    ne.trace_record("Prefill", "B", 0, 17)
    ne.trace_record("Prefill", "E", 0, 17)
    ne.trace_record("UsableBlockNum", "C", 0, 99)
    ne.trace_disable()
    events = json.load(open(path))
    assert [e["name"] for e in events[:3]] == ["Prefill", "Prefill", "UsableBlockNum"] and events[2]["args"]["value"] == 99


# ----------------------------------------------------------------------------------- config
REFERENCE_STYLE_YAML = """
setting:
  global:
    tensor_para_size: 2
    pipeline_para_size: 1
    enable_lora_adapter: false
    embed_tokens_use_cpu: false
    enable_cuda_graph: false
  batch_scheduler:
    schedule_strategy: 0
    waiting_timeout_in_ms: 3600000
    max_waiting_queue_len: 1200
    max_step_tokens: 4096
    max_batch_size: 128
    max_token_len: 2048
    swapout_block_threshold: 1.0
    swapin_block_threshold: 2.0
    launch_block_threshold: 2.0
    enable_auto_prefix_cache: true
    split_fuse_token_num: 256
    swap_threadpool_size: 8
    preempt_mode: 0
    min_flexible_cache_num: 0
  block_manager:
    block_token_num: 16
    reserved_device_memory_ratio: 0.01
    lora_deivce_memory_ratio: 0.0
    lora_host_memory_factor: 10.0
    block_device_memory_ratio: -1.0
    block_host_memory_factor: 2.0
  quantization_config:
    gptq_backend: cutlass
    kv_cache:
      dtype: fp8_e4m3
    weight:
      quant_method: auto
  profiler:
    export_interval_millis: 30000
    export_timeout_millis: 1000
    attributes:
      instance: "1.1.1.1"
      version: "1.1"
  endpoint_type: python
  some_future_key: 1
model_spec:
  base_model:
    model_dir: ./model
  plugin_model:
    enable_tensorrt: true
    plugin_thread_pool_size: 1
"""


def test_yaml_config_schema_and_defaults(tmp_path):
    p = tmp_path / "ksana_llm.yaml"
    p.write_text(REFERENCE_STYLE_YAML)
    c = cfgmod.load_yaml_config(str(p))
    assert c.global_.tensor_para_size == 2 and c.batch_scheduler.max_batch_size == 128
    assert c.batch_scheduler.split_fuse_token_num == 256 and c.batch_scheduler.enable_auto_prefix_cache
    assert c.block_manager.block_host_memory_factor == 2.0 and c.quantization.kv_cache_dtype == "fp8_e4m3"
    assert c.profiler.attributes == {"instance": "1.1.1.1", "version": "1.1"}
    assert c.model_dir == str(tmp_path / "model") and c.tokenizer_dir == c.model_dir
    d = cfgmod.EngineConfig()            # defaults of the reference's structs
    assert (d.batch_scheduler.max_batch_size, d.batch_scheduler.max_waiting_queue_len, d.batch_scheduler.waiting_timeout_in_ms,
            d.batch_scheduler.max_step_tokens, d.block_manager.reserved_device_memory_ratio,
            d.block_manager.block_host_memory_factor) == (8, 256, 600000, 4096, 0.05, 10.0)
    with pytest.raises(ValueError):
        cfgmod.load_yaml_config({"setting": {"quantization_config": {"kv_cache": {"dtype": "int3"}}}})


def test_hf_model_config_variants():
    llama3 = {"model_type": "llama", "hidden_size": 8192, "num_hidden_layers": 80, "num_attention_heads": 64,
              "num_key_value_heads": 8, "intermediate_size": 28672, "vocab_size": 128256, "rope_theta": 500000.0,
              "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "eos_token_id": [128001, 128009],
              "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 8192}}
    m = cfgmod.model_config_from_hf(llama3)
    assert (m.head_dim, m.num_kv_heads, m.eos_token_ids) == (128, 8, [128001, 128009]) and m.rope_scaling["factor"] == 8.0
    q = cfgmod.model_config_from_hf({"model_type": "qwen2", "hidden_size": 8192, "num_attention_heads": 64,
                                     "num_key_value_heads": 8, "num_hidden_layers": 80, "intermediate_size": 29568,
                                     "vocab_size": 152064})
    assert q.model_type == "qwen" and q.qkv_bias
    g = cfgmod.model_config_from_hf({"model_type": "gpt2", "n_embd": 768, "n_layer": 12, "n_head": 12, "vocab_size": 50257})
    assert g.norm_type == "layernorm" and not g.gated_mlp and g.position_embedding == "learned" and g.tie_word_embeddings
    b = cfgmod.model_config_from_hf({"model_type": "baichuan", "hidden_size": 5120, "num_attention_heads": 40,
                                     "num_hidden_layers": 40, "intermediate_size": 13696, "vocab_size": 125696})
    assert b.position_embedding == "alibi" and b.lm_head_norm
    glm = cfgmod.model_config_from_hf({"model_type": "chatglm", "hidden_size": 4096, "num_attention_heads": 32,
                                       "num_layers": 28, "ffn_hidden_size": 13696, "multi_query_group_num": 2,
                                       "multi_query_attention": True, "padded_vocab_size": 65024, "kv_channels": 128})
    assert glm.rotary_dim == 64 and not glm.rope_neox and glm.num_kv_heads == 2
    ds = cfgmod.model_config_from_hf({"model_type": "deepseek_v3", "hidden_size": 7168, "num_hidden_layers": 61,
                                      "num_attention_heads": 128, "n_routed_experts": 256, "num_experts_per_tok": 8,
                                      "moe_intermediate_size": 2048, "n_shared_experts": 1, "kv_lora_rank": 512,
                                      "q_lora_rank": 1536, "qk_nope_head_dim": 128, "qk_rope_head_dim": 64,
                                      "v_head_dim": 128, "first_k_dense_replace": 3, "n_group": 8, "topk_group": 4,
                                      "intermediate_size": 18432, "vocab_size": 129280,
                                      "quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}})
    assert ds.is_mla and ds.is_moe and ds.moe_scoring == "sigmoid" and ds.fp8_checkpoint and ds.head_dim == 192
    assert cfgmod.kv_block_bytes(m, 16, 8, 1, 2) == 80 * 1 * 128 * 16 * 2 * 2
    with pytest.raises(ValueError):
        cfgmod.check_tp(m, 3)


def test_kv_scale_file(tmp_path):
    p = tmp_path / "kv_cache_scales.json"
    p.write_text(json.dumps({"kv_cache": {"dtype": "float8_e4m3fn", "scaling_factor": {"0": {"0": 0.5, "1": 0.25}}}}))
    assert cfgmod.load_kv_scales(str(p), 2) == [[0.5, 0.5], [0.25, 0.25]]


def test_native_msgpack_matches_the_python_codec_and_validates_forward_bodies():
    import msgpack
    import pytest
    from ksanallm_b200.utils import native_engine as ne
    docs = [None, True, 0, 127, 128, 255, 256, 65535, 65536, 2**32, 2**63 - 1, 2**64 - 1, -1, -32, -33, -129, -32769, -2**31 - 1,
            -2**63, 1.5, -0.25, "", "héllo", "x" * 40, "y" * 300, b"", b"\x00\x01" * 200, [], [1, [2, [3]]], list(range(20)),
            {"a": 1, "b": {"c": [1.0, None, b"zz"]}}, {str(i): i for i in range(20)}]
    for d in docs:
        packed = ne.msgpack_pack(d)
        assert msgpack.unpackb(packed, raw=False, strict_map_key=False) == d
        assert ne.msgpack_unpack(msgpack.packb(d, use_bin_type=True)) == d
    assert ne.msgpack_unpack(msgpack.packb(1.5, use_single_float=True)) == 1.5
    big = {"requests": [{"input_tokens": list(range(70000)), "request_target": [{"target_name": "logits"}]}]}
    assert ne.unpack_forward_body(msgpack.packb(big))["requests"][0]["input_tokens"][-1] == 69999
    for bad in (b"\xc1", b"\x92\x01", msgpack.packb(1) + b"\x00", b"\xd4\x01\x00"):
        with pytest.raises(RuntimeError):
            ne.msgpack_unpack(bad)
    ok = {"requests": [{"input_tokens": [1, 2, 3], "request_target": [
        {"target_name": "transformer", "slice_pos": [[0, 1]], "token_reduce_mode": "GATHER_ALL"}]}]}
    assert ne.unpack_forward_body(msgpack.packb(ok)) == ok
    for broken, why in ((dict(requests=[]), "no requests"),
                        (dict(requests=[{"input_tokens": [1], "request_target": []}]), "request_target is empty"),
                        (dict(requests=[{"request_target": [{"target_name": "logits"}]}]), "input_tokens or a prompt"),
                        (dict(requests=[{"input_tokens": [1], "request_target": [{"target_name": "bogus"}]}]), "unknown target_name"),
                        (dict(requests=[{"input_tokens": [1], "request_target": [{"target_name": "logits", "slice_pos": [[1]]}]}]),
                         "slice_pos")):
        with pytest.raises(ValueError, match=why):
            ne.unpack_forward_body(msgpack.packb(broken))


def test_stop_checker_incremental_search():
    """Native stop-string checker: pieces arrive one by one, a stop string may straddle pieces, the earliest
    match wins, half a UTF-8 character is reported as incomplete."""
    from ksanallm_b200.utils import native_engine as ne
    c = ne.StopChecker(["END", "stop here", ""])
    assert c.append("abc E") == -1 and c.append("N") == -1
    assert c.append("D tail") == 4 and c.kept() == "abc "
    assert c.append("more END") == 4                      # stays on the first hit
    c.reset()
    assert c.append("x stop") == -1 and c.append(" he") == -1 and c.append("re END") == 2 and c.kept() == "x "
    c2 = ne.StopChecker(["é!"])
    assert c2.append("caf") == -1 and c2.append("é") == -1 and c2.append("!") == 3 and c2.kept() == "caf"
    assert ne.StopChecker.ends_incomplete("ab�") and not ne.StopChecker.ends_incomplete("abé")
    assert not ne.StopChecker.ends_incomplete("")
    none = ne.StopChecker([])
    assert none.append("anything") == -1 and none.kept() == "anything"


def test_example_configurations_load():
    """Every YAML under examples/ goes through the parser and keeps its parallel layout."""
    import glob
    import os
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
    files = sorted(glob.glob(os.path.join(root, "*.yaml")) + glob.glob(os.path.join(root, "*", "*.yaml")))
    assert len(files) >= 6
    seen = {}
    for f in files:
        c = cfgmod.load_yaml_config(f)
        seen[os.path.basename(f)] = c
        assert c.batch_scheduler.max_batch_size >= 1 and c.block_manager.block_token_num in (16, 32, 64, 128)
    assert seen["ksana_llm.yaml"].batch_scheduler.max_batch_size >= 1
    assert seen["ksana_llm_70b_fp8_tp8.yaml"].global_.tensor_para_size == 8
    assert seen["ksana_llm_70b_fp8_tp8.yaml"].quantization.weight_quant_method == "fp8_block"
    assert seen["ksana_llm_pipeline.yaml"].global_.pipeline_para_size == 2
    assert seen["ksana_llm_deepseek_v3_ep8.yaml"].global_.attn_data_para_size == 8
    assert seen["ksana_llm_deepseek_v3_ep8.yaml"].global_.expert_para_size == 8


def test_import_compatibility_package():
    """`import ksana_llm` exposes the serving surface of the reference's Python package."""
    import ksana_llm
    from ksanallm_b200.serving.auto_model import AutoModel
    assert ksana_llm.AutoModel is AutoModel
    assert {"AutoModel", "EndpointConfig", "PluginConfig"} <= set(ksana_llm.__all__)
    assert ksana_llm.EndpointConfig().endpoint == "python" and ksana_llm.EndpointConfig(endpoint="trpc", port=9000).type == "trpc"
    assert ksana_llm.PluginConfig(thread_pool_size=4).thread_pool_size == 4
    for bad in ("/no/such/file.yaml", __file__):               # missing, and not a YAML file
        with pytest.raises(RuntimeError):
            ksana_llm.AutoModel.from_config(bad)


def test_lost_worker_rank_ends_the_service(tmp_path):
    """Failure detection reaches the engine (host only): rank 1 of a two-rank CPU engine exits between two steps; rank
    0's liveness monitor sees the closed control connection, the requests in flight are answered with RET_RUNTIME and
    the process leaves with a non-zero code instead of waiting forever in the step-plan broadcast."""
    import json
    import socket
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    out = str(tmp_path / "lifetime.json")
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), KSANA_CONTROL_PORT=str(port + 1), KSANA_HEARTBEAT_INTERVAL_MS="100",
                   KSANA_HEARTBEAT_TIMEOUT_MS="2000", OMP_NUM_THREADS="1", DISABLE_WARMUP="1", KLLM_LOG_FILE="stderr")
        procs.append(subprocess.Popen([sys.executable, os.path.join(root, "tests", "lifetime_worker.py"), out], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert procs[1].returncode == 0, outs[1][-2000:]
    assert procs[0].returncode == 1, outs[0][-3000:]
    got = json.load(open(out))
    assert "lost" in got["reason"] and got["fatal"]
    assert all(code == 12 and done for code, done, _ in got["statuses"]), got
    assert "service shutdown" in outs[0]


def test_native_logger_levels_file_and_python_bridge(tmp_path):
    """KLLM_LOG_LEVEL / KLLM_LOG_FILE semantics of the native logger and the Python bridge on top of it."""
    import logging
    from ksanallm_b200.utils import logger
    path = str(tmp_path / "logs" / "engine.log")          # the directory is created on demand
    old_file, old_level = logger.log_file(), ne.log_level()
    try:
        logger.set_file(path)
        logger.set_level("WARNING")
        logger.info("not written")
        logger.warning("disk almost full")
        logger.error("step failed")
        assert not ne.log_enabled(logger.INFO) and ne.log_enabled(logger.ERROR)
        logger.set_level("DEBUG")
        logger.debug("details")
        h = logger.NativeLogHandler()
        lg = logging.getLogger("ksana-test")
        lg.addHandler(h)
        lg.setLevel(logging.INFO)
        lg.info("from python logging %d", 7)
        lg.removeHandler(h)
        logger.set_file("stderr")
        text = open(path).read().splitlines()
    finally:
        logger.set_file(old_file)
        ne.set_log_level(["DEBUG", "INFO", "WARNING", "ERROR", "FATAL"][old_level])
    assert len(text) == 4 and "not written" not in "".join(text)
    assert " WARNING " in text[0] and text[0].endswith("] disk almost full") and "test_host_components.py:" in text[0]
    assert " ERROR " in text[1] and " DEBUG " in text[2]
    assert "from python logging 7" in text[3] and "ksana-test" in text[3]


def test_weight_maps_accept_dollar_groups(tmp_path):
    """A weight map written for the reference engine names capture groups as $1 (std::regex_replace); such a file
    loads and renames like the same map written with Python's \\1."""
    from ksanallm_b200.models.weights import apply_weight_map, load_weight_map
    ref_style = {"transformer.h.(\\d+).ln_(\\d).weight": "model.layers.$1.norm$2.weight", "transformer.wte.weight": "model.embed_tokens.weight"}
    py_style = {"transformer.h.(\\d+).ln_(\\d).weight": "model.layers.\\1.norm\\2.weight", "transformer.wte.weight": "model.embed_tokens.weight"}
    pa, pb = tmp_path / "a.json", tmp_path / "b.json"
    pa.write_text(json.dumps(ref_style))
    pb.write_text(json.dumps(py_style))
    ra, rb = load_weight_map("x", str(pa)), load_weight_map("x", str(pb))
    for name in ("transformer.h.12.ln_2.weight", "transformer.wte.weight", "lm_head.weight"):
        assert apply_weight_map(name, ra) == apply_weight_map(name, rb)
    assert apply_weight_map("transformer.h.12.ln_2.weight", ra) == "model.layers.12.norm2.weight"


def test_otlp_http_export_of_spans_and_metrics():
    """Export targets that are http:// URLs speak OTLP/HTTP with JSON bodies: finished spans arrive at /v1/traces as
    one ExportTraceServiceRequest (resource attributes, ids, parent from the traceparent header, unix-nanosecond times,
    span attributes) and the periodic metrics export at /v1/metrics (counters as cumulative monotonic sums,
    distributions as histograms with count / sum / min / max). A collector that is away costs dropped requests,
    never a blocked caller."""
    import json
    import socket
    import threading
    import time
    from http.server import BaseHTTPRequestHandler, HTTPServer

    got = {"/v1/traces": [], "/v1/metrics": []}

    class Collector(BaseHTTPRequestHandler):
        def do_POST(self):
            body = self.rfile.read(int(self.headers["Content-Length"]))
            assert self.headers["Content-Type"] == "application/json"
            got[self.path].append(json.loads(body))
            self.send_response(200)
            self.send_header("Content-Length", "2")
            self.end_headers()
            self.wfile.write(b"{}")

        def log_message(self, *a):
            pass

    srv = HTTPServer(("127.0.0.1", 0), Collector)
    port = srv.server_address[1]
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    try:
        ne.metrics_reset()
        ne.metrics_set_attributes({"instance": "node-7"})
        ne.otlp_configure({"instance": "node-7"}, 500)
        ne.span_set_sink(f"http://127.0.0.1:{port}/v1/traces")
        parent = "00-0af7651916cd43dd8448eb211c80319c-b7ad6b7169203331-01"
        t_before = time.time_ns()
        sid = ne.span_start("generate", parent)
        time.sleep(0.01)
        ne.span_end(sid, {"output_tokens": "5"})
        sid2 = ne.span_start("forward", "")
        ne.span_end(sid2)
        ne.report_counter("forward_req_total_num", 3)
        ne.report_metric("time_to_first_token_ms", 12.5)
        ne.report_metric("time_to_first_token_ms", 7.5)
        ne.metrics_start_export(f"http://127.0.0.1:{port}/v1/metrics", 50)
        deadline = time.time() + 10
        while time.time() < deadline and not (got["/v1/traces"] and got["/v1/metrics"]):
            ne.otlp_flush(200)
            time.sleep(0.05)
        ne.metrics_stop_export()
        ne.otlp_flush(2000)
    finally:
        ne.span_set_sink("")
        srv.shutdown()
    spans = [s for req in got["/v1/traces"] for rs in req["resourceSpans"] for ss in rs["scopeSpans"] for s in ss["spans"]]
    res_attrs = {a["key"]: a["value"]["stringValue"] for a in got["/v1/traces"][0]["resourceSpans"][0]["resource"]["attributes"]}
    assert res_attrs["instance"] == "node-7" and res_attrs["service.name"] == "ksana_llm"
    gen = next(s for s in spans if s["name"] == "generate")
    assert gen["traceId"] == "0af7651916cd43dd8448eb211c80319c" and gen["parentSpanId"] == "b7ad6b7169203331"
    assert gen["spanId"] == sid and len(gen["spanId"]) == 16
    assert int(gen["endTimeUnixNano"]) - int(gen["startTimeUnixNano"]) >= 9_000_000
    assert abs(int(gen["startTimeUnixNano"]) - t_before) < 5_000_000_000          # wall-clock time, not a monotonic one
    assert {a["key"]: a["value"]["stringValue"] for a in gen["attributes"]} == {"output_tokens": "5"}
    fwd = next(s for s in spans if s["name"] == "forward")
    assert "parentSpanId" not in fwd and len(fwd["traceId"]) == 32
    metrics = {m["name"]: m for req in got["/v1/metrics"] for rm in req["resourceMetrics"] for sm in rm["scopeMetrics"]
               for m in sm["metrics"]}
    c = metrics["ksana_forward_req_total_num"]["sum"]
    assert c["isMonotonic"] and c["aggregationTemporality"] == 2 and c["dataPoints"][0]["asDouble"] == 3
    h = metrics["ksana_time_to_first_token_ms"]["histogram"]["dataPoints"][0]
    assert h["count"] == "2" and h["sum"] == 20 and h["min"] == 7.5 and h["max"] == 12.5
    # nobody listens: the request is dropped after the timeout and counted, the caller never waits
    sent0, dropped0 = ne.otlp_stats()
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    dead_port = sock.getsockname()[1]
    sock.close()
    ne.span_set_sink(f"http://127.0.0.1:{dead_port}/v1/traces")
    t0 = time.perf_counter()
    ne.span_end(ne.span_start("lost", ""))
    assert time.perf_counter() - t0 < 0.5
    ne.otlp_flush(3000)
    ne.span_set_sink("")
    sent1, dropped1 = ne.otlp_stats()
    assert dropped1 == dropped0 + 1 and sent1 == sent0


def test_native_batch_loop_sleeps_wakes_and_survives_errors():
    """The engine's loop thread in C++: runs the step callable while it reports work, sleeps on its condition variable
    while the idle callable says so (no spinning), wakes within milliseconds of `notify`, hands an exception that
    escapes a step to the error callable and keeps going, and stops promptly."""
    import threading
    import time
    work = {"n": 0, "pending": 0, "errors": []}
    lock = threading.Lock()
    woke = threading.Event()

    def step():
        with lock:
            if work["pending"] == 0:
                return False
            work["pending"] -= 1
            work["n"] += 1
            if work["n"] == 3:
                raise ValueError("third step fails")
        woke.set()
        return True

    loop = ne.BatchLoop()
    loop.start(step, lambda: work["pending"] == 0, lambda msg: work["errors"].append(msg))
    try:
        time.sleep(0.3)
        assert loop.running and loop.steps == 0 and loop.sleeps <= 10         # idle: asleep, not polling
        with lock:
            work["pending"] = 5
        t0 = time.perf_counter()
        loop.notify()
        assert woke.wait(5.0) and time.perf_counter() - t0 < 1.0
        deadline = time.time() + 5
        while time.time() < deadline and work["pending"]:
            time.sleep(0.01)
        assert work["pending"] == 0 and work["n"] == 5
        assert loop.steps == 4                                              # the failing step does not count as run
        assert len(work["errors"]) == 1 and "third step fails" in work["errors"][0]
    finally:
        t0 = time.perf_counter()
        loop.stop()
        assert time.perf_counter() - t0 < 3.0 and not loop.running
    loop.stop()                                                             # twice is fine


def test_clock_record_parser_and_breakdown_helpers():
    """The nvidia-smi clock record (median SM clock, maximum, throttle reasons that were active in any sample; absent
    tool reported as such) and the launch-class key of the step breakdown tool."""
    import importlib.util
    import os
    from ksanallm_b200.utils.clocks import ClockSampler
    c = ClockSampler(0)
    c.lines = ["0, 1965, 1965, 410.5, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
               "0, 1470, 1965, 998.2, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1455, 1965, 1001.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "garbage line"]
    c.proc = type("P", (), {"terminate": lambda s: None, "wait": lambda s, timeout=0: None, "kill": lambda s: None})()
    rec = c.stop()
    assert rec == {"sm_mhz": 1470.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    off = ClockSampler(0, enabled=False)
    off.start()
    assert off.stop()["sm_mhz"] is None
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("step_breakdown", os.path.join(root, "benchmarks", "step_breakdown.py"))
    sb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sb)
    key = sb._class_key("ksana_gemm_smallm", (2, 140737488355328, 8192, None, 64, True, 1280, 0.5, 9999999999))
    assert key == "gemm_smallm(2,8192,64,1280)"          # pointers, floats, flags and huge values do not split classes


def test_native_waiter_and_stream_channel_behave_like_event_and_queue():
    """The request path's blocking primitives in C++: `Waiter` (set / is_set / wait with a timeout in seconds) and
    `StreamChannel` (put / get with a timeout raising queue.Empty, FIFO order, any Python object as an item); a waiting
    thread holds no interpreter lock, so other threads keep running meanwhile."""
    import queue
    import threading
    import time
    w = ne.Waiter()
    assert not w.is_set()
    t0 = time.perf_counter()
    assert w.wait(0.05) is False and 0.04 < time.perf_counter() - t0 < 2.0
    ticks = []
    stop = threading.Event()

    def spin():
        while not stop.is_set():
            ticks.append(1)
            time.sleep(0.001)

    th = threading.Thread(target=spin)
    th.start()
    threading.Timer(0.1, w.set).start()
    assert w.wait(5.0) and w.is_set() and w.wait() is True
    stop.set()
    th.join()
    assert len(ticks) > 5                       # the spinner ran while the main thread was blocked in wait()
    w.clear()
    assert not w.is_set()
    c = ne.StreamChannel()
    with pytest.raises(queue.Empty):
        c.get(timeout=0.05)
    items = [("step", [[1, 2], [3]]), {"k": "v"}, None, 7]
    for it in items:
        c.put(it)
    assert c.qsize() == 4 and [c.get(timeout=1) for _ in items] == items and c.empty()
    threading.Timer(0.05, lambda: c.put("late")).start()
    assert c.get(timeout=5) == "late"


@pytest.mark.parametrize("size,max_tokens,hidden", [(1, 512, 1024), (2, 512, 1024), (4, 16384, 8192), (8, 16384, 8192),
                                                    (8, 64, 8192), (3, 1000, 5120)])
def test_symmetric_buffer_layout_for_every_group_size(size, max_tokens, hidden):
    """Layout arithmetic of the peer-mapped buffer (no device needed): regions do not overlap, every region starts on
    a 256-byte boundary (16-byte vector and multimem accesses), a receive slot holds a rank's share of a large batch
    and every row of a decode-sized one, and the two slot sets hold one slot per rank each."""
    from ksanallm_b200.parallel.symm import CAND_MAX_K, FLAG_BYTES, ONE_SHOT_ROWS, SymmetricComm
    lay = SymmetricComm.layout(size, max_tokens, hidden)
    row = hidden * 2
    assert lay["slot_rows"] >= ONE_SHOT_ROWS and lay["slot_rows"] * size >= max_tokens
    assert lay["slot_bytes"] >= lay["slot_rows"] * row
    regions = [(0, FLAG_BYTES)]
    for base in lay["slots_off"]:
        regions += [(base + r * lay["slot_bytes"], lay["slot_bytes"]) for r in range(size)]
    regions += [(lay["h_off"], max_tokens * row), (lay["y_off"], max_tokens * row), (lay["yq_off"], max_tokens * hidden),
                (lay["ys_off"], (hidden // 128 + 1) * lay["scale_ld"] * 4), (lay["stage_off"], lay["stage_bytes"]),
                (lay["cand_off"], lay["cand_words"] * 4)]
    regions.sort()
    for (a, n), (b, _) in zip(regions, regions[1:]):
        assert a + n <= b, (a, n, b)
    assert regions[-1][0] + regions[-1][1] <= lay["total"]
    assert all(start % 256 == 0 for start, _ in regions)
    assert lay["scale_ld"] >= max_tokens and lay["scale_ld"] % 4 == 0
    assert lay["cand_words"] >= 2 * min(max_tokens, 1024) * CAND_MAX_K
    # a partial product of all rows fits the slot area of one parity (pull mode writes it there in one piece)
    assert size * lay["slot_bytes"] >= max_tokens * row


def test_row_parallel_form_by_group_size_and_batch(monkeypatch):
    """Which form a row-parallel linear takes, decided on the host: every rank reduces all rows itself up to 64 rows
    while it pulls at most 8 MB; the GEMM pushes its rows from 4 ranks on (2 ranks pull); the switches override."""
    from ksanallm_b200.parallel.symm import SymmetricComm
    for var in ("KSANA_PUSH", "KSANA_PUSH_PREFILL", "KSANA_ONE_SHOT_ROWS"):
        monkeypatch.delenv(var, raising=False)

    def comm(size, hidden=8192):
        c = SymmetricComm.__new__(SymmetricComm)          # decisions only: no device, no buffer
        c.size, c.hidden = size, hidden
        return c

    for size in (2, 4, 8):
        assert comm(size).one_shot(64) and not comm(size).one_shot(65)
    assert comm(8).one_shot(64) and not comm(8, hidden=16384).one_shot(64)        # 14.7 MB to pull: split over the ranks
    assert [comm(n).push_decode for n in (2, 4, 8)] == [False, True, True]
    assert not comm(8).push_prefill
    monkeypatch.setenv("KSANA_PUSH", "0")
    assert not comm(8).push_decode
    monkeypatch.setenv("KSANA_PUSH", "1")
    assert comm(2).push_decode
    monkeypatch.setenv("KSANA_PUSH_PREFILL", "1")
    assert comm(4).push_prefill
    monkeypatch.setenv("KSANA_ONE_SHOT_ROWS", "16")
    assert comm(4).one_shot(16) and not comm(4).one_shot(17)
