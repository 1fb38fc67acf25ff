"""The serving benchmark client against a live (CPU, tiny model) server: statistics and both request modes."""
import math
import os
import socket
import sys
import threading
import time

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks"))
import benchmark_throughput as bt  # noqa: E402
from helpers import ByteTokenizer, tiny_model_cfg  # noqa: E402


def test_summary_statistics():
    recs = []
    for i in range(4):
        r = bt.RequestRecord(prompt_len=10, output_len=5, start=0.0, first_token=0.1 * (i + 1), end=1.0 + i)
        r.chunk_times = [r.first_token, r.first_token + 0.2, r.first_token + 0.5]
        recs.append(r)
    bad = bt.RequestRecord(prompt_len=3, ok=False)
    s = bt.summarize(recs + [bad], wall=4.0, percentiles=(50, 99))
    assert s["finished"] == 4 and s["failed"] == 1
    assert s["request_throughput"] == 1.0 and s["token_throughput"] == 15.0
    assert math.isclose(s["avg_latency_s"], 2.5) and math.isclose(s["p50_latency_s"], 2.5)
    assert math.isclose(s["avg_ttft_s"], 0.25)
    assert math.isclose(recs[0].tpot, (1.0 - 0.1) / 4)
    assert math.isclose(s["avg_itl_s"], 0.25)
    assert bt.percentile([1, 2, 3, 4], 100) == 4 and math.isnan(bt.percentile([], 50))
    w = bt.synthetic_prompts("5:20:7:0.5", 300, seed=1)
    assert len(w) == 5 and all(o == 7 and all(3 <= t < 300 for t in p) for p, o in w)


@pytest.fixture(scope="module")
def server():
    import uvicorn
    from ksanallm_b200.config import EngineConfig
    from ksanallm_b200.llm import LLM
    from ksanallm_b200.serving.serving_model import ServingModel
    from ksanallm_b200.serving.serving_server import create_app
    tok = ByteTokenizer()
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size = 8
    ec.batch_scheduler.max_token_len = 128
    ec.block_manager.device_blocks_num = 128
    llm = LLM(ec, tiny_model_cfg(), weights="random", device="cpu", dtype=torch.float32, tokenizer=tok)
    model = ServingModel("", llm=llm, tokenizer=tok)
    model.init_serving()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    srv = uvicorn.Server(uvicorn.Config(create_app(model, tok), host="127.0.0.1", port=port, log_level="warning"))
    th = threading.Thread(target=srv.run, daemon=True)
    th.start()
    for _ in range(200):
        if srv.started:
            break
        time.sleep(0.05)
    assert srv.started
    yield port
    srv.should_exit = True
    th.join(timeout=10)
    model.shutdown()


@pytest.mark.parametrize("extra", [["--stream", "--request_rate", "50", "--random"], ["--mode", "sync", "--concurrency", "3"]])
def test_client_against_live_server(server, tmp_path, extra):
    perf = tmp_path / "perf.csv"
    args = bt.args_config(["--port", str(server), "--synthetic", "6:12:5", "--vocab_size", "250", "--perf_csv", str(perf),
                           "--output_csv", str(tmp_path / "out.csv"), "--client_timeout", "60"] + extra)
    res = bt.run_benchmark(args)
    assert len(res) == 1
    s = res[0]
    assert s["finished"] == 6 and s["failed"] == 0
    assert s["avg_output_tokens"] == 5 and s["avg_input_tokens"] == 12
    assert s["token_throughput"] > 0
    if "--stream" in extra:
        assert s["avg_ttft_s"] > 0 and s["p99_ttft_s"] >= s["p50_ttft_s"] and "avg_tpot_s" in s
    assert perf.exists() and (tmp_path / "out.csv").read_text().count("\n") == 7


def test_client_text_prompts_chat_template_stop_strings_and_regex(server, tmp_path):
    """Text prompts from a CSV file wrapped by the tokenizer's chat template, a stop string and a structured-output
    expression read from a file: all reach the server in the request body and the run completes."""
    csv_path = tmp_path / "prompts.csv"
    csv_path.write_text("id,prompt\n1,hello there\n2,second prompt\n3,third\n", encoding="utf-8")
    regex_path = tmp_path / "regex.txt"
    regex_path.write_text("[a-c]{3}\n", encoding="utf-8")
    args = bt.args_config(["--port", str(server), "--input_csv", str(csv_path), "--col_idx", "1", "--max_new_tokens", "6",
                           "--mode", "sync", "--concurrency", "2", "--client_timeout", "60", "--stop_strings", "zzzz",
                           "--structured_output_file", str(regex_path), "--chat_template", "--tokenizer_path", "unused"])
    bt._TOKENIZER = ByteTokenizer()                       # stands in for AutoTokenizer.from_pretrained
    try:
        wrapped = bt.apply_chat_template(args, "hello there")
        assert wrapped == "<user>hello there<assistant>"
        res = bt.run_benchmark(args)
    finally:
        bt._TOKENIZER = None
    assert args.structured_output_regex == "[a-c]{3}"
    body = bt.build_payload(args, wrapped)
    assert body["structured_output_regex"] == "[a-c]{3}" and body["sampling_config"]["stop_strings"] == ["zzzz"]
    assert res[0]["finished"] == 3 and res[0]["failed"] == 0


@pytest.mark.parametrize("config,extra", [("b", ["--requests", "8", "--input-len", "24", "--output-len", "6"]),
                                          ("d", ["--requests", "5", "--output-len", "4"]),
                                          ("e", ["--requests", "6", "--input-len", "40", "--output-len", "8"])])
def test_offline_configurations_toy_mode(config, extra):
    """The offline configuration script end to end on the CPU (toy-sized models of the named architectures): every
    request finishes, the shared-prefix load hits the prefix cache."""
    import json
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "benchmarks", "offline_configs.py"), "--config", config] + extra,
                       capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    assert res["config"] == config and res["finished_ok"] == res["requests"] and res["output_tokens"] > 0
    if config == "d":
        assert res["prefix_hit_tokens"] > 0


def test_command_line_clients_against_live_server(server, capsys):
    """serving_generate_client.py and serving_forward_client.py (the reference's client script names) against the
    live server: blocking and streaming generation, a logits target with perplexity, a hidden-state target."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import serving_forward_client
    import serving_generate_client
    res = serving_generate_client.main(["--port", str(server), "--host", "127.0.0.1", "--prompt", "hello", "--max_new_tokens", "5"])
    assert len(res["output_token_ids"][0]) == 5
    res = serving_generate_client.main(["--port", str(server), "--host", "127.0.0.1", "--input_tokens", "5", "6", "7",
                                        "--max_new_tokens", "4", "--stream"])
    assert res["chunks"] and len(res["chunks"][-1]["output_token_ids"][0]) == 4
    doc = serving_forward_client.main(["--port", str(server), "--host", "127.0.0.1", "--input_tokens", "5", "6", "7", "8", "9",
                                       "--target", "logits", "--reduce", "GATHER_TOKEN_ID", "--slice", "0", "3"])
    t = doc["responses"][0]["response"][0]
    assert t["target_name"] == "logits" and t["tensor"].shape[0] == 4
    doc = serving_forward_client.main(["--port", str(server), "--host", "127.0.0.1", "--prompt", "abcdef", "--target", "layernorm",
                                       "--slice", "0", "1"])
    assert doc["responses"][0]["response"][0]["tensor"].shape[0] == 2
    assert "perplexity" in capsys.readouterr().out
    # the example clients (examples/api_client.py, examples/streaming_client.py)
    import importlib.util
    for name in ("api_client", "streaming_client"):
        spec = importlib.util.spec_from_file_location(name, os.path.join(root, "examples", name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        for extra in ([], ["--stream"]):
            assert mod.main(["--host", "127.0.0.1", "--port", str(server), "--prompt", "hello there"] + extra) == 0
        out = capsys.readouterr().out
        assert ("Answer 0" in out) if name == "api_client" else ("[" in out)
    spec = importlib.util.spec_from_file_location("openai_client", os.path.join(root, "examples", "openai_client.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for extra in ([], ["--stream"]):
        assert mod.main(["--host", "127.0.0.1", "--port", str(server), "--max_tokens", "5", "hello there"] + extra) == 0
    capsys.readouterr()
    # the concurrent example client beside the 7B sample configuration (examples/llama7b/serving_client.py)
    spec = importlib.util.spec_from_file_location("llama7b_client", os.path.join(root, "examples", "llama7b", "serving_client.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for extra in ([], ["--stream"]):
        old_argv = sys.argv
        sys.argv = ["serving_client.py", "--port", str(server), "--max_new_tokens", "4", "--prompt", "hello", "--prompt", "abc"] + extra
        try:
            mod.main()
        finally:
            sys.argv = old_argv
        out = capsys.readouterr().out
        assert "2 requests in" in out and "request failed" not in out and "HTTP " not in out


def test_prompt_sets_and_prefix_cache_reader(tmp_path):
    """The shipped prompt sets load through the client's CSV reader; the prefix-cache set shares its preamble token
    for token, and its engine configuration parses."""
    import importlib.util
    from ksanallm_b200.config import load_yaml_config
    bench_dir = os.path.dirname(os.path.abspath(bt.__file__))
    spec = importlib.util.spec_from_file_location("prefix_cache_reader", os.path.join(bench_dir, "prefix_cache_reader.py"))
    reader = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(reader)
    assert reader.common_prefix_len([[1, 2, 3, 4], [1, 2, 9], [1, 2, 3]]) == 2
    assert reader.common_prefix_len([]) == 0 and reader.common_prefix_len([[5, 6]]) == 2
    path = os.path.join(bench_dir, "prefix_cache_input.csv")
    shared, prompts = reader.load_prompts(path, tokenizer=ByteTokenizer(), count=50)
    assert len(prompts) == 50 and len(set(prompts)) == 24 and prompts[24] == prompts[0]
    assert shared > 700 and all(p.startswith("[INST]You are the assistant") and p.endswith("[/INST]") for p in prompts)
    assert reader.load_prompts(path, count=0)[0] == 0                       # no tokenizer: nothing measured
    bad = tmp_path / "bad.csv"
    bad.write_text("description\nid,text\n0,hello\n")
    with pytest.raises(ValueError):
        reader.load_prompts(str(bad))
    qs = bt.read_prompts(os.path.join(bench_dir, "benchmark_input.csv"), 0, 0, False, 0)
    assert len(qs) == 32 and all(q.startswith("Think about") for q in qs)
    # the chat-style set is what its generator produces (same seed, bit for bit), long-tailed in length
    spec = importlib.util.spec_from_file_location("make_chat_prompts", os.path.join(bench_dir, "make_chat_prompts.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    chat = bt.read_prompts(os.path.join(bench_dir, "chat_prompts_500.csv"), 0, 0, False, 0)
    assert chat == gen.build(500, 0)
    lens = sorted(len(q) for q in chat)
    assert lens[250] < 400 and lens[-1] > 3000 and lens[0] > 10
    ec = load_yaml_config(os.path.join(bench_dir, "prefix_cache_config.yaml"))
    assert ec.batch_scheduler.enable_auto_prefix_cache and ec.batch_scheduler.max_batch_size == 256


@pytest.mark.parametrize("config,extra", [("b", ["--requests", "6", "--input-len", "20", "--output-len", "5"]),
                                          ("e", ["--requests", "4", "--input-len", "24", "--output-len", "4"])])
def test_offline_configurations_two_ranks_exit(config, extra):
    """Two tensor-parallel ranks of the offline configuration script (CPU, gloo): the result line is printed and both
    processes leave on their own (the worker rank is released by the end-of-batch signal, not by a stop signal)."""
    import json
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    port = 29750 + (0 if config == "b" else 1)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(root, "benchmarks", "offline_configs.py"), "--config", config] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    res = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    assert res["n_gpus"] == 2 and res["finished_ok"] == res["requests"]


@pytest.fixture(scope="module")
def foreign_servers():
    """Stand-ins for other serving stacks: each answers in that stack's own request / answer format."""
    import json
    import uvicorn
    from fastapi import FastAPI, Request
    from fastapi.responses import JSONResponse, StreamingResponse
    app = FastAPI()
    seen = {}

    @app.post("/generate")
    async def generate(req: Request):
        body = await req.json()
        if "sampling_params" in body:                       # sglang
            seen["sglang"] = body
            return JSONResponse({"text": " four words of text", "meta_info": {"prompt_tokens": 7, "completion_tokens": 4}})
        seen["vllm"] = body                                  # vllm: the prompt is echoed, chunks end with a zero byte
        words = [" one", " two", " three"]
        if body.get("stream"):
            async def chunks():
                text = body["prompt"]
                for w in words:
                    text += w
                    yield json.dumps({"text": [text]}).encode() + b"\0"
            return StreamingResponse(chunks())
        return JSONResponse({"text": [body["prompt"] + "".join(words)]})

    @app.post("/v2/models/ensemble/generate_stream")
    async def trt(req: Request):
        seen["trt-llm"] = await req.json()

        async def events():
            for i in range(1, 4):
                yield ("data: " + json.dumps({"text_output": "tok " * i}) + "\n\n").encode()
        return StreamingResponse(events(), media_type="text/event-stream")

    @app.post("/v1/chat")
    async def chat(req: Request):
        seen["chat"] = await req.json()

        async def events():
            for w in ("Hel", "lo ", "you"):
                yield ("data: " + json.dumps({"choices": [{"delta": {"content": w}}]}) + "\n\n").encode()
            yield ("data: " + json.dumps({"choices": [{"delta": {"content": ""}}],
                                          "usage": {"prompt_tokens": 5, "completion_tokens": 3}}) + "\n\n").encode()
            yield b"data: [DONE]\n\n"
        return StreamingResponse(events(), media_type="text/event-stream")

    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    srv = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
    th = threading.Thread(target=srv.run, daemon=True)
    th.start()
    for _ in range(200):
        if srv.started:
            break
        time.sleep(0.05)
    assert srv.started
    yield port, seen
    srv.should_exit = True
    th.join(timeout=10)


@pytest.mark.parametrize("backend,stream,n_in,n_out", [("vllm", True, 0, 0), ("vllm", False, 0, 0), ("sglang", False, 7, 4),
                                                       ("trt-llm", True, 0, 0), ("vllm-server", True, 5, 3)])
def test_client_speaks_other_backends(foreign_servers, tmp_path, backend, stream, n_in, n_out):
    """--backend picks the URL, the request body and the answer format of another serving stack; latency statistics
    come out the same way, token counts from the answer where the stack reports them."""
    port, seen = foreign_servers
    csv_path = tmp_path / "prompts.csv"
    csv_path.write_text("question\nwhat is this\nand that\n", encoding="utf-8")
    out_csv = tmp_path / "out.csv"
    argv = ["--port", str(port), "--backend", backend, "--input_csv", str(csv_path), "--max_new_tokens", "9",
            "--client_timeout", "30", "--output_csv", str(out_csv)] + (["--stream"] if stream else [])
    res = bt.run_benchmark(bt.args_config(argv))
    s = res[0]
    assert s["finished"] == 2 and s["failed"] == 0
    assert s["avg_input_tokens"] == n_in and s["avg_output_tokens"] == n_out
    if stream:
        assert s["avg_ttft_s"] > 0
    text = out_csv.read_text()
    if backend == "vllm":
        assert seen["vllm"]["max_tokens"] == 9 and "one two three" in text and "what is this one" not in text
    elif backend == "sglang":
        assert seen["sglang"]["sampling_params"]["max_new_tokens"] == 9 and "four words of text" in text
    elif backend == "trt-llm":
        assert seen["trt-llm"]["text_input"] in ("what is this", "and that") and "tok tok tok" in text
    else:
        assert seen["chat"]["messages"][0]["role"] == "user" and "Hello you" in text


@pytest.mark.parametrize("stream", [False, True])
def test_client_chat_server_backend_against_this_server(server, tmp_path, stream):
    """The client's chat-server format (``--backend ksana-server``: OpenAI-style body to /v1/chat, usage counts and
    server-sent events in the answer) against this package's own server."""
    csv_path = tmp_path / "prompts.csv"
    csv_path.write_text("prompt\nhello there\nsecond prompt\nthird one\n", encoding="utf-8")
    args = bt.args_config(["--port", str(server), "--backend", "ksana-server", "--input_csv", str(csv_path), "--max_new_tokens", "5",
                           "--client_timeout", "60", "--ignore_eos"] +
                          (["--stream", "--request_rate", "50"] if stream else ["--mode", "sync", "--concurrency", "2"]))
    s = bt.run_benchmark(args)[0]
    assert s["finished"] == 3 and s["failed"] == 0 and s["avg_output_tokens"] == 5
    if stream:
        assert s["avg_ttft_s"] > 0
