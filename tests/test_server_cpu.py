"""HTTP surface on CPU: /generate (blocking + zero-byte-delimited streaming), /forward (msgpack), errors, metrics."""
import json

import msgpack
import pytest
import torch

from helpers import ByteTokenizer, tiny_model_cfg
from ksanallm_b200.config import EngineConfig
from ksanallm_b200.llm import LLM
from ksanallm_b200.serving.clients import perplexity_from_forward
from ksanallm_b200.serving.request_packer import unpack_tensor
from ksanallm_b200.serving.serving_model import ServingModel, make_sampling_config
from ksanallm_b200.serving.serving_server import create_app


@pytest.fixture(scope="module")
def client():
    from fastapi.testclient import TestClient
    tok = ByteTokenizer()
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size = 8
    ec.batch_scheduler.max_token_len = 128
    ec.block_manager.device_blocks_num = 128
    ec.block_manager.host_blocks_num = 16
    llm = LLM(ec, tiny_model_cfg(), weights="random", device="cpu", dtype=torch.float32, tokenizer=tok)
    model = ServingModel("", llm=llm, tokenizer=tok)
    model.init_serving()
    with TestClient(create_app(model, tok)) as c:
        yield c
    model.shutdown()


def test_generate_blocking(client):
    r = client.post("/generate", json={"prompt": "hello", "stream": False,
                                       "sampling_config": {"max_new_tokens": 6, "ignore_eos": True, "logprobs": 2}})
    assert r.status_code == 200
    body = r.json()
    assert set(body) == {"texts", "output_token_ids", "logprobs", "input_token_ids"}
    assert len(body["output_token_ids"]) == 1 and len(body["output_token_ids"][0]) == 6
    assert body["input_token_ids"] == ByteTokenizer().encode("hello")
    assert len(body["logprobs"][0]) == 6 and len(body["logprobs"][0][0]) == 2
    r2 = client.post("/generate", json={"input_tokens": body["input_token_ids"], "stream": False,
                                        "sampling_config": {"max_new_tokens": 6, "ignore_eos": True}})
    assert r2.json()["output_token_ids"] == body["output_token_ids"]       # greedy is deterministic


def test_generate_streaming_chunks(client):
    with client.stream("POST", "/generate", json={"prompt": "abc", "stream": True,
                                                  "sampling_config": {"max_new_tokens": 5, "ignore_eos": True}}) as r:
        raw = b"".join(r.iter_bytes())
    chunks = [json.loads(c) for c in raw.split(b"\0") if c]
    assert len(chunks) >= 1 and len(chunks[-1]["output_token_ids"][0]) == 5
    lens = [len(c["output_token_ids"][0]) for c in chunks]
    assert lens == sorted(lens)


def test_generate_chat_messages_and_n(client):
    r = client.post("/generate", json={"messages": [{"role": "user", "content": "hi"}], "stream": False,
                                       "sampling_config": {"max_new_tokens": 3, "ignore_eos": True, "topk": 20,
                                                           "temperature": 1.3, "num_return_sequences": 2}})
    assert r.status_code == 200 and len(r.json()["output_token_ids"]) == 2


def test_generate_errors_are_http_500_with_code(client):
    r = client.post("/generate", json={"prompt": "x", "stream": False, "sampling_config": {"topk": 5000}})
    assert r.status_code == 500 and r.json()["code"] == 1 and "topk" in r.json()["message"]
    r = client.post("/generate", json={"input_tokens": list(range(3, 203)), "stream": False, "sampling_config": {}})
    assert r.status_code == 500 and r.json()["code"] == 6


def test_forward_msgpack_roundtrip(client):
    toks = ByteTokenizer().encode("perplexity")
    req = {"requests": [{"input_tokens": toks, "request_target": [
        {"target_name": "logits", "slice_pos": [[0, len(toks) - 2]], "token_reduce_mode": "GATHER_TOKEN_ID"},
        {"target_name": "layernorm", "token_reduce_mode": "GATHER_ALL"}]}]}
    r = client.post("/forward", content=msgpack.packb(req, use_bin_type=True))
    assert r.status_code == 200
    doc = msgpack.unpackb(r.content, raw=False)
    assert doc["code"] == 0 and doc["responses"][0]["input_token_ids"] == toks
    tensors = {t["target_name"]: unpack_tensor(t["tensor"]) for t in doc["responses"][0]["response"]}
    assert tensors["logits"].shape == (len(toks) - 1,) and tensors["layernorm"].shape == (1, 64)
    for t in doc["responses"][0]["response"]:
        t["tensor"] = unpack_tensor(t["tensor"])
    assert perplexity_from_forward(doc)[0] > 1.0
    bad = {"requests": [{"input_tokens": toks, "request_target": [{"target_name": "logits", "slice_pos": [[0, len(toks) - 1]],
                                                                   "token_reduce_mode": "GATHER_TOKEN_ID"}]}]}
    r = client.post("/forward", content=msgpack.packb(bad, use_bin_type=True))
    assert r.status_code == 500 and msgpack.unpackb(r.content, raw=False)["code"] == 1


def test_metrics_endpoint_and_sampling_mapping(client):
    text = client.get("/metrics").text
    assert "ksana_forward_req_total_num_count" in text and "ksana_time_to_first_token_ms_count" in text
    c = make_sampling_config({"top_k": 40, "do_sample": False, "max_new_tokens": -1})
    assert c.topk == 1 and c.max_new_tokens == 1024
    c = make_sampling_config({"top_k": 40, "do_sample": True, "top_p": 0.9, "stop_token_ids": [2]})
    assert c.topk == 40 and abs(c.topp - 0.9) < 1e-6 and c.stop_token_ids == [2]


def test_statistics_file_receives_metric_lines(tmp_path, monkeypatch):
    """With KLLM_STAT_FILE set and no collector configured, the metrics go to that file: one JSON line per export
    interval, naming the request counters."""
    import time
    stat = tmp_path / "stats" / "ksana_stat.log"
    monkeypatch.setenv("KLLM_STAT_FILE", str(stat))
    tok = ByteTokenizer()
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size = 4
    ec.batch_scheduler.max_token_len = 64
    ec.block_manager.device_blocks_num = 32
    ec.profiler.export_interval_millis = 50
    llm = LLM(ec, tiny_model_cfg(), weights="random", device="cpu", dtype=torch.float32, tokenizer=tok)
    model = ServingModel("", llm=llm, tokenizer=tok)
    model.init_serving()
    try:
        req = llm.engine.add_request(tok.encode("hello"), make_sampling_config({"max_new_tokens": 3, "ignore_eos": True}))
        assert req.done.wait(30)
        deadline = time.time() + 10
        while time.time() < deadline and not (stat.exists() and stat.read_text().strip()):
            time.sleep(0.05)
    finally:
        model.shutdown()
    lines = [json.loads(x) for x in stat.read_text().splitlines() if x.strip()]
    assert lines and any("forward_req_total_num" in json.dumps(x) for x in lines)


def test_tokenizer_loading_rules(tmp_path, monkeypatch):
    """Which loader a tokenizer directory gets: the class named LlamaTokenizer itself (with the automatic choice as a
    fallback), a processor for multimodal checkpoints (its text tokenizer serves, the processor stays reachable),
    AutoTokenizer otherwise."""
    import transformers
    from ksanallm_b200.serving.serving_server import load_tokenizer
    calls = []

    class Tok:
        is_fast = True

    class Proc:
        def __init__(self):
            self.tokenizer = Tok()

    monkeypatch.setattr(transformers.AutoTokenizer, "from_pretrained", classmethod(lambda cls, d, **kw: calls.append(("auto", kw)) or Tok()))
    monkeypatch.setattr(transformers.AutoProcessor, "from_pretrained", classmethod(lambda cls, d, **kw: calls.append(("processor", kw)) or Proc()))
    monkeypatch.setattr(transformers.LlamaTokenizer, "from_pretrained", classmethod(lambda cls, d, **kw: calls.append(("llama", kw)) or Tok()))
    plain = tmp_path / "plain"
    plain.mkdir()
    assert isinstance(load_tokenizer(str(plain)), Tok) and calls[-1] == ("auto", {"trust_remote_code": True})
    llama = tmp_path / "llama"
    llama.mkdir()
    (llama / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "LlamaTokenizer"}))
    assert isinstance(load_tokenizer(str(llama)), Tok) and calls[-1][0] == "llama"

    def broken(cls, d, **kw):
        raise OSError("no sentencepiece model")
    monkeypatch.setattr(transformers.LlamaTokenizer, "from_pretrained", classmethod(broken))
    assert isinstance(load_tokenizer(str(llama)), Tok) and calls[-1][0] == "auto"
    vl = tmp_path / "vl"
    vl.mkdir()
    (vl / "preprocessor_config.json").write_text("{}")
    tok = load_tokenizer(str(vl))
    assert isinstance(tok, Tok) and isinstance(tok.processor, Proc) and calls[-1][0] == "processor"


def test_many_open_requests_hold_no_threads():
    """Forty requests in flight at once (half of them streaming) through a front whose executor has two threads: all
    of them complete with full-length answers, and the process grows by no thread per open request, because a request
    that is running waits on the event loop, not on a thread."""
    import asyncio
    import threading
    import httpx
    tok = ByteTokenizer()
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size = 64
    ec.batch_scheduler.max_token_len = 128
    ec.block_manager.device_blocks_num = 512
    llm = LLM(ec, tiny_model_cfg(), weights="random", device="cpu", dtype=torch.float32, tokenizer=tok)
    model = ServingModel("", llm=llm, tokenizer=tok)
    model.init_serving()
    from concurrent.futures import ThreadPoolExecutor
    app = create_app(model, tok, executor=ThreadPoolExecutor(max_workers=2))
    peak = [0]

    async def run():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://test") as c:
            async def one(i):
                r = await c.post("/generate", json={"prompt": "request number %d" % i, "stream": i % 2 == 0,
                                                    "sampling_config": {"max_new_tokens": 24, "ignore_eos": True}}, timeout=120)
                peak[0] = max(peak[0], threading.active_count())
                assert r.status_code == 200
                if i % 2 == 0:
                    chunks = [json.loads(x) for x in r.content.split(b"\0") if x]
                    return chunks[-1]["output_token_ids"][0]
                return r.json()["output_token_ids"][0]
            return await asyncio.gather(*[one(i) for i in range(40)])

    before = threading.active_count()
    try:
        outs = asyncio.run(run())
    finally:
        model.shutdown()
    assert len(outs) == 40 and all(len(o) == 24 for o in outs)
    assert peak[0] - before <= 6, (before, peak[0])       # executor threads and the loop's helpers, not 40


def test_closing_a_stream_follower_aborts_its_request():
    """A client that leaves mid-stream: closing the follower aborts the request in the engine, which then ends it with
    the aborted status instead of generating to the end."""
    import asyncio
    tok = ByteTokenizer()
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size = 4
    ec.batch_scheduler.max_token_len = 2048
    ec.block_manager.device_blocks_num = 256
    llm = LLM(ec, tiny_model_cfg(), weights="random", device="cpu", dtype=torch.float32, tokenizer=tok)
    model = ServingModel("", llm=llm, tokenizer=tok)
    model.init_serving()

    async def run():
        status, follower = await model.generate_async(inputs=tok.encode("a long story"), streamer=True,
                                                      generation_config={"max_new_tokens": 1500, "ignore_eos": True})
        assert status.OK()
        first = await follower.__anext__()
        assert 1 <= len(first.output_tokens[0]) < 1500
        req = follower.req
        follower.close()
        for _ in range(600):
            if req.done.is_set():
                break
            await asyncio.sleep(0.01)
        return req

    try:
        req = asyncio.run(run())
    finally:
        model.shutdown()
    assert req.done.is_set() and req.aborted and len(req.outputs[0].tokens) < 1500


def test_streamed_outputs_pass_through_the_plugin():
    """Every streamed output is handed to the plug-in's post-processing (here it appends a marker token), in the
    event-loop form and in the blocking iterator."""
    import asyncio

    class Marker:
        loaded = True
        calls = 0

        def preprocess(self, **kw):
            # a plug-in may ask for tensors of the prompt as well (same target description as /forward takes)
            kw["ksana_python_input"].request_target = {"layernorm": {"slice_pos": [[0, 1]], "token_reduce_mode": "GATHER_ALL"}}

        def postprocess(self, ksana_python_input, ksana_python_output, **kw):
            Marker.calls += 1
            ksana_python_output.output_tokens = [t + [7777] for t in ksana_python_output.output_tokens]

    tok = ByteTokenizer()
    ec = EngineConfig()
    ec.batch_scheduler.max_batch_size = 4
    ec.batch_scheduler.max_token_len = 64
    ec.block_manager.device_blocks_num = 32
    llm = LLM(ec, tiny_model_cfg(), weights="random", device="cpu", dtype=torch.float32, tokenizer=tok)
    model = ServingModel("", llm=llm, tokenizer=tok)
    model.init_serving()
    model.plugin = Marker()

    async def run(blocking_iterator):
        gen = {"max_new_tokens": 6, "ignore_eos": True}
        if blocking_iterator:
            status, it = model.generate(inputs=tok.encode("hi"), generation_config=gen, streamer=True)
        else:
            status, it = await model.generate_async(inputs=tok.encode("hi"), generation_config=gen, streamer=True)
        assert status.OK()
        outs = [o async for o in it]
        return outs

    try:
        for blocking_iterator in (False, True):
            outs = asyncio.run(run(blocking_iterator))
            assert outs and all(o.output_tokens[0][-1] == 7777 for o in outs)
            assert len(outs[-1].output_tokens[0]) == 7
            assert tuple(outs[-1].response["layernorm"].shape) == (2, 64)
    finally:
        model.shutdown()
    assert Marker.calls >= 2


def test_server_command_line_rules(tmp_path):
    """--endpoint on the command line wins over the YAML's endpoint_type (which wins over "python"); the access log
    flag takes the forms launch scripts of the reference use."""
    from ksanallm_b200.serving.serving_server import args_config
    y = tmp_path / "c.yaml"
    y.write_text("setting:\n  endpoint_type: TRPC\nmodel_spec:\n  base_model:\n    model_dir: /tmp/none\n")
    a = args_config(["--config_file", str(y)])
    assert a.endpoint == "trpc" and a.access_log is True and a.tokenizer_dir == a.model_dir
    a = args_config(["--config_file", str(y), "--endpoint", "Python", "--access-log", "False"])
    assert a.endpoint == "python" and a.access_log is False
    assert args_config(["--config_file", str(y), "--no-access-log"]).access_log is False
    y.write_text("model_spec:\n  base_model:\n    model_dir: /tmp/none\n")
    assert args_config(["--config_file", str(y)]).endpoint == "python"


def test_openai_style_routes(client):
    """/v1/models, /v1/completions and /v1/chat/completions: blocking answers with usage counts, greedy at temperature
    0 (equal to /generate's greedy tokens), n choices, server-sent events whose deltas add up to the blocking text."""
    assert client.get("/v1/models").json()["data"][0]["object"] == "model"
    greedy = client.post("/generate", json={"prompt": "hello", "stream": False,
                                            "sampling_config": {"max_new_tokens": 6}}).json()
    r = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 6, "temperature": 0})
    assert r.status_code == 200, r.text
    body = r.json()
    assert body["object"] == "text_completion" and body["id"].startswith("cmpl-") and len(body["choices"]) == 1
    assert body["choices"][0]["text"] == greedy["texts"][0]
    assert body["usage"] == {"prompt_tokens": len(greedy["input_token_ids"]), "completion_tokens": len(greedy["output_token_ids"][0]),
                             "total_tokens": len(greedy["input_token_ids"]) + len(greedy["output_token_ids"][0])}
    assert body["choices"][0]["finish_reason"] in ("length", "stop")
    # token ids as the prompt, three sampled choices
    r = client.post("/v1/completions", json={"prompt": greedy["input_token_ids"], "max_tokens": 4, "n": 3, "seed": 5,
                                             "ignore_eos": True})
    assert r.status_code == 200 and [c["index"] for c in r.json()["choices"]] == [0, 1, 2]
    assert r.json()["usage"]["completion_tokens"] == 12
    # chat: blocking, then the same request streamed
    req = {"messages": [{"role": "user", "content": "hi there"}], "max_tokens": 8, "temperature": 0, "ignore_eos": True}
    chat = client.post("/v1/chat/completions", json=req).json()
    assert chat["object"] == "chat.completion" and chat["choices"][0]["message"]["role"] == "assistant"
    assert chat["choices"][0]["finish_reason"] == "length" and chat["usage"]["completion_tokens"] == 8
    with client.stream("POST", "/v1/chat/completions", json=dict(req, stream=True)) as resp:
        assert resp.headers["content-type"].startswith("text/event-stream")
        raw = b"".join(resp.iter_bytes()).decode()
    events = [e[len("data: "):] for e in raw.split("\n\n") if e.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert all(c["object"] == "chat.completion.chunk" for c in chunks) and chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
    assert text == chat["choices"][0]["message"]["content"] and chunks[-1]["choices"][0]["finish_reason"] == "length"
    # errors in the OpenAI shape
    bad = client.post("/v1/completions", json={"prompt": {"not": "a prompt"}})
    assert bad.status_code == 400 and bad.json()["error"]["type"] == "invalid_request_error"
    assert client.post("/v1/chat/completions", json={"messages": []}).status_code == 400
    long_prompt = client.post("/v1/completions", json={"prompt": [5] * 500, "max_tokens": 2})        # the model takes 128
    assert long_prompt.status_code == 400 and long_prompt.json()["error"]["type"] == "invalid_request_error"
