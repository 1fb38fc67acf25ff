"""HTTP front: ``POST /generate`` (JSON in; JSON out, or a stream of JSON chunks each terminated by a
zero byte) and ``POST /forward`` (msgpack in / out), plus ``GET /metrics`` (Prometheus text) and OpenAI-style
``/v1/completions``, ``/v1/chat/completions`` and ``/v1/models``.

Request / response fields, the chunk framing and the HTTP 500 ``{"message", "code"}`` error body follow
src/ksana_llm/python/serving_server.py:41-449. Only node rank 0 serves HTTP; other ranks follow the
engine's broadcast step plans.

  python -m ksanallm_b200.serving.serving_server --config_file ksana_llm.yaml --port 8080
"""
from __future__ import annotations

import argparse
import json
import os
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, List, Optional

import msgpack
import yaml
from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, Response, StreamingResponse

from ..utils import logger
from ..utils import native_engine as ne
from .plugin import PluginConfig
from .serving_model import EndpointConfig, ServingModel

TRACE_HEADERS = ("x-remote-ip", "traceparent")
TIMEOUT_KEEP_ALIVE = 5          # seconds an idle client connection is kept open


def _flag(text: str) -> bool:
    """Boolean command-line value: "false", "0", "no" and "off" (any case) are False, everything else True."""
    return str(text).strip().lower() not in ("false", "0", "no", "off", "")


def args_config(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--config_file", type=str, default="examples/ksana_llm.yaml", help="serving config file")
    p.add_argument("--tokenizer_dir", type=str, default=None, help="tokenizer dir (default: the model dir)")
    p.add_argument("--host", type=str, default="0.0.0.0")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--endpoint", type=str, default=None,
                   help="server endpoint type (python, or the name of an RPC endpoint plug-in); default: the YAML's "
                        "setting.endpoint_type, else python")
    p.add_argument("--access-log", nargs="?", const=True, default=True, type=_flag,
                   help="endpoint access log: --access-log, --access-log false, --no-access-log")
    p.add_argument("--no-access-log", dest="access_log", action="store_false")
    p.add_argument("--ssl-keyfile", type=str, default=None)
    p.add_argument("--ssl-certfile", type=str, default=None)
    p.add_argument("--root-path", type=str, default=None)
    p.add_argument("--random-weights", action="store_true", help="serve a random-init model (tests, benchmarks)")
    args = p.parse_args(argv)
    prepare_config(args)
    return args


def prepare_config(args):
    """Resolve model / tokenizer dirs and the plugin settings from the YAML."""
    args.config_file = os.path.abspath(args.config_file)
    with open(args.config_file, "r", encoding="utf-8") as f:
        doc = yaml.safe_load(f) or {}
    base = (doc.get("model_spec") or {}).get("base_model") or {}
    model_dir = str(base.get("model_dir", ""))
    if model_dir and not os.path.isabs(model_dir):
        model_dir = os.path.normpath(os.path.join(os.path.dirname(args.config_file), model_dir))
    args.model_dir = model_dir
    if args.tokenizer_dir is None:
        args.tokenizer_dir = base.get("tokenizer_dir") or model_dir
    plugin = (doc.get("model_spec") or {}).get("plugin_model") or {}
    args.plugin_enable_trt = bool(plugin.get("enable_tensorrt", True))
    args.plugin_thread_pool_size = int(plugin.get("plugin_thread_pool_size", 1))
    if args.endpoint is None:                  # the command line wins over the YAML
        args.endpoint = (doc.get("setting") or {}).get("endpoint_type") or "python"
    args.endpoint = str(args.endpoint).lower()
    args.model_type = ""
    cfg_path = os.path.join(model_dir, "config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path, "r", encoding="utf-8") as f:
            mc = json.load(f)
        args.model_type = mc.get("model_type", "")
        if args.model_type == "qwen" and "visual" in mc:
            args.model_type = "qwen_vl"


def load_tokenizer(tokenizer_dir: str):
    """Tokenizer of a checkpoint directory, by the reference server's rules (src/ksana_llm/python/serving_server.py:381-390):
    a directory whose tokenizer_config.json names ``LlamaTokenizer`` gets that class itself (the automatic choice may
    convert it to a fast tokenizer that splits some inputs differently); a directory with a ``preprocessor_config.json``
    (multimodal checkpoints) is loaded as a processor, whose text tokenizer serves the server while the processor
    stays reachable as ``tokenizer.processor`` for plug-ins; everything else through ``AutoTokenizer``."""
    import transformers
    cfg = {}
    cfg_path = os.path.join(tokenizer_dir, "tokenizer_config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path, "r", encoding="utf-8") as f:
            cfg = json.load(f)
    tok = None
    if cfg.get("tokenizer_class", "") == "LlamaTokenizer":
        try:
            tok = transformers.LlamaTokenizer.from_pretrained(tokenizer_dir)
        except Exception as e:      # noqa: BLE001 - e.g. no sentencepiece model in the directory: the automatic choice still works
            logger.warning(f"LlamaTokenizer could not be loaded from {tokenizer_dir} ({e}); using AutoTokenizer")
    elif os.path.exists(os.path.join(tokenizer_dir, "preprocessor_config.json")):
        proc = transformers.AutoProcessor.from_pretrained(tokenizer_dir, trust_remote_code=True)
        tok = getattr(proc, "tokenizer", proc)
        if tok is not proc:
            tok.processor = proc
    if tok is None:
        tok = transformers.AutoTokenizer.from_pretrained(tokenizer_dir, trust_remote_code=True)
    if not getattr(tok, "is_fast", True):
        logger.warning(f"using a slow tokenizer for {tokenizer_dir}: tokenisation may take a noticeable share of the request time")
    return tok


def _sampling_dict(sampling_config: Optional[dict], tokenizer) -> dict:
    sc = dict(sampling_config or {})
    stop_token_ids = list(sc.get("stop_token_ids", []) or [])
    ignore_eos = bool(sc.get("ignore_eos", False))
    eos = getattr(tokenizer, "eos_token_id", None) if tokenizer is not None else None
    if eos is not None and not ignore_eos and eos not in stop_token_ids:
        stop_token_ids.append(eos)
    return {
        "top_k": sc.get("topk", 1), "do_sample": sc.get("do_sample", None), "top_p": sc.get("topp", 1.0),
        "temperature": sc.get("temperature", 1.0), "max_new_tokens": sc.get("max_new_tokens", -1),
        "logprobs_num": sc.get("logprobs", 0), "repetition_penalty": sc.get("repetition_penalty", 1.0),
        "no_repeat_ngram_size": sc.get("no_repeat_ngram_size", 0),
        "encoder_no_repeat_ngram_size": sc.get("encoder_no_repeat_ngram_size", 0),
        "num_beams": sc.get("num_beams", 1), "num_return_sequences": sc.get("num_return_sequences", 1),
        "length_penalty": sc.get("length_penalty", 1.0), "stop_strings": sc.get("stop_strings", []),
        "stop_token_ids": stop_token_ids, "ignore_eos": ignore_eos, "seed": sc.get("seed", 0),
    }


def _decode(tokenizer, tokens: List[int], strip_partial: bool = False) -> str:
    if tokenizer is None:
        return ""
    text = tokenizer.decode(tokens, skip_special_tokens=True)
    return text.rstrip("�") if strip_partial else text


def create_app(model: ServingModel, tokenizer, executor: Optional[ThreadPoolExecutor] = None):
    app = FastAPI()
    executor = executor or ThreadPoolExecutor(max_workers=256)

    def trace_ctx(request) -> Dict[str, str]:
        return {h: request.headers.get(h) for h in TRACE_HEADERS if request.headers.get(h) is not None}

    def to_json(out) -> dict:
        return {"texts": [_decode(tokenizer, t) for t in out.output_tokens], "output_token_ids": out.output_tokens,
                "logprobs": out.logprobs, "input_token_ids": out.input_tokens}

    def render_messages(messages) -> Optional[List[int]]:
        if tokenizer is None or not hasattr(tokenizer, "apply_chat_template"):
            return None
        ids = tokenizer.apply_chat_template(messages, tokenize=True, add_generation_prompt=True)
        if hasattr(ids, "keys"):                       # newer tokenizers return an encoding object, not a list
            ids = ids["input_ids"]
        if len(ids) and isinstance(ids[0], (list, tuple)):
            ids = ids[0]
        return [int(t) for t in ids]

    async def process_request(request_dict: Dict[str, Any], req_ctx: Dict[str, str]):
        model_name = request_dict.pop("model_name", "")
        prompt_text = request_dict.pop("prompt", None)
        messages = request_dict.pop("messages", None)
        enable_streaming = request_dict.pop("stream", True)
        sampling_config = request_dict.pop("sampling_config", None)
        regex = request_dict.pop("structured_output_regex", None)
        input_tokens = request_dict.pop("input_tokens", None)
        if input_tokens is None and prompt_text is not None and tokenizer is not None:
            input_tokens = tokenizer.encode(prompt_text, add_special_tokens=True)
        if input_tokens is None and messages is not None and (model.plugin is None or not model.plugin.loaded):
            input_tokens = render_messages(messages)
        kwargs = {"input_refit_embedding": {}, "additional_params": request_dict.pop("additional_params", None) or {},
                  "prompt": prompt_text}
        emb = request_dict.pop("input_refit_embedding", None)
        if emb is not None:
            for k in ("pos", "embeddings"):
                if k in emb:
                    kwargs["input_refit_embedding"][k] = emb[k]
        if regex is not None:
            kwargs["structured_output_regex"] = regex
        gen = _sampling_dict(sampling_config, tokenizer)
        # no thread waits while the request runs: the engine posts pieces and the end to this event loop
        status, result = await model.generate_async(model_name=model_name, inputs=input_tokens, generation_config=gen,
                                                    messages=messages, streamer=True if enable_streaming else None,
                                                    req_ctx=req_ctx, executor=executor, **kwargs)
        if not status.OK():
            return status, None, enable_streaming
        if enable_streaming:
            async def stream_results():
                try:
                    async for out in result:
                        if out is None:
                            return
                        body = {"texts": [_decode(tokenizer, t, True) for t in out.output_tokens],
                                "output_token_ids": out.output_tokens, "logprobs": out.logprobs,
                                "input_token_ids": out.input_tokens}
                        yield json.dumps(body).encode() + b"\0"
                finally:
                    result.close()          # a client that went away mid-stream: the request is aborted
            return status, stream_results(), True
        return status, to_json(result), False

    @app.post("/generate")
    async def generate(request: Request):
        req_ctx = trace_ctx(request)
        request_dict = await request.json()
        status, results, streaming = await process_request(request_dict, req_ctx)
        if not status.OK():
            return JSONResponse({"message": status.GetMessage(), "code": status.GetCode().value}, status_code=500)
        if streaming:
            return StreamingResponse(results)
        return JSONResponse(results)

    @app.post("/forward")
    async def forward(request: Request):
        req_ctx = trace_ctx(request)
        body = await request.body()
        status, response_bytes = await model.forward_async(body, req_ctx, executor=executor)
        if status.OK() and response_bytes is not None:
            return Response(content=response_bytes, media_type="application/x-msgpack")
        err = msgpack.packb({"message": status.GetMessage(), "code": status.GetCode().value})
        return Response(content=err, status_code=500, media_type="application/x-msgpack")

    # ------------------------------------------------------------------ OpenAI-style routes
    # /v1/completions, /v1/chat/completions (blocking and server-sent events) and /v1/models over the same engine
    # path as /generate. The reference's server takes OpenAI-style ``messages`` in /generate only; these routes are
    # for clients that speak the OpenAI wire format itself.
    served_name = os.path.basename(os.path.normpath(getattr(model.llm.engine_cfg, "model_dir", "") or "")) or "ksana_llm"

    def openai_error(message: str, status: int = 400, kind: str = "invalid_request_error"):
        return JSONResponse({"error": {"message": message, "type": kind, "param": None, "code": None}}, status_code=status)

    def openai_sampling(body: dict, default_max: int) -> dict:
        temperature = body.get("temperature")
        temperature = 1.0 if temperature is None else float(temperature)
        greedy = temperature <= 0.0
        stop = body.get("stop") or []
        stop = [stop] if isinstance(stop, str) else list(stop)
        max_tokens = body.get("max_completion_tokens") or body.get("max_tokens") or body.get("max_new_tokens") or default_max
        sc = {"topk": 1 if greedy else int(body.get("top_k") or 50), "temperature": 1.0 if greedy else temperature,
              "topp": float(body.get("top_p") or 1.0), "max_new_tokens": int(max_tokens),
              "num_return_sequences": int(body.get("n") or 1), "stop_strings": stop,
              "repetition_penalty": float(body.get("repetition_penalty") or 1.0), "seed": int(body.get("seed") or 0),
              "ignore_eos": bool(body.get("ignore_eos", False)), "do_sample": not greedy,
              "stop_token_ids": [int(t) for t in (body.get("stop_token_ids") or [])]}
        return _sampling_dict(sc, tokenizer)

    async def openai_generate(kind: str, body: dict, input_tokens: List[int], req_ctx: Dict[str, str]):
        import time as _time
        import uuid
        gen = openai_sampling(body, 16 if kind == "text_completion" else 1024)
        stream = bool(body.get("stream", False))
        rid = ("cmpl-" if kind == "text_completion" else "chatcmpl-") + uuid.uuid4().hex[:24]
        created = int(_time.time())
        name = body.get("model") or served_name
        status, result = await model.generate_async(model_name=name, inputs=input_tokens, generation_config=gen,
                                                    streamer=True if stream else None, req_ctx=req_ctx, executor=executor,
                                                    prompt=body.get("prompt") if isinstance(body.get("prompt"), str) else None,
                                                    **({"structured_output_regex": body["structured_output_regex"]}
                                                       if body.get("structured_output_regex") else {}))
        if not status.OK():
            code = status.GetCode().value
            if code in (1, 6):            # a bad argument, a prompt beyond the model's length: the client's to fix
                return openai_error(status.GetMessage(), 400, "invalid_request_error")
            if code in (5, 7):            # waiting queue full, waited too long: try again later
                return openai_error(status.GetMessage(), 503, "server_overloaded")
            return openai_error(status.GetMessage(), 500, "server_error")

        def finish_reason(tokens) -> str:
            return "length" if len(tokens) >= gen["max_new_tokens"] else "stop"

        def choice(i: int, text: str, reason, delta: bool):
            if kind == "text_completion":
                return {"index": i, "text": text, "logprobs": None, "finish_reason": reason}
            key = "delta" if delta else "message"
            msg = {"content": text} if delta else {"role": "assistant", "content": text}
            return {"index": i, key: msg, "logprobs": None, "finish_reason": reason}

        if not stream:
            texts = [_decode(tokenizer, t) for t in result.output_tokens]
            n_out = sum(len(t) for t in result.output_tokens)
            return JSONResponse({
                "id": rid, "object": kind if kind == "text_completion" else "chat.completion", "created": created, "model": name,
                "choices": [choice(i, texts[i], finish_reason(result.output_tokens[i]), False) for i in range(len(texts))],
                "usage": {"prompt_tokens": len(result.input_tokens), "completion_tokens": n_out,
                          "total_tokens": len(result.input_tokens) + n_out}})

        obj = "text_completion" if kind == "text_completion" else "chat.completion.chunk"

        async def events():
            sent: Dict[int, str] = {}
            last = None
            try:
                if kind != "text_completion":
                    first = {"id": rid, "object": obj, "created": created, "model": name,
                             "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]}
                    yield b"data: " + json.dumps(first).encode() + b"\n\n"
                async for out in result:
                    last = out
                    choices = []
                    for i, toks in enumerate(out.output_tokens):
                        text = _decode(tokenizer, toks, True)
                        piece = text[len(sent.get(i, "")):]
                        if piece:
                            sent[i] = text
                            choices.append(choice(i, piece, None, True))
                    if choices:
                        chunk = {"id": rid, "object": obj, "created": created, "model": name, "choices": choices}
                        yield b"data: " + json.dumps(chunk).encode() + b"\n\n"
                if last is not None:
                    # what the per-step decoding held back (an incomplete character at the tail) goes out with the end
                    tails = []
                    for i, t in enumerate(last.output_tokens):
                        full = _decode(tokenizer, t)
                        tails.append(full[len(sent.get(i, "")):] if full.startswith(sent.get(i, "")) else "")
                    n_out = sum(len(t) for t in last.output_tokens)
                    final = {"id": rid, "object": obj, "created": created, "model": name,
                             "choices": [choice(i, tails[i], finish_reason(t), True) for i, t in enumerate(last.output_tokens)],
                             "usage": {"prompt_tokens": len(last.input_tokens), "completion_tokens": n_out,
                                       "total_tokens": len(last.input_tokens) + n_out}}
                    yield b"data: " + json.dumps(final).encode() + b"\n\n"
                yield b"data: [DONE]\n\n"
            finally:
                result.close()
        return StreamingResponse(events(), media_type="text/event-stream")

    @app.get("/v1/models")
    async def openai_models():
        return JSONResponse({"object": "list", "data": [{"id": served_name, "object": "model", "owned_by": "ksana_llm"}]})

    @app.post("/v1/completions")
    async def openai_completions(request: Request):
        body = await request.json()
        prompt = body.get("prompt")
        if isinstance(prompt, list) and prompt and all(isinstance(t, int) for t in prompt):
            tokens = [int(t) for t in prompt]
        elif isinstance(prompt, list) and len(prompt) == 1 and isinstance(prompt[0], str):
            prompt = prompt[0]
            tokens = None
        elif isinstance(prompt, str):
            tokens = None
        else:
            return openai_error("prompt must be a string, a list with one string, or a list of token ids")
        if tokens is None:
            if tokenizer is None:
                return openai_error("this server has no tokenizer: send the prompt as a list of token ids")
            tokens = tokenizer.encode(prompt, add_special_tokens=True)
        return await openai_generate("text_completion", body, tokens, trace_ctx(request))

    @app.post("/v1/chat")                    # the path the benchmark client's "ksana-server" / "vllm-server" backends use
    @app.post("/v1/chat/completions")
    async def openai_chat(request: Request):
        body = await request.json()
        messages = body.get("messages")
        if not isinstance(messages, list) or not messages:
            return openai_error("messages must be a non-empty list")
        tokens = render_messages(messages)
        if tokens is None:
            return openai_error("this server's tokenizer has no chat template")
        return await openai_generate("chat.completion", body, tokens, trace_ctx(request))

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(ne.metrics_prometheus())

    @app.get("/health")
    async def health():
        return JSONResponse({"status": "ok"})

    return app


def main(argv=None):
    args = args_config(argv)
    logger.install_logging_handler()          # uvicorn / serving records go to the engine's log sink (KLLM_LOG_FILE)
    logger.info(f"serving_server starting: config {args.config_file}, endpoint {args.endpoint} on {args.host}:{args.port}")
    tokenizer = load_tokenizer(args.tokenizer_dir) if args.tokenizer_dir and os.path.isdir(args.tokenizer_dir) else None
    model = ServingModel(args.config_file, tokenizer=tokenizer)
    plugin_config = PluginConfig(model_dir=args.model_dir, config_file=args.config_file, plugin_name=args.model_type,
                                 enable_trt=args.plugin_enable_trt, thread_pool_size=args.plugin_thread_pool_size)
    endpoint_config = EndpointConfig(args.endpoint, args.host, args.port, args.access_log)
    model.init_serving(plugin_config, endpoint_config, weights="random" if args.random_weights else "checkpoint")
    rank = int(os.environ.get("RANK", "0"))
    node_rank = int(os.environ.get("NODE_RANK", "0"))
    if rank != 0 or node_rank != 0:
        print("Uvicorn running on NONE.", flush=True)      # the line launch scripts wait for, from a rank without a port
        while model.llm.follow():      # worker ranks: execute broadcast step plans until the stop signal
            pass
        if getattr(model.llm, "coordinator", None) is not None:
            model.llm.coordinator.close()
        return
    if args.endpoint != "python":
        # an RPC endpoint plug-in serves on the configured host and port itself: no HTTP front beside it
        import signal
        for sig in (signal.SIGTERM, signal.SIGINT):
            signal.signal(sig, lambda *_: model.shutdown())
        logger.info(f"endpoint {args.endpoint} serving on {args.host}:{args.port}")
        while not model.wait_for_shutdown(1.0):
            pass
        return
    import uvicorn
    app = create_app(model, tokenizer)
    log_level = os.environ.get("KLLM_LOG_LEVEL", "INFO").lower()
    if log_level in ("debug", "info", "warning", "error"):
        pass
    else:
        log_level = "info"
    try:
        uvicorn.run(app, host=args.host, port=args.port, log_level=log_level, access_log=args.access_log,
                    timeout_keep_alive=TIMEOUT_KEEP_ALIVE, ssl_keyfile=args.ssl_keyfile, ssl_certfile=args.ssl_certfile,
                    root_path=args.root_path or "")
    finally:
        model.shutdown()


if __name__ == "__main__":
    main()
