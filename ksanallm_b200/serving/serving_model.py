"""The serving object behind the HTTP front and the Python package API: owns the LLM (model + engine
loop), converts generation configs into native SamplingConfig objects, runs plugin pre/post-processing,
and exposes blocking, streaming and forward (tensor extraction) calls.

Public behaviour follows src/ksana_llm/python/ksana_llm/serving_model.py:22-233 and the service layer
behind it (src/ksana_llm/endpoints/local/local_endpoint.cpp:31-128,
src/ksana_llm/endpoints/streaming/streaming_iterator.cpp:17-100): generate returns (Status, output) where
output carries input_tokens / output_tokens / logprobs per returned sequence; the streaming iterator yields
the cumulative outputs after every step and aborts the request when it is dropped.
"""
from __future__ import annotations

import asyncio
import logging
import os
import threading
from functools import partial
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from ..config import load_model_config, load_yaml_config
from ..llm import LLM
from ..runtime.sampler import beam_final_order
from ..utils import native_engine as ne
from .forward_api import verify_request_target
from .plugin import KsanaPlugin, PluginConfig
from .request_packer import pack_responses, unpack_requests

logger = logging.getLogger(__name__)


@dataclass
class EndpointConfig:
    endpoint: str = "python"      # "python": the HTTP front of this package; another name: an RPC endpoint plug-in
    host: str = "0.0.0.0"
    port: int = 8080
    access_log: bool = True

    @property
    def type(self) -> str:
        return self.endpoint


class Status:
    def __init__(self, code: int = 0, message: str = ""):
        self.code, self.message = int(code), message

    def OK(self) -> bool:
        return self.code == 0

    def GetCode(self):
        return self

    @property
    def value(self) -> int:
        return self.code

    def GetMessage(self) -> str:
        return self.message

    def ToString(self) -> str:
        return "OK" if self.OK() else f"{self.code}: {self.message}"


class _Record:
    """An attribute record that also answers like a dict: plug-ins written for the reference set attributes
    (``ksana_python_input.input_tokens = ...``), the plug-ins of this package index (``inp["input_tokens"]``)."""

    def __getitem__(self, key):
        try:
            return getattr(self, key)
        except AttributeError:
            raise KeyError(key) from None

    def __setitem__(self, key, value):
        setattr(self, key, value)

    def __contains__(self, key):
        return hasattr(self, key)

    def get(self, key, default=None):
        return getattr(self, key, default)

    def setdefault(self, key, default=None):
        if not hasattr(self, key):
            setattr(self, key, default)
        return getattr(self, key)


class InputRefitEmbedding(_Record):
    """Embeddings a plug-in splices over prompt positions: ``pos`` (start position of every piece), the pieces as
    nested lists (``embeddings``) or tensors (``embedding_tensors``), and ``additional_tensors`` (multimodal rotary
    positions [3, T] first), as in src/ksana_llm/python/ksana_plugin/qwen2_vl/ksana_plugin.py:128-135."""

    def __init__(self, pos=None, embeddings=None):
        self.pos = list(pos or [])
        self.embeddings = embeddings if embeddings is not None else []
        self.embedding_tensors = ()
        self.additional_tensors = []

    def pieces(self):
        return self.embedding_tensors if len(self.embedding_tensors) else self.embeddings


class KsanaPythonInput(_Record):
    """What a plug-in's ``preprocess`` receives and may rewrite."""

    def __init__(self, input_tokens=None, sampling_config=None, model_name: str = "", input_refit_embedding=None,
                 structured_output_regex: str = "", additional_params=None, prompt=None):
        self.model_name = model_name
        self.input_tokens = list(input_tokens or [])
        self.sampling_config = sampling_config
        self.input_refit_embedding = input_refit_embedding or {}
        self.structured_output_regex = structured_output_regex
        self.request_target = {}         # target name -> {"token_id" | "slice_pos", "token_reduce_mode"} (as /forward takes)
        self.additional_params = additional_params or {}
        self.prompt = prompt

    def __setattr__(self, key, value):
        if key == "input_refit_embedding" and not isinstance(value, InputRefitEmbedding):
            value = InputRefitEmbedding((value or {}).get("pos"), (value or {}).get("embeddings"))
        object.__setattr__(self, key, value)


@dataclass
class KsanaPythonOutput:
    input_tokens: List[int] = field(default_factory=list)
    output_tokens: List[List[int]] = field(default_factory=list)
    logprobs: List[list] = field(default_factory=list)
    response: Dict[str, Any] = field(default_factory=dict)
    embedding: List[Any] = field(default_factory=list)
    finished: bool = False


def make_sampling_config(gen: Any) -> "ne.SamplingConfig":
    """HF-style generation config (object or dict) -> native SamplingConfig. ``do_sample=False`` (or unset
    with default top-k) means greedy, i.e. topk=1 (serving_model.py:220-233 of the reference)."""
    get = (lambda k, d=None: gen.get(k, d)) if isinstance(gen, dict) else (lambda k, d=None: getattr(gen, k, d))
    c = ne.SamplingConfig()
    c.topk = int(get("top_k", get("topk", 1)) or 1)
    c.topp = float(get("top_p", get("topp", 1.0)) or 1.0)
    c.temperature = float(get("temperature", 1.0) or 1.0)
    do_sample = get("do_sample", None)
    if do_sample is False or c.topk == 1:
        # greedy: the other sampling knobs go back to neutral as well, so that reported log-probabilities are those of
        # the unscaled distribution
        c.topk, c.topp, c.temperature = 1, 1.0, 1.0
    mx = get("max_new_tokens", -1)
    c.max_new_tokens = int(mx) if mx is not None and int(mx) > 0 else 1024
    c.logprobs_num = int(get("logprobs_num", get("logprobs", 0)) or 0)
    c.repetition_penalty = float(get("repetition_penalty", 1.0) or 1.0)
    c.no_repeat_ngram_size = int(get("no_repeat_ngram_size", 0) or 0)
    c.encoder_no_repeat_ngram_size = int(get("encoder_no_repeat_ngram_size", 0) or 0)
    c.num_beams = int(get("num_beams", 1) or 1)
    c.num_return_sequences = int(get("num_return_sequences", 1) or 1)
    c.length_penalty = float(get("length_penalty", 1.0) or 1.0)
    c.stop_strings = list(get("stop_strings", []) or [])
    c.stop_token_ids = [int(t) for t in (get("stop_token_ids", []) or [])]
    c.ignore_eos = bool(get("ignore_eos", False))
    seed = get("seed", 0)
    c.seed = int(seed) if seed else 0
    return c


class PyAsyncStreamingIterator:
    """Async iterator over a streaming request. Dropping it (client disconnect) aborts the request."""

    def __init__(self, engine, req, output_fn, postprocess=None):
        self.engine, self.req, self.output_fn, self.postprocess = engine, req, output_fn, postprocess
        self._done = False

    def __aiter__(self):
        return self

    def _next_blocking(self):
        item = self.req.stream_queue.get()
        return item

    async def __anext__(self):
        if self._done:
            raise StopAsyncIteration
        loop = asyncio.get_event_loop()
        item = await loop.run_in_executor(None, self._next_blocking)
        if item is None:
            self._done = True
            raise StopAsyncIteration
        out = self.output_fn(self.req)
        if self.postprocess is not None:
            await loop.run_in_executor(None, self.postprocess, out)
        return out

    def __del__(self):
        if not self._done and not self.req.done.is_set():
            self.engine.abort(self.req)


class AsyncRequestFollower:
    """Event-loop side of a request: the engine's loop thread calls :meth:`post` with every streamed piece and with
    None at the end; the items cross to the event loop through ``call_soon_threadsafe`` into an ``asyncio.Queue``.
    As an async iterator it yields the request's output after every piece (streaming); :meth:`finished` waits for
    the end (blocking requests). Closing or dropping it before the end (client disconnect) aborts the request."""

    def __init__(self, loop, engine, output_fn, postprocess=None, executor=None):
        self.loop, self.engine, self.output_fn = loop, engine, output_fn
        self.postprocess, self.executor = postprocess, executor      # the plug-in's hook for every streamed output
        self.queue: asyncio.Queue = asyncio.Queue()
        self.req = None
        self._done = False
        self._end_seen = False

    def post(self, item) -> None:             # engine loop thread
        try:
            self.loop.call_soon_threadsafe(self.queue.put_nowait, item)
        except RuntimeError:                  # the event loop is gone (server shutting down): nobody is listening
            pass

    async def finished(self) -> None:
        while not self._done:
            if await self.queue.get() is None:
                self._done = True

    def __aiter__(self):
        return self

    async def __anext__(self):
        if self._done or self._end_seen:
            self._done = True
            raise StopAsyncIteration
        if await self.queue.get() is None:
            self._done = True
            raise StopAsyncIteration
        # pieces that piled up while the consumer was busy collapse into one output (each stands for "all tokens so
        # far"); an end marker among them is honoured on the next call, after this last output
        while not self.queue.empty():
            if self.queue.get_nowait() is None:
                self._end_seen = True
                break
        out = self.output_fn(self.req)
        if self.postprocess is not None:
            await self.loop.run_in_executor(self.executor, self.postprocess, out)
        return out

    def close(self) -> None:
        if not self._done and self.req is not None and not self.req.done.is_set():
            self.engine.abort(self.req)
        self._done = True

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


class ServingModel:
    def __init__(self, config_file: str, llm: Optional[LLM] = None, tokenizer=None):
        self._config_file = config_file
        self.llm = llm
        self.tokenizer = tokenizer
        self.plugin: Optional[KsanaPlugin] = None
        self._stopped = threading.Event()
        self.endpoint_config = EndpointConfig()
        self.model_cfg = llm.model_cfg if llm is not None else None

    # ------------------------------------------------------------------ lifecycle
    def init_serving(self, plugin_config: Optional[PluginConfig] = None, endpoint_config: Optional[EndpointConfig] = None,
                     weights="checkpoint", device: Optional[str] = None):
        if endpoint_config is not None:
            self.endpoint_config = endpoint_config
        if self.llm is None:
            cfg = load_yaml_config(self._config_file)
            if self.tokenizer is None:
                # AutoModel.from_config(yaml) users pass no tokenizer: take the one beside the checkpoint (stop strings,
                # structured output and text prompts of /forward need it)
                tdir = getattr(cfg, "tokenizer_dir", "") or getattr(cfg, "model_dir", "")
                if tdir and os.path.isdir(tdir) and any(os.path.exists(os.path.join(tdir, f)) for f in
                                                        ("tokenizer.json", "tokenizer.model", "tokenizer_config.json", "vocab.json")):
                    try:
                        from transformers import AutoTokenizer
                        self.tokenizer = AutoTokenizer.from_pretrained(tdir, trust_remote_code=True)
                    except Exception as e:          # noqa: BLE001 - a broken tokenizer directory must not stop token-id serving
                        logger.warning("tokenizer in %s could not be loaded: %s", tdir, e)
            self.llm = LLM(cfg, None, weights=weights, device=device, tokenizer=self.tokenizer)
            self.model_cfg = self.llm.model_cfg
        self.llm.engine.tokenizer = self.tokenizer
        if plugin_config is not None:
            self.plugin = KsanaPlugin(plugin_config)
        prof = self.llm.engine_cfg.profiler
        if prof.attributes:
            ne.metrics_set_attributes(dict(prof.attributes))
        # http:// export targets speak OTLP/HTTP with JSON bodies to a collector (/v1/traces, /v1/metrics)
        ne.otlp_configure({str(k): str(v) for k, v in (prof.attributes or {}).items()}, int(prof.export_timeout_millis))
        stat_file = os.environ.get("KLLM_STAT_FILE", "")
        if prof.metrics_export_url:
            ne.metrics_start_export(prof.metrics_export_url, prof.export_interval_millis)
        elif stat_file:
            # no collector configured: one JSON line of all metrics per interval appended to the statistics file
            # (the variable names it as for the reference's profile writer, src/ksana_llm/profiler/writer.cpp:10-19)
            if os.path.dirname(stat_file):
                os.makedirs(os.path.dirname(stat_file), exist_ok=True)
            ne.metrics_start_export(stat_file, prof.export_interval_millis)
        if prof.trace_export_url:
            ne.span_set_sink(prof.trace_export_url)
        from ..utils import version_reporter
        version_reporter.init(self.llm.engine_cfg.global_.is_version_report)
        if self.llm.rank == 0:
            self.llm.engine.start()
            self._start_rpc_endpoint()

    def _start_rpc_endpoint(self):
        """An ``endpoint_type`` other than "python" names a plug-in: ``lib<name>_endpoint.so`` exporting
        ``Create<Name>Endpoint`` (looked up in the model directory, then on the loader path), which serves requests
        through its own transport and calls back into this model
        (src/ksana_llm/endpoints/endpoint_factory.cpp:19-39, src/ksana_llm/service/inference_server.cpp:96-118)."""
        kind = (self.endpoint_config.endpoint or "python").lower()
        self.rpc_endpoint = None
        if kind in ("python", "", "none"):
            return
        import json
        search = self.llm.engine_cfg.model_dir or ""
        self.rpc_endpoint = ne.EndpointPlugin(kind, search)

        def handler(which: str, body: bytes):
            try:
                if which == "forward":
                    status, out = self.forward(body)
                    return (200 if status.OK() else 500), (out or b"")
                req = json.loads(body.decode("utf-8"))
                status, out = self.generate(inputs=req.get("input_tokens"), generation_config=req.get("sampling_config") or {},
                                            messages=req.get("messages"))
                if not status.OK():
                    return 500, json.dumps({"message": status.message, "code": status.code}).encode()
                return 200, json.dumps({"output_token_ids": out.output_tokens, "input_token_ids": out.input_tokens,
                                        "logprobs": out.logprobs}).encode()
            except Exception as e:  # noqa: BLE001 - a transport plug-in gets an error reply, never an exception
                return 500, str(e).encode()

        rc = self.rpc_endpoint.start(handler, self.shutdown, self.endpoint_config.host, int(self.endpoint_config.port))
        if rc != 0:
            raise RuntimeError(f"endpoint plug-in {self.rpc_endpoint.path} failed to start (code {rc})")

    def wait_for_shutdown(self, timeout: Optional[float] = None) -> bool:
        """Blocks until :meth:`shutdown` has run (the process of an RPC endpoint has nothing else to do)."""
        return self._stopped.wait(timeout)

    def shutdown(self):
        self._stopped.set()
        ep = getattr(self, "rpc_endpoint", None)
        if ep is not None:
            self.rpc_endpoint = None
            ep.stop()
        if self.llm is not None:
            self.llm.shutdown(stop_followers=True)
        ne.metrics_stop_export()

    # ------------------------------------------------------------------ generate
    def _output_of(self, req) -> KsanaPythonOutput:
        outs = list(req.outputs)
        cfg = req.cfg
        if cfg.num_beams > 1 and req.all_finished():
            order = beam_final_order(outs, cfg.length_penalty)
            outs = [outs[i] for i in order][:max(cfg.num_return_sequences, 1)]
        return KsanaPythonOutput(input_tokens=list(req.prompt), output_tokens=[list(o.tokens) for o in outs],
                                 logprobs=[list(o.logprobs) for o in outs], finished=req.all_finished(),
                                 response=dict(req.response))

    def _submit(self, inputs, generation_config, streamer, messages, req_ctx, kwargs, listener=None):
        """Validation, the plug-in's preprocessing and the hand-over to the engine: (Status, request, plug-in input)."""
        gen = generation_config if generation_config is not None else {}
        sampling = make_sampling_config(gen)
        code, msg = sampling.verify_args()
        if code != 0:
            return Status(code, msg), None, None
        ksana_input = KsanaPythonInput(inputs, sampling, kwargs.get("model_name") or "", kwargs.get("input_refit_embedding"),
                                       kwargs.get("structured_output_regex") or "", kwargs.get("additional_params"),
                                       kwargs.get("prompt"))
        # a request that brings its own spliced embeddings is not pre-processed again (as in the reference)
        if self.plugin is not None and not ksana_input.input_refit_embedding.pos:
            self.plugin.preprocess(ksana_python_input=ksana_input, messages=messages,
                                   additional_params=ksana_input.additional_params, prompt=ksana_input.prompt or "")
        tokens = list(ksana_input.input_tokens)
        if not tokens:
            return Status(1, "empty input tokens"), None, None
        refit = None
        emb = ksana_input.input_refit_embedding
        if emb.pos and emb.pieces() is not None and len(emb.pieces()):
            refit = (list(emb.pos), [torch.as_tensor(e, dtype=torch.float32) for e in emb.pieces()])
        extra = ksana_input.get("additional_tensors")
        mrope = extra.get("mrope_positions") if isinstance(extra, dict) else None
        if mrope is None and len(emb.additional_tensors):
            mrope = emb.additional_tensors[0]          # rotary positions [3, T] of a multimodal prompt
        span = ne.span_start("generate", (req_ctx or {}).get("traceparent", ""))
        req = self.llm.engine.add_request(tokens, sampling, stream=bool(streamer),
                                          structured_regex=ksana_input.structured_output_regex or "",
                                          request_target=dict(ksana_input.request_target) or None,
                                          refit=refit, mrope_positions=mrope, listener=listener)
        req.span_id = span
        if req.done.is_set() and req.status_code != 0:
            return Status(req.status_code, req.status_message), None, None
        return Status(), req, ksana_input

    def _stream_postprocess(self, ksana_input):
        """The plug-in's post-processing as a one-argument call for every streamed output (the reference's streaming
        iterator runs it on each piece, src/ksana_llm/python/ksana_llm/serving_model.py:45-58); None without a plug-in."""
        if self.plugin is None or not self.plugin.loaded:
            return None
        return lambda out: self.plugin.postprocess(ksana_python_input=ksana_input, ksana_python_output=out)

    def generate(self, model_name: str = "", inputs: Optional[List[int]] = None, generation_config: Any = None,
                 streamer=None, messages=None, req_ctx: Optional[Dict[str, str]] = None, **kwargs):
        """Returns (Status, KsanaPythonOutput) or, with ``streamer``, (Status, async iterator). The calling thread
        waits for the result; the HTTP front uses :meth:`generate_async`, which holds no thread while a request runs."""
        status, req, ksana_input = self._submit(inputs, generation_config, streamer, messages, req_ctx, kwargs)
        if not status.OK():
            return status, None
        if streamer:
            return Status(), PyAsyncStreamingIterator(self.llm.engine, req, self._output_of,
                                                      self._stream_postprocess(ksana_input))
        req.done.wait()
        if req.status_code != 0:
            return Status(req.status_code, req.status_message), None
        out = self._output_of(req)
        if self.plugin is not None:
            self.plugin.postprocess(ksana_python_input=ksana_input, ksana_python_output=out)
        return Status(), out

    async def generate_async(self, model_name: str = "", inputs: Optional[List[int]] = None, generation_config: Any = None,
                             streamer=None, messages=None, req_ctx: Optional[Dict[str, str]] = None, executor=None,
                             **kwargs):
        """:meth:`generate` for callers on an asyncio event loop. Preparation (validation, plug-in, hand-over to the
        engine) runs on ``executor``; from then on the engine's loop thread posts every streamed piece and the end of
        the request to the event loop, so that a request in flight occupies no thread: thousands of open requests
        cost thousands of small queues, not thousands of blocked threads. Same return values as :meth:`generate`."""
        loop = asyncio.get_running_loop()
        follower = AsyncRequestFollower(loop, self.llm.engine, self._output_of)
        status, req, ksana_input = await loop.run_in_executor(
            executor, partial(self._submit, inputs, generation_config, streamer, messages, req_ctx, kwargs, follower.post))
        if not status.OK():
            return status, None
        follower.req = req
        if streamer:
            follower.postprocess, follower.executor = self._stream_postprocess(ksana_input), executor
            return Status(), follower
        await follower.finished()
        if req.status_code != 0:
            return Status(req.status_code, req.status_message), None
        out = self._output_of(req)
        if self.plugin is not None:
            await loop.run_in_executor(executor, partial(self.plugin.postprocess, ksana_python_input=ksana_input,
                                                         ksana_python_output=out))
        return Status(), out

    # ------------------------------------------------------------------ forward
    def _forward_submit(self, request_bytes: bytes, listener=None):
        """Decoding, validation and hand-over of a /forward batch: (Status, requests in flight)."""
        try:
            reqs_in = unpack_requests(request_bytes, self.tokenizer)
        except Exception as e:  # noqa: BLE001
            return Status(1, f"failed to parse request: {e}"), None
        engine = self.llm.engine
        if getattr(engine.model, "dp", None) is not None:
            # attention data parallelism spreads the rows of a step over the ranks; request targets address rows of
            # the whole step, so they are served by tensor- or pipeline-parallel deployments only
            return Status(1, "request targets are not supported with attention data parallelism"), None
        pending = []
        for r in reqs_in:
            code, msg = verify_request_target(r["request_target"], len(r["input_tokens"]))
            if code != 0:
                return Status(code, msg), None
        for r in reqs_in:
            s = ne.SamplingConfig()
            s.max_new_tokens = 1
            refit = None
            emb = r.get("input_refit_embedding") or {}
            if emb.get("pos") and emb.get("embeddings") is not None:
                refit = (list(emb["pos"]), [torch.as_tensor(e, dtype=torch.float32) for e in emb["embeddings"]])
            pending.append(engine.add_request(r["input_tokens"], s, request_target=r["request_target"], refit=refit,
                                              listener=listener))
        return Status(), pending

    @staticmethod
    def _forward_pack(pending):
        for req in pending:
            if req.status_code != 0:
                return Status(req.status_code, req.status_message), None
        return Status(), pack_responses([(req.prompt, req.response) for req in pending])

    def forward(self, request_bytes: bytes, req_ctx: Optional[Dict[str, str]] = None):
        """msgpack batch of prefill-only requests with request targets -> msgpack responses."""
        status, pending = self._forward_submit(request_bytes)
        if not status.OK():
            return status, None
        for req in pending:
            req.done.wait()
        return self._forward_pack(pending)

    async def forward_async(self, request_bytes: bytes, req_ctx: Optional[Dict[str, str]] = None, executor=None):
        """:meth:`forward` for callers on an event loop: decoding and packing run on ``executor``, and no thread waits
        while the batch is in the engine (every request posts its end to the loop)."""
        loop = asyncio.get_running_loop()
        ends: asyncio.Queue = asyncio.Queue()

        def post(item):                       # engine loop thread; only the end of a request matters here
            if item is None:
                try:
                    loop.call_soon_threadsafe(ends.put_nowait, None)
                except RuntimeError:
                    pass
        status, pending = await loop.run_in_executor(executor, partial(self._forward_submit, request_bytes, post))
        if not status.OK():
            return status, None
        for _ in pending:
            await ends.get()
        return await loop.run_in_executor(executor, partial(self._forward_pack, pending))
