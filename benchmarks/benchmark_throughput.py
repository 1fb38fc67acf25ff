"""Serving benchmark client for the /generate endpoint: request-rate / concurrency controlled load, streaming or
blocking requests, throughput and latency statistics.

Same measurement definitions and the same main flags as the reference's benchmarks/benchmark_throughput.py
(argument list :127-275, statistics :59-123 and :809-880), so existing run scripts keep working:

  request throughput   = finished requests / wall time
  token throughput     = (input tokens + output tokens) / wall time
  latency              = per request, send to last byte
  TTFT                 = send to the first streamed chunk that carries a token           (--stream only)
  ITL                  = gaps between consecutive streamed chunks
  TPOT                 = (latency - TTFT) / (output tokens - 1)

Prompts come from a CSV column (--input_csv / --col_idx, e.g. the reference's share_gpt_500.csv) or are synthetic
token-id prompts (--synthetic N:IN_LEN:OUT_LEN[:SIGMA], log-normal lengths around IN_LEN when SIGMA > 0), which need
no tokenizer on either side. Requests are sent by an asyncio client (aiohttp); ``--mode sync`` uses blocking
``requests`` calls from a thread pool of ``--concurrency`` workers instead.

  python benchmarks/benchmark_throughput.py --port 8080 --synthetic 500:512:128 --request_rate 8 --stream
"""
from __future__ import annotations

import argparse
import asyncio
import csv
import json
import math
import random
import os
import sys
import time
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class RequestRecord:
    prompt_len: int = 0
    output_len: int = 0
    start: float = 0.0
    first_token: Optional[float] = None
    end: float = 0.0
    chunk_times: List[float] = field(default_factory=list)
    ok: bool = True
    error: str = ""
    text: str = ""

    @property
    def latency(self) -> float:
        return self.end - self.start

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token is None else self.first_token - self.start

    @property
    def tpot(self) -> Optional[float]:
        if self.first_token is None or self.output_len < 2:
            return None
        return (self.end - self.first_token) / (self.output_len - 1)

    @property
    def itls(self) -> List[float]:
        return [b - a for a, b in zip(self.chunk_times[:-1], self.chunk_times[1:])]


def percentile(values: List[float], p: float) -> float:
    if not values:
        return float("nan")
    v = sorted(values)
    k = (len(v) - 1) * p / 100.0
    lo, hi = math.floor(k), math.ceil(k)
    return v[lo] if lo == hi else v[lo] + (v[hi] - v[lo]) * (k - lo)


def summarize(records: List[RequestRecord], wall: float, percentiles=(50, 99)) -> dict:
    """Aggregate statistics of one benchmark iteration."""
    done = [r for r in records if r.ok]
    n_in = sum(r.prompt_len for r in done)
    n_out = sum(r.output_len for r in done)
    lat = [r.latency for r in done]
    out = {
        "requests": len(records), "finished": len(done), "failed": len(records) - len(done), "wall_s": wall,
        "request_throughput": len(done) / wall if wall > 0 else 0.0,
        "token_throughput": (n_in + n_out) / wall if wall > 0 else 0.0,
        "output_token_throughput": n_out / wall if wall > 0 else 0.0,
        "avg_latency_s": sum(lat) / len(lat) if lat else float("nan"),
        "avg_input_tokens": n_in / len(done) if done else 0.0,
        "avg_output_tokens": n_out / len(done) if done else 0.0,
    }
    ttft = [r.ttft for r in done if r.ttft is not None]
    tpot = [r.tpot for r in done if r.tpot is not None]
    itl = [x for r in done for x in r.itls]
    for name, vals in (("latency_s", lat), ("ttft_s", ttft), ("tpot_s", tpot), ("itl_s", itl)):
        if not vals:
            continue
        if name != "latency_s":
            out[f"avg_{name}"] = sum(vals) / len(vals)
        for p in percentiles:
            out[f"p{p:g}_{name}"] = percentile(vals, p)
    return out


def synthetic_prompts(spec: str, vocab: int, seed: int):
    """N:IN_LEN:OUT_LEN[:SIGMA] -> list of (token ids, max_new_tokens)."""
    parts = spec.split(":")
    n, in_len, out_len = int(parts[0]), int(parts[1]), int(parts[2])
    sigma = float(parts[3]) if len(parts) > 3 else 0.0
    rng = random.Random(seed)
    prompts = []
    for _ in range(n):
        L = in_len if sigma <= 0 else max(1, int(round(rng.lognormvariate(math.log(in_len), sigma))))
        prompts.append(([rng.randrange(3, vocab) for _ in range(L)], out_len))
    return prompts


def read_prompts(path: str, col_idx: int, prompt_num: int, shuffle: bool, seed: int) -> List[str]:
    with open(path, "r", encoding="utf-8", newline="") as f:
        rows = list(csv.reader(f))
    prompts = [r[col_idx] for r in rows[1:] if len(r) > col_idx and r[col_idx]]
    if shuffle:
        random.Random(seed).shuffle(prompts)
    return prompts[:prompt_num] if prompt_num > 0 else prompts


_TOKENIZER = None


def load_tokenizer(args):
    global _TOKENIZER
    if _TOKENIZER is None:
        if not args.tokenizer_path:
            raise SystemExit("--chat_template needs --tokenizer_path")
        from transformers import AutoTokenizer
        _TOKENIZER = AutoTokenizer.from_pretrained(args.tokenizer_path, trust_remote_code=True)
    return _TOKENIZER


def apply_chat_template(args, prompt: str, tokenizer=None) -> str:
    """The prompt as the single user turn of a conversation, rendered to text with the generation prompt appended."""
    tok = tokenizer or load_tokenizer(args)
    return tok.apply_chat_template([{"role": "user", "content": prompt}], tokenize=False, add_generation_prompt=True)


def build_payload(args, prompt, max_new_tokens: Optional[int] = None) -> dict:
    builder = BACKENDS[getattr(args, "backend", "ksana")][1]
    if builder is not None:
        if not isinstance(prompt, str):
            raise SystemExit("--synthetic token-id prompts need --backend ksana (other servers take text)")
        return builder(args, prompt, max_new_tokens or args.max_new_tokens)
    sampling = {
        "temperature": args.temperature, "topk": args.topk, "topp": args.topp,
        "max_new_tokens": max_new_tokens or args.max_new_tokens, "repetition_penalty": args.repetition_penalty,
        "no_repeat_ngram_size": args.no_repeat_ngram_size, "encoder_no_repeat_ngram_size": args.encoder_no_repeat_ngram_size,
        "length_penalty": args.length_penalty, "num_beams": args.num_beams,
        "num_return_sequences": args.num_return_sequences, "logprobs": args.logprobs, "ignore_eos": args.ignore_eos,
        "stop_token_ids": args.stop_token_ids or [],
    }
    if args.stop_strings:
        sampling["stop_strings"] = list(args.stop_strings)
    body = {"sampling_config": sampling, "stream": bool(args.stream)}
    if args.structured_output_regex:
        body["structured_output_regex"] = args.structured_output_regex
    if isinstance(prompt, str):
        body["prompt"] = prompt
    else:
        body["input_tokens"] = list(prompt)
    return body


# ---------------------------------------------------------------------------------------------------------------
# Other servers behind the same load generator (the reference's --backend values, benchmarks/benchmark_throughput.py
# :390-470 request bodies and :565-605 answers). An adapter names the URL path, builds the request body from the
# common flags and reads prompt / output token counts and the text out of the last JSON object of the answer. Token
# counts the server does not report are taken from --tokenizer_path when one is given, else they stay zero.
def _body_vllm(args, prompt, n_new):
    return {"prompt": prompt, "n": 1, "temperature": args.temperature, "max_tokens": n_new, "logprobs": args.logprobs or None,
            "repetition_penalty": args.repetition_penalty, "stop_token_ids": args.stop_token_ids or [],
            "ignore_eos": args.ignore_eos, "min_tokens": n_new if args.ignore_eos else 0, "skip_special_tokens": False,
            "spaces_between_special_tokens": False, "top_p": args.topp, "top_k": args.topk, "stream": bool(args.stream)}


def _body_trt(args, prompt, n_new):
    return {"accumulate_tokens": True, "text_input": prompt, "max_tokens": n_new, "temperature": args.temperature,
            "min_tokens": n_new if args.ignore_eos else 0, "bad_words": "", "stop_words": "", "top_p": args.topp,
            "top_k": args.topk, "stream": bool(args.stream)}


def _body_sglang(args, prompt, n_new):
    return {"text": prompt, "stream": bool(args.stream),
            "sampling_params": {"n": 1, "temperature": args.temperature, "max_new_tokens": n_new,
                                "stop_token_ids": args.stop_token_ids or [], "ignore_eos": args.ignore_eos,
                                "top_p": args.topp, "top_k": args.topk, "skip_special_tokens": False,
                                "spaces_between_special_tokens": False, "repetition_penalty": args.repetition_penalty}}


def _body_chat_server(args, prompt, n_new):
    return {"model": "default_model", "prompt": prompt, "messages": [{"role": "user", "content": prompt}],
            "top_p": args.topp, "temperature": args.temperature, "top_k": args.topk,
            "repetition_penalty": args.repetition_penalty, "logprobs": args.logprobs, "n": 1, "task_id": time.time(),
            "delete_prompt_from_output": 1, "stream": bool(args.stream), "stop_token_ids": args.stop_token_ids or [],
            "max_new_tokens": n_new, "max_tokens": n_new, "ignore_eos": args.ignore_eos,
            "structured_output_regex": args.structured_output_regex or None}


def _count(tok, text):
    return len(tok.encode(text)) if (tok is not None and text) else 0


def _read_prompt_echo(body, prompt, tok, strip_prompt):
    text = (body.get("text") or [""])
    text = text[0] if isinstance(text, list) else text
    if strip_prompt and isinstance(prompt, str) and text.startswith(prompt):
        text = text[len(prompt):]
    outs = body.get("output_token_ids")
    n_out = len(outs[0]) if outs else _count(tok, text)
    return _count(tok, prompt if isinstance(prompt, str) else ""), n_out, text.strip()


def _read_trt(body, prompt, tok, _):
    text = (body.get("text_output") or "").strip()
    return _count(tok, prompt if isinstance(prompt, str) else ""), _count(tok, text), text


def _read_sglang(body, prompt, tok, _):
    meta = body.get("meta_info") or {}
    return int(meta.get("prompt_tokens", 0)), int(meta.get("completion_tokens", 0)), (body.get("text") or "").strip()


def _read_chat_server(body, prompt, tok, streamed_text):
    usage = body.get("usage") or {}
    choice = (body.get("choices") or [{}])[0]
    text = streamed_text if streamed_text else ((choice.get("message") or choice.get("delta") or {}).get("content")
                                                or choice.get("text") or "")
    n_out = int(usage.get("completion_tokens", 0)) or _count(tok, text)
    return int(usage.get("prompt_tokens", 0)), n_out, text


BACKENDS = {
    # name: (url path; "+_stream" marks a path that gets that suffix for streaming), body builder, answer reader,
    #        strip the echoed prompt from the text
    "ksana": ("/generate", None, None, False),
    "vllm": ("/generate", _body_vllm, _read_prompt_echo, True),
    "mindie-service": ("/generate", _body_vllm, _read_prompt_echo, True),
    "evart": ("/generate", _body_vllm, _read_prompt_echo, False),
    "trt-llm": ("/v2/models/ensemble/generate+_stream", _body_trt, _read_trt, False),
    "sglang": ("/generate", _body_sglang, _read_sglang, False),
    "ksana-server": ("/v1/chat", _body_chat_server, _read_chat_server, False),
    "vllm-server": ("/v1/chat", _body_chat_server, _read_chat_server, False),
}


def backend_url(args) -> str:
    path = BACKENDS[args.backend][0]
    if path.endswith("+_stream"):
        path = path[:-len("+_stream")] + ("_stream" if args.stream else "")
    return f"http://{args.host}:{args.port}{path}"


def iter_json_objects(buf: bytes):
    """Splits what has arrived of a streamed answer into complete JSON objects and the unfinished rest. Servers frame
    their objects with zero bytes (this engine), with "data: " lines (server-sent events) or with new lines."""
    out = []
    while True:
        hits = [(i, len(sep)) for sep in (b"\0", b"\n\n", b"\n") for i in [buf.find(sep)] if i >= 0]
        if not hits:
            break
        at, width = min(hits)
        piece, rest = buf[:at].strip(), buf[at + width:]
        if piece.startswith(b"data:"):
            piece = piece[5:].strip()
        if piece and piece != b"[DONE]":
            try:
                out.append(json.loads(piece))
            except ValueError:
                break                  # a separator inside an unfinished object: wait for more bytes
        buf = rest
    return out, buf


def _finish(rec: RequestRecord, body: Optional[dict], args=None, prompt=None, tok=None, streamed_text=""):
    if body is None:
        return
    reader = BACKENDS[getattr(args, "backend", "ksana")][2] if args is not None else None
    if reader is not None:
        if "error" in body:
            rec.ok, rec.error = False, str(body["error"])[:200]
            return
        extra = streamed_text if reader is _read_chat_server else BACKENDS[args.backend][3]
        n_in, n_out, rec.text = reader(body, prompt, tok, extra)
        rec.output_len = n_out
        if rec.prompt_len == 0:
            rec.prompt_len = n_in
        return
    outs = body.get("output_token_ids") or []
    rec.output_len = sum(len(o) for o in outs)
    if rec.prompt_len == 0:
        rec.prompt_len = len(body.get("input_token_ids") or [])
    texts = body.get("texts") or []
    rec.text = texts[0] if texts else ""


async def send_async(session, url: str, payload: dict, rec: RequestRecord, args=None, prompt=None, tok=None):
    """One request. This engine streams JSON objects separated by a zero byte (one per engine step); the other
    backends' framings are handled by ``iter_json_objects``."""
    rec.start = time.perf_counter()
    foreign = args is not None and BACKENDS[args.backend][1] is not None
    try:
        async with session.post(url, json=payload) as resp:
            if resp.status != 200:
                rec.ok, rec.error = False, f"HTTP {resp.status}: {(await resp.text())[:200]}"
                rec.end = time.perf_counter()
                return
            if payload.get("stream") and foreign:
                buf, last, text = b"", None, ""
                async for chunk in resp.content.iter_any():
                    buf += chunk
                    objs, buf = iter_json_objects(buf)
                    now = time.perf_counter()
                    for obj in objs:
                        last = obj
                        delta = ((obj.get("choices") or [{}])[0].get("delta") or {}).get("content") if "choices" in obj else None
                        if delta:
                            text += delta
                        if rec.first_token is None:
                            rec.first_token = now
                        rec.chunk_times.append(now)
                tail = buf.strip(b"\0 \n")
                if tail.startswith(b"data:"):
                    tail = tail[5:].strip()
                if tail and tail != b"[DONE]":
                    try:
                        last = json.loads(tail)
                    except ValueError:
                        pass
                _finish(rec, last, args, prompt, tok, text)
            elif payload.get("stream"):
                buf, last = b"", None
                async for chunk in resp.content.iter_any():
                    buf += chunk
                    while b"\0" in buf:
                        piece, buf = buf.split(b"\0", 1)
                        if not piece:
                            continue
                        now = time.perf_counter()
                        last = json.loads(piece)
                        if any(len(o) for o in last.get("output_token_ids") or []):
                            if rec.first_token is None:
                                rec.first_token = now
                            rec.chunk_times.append(now)
                if buf.strip(b"\0"):
                    last = json.loads(buf.strip(b"\0"))
                _finish(rec, last)
            else:
                _finish(rec, await resp.json(content_type=None), args, prompt, tok)
    except Exception as e:  # noqa: BLE001 - a failed request is a data point, not a crash
        rec.ok, rec.error = False, repr(e)
    rec.end = time.perf_counter()


async def run_async(args, url: str, work: list) -> List[RequestRecord]:
    import aiohttp
    records = [RequestRecord(prompt_len=0 if isinstance(p, str) else len(p)) for p, _ in work]
    sem = asyncio.Semaphore(args.concurrency) if args.request_rate == float("inf") and args.concurrency > 0 else None
    rng = random.Random(args.seed)
    timeout = aiohttp.ClientTimeout(total=args.client_timeout)
    async with aiohttp.ClientSession(timeout=timeout) as session:
        tok = _counting_tokenizer(args)

        async def one(i):
            payload = build_payload(args, work[i][0], work[i][1])
            if sem is None:
                await send_async(session, url, payload, records[i], args, work[i][0], tok)
            else:
                async with sem:
                    await send_async(session, url, payload, records[i], args, work[i][0], tok)

        tasks = []
        for i in range(len(work)):
            tasks.append(asyncio.create_task(one(i)))
            if args.request_rate != float("inf"):
                gap = rng.expovariate(args.request_rate) if args.random else 1.0 / args.request_rate
                await asyncio.sleep(gap)
        await asyncio.gather(*tasks)
    return records


def _counting_tokenizer(args):
    """Tokenizer for the token counts of servers that do not report them (None without --tokenizer_path)."""
    if BACKENDS[args.backend][1] is None or not getattr(args, "tokenizer_path", None):
        return None
    return load_tokenizer(args)


def run_sync(args, url: str, work: list) -> List[RequestRecord]:
    import requests
    from concurrent.futures import ThreadPoolExecutor
    records = [RequestRecord(prompt_len=0 if isinstance(p, str) else len(p)) for p, _ in work]
    tok = _counting_tokenizer(args)

    def one(i):
        rec = records[i]
        payload = build_payload(args, work[i][0], work[i][1])
        payload["stream"] = False
        rec.start = time.perf_counter()
        try:
            r = requests.post(url, json=payload, timeout=args.client_timeout)
            if r.status_code != 200:
                rec.ok, rec.error = False, f"HTTP {r.status_code}"
            else:
                _finish(rec, r.json(), args, work[i][0], tok)
        except Exception as e:  # noqa: BLE001
            rec.ok, rec.error = False, repr(e)
        rec.end = time.perf_counter()

    with ThreadPoolExecutor(max_workers=max(1, args.concurrency)) as ex:
        list(ex.map(one, range(len(work))))
    return records


def args_config(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--input_csv", default=None)
    p.add_argument("--col_idx", type=int, default=0)
    p.add_argument("--prefix_cache_csv", default=None,
                   help="prompt set with a shared preamble (see prefix_cache_reader.py); the shared token count is "
                        "reported when --tokenizer_path is given")
    p.add_argument("--output_csv", default=None, help="per-request outputs (prompt length, output length, latency, text)")
    p.add_argument("--perf_csv", default=None, help="one row of summary statistics per iteration")
    p.add_argument("--request_rate", type=float, default=float("inf"), help="requests per second; inf = all at once")
    p.add_argument("--request_rate_step", type=float, default=1.0)
    p.add_argument("--request_rate_num_iters", type=int, default=1, help="iterations, each request_rate_step faster")
    p.add_argument("--max_avg_latency", type=float, default=float("inf"), help="stop the rate sweep beyond this (s)")
    p.add_argument("--max_first_token_latency", type=float, default=float("inf"))
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--random", action="store_true", help="Poisson arrivals instead of a fixed gap")
    p.add_argument("--shuffle", action="store_true")
    p.add_argument("--percentiles", type=float, nargs="+", default=[99])
    p.add_argument("--concurrency", type=int, default=1, help="in-flight requests when no request rate is given")
    p.add_argument("--warmup_num_iters", type=int, default=0)
    p.add_argument("--repeat_num_iters", type=int, default=1)
    p.add_argument("--mode", default="async", choices=["async", "sync"])
    p.add_argument("--stream", action="store_true")
    p.add_argument("--backend", default="ksana", choices=sorted(BACKENDS),
                   help="server to load: this engine's /generate (default), or vllm / trt-llm / sglang / evart / "
                        "mindie-service / ksana-server / vllm-server with their own request and answer formats")
    p.add_argument("--prompt_num", type=int, default=0)
    p.add_argument("--model_type", default="llama")
    p.add_argument("--synthetic", default=None, help="N:IN_LEN:OUT_LEN[:SIGMA] synthetic token-id prompts")
    p.add_argument("--vocab_size", type=int, default=32000)
    p.add_argument("--max_new_tokens", type=int, default=1024)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--topk", type=int, default=1)
    p.add_argument("--topp", type=float, default=1.0)
    p.add_argument("--repetition_penalty", type=float, default=1.0)
    p.add_argument("--no_repeat_ngram_size", type=int, default=0)
    p.add_argument("--encoder_no_repeat_ngram_size", type=int, default=0)
    p.add_argument("--length_penalty", type=float, default=1.0)
    p.add_argument("--num_beams", type=int, default=1)
    p.add_argument("--num_return_sequences", type=int, default=1)
    p.add_argument("--logprobs", type=int, default=0)
    p.add_argument("--stop_token_ids", type=int, nargs="*", default=None)
    p.add_argument("--stop_strings", type=str, nargs="*", default=None, help="strings that end a generation")
    p.add_argument("--structured_output_regex", type=str, default=None, help="regular expression the outputs must match")
    p.add_argument("--structured_output_file", type=str, default=None, help="file holding that regular expression")
    p.add_argument("--tokenizer_path", type=str, default=None,
                   help="Hugging Face tokenizer: needed by --chat_template, and used to count tokens of text-only answers")
    p.add_argument("--chat_template", action="store_true",
                   help="wrap every prompt as one user message with the tokenizer's chat template")
    p.add_argument("--ignore_eos", action="store_true")
    p.add_argument("--client_timeout", type=float, default=3600.0)
    return p.parse_args(argv)


def run_benchmark(args) -> List[dict]:
    url = backend_url(args)
    if args.structured_output_file:
        with open(args.structured_output_file, "r", encoding="utf-8") as f:
            args.structured_output_regex = f.read().strip()
    if args.synthetic:
        work = synthetic_prompts(args.synthetic, args.vocab_size, args.seed)
        args.ignore_eos = True
    elif args.input_csv:
        work = [(p, None) for p in read_prompts(args.input_csv, args.col_idx, args.prompt_num, args.shuffle, args.seed)]
        if args.chat_template:
            work = [(apply_chat_template(args, p), n) for p, n in work]
    elif args.prefix_cache_csv:
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from prefix_cache_reader import load_prompts
        shared, prompts = load_prompts(args.prefix_cache_csv, getattr(args, "tokenizer_path", None) or None,
                                       args.prompt_num or 220)
        print(f"prefix-cache prompt set: {len(prompts)} prompts, {shared} shared prefix tokens")
        work = [(p, None) for p in prompts]
    else:
        raise SystemExit("give --input_csv, --prefix_cache_csv or --synthetic")
    pct = sorted(set([50.0] + list(args.percentiles)))
    results = []
    rate = args.request_rate
    for it in range(max(1, args.request_rate_num_iters)):
        for rep in range(args.warmup_num_iters + args.repeat_num_iters):
            t0 = time.perf_counter()
            records = asyncio.run(run_async(args, url, work)) if args.mode == "async" else run_sync(args, url, work)
            wall = time.perf_counter() - t0
            if rep < args.warmup_num_iters:
                continue
            s = summarize(records, wall, pct)
            s["request_rate"] = rate
            results.append(s)
            print(json.dumps(s))
            if args.output_csv:
                with open(args.output_csv, "w", encoding="utf-8", newline="") as f:
                    w = csv.writer(f)
                    w.writerow(["prompt_len", "output_len", "latency_s", "ttft_s", "ok", "text"])
                    for r in records:
                        w.writerow([r.prompt_len, r.output_len, f"{r.latency:.6f}", "" if r.ttft is None else f"{r.ttft:.6f}",
                                    int(r.ok), r.text])
        last = results[-1]
        if last["avg_latency_s"] > args.max_avg_latency or last.get("avg_ttft_s", 0.0) > args.max_first_token_latency:
            break
        if rate != float("inf"):
            rate += args.request_rate_step
            args.request_rate = rate
    if args.perf_csv and results:
        keys = sorted({k for r in results for k in r})
        with open(args.perf_csv, "w", encoding="utf-8", newline="") as f:
            w = csv.DictWriter(f, fieldnames=keys)
            w.writeheader()
            w.writerows(results)
    return results


if __name__ == "__main__":
    run_benchmark(args_config())
    sys.exit(0)
