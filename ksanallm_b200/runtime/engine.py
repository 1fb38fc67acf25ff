"""The engine loop: C++ scheduler -> step metadata upload -> model forward -> fused sampler ->
scheduler post-step -> per-request notification.

One engine step corresponds to the reference's ``BatchManager::MainProcess`` iteration
(src/ksana_llm/batch_manager/batch_manager.cpp:111-241) plus ``LlmRuntime::Step``
(src/ksana_llm/runtime/llm_runtime.cpp:387-445). Differences: the scheduler's plan is a flat
int32 image uploaded with one pinned host->device copy (instead of many small copies built in
``ModelInput::ParseFromRequests``), swap/copy lists are executed by one gather/scatter kernel on the
compute stream, and in multi-rank runs rank 0 broadcasts the same image to the other ranks.
"""
from __future__ import annotations

import os
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import numpy as np
import torch

from ..config import EngineConfig, ModelConfig
from ..models.common import LogitCandidates, StepInput
from ..ops import dispatch as ops
from ..ops import checks as _checks
from ..ops import native
from ..utils import logger, nvtx
from ..utils import native_engine as ne
from .sampler import DeviceStepError, Sampler, SamplingParams
from .structured import StructuredOutput


@dataclass
class SequenceOutput:
    tokens: List[int] = field(default_factory=list)
    logprobs: List[list] = field(default_factory=list)       # per token: [(id, logprob), ...]
    finished: bool = False
    cum_logprob: float = 0.0


class Request:
    """Python-side request record: outputs per sibling sequence, completion / streaming signalling."""

    def __init__(self, req_id: int, prompt: List[int], cfg, n_seqs: int, stream: bool = False, listener=None):
        self.req_id = req_id
        # ``listener(item)``: called on the engine's loop thread with every streamed piece (streaming requests) and
        # with None on completion, in place of a queue that some thread would have to block on (the HTTP front hands
        # the items to its event loop). It must not block.
        self.listener = listener
        self.stream = stream
        self.prompt = list(prompt)
        self.cfg = cfg
        self.outputs = [SequenceOutput() for _ in range(n_seqs)]
        self.seq_ids: List[int] = []
        self.status_code = 0
        self.status_message = ""
        # native waiter / channel (condition variables outside the interpreter; same methods as threading.Event and
        # queue.Queue), the interpreter's own primitives when the runtime library lacks them
        self.done = ne.Waiter() if hasattr(ne, "Waiter") else threading.Event()
        self.stream_queue = ((ne.StreamChannel() if hasattr(ne, "StreamChannel") else queue.Queue())
                             if (stream and listener is None) else None)
        self.arrive = time.time()
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self.structured: Optional[StructuredOutput] = None
        self.aborted = False
        # /forward style extraction
        self.request_target: Optional[dict] = None
        self.targets_done = False                        # the targets are taken from the prefill step, once
        self.response: Dict[str, torch.Tensor] = {}
        self.refit: Optional[tuple] = None               # (positions, embeddings)
        self.mrope_positions = None
        self.span_id: Optional[str] = None
        self.prefix_hit = 0

    def all_finished(self) -> bool:
        return all(o.finished for o in self.outputs)

    def emit(self, item) -> None:
        """A streamed piece (("step", tokens of every output so far)) or the end marker (None) to whoever follows
        this request."""
        if self.stream_queue is not None:
            self.stream_queue.put(item)
        if self.listener is not None and (item is None or self.stream):
            try:
                self.listener(item)
            except Exception as e:  # noqa: BLE001 - a follower that went away must not stop the step loop
                logger.warning(f"listener of request {self.req_id} failed: {e!r}")


class ModelRunner:
    """Owns the model, its KV cache and the per-step device metadata."""

    def __init__(self, model, block_tokens: int, num_blocks: int, num_host_blocks: int, kv_dtype=None):
        self.model = model
        self.device = model.device
        self.cuda = self.device.type == "cuda"
        self.block_tokens = block_tokens
        model.allocate_kv_cache(num_blocks, block_tokens, kv_dtype)
        self.block_bytes = model.block_bytes()
        self.host_cache = None
        if num_host_blocks > 0:
            self.host_cache = torch.zeros(num_host_blocks, self.block_bytes, dtype=torch.uint8,
                                          pin_memory=self.cuda)
        self._ring: list = []
        self._ring_pos = 0
        self._swap_stream = None
        self.exchange_candidates = os.environ.get("KSANA_SHARD_SAMPLING", "1") != "0"
        self.pipeline = None             # parallel.pipeline.PipelineRunner when the job has several stages
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    STAGE_RING = 16       # several steps of uploads may be queued behind the step in flight (pipelined stepping)

    def _stage_buffer(self, n: int):
        """Next pinned staging buffer of the ring with room for ``n`` int32 words. A buffer is rewritten only after
        the copy that last read it has completed (its event), so several asynchronous uploads of one step - block
        lists, the step image, sampler parameters - never share host memory that a DMA may still be reading."""
        ring = self._ring
        if not ring:
            ring.extend([None, 0, None] for _ in range(self.STAGE_RING))        # [buffer, capacity, event]
        self._ring_pos = (self._ring_pos + 1) % self.STAGE_RING
        slot = ring[self._ring_pos]
        if slot[2] is not None:
            slot[2].synchronize()
        if n > slot[1]:
            slot[1] = max(n * 2, 1 << 16)
            slot[0] = torch.empty(slot[1], dtype=torch.int32, pin_memory=True)
            slot[2] = torch.cuda.Event()
        return slot

    def _stage(self, arr: np.ndarray, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """int32 host array -> device through a pinned staging buffer, one asynchronous H2D copy. ``out``: device
        tensor to fill (CUDA-graph inputs); otherwise a new device tensor is returned."""
        n = int(arr.size)
        if not self.cuda:
            return torch.from_numpy(arr.copy())
        slot = self._stage_buffer(n)
        host = slot[0][:n]
        host.numpy()[:] = arr.reshape(-1)
        self.h2d_bytes += n * 4
        if out is None:
            out = host.to(self.device, non_blocking=True)
        else:
            out.copy_(host, non_blocking=True)
        slot[2].record()
        return out

    def apply_block_ops(self, plan) -> None:
        """Block copies of forks decided after the previous step, then swap-outs, swap-ins and the copies decided by
        this plan, in that order. On a GPU the four lists travel in one staged upload; a swap is one kernel per
        direction that moves the blocks between the cache and the pinned host pool over PCIe (no staging copy, no
        host synchronisation), issued on a side stream that the compute stream joins before the forward."""
        pre = np.asarray(getattr(plan, "pre_copies", ()), dtype=np.int32)
        so, si, cp = np.asarray(plan.swap_out, dtype=np.int32), np.asarray(plan.swap_in, dtype=np.int32), \
            np.asarray(plan.copies, dtype=np.int32)
        if not (pre.size or so.size or si.size or cp.size):
            return
        cache = self.model.kv_cache
        flat = cache.view(cache.shape[0], -1)
        if (so.size or si.size) and self.host_cache is None:
            raise RuntimeError("swap requested without a host block pool")
        pre3, cp3 = pre.reshape(-1, 3), cp.reshape(-1, 3)
        if self.cuda:
            pre2 = np.ascontiguousarray(pre3[:, :2]).reshape(-1)
            cp2 = np.ascontiguousarray(cp3[:, :2]).reshape(-1)
            dev = self._stage(np.concatenate([pre2, so.reshape(-1), si.reshape(-1), cp2]))
            o = pre2.size
            if pre2.size:
                native.copy_blocks(cache, dev[:o], self.block_bytes)
            if so.size or si.size:
                if self._swap_stream is None:
                    self._swap_stream = torch.cuda.Stream(device=self.device)
                main = torch.cuda.current_stream()
                self._swap_stream.wait_stream(main)
                with torch.cuda.stream(self._swap_stream):
                    if so.size:
                        native.swap_blocks(cache, self.host_cache, dev[o:o + so.size], self.block_bytes, to_host=True)
                    if si.size:
                        native.swap_blocks(cache, self.host_cache, dev[o + so.size:o + so.size + si.size],
                                           self.block_bytes, to_host=False)
                dev.record_stream(self._swap_stream)
                main.wait_stream(self._swap_stream)
            if cp2.size:
                native.copy_blocks(cache, dev[o + so.size + si.size:], self.block_bytes)
        else:
            raw = flat.view(torch.uint8) if flat.dtype != torch.uint8 else flat
            for sblk, dblk, _ in pre3:
                flat[int(dblk)].copy_(flat[int(sblk)])
            if so.size:
                p2 = so.reshape(-1, 2).astype(np.int64)
                self.host_cache[torch.from_numpy(p2[:, 1])] = raw[torch.from_numpy(p2[:, 0])]
            if si.size:
                p2 = si.reshape(-1, 2).astype(np.int64)
                raw[torch.from_numpy(p2[:, 0])] = self.host_cache[torch.from_numpy(p2[:, 1])]
            for sblk, dblk, _ in cp3:
                flat[int(dblk)].copy_(flat[int(sblk)])
        for t3 in (pre3, cp3):
            if t3.size and (t3[:, 2] != 0).any():
                self.model.rerotate_blocks(t3)

    def _stage_plan(self, plan) -> torch.Tensor:
        """The step's device metadata (ids, positions, slots, sequence offsets, lengths, block table, sample rows) in
        one upload. A scheduler plan writes its image straight into the pinned staging buffer."""
        if self.cuda and hasattr(plan, "write_step_image"):
            n = int(plan.step_image_words())
            slot = self._stage_buffer(n)
            plan.write_step_image(slot[0].data_ptr(), slot[1])
            self.h2d_bytes += n * 4
            dev = slot[0][:n].to(self.device, non_blocking=True)
            slot[2].record()
            return dev
        parts = [plan.input_ids, plan.positions, plan.slots, plan.cu_q, plan.kv_lens, plan.block_table, plan.sample_rows]
        return self._stage(np.concatenate([np.asarray(p, dtype=np.int32).reshape(-1) for p in parts]))

    def _patch_ids(self, ids: torch.Tensor, patch) -> None:
        """Pipelined steps: rows whose input token the host does not know yet (sampled by the step still in flight)
        take it from that step's sampler output on the device. ``patch`` = (rows, src, previous tokens)."""
        rows, src, prev = patch
        if rows.size == 0:
            return
        if self.cuda:
            idx = self._stage(np.concatenate([rows, src]).astype(np.int32))
            native.patch_ids(ids, idx[:rows.size], idx[rows.size:], prev)
        else:
            ids[torch.from_numpy(rows.astype(np.int64))] = prev[torch.from_numpy(src.astype(np.int64))].to(ids.dtype)

    def build_step(self, plan, extra: Optional[dict] = None, patch=None) -> StepInput:
        T, nseq = plan.num_tokens, len(plan.seq_ids)
        nsamp = plan.sample_rows.size
        dev = self._stage_plan(plan)
        if patch is not None:
            self._patch_ids(dev[:T], patch)
        o = 0

        def take(n):
            nonlocal o
            v = dev[o:o + n]
            o += n
            return v

        input_ids, positions, slots = take(T), take(T), take(T)
        cu_q, kv_lens = take(nseq + 1), take(nseq)
        table = take(nseq * plan.max_blocks).view(nseq, plan.max_blocks)
        rows = take(nsamp)
        step = StepInput(input_ids, positions, slots, cu_q, kv_lens, table, plan.num_multi, plan.num_single, T,
                         plan.num_multi_tokens, plan.max_q_len, logits_rows=rows)
        kv_lens = np.asarray(plan.kv_lens)
        step.max_kv_len = int(kv_lens.max()) if nseq else 0
        step.sample_k = self.candidate_k(plan, extra)
        if plan.num_single:
            max_kv = int(kv_lens[plan.num_multi:].max())
            step.decode_splits = ops.decode_splits(plan.num_single, self.model.Hkv, max_kv)
        if extra:
            for k, v in extra.items():
                setattr(step, k, v)
        return step

    CANDIDATE_KS = (1, 8, 64)

    def candidate_k(self, plan, extra) -> int:
        """How many per-shard sampling candidates a tensor-parallel step exchanges instead of whole logits rows
        (0: whole rows). Needs the peer-memory path, a step whose sampling looks only at the largest logits (no
        penalties or bans, which edit whole rows) and nobody else reading the logits (request targets, hooks)."""
        model = self.model
        symm = getattr(getattr(model, "comm", None), "symm", None)
        if (not self.cuda or symm is None or getattr(model, "tp_size", 1) <= 1 or extra or self.pipeline is not None
                or not self.exchange_candidates or plan.sample_full or plan.sample_k <= 0):
            return 0
        for k in self.CANDIDATE_KS:
            if plan.sample_k <= k:
                return k
        return 0

    # ------------------------------------------------------------------ CUDA-graph decode
    GRAPH_SIZES = (1, 2, 4, 8, 16, 32, 64, 128, 256)

    def enable_graphs(self, max_batch: int, max_token_len: int):
        """Whole-model CUDA graphs for pure-decode steps, one per padded batch size (the reference captures
        per-layer graphs for batch sizes 1..3 only: src/ksana_llm/runtime/cuda_graph_runner.cpp:11-30)."""
        if not self.cuda or self.pipeline is not None or getattr(self.model, "dp", None) is not None:
            return
        self.graphs = {}
        self.graph_max_batch = max_batch
        self.graph_max_blocks = (max_token_len + self.block_tokens - 1) // self.block_tokens + 1
        self.graph_max_kv = max_token_len

    def release_graphs(self):
        """Drop the captured graphs (before tearing down process groups / the device context)."""
        if getattr(self, "graphs", None):
            self.graphs.clear()
            if self.cuda:
                torch.cuda.synchronize(self.device)

    def _graph_for(self, bs: int, kx: int = 0):
        g = self.graphs.get((bs, kx))
        if g is not None:
            return g
        mb = self.graph_max_blocks
        n = 4 * bs + bs * mb
        img = torch.zeros(n, dtype=torch.int32, device=self.device)
        ids, pos, slots, kvl = img[0:bs], img[bs:2 * bs], img[2 * bs:3 * bs], img[3 * bs:4 * bs]
        table = img[4 * bs:].view(bs, mb)
        slots.fill_(-1)
        cu_q = torch.arange(bs + 1, dtype=torch.int32, device=self.device)
        step = StepInput(ids, pos, slots, cu_q, kvl, table, 0, bs, bs, 0, 1, logits_rows=None)
        step.decode_splits = ops.decode_splits(bs, self.model.Hkv, self.graph_max_kv)
        step.max_kv_len = self.graph_max_kv
        step.sample_k = kx
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.model.forward(step)          # warm-up: lazy initialisations must not happen under capture
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = self.model.forward(step)
        # the captured kernels hold raw pointers to every tensor of `step` (cu_q is not part of `img`): keep the
        # step alive with the graph, or its memory is handed to later allocations and a replay reads garbage offsets
        g = (graph, img, logits, mb, step)
        self.graphs[(bs, kx)] = g
        return g

    def _try_graph(self, plan, patch=None) -> Optional[torch.Tensor]:
        nseq = len(plan.seq_ids)
        if getattr(self, "graphs", None) is None or plan.num_multi or nseq == 0 or nseq > self.graph_max_batch:
            return None
        if plan.sample_rows.size != nseq or plan.max_blocks > self.graph_max_blocks:
            return None
        bs = next(b for b in self.GRAPH_SIZES if b >= nseq)
        graph, img, logits, mb, _step = self._graph_for(bs, self.candidate_k(plan, None))
        n = 4 * bs + bs * mb
        if hasattr(plan, "write_decode_image"):
            slot = self._stage_buffer(n)                  # the plan writes the padded image into pinned memory itself
            plan.write_decode_image(slot[0].data_ptr(), slot[1], bs, mb)
            self.h2d_bytes += n * 4
            img.copy_(slot[0][:n], non_blocking=True)
            slot[2].record()
        else:
            host = np.zeros(n, dtype=np.int32)
            host[0:nseq] = plan.input_ids
            host[bs:bs + nseq] = plan.positions
            host[2 * bs:3 * bs] = -1
            host[2 * bs:2 * bs + nseq] = plan.slots
            host[3 * bs:3 * bs + nseq] = plan.kv_lens
            tbl = host[4 * bs:].reshape(bs, mb)
            tbl[:nseq, :plan.max_blocks] = np.asarray(plan.block_table).reshape(nseq, plan.max_blocks)
            self._stage(host, out=img)
        if patch is not None:
            self._patch_ids(img[:bs], patch)
        graph.replay()
        self.graph_replays = getattr(self, "graph_replays", 0) + 1
        if isinstance(logits, LogitCandidates):
            return LogitCandidates(logits.values[:nseq], logits.ids[:nseq])
        return logits[:nseq]

    @torch.inference_mode()
    def execute(self, plan, extra: Optional[dict] = None, patch=None) -> torch.Tensor:
        dp = getattr(self.model, "dp", None)
        if dp is not None:
            # attention data parallelism: this rank runs only its own sequences and only its own pool's swap / copy
            # entries (the plan names device blocks as rank * blocks_per_rank + block); rank 0 collects the logits rows
            sub = dp.sub_plan(plan)
            self.apply_block_ops(sub)
            if plan.empty():
                return None
            local = None
            if sub.num_tokens:
                local = self.model.forward(self.build_step(sub, None))
            else:
                self.model.forward_empty_dp()
            return dp.gather_logits(local, self.model.cfg.vocab_size, self.device)
        self.apply_block_ops(plan)
        if plan.empty():
            return None                      # a plan may carry block operations only (everything else was preempted)
        if extra is None:
            out = self._try_graph(plan, patch)
            if out is not None:
                return out
        step = self.build_step(plan, extra, patch)
        if _checks.enabled():
            _checks.check_step(step, self.model)
        if self.pipeline is not None:
            return self.pipeline.forward(step, plan)
        return self.model.forward(step)


class LLMEngine:
    def __init__(self, model, model_cfg: ModelConfig, cfg: EngineConfig, num_blocks: int, num_host_blocks: int = 0,
                 tokenizer=None, kv_dtype=None, rank: int = 0, world_size: int = 1, control_group=None, pipeline=None):
        self.model, self.model_cfg, self.cfg = model, model_cfg, cfg
        self.tokenizer = tokenizer
        self.rank, self.world_size, self.control_group = rank, world_size, control_group
        bs = cfg.batch_scheduler
        sc = ne.SchedulerConfig()
        for k in ("schedule_strategy", "waiting_timeout_in_ms", "max_waiting_queue_len", "max_step_tokens",
                  "max_batch_size", "swapout_block_threshold", "swapin_block_threshold", "launch_block_threshold",
                  "preempt_mode", "split_fuse_token_num", "min_flexible_cache_num"):
            setattr(sc, k, getattr(bs, k))
        sc.max_token_len = min(bs.max_token_len, model_cfg.max_token_len) if model_cfg.max_token_len else bs.max_token_len
        sc.enable_prefix_cache = bool(bs.enable_auto_prefix_cache)
        sc.block_token_num = cfg.block_manager.block_token_num
        sc.eos_token_ids = list(model_cfg.eos_token_ids)
        dp = getattr(model, "dp", None)
        if dp is not None and getattr(dp, "size", 1) > 1:
            sc.dp_size = int(dp.size)          # every data-parallel rank's cache only holds its own sequences
            dp.blocks_per_rank = int(num_blocks)
        self.sched_cfg = sc
        if num_blocks * sc.block_token_num < sc.max_token_len:
            raise ValueError(f"{num_blocks} KV blocks of {sc.block_token_num} tokens cannot hold max_token_len "
                             f"{sc.max_token_len}")
        self.scheduler = ne.Scheduler(sc, num_blocks, num_host_blocks) if rank == 0 else None
        self.runner = ModelRunner(model, sc.block_token_num, num_blocks, num_host_blocks, kv_dtype)
        self.runner.pipeline = pipeline
        if cfg.global_.enable_cuda_graph:
            self.runner.enable_graphs(bs.max_batch_size, sc.max_token_len)
        self.sampler = Sampler(model.device, model_cfg.vocab_size, stage=self.runner._stage)
        self.requests: Dict[int, Request] = {}
        self.seq_to_req: Dict[int, tuple] = {}
        self._next_req = 1
        self._lock = threading.Lock()
        self._wake = threading.Condition()
        self._native_loop = None
        self._exit_hook = False
        self._loop_bound = False
        self._thread: Optional[threading.Thread] = None
        self._stop = False
        self.steps = 0
        self.fsm_controller = ne.FsmController()
        self.step_hook: Optional[Callable] = None
        self.last_logits: Optional[torch.Tensor] = None
        self.fatal: Optional[str] = None          # set when the tensor-parallel group can no longer serve (see _device_fault)
        # pipelined stepping (see _step_pipelined): the step whose tokens the host has not read yet, and how many
        # active requests need synchronous steps
        self.pipelined = os.environ.get("KSANA_PIPELINED_STEPS", "1") != "0"
        self._flight: Optional[dict] = None
        self._nonplain = 0
        self.host_ms: Dict[str, float] = {}      # host wall time of the step loop by phase (milliseconds, summed)

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: List[int], sampling=None, stream: bool = False, structured_regex: str = "",
                    request_target: Optional[dict] = None, refit=None, mrope_positions=None, listener=None) -> Request:
        cfg = sampling or ne.SamplingConfig()
        cfg.verify_args()          # normalises in place (e.g. beams need as many log-probs as beams); errors resurface below
        with self._lock:
            req_id = self._next_req
            self._next_req += 1
        n = max(cfg.num_beams, cfg.num_return_sequences, 1)
        req = Request(req_id, prompt, cfg, n, stream, listener)
        req.request_target, req.refit, req.mrope_positions = request_target, refit, mrope_positions
        # plain = nothing needs the host between a step's sampling and the next forward (see _step_pipelined)
        req.plain = (n == 1 and cfg.num_beams == 1 and not cfg.stop_strings and not structured_regex and
                     cfg.repetition_penalty == 1.0 and cfg.no_repeat_ngram_size == 0 and
                     cfg.encoder_no_repeat_ngram_size == 0 and cfg.logprobs_num == 0 and not request_target and
                     refit is None and mrope_positions is None)
        if structured_regex:
            req.structured = StructuredOutput(self.fsm_controller.get_or_create(structured_regex), self.tokenizer)
        if cfg.seed == 0:
            cfg.seed = int.from_bytes(os.urandom(7), "little") | 1
        if self.fatal is not None:
            code, msg, seq_ids = 12, f"engine stopped after a device error: {self.fatal}", []
        elif getattr(self.model, "dp", None) is not None and (request_target or refit is not None or mrope_positions is not None):
            # attention data parallelism hands each rank the rows of its own sequences; per-row extras address the
            # rows of the whole step and are not re-indexed per rank
            code, msg, seq_ids = 1, "request targets and spliced embeddings are not supported with attention data parallelism", []
        else:
            code, msg, seq_ids = self.scheduler.add_request(req_id, list(prompt), cfg)
        ne.report_counter("forward_req_total_num", 1)
        if code != 0:
            req.status_code, req.status_message = code, msg
            for o in req.outputs:
                o.finished = True
            ne.report_counter("forward_req_error_num", 1)
            self._complete(req)
            return req
        req.seq_ids = list(seq_ids)
        with self._lock:
            self.requests[req_id] = req
            for i, sid in enumerate(seq_ids):
                self.seq_to_req[sid] = (req, i)
            if not req.plain:
                self._nonplain += 1
        if req.structured is not None:
            init = req.structured.initial_tokens()
            if init:
                req.outputs[0].tokens = list(init)
                self.scheduler.replace_generated(seq_ids[0], list(init))
        ne.report_counter("metric_input_tokens_num", len(prompt))
        self._notify_loop()
        return req

    def abort(self, req: Request):
        req.aborted = True
        self.scheduler.abort(req.req_id)
        self._notify_loop()

    def _complete(self, req: Request):
        req.finish_time = time.time()
        req.done.set()
        req.emit(None)
        if req.span_id:
            ne.span_end(req.span_id, {"code": str(req.status_code)})
        with self._lock:
            if self.requests.pop(req.req_id, None) is not None and not getattr(req, "plain", True):
                self._nonplain -= 1
            for sid in req.seq_ids:
                self.seq_to_req.pop(sid, None)

    # ------------------------------------------------------------------ one step
    def _handle_events(self, events, lp_by_seq=None):
        touched = set()
        for seq_id, req_id, index, token, finished, code, message in events:
            ent = self.seq_to_req.get(seq_id)
            if ent is None:
                continue
            req, i = ent
            out = req.outputs[i]
            if token >= 0 and not out.finished:
                out.tokens.append(int(token))
                if lp_by_seq is not None and seq_id in lp_by_seq:
                    out.logprobs.append(lp_by_seq[seq_id])
                if req.first_token_time is None:
                    req.first_token_time = time.time()
                    ne.report_metric("time_to_first_token_ms", (req.first_token_time - req.arrive) * 1000.0)
            if finished:
                out.finished = True
                if code == 0 and req.cfg.stop_strings and self.tokenizer is not None:
                    self._final_stop_check(out, req.cfg)
                if code != 0:
                    req.status_code, req.status_message = code, message
                    ne.report_counter({4: "forward_req_aborted_num", 7: "forward_req_timeout_num"}.get(code, "forward_req_error_num"), 1)
            touched.add(req.req_id)
            if not finished and token >= 0:
                self._post_token_hooks(req, i, seq_id)
        for rid in touched:
            req = self.requests.get(rid)
            if req is None:
                continue
            if req.stream:
                # queue followers get the tokens so far; a listener reads the request itself on its own thread
                req.emit(("step", [list(o.tokens) for o in req.outputs] if req.stream_queue is not None else None))
            if req.all_finished():
                n_out = sum(len(o.tokens) for o in req.outputs)
                ne.report_counter("metric_output_token_num", n_out)
                if req.first_token_time and n_out > 1:
                    ne.report_metric("time_to_per_output_token_ms",
                                     (time.time() - req.first_token_time) * 1000.0 / max(1, n_out - 1))
                ne.report_metric("forward_cost_time_ms", (time.time() - req.arrive) * 1000.0)
                self._complete(req)

    def _final_stop_check(self, out, cfg):
        """The last token of a sequence can complete a stop string too (and text held back as half a character is
        final now): one search over the whole text (src/ksana_llm/batch_scheduler/strategy/continuous_batching.cpp:32-55
        checks complete stop strings when a request finishes)."""
        checker = ne.StopChecker(list(cfg.stop_strings))
        if checker.append(self.tokenizer.decode(out.tokens, skip_special_tokens=True)) >= 0:
            out.tokens = list(self.tokenizer.encode(checker.kept(), add_special_tokens=False))

    def _post_token_hooks(self, req: Request, i: int, seq_id: int):
        """Stop strings and structured output act on decoded text, which needs the tokenizer."""
        out = req.outputs[i]
        cfg = req.cfg
        if cfg.stop_strings and self.tokenizer is not None:
            # incremental detokenisation: only the tokens since the last complete character are decoded again, and
            # the native checker searches only the tail that the new text can complete. Bytes that never complete a
            # character (they decode to U+FFFD whatever follows) break the increments: such an output falls back
            # to decoding and searching its whole text per token.
            st = getattr(out, "_stop_state", None)
            if st is None:
                st = out._stop_state = [ne.StopChecker(list(cfg.stop_strings)), 0, 0, False]   # checker, prefix, read, whole
            checker, prefix, read, whole = st
            hit = -1
            if not whole:
                before = self.tokenizer.decode(out.tokens[prefix:read], skip_special_tokens=True) if read > prefix else ""
                now = self.tokenizer.decode(out.tokens[prefix:], skip_special_tokens=True)
                if not ne.StopChecker.ends_incomplete(now):
                    if now.startswith(before):
                        st[1], st[2] = read, len(out.tokens)
                        hit = checker.append(now[len(before):])
                    else:
                        whole = st[3] = True
                elif len(out.tokens) - read >= 4 or len(out.tokens) >= cfg.max_new_tokens:
                    whole = st[3] = True
            if whole:
                checker.reset()
                hit = checker.append(self.tokenizer.decode(out.tokens, skip_special_tokens=True))
            if hit >= 0:
                kept = self.tokenizer.encode(checker.kept(), add_special_tokens=False)
                out.tokens = list(kept)
                self.scheduler.finish_sequence(seq_id, -1, 0, "")
                out.finished = True
                return
        if req.structured is not None:
            action = req.structured.after_token(out.tokens)
            if action.final:
                out.tokens = action.tokens
                self.scheduler.finish_sequence(seq_id, -1, 0, "")
                out.finished = True
            elif action.changed:
                out.tokens = action.tokens
                self.scheduler.replace_generated(seq_id, action.tokens)

    def _gather_extras(self, plan) -> Optional[dict]:
        """Per-step optional inputs, as host tensors: plugin embeddings to splice in, multimodal rotary positions,
        and for /forward targets the flag that keeps the hidden states plus the row ranges [first row, rows] whose
        logits are computed for every position after the forward (a collective under tensor parallelism, so the
        worker ranks get the same list and run it too)."""
        extra = {}
        refit_pos, refit_emb, want_hidden, full_logits = [], [], False, []
        mrope = None
        row0 = 0
        for k, sid in enumerate(plan.seq_ids.tolist()):
            ent = self.seq_to_req.get(sid)
            ql = int(plan.q_lens[k])
            if ent is not None:
                req, _ = ent
                start = int(plan.kv_lens[k]) - ql
                if req.refit is not None:
                    for pos, emb in zip(*req.refit):
                        n = emb.shape[0] if emb.dim() > 1 else 1
                        e2 = emb.reshape(n, -1)
                        for j in range(n):
                            p = int(pos) + j
                            if start <= p < start + ql:
                                refit_pos.append(row0 + p - start)
                                refit_emb.append(e2[j])
                if req.mrope_positions is not None:
                    if mrope is None:
                        mrope = torch.zeros(3, plan.num_tokens, dtype=torch.int32)
                        mrope[:] = torch.from_numpy(np.asarray(plan.positions)).to(torch.int32)
                    mp = torch.as_tensor(req.mrope_positions, dtype=torch.int32)
                    end = min(start + ql, mp.shape[1])
                    if end > start:
                        mrope[:, row0:row0 + end - start] = mp[:, start:end]
                    if start + ql > mp.shape[1]:     # generated tokens continue from the last multimodal position
                        base = int(mp.max()) + 1 - mp.shape[1]
                        s2 = max(start, mp.shape[1])
                        mrope[:, row0 + s2 - start:row0 + ql] = torch.arange(s2, start + ql, dtype=torch.int32) + base
                if req.request_target and not req.targets_done:
                    want_hidden = True
                    if "logits" in req.request_target:
                        full_logits.append([row0, ql])
            row0 += ql
        if refit_pos:
            extra["refit_positions"] = torch.tensor(refit_pos, dtype=torch.int32)
            extra["refit_embeddings"] = torch.stack(refit_emb).float().cpu()
        if mrope is not None:
            extra["mrope_positions"] = mrope
        if want_hidden:
            extra["want_hidden"] = True
        if full_logits:
            extra["full_logits"] = full_logits
        return extra or None

    def run_with_extras(self, plan, extra: Optional[dict], patch=None):
        """The forward of one step with its optional inputs moved to the device; returns (logits, the all-position
        logits of the ``full_logits`` row ranges in order). Every rank of the engine calls this with the same plan
        and extras, so the collectives inside line up."""
        step_extra = None
        if extra:
            dev = self.model.device
            step_extra = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in extra.items() if k != "full_logits"}
        logits = self.runner.execute(plan, step_extra or None, patch)
        ranges = (extra or {}).get("full_logits", [])
        pipe = self.runner.pipeline
        if pipe is not None and extra and extra.get("want_hidden"):
            return logits, pipe.collect_targets(ranges)       # the states live on the last stage
        full = [self.model.compute_logits(self.model.step_normed[r0:r0 + n]) for r0, n in ranges]
        return logits, full

    # ------------------------------------------------------------------ pipelined stepping
    # The host work between two steps (read the tokens, post-process, schedule, pack, broadcast, launch) is off the
    # device's critical path whenever the running requests are plain: the next step is planned and launched while the
    # device still runs the current one. The scheduler gives every sampling sequence a placeholder token
    # (Scheduler::Advance), the next step's decode rows take their input ids from the sampler's device buffer, and the
    # tokens are read and post-processed (Scheduler::Resolve) while that next step executes. Counterpart of the
    # reference's separate scheduling / execution threads (src/ksana_llm/batch_manager/batch_manager.cpp:111-241) with
    # one thread and one step of look-ahead. Anything that needs the host between sampling and the next forward
    # (beams, parallel sampling forks, stop strings, structured output, penalties, log-probs, request targets, hooks)
    # drains the pipeline and steps synchronously.
    AUX_MAGIC = 0x4B535058

    def _pipelining_possible(self) -> bool:
        return (self.pipelined and self.runner.pipeline is None and getattr(self.model, "dp", None) is None
                and self.step_hook is None and self._nonplain == 0)

    def _resolve_flight(self) -> None:
        """Second half of a pipelined step: its tokens reach the host, the scheduler puts them in place of the
        placeholders and the requests hear about them."""
        fl, self._flight = self._flight, None
        if fl is None:
            return
        t0 = time.perf_counter()
        try:
            tokens = self.sampler.finish_plain(fl["handle"])
        except DeviceStepError as e:
            self._device_fault(e)
            return
        t1 = time.perf_counter()
        events = self.scheduler.resolve(fl["plan"], tokens)
        self._handle_events(events, None)
        self.steps += 1
        tm = self.host_ms
        tm["sample_and_wait"] = tm.get("sample_and_wait", 0.0) + (t1 - t0) * 1000.0
        tm["post_step"] = tm.get("post_step", 0.0) + (time.perf_counter() - t1) * 1000.0
        tm["steps"] = tm.get("steps", 0) + 1

    def _plain_params(self, plan, pending: set):
        params = []
        for sid in plan.sample_seq_ids.tolist():
            ent = self.seq_to_req.get(sid)
            req, i = ent if ent else (None, 0)
            sp = SamplingParams.from_request(req, i)
            if sid in pending:
                sp.step += 1                 # its previous token is still on the device: not in the request's list yet
            params.append(sp)
        return params

    def _patch_for(self, plan, fl):
        """(rows, src, previous tokens) for the rows of ``plan`` whose input id is a placeholder, or None."""
        ids = np.asarray(plan.input_ids)
        rows = np.nonzero(ids < 0)[0].astype(np.int32)
        if rows.size == 0:
            return None
        if fl is None:
            raise RuntimeError("a step plan carries placeholder tokens but no step is in flight")
        where = {sid: k for k, sid in enumerate(fl["plan"].sample_seq_ids.tolist())}
        cu = np.asarray(plan.cu_q)
        seq_of_row = np.searchsorted(cu, rows, side="right") - 1
        seq_ids = np.asarray(plan.seq_ids)
        src = np.array([where[int(seq_ids[k])] for k in seq_of_row], dtype=np.int32)
        return rows, src, fl["handle"]["tokens_dev"]

    def _step_pipelined(self) -> bool:
        tm = self.host_ms
        t0 = time.perf_counter()
        fl = self._flight
        with nvtx.annotate("schedule"):
            plan = self.scheduler.schedule()
        t1 = time.perf_counter()
        if plan.events:
            self._handle_events(plan.events)
        if plan.empty():
            if plan.has_block_ops():
                if self.world_size > 1:
                    self._broadcast_plan(plan, None)
                self.runner.execute(plan, None)
            if fl is not None:
                self._resolve_flight()
                return True
            return plan.has_block_ops()
        extra = self._gather_extras(plan)
        plain = (not extra and self.scheduler.can_pipeline(plan) and self._pipelining_possible())
        patch = self._patch_for(plan, fl)
        image = None
        if plain:
            pending = set(fl["plan"].sample_seq_ids.tolist()) if fl is not None else set()
            image = Sampler.params_image(self._plain_params(plan, pending))
        t2 = time.perf_counter()
        if self.world_size > 1:
            self._broadcast_plan(plan, extra, self._pack_aux(patch, image))
        t3 = time.perf_counter()
        phase = "Prefill" if plan.num_multi else "Decode"
        with nvtx.annotate(phase):
            logits, self._step_full_logits = self.run_with_extras(plan, extra, patch)
        self.last_logits = logits
        nsamp = int(plan.sample_rows.size)
        if plain:
            handle = self.sampler.launch_plain(logits, image, nsamp) if nsamp else {"tokens_dev": None, "B": 0, "code": 0}
            t4 = time.perf_counter()
            if fl is not None:
                self._resolve_flight()                   # overlaps with the step just launched
            if self.fatal is None:
                self.scheduler.advance(plan)
                self._flight = {"plan": plan, "handle": handle, "phase": phase}
            for k, v in (("schedule", t1 - t0), ("extras", t2 - t1), ("broadcast", t3 - t2), ("launch", t4 - t3)):
                tm[k] = tm.get(k, 0.0) + v * 1000.0
            # most of this iteration was spent waiting for the step launched by the previous one
            self._phase_wall(fl["phase"] if fl is not None else phase, t0)
            return True
        # a step that needs the host between sampling and the next forward: finish what is in flight, then the
        # synchronous second half
        t4 = time.perf_counter()
        if fl is not None:
            self._resolve_flight()
            if self.fatal is not None:
                return True
        try:
            tokens, parents, lp_by_seq = self._sample(plan, logits)
        except DeviceStepError as e:
            self._device_fault(e)
            return True
        t5 = time.perf_counter()
        self._extract_targets(plan, logits)
        events = self.scheduler.post_step(plan, tokens, parents)
        t6 = time.perf_counter()
        self._handle_events(events, lp_by_seq)
        self.steps += 1
        if self.step_hook:
            self.step_hook(plan, logits)
        for k, v in (("schedule", t1 - t0), ("extras", t2 - t1), ("broadcast", t3 - t2), ("launch", t4 - t3),
                     ("sample_and_wait", t5 - t4), ("post_step", t6 - t5), ("events", time.perf_counter() - t6)):
            tm[k] = tm.get(k, 0.0) + v * 1000.0
        tm["steps"] = tm.get("steps", 0) + 1
        self._phase_wall(phase, t0)
        return True

    def _phase_wall(self, phase: str, t0: float):
        """Wall time of one loop iteration, booked to the phase (Prefill / Decode) it mostly served."""
        tm = self.host_ms
        tm[phase + "_wall"] = tm.get(phase + "_wall", 0.0) + (time.perf_counter() - t0) * 1000.0
        tm[phase + "_n"] = tm.get(phase + "_n", 0) + 1

    def _pack_aux(self, patch, image) -> Optional[np.ndarray]:
        """What the worker ranks need beside the plan in a pipelined step: the rows to patch from their own copy of
        the previous step's tokens, and the sampler's parameters (they run the same sampler on the same logits, so
        every rank holds the tokens the next step reads). Layout: magic, n_patch, n_sample_words, rows, src, image."""
        if patch is None and image is None:
            return None
        rows, src = (patch[0], patch[1]) if patch is not None else (np.zeros(0, np.int32), np.zeros(0, np.int32))
        img = image if image is not None else np.zeros(0, np.int32)
        return np.concatenate([np.array([self.AUX_MAGIC, rows.size, img.size], dtype=np.int32), rows, src, img])

    def follow_step(self, plan, extra: Optional[dict], aux: Optional[np.ndarray]):
        """Worker ranks: one broadcast step. Pipelined steps also sample (no read-back) so that the next step can take
        its input ids from this rank's own device buffer."""
        patch, image = None, None
        if aux is not None and aux.size >= 3 and int(aux[0]) == self.AUX_MAGIC:
            n_patch, n_img = int(aux[1]), int(aux[2])
            if n_patch:
                prev = self._flight["handle"]["tokens_dev"] if self._flight else None
                if prev is None:
                    raise RuntimeError("worker rank: a pipelined step refers to tokens this rank never sampled")
                patch = (aux[3:3 + n_patch].copy(), aux[3 + n_patch:3 + 2 * n_patch].copy(), prev)
            if n_img:
                image = aux[3 + 2 * n_patch:3 + 2 * n_patch + n_img].copy()
        out = self.run_with_extras(plan, extra, patch)
        if image is not None:
            nsamp = int(plan.sample_rows.size)
            self._flight = {"plan": None, "handle": self.sampler.launch_plain(out[0], image, nsamp, read_back=False)
                            if nsamp else {"tokens_dev": None, "B": 0}}
        else:
            self._flight = None
        return out

    def step(self) -> bool:
        """Runs one engine step. Returns False when there was nothing to run."""
        if self._flight is not None or self._pipelining_possible():
            if self._flight is not None and not self._pipelining_possible():
                self._resolve_flight()       # something that needs synchronous steps arrived: drain first
            else:
                return self._step_pipelined()
        tm = self.host_ms
        t0 = time.perf_counter()
        with nvtx.annotate("schedule"):
            plan = self.scheduler.schedule()
        t1 = time.perf_counter()
        ne.report_metric("batch_manager_schedule_ms", (t1 - t0) * 1000.0)
        if plan.events:
            self._handle_events(plan.events)
        if plan.empty():
            if plan.has_block_ops():         # copies / swaps decided without a forward to run: execute them alone
                if self.world_size > 1:
                    self._broadcast_plan(plan, None)
                self.runner.execute(plan, None)
                return True
            return False
        ne.trace_record("SchedBegin", "i", 0, float(plan.num_tokens))
        ne.report_metric("batch_scheduler_batch_size", float(len(plan.seq_ids)))
        ne.report_metric("token_num_in_batch", float(plan.num_tokens))
        extra = self._gather_extras(plan)
        if self.step_hook is not None:
            plan.sample_full = True          # a hook reads whole logits rows: every rank gathers them (the flag travels with the plan)
        t2 = time.perf_counter()
        if self.world_size > 1:
            self._broadcast_plan(plan, extra)
        t3 = time.perf_counter()
        phase = "Prefill" if plan.num_multi else "Decode"
        ne.trace_record(phase, "B", 0, float(plan.num_tokens))
        with nvtx.annotate(phase):
            logits, self._step_full_logits = self.run_with_extras(plan, extra)
        t4 = time.perf_counter()
        self.last_logits = logits
        try:
            with nvtx.annotate("sample"):
                tokens, parents, lp_by_seq = self._sample(plan, logits)
        except DeviceStepError as e:
            self._device_fault(e)
            return True
        t5 = time.perf_counter()
        ne.trace_record(phase, "E", 0, float(plan.num_tokens))
        self._extract_targets(plan, logits)
        events = self.scheduler.post_step(plan, tokens, parents)
        t6 = time.perf_counter()
        self._handle_events(events, lp_by_seq)
        self.steps += 1
        if self.step_hook:
            self.step_hook(plan, logits)
        t7 = time.perf_counter()
        for k, v in (("schedule", t1 - t0), ("extras", t2 - t1), ("broadcast", t3 - t2), ("launch", t4 - t3),
                     ("sample_and_wait", t5 - t4), ("post_step", t6 - t5), ("events", t7 - t6)):
            tm[k] = tm.get(k, 0.0) + v * 1000.0
        tm["steps"] = tm.get("steps", 0) + 1
        self._phase_wall(phase, t0)
        return True

    def _sample(self, plan, logits):
        sample_seq_ids = plan.sample_seq_ids.tolist()
        nsamp = len(sample_seq_ids)
        if nsamp == 0:
            return [], [], {}
        # logits rows: one per plan.sample_rows entry (siblings repeat their leader's row)
        params, reqs = [], []
        for sid in sample_seq_ids:
            ent = self.seq_to_req.get(sid)
            req, i = ent if ent else (None, 0)
            reqs.append((req, i))
            params.append(SamplingParams.from_request(req, i))
        return self.sampler.sample(logits, params, reqs, sample_seq_ids)

    def _extract_targets(self, plan, logits):
        """/forward request targets: copies of the requested slices (see serving.forward_api)."""
        from ..serving.forward_api import extract_targets
        extract_targets(self, plan, logits)

    def full_logits_for(self, req, row0: int, ql: int) -> torch.Tensor:
        """Logits of every position of one sequence of the current step (perplexity-style targets): computed right
        after the forward, in plan order, by ``run_with_extras``."""
        return self._step_full_logits.pop(0)

    def _broadcast_plan(self, plan, extra: Optional[dict] = None, aux: Optional[np.ndarray] = None):
        """The plan image for the worker ranks; ``aux`` (pipelined steps) rides behind it in the same message, followed
        by its length, and a plan without one ends with a zero."""
        from ..parallel.control import broadcast_plan, pack_extras
        img = plan.pack()
        tail = np.concatenate([aux, [aux.size]]).astype(np.int32) if aux is not None else np.zeros(1, dtype=np.int32)
        broadcast_plan(self.control_group, np.concatenate([img, tail]), extras=pack_extras(extra))

    # ------------------------------------------------------------------ loop
    def start(self):
        """Starts the step loop: a native thread (``BatchLoop``: sleeps on a condition variable while idle, woken by
        ``add_request`` / ``abort``), or a Python thread with ``KSANA_NATIVE_LOOP=0``."""
        if self._thread is not None or self._native_loop is not None:
            return
        self._stop = False
        if os.environ.get("KSANA_NATIVE_LOOP", "1") != "0" and hasattr(ne, "BatchLoop"):
            self._native_loop = ne.BatchLoop()
            self._native_loop.start(self._loop_step, self._loop_idle, self._loop_error)
            if not self._exit_hook:
                # a native thread must not ask for the interpreter lock while the interpreter shuts down: a process
                # that ends without stop() joins the loop first
                import atexit
                import weakref
                ref = weakref.ref(self)
                atexit.register(lambda: ref() is not None and ref().stop())
                self._exit_hook = True
            return
        self._thread = threading.Thread(target=self._loop, name="ksana-engine", daemon=True)
        self._thread.start()

    def _loop_step(self) -> bool:
        if self._stop:
            return False
        self._bind_loop_thread()
        return bool(self.step())

    def _bind_loop_thread(self):
        """The current CUDA device is a per-thread setting: the loop thread adopts the model's device once."""
        if not self._loop_bound:
            self._loop_bound = True
            dev = getattr(self.runner, "device", None)
            if dev is not None and torch.device(dev).type == "cuda":
                torch.cuda.set_device(dev)

    def _loop_idle(self) -> bool:
        return bool(self.scheduler.idle()) and not self._stop

    def _loop_error(self, message: str):
        logger.error(f"engine step failed: {message}")
        self._fail_all(12, f"engine step failed: {message}")

    def _notify_loop(self):
        with self._wake:
            self._wake.notify_all()
        if self._native_loop is not None:
            self._native_loop.notify()

    def _loop(self):
        while not self._stop:
            try:
                self._bind_loop_thread()
                ran = self.step()
            except Exception as e:  # noqa: BLE001 - the loop must survive and fail the affected requests
                import traceback
                traceback.print_exc()
                logger.error(f"engine step failed: {e!r}")
                self._fail_all(12, f"engine step failed: {e}")
                ran = False
            if not ran:
                with self._wake:
                    if self.scheduler.idle() and not self._stop:
                        self._wake.wait(timeout=0.05)
                    else:
                        self._wake.wait(timeout=0.001)

    def _device_fault(self, err: DeviceStepError):
        """A kernel of the step reported through the device error word (read back with the sampled tokens): the
        step's logits are not trustworthy, so every request in flight ends with RET_RUNTIME instead of sampled
        garbage (the reference turns a failed forward into an error status for the batch the same way:
        src/ksana_llm/runtime/llm_runtime.cpp:387-445). With several ranks a wait on a peer that ran out leaves the
        ranks' collective epochs out of step, so the engine also refuses new requests and releases the workers."""
        ne.report_counter("forward_req_error_num", len(self.requests))
        logger.error(f"device error during an engine step ({len(self.requests)} requests in flight): {err}")
        self._fail_all(12, f"device error during the step: {err}")
        if self.world_size > 1 or err.code == 3:
            self.fatal = str(err)
            if self.world_size > 1:
                from ..parallel.control import broadcast_plan
                try:
                    broadcast_plan(self.control_group, None)
                except Exception:  # noqa: BLE001 - the workers may be gone already
                    pass

    def on_service_stop(self, reason: str):
        """Stop hook of the service lifetime (parallel.coordinator): a peer rank is gone, so no step can complete any
        more. Every request in flight is answered with RET_RUNTIME and new ones are refused."""
        self.fatal = reason
        self._stop = True
        if self.scheduler is not None:
            self._fail_all(12, f"service stopped: {reason}")

    def _fail_all(self, code: int, message: str):
        for req in list(self.requests.values()):
            req.status_code, req.status_message = code, message
            self.scheduler.abort(req.req_id)
            for o in req.outputs:
                o.finished = True
            self._complete(req)

    def stop(self):
        self._stop = True
        self._notify_loop()
        if self._native_loop is not None:
            self._native_loop.stop()
            self._native_loop = None
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None

    # ------------------------------------------------------------------ conveniences
    def generate(self, prompts: List[List[int]], sampling=None, timeout: Optional[float] = None) -> List[Request]:
        """Offline batch generation: steps on the calling thread, or waits for the background loop where one runs."""
        reqs = [self.add_request(p, _clone_cfg(sampling)) for p in prompts]
        if self._thread is None and self._native_loop is None:
            deadline = time.time() + timeout if timeout else None
            while not all(r.done.is_set() for r in reqs):
                if not self.step() and self.scheduler.idle():
                    break
                if deadline and time.time() > deadline:
                    break
            if self._flight is not None:          # a last step of rows that turned out to be finished: collect it
                self._resolve_flight()
        else:
            for r in reqs:
                r.done.wait(timeout)
        return reqs


def _clone_cfg(cfg):
    if cfg is None:
        return None
    c = ne.SamplingConfig()
    for k in ("topk", "num_beams", "num_return_sequences", "topp", "temperature", "repetition_penalty",
              "length_penalty", "no_repeat_ngram_size", "encoder_no_repeat_ngram_size", "max_new_tokens",
              "logprobs_num", "stop_token_ids", "stop_strings", "ignore_eos", "seed"):
        setattr(c, k, getattr(cfg, k))
    return c
