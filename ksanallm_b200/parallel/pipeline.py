"""Pipeline parallelism: contiguous layer ranges per stage, hidden states handed from stage to stage with
point-to-point sends (NCCL on GPUs, gloo on CPU), several micro-batches in flight.

The reference pipelines only across nodes: layer ranges per node (src/ksana_llm/distributed/control_channel.cpp:510-580),
hidden states copied device -> pinned host -> TCP -> pinned host -> device (src/ksana_llm/distributed/data_channel.cpp:148-176),
one batch in flight (src/ksana_llm/batch_manager/batch_manager.cpp:111-277), the master running embedding, lm_head and
sampling. Here a stage is a group of ``tp`` ranks anywhere in the job, the hand-off is ``isend`` / ``irecv`` between the
ranks with the same tensor-parallel index of neighbouring stages (device to device, no host staging), and a step's
sequences are cut into micro-batches so that stage ``s`` works on micro-batch ``m+1`` while its output for ``m``
is on the wire and stage ``s+1`` works on ``m``. The last stage computes the logits of all micro-batches in one
lm_head call and sends them to rank 0, which samples.

Rank layout: ``rank = pp_rank * tp + tp_rank``; rank 0 is (stage 0, tp 0) and owns the scheduler and the sampler.
"""
from __future__ import annotations

from dataclasses import replace
from typing import List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..models.common import StepInput


def stage_layers(num_layers: int, pp_size: int, pp_rank: int) -> Tuple[int, int]:
    """Inclusive layer range of a stage: quotient layers each, the first ``remainder`` stages one more."""
    q, r = divmod(num_layers, pp_size)
    lo = pp_rank * q + min(pp_rank, r)
    n = q + (1 if pp_rank < r else 0)
    if n <= 0:
        raise ValueError(f"{num_layers} layers cannot be split over {pp_size} pipeline stages")
    return lo, lo + n - 1


def split_sequences(q_lens: np.ndarray, parts: int) -> List[Tuple[int, int]]:
    """Cuts sequences [0, n) into at most ``parts`` contiguous ranges of roughly equal token counts."""
    n = int(len(q_lens))
    if n == 0:
        return []
    parts = max(1, min(parts, n))
    total = int(q_lens.sum())
    cuts, acc, k = [0], 0, 1
    for i in range(n):
        acc += int(q_lens[i])
        if k < parts and acc * parts >= total * k and i + 1 < n:
            cuts.append(i + 1)
            k += 1
    cuts.append(n)
    return [(a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]


def micro_step(step: StepInput, cu_host: np.ndarray, a: int, b: int, kv_host: Optional[np.ndarray] = None) -> StepInput:
    """The sub-step of sequences [a, b): views of the step's device tensors, offsets rebased (one tiny device op)."""
    t0, t1 = int(cu_host[a]), int(cu_host[b])
    nm = min(max(step.num_multi - a, 0), b - a)
    nm_tok = int(cu_host[a + nm]) - t0
    q_lens = np.diff(cu_host[a:b + 1])
    sub = replace(step,
                  input_ids=step.input_ids[t0:t1], positions=step.positions[t0:t1], slots=step.slots[t0:t1],
                  cu_q=step.cu_q[a:b + 1] - t0, kv_lens=step.kv_lens[a:b], block_table=step.block_table[a:b],
                  num_multi=nm, num_single=(b - a) - nm, num_tokens=t1 - t0, num_multi_tokens=nm_tok,
                  max_q_len=int(q_lens.max()) if len(q_lens) else 0, logits_rows=None, want_hidden=False,
                  refit_positions=None, refit_embeddings=None, decode_workspace=None)
    if step.mrope_positions is not None:
        sub.mrope_positions = step.mrope_positions[:, t0:t1]
    if kv_host is not None and b > a:
        sub.max_kv_len = int(kv_host[a:b].max())
    return sub


class PipelineRunner:
    """Executes one engine step on this rank's stage."""

    def __init__(self, model, pp_rank: int, pp_size: int, tp_rank: int, tp_size: int, group=None, micro_batches: int = 2):
        self.model = model
        self.pp_rank, self.pp_size, self.tp_rank, self.tp_size = pp_rank, pp_size, tp_rank, tp_size
        self.group = group
        self.micro_batches = max(1, micro_batches)
        self.first, self.last = pp_rank == 0, pp_rank == pp_size - 1
        self.prev = (pp_rank - 1) * tp_size + tp_rank
        self.next = (pp_rank + 1) * tp_size + tp_rank
        self.logits_src = (pp_size - 1) * tp_size           # (last stage, tp 0) sends the logits to rank 0
        self.sent_bytes = 0

    def forward(self, step: StepInput, plan) -> Optional[torch.Tensor]:
        """Returns the fp32 logits on rank 0 (and on the last stage), None elsewhere."""
        model = self.model
        cu = np.asarray(plan.cu_q, dtype=np.int64)
        kvh = np.asarray(plan.kv_lens, dtype=np.int64)
        q_lens = np.diff(cu)
        if step.refit_positions is not None and step.refit_positions.numel() > 0:
            ranges = [(0, len(q_lens))]                      # row indices of plugin embeddings refer to the whole step
        else:
            ranges = split_sequences(q_lens, self.micro_batches)
        H = model.cfg.hidden_size
        dev, dt = model.device, model.dtype
        recv_bufs, recv_reqs = [], []
        if not self.first:
            for a, b in ranges:
                buf = torch.empty(int(cu[b] - cu[a]), H, dtype=dt, device=dev)
                recv_bufs.append(buf)
                recv_reqs.append(dist.irecv(buf, src=self.prev, group=self.group))
        sends, outs = [], []
        for i, (a, b) in enumerate(ranges):
            whole = len(ranges) == 1
            sub = step if whole else micro_step(step, cu, a, b, kvh)
            h_in = None
            if not self.first:
                recv_reqs[i].wait()
                h_in = recv_bufs[i]
            h = model.forward_layers(sub, h_in)
            if self.last:
                outs.append(h)
            else:
                h = h.contiguous()
                sends.append((dist.isend(h, dst=self.next, group=self.group), h))
                self.sent_bytes += h.numel() * h.element_size()
        logits = None
        if self.last:
            h_all = outs[0] if len(outs) == 1 else torch.cat(outs, 0)
            logits = model.lm_head_forward(h_all, step)
            if self.pp_size > 1 and self.tp_rank == 0:
                logits = logits.contiguous()
                dist.send(logits, dst=0, group=self.group)
        for req, _keep in sends:
            req.wait()
        if self.first and self.pp_size > 1 and self.tp_rank == 0:
            rows = int(step.logits_rows.numel()) if step.logits_rows is not None else int(cu[-1])
            logits = torch.empty(rows, model.cfg.vocab_size, dtype=torch.float32, device=dev)
            dist.recv(logits, src=self.logits_src, group=self.group)
        return logits

    def collect_targets(self, full_ranges) -> list:
        """Collective over the engine's ranks after a step that kept its hidden states (request targets). Only the
        last stage has the final hidden states, the final norm and the lm_head, while rank 0 answers the requests:
        the last stage computes the all-position logits of the row ranges ``full_ranges`` ([first row, rows] each)
        and its tensor-parallel rank 0 sends hidden states, normed states and those logits to rank 0, which keeps
        the states on its model object and returns the logits list (other ranks return [])."""
        model = self.model
        if self.pp_size == 1:
            return [model.compute_logits(model.step_normed[r0:r0 + n]) for r0, n in full_ranges]
        full = []
        if self.last:
            full = [model.compute_logits(model.step_normed[r0:r0 + n]).contiguous() for r0, n in full_ranges]
            if self.tp_rank == 0:
                shape = torch.tensor(list(model.step_hidden.shape), dtype=torch.int64, device=model.step_hidden.device)
                dist.send(shape, dst=0, group=self.group)
                for t in (model.step_hidden, model.step_normed):
                    dist.send(t.contiguous(), dst=0, group=self.group)
                for t in full:
                    dist.send(t, dst=0, group=self.group)
        if self.first and self.tp_rank == 0:
            dev = model.device
            shape = torch.zeros(2, dtype=torch.int64, device=dev)
            dist.recv(shape, src=self.logits_src, group=self.group)
            T, H = int(shape[0]), int(shape[1])
            model.step_hidden = torch.empty(T, H, dtype=model.dtype, device=dev)
            model.step_normed = torch.empty(T, H, dtype=model.dtype, device=dev)
            dist.recv(model.step_hidden, src=self.logits_src, group=self.group)
            dist.recv(model.step_normed, src=self.logits_src, group=self.group)
            full = []
            for _r0, n in full_ranges:
                t = torch.empty(n, model.cfg.vocab_size, dtype=torch.float32, device=dev)
                dist.recv(t, src=self.logits_src, group=self.group)
                full.append(t)
        return full

