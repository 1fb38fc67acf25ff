"""Attention data parallelism with expert parallelism (DeepSeek-style serving layout).

The reference has neither (one tensor-parallel group serves every request, experts are sliced by tensor
parallelism: src/ksana_llm/models/common_moe/common_moe_model.cpp:35-63). Here every rank of the group owns a
disjoint set of sequences for everything except the routed experts:

  * attention, dense MLPs, shared experts, norms, lm_head: replicated weights, each rank computes only the rows of
    its own sequences (their KV lives only in that rank's cache);
  * routed experts: whole experts per rank (expert parallelism). At an MoE block every rank contributes its rows to an
    all-gather (dispatch), runs its own experts over all rows, and a reduce-scatter returns to every rank the summed
    expert outputs of its own rows (combine).

Sequence ownership is ``seq_id % size``: stable for the lifetime of a sequence and known to every rank from the
broadcast step plan, as are all ranks' row counts, so no sizes are exchanged at run time. Rank 0 schedules and
samples; the other ranks send it the logits rows of their sequences each step. The scheduler keeps one KV block pool
(with its own prefix tree and host swap pool) per rank, so the group holds ``size`` times the sequences of one GPU;
block ids in a sequence's table are ids of its owner's pool.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist


class AttentionDP:
    def __init__(self, rank: int, size: int, group=None, symm=None):
        self.rank, self.size, self.group = rank, size, group
        self.symm = symm                             # parallel.symm.SymmetricComm: dispatch / combine over peer memory
        self.counts: List[int] = [0] * size          # rows per rank of the step being executed
        self.blocks_per_rank = 0                     # device blocks of one rank's pool (set by the engine)
        self.gathered_bytes = 0

    # ------------------------------------------------------------------ step plan -> this rank's share
    def owner(self, seq_ids: np.ndarray) -> np.ndarray:
        return np.asarray(seq_ids, dtype=np.int64) % self.size

    def sub_plan(self, plan):
        """The plan restricted to this rank's sequences (same field names as the scheduler's plan), plus the
        bookkeeping ``gather_logits`` needs. Rows keep the plan's order: multi-token sequences first."""
        seq_ids = np.asarray(plan.seq_ids, dtype=np.int64)
        own = self.owner(seq_ids)
        cu = np.asarray(plan.cu_q, dtype=np.int64)
        q_lens = np.diff(cu)
        self.counts = [int(q_lens[own == r].sum()) for r in range(self.size)]
        mine = np.nonzero(own == self.rank)[0]
        rows = np.concatenate([np.arange(cu[i], cu[i + 1]) for i in mine]) if len(mine) else np.zeros(0, dtype=np.int64)
        new_row = np.full(int(cu[-1]) + 1, -1, dtype=np.int64)
        new_row[rows] = np.arange(len(rows))
        sample_rows = np.asarray(plan.sample_rows, dtype=np.int64)
        sample_seq = np.asarray(plan.sample_seq_ids, dtype=np.int64)
        sample_owner = self.owner(sample_seq)
        my_samples = np.nonzero(sample_owner == self.rank)[0]
        nm = int((mine < plan.num_multi).sum())
        ql = q_lens[mine]
        table = np.asarray(plan.block_table, dtype=np.int32).reshape(len(seq_ids), plan.max_blocks)
        sub = SimpleNamespace(
            seq_ids=seq_ids[mine].astype(np.int32), q_lens=ql.astype(np.int32),
            kv_lens=np.asarray(plan.kv_lens, dtype=np.int32)[mine],
            input_ids=np.asarray(plan.input_ids, dtype=np.int32)[rows], positions=np.asarray(plan.positions, dtype=np.int32)[rows],
            slots=np.asarray(plan.slots, dtype=np.int32)[rows],
            cu_q=np.concatenate([[0], np.cumsum(ql)]).astype(np.int32),
            block_table=table[mine].reshape(-1), max_blocks=plan.max_blocks,
            sample_rows=new_row[sample_rows[my_samples]].astype(np.int32), sample_seq_ids=sample_seq[my_samples].astype(np.int32),
            num_multi=nm, num_single=len(mine) - nm, num_tokens=int(len(rows)), num_multi_tokens=int(ql[:nm].sum()),
            max_q_len=int(ql.max()) if len(ql) else 0,
            swap_out=self._mine(plan.swap_out, 2, (0,)), swap_in=self._mine(plan.swap_in, 2, (0,)),
            copies=self._mine(plan.copies, 3, (0, 1)), pre_copies=self._mine(getattr(plan, "pre_copies", ()), 3, (0, 1)))
        self._sample_owner = sample_owner
        self._sample_counts = [int((sample_owner == r).sum()) for r in range(self.size)]
        return sub

    def _mine(self, flat, width: int, block_cols) -> np.ndarray:
        """Swap / copy entries of this rank. The scheduler keeps one block pool per rank and writes a device block of
        these lists as ``rank * blocks_per_rank + block``; entries of other ranks are dropped, ours lose the offset."""
        a = np.asarray(flat, dtype=np.int32).reshape(-1, width)
        if a.size == 0 or not self.blocks_per_rank:
            return np.asarray(flat, dtype=np.int32)
        keep = (a[:, block_cols[0]] // self.blocks_per_rank) == self.rank
        a = a[keep].copy()
        for c in block_cols:
            a[:, c] -= self.rank * self.blocks_per_rank
        return a.reshape(-1)

    # ------------------------------------------------------------------ logits back to the scheduler rank
    def gather_logits(self, local: Optional[torch.Tensor], vocab: int, device) -> Optional[torch.Tensor]:
        """Collective. ``local``: this rank's fp32 logits rows [n_local, vocab] (None when it has none). Rank 0
        gets all rows in the plan's sample order; other ranks get None."""
        n_max = max(self._sample_counts) if self._sample_counts else 0
        if n_max == 0:
            return None if self.rank else torch.zeros(0, vocab, dtype=torch.float32, device=device)
        pad = torch.zeros(n_max, vocab, dtype=torch.float32, device=device)
        if local is not None and local.shape[0]:
            pad[: local.shape[0]] = local
        out = torch.empty(self.size * n_max, vocab, dtype=torch.float32, device=device)
        dist.all_gather_into_tensor(out, pad, group=self.group)
        if self.rank != 0:
            return None
        idx = np.zeros(len(self._sample_owner), dtype=np.int64)
        seen = [0] * self.size
        for j, r in enumerate(self._sample_owner):
            idx[j] = r * n_max + seen[r]
            seen[r] += 1
        return out[torch.from_numpy(idx).to(device)]

    # ------------------------------------------------------------------ MoE block: dispatch / experts / combine
    def moe(self, model, mw, x: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        """h += routed experts(x) + shared expert(x) for this rank's rows ``x`` [T_r, H]."""
        from ..models.moe import moe_partial, shared_expert
        from ..ops import dispatch as ops
        t_max = max(self.counts)
        T, H = x.shape
        if t_max == 0:
            return h
        pad = x if T == t_max else torch.cat([x, x.new_zeros(t_max - T, H)], 0)
        if self.symm is not None and x.is_cuda:
            # peer-memory path: rows pulled from the peers' staging areas (dispatch), this rank's experts run over
            # all rows with their weighted outputs written into its peer-visible slot, and one kernel pulls this
            # rank's rows from every peer, sums them and adds them to the residual (combine)
            gathered = self.symm.all_gather_rows(pad.contiguous())
            if gathered is not None:
                self.gathered_bytes += gathered.numel() * gathered.element_size()
                out_rows = h.contiguous() if T else h
                if mw.shared_gate_up is not None and T:
                    out_rows = ops.add(out_rows, shared_expert(model, mw, x).contiguous())
                if self.symm.reduce_rows_into(lambda part: moe_partial(model, mw, gathered, into=part, shared=False),
                                              self.size * t_max, self.rank * t_max, out_rows):
                    return out_rows
                raise RuntimeError("expert combine does not fit the symmetric buffer (raise max_step_tokens head room)")
        gathered = torch.empty(self.size * t_max, H, dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(gathered, pad.contiguous(), group=self.group)        # dispatch
        self.gathered_bytes += gathered.numel() * gathered.element_size()
        part = moe_partial(model, mw, gathered, shared=False)                              # this rank's experts, all rows
        if x.is_cuda:
            mine = torch.empty(t_max, H, dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(mine, part.contiguous(), group=self.group)          # combine
        else:                                   # CPU process groups have no reduce-scatter: sum everything, keep our rows
            part = part.contiguous()
            dist.all_reduce(part, group=self.group)
            mine = part[self.rank * t_max:(self.rank + 1) * t_max]
        out = mine[:T]
        if mw.shared_gate_up is not None and T:
            out = out + shared_expert(model, mw, x)
        return ops.add(h, out.contiguous()) if T else h
