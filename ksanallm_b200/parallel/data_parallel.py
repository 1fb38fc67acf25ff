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
        # "allgather": every rank sees every row (dispatch = all-gather, combine = reduce-scatter; over peer memory with
        # the fused backend). "alltoall": a row travels only to the ranks that hold one of its experts and only their
        # weighted outputs travel back (library all-to-all collectives with per-step sizes; KSANA_EP_DISPATCH=alltoall)
        import os
        self.dispatch = os.environ.get("KSANA_EP_DISPATCH", "allgather")
        self.dispatched_rows = 0                     # rows sent to other ranks (all-to-all) since the start

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
        if self.dispatch == "alltoall":
            return self._moe_alltoall(model, mw, x, h)
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

    def _moe_alltoall(self, model, mw, x: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        """Expert-parallel block as an all-to-all. Every rank routes its own rows, sends a row once to each rank that
        holds at least one of the row's chosen experts (with the choices restricted to that rank's experts), the
        owners run their experts on what they received and send one weighted sum per received row back, and the home
        rank adds up what returns. With group-limited routing a row reaches at most ``topk_group`` ranks instead of
        all of them. Sizes differ per step, so the row counts are exchanged first (one small all-to-all and a host
        read); every rank takes part in every collective, also with no rows of its own."""
        from ..models.moe import moe_partial, route, shared_expert
        from ..ops import dispatch as ops
        T, H = x.shape
        K = model.cfg.num_experts_per_tok
        dev = x.device
        per = mw.expert_hi - mw.expert_lo                     # experts per rank (whole experts, equal shares)
        if T:
            ids, w = route(model, mw, x)
            dest = (ids.long() // per).clamp_(0, self.size - 1)                  # [T, K] owner rank of every choice
        send_idx, send_counts = [], []
        for d in range(self.size):
            idx = (dest == d).any(dim=1).nonzero(as_tuple=True)[0] if T else torch.zeros(0, dtype=torch.long, device=dev)
            send_idx.append(idx)
            send_counts.append(int(idx.numel()))
        order = torch.cat(send_idx) if T else torch.zeros(0, dtype=torch.long, device=dev)
        n_send = int(order.numel())
        rows = x[order].contiguous() if n_send else x.new_zeros(0, H)
        if n_send:
            to = torch.repeat_interleave(torch.arange(self.size, device=dev), torch.tensor(send_counts, device=dev))
            here = dest[order] == to.unsqueeze(1)                                 # choices that live on the target rank
            s_ids = torch.where(here, ids[order].to(torch.int32), torch.full_like(ids[order], -1, dtype=torch.int32)).contiguous()
            s_w = torch.where(here, w[order], torch.zeros_like(w[order])).contiguous()
        else:
            s_ids = torch.zeros(0, K, dtype=torch.int32, device=dev)
            s_w = torch.zeros(0, K, dtype=torch.float32, device=dev)
        cnt_out = torch.tensor(send_counts, dtype=torch.int64, device=dev)
        cnt_in = torch.empty(self.size, dtype=torch.int64, device=dev)
        dist.all_to_all_single(cnt_in, cnt_out, group=self.group)
        recv_counts = [int(c) for c in cnt_in.tolist()]
        n_recv = sum(recv_counts)
        r_rows = torch.empty(n_recv, H, dtype=x.dtype, device=dev)
        r_ids = torch.empty(n_recv, K, dtype=torch.int32, device=dev)
        r_w = torch.empty(n_recv, K, dtype=torch.float32, device=dev)
        for out_t, in_t in ((r_rows, rows), (r_ids, s_ids), (r_w, s_w)):
            dist.all_to_all_single(out_t, in_t, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=self.group)
        self.dispatched_rows += n_send - send_counts[self.rank]
        self.gathered_bytes += (n_recv - recv_counts[self.rank]) * H * x.element_size()
        if n_recv:
            part = moe_partial(model, mw, r_rows, shared=False, routing=(r_ids, r_w)).contiguous()
        else:
            part = x.new_zeros(0, H)
        back = torch.empty(n_send, H, dtype=x.dtype, device=dev)
        dist.all_to_all_single(back, part, output_split_sizes=send_counts, input_split_sizes=recv_counts, group=self.group)
        if not T:
            return h
        out = torch.zeros(T, H, dtype=torch.float32, device=dev)
        out.index_add_(0, order, back.float())
        if mw.shared_gate_up is not None:
            out = out + shared_expert(model, mw, x).float()
        return ops.add(h, out.to(x.dtype).contiguous())
