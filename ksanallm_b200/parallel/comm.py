"""Tensor-parallel communication. Two backends behind one interface:

* ``nccl``  - library collectives through torch.distributed (NCCL on GPUs, gloo on CPU). This is the
  op sequence of the reference (src/ksana_llm/models/base/model_communicator.cpp:64-123,
  src/ksana_llm/layers/nvidia/nccl_all_reduce_sum_layer.cpp:23-31, nccl_all_gather_layer.cpp:28-45)
  and serves as the baseline and the fallback.
* ``fused`` - hand-written kernels over peer-mapped symmetric buffers (see :mod:`.symm`): the
  row-parallel GEMM's partial sums are reduced across GPUs and the residual is added inside one
  kernel; small messages use a one-shot all-reduce. Every wait on a peer flag is bounded.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import dispatch as ops


class TPComm:
    def __init__(self, group=None, rank: int = 0, size: int = 1, backend: str = "nccl", device=None,
                 max_tokens: int = 16384, hidden: int = 8192):
        self.group, self.rank, self.size, self.backend = group, rank, size, backend
        self.device = device
        self.symm = None
        if backend == "fused" and size > 1 and device is not None and torch.device(device).type == "cuda":
            from .symm import SymmetricComm
            self.symm = SymmetricComm(group, rank, size, device, max_tokens, hidden)

    # ---- primitives
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        if self.symm is not None and self.symm.fits(x):
            return self.symm.all_reduce(x)
        dist.all_reduce(x, group=self.group)
        return x

    def all_gather_last_dim(self, x: torch.Tensor, valid: Optional[int] = None) -> torch.Tensor:
        """[M, n] shards -> [M, size*valid] (each shard contributes its first ``valid`` columns)."""
        if self.size == 1:
            return x
        x = x.contiguous()
        if self.symm is not None and x.is_cuda:
            out = self.symm.all_gather_cols(x, valid or x.shape[1])
            if out is not None:
                return out
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x, group=self.group)
        v = valid or x.shape[1]
        return torch.cat([p[:, :v] for p in parts], dim=1)

    # ---- fused-with-compute entry points used by the model code
    def row_parallel_linear(self, x, W, h: torch.Tensor) -> torch.Tensor:
        """h += all_reduce(x W^T). Baseline: GEMM, library all-reduce, add. Fused backend: the partial
        product is written into the symmetric buffer (or pushed to the peers by the GEMM's epilogue) and one kernel
        reduces over the ranks and adds the residual, for the batch sizes that every rank reduces itself; larger
        batches outside the fused forward (whose residual stream lives in the symmetric buffer) use the library."""
        if self.symm is not None and self.symm.one_shot(h.shape[0]) and h.is_contiguous():
            return self.symm.row_parallel_norm(x, W, h, None)[0]
        return self._rp_nccl(x, W, h)

    def _rp_nccl(self, x, W, h):
        partial = ops.linear(x, W)
        dist.all_reduce(partial, group=self.group)
        return ops.add(h, partial)
