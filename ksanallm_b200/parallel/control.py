"""Step-plan distribution between the ranks of one engine: rank 0 owns the scheduler and sends the
packed plan image (see StepPlan::Pack) to the other ranks each step; ``None`` tells them to stop.
A CPU (gloo) process group carries it, so no device synchronisation is involved."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.distributed as dist


def broadcast_plan(group, image: Optional[np.ndarray], src: int = 0):
    """Collective. On the source ``image`` is the packed plan (or None to stop); returns the image
    (np.int32 array) on every rank, or None for the stop signal."""
    rank = dist.get_rank()
    if rank == src:
        n = -1 if image is None else int(image.size)
        hdr = torch.tensor([n], dtype=torch.int64)
        dist.broadcast(hdr, src=src, group=group)
        if n > 0:
            dist.broadcast(torch.from_numpy(np.ascontiguousarray(image, dtype=np.int32)), src=src, group=group)
        return image
    hdr = torch.zeros(1, dtype=torch.int64)
    dist.broadcast(hdr, src=src, group=group)
    n = int(hdr.item())
    if n < 0:
        return None
    buf = torch.empty(n, dtype=torch.int32)
    if n > 0:
        dist.broadcast(buf, src=src, group=group)
    return buf.numpy()
