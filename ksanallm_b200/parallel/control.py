"""Step-plan distribution between the ranks of one engine: rank 0 owns the scheduler and sends the
packed plan image (see StepPlan::Pack) to the other ranks each step; ``None`` tells them to stop.
A CPU (gloo) process group carries it, so no device synchronisation is involved."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.distributed as dist


def broadcast_plan(group, image: Optional[np.ndarray], src: int = 0, extras: Optional[bytes] = None,
                   with_extras: bool = False):
    """Collective. On the source ``image`` is the packed plan (or None to stop) and ``extras`` an optional byte
    string that goes with it (the step's optional inputs, see ``pack_extras``). Returns the image (np.int32 array)
    on every rank, or None for the stop signal; with ``with_extras`` the pair (image, extras bytes or None)."""
    rank = dist.get_rank()
    if rank == src:
        n = -1 if image is None else int(image.size)
        ne_ = len(extras) if (extras and n > 0) else 0
        hdr = torch.tensor([n, ne_], dtype=torch.int64)
        dist.broadcast(hdr, src=src, group=group)
        if n > 0:
            dist.broadcast(torch.from_numpy(np.ascontiguousarray(image, dtype=np.int32)), src=src, group=group)
        if ne_:
            dist.broadcast(torch.frombuffer(bytearray(extras), dtype=torch.uint8), src=src, group=group)
        return (image, extras) if with_extras else image
    hdr = torch.zeros(2, dtype=torch.int64)
    dist.broadcast(hdr, src=src, group=group)
    n, ne_ = int(hdr[0]), int(hdr[1])
    if n < 0:
        return (None, None) if with_extras else None
    buf = torch.empty(n, dtype=torch.int32)
    if n > 0:
        dist.broadcast(buf, src=src, group=group)
    blob = None
    if ne_:
        eb = torch.empty(ne_, dtype=torch.uint8)
        dist.broadcast(eb, src=src, group=group)
        blob = eb.numpy().tobytes()
    return (buf.numpy(), blob) if with_extras else buf.numpy()


def pack_extras(extra: Optional[dict]) -> Optional[bytes]:
    """Byte image of a step's optional inputs (host tensors, flags, row ranges) for the worker ranks."""
    if not extra:
        return None
    import io
    f = io.BytesIO()
    torch.save({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in extra.items()}, f)
    return f.getvalue()


def unpack_extras(blob: Optional[bytes]) -> Optional[dict]:
    if not blob:
        return None
    import io
    return torch.load(io.BytesIO(blob), weights_only=True)
