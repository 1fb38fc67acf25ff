"""Step-plan distribution between the ranks of one engine: rank 0 owns the scheduler and sends the
packed plan image (see StepPlan::Pack) to the other ranks each step; ``None`` tells them to stop.
A CPU (gloo) process group carries it, so no device synchronisation is involved."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.distributed as dist


INLINE_WORDS = 16384          # plans up to this many int32 words travel inside the header message (one collective)


def broadcast_plan(group, image: Optional[np.ndarray], src: int = 0, extras: Optional[bytes] = None,
                   with_extras: bool = False):
    """Collective. On the source ``image`` is the packed plan (or None to stop) and ``extras`` an optional byte
    string that goes with it (the step's optional inputs, see ``pack_extras``). Returns the image (np.int32 array)
    on every rank, or None for the stop signal; with ``with_extras`` the pair (image, extras bytes or None).

    One fixed-size message per step in the common case: words 0 / 1 carry the plan's length (-1: stop) and the
    extras' length, and a plan of up to INLINE_WORDS words (every decode step, most prefill steps) follows in the same
    message. Longer plans and extras go in a second / third message whose sizes the first one announced."""
    rank = dist.get_rank()
    head = torch.zeros(2 + INLINE_WORDS, dtype=torch.int32)
    if rank == src:
        n = -1 if image is None else int(image.size)
        ne_ = len(extras) if (extras and n > 0) else 0
        head[0], head[1] = n, ne_
        img = None
        if n > 0:
            img = torch.from_numpy(np.ascontiguousarray(image, dtype=np.int32).reshape(-1))
            if n <= INLINE_WORDS:
                head[2:2 + n] = img
        dist.broadcast(head, src=src, group=group)
        if n > INLINE_WORDS:
            dist.broadcast(img, src=src, group=group)
        if ne_:
            dist.broadcast(torch.frombuffer(bytearray(extras), dtype=torch.uint8), src=src, group=group)
        return (image, extras) if with_extras else image
    dist.broadcast(head, src=src, group=group)
    n, ne_ = int(head[0]), int(head[1])
    if n < 0:
        return (None, None) if with_extras else None
    if n <= INLINE_WORDS:
        buf = head[2:2 + n].clone()
    else:
        buf = torch.empty(n, dtype=torch.int32)
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
