"""Debug-mode validation of everything a step hands to the kernels as an index.

The kernels trust the step metadata (block tables, cache slots, token ids, row indices). With
``KSANA_CHECK_INPUTS=1`` the runner validates it on the host before every forward pass and raises with the first
violation, so that a scheduler or plug-in bug surfaces as a Python exception instead of an out-of-range device
access. This is the engine's own bounds-check mode, for runs where no device-side sanitizer is at hand.
The checks synchronise with the device and are meant for tests and debugging, not for serving.
"""
from __future__ import annotations

import os
from typing import List

import torch


def enabled() -> bool:
    return os.environ.get("KSANA_CHECK_INPUTS", "0") not in ("", "0", "false", "False")


def step_violations(step, num_blocks: int, block_tokens: int, vocab_size: int, max_positions: int) -> List[str]:
    """All violations found in a StepInput (empty list = consistent)."""
    bad: List[str] = []
    T = int(step.input_ids.shape[0])
    nseq = int(step.kv_lens.shape[0])
    cu = step.cu_q.long().cpu()
    kv = step.kv_lens.long().cpu()
    ids = step.input_ids.long().cpu()
    pos = step.positions.long().cpu()
    slots = step.slots.long().cpu()
    table = step.block_table.long().cpu()
    if T != step.num_tokens:
        bad.append(f"num_tokens {step.num_tokens} != rows {T}")
    if step.num_multi + step.num_single != nseq:
        bad.append(f"num_multi + num_single = {step.num_multi + step.num_single} != sequences {nseq}")
    if cu.numel() != nseq + 1 or int(cu[0]) != 0 or (nseq and int(cu[-1]) != T) or bool((cu[1:] < cu[:-1]).any()):
        bad.append("cu_q is not a non-decreasing prefix sum ending at the row count")
        return bad
    q_lens = cu[1:] - cu[:-1]
    if nseq and bool((q_lens > kv).any()):
        bad.append("a sequence has more new rows than cached + new tokens (q_len > kv_len)")
    if nseq and int(q_lens.max()) > max(step.max_q_len, 0):
        bad.append(f"max_q_len {step.max_q_len} is smaller than the longest row count {int(q_lens.max())}")
    if step.num_multi < nseq and bool((q_lens[step.num_multi:] != 1).any()):
        bad.append("a single-token sequence has a row count other than 1")
    if T and (int(ids.min()) < 0 or int(ids.max()) >= vocab_size):
        bad.append(f"token id outside [0, {vocab_size})")
    if T and (int(pos.min()) < 0 or int(pos.max()) >= max_positions):
        bad.append(f"position outside [0, {max_positions})")
    live = slots[slots >= 0]
    if live.numel():
        if int(live.max()) >= num_blocks * block_tokens:
            bad.append(f"cache slot beyond the {num_blocks} blocks of the cache")
        if live.unique().numel() != live.numel():
            bad.append("two rows write the same cache slot")
    if bool((slots < -1).any()):
        bad.append("cache slot below -1")
    for s in range(nseq):
        need = (int(kv[s]) + block_tokens - 1) // block_tokens
        if need > table.shape[1]:
            bad.append(f"sequence {s}: {need} blocks needed, block table has {table.shape[1]} columns")
            continue
        used = table[s, :need]
        if need and (int(used.min()) < 0 or int(used.max()) >= num_blocks):
            bad.append(f"sequence {s}: block id outside [0, {num_blocks})")
            continue
        # the rows written this step must land in the blocks the table names for their positions
        q0, q1 = int(cu[s]), int(cu[s + 1])
        for r in range(q0, q1):
            sl = int(slots[r])
            if sl < 0:
                continue
            p = int(kv[s]) - (q1 - r)
            if sl != int(table[s, p // block_tokens]) * block_tokens + p % block_tokens:
                bad.append(f"sequence {s}: row {r} writes slot {sl}, its block table says otherwise")
                break
    if step.logits_rows is not None and step.logits_rows.numel():
        lr = step.logits_rows.long().cpu()
        if int(lr.min()) < 0 or int(lr.max()) >= T:
            bad.append("a logits row index is outside the step's rows")
    if step.refit_positions is not None and step.refit_positions.numel():
        rp = step.refit_positions.long().cpu()
        if int(rp.min()) < 0 or int(rp.max()) >= T:
            bad.append("an embedding-refit row index is outside the step's rows")
    return bad


def check_step(step, model) -> None:
    cache = model.kv_cache
    bad = step_violations(step, int(cache.shape[0]), model.block_tokens, model.cfg.vocab_size,
                          int(model.cos_sin.shape[0]) if model.cos_sin is not None else 1 << 30)
    if bad:
        raise RuntimeError("inconsistent step metadata: " + "; ".join(bad))
