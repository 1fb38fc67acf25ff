"""``/forward`` request targets: validation rules and extraction of the requested tensors.

Rules follow src/ksana_llm/utils/request.cpp:89-181: targets are ``layernorm`` / ``transformer`` /
``logits``; a target gives ``token_id`` or ``slice_pos`` (not both); ``logits`` supports only
GATHER_TOKEN_ID with ``slice_pos`` that does not include the last position; ``transformer`` and
``layernorm`` support only GATHER_ALL. Logits targets return, for each requested position p, the
probability of the next input token: softmax(logits[p])[input[p+1]]
(src/ksana_llm/samplers/sampler.cpp:240-279), which is what perplexity evaluation needs.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

VALID_TARGETS = ("layernorm", "transformer", "logits")


def verify_request_target(targets: Dict[str, dict], input_len: int) -> Tuple[int, str]:
    for name, t in targets.items():
        if name not in VALID_TARGETS:
            return 1, f"Invalid target name {name}"
        token_id = t.get("token_id") or []
        slice_pos = t.get("slice_pos") or []
        mode = t.get("token_reduce_mode", "GATHER_ALL")
        if token_id and slice_pos:
            return 1, f"Unable to set both token_id and slice_pos at the same time for target {name}"
        if mode not in ("GATHER_ALL", "GATHER_TOKEN_ID"):
            return 1, f"Unsupported token_reduce_mode {mode}"
        norm = []
        for a, b in slice_pos:
            a = a + input_len if a < 0 else a
            b = b + input_len if b < 0 else b
            if a > b or a < 0 or b >= input_len:
                return 1, f"Invalid slice_pos [{a}, {b}] for input of {input_len} tokens in target {name}"
            if norm and a <= norm[-1][1]:
                return 1, f"slice_pos intervals of target {name} overlap or are unordered"
            norm.append([a, b])
        t["slice_pos"] = norm
        if name == "logits":
            if mode != "GATHER_TOKEN_ID":
                return 1, "The output of the 'logits' target only supports GATHER_TOKEN_ID"
            if token_id:
                return 1, "The 'logits' target does not support token_id"
            if norm and norm[-1][1] >= input_len - 1:
                return 1, "slice_pos of the 'logits' target may not include the last input position"
        elif mode != "GATHER_ALL":
            return 1, f"The output of the '{name}' target only supports GATHER_ALL"
    return 0, ""


def target_positions(t: dict, input_len: int) -> List[int]:
    pos = []
    for a, b in t.get("slice_pos") or []:
        pos.extend(range(a, b + 1))
    if not pos and not (t.get("token_id") or []):
        pos = [input_len - 1]
    return pos


def extract_targets(engine, plan, logits) -> None:
    """Called after the forward of a step. Sequences with request targets run as single-step prefill
    (their whole prompt is in this step), so hidden rows are addressed by position directly."""
    model = engine.model
    row0 = 0
    for k, sid in enumerate(plan.seq_ids.tolist()):
        ql = int(plan.q_lens[k])
        ent = engine.seq_to_req.get(sid)
        if ent is not None and ent[0].request_target and not ent[0].targets_done:
            req = ent[0]
            req.targets_done = True          # later (decode) steps of a generating request carry no prompt rows
            hidden_all = getattr(model, "step_hidden", None)
            for name, t in req.request_target.items():
                pos = target_positions(t, len(req.prompt))
                if name == "logits":
                    full = engine.full_logits_for(req, row0, ql)
                    p = torch.tensor(pos, dtype=torch.long)
                    nxt = torch.tensor([req.prompt[i + 1] for i in pos], dtype=torch.long)
                    probs = torch.softmax(full[p].float(), dim=-1)
                    req.response[name] = probs[torch.arange(len(pos)), nxt].cpu()
                else:
                    src = model.step_hidden if name == "transformer" else model.step_normed
                    token_id = t.get("token_id") or []
                    if token_id:
                        sel = [i for i, tok in enumerate(req.prompt) if tok in set(token_id)]
                    else:
                        sel = pos
                    idx = torch.tensor([row0 + i for i in sel], dtype=torch.long, device=src.device)
                    req.response[name] = src[idx].float().cpu()
        row0 += ql
