"""Token selection for one engine step. The device work is the fused sampler kernel (penalties and
bans edit the fp32 logits first); the host part keeps the per-request bookkeeping: penalty token
lists, n-gram bans, log-prob collection and beam expansion.

Order of operations and semantics follow the reference sampler
(src/ksana_llm/samplers/sampler.cpp:82-400; beam search:
src/ksana_llm/samplers/beam_search/beam_search_sampling.cpp:10-113): repetition penalty,
n-gram bans, top-N log-probs over the temperature-scaled logits, then argmax / top-k / top-p.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from ..ops import native, reference as ref


@dataclass
class SamplingParams:
    temperature: float = 1.0
    topk: int = 1
    topp: float = 1.0
    repetition_penalty: float = 1.0
    no_repeat_ngram_size: int = 0
    encoder_no_repeat_ngram_size: int = 0
    logprobs_num: int = 0
    num_beams: int = 1
    length_penalty: float = 1.0
    seed: int = 1
    step: int = 0
    index: int = 0

    @staticmethod
    def from_request(req, index: int) -> "SamplingParams":
        if req is None:
            return SamplingParams()
        c = req.cfg
        out = req.outputs[index]
        return SamplingParams(c.temperature, c.topk, c.topp, c.repetition_penalty, c.no_repeat_ngram_size,
                              c.encoder_no_repeat_ngram_size, c.logprobs_num, c.num_beams, c.length_penalty,
                              (int(c.seed) + 7919 * index) & ((1 << 62) - 1), len(out.tokens), index)


def banned_ngram_tokens(history: List[int], n: int) -> List[int]:
    """Tokens that would complete an n-gram already present in ``history``."""
    if n <= 0 or len(history) + 1 < n:
        return []
    if n == 1:
        return list(set(history))
    prefix = tuple(history[len(history) - (n - 1):])
    banned = set()
    for i in range(len(history) - n + 1):
        if tuple(history[i:i + n - 1]) == prefix:
            banned.add(history[i + n - 1])
    return list(banned)


def banned_encoder_ngram_tokens(prompt: List[int], generated: List[int], n: int) -> List[int]:
    """Tokens that would reproduce an n-gram of the prompt."""
    if n <= 0:
        return []
    if n == 1:
        return list(set(prompt))
    if len(generated) < n - 1:
        return []
    prefix = tuple(generated[len(generated) - (n - 1):])
    banned = set()
    for i in range(len(prompt) - n + 1):
        if tuple(prompt[i:i + n - 1]) == prefix:
            banned.add(prompt[i + n - 1])
    return list(banned)


class DeviceStepError(RuntimeError):
    """A kernel of the step reported through the device error word: a bounded wait ran out (a peer or a copy never
    arrived) or an index guard skipped an out-of-range access. The step's results are invalid."""

    def __init__(self, code: int):
        self.code = int(code)
        super().__init__(native.describe_err_code(self.code))


class Sampler:
    def __init__(self, device, vocab_size: int, stage=None):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.vocab = vocab_size
        self.d2h_bytes = 0
        self._cpu_rng = torch.Generator().manual_seed(1234)
        self._stage = stage                  # int32 host array -> device through pinned staging (ModelRunner._stage)
        self._host_out = None                # pinned read-back area: tokens, then the device error word
        self._host_cap = 0
        self._done = None
        self._plain_slots = [[None, None], [None, None]]     # two read-back areas: a step in flight and the next one
        self._plain_next = 0

    @staticmethod
    def params_image(params: List[SamplingParams]) -> np.ndarray:
        """The sampler kernel's per-row parameters as 6 int32 words per row: temperature, top-k, top-p, draw counter
        (all rows of one kind together), then the 64-bit seeds."""
        B = len(params)
        img = np.empty(6 * B, dtype=np.int32)
        img[0:B] = np.array([p.temperature for p in params], dtype=np.float32).view(np.int32)
        img[B:2 * B] = [p.topk for p in params]
        img[2 * B:3 * B] = np.array([p.topp for p in params], dtype=np.float32).view(np.int32)
        img[3 * B:4 * B] = [p.step for p in params]
        img[4 * B:6 * B] = np.array([p.seed for p in params], dtype=np.int64).view(np.int32)
        return img

    def _image_views(self, dev: torch.Tensor, B: int):
        o = 4 * B                                             # seeds are 64-bit: an even word offset keeps them aligned
        return (dev[0:B].view(torch.float32), dev[B:2 * B], dev[2 * B:3 * B].view(torch.float32), dev[3 * B:4 * B],
                dev[o:o + 2 * B].view(torch.int64))

    # ------------------------------------------------------------------ plain rows, in two halves (pipelined steps)
    def launch_plain(self, logits, image: np.ndarray, B: int, read_back: bool = True) -> dict:
        """Sampling of rows that need nothing but the kernel (no penalties, bans, log-probs or beams), without waiting
        for the result: returns a handle whose ``tokens_dev`` (int32 [B] on the device) the next step can read its
        input ids from, and which ``finish_plain`` turns into host tokens later. ``read_back`` False (worker ranks):
        nothing is copied to the host."""
        merged = None
        if not torch.is_tensor(logits):
            merged, logits = logits, logits.values
        logits = logits[:B]
        if not self.cuda:
            view = torch.from_numpy(image)
            temp, topk, topp = view[0:B].view(torch.float32), view[B:2 * B], view[2 * B:3 * B].view(torch.float32)
            u = torch.rand(B, generator=self._cpu_rng)
            tok, _, _ = ref.sample(logits.float(), temp, topk, topp, u, 0)
            code = int(native.err_flag(self.device).item())
            return {"tokens_dev": tok.to(torch.int32), "B": B, "code": code}
        dev = self._stage(image) if self._stage is not None else torch.from_numpy(image).to(self.device)
        temp, topk, topp, steps, seeds = self._image_views(dev, B)
        out = torch.empty(B, dtype=torch.int32, device=self.device)
        if merged is not None:
            native.sample_merged(logits, merged.ids[:B], temp, topk, topp, seeds, steps, out)
        else:
            native.sample(logits, temp, topk, topp, seeds, steps, out)
        handle = {"tokens_dev": out, "B": B}
        if read_back:
            slot = self._plain_slots[self._plain_next]
            self._plain_next ^= 1
            if slot[0] is None or slot[0].numel() < B + 1:
                slot[0] = torch.empty(max(2 * (B + 1), 1024), dtype=torch.int32, pin_memory=True)
                slot[1] = torch.cuda.Event()
            slot[0][:B].copy_(out, non_blocking=True)
            slot[0][B:B + 1].copy_(native.err_flag(self.device), non_blocking=True)
            slot[1].record()
            handle["slot"] = slot
            self.d2h_bytes += (B + 1) * 4
        return handle

    def finish_plain(self, handle: dict) -> List[int]:
        """Waits for a ``launch_plain`` result (the step's only host synchronisation); raises DeviceStepError when a
        kernel of that step reported through the error word."""
        B = handle["B"]
        if B == 0 or handle.get("tokens_dev") is None:
            return []
        if "slot" not in handle:
            code = handle.get("code", 0)
            if code:
                native.clear_err_flag(self.device)
                raise DeviceStepError(code)
            return handle["tokens_dev"].tolist()
        host, ev = handle["slot"]
        ev.synchronize()
        arr = host[:B + 1].numpy()
        code = int(arr[B])
        if code != 0:
            native.clear_err_flag(self.device)
            raise DeviceStepError(code)
        return arr[:B].tolist()

    def _upload_params(self, params: List[SamplingParams]):
        """temperature / top-k / top-p / step counters / seeds of all rows in one staged host->device copy."""
        B = len(params)
        img = np.empty(6 * B, dtype=np.int32)
        img[0:B] = np.array([p.temperature for p in params], dtype=np.float32).view(np.int32)
        img[B:2 * B] = [p.topk for p in params]
        img[2 * B:3 * B] = np.array([p.topp for p in params], dtype=np.float32).view(np.int32)
        img[3 * B:4 * B] = [p.step for p in params]
        o = 4 * B                                             # seeds are 64-bit: an even word offset keeps them 8-byte aligned
        img[o:o + 2 * B] = np.array([p.seed for p in params], dtype=np.int64).view(np.int32)
        if self._stage is not None:
            dev = self._stage(img)
        else:
            dev = torch.from_numpy(img).to(self.device)
        return (dev[0:B].view(torch.float32), dev[B:2 * B], dev[2 * B:3 * B].view(torch.float32), dev[3 * B:4 * B],
                dev[o:o + 2 * B].view(torch.int64))

    def _read_back(self, out: torch.Tensor):
        """Sampled tokens and the device error word through pinned memory: two asynchronous copies and one event
        wait (the step's only host synchronisation). Raises DeviceStepError when a kernel of the step reported."""
        B = out.numel()
        if self._host_out is None or self._host_cap < B + 1:
            self._host_cap = max(2 * (B + 1), 1024)
            self._host_out = torch.empty(self._host_cap, dtype=torch.int32, pin_memory=True)
            self._done = torch.cuda.Event()
        host = self._host_out
        host[:B].copy_(out, non_blocking=True)
        host[B:B + 1].copy_(native.err_flag(self.device), non_blocking=True)
        self._done.record()
        self._done.synchronize()
        self.d2h_bytes += (B + 1) * 4
        arr = host[:B + 1].numpy()
        code = int(arr[B])
        if code != 0:
            native.clear_err_flag(self.device)
            raise DeviceStepError(code)
        return arr[:B].tolist()

    def _csr(self, lists: List[List[int]]):
        offs = np.zeros(len(lists) + 1, dtype=np.int32)
        for i, l in enumerate(lists):
            offs[i + 1] = offs[i] + len(l)
        ids = np.fromiter((t for l in lists for t in l), dtype=np.int32, count=int(offs[-1]))
        return (torch.from_numpy(offs).to(self.device), torch.from_numpy(ids).to(self.device))

    @torch.inference_mode()
    def sample(self, logits, params: List[SamplingParams], reqs, seq_ids: List[int]):
        B = len(params)
        merged = None
        if not torch.is_tensor(logits):
            # per-shard top-k candidates gathered from the tensor-parallel ranks (models.common.LogitCandidates): the
            # engine only asks for them when no row edits its logits first, so the penalty / ban passes are skipped
            merged, logits = logits, logits.values
        logits = logits[:B]
        # 1. repetition penalty over the distinct tokens seen so far
        if merged is None and any(p.repetition_penalty != 1.0 for p in params):
            lists = []
            for p, (req, i) in zip(params, reqs):
                seen = set(req.prompt) | set(req.outputs[i].tokens) if (req is not None and p.repetition_penalty != 1.0) else set()
                lists.append([t for t in seen if 0 <= t < self.vocab])
            pen = torch.tensor([p.repetition_penalty for p in params], dtype=torch.float32, device=self.device)
            offs, ids = self._csr(lists)
            if self.cuda:
                native.repetition_penalty(logits, offs, ids, pen)
            else:
                for b, l in enumerate(lists):
                    if l:
                        logits[b, torch.tensor(l)] *= 1.0 / params[b].repetition_penalty
        # 2. n-gram bans
        if merged is None and any(p.no_repeat_ngram_size > 0 or p.encoder_no_repeat_ngram_size > 0 for p in params):
            lists = []
            for p, (req, i) in zip(params, reqs):
                ban = []
                if req is not None:
                    gen = req.outputs[i].tokens
                    if p.no_repeat_ngram_size > 0:
                        ban += banned_ngram_tokens(list(req.prompt) + list(gen), p.no_repeat_ngram_size)
                    if p.encoder_no_repeat_ngram_size > 0:
                        ban += banned_encoder_ngram_tokens(list(req.prompt), list(gen), p.encoder_no_repeat_ngram_size)
                lists.append([t for t in set(ban) if 0 <= t < self.vocab])
            offs, ids = self._csr(lists)
            if self.cuda:
                native.ban_tokens(logits, offs, ids)
            else:
                for b, l in enumerate(lists):
                    if l:
                        logits[b, torch.tensor(l)] = float("-inf")
        # 3. fused temperature / top-k / top-p / draw (+ top-N log-probs)
        N = max(p.logprobs_num for p in params)
        if self.cuda:
            temp, topk, topp, steps, seeds = self._upload_params(params)
            out = torch.empty(B, dtype=torch.int32, device=self.device)
            lp_ids = torch.empty(B, max(N, 1), dtype=torch.int32, device=self.device) if N else None
            lp_vals = torch.empty(B, max(N, 1), dtype=torch.float32, device=self.device) if N else None
            if merged is not None:
                native.sample_merged(logits, merged.ids[:B], temp, topk, topp, seeds, steps, out, num_logprobs=N,
                                     lp_ids=lp_ids, lp_vals=lp_vals)
            else:
                native.sample(logits, temp, topk, topp, seeds, steps, out, num_logprobs=N, lp_ids=lp_ids, lp_vals=lp_vals)
            tokens = self._read_back(out)      # the step's device->host result read (the only host synchronisation)
            if N:
                lp_ids_h, lp_vals_h = lp_ids.cpu(), lp_vals.cpu()
                self.d2h_bytes += B * N * 8
        else:
            temp = torch.tensor([p.temperature for p in params], dtype=torch.float32)
            topk = torch.tensor([p.topk for p in params], dtype=torch.int32)
            topp = torch.tensor([p.topp for p in params], dtype=torch.float32)
            u = torch.rand(B, generator=self._cpu_rng)
            tok, lp_ids_h, lp_vals_h = ref.sample(logits.float(), temp, topk, topp, u, N)
            tokens = tok.tolist()
            code = int(native.err_flag(self.device).item())      # same contract as the device path
            if code != 0:
                native.clear_err_flag(self.device)
                raise DeviceStepError(code)
        parents = [-1] * B
        lp_by_seq: Dict[int, list] = {}
        if N:
            for b, sid in enumerate(seq_ids):
                n = params[b].logprobs_num
                if n:
                    lp_by_seq[sid] = [(int(lp_ids_h[b, j]), float(lp_vals_h[b, j])) for j in range(n)]
            self._beam_search(params, reqs, seq_ids, tokens, parents, lp_by_seq)
        return tokens, parents, lp_by_seq

    def _beam_search(self, params, reqs, seq_ids, tokens, parents, lp_by_seq):
        """Beam expansion per request group: candidates = beams x their top log-probs, keep the best
        ``num_beams`` by cumulative log-prob, re-parent sequences whose history changes."""
        groups: Dict[int, List[int]] = {}
        for b, (req, i) in enumerate(reqs):
            if req is not None and params[b].num_beams > 1:
                groups.setdefault(req.req_id, []).append(b)
        for rid, rows in groups.items():
            req = reqs[rows[0]][0]
            nb = params[rows[0]].num_beams
            first = all(len(req.outputs[reqs[b][1]].tokens) == 0 for b in rows)
            cands = []
            for b in rows:
                out = req.outputs[reqs[b][1]]
                for tok, lp in lp_by_seq.get(seq_ids[b], []):
                    if tok >= 0:
                        cands.append((out.cum_logprob + lp, b, tok))
                if first:
                    break          # all beams share one history: expand it once
            cands.sort(key=lambda c: -c[0])
            chosen = cands[:len(rows)] if len(cands) >= len(rows) else (cands * len(rows))[:len(rows)]
            snapshot = {b: (list(req.outputs[reqs[b][1]].tokens), list(req.outputs[reqs[b][1]].logprobs)) for b in rows}
            for slot, (score, src_b, tok) in zip(rows, chosen):
                out = req.outputs[reqs[slot][1]]
                tokens[slot] = tok
                if src_b != slot and not first:
                    parents[slot] = seq_ids[src_b]
                    out.tokens, out.logprobs = list(snapshot[src_b][0]), list(snapshot[src_b][1])
                out.cum_logprob = score


def beam_final_order(outputs, length_penalty: float) -> List[int]:
    """Final ranking of a beam group: cumulative log-prob / len^length_penalty, best first."""
    scores = [o.cum_logprob / (max(len(o.tokens), 1) ** length_penalty) for o in outputs]
    return sorted(range(len(outputs)), key=lambda i: -scores[i])
