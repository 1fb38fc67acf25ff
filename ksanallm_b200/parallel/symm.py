"""Symmetric (peer-mapped) buffers and the fused tensor-parallel paths built on them.

Every rank allocates one buffer of identical layout with ``torch.distributed._symmetric_memory`` and
maps all peers' buffers, so the kernels in ``comm.cu`` and the GEMM push epilogues address peers with
plain pointers over NVLink. Layout (bytes):

    [0, 4 KiB)              flag pad (per kind and peer: last signalled epoch)
    slots[2][size]          receive slots for partial products (double buffered by call parity)
    h, y, yq, yscale        all-gathered residual stream / normalised activations (large batches)
    stage                   staging area for the plain all-reduce

Row-parallel linear:
  * up to ``ONE_SHOT_ROWS`` rows: the GEMM writes its partial product into its own symmetric buffer; after
    one flag exchange every rank pulls all rows from every peer, sums them in rank order, adds the residual
    and normalises all rows itself (no gather phase);
  * more rows: the GEMM writes its partial product into its own symmetric buffer; one kernel per rank then
    pulls the rows it owns from every peer (coalesced peer loads: reduce-scatter), adds the residual,
    normalises (+ FP8 quantises) and pushes the result rows to every peer (all-gather), followed by one more
    flag exchange. The residual stream stays sharded by rows: only its owner ever reads it. With ``PUSH_EPILOGUE``
    (KSANA_PUSH_PREFILL=1) the GEMM's epilogue stores each partial row piece straight into the receive slot of the
    rank that owns the row (64 contiguous bytes per row and store, turned through shared memory; one 16-byte piece
    per row and thread ran NVLink at a fraction of its rate), so the reduce-scatter traffic overlaps the tiles still
    being computed and the reduce kernel reads local memory only.
Every wait is bounded in the kernels; a timeout sets the device error word (see native.check_err_flag).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native
from ..ops.dispatch import LinearWeight, QTensor, linear, quantize

FLAG_BYTES = 4096
ONE_SHOT_ROWS = 64             # at most this many rows are reduced by every rank itself (one flag exchange) ...
ONE_SHOT_PULL_BYTES = 8 << 20  # ... and only while a rank then pulls no more than this from its peers: beyond it the
                               # rows are split over the ranks (reduce-scatter, norm, all-gather), which moves
                               # 2/size of the bytes at the price of a second flag exchange and a second launch.
                               # Measured on 8 GPUs at 64 rows x 8192 (7 MB pulled per rank): one-shot 23.6 us per
                               # reduce and the fastest whole step; split 22.8 us (in-switch sums) / 23.9 us (peer
                               # loads) per reduce but a slower step
CAND_MAX_K = 64                # sampling candidates exchanged per row and shard at most (beyond: whole shards)
PUSH_MIN_RANKS = 4             # decode-sized batches on this many ranks or more: the row-parallel GEMM's epilogue
                               # pushes its partial rows into every rank's receive slot (posted NVLink stores that
                               # overlap with the tiles still being computed) and the reduce kernel reads local
                               # memory only; below, every rank pulls the partial rows from its peers instead
PUSH_EPILOGUE = False          # large batches: reduce-scatter by GEMM-epilogue pushes (64 contiguous bytes per row
                               # and store) instead of owner pulls; KSANA_PUSH_PREFILL=0 / 1 overrides


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class SymmetricComm:
    @staticmethod
    def layout(size: int, max_tokens: int, hidden: int) -> dict:
        """Byte offsets of the regions of the symmetric buffer (identical on every rank) for a group of ``size`` ranks:
        pure arithmetic, no device involved."""
        rows_rs = (max_tokens + size - 1) // size
        slot_rows = max(rows_rs, ONE_SHOT_ROWS)
        slot_bytes = _align(slot_rows * hidden * 2)
        off = FLAG_BYTES
        slots_off = [off, off + size * slot_bytes]
        off += 2 * size * slot_bytes
        h_off = off; off += _align(max_tokens * hidden * 2)
        y_off = off; off += _align(max_tokens * hidden * 2)
        yq_off = off; off += _align(max_tokens * hidden)
        scale_ld = _align(max_tokens, 4)
        ys_off = off; off += _align((hidden // 128 + 1) * scale_ld * 4)
        stage_off = off
        stage_bytes = _align(max_tokens * hidden * 2)
        off += stage_bytes
        # sampling candidates of the vocabulary shards (values and token ids, fp32 / int32 words): a region of its
        # own, so that nothing else ever writes it between a step's exchange and the next step's
        cand_off = off
        cand_words = 2 * min(max_tokens, 1024) * CAND_MAX_K
        off += _align(cand_words * 4)
        return dict(slot_rows=slot_rows, slot_bytes=slot_bytes, slots_off=slots_off, h_off=h_off, y_off=y_off, yq_off=yq_off,
                    scale_ld=scale_ld, ys_off=ys_off, stage_off=stage_off, stage_bytes=stage_bytes, cand_off=cand_off,
                    cand_words=cand_words, total=off)

    def __init__(self, group, rank: int, size: int, device, max_tokens: int = 16384, hidden: int = 8192):
        import torch.distributed._symmetric_memory as symm_mem
        self.group, self.rank, self.size, self.device = group, rank, size, torch.device(device)
        self.max_tokens, self.hidden = max_tokens, hidden
        lay = self.layout(size, max_tokens, hidden)
        self.slot_rows, self.slot_bytes, self.slots_off = lay["slot_rows"], lay["slot_bytes"], lay["slots_off"]
        self.h_off, self.y_off, self.yq_off, self.ys_off = lay["h_off"], lay["y_off"], lay["yq_off"], lay["ys_off"]
        self.scale_ld, self.stage_off, self.stage_bytes = lay["scale_ld"], lay["stage_off"], lay["stage_bytes"]
        self.cand_off, self.cand_words, self.total = lay["cand_off"], lay["cand_words"], lay["total"]
        self.buf = symm_mem.empty(self.total, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.data_ptrs = (C.c_ulonglong * 8)(*(ptrs + [0] * (8 - size)))
        self.flag_ptrs = (C.c_ulonglong * 8)(*(ptrs + [0] * (8 - size)))       # flags live at offset 0
        # NVLS: multicast address of the buffer when the platform bound one (in-switch reductions); opt-in
        self.mc_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        # in-switch reduction / replication pays from four ranks on (with two there is nothing to save); KSANA_NVLS=0 / 1
        # overrides
        self.ctrs = torch.zeros(16, dtype=torch.int32, device=self.device)
        # address of this rank's "partial rows delivered" flag (kind 0) in every rank's flag pad
        self.sig_flag_ptrs = (C.c_ulonglong * 8)(*[(ptrs[r] + 4 * rank if r < size else 0) for r in range(8)])
        self.parity = 0
        dist.barrier(group)
        # local views
        self.h = self._view(self.h_off, (max_tokens, hidden), torch.bfloat16)
        self.y = self._view(self.y_off, (max_tokens, hidden), torch.bfloat16)
        self.yq = self._view(self.yq_off, (max_tokens, hidden), torch.float8_e4m3fn)
        self.ys = self._view(self.ys_off, (hidden // 128 + 1, self.scale_ld), torch.float32)
        self.stage = self._view(self.stage_off, (self.stage_bytes // 2,), torch.bfloat16)

    # The switches below are read from the environment at every call (a dictionary lookup), so that one process can
    # time several settings; all ranks must hold the same values.
    @property
    def use_nvls(self) -> bool:
        want = os.environ.get("KSANA_NVLS")
        return bool(self.mc_ptr) and (want == "1" or (want is None and self.size >= 4))

    @property
    def push_signal(self) -> bool:
        return os.environ.get("KSANA_PUSH_SIGNAL", "0") == "1"

    @property
    def push_decode(self) -> bool:
        """Decode-sized batches: whether the row-parallel GEMM's epilogue pushes its rows to every rank (default from
        ``PUSH_MIN_RANKS`` ranks on) instead of every rank pulling them; ``KSANA_PUSH=0 / 1`` overrides."""
        want = os.environ.get("KSANA_PUSH")
        return self.size >= PUSH_MIN_RANKS if want is None else want == "1"

    @property
    def push_prefill(self) -> bool:
        want = os.environ.get("KSANA_PUSH_PREFILL")
        return PUSH_EPILOGUE if want is None else want == "1"

    def one_shot(self, M: int) -> bool:
        """Whether a row-parallel result of M rows is reduced by every rank itself (all rows pulled from every peer)
        instead of reduce-scatter + all-gather."""
        forced = os.environ.get("KSANA_ONE_SHOT_ROWS")
        if forced is not None:
            return M <= int(forced)
        return M <= ONE_SHOT_ROWS and M * (self.size - 1) * self.hidden * 2 <= ONE_SHOT_PULL_BYTES

    def _view(self, off: int, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty(0, dtype=dtype).element_size()
        return self.buf[off:off + n * esz].view(dtype).view(*shape)

    def fits(self, x: torch.Tensor) -> bool:
        return x.is_cuda and x.dtype == torch.bfloat16 and x.numel() * 2 <= self.stage_bytes and x.numel() % 8 == 0

    # ------------------------------------------------------------------ plain collectives
    def barrier(self):
        rc = native.lib().ksana_comm_barrier(self.data_ptrs, self.flag_ptrs, self.rank, self.size, self.ctrs.data_ptr(),
                                             native.err_flag(self.device).data_ptr(), native._st())
        native._check(rc, "ksana_comm_barrier")

    def all_reduce(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, nvls: Optional[bool] = None) -> torch.Tensor:
        """x (bf16, contiguous) summed over ranks (+ residual): one-shot pull over peer memory, or - ``nvls`` /
        KSANA_NVLS=1 and a multicast binding of the buffer - one in-switch reduction per 16 bytes
        (multimem.ld_reduce)."""
        n = x.numel()
        self.stage[:n].copy_(x.reshape(-1))
        out = torch.empty_like(x)
        if nvls if nvls is not None else self.use_nvls:
            rc = native.lib().ksana_allreduce_nvls(self.data_ptrs, self.flag_ptrs, self.rank, self.size,
                                                   self.ctrs.data_ptr(), self.mc_ptr, self.stage_off, out.data_ptr(),
                                                   residual.data_ptr() if residual is not None else None, n,
                                                   native.err_flag(self.device).data_ptr(), native._st())
            native._check(rc, "ksana_allreduce_nvls")
            self.barrier()
            return out
        rc = native.lib().ksana_allreduce_pull(self.data_ptrs, self.flag_ptrs, self.rank, self.size,
                                               self.ctrs.data_ptr(), self.stage_off, out.data_ptr(),
                                               residual.data_ptr() if residual is not None else None, n,
                                               native.err_flag(self.device).data_ptr(), native._st())
        native._check(rc, "ksana_allreduce_pull")
        # the staging area is reused by the next call: peers must be done reading it
        self.barrier()
        return out

    def all_gather_cols(self, x: torch.Tensor, valid: int) -> Optional[torch.Tensor]:
        """[rows, n] fp32 shards -> [rows, size * valid] by pulling the peers' staged shards. None if it does not fit."""
        rows, n = x.shape
        if x.dtype != torch.float32 or rows * n * 4 > self.stage_bytes:
            return None
        stage = self.stage.view(torch.float32)[: rows * n].view(rows, n)
        stage.copy_(x)
        out = torch.empty(rows, self.size * valid, dtype=torch.float32, device=self.device)
        rc = native.lib().ksana_allgather_pull(self.data_ptrs, self.flag_ptrs, self.rank, self.size,
                                               self.ctrs.data_ptr(), self.stage_off, out.data_ptr(), rows, valid, n,
                                               self.size * valid, native.err_flag(self.device).data_ptr(), native._st())
        native._check(rc, "ksana_allgather_pull")
        self.barrier()          # peers are done reading the stage before it is written again
        return out

    def candidate_stage(self, B: int, k: int):
        """Where this rank writes its shard's sampling candidates: (values fp32 [B, k], token ids int32 [B, k]),
        views of the symmetric buffer. None if B x k does not fit the region."""
        if 2 * B * k > self.cand_words or k > CAND_MAX_K:
            return None
        words = self.buf[self.cand_off: self.cand_off + 2 * B * k * 4]
        return words[: B * k * 4].view(torch.float32).view(B, k), words[B * k * 4:].view(torch.int32).view(B, k)

    def gather_candidates(self, B: int, k: int):
        """Collective: every rank's staged candidates -> (values [B, size * k], token ids [B, size * k]) on every rank,
        rank r's candidates in columns [r * k, (r + 1) * k). One pull kernel (its flag exchange makes the peers'
        staged rows visible); the region is written once per forward pass, and the flag exchanges of the next pass's
        layers lie between two uses, so no trailing barrier is needed."""
        out = torch.empty(2 * B, self.size * k, dtype=torch.float32, device=self.device)
        rc = native.lib().ksana_allgather_pull(self.data_ptrs, self.flag_ptrs, self.rank, self.size,
                                               self.ctrs.data_ptr(), self.cand_off, out.data_ptr(), 2 * B, k, k,
                                               self.size * k, native.err_flag(self.device).data_ptr(), native._st())
        native._check(rc, "ksana_allgather_pull")
        return out[:B], out[B:].view(torch.int32)

    def all_gather_rows(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """[rows, H] bf16 (the same ``rows`` on every rank) -> [size * rows, H]: rank r's rows at r * rows, pulled
        from the peers' staging areas (raw 32-bit copies). None if it does not fit the staging area."""
        rows, H = x.shape
        if x.dtype != torch.bfloat16 or H % 2 or rows * H * 2 > self.stage_bytes or rows == 0:
            return None
        n = rows * H // 2                                    # 32-bit words per rank
        self.stage[: rows * H].copy_(x.reshape(-1))
        out = torch.empty(self.size * rows, H, dtype=torch.bfloat16, device=self.device)
        rc = native.lib().ksana_allgather_pull(self.data_ptrs, self.flag_ptrs, self.rank, self.size,
                                               self.ctrs.data_ptr(), self.stage_off, out.data_ptr(), 1, n, n,
                                               self.size * n, native.err_flag(self.device).data_ptr(), native._st())
        native._check(rc, "ksana_allgather_pull")
        self.barrier()          # peers are done reading the stage before it is written again
        return out

    def reduce_rows_into(self, write_partial, M: int, row_begin: int, h_rows: torch.Tensor) -> bool:
        """Reduce-scatter with the residual add fused: every rank fills its partial result for all ``M`` rows
        (``write_partial(part)``, part = [M, hidden] view of its peer-visible slot); this rank then pulls rows
        ``[row_begin, row_begin + len(h_rows))`` from every peer, sums them in rank order and adds them to ``h_rows``
        in place. False if M does not fit the slots."""
        H = self.hidden
        if M * H * 2 > self.size * self.slot_bytes or h_rows.dtype != torch.bfloat16:
            return False
        parity = self.parity
        self.parity ^= 1
        part = self.buf[self.slots_off[parity]: self.slots_off[parity] + M * H * 2].view(torch.bfloat16).view(M, H)
        write_partial(part)
        n = int(h_rows.shape[0])
        # the kernel addresses the residual by global row: bias the pointer so that row_begin lands on h_rows[0]
        h_base = h_rows.data_ptr() - row_begin * H * 2 if n else 0
        rc = native.lib().ksana_reduce_norm(self.data_ptrs, self.flag_ptrs, self.rank, self.size, self.ctrs.data_ptr(),
                                            self.slots_off[parity], self.slot_bytes, row_begin, n, M, H, h_base or None,
                                            None, None, 0.0, 0, None, None, None, 0, 4, self.h_off, self.y_off,
                                            self.yq_off, self.ys_off, self.mc_ptr if self.use_nvls else 0,
                                            native.err_flag(self.device).data_ptr(), native._st())
        native._check(rc, "ksana_reduce_norm")
        return True

    # ------------------------------------------------------------------ fused row-parallel linear
    def begin_forward(self):
        self.parity = 0

    def _push_ptrs(self, parity: int):
        base = self.slots_off[parity] + self.rank * self.slot_bytes
        return (C.c_ulonglong * 8)(*[int(self.handle.buffer_ptrs[r]) + base if r < self.size else 0 for r in range(8)])

    def row_parallel_norm(self, x, W: LinearWeight, h: torch.Tensor, norm_w, norm_b=None, eps: float = 1e-6,
                          layernorm: bool = False, quant_for: Optional[LinearWeight] = None, want_y: bool = True,
                          gather_h: bool = False):
        """h += sum_ranks(x W^T); y = norm(h) in the form the next linear wants. Returns (h, y).

        ``h`` must be the symmetric residual view (``self.h[:M]``) when M > ONE_SHOT_ROWS; there every rank
        keeps only the rows it owns up to date unless ``gather_h`` asks for the full residual stream."""
        M = x.q.shape[0] if isinstance(x, QTensor) else x.shape[0]
        return self._partial_norm(x, W, M, W.out_features, h, norm_w, norm_b, eps, layernorm, quant_for, gather_h)

    def partial_norm(self, write_partial, M: int, h: torch.Tensor, norm_w, norm_b=None, eps: float = 1e-6,
                     layernorm: bool = False, quant_for: Optional[LinearWeight] = None, gather_h: bool = False):
        """h += sum_ranks(partial); y = norm(h). ``write_partial(part)`` fills this rank's partial result
        ``part`` ([M, hidden] bf16, a view of the symmetric slot) - e.g. the top-k weighted combine of the experts
        this rank owns - and the same reduce kernel as for row-parallel GEMMs pulls, sums, adds the residual and
        normalises. Returns (h, y)."""
        return self._partial_norm(write_partial, None, M, self.hidden, h, norm_w, norm_b, eps, layernorm, quant_for,
                                  gather_h)

    def _partial_norm(self, x, W, M, H, h, norm_w, norm_b, eps, layernorm, quant_for, gather_h):
        writer = x if W is None else None
        parity = self.parity
        self.parity ^= 1
        push = self._push_ptrs(parity)
        err = native.err_flag(self.device).data_ptr()
        st = native._st()
        lib = native.lib()
        if writer is None and W.fp8 and not isinstance(x, QTensor):
            x = quantize(x)
        one_shot = self.one_shot(M)
        gemm_signals = False
        plain_w = writer is None and not W.nvfp4 and not W.w4a16
        push_mode = plain_w and (self.push_decode if one_shot else self.push_prefill)
        rows_per = M if one_shot else (M + self.size - 1) // self.size
        bias = W.bias.data_ptr() if (writer is None and W.bias is not None and self.rank == 0) else None
        if writer is not None:
            part = self.buf[self.slots_off[parity]: self.slots_off[parity] + M * H * 2].view(torch.bfloat16).view(M, H)
            writer(part)
        elif not push_mode:
            # partial product [M, H] into this rank's own symmetric buffer (the slot area of this parity); the
            # reduce kernel of every row owner (one-shot: of every rank) pulls it from there
            part = self.buf[self.slots_off[parity]: self.slots_off[parity] + M * H * 2].view(torch.bfloat16).view(M, H)
            linear(x, W if self.rank == 0 else W.without_bias(), out=part)
        elif one_shot and W.fp8 and W.ue8m0 and M >= native.MX_MIN_M and not native._skinny_wins_mx(M, H, W.in_features):
            # the tiled kernel is the faster GEMM for this shape: its epilogue broadcasts the rows (push_rows = 0)
            native.gemm_mxfp8(x.q, x.s, W.wq, W.ws, bias=W.bias if self.rank == 0 else None, push=push,
                              push_n=self.size, push_rows=0, ldd=H)
            rc = 0
        elif one_shot:
            scratch, counters = native.gemm_workspace(self.device)
            gemm_signals = self.push_signal
            if W.fp8:
                head = (2 if W.ue8m0 else 1, x.q.data_ptr(), x.q.stride(0), x.s.data_ptr(), x.s.stride(0), W.wq.data_ptr(),
                        W.wq.stride(0), W.ws.data_ptr())
            else:
                head = (0, x.data_ptr(), x.stride(0), None, 0, W.w.data_ptr(), W.w.stride(0), None)
            tail = (H, bias, M, H, W.in_features, scratch.data_ptr(), scratch.numel() * 4, counters.data_ptr(),
                    counters.numel(), push, self.size)
            if gemm_signals:
                # the GEMM's last CTA raises this rank's flag at the peers once its pushes are out: the reduce kernel
                # below then only waits (gather bit 4)
                rc = lib.ksana_gemm_smallm_push_signal(*head, *tail, self.sig_flag_ptrs, self.ctrs.data_ptr(),
                                                       self.ctrs[12:13].data_ptr(), err, st)
            else:
                rc = lib.ksana_gemm_smallm_push(*head, *tail, err, st)
            native._check(rc, "ksana_gemm_smallm_push")
        else:
            if W.fp8 and W.ue8m0 and M >= native.MX_MIN_M:
                tall = (native.MX_TALL_MIN_M > 0 and M >= native.MX_TALL_MIN_M and
                        native._tall_wins(M, H, W.in_features))
                (native.gemm_mxfp8_tall if tall else native.gemm_mxfp8)(
                    x.q, x.s, W.wq, W.ws, bias=W.bias if self.rank == 0 else None, push=push, push_n=self.size,
                    push_rows=rows_per, ldd=H)
                rc = 0
            elif W.fp8:
                rc = lib.ksana_gemm_fp8_block_push(x.q.data_ptr(), x.q.stride(0), x.s.data_ptr(), x.s.stride(0),
                                                   W.wq.data_ptr(), W.wq.stride(0), W.ws.data_ptr(), H, bias, M, H,
                                                   W.in_features, 0, push, self.size, rows_per, err, st)
            else:
                rc = lib.ksana_gemm_bf16_push(x.data_ptr(), x.stride(0), W.w.data_ptr(), W.w.stride(0), H, bias, M, H,
                                              W.in_features, 0, push, self.size, rows_per, err, st)
            native._check(rc, "ksana_gemm_push")
        want_q = quant_for is not None and quant_for.fp8 and H % 128 == 0 and norm_w is not None
        if one_shot:
            row_begin, row_count, gather = 0, M, (4 if (writer is not None or not push_mode) else 0)
            if push_mode and writer is None and self.push_signal and gemm_signals:
                gather |= 16
            y = torch.empty(M, H, dtype=torch.bfloat16, device=self.device) if (norm_w is not None and not want_q) else None
            yq = torch.empty(M, H, dtype=torch.float8_e4m3fn, device=self.device) if want_q else None
            scale_ld = (M + 3) // 4 * 4
            ys = torch.empty(H // 128, scale_ld, dtype=torch.float32, device=self.device) if want_q else None
        else:
            row_begin = min(self.rank * rows_per, M)
            row_count = max(0, min(rows_per, M - row_begin))
            gather = 1 | (2 if gather_h else 0) | (4 if (writer is not None or not push_mode) else 0)
            assert h.data_ptr() == self.h.data_ptr(), "large-batch row-parallel linear needs the symmetric residual view"
            y = self.y[:M] if (norm_w is not None and not want_q) else None
            yq = self.yq[:M] if want_q else None
            ys = self.ys if want_q else None
            scale_ld = self.scale_ld
        rc = lib.ksana_reduce_norm(self.data_ptrs, self.flag_ptrs, self.rank, self.size, self.ctrs.data_ptr(),
                                   self.slots_off[parity], self.slot_bytes, row_begin, row_count, M, H, h.data_ptr(),
                                   norm_w.data_ptr() if norm_w is not None else None,
                                   norm_b.data_ptr() if norm_b is not None else None, float(eps), int(layernorm),
                                   y.data_ptr() if y is not None else None, yq.data_ptr() if yq is not None else None,
                                   ys.data_ptr() if ys is not None else None, scale_ld, gather, self.h_off, self.y_off,
                                   self.yq_off, self.ys_off, self.mc_ptr if self.use_nvls else 0, err, st)
        native._check(rc, "ksana_reduce_norm")
        if norm_w is None:
            return h, None
        return h, (QTensor(yq, ys) if want_q else y)
