"""ctypes bindings to ``libksana_kernels.so`` (the hand-written sm_100a kernels).

Every wrapper takes torch CUDA tensors, passes raw pointers plus the current CUDA stream and
raises if the native library is missing or a launch is rejected, so a GPU box can never fall
back silently to PyTorch ops.
"""
from __future__ import annotations

import ctypes as C
import math
from pathlib import Path
from typing import Optional

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libksana_kernels.so"

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float

_SIGS = {
    "ksana_gemm_bf16": [vp, i32, vp, i32, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp],
    "ksana_gemm_pair": [i32, vp, i32, vp, i32, vp, i32, vp, vp, i32, vp, vp, i32, i32, i32, i32, vp, i32, i32, vp, vp],
    "ksana_gemm_nvfp4": [vp, i32, vp, i32, vp, vp, i32, vp, i32, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp],
    "ksana_gemm_bf16_batched": [vp, i64, i64, vp, i64, i64, vp, i64, i64, i32, i32, i32, i32, vp, vp],
    "ksana_gemm_grouped_nvfp4": [vp, i32, vp, i32, vp, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, vp, i32, vp, vp],
    "ksana_quant_nvfp4": [vp, i32, vp, i32, vp, i32, vp, i32, i32, vp],
    "ksana_gemm_mxfp8": [vp, i32, vp, i32, vp, i32, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, vp, i32, i32, vp,
                         vp],
    "ksana_gemm_bf16_tall": [vp, i32, vp, i32, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, vp, vp],
    "ksana_gemm_mxfp8_tall": [vp, i32, vp, i32, vp, i32, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, vp, i32, i32, vp,
                              vp],
    "ksana_gemm_mxfp8_pair": [vp, i32, vp, i32, vp, i32, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, vp, i32, i32, vp, vp],
    "ksana_gemm_fp8_block": [vp, i32, vp, i32, vp, i32, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp],
    "ksana_gemm_smallm": [i32, vp, i32, vp, i32, vp, i32, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, vp, i64, vp, i32,
                          vp, vp],
    "ksana_gemm_grouped": [i32, vp, i32, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, vp, i32, vp, vp],
    "ksana_moe_route": [vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, i32, vp],
    "ksana_moe_align": [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp],
    "ksana_moe_permute": [vp, vp, vp, i32, i32, i32, i32, vp, vp],
    "ksana_moe_combine": [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp],
    "ksana_gemm_smallm_push": [i32, vp, i32, vp, i32, vp, i32, vp, i32, vp, i32, i32, i32, vp, i64, vp, i32, vp, i32, vp, vp],
    "ksana_gemm_smallm_push_signal": [i32, vp, i32, vp, i32, vp, i32, vp, i32, vp, i32, i32, i32, vp, i64, vp, i32, vp, i32,
                                      vp, vp, vp, vp, vp],
    "ksana_gemm_fp8_block_push": [vp, i32, vp, i32, vp, i32, vp, i32, vp, i32, i32, i32, i32, vp, i32, i32, vp, vp],
    "ksana_gemm_bf16_push": [vp, i32, vp, i32, i32, vp, i32, i32, i32, i32, vp, i32, i32, vp, vp],
    "ksana_reduce_norm": [vp, vp, i32, i32, vp, i64, i64, i32, i32, i32, i32, vp, vp, vp, f32, i32, vp, vp, vp, i32, i32,
                          i64, i64, i64, i64, C.c_ulonglong, vp, vp],
    "ksana_comm_barrier": [vp, vp, i32, i32, vp, vp, vp],
    "ksana_allreduce_pull": [vp, vp, i32, i32, vp, i64, vp, vp, i64, vp, vp],
    "ksana_allreduce_nvls": [vp, vp, i32, i32, vp, C.c_ulonglong, i64, vp, vp, i64, vp, vp],
    "ksana_allgather_pull": [vp, vp, i32, i32, vp, i64, vp, i32, i32, i32, i32, vp, vp],
    "ksana_norm": [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, i32, vp],
    "ksana_act_mul": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp],
    "ksana_quant_fp8": [vp, vp, vp, i32, i32, i32, i32, vp],
    "ksana_embedding": [vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, vp],
    "ksana_gather_rows": [vp, vp, vp, i32, i32, i32, vp, vp],
    "ksana_refit_rows": [vp, vp, vp, i32, i32, vp],
    "ksana_rope_kv_append": [vp, vp, i32, vp, vp, vp, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, f32, f32,
                             i32, vp],
    "ksana_copy_blocks": [vp, vp, i32, i64, i32, vp, vp],
    "ksana_swap_blocks": [vp, vp, vp, i32, i64, i32, i32, i32, vp, vp],
    "ksana_add": [vp, vp, vp, vp, i64, i32, vp],
    "ksana_patch_ids": [vp, vp, vp, vp, i32, i32, i32, vp, vp],
    "ksana_smallm_estimate": [i32, i32, i32, i32, vp],
    "ksana_absmax_scale": [vp, i32, i32, i64, f32, f32, vp, vp, vp],
    "ksana_rerotate_blocks": [vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp],
    "ksana_cast_f32": [vp, vp, i64, vp],
    "ksana_paged_prefill_tc": [vp, i64, i64, vp, i64, vp, i64, i32, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, f32, i64,
                               vp, vp],
    "ksana_paged_prefill": [vp, i64, vp, i64, vp, i64, i32, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32,
                            f32, f32, i64, vp, vp],
    "ksana_paged_decode": [vp, i64, vp, i64, vp, i64, i32, vp, i32, vp, vp, i32, i32, i32, i32, f32, i32, f32, f32,
                           i32, vp, vp, i64, vp, vp, i32, vp, vp],
    "ksana_mla_attention": [vp, i64, vp, i64, vp, i64, i32, vp, i32, vp, vp, i32, i32, i32, f32, i64, i32, vp, vp, vp, vp],
    "ksana_mla_rope_append": [vp, i64, i32, vp, i64, vp, f32, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, i64, vp, vp],
    "ksana_gemm_smallm_w4": [vp, i32, vp, vp, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, vp, i64, vp, i32, vp, vp],
    "ksana_w4_gemv": [vp, i64, vp, vp, vp, vp, vp, i64, vp, i64, i32, i32, i32, i32, vp],
    "ksana_w4_dequant": [vp, vp, vp, vp, i64, i32, i32, i32, vp],
    "ksana_sample": [vp, i64, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp, i32, i32, vp],
    "ksana_sample_merged": [vp, i64, vp, i64, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp, i32, i32, vp],
    "ksana_shard_topk": [vp, i64, vp, i32, i32, i32, i32, vp, vp, vp],
    "ksana_repetition_penalty": [vp, i64, vp, vp, vp, vp, i32, i32, vp],
    "ksana_ban_tokens": [vp, i64, vp, vp, vp, i32, i32, vp],
}

_launches = 0


def launch_count() -> int:
    """Number of native kernel launches issued through this module (bench accounting)."""
    return _launches


def available() -> bool:
    return _LIB_PATH.exists()


_recorder = None


class _RecordingLib:
    """Stand-in for the library handle while a launch recorder is installed: every entry point called through it
    is appended to the recorder as (name, function, arguments) before it runs."""

    def __init__(self, real, rec):
        self._real, self._rec = real, rec

    def __getattr__(self, name):
        fn = getattr(self._real, name)
        rec = self._rec

        def call(*args):
            rec.append((name, fn, args))
            return fn(*args)
        return call


class recording:
    """Context manager: collects every native launch issued inside it into ``calls`` (used by the step breakdown
    in benchmarks/step_breakdown.py, which replays subsets of a step's launches in graphs of their own)."""

    def __init__(self, calls: list):
        self.calls = calls

    def __enter__(self):
        global _recorder
        _recorder = self.calls
        return self.calls

    def __exit__(self, *exc):
        global _recorder
        _recorder = None
        return False


def lib():
    if _recorder is not None:
        return _RecordingLib(_load(), _recorder)
    return _load()


def _load():
    global _LIB
    if _LIB is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"native kernel library {_LIB_PATH} is missing: run `python -m ksanallm_b200.build` "
                "(CUDA tensors are never served by a PyTorch fallback)")
        _LIB = C.CDLL(str(_LIB_PATH))
        for name, sig in _SIGS.items():
            fn = getattr(_LIB, name, None)
            if fn is not None:
                fn.argtypes = sig
                fn.restype = C.c_int
    return _LIB


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _st():
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, name: str):
    global _launches
    _launches += 1
    if rc != 0:
        raise RuntimeError(f"{name} rejected its arguments or failed to launch (code {rc})")


_err_flags = {}


def err_flag(device) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits set when a wait gave up."""
    d = torch.device(device)
    key = (d.type, d.index or 0)
    if key not in _err_flags:
        _err_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _err_flags[key]


def describe_err_code(code: int) -> str:
    if code >= 1000000:
        names = {11: "block-table entry", 12: "sequence row range", 13: "position", 14: "cache slot", 15: "expert id",
                 16: "expert destination row", 17: "gather row index"}
        return (f"a kernel skipped an out-of-range {names.get(code // 1000000, 'index')} "
                f"(value mod 1e6 = {code % 1000000}); the step's results are invalid")
    what = {2: "a tensor-core GEMM gave up waiting for its operands", 3: "a wait for a peer GPU's flag ran out",
            4: "an attention kernel gave up waiting for its K/V tiles"}.get(code, "a device-side bounded wait timed out")
    return f"{what} (kernel reported error status {code})"


def clear_err_flag(device) -> None:
    with torch.inference_mode():              # the word may have been created inside the engine's inference mode
        err_flag(device).zero_()


def check_err_flag(device) -> None:
    """Reads the device error word (synchronises the stream); raises and clears it when a kernel reported."""
    code = int(err_flag(device).item())
    if code != 0:
        clear_err_flag(device)
        raise RuntimeError(describe_err_code(code))


# ------------------------------------------------------------------------------------- GEMM
import os as _os

SMALL_M_FP8 = int(_os.environ.get("KSANA_SKINNY_MAX_M", "32"))   # FP8: rows up to which the skinny stream-K kernel always runs
SMALL_M_BF16 = 128                 # bf16: no per-K-block promotion, the skinny kernel wins up to a full token tile
_SCRATCH_BYTES = 64 << 20
_COUNTERS = 4096
_workspaces = {}


def gemm_workspace(device):
    """Per-device scratch for tiles whose K range is cut across CTAs (fp32 partial tiles) and the tile
    arrival counters (zeroed once; the kernel leaves them zero). Launches that share it must be
    ordered on one stream. ``splits`` of the GEMM wrappers: 0 = automatic, > 0 = number of persistent
    CTAs, < 0 = force the skinny kernel for M up to 128."""
    key = torch.device(device).index or 0
    if key not in _workspaces:
        _workspaces[key] = (torch.empty(_SCRATCH_BYTES // 4, dtype=torch.float32, device=device),
                            torch.zeros(_COUNTERS, dtype=torch.int32, device=device))
    return _workspaces[key]


def _gemm_smallm(kind, x, xs, w, ws, out, out_f32, bias, residual, M, N, K, splits):
    dst = out if out_f32 is None else out_f32
    scratch, counters = gemm_workspace(x.device)
    rc = lib().ksana_gemm_smallm(kind, _p(x), x.stride(0), _p(xs), xs.stride(0) if xs is not None else 0, _p(w),
                                 w.stride(0), _p(ws), _p(out) if out_f32 is None else None, _p(out_f32), dst.stride(0),
                                 _p(bias), _p(residual), residual.stride(0) if residual is not None else 0, M, N, K,
                                 max(splits, 0), _p(scratch), scratch.numel() * 4, _p(counters), counters.numel(),
                                 _p(err_flag(x.device)), _st())
    _check(rc, "ksana_gemm_smallm")
    return dst


PAIR_MIN_M = 0                     # CTA-pair (cta_group::2) kernel from this many rows; 0 disables it


def gemm_pair(kind, x, xs, w, ws, out, bias=None, residual=None, push=None, push_n=0, push_rows=0):
    """CTA-pair tcgen05 GEMM (256 x 256 tiles over two SMs). kind 0: bf16, 1: block-scaled FP8. bf16 output only."""
    M, K = x.shape
    N = w.shape[0]
    rc = lib().ksana_gemm_pair(kind, _p(x), x.stride(0), _p(xs), xs.stride(0) if xs is not None else 0, _p(w),
                               w.stride(0), _p(ws), _p(out), out.stride(0) if out is not None else N, _p(bias),
                               _p(residual), residual.stride(0) if residual is not None else 0, M, N, K, push, push_n,
                               push_rows, _p(err_flag(x.device)), _st())
    _check(rc, "ksana_gemm_pair")
    return out


BF16_TALL_MIN_M = 0                # 256 x 256-tile bf16 kernel from this many rows; 0 disables it


def gemm_bf16_tall(x, w, out=None, bias=None, residual=None, out_f32=None, max_ctas=0):
    """bf16 GEMM with 256 x 256 tiles per CTA (two 128-row MMAs share every weight tile)."""
    M, K = x.shape
    N = w.shape[0]
    dst = out if out_f32 is None else out_f32
    rc = lib().ksana_gemm_bf16_tall(_p(x), x.stride(0), _p(w), w.stride(0), _p(out) if out_f32 is None else None,
                                    _p(out_f32), dst.stride(0), _p(bias), _p(residual),
                                    residual.stride(0) if residual is not None else 0, M, N, K, max_ctas,
                                    _p(err_flag(x.device)), _st())
    _check(rc, "ksana_gemm_bf16_tall")
    return dst


def _pair_ok(M, N, K, kind, bn, out_f32, max_ctas):
    return (PAIR_MIN_M > 0 and M >= PAIR_MIN_M and bn == 0 and max_ctas == 0 and out_f32 is None and N % 8 == 0
            and N >= 256 and K % (128 if kind else 8) == 0)


def gemm_bf16(x, w, out=None, bias=None, residual=None, out_f32=None, bn=0, max_ctas=0, splits=0):
    """out[M,N] = x[M,K] @ w[N,K]^T (+bias)(+residual). bf16 in, bf16 (or fp32) out."""
    M, K = x.shape
    N = w.shape[0]
    assert x.stride(1) == 1 and w.stride(1) == 1 and w.shape[1] == K
    if out is None and out_f32 is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    dst = out if out_f32 is None else out_f32
    if (M <= SMALL_M_BF16 or splits < 0) and M <= 128 and bn == 0 and K % 8 == 0:
        return _gemm_smallm(0, x, None, w, None, out, out_f32, bias, residual, M, N, K, splits)
    if (BF16_TALL_MIN_M > 0 and M >= BF16_TALL_MIN_M and bn == 0 and splits == 0 and N % 8 == 0 and K % 8 == 0
            and ((M + 255) // 256) * ((N + 255) // 256) >= 148):
        return gemm_bf16_tall(x, w, out, bias, residual, out_f32, max_ctas)
    if _pair_ok(M, N, K, 0, bn, out_f32, max_ctas):
        return gemm_pair(0, x, None, w, None, out, bias, residual)
    rc = lib().ksana_gemm_bf16(_p(x), x.stride(0), _p(w), w.stride(0), _p(out) if out_f32 is None else None,
                               _p(out_f32), dst.stride(0), _p(bias), _p(residual),
                               residual.stride(0) if residual is not None else 0, M, N, K, bn, max_ctas,
                               _p(err_flag(x.device)), _st())
    _check(rc, "ksana_gemm_bf16")
    return dst


MX_MIN_M = 33                      # hardware-scaled kernel from this many rows (below: the skinny stream-K kernel)


def gemm_mxfp8(xq, xs, wq, ws, out=None, bias=None, residual=None, out_f32=None, bn=0, max_ctas=0, push=None,
               push_n=0, push_rows=0, ldd=None):
    """FP8 GEMM whose power-of-two scales are applied by the tensor cores (tcgen05 block_scale MMA)."""
    M, K = xq.shape
    N = wq.shape[0]
    dst = out if out_f32 is None else out_f32
    rc = lib().ksana_gemm_mxfp8(_p(xq), xq.stride(0), _p(xs), xs.stride(0), _p(wq), wq.stride(0), _p(ws),
                                _p(out) if out_f32 is None else None, _p(out_f32),
                                dst.stride(0) if dst is not None else ldd, _p(bias), _p(residual),
                                residual.stride(0) if residual is not None else 0, M, N, K, bn, max_ctas, push, push_n,
                                push_rows, _p(err_flag(xq.device)), _st())
    _check(rc, "ksana_gemm_mxfp8")
    return dst


MX_TALL_MIN_M = 512                # 256 x 224-tile hardware-scaled kernel from this many rows (measured faster); 0 disables it


def _tall_wins(M, N, K, max_ctas=0, sms=148):
    """256 x 224 tiles against 128 x 256 tiles for one problem, from measured behaviour: the tall tile does 1.75
    times the MMA work at about 1.18 times the rate but cannot overlap its accumulator drain (about three K
    blocks of time per tile), so it needs a long K and a tile count that fills its last wave."""
    if K < 4096:
        return False
    ctas = min(sms, max_ctas) if max_ctas > 0 else sms
    kb = K // 128
    t_tall = ((M + 255) // 256) * ((N + 223) // 224)
    t_std = ((M + 127) // 128) * ((N + 255) // 256)
    if t_tall < ctas:
        return False
    tall = -(-t_tall // ctas) * (1.75 * kb + 3.0) / 1.18
    std = -(-t_std // ctas) * (kb + 0.5)
    return tall < std


def gemm_mxfp8_tall(xq, xs, wq, ws, out=None, bias=None, residual=None, out_f32=None, max_ctas=0, push=None, push_n=0,
                    push_rows=0, ldd=None):
    """Hardware-scaled FP8 GEMM with 256 x 224 tiles per CTA (less operand traffic per MMA than 128 x 256)."""
    M, K = xq.shape
    N = wq.shape[0]
    dst = out if out_f32 is None else out_f32
    rc = lib().ksana_gemm_mxfp8_tall(_p(xq), xq.stride(0), _p(xs), xs.stride(0), _p(wq), wq.stride(0), _p(ws),
                                     _p(out) if out_f32 is None else None, _p(out_f32),
                                     dst.stride(0) if dst is not None else ldd, _p(bias), _p(residual),
                                     residual.stride(0) if residual is not None else 0, M, N, K, max_ctas, push, push_n,
                                     push_rows, _p(err_flag(xq.device)), _st())
    _check(rc, "ksana_gemm_mxfp8_tall")
    return dst


MX_PAIR_MIN_M = 0                  # CTA-pair hardware-scaled kernel from this many rows; 0 disables it


def gemm_mxfp8_pair(xq, xs, wq, ws, out=None, bias=None, residual=None, out_f32=None, push=None, push_n=0, push_rows=0,
                    ldd=None):
    """Hardware-scaled FP8 GEMM on CTA pairs (256 x 256 tiles over two SMs, tcgen05 cta_group::2 block_scale MMA)."""
    M, K = xq.shape
    N = wq.shape[0]
    dst = out if out_f32 is None else out_f32
    rc = lib().ksana_gemm_mxfp8_pair(_p(xq), xq.stride(0), _p(xs), xs.stride(0), _p(wq), wq.stride(0), _p(ws),
                                     _p(out) if out_f32 is None else None, _p(out_f32),
                                     dst.stride(0) if dst is not None else ldd, _p(bias), _p(residual),
                                     residual.stride(0) if residual is not None else 0, M, N, K, push, push_n,
                                     push_rows, _p(err_flag(xq.device)), _st())
    _check(rc, "ksana_gemm_mxfp8_pair")
    return dst


def _skinny_wins_mx(M, N, K, sms=148):
    """Rows 33..128 with tensor-core-applied scales: skinny stream-K kernel or tiled kernel, from their measured
    behaviour in CUDA graphs of decode steps (microseconds). Tiled: about 6.5 + 0.37 per 128-deep K block and wave of
    128 x 128 tiles (0.69 with 128 x 256 tiles); one CTA walks the whole K range of its tile, so few tiles leave
    SMs idle. Skinny: the (tile, K block) units are spread evenly over the SMs at about 0.62 per K block and CTA for 64
    rows (0.9 for 128), plus a higher fixed cost and the cross-CTA reduction of cut tiles."""
    kb = K // 128
    t128 = (N + 127) // 128
    t256 = (N + 255) // 256
    if t256 >= 100:
        tiled = 6.5 + -(-t256 // sms) * kb * 0.69
    else:
        tiled = 6.5 + -(-t128 // sms) * kb * 0.37
    units = t128 * kb
    ctas = min(sms, max(1, units // 4))
    per_cta = -(-units // ctas)
    pieces = -(-kb // max(1, per_cta)) + 1 if per_cta < kb else 1
    skinny = 11.5 + 0.15 * pieces + per_cta * (0.62 if M <= 64 else 0.9)
    return skinny < tiled


def gemm_fp8(xq, xs, wq, ws, out=None, bias=None, residual=None, out_f32=None, bn=0, max_ctas=0, splits=0,
             hw_scale=False):
    """Block-scaled FP8 GEMM. xq [M,K] e4m3, xs [K/128, ld] fp32; wq [N,K] e4m3, ws [ceil(N/128), K/128] fp32.
    hw_scale: every scale is a power of two, so the tensor cores may apply them (large-M path)."""
    M, K = xq.shape
    N = wq.shape[0]
    if out is None and out_f32 is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=xq.device)
    dst = out if out_f32 is None else out_f32
    if hw_scale:
        # power-of-two scales: both kernels let the tensor cores apply them. Skinny stream-K kernel for decode-sized
        # M and wherever the tiled kernel would leave most SMs idle; tiled kernel otherwise (256-wide tiles when
        # they fill the SMs).
        t256 = ((M + 127) // 128) * ((N + 255) // 256)
        skinny = M <= SMALL_M_FP8 or (M <= 128 and _skinny_wins_mx(M, N, K))
        if (skinny or splits != 0) and M <= 128 and bn == 0:
            return _gemm_smallm(2, xq, xs, wq, ws, out, out_f32, bias, residual, M, N, K, splits)
        if MX_TALL_MIN_M > 0 and M >= MX_TALL_MIN_M and bn == 0 and _tall_wins(M, N, K, max_ctas):
            return gemm_mxfp8_tall(xq, xs, wq, ws, out, bias, residual, out_f32, max_ctas)
        if MX_PAIR_MIN_M > 0 and M >= MX_PAIR_MIN_M and bn == 0 and max_ctas == 0 and t256 >= 148:
            return gemm_mxfp8_pair(xq, xs, wq, ws, out, bias, residual, out_f32)
        if bn == 0 or bn >= 128:
            return gemm_mxfp8(xq, xs, wq, ws, out, bias, residual, out_f32, bn or (256 if t256 >= 100 else 128),
                              max_ctas)
    skinny = M <= SMALL_M_FP8 or (M <= 64 and K >= 16384 and N <= 16384)
    if (skinny or splits < 0) and M <= 128 and bn == 0:
        return _gemm_smallm(1, xq, xs, wq, ws, out, out_f32, bias, residual, M, N, K, splits)
    if bn == 0 and M <= 128:
        bn = 128 if N >= 10240 else 64     # decode-sized rows on the tiled kernel: measured best tile widths
    rc = lib().ksana_gemm_fp8_block(_p(xq), xq.stride(0), _p(xs), xs.stride(0), _p(wq), wq.stride(0), _p(ws),
                                    _p(out) if out_f32 is None else None, _p(out_f32), dst.stride(0), _p(bias),
                                    _p(residual), residual.stride(0) if residual is not None else 0, M, N, K, bn,
                                    max_ctas, _p(err_flag(xq.device)), _st())
    _check(rc, "ksana_gemm_fp8_block")
    return dst


_absmax_acc = {}


def absmax_scale(x, divisor: float, floor: float = 1e-12):
    """max(|x|) / divisor (at least ``floor``) of a bf16 matrix as an fp32 scalar tensor on the device: the tensor
    scale of an NVFP4 activation, without a host round trip or a widened copy of ``x``."""
    rows, cols = x.shape
    key = (x.device.type, x.device.index)
    acc = _absmax_acc.get(key)
    if acc is None:
        acc = _absmax_acc[key] = torch.zeros(1, dtype=torch.int32, device=x.device)
    scale = torch.empty((), dtype=torch.float32, device=x.device)
    _check(lib().ksana_absmax_scale(_p(x), rows, cols, x.stride(0), float(divisor), float(floor), _p(acc), _p(scale),
                                    _st()), "ksana_absmax_scale")
    return scale


def quant_nvfp4(x, tensor_scale):
    """bf16 [M, K] -> (packed e2m1 [M, K/2] uint8, e4m3 block scales [M, K/16], tensor_scale). K % 16 == 0.
    ``tensor_scale``: fp32 scalar tensor on the device (calibrated or amax / (448 * 6))."""
    M, K = x.shape
    q = torch.empty(M, K // 2, dtype=torch.uint8, device=x.device)
    bs = torch.empty(M, K // 16, dtype=torch.float8_e4m3fn, device=x.device)
    _check(lib().ksana_quant_nvfp4(_p(x), x.stride(0), _p(q), q.stride(0), _p(bs), bs.stride(0), _p(tensor_scale), M, K,
                                   _st()), "ksana_quant_nvfp4")
    return q, bs, tensor_scale


def gemm_nvfp4(aq, a_bs, a_ts, wq, w_bs, w_ts, out=None, bias=None, residual=None, out_f32=None, bn=0, max_ctas=0):
    """NVFP4 x NVFP4 GEMM (e2m1 values, e4m3 scales per 16 elements, fp32 tensor scales) on the block-scaled tensor
    cores. aq [M, K/2], wq [N, K/2] packed bytes; K % 256 == 0."""
    M, N, K = aq.shape[0], wq.shape[0], aq.shape[1] * 2
    if out is None and out_f32 is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
    dst = out if out_f32 is None else out_f32
    rc = lib().ksana_gemm_nvfp4(_p(aq), aq.stride(0), _p(a_bs), a_bs.stride(0), _p(a_ts), _p(wq), wq.stride(0), _p(w_bs),
                                w_bs.stride(0), _p(w_ts), _p(out) if out_f32 is None else None, _p(out_f32),
                                dst.stride(0), _p(bias), _p(residual), residual.stride(0) if residual is not None else 0,
                                M, N, K, bn, max_ctas, _p(err_flag(aq.device)), _st())
    _check(rc, "ksana_gemm_nvfp4")
    return dst


def gemm_bf16_batched(a, w, out):
    """out[b] = a[b] @ w[b]^T for every b: a [B, M, K], w [B, N, K], out [B, M, N], bf16 views with unit stride in the
    last dimension and any (16-byte aligned) strides in the others, e.g. head-interleaved activations
    ``x.view(T, H, D).transpose(0, 1)``. One launch of the tcgen05 GEMM over all batch entries' tiles."""
    B, M, K = a.shape
    N = w.shape[1]
    assert w.shape[0] == B and w.shape[2] == K and tuple(out.shape) == (B, M, N)
    assert a.stride(2) == 1 and w.stride(2) == 1 and out.stride(2) == 1
    rc = lib().ksana_gemm_bf16_batched(_p(a), a.stride(1), a.stride(0), _p(w), w.stride(1), w.stride(0), _p(out),
                                       out.stride(1), out.stride(0), B, M, N, K, _p(err_flag(a.device)), _st())
    _check(rc, "ksana_gemm_bf16_batched")
    return out


def gemm_grouped_nvfp4(aq, a_bs, a_ts, wq, w_bs, w_ts, tile_expert, E, N, out=None, bn=0):
    """Expert-major NVFP4 rows ``aq`` [cap, K/2] (128-row tiles, one expert each, ``tile_expert`` < 0: unused) times
    the experts' stacked NVFP4 matrices ``wq`` [E * N, K/2] with block scales ``w_bs`` [E * N, K/16] and one tensor
    scale per expert ``w_ts`` [E]. Rows of unused tiles are left untouched."""
    cap, K = aq.shape[0], aq.shape[1] * 2
    if out is None:
        out = torch.zeros(cap, N, dtype=torch.bfloat16, device=aq.device)
    rc = lib().ksana_gemm_grouped_nvfp4(_p(aq), aq.stride(0), _p(a_bs), a_bs.stride(0), _p(a_ts), _p(wq), wq.stride(0),
                                        _p(w_bs), w_bs.stride(0), _p(w_ts), _p(out), out.stride(0), cap, N, K, E,
                                        _p(tile_expert), bn, _p(err_flag(aq.device)), _st())
    _check(rc, "ksana_gemm_grouped_nvfp4")
    return out


W4_TENSOR_CORE = True        # rows 3..128: expand-in-kernel + tcgen05 (the CUDA-core GEMV is compute bound beyond 2 rows)
W4_GEMV_MAX_M = 32          # up to this many rows the 4-bit weights are streamed by the GEMV kernel (8 rows per pass)
_w4_scratch = {}


def linear_w4(x, q4, scale, zs, out=None, bias=None, residual=None):
    """y = x W^T (+bias, +residual) for 4-bit group-quantised W (see csrc/kernels/w4a16.cu)."""
    M, K = x.shape
    N = q4.shape[0]
    g = K // scale.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    if W4_TENSOR_CORE and 2 < M <= 128 and g % 64 == 0 and K % 64 == 0:
        # weight stream on the tensor cores: four warps expand the packed tiles to bf16 in shared memory, the rest is
        # the stream-K skinny GEMM
        scratch, counters = gemm_workspace(x.device)
        rc = lib().ksana_gemm_smallm_w4(_p(x), x.stride(0), _p(q4), _p(scale), _p(zs), g, _p(out), out.stride(0), _p(bias),
                                        _p(residual), residual.stride(0) if residual is not None else 0, M, N, K,
                                        _p(scratch), scratch.numel() * 4, _p(counters), counters.numel(),
                                        _p(err_flag(x.device)), _st())
        _check(rc, "ksana_gemm_smallm_w4")
        return out
    if M <= W4_GEMV_MAX_M:
        rc = lib().ksana_w4_gemv(_p(x), x.stride(0), _p(q4), _p(scale), _p(zs), _p(bias), _p(residual),
                                 residual.stride(0) if residual is not None else 0, _p(out), out.stride(0), M, N, K, g, _st())
        _check(rc, "ksana_w4_gemv")
        return out
    # compute-bound: expand once into a per-device scratch matrix shared by all layers, then the tcgen05 bf16 GEMM
    key = (x.device.index or 0)
    buf = _w4_scratch.get(key)
    if buf is None or buf.numel() < N * K:
        buf = torch.empty(N * K, dtype=torch.bfloat16, device=x.device)
        _w4_scratch[key] = buf
    w = buf[: N * K].view(N, K)
    _check(lib().ksana_w4_dequant(_p(q4), _p(scale), _p(zs), _p(w), K, N, K, g, _st()), "ksana_w4_dequant")
    return gemm_bf16(x, w, out=out, bias=bias, residual=residual)


def quant_fp8(x, q=None, s=None):
    M, K = x.shape
    if q is None:
        q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    if s is None:
        s = torch.empty(K // 128, max(4, (M + 3) // 4 * 4), dtype=torch.float32, device=x.device)
    _check(lib().ksana_quant_fp8(_p(x), _p(q), _p(s), s.stride(0), M, K, x.stride(0), _st()), "ksana_quant_fp8")
    return q, s


# -------------------------------------------------------------------------------- elementwise
def norm(x, w, eps, residual=None, beta=None, out=None, layernorm=False, quant=False, q=None, s=None,
         want_out=True):
    """y = norm(x (+residual, updated in place)) * w (+beta); optionally also the FP8 operand of y."""
    M, H = x.shape
    if want_out and out is None:
        out = torch.empty(M, H, dtype=torch.bfloat16, device=x.device)
    if quant:
        if q is None:
            q = torch.empty(M, H, dtype=torch.float8_e4m3fn, device=x.device)
        if s is None:
            s = torch.empty(H // 128, max(4, (M + 3) // 4 * 4), dtype=torch.float32, device=x.device)
    rc = lib().ksana_norm(_p(x), _p(residual), _p(w), _p(beta), _p(out) if want_out else None, _p(q) if quant else None,
                          _p(s) if quant else None, s.stride(0) if quant else 0, M, H, float(eps), int(layernorm),
                          _st())
    _check(rc, "ksana_norm")
    return (out, q, s) if quant else out


_ACTS = {"silu": 0, "swiglu": 0, "gelu": 1, "gelu_new": 1, "gelu_pytorch_tanh": 1, "relu": 2}


def act_mul(x, act="silu", gated=True, out=None, quant=False, q=None, s=None, want_out=True):
    M = x.shape[0]
    inter = x.shape[1] // 2 if gated else x.shape[1]
    if want_out and out is None:
        out = torch.empty(M, inter, dtype=torch.bfloat16, device=x.device)
    if quant:
        if q is None:
            q = torch.empty(M, inter, dtype=torch.float8_e4m3fn, device=x.device)
        if s is None:
            s = torch.empty(inter // 128, max(4, (M + 3) // 4 * 4), dtype=torch.float32, device=x.device)
    rc = lib().ksana_act_mul(_p(x), _p(out) if want_out else None, _p(q) if quant else None, _p(s) if quant else None,
                             s.stride(0) if quant else 0, M, inter, x.stride(0), _ACTS[act], int(gated), _st())
    _check(rc, "ksana_act_mul")
    return (out, q, s) if quant else out


def embedding(ids, table, out=None, vocab_lo=0, vocab_hi=None, positions=None, pos_table=None, scale=1.0):
    T, H = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=table.device)
    hi = vocab_lo + table.shape[0] if vocab_hi is None else vocab_hi
    rc = lib().ksana_embedding(_p(ids), _p(table), _p(positions), _p(pos_table), _p(out), T, H, vocab_lo, hi,
                               float(scale), _st())
    _check(rc, "ksana_embedding")
    return out


def gather_rows(x, idx, out=None):
    R, H = idx.numel(), x.shape[1]
    if out is None:
        out = torch.empty(R, H, dtype=torch.bfloat16, device=x.device)
    _check(lib().ksana_gather_rows(_p(x), _p(idx), _p(out), R, H, int(x.shape[0]), _p(err_flag(x.device)), _st()),
           "ksana_gather_rows")
    return out


def refit_rows(hidden, pos, emb):
    _check(lib().ksana_refit_rows(_p(hidden), _p(pos), _p(emb), pos.numel(), hidden.shape[1], _st()),
           "ksana_refit_rows")


def patch_ids(ids, rows, src, prev_tokens):
    """ids[rows[i]] = prev_tokens[src[i]] on the device (all int32)."""
    _check(lib().ksana_patch_ids(_p(ids), _p(rows), _p(src), _p(prev_tokens), rows.numel(), ids.numel(),
                                 prev_tokens.numel(), _p(err_flag(ids.device)), _st()), "ksana_patch_ids")


def rerotate_blocks(cache, triples, cos_sin, rot_dim, neox):
    """Rotate the K rows of the destination blocks of ``triples`` (int32 [n, 3] on the device: source block,
    destination block, position delta) by their position deltas, in place. ``cache``: [blocks, layers, 2, kv heads,
    block tokens, head dim], bf16 or e4m3; ``cos_sin``: [max_pos, rot_dim] fp32."""
    nb, layers, _, hkv, bt, D = cache.shape
    _check(lib().ksana_rerotate_blocks(_p(cache), _p(triples), triples.shape[0], _p(cos_sin), cos_sin.shape[0], layers,
                                       hkv, bt, D, rot_dim, int(bool(neox)), cache.element_size(), nb,
                                       _p(err_flag(cache.device)), _st()), "ksana_rerotate_blocks")


def add(a, b=None, bias=None, out=None):
    if out is None:
        out = torch.empty_like(a)
    H = a.shape[-1]
    _check(lib().ksana_add(_p(a), _p(b), _p(bias), _p(out), a.numel() // H, H, _st()), "ksana_add")
    return out


def cast_f32(x, out=None):
    if out is None:
        out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    _check(lib().ksana_cast_f32(_p(x), _p(out), x.numel(), _st()), "ksana_cast_f32")
    return out


# ---------------------------------------------------------------------------- attention path
def rope_kv_append(qkv, positions, slots, cos_sin, cache_layer, block_stride, block_tokens, Hq, Hkv, D, rot_dim,
                   neox=True, mrope_sections=None, k_scale=1.0, v_scale=1.0, apply_rope=True):
    """In-place RoPE on q,k of qkv [T,(Hq+2Hkv)*D] and append of k,v into the layer's paged cache."""
    T = qkv.shape[0]
    fp8 = cache_layer is not None and cache_layer.dtype != torch.bfloat16
    pos_stride, s0, s1 = 0, 0, 0
    if mrope_sections is not None:
        pos_stride = positions.stride(0)
        s0, s1 = mrope_sections[0], mrope_sections[0] + mrope_sections[1]
    rc = lib().ksana_rope_kv_append(_p(qkv), _p(positions), pos_stride, _p(slots), _p(cos_sin), _p(cache_layer),
                                    block_stride, block_tokens, T, Hq, Hkv, D, rot_dim, int(neox), s0, s1, int(fp8),
                                    float(k_scale), float(v_scale), int(apply_rope), _st())
    _check(rc, "ksana_rope_kv_append")


def _cache_rows(cache_layer, block_stride, D):
    """Rows of D elements addressable from the layer's base pointer (bounds of the TMA tensor map)."""
    return int(cache_layer.shape[0]) * int(block_stride) // int(D)


PREFILL_TC = True                  # prefill attention on tcgen05 where the kernel covers the configuration


def paged_prefill(q, q_stride, out, cache_layer, block_stride, block_tokens, block_table, cu_q, kv_lens, B, max_q_len,
                  Hq, Hkv, D, scale, alibi=None, k_scale=1.0, v_scale=1.0):
    fp8 = cache_layer.dtype != torch.bfloat16
    if PREFILL_TC and not fp8 and D == 128:
        # tcgen05 kernel (head dim 128, bf16 cache, group size dividing 128); -100 = configuration not covered
        rc = lib().ksana_paged_prefill_tc(_p(q), q_stride, q.shape[0], _p(out), out.stride(0), _p(cache_layer),
                                          block_stride, block_tokens, _p(block_table), block_table.stride(0),
                                          _p(cu_q), _p(kv_lens), _p(alibi), B, max_q_len, Hq, Hkv, D, float(scale),
                                          _cache_rows(cache_layer, block_stride, D), _p(err_flag(q.device)), _st())
        if rc != -100:
            _check(rc, "ksana_paged_prefill_tc")
            return
    rc = lib().ksana_paged_prefill(_p(q), q_stride, _p(out), out.stride(0), _p(cache_layer), block_stride,
                                   block_tokens, _p(block_table), block_table.stride(0), _p(cu_q), _p(kv_lens),
                                   _p(alibi), B, max_q_len, Hq, Hkv, D, float(scale), int(fp8), float(k_scale),
                                   float(v_scale), _cache_rows(cache_layer, block_stride, D), _p(err_flag(q.device)), _st())
    _check(rc, "ksana_paged_prefill")


def paged_decode(q, q_stride, out, cache_layer, block_stride, block_tokens, block_table, kv_lens, B, Hq, Hkv, D, scale,
                 alibi=None, k_scale=1.0, v_scale=1.0, num_splits=1, part_o=None, part_ml=None, out_q=None,
                 out_scale=None):
    """``out_q`` / ``out_scale`` (head dim 128): the output also (or, with ``out`` None, only) as the FP8 operand of the
    next GEMM: e4m3 [B, Hq * D] and scales [Hq, ld]."""
    fp8 = cache_layer.dtype != torch.bfloat16
    rc = lib().ksana_paged_decode(_p(q), q_stride, _p(out), out.stride(0) if out is not None else Hq * D, _p(cache_layer),
                                  block_stride, block_tokens,
                                  _p(block_table), block_table.stride(0), _p(kv_lens), _p(alibi), B, Hq, Hkv, D,
                                  float(scale), int(fp8), float(k_scale), float(v_scale), num_splits, _p(part_o),
                                  _p(part_ml), _cache_rows(cache_layer, block_stride, D), _p(out_q), _p(out_scale),
                                  out_scale.stride(0) if out_scale is not None else 0, _p(err_flag(q.device)), _st())
    _check(rc, "ksana_paged_decode")


def mla_rope_append(q, nope, kv, norm_w, eps, positions, slots, cos_sin, qfull, cache_layer, block_stride, block_tokens, G):
    """Latent RMSNorm + rotary key rotation + append to the paged latent cache, and q_pe rotation into ``qfull``
    ([T, G, 576]; its first 512 columns are filled by the caller). q: [T, G*(nope+64)], kv: [T, 576]."""
    T = q.shape[0]
    rc = lib().ksana_mla_rope_append(_p(q), q.stride(0), nope, _p(kv), kv.stride(0), _p(norm_w), float(eps), _p(positions),
                                     _p(slots), _p(cos_sin), _p(qfull), _p(cache_layer), block_stride, block_tokens, T, G,
                                     int(cos_sin.shape[0]), int(cache_layer.shape[0]) * block_tokens,
                                     _p(err_flag(q.device)), _st())
    _check(rc, "ksana_mla_rope_append")


def mla_splits(num_seqs: int, max_q_len: int, max_kv: int, sms: int = 148) -> int:
    """KV splits for the latent-attention kernel: only pure decode steps split; the count minimises the number of
    CTA waves times the tiles per CTA, and a split never holds fewer than 4 tiles of 64 tokens."""
    if max_q_len != 1 or num_seqs <= 0:
        return 1
    tiles = max(1, (max_kv + 63) // 64)
    most = max(1, min(32, tiles // 4))
    best, best_cost = 1, None
    for n in range(1, most + 1):
        waves = (2 * num_seqs * n + sms - 1) // sms            # one CTA per SM, two output halves per sequence
        cost = waves * ((tiles + n - 1) // n + 2)              # tile times of the longest CTA chain (+ set-up)
        if best_cost is None or cost < best_cost:
            best, best_cost = n, cost
    return best


def mla_attention(qfull, out, cache_layer, block_stride, block_tokens, block_table, cu_q, kv_lens, B, max_q_len, G, scale,
                  nsplit=1) -> bool:
    """Absorbed multi-head latent attention on tcgen05 (see csrc/kernels/mla_attention.cu). qfull [T, G, 576],
    out [T, G, 512]. Returns False when the kernel does not cover the configuration."""
    T = qfull.shape[0]
    po = pml = None
    if nsplit > 1:
        po = torch.empty(nsplit * T * G * 512, dtype=torch.float32, device=qfull.device)
        pml = torch.empty(nsplit * T * G * 2, dtype=torch.float32, device=qfull.device)
    rc = lib().ksana_mla_attention(_p(qfull), T, _p(out), out.stride(0), _p(cache_layer), block_stride, block_tokens,
                                   _p(block_table), block_table.stride(0), _p(cu_q), _p(kv_lens), B, max_q_len, G,
                                   float(scale), _cache_rows(cache_layer, block_stride, 576), nsplit, _p(po), _p(pml),
                                   _p(err_flag(qfull.device)), _st())
    if rc == -100:
        return False
    _check(rc, "ksana_mla_attention")
    return True


def copy_blocks(cache, pairs, block_bytes):
    """pairs: int32 [n, 2] (source block, destination block) on the device; ids outside the cache are skipped and
    recorded in the error word."""
    _check(lib().ksana_copy_blocks(_p(cache), _p(pairs), pairs.numel() // 2, block_bytes, int(cache.shape[0]),
                                   _p(err_flag(cache.device)), _st()), "ksana_copy_blocks")


def swap_blocks(cache, host_pool, pairs, block_bytes, to_host: bool):
    """Whole cache blocks between the device cache and the pinned host block pool, one launch per list. ``pairs``:
    int32 [n, 2] (device block, host block) on the device; ``host_pool``: pinned uint8 [host_blocks, block_bytes]
    (the kernel reads / writes it over PCIe, no staging copy). Bad ids are skipped and recorded in the error word."""
    _check(lib().ksana_swap_blocks(_p(cache), host_pool.data_ptr(), _p(pairs), pairs.numel() // 2, block_bytes,
                                   0 if to_host else 1, int(cache.shape[0]), int(host_pool.shape[0]),
                                   _p(err_flag(cache.device)), _st()), "ksana_swap_blocks")


# ----------------------------------------------------------------------------------- sampler
def sample(logits, temperature, top_k, top_p, seeds, steps, out_tokens, row_idx=None, num_logprobs=0, lp_ids=None,
           lp_vals=None):
    B = out_tokens.numel()
    rc = lib().ksana_sample(_p(logits), logits.stride(0), _p(row_idx), _p(temperature), _p(top_k), _p(top_p),
                            _p(seeds), _p(steps), _p(out_tokens), num_logprobs, _p(lp_ids), _p(lp_vals), B,
                            logits.shape[1], _st())
    _check(rc, "ksana_sample")


def sample_merged(cand_vals, cand_ids, temperature, top_k, top_p, seeds, steps, out_tokens, num_logprobs=0, lp_ids=None,
                  lp_vals=None):
    """The sampler over candidate lists gathered from the vocabulary shards: cand_vals [B, C] fp32 logits and
    cand_ids [B, C] int32 token ids of the same columns."""
    B = out_tokens.numel()
    rc = lib().ksana_sample_merged(_p(cand_vals), cand_vals.stride(0), _p(cand_ids), cand_ids.stride(0), None,
                                   _p(temperature), _p(top_k), _p(top_p), _p(seeds), _p(steps), _p(out_tokens),
                                   num_logprobs, _p(lp_ids), _p(lp_vals), B, cand_vals.shape[1], _st())
    _check(rc, "ksana_sample_merged")


def shard_topk(logits, vocab, k, idx_offset, out_vals, out_ids):
    """This vocabulary shard's k largest logits per row and their token ids (column + idx_offset):
    out_vals fp32 [B, k], out_ids int32 [B, k], sorted by value (descending) then id."""
    B = logits.shape[0]
    rc = lib().ksana_shard_topk(_p(logits), logits.stride(0), None, B, vocab, k, idx_offset, _p(out_vals), _p(out_ids),
                                _st())
    _check(rc, "ksana_shard_topk")


def repetition_penalty(logits, offsets, ids, penalty, row_idx=None):
    B = penalty.numel()
    rc = lib().ksana_repetition_penalty(_p(logits), logits.stride(0), _p(row_idx), _p(offsets), _p(ids), _p(penalty),
                                        B, logits.shape[1], _st())
    _check(rc, "ksana_repetition_penalty")


def ban_tokens(logits, offsets, ids, row_idx=None):
    B = offsets.numel() - 1
    rc = lib().ksana_ban_tokens(_p(logits), logits.stride(0), _p(row_idx), _p(offsets), _p(ids), B, logits.shape[1],
                                _st())
    _check(rc, "ksana_ban_tokens")


# --------------------------------------------------------------------------- mixture of experts
def gemm_grouped(a, w, tile_expert, E, N, out=None, a_scale=None, w_scale=None, bn=0):
    """Expert-major rows of ``a`` [cap, K] (128-row tiles, one expert each) times stacked W [E*N, K]."""
    cap, K = a.shape
    kind = 0 if a_scale is None else 1
    if out is None:
        out = torch.empty(cap, N, dtype=torch.bfloat16, device=a.device)
    rc = lib().ksana_gemm_grouped(kind, _p(a), a.stride(0), _p(a_scale), a_scale.stride(0) if a_scale is not None else 0,
                                  _p(w), w.stride(0), _p(w_scale), _p(out), out.stride(0), cap, N, K, E,
                                  _p(tile_expert), bn, _p(err_flag(a.device)), _st())
    _check(rc, "ksana_gemm_grouped")
    return out


def moe_route(logits, K, scoring="softmax", renorm=True, scale=1.0, bias=None, n_group=1, topk_group=1):
    T, E = logits.shape
    ids = torch.empty(T, K, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, K, dtype=torch.float32, device=logits.device)
    rc = lib().ksana_moe_route(_p(logits), _p(bias), _p(ids), _p(w), T, E, K, 0 if scoring == "softmax" else 1,
                               int(renorm), float(scale), n_group, topk_group, _st())
    _check(rc, "ksana_moe_route")
    return ids, w


def moe_align(topk_ids, E, expert_lo=0, expert_hi=None):
    TK = topk_ids.numel()
    hi = E if expert_hi is None else expert_hi
    max_tiles = (TK + (hi - expert_lo) * 127 + 127) // 128
    dev = topk_ids.device
    dst_row = torch.empty(TK, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    total = torch.empty(1, dtype=torch.int32, device=dev)
    rc = lib().ksana_moe_align(_p(topk_ids), _p(dst_row), _p(tile_expert), _p(offsets), _p(total), TK, E, max_tiles,
                               expert_lo, hi, _p(err_flag(dev)), _st())
    _check(rc, "ksana_moe_align")
    return dst_row, tile_expert, offsets, total, max_tiles * 128


def moe_permute(x, dst_row, K, cap, zero=False):
    """``zero``: padding rows are zero instead of undefined (for consumers that reduce over the whole tensor)."""
    T, H = x.shape
    perm = (torch.zeros if zero else torch.empty)(cap, H, dtype=torch.bfloat16, device=x.device)
    _check(lib().ksana_moe_permute(_p(x), _p(dst_row), _p(perm), T, K, H, cap, _p(err_flag(x.device)), _st()),
           "ksana_moe_permute")
    return perm


def moe_combine(y, dst_row, topk_w, out, K, accumulate):
    T, H = out.shape
    _check(lib().ksana_moe_combine(_p(y), _p(dst_row), _p(topk_w), _p(out), T, K, H, int(accumulate), int(y.shape[0]),
                                   _p(err_flag(out.device)), _st()), "ksana_moe_combine")
    return out
