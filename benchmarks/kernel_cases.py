"""Small, self-contained launches of the hot kernels for profiling (each case runs its kernel twice).

  python benchmarks/kernel_cases.py [case ...]
  ncu --set full --clock-control none -k regex:<kernel> -c <n> -o prof python benchmarks/kernel_cases.py <case>

Cases keep a few hundred MB on the device: larger than L2 where DRAM figures matter, small enough for a
multi-pass capture to finish in a minute or two.
"""
from __future__ import annotations

import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ksanallm_b200.ops import native, reference as ref  # noqa: E402

DEV = "cuda"


def _w8(n, k):
    wq = (torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.05).to(torch.float8_e4m3fn)
    return wq, torch.ones((n + 127) // 128, k // 128, device=DEV)


def case_skinny_fp8():       # decode gate|up shard: 8 tokens, 235 MB of FP8 weights streamed once
    wq, ws = _w8(28672, 8192)
    xq, xs = native.quant_fp8(torch.randn(8, 8192, device=DEV, dtype=torch.bfloat16))
    y = torch.empty(8, 28672, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        native.gemm_fp8(xq, xs, wq, ws, out=y)


def case_skinny_mx_m64():    # decode at batch 64 with tensor-core-applied scales: 470 MB of FP8 weights streamed once
    wq, ws = _w8(57344, 8192)
    xq, xs = native.quant_fp8(torch.randn(64, 8192, device=DEV, dtype=torch.bfloat16))
    y = torch.empty(64, 57344, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        native.gemm_fp8(xq, xs, wq, ws, out=y, splits=-1, hw_scale=True)


def case_gemm_mxfp8():       # prefill-sized hardware-scaled FP8 GEMM: 4096 x 10240 x 8192
    wq, ws = _w8(10240, 8192)
    xq, xs = native.quant_fp8(torch.randn(4096, 8192, device=DEV, dtype=torch.bfloat16))
    y = torch.empty(4096, 10240, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        native.gemm_mxfp8(xq, xs, wq, ws, y)


def case_gemm_mxfp8_pair():  # the same GEMM on CTA pairs (256 x 256 tiles over two SMs)
    wq, ws = _w8(10240, 8192)
    xq, xs = native.quant_fp8(torch.randn(4096, 8192, device=DEV, dtype=torch.bfloat16))
    y = torch.empty(4096, 10240, device=DEV, dtype=torch.bfloat16)

    def run():
        native.gemm_mxfp8_pair(xq, xs, wq, ws, y)
    run.flops = 2 * 4096 * 10240 * 8192
    for _ in range(2):
        run()
    return run


def case_gemm_mxfp8_tall():  # the same GEMM with 256 x 224 tiles per CTA
    wq, ws = _w8(10240, 8192)
    xq, xs = native.quant_fp8(torch.randn(4096, 8192, device=DEV, dtype=torch.bfloat16))
    y = torch.empty(4096, 10240, device=DEV, dtype=torch.bfloat16)

    def run():
        native.gemm_mxfp8_tall(xq, xs, wq, ws, y)
    run.flops = 2 * 4096 * 10240 * 8192
    for _ in range(2):
        run()
    return run


def case_gemm_mxfp8_big():   # a prefill step of the 70B model: 16384 x 10240 x 8192
    wq, ws = _w8(10240, 8192)
    xq, xs = native.quant_fp8(torch.randn(16384, 8192, device=DEV, dtype=torch.bfloat16))
    y = torch.empty(16384, 10240, device=DEV, dtype=torch.bfloat16)

    def run():
        native.gemm_mxfp8(xq, xs, wq, ws, y, bn=256)
    run.flops = 2 * 16384 * 10240 * 8192
    for _ in range(2):
        run()
    return run


def case_gemm_mxfp8_pair_big():
    wq, ws = _w8(10240, 8192)
    xq, xs = native.quant_fp8(torch.randn(16384, 8192, device=DEV, dtype=torch.bfloat16))
    y = torch.empty(16384, 10240, device=DEV, dtype=torch.bfloat16)

    def run():
        native.gemm_mxfp8_pair(xq, xs, wq, ws, y)
    run.flops = 2 * 16384 * 10240 * 8192
    for _ in range(2):
        run()
    return run


def case_skinny_bf16():
    w = torch.randn(14336, 8192, device=DEV, dtype=torch.bfloat16) * 0.05
    x = torch.randn(8, 8192, device=DEV, dtype=torch.bfloat16)
    y = torch.empty(8, 14336, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        native.gemm_bf16(x, w, out=y)


def case_gemm_fp8():         # prefill-sized FP8 GEMM: 4096 x 10240 x 8192 (256-wide tiles, split epilogue)
    wq, ws = _w8(10240, 8192)
    xq, xs = native.quant_fp8(torch.randn(4096, 8192, device=DEV, dtype=torch.bfloat16))
    y = torch.empty(4096, 10240, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        native.gemm_fp8(xq, xs, wq, ws, out=y)


def case_gemm_bf16():
    w = torch.randn(8192, 8192, device=DEV, dtype=torch.bfloat16) * 0.05
    x = torch.randn(4096, 8192, device=DEV, dtype=torch.bfloat16)
    y = torch.empty(4096, 8192, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        native.gemm_bf16(x, w, out=y)


def _paged(B, kv_len, Hq, Hkv, D, q_len):
    bt = 16
    nblk = (kv_len + bt - 1) // bt
    cache = torch.randn(B * nblk, 2, Hkv, bt, D, device=DEV, dtype=torch.bfloat16)
    table = torch.arange(B * nblk, device=DEV, dtype=torch.int32).view(B, nblk)
    q = torch.randn(B * q_len, (Hq + 2 * Hkv) * D, device=DEV, dtype=torch.bfloat16)
    cu = torch.arange(0, (B + 1) * q_len, q_len, device=DEV, dtype=torch.int32)
    kvl = torch.full((B,), kv_len, device=DEV, dtype=torch.int32)
    out = torch.empty(B * q_len, Hq * D, device=DEV, dtype=torch.bfloat16)
    return q, cache, table, cu, kvl, out


def case_decode_attn():      # 64 sequences x 2304 cached tokens, 64 q / 8 kv heads: 604 MB of K/V read once
    B, kv, Hq, Hkv, D = 64, 2304, 64, 8, 128
    q, cache, table, cu, kvl, out = _paged(B, kv, Hq, Hkv, D, 1)
    splits = 1
    for _ in range(2):
        native.paged_decode(q, q.stride(0), out, cache, cache.stride(0), 16, table, kvl, B, Hq, Hkv, D, 1 / math.sqrt(D),
                            num_splits=splits)


def case_prefill_attn():     # 4 sequences x 2048 new tokens, 64 q / 8 kv heads
    B, kv, Hq, Hkv, D = 4, 2048, 64, 8, 128
    q, cache, table, cu, kvl, out = _paged(B, kv, Hq, Hkv, D, kv)
    for _ in range(2):
        native.paged_prefill(q, q.stride(0), out, cache, cache.stride(0), 16, table, cu, kvl, B, kv, Hq, Hkv, D,
                             1 / math.sqrt(D))


def _mla(B, q_len, kv_len, G, nsplit):
    bt = 16
    nblk = (kv_len + bt - 1) // bt
    cache = torch.randn(B * nblk, 1, bt, 576, device=DEV, dtype=torch.bfloat16) * 0.5
    layer = cache[:, 0]
    table = torch.arange(B * nblk, device=DEV, dtype=torch.int32).view(B, nblk)
    q = torch.randn(B * q_len, G, 576, device=DEV, dtype=torch.bfloat16) * 0.3
    cu = torch.arange(0, (B + 1) * q_len, q_len, device=DEV, dtype=torch.int32)
    kvl = torch.full((B,), kv_len, device=DEV, dtype=torch.int32)
    out = torch.empty(B * q_len, G, 512, device=DEV, dtype=torch.bfloat16)

    def run():
        native.mla_attention(q, out, layer, layer.stride(0), bt, table, cu, kvl, B, q_len, G, 1 / math.sqrt(192), nsplit)
    # work per launch: causal pairs x heads x (576 + 512) x 2 flops; cache bytes read once
    pairs = B * (q_len * (kv_len - q_len) + q_len * (q_len + 1) // 2)
    run.flops = pairs * G * (576 + 512) * 2
    run.bytes = B * kv_len * 576 * 2
    return run


def case_mla_decode():       # DeepSeek-V3 decode, all 128 heads on one GPU: 32 sequences x 4096 cached tokens (151 MB)
    run = _mla(32, 1, 4096, 128, native.mla_splits(32, 1, 4096))
    for _ in range(2):
        run()
    return run


def case_mla_decode_tp8():   # 16 heads per rank (TP8): 64 sequences x 4096 cached tokens (302 MB)
    run = _mla(64, 1, 4096, 16, native.mla_splits(64, 1, 4096))
    for _ in range(2):
        run()
    return run


def case_mla_prefill():      # 2 sequences x 2048 new tokens, 128 heads (absorbed form)
    run = _mla(2, 2048, 2048, 128, 1)
    for _ in range(2):
        run()
    return run


def _w4_case(M):
    N, K, g = 28672, 8192, 128
    q4 = torch.randint(0, 256, (N, K // 2), device=DEV, dtype=torch.uint8)
    scale = torch.full((N, K // g), 0.01, device=DEV, dtype=torch.float16)
    zs = torch.full((N, K // g), 0.08, device=DEV, dtype=torch.float16)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    y = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)

    def run():
        native.linear_w4(x, q4, scale, zs, out=y)
    run.bytes = N * K // 2 + 2 * N * (K // g) * 2
    run.flops = 2 * M * N * K
    for _ in range(2):
        run()
    return run


def case_w4_gemv():          # 4-bit weight-only decode GEMM: 8 rows x 28672 x 8192 (117 MB of packed weights)
    return _w4_case(8)


def case_w4_m128():          # the same weights at a decode batch of 128
    return _w4_case(128)


def case_norm_quant():       # residual add + RMSNorm + FP8 quantisation of 16384 x 8192 activations (805 MB moved)
    x = torch.randn(16384, 8192, device=DEV, dtype=torch.bfloat16)
    r = torch.randn(16384, 8192, device=DEV, dtype=torch.bfloat16)
    w = torch.ones(8192, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        native.norm(x, w, 1e-5, residual=r, quant=True, want_out=False)


def case_sampler():
    logits = torch.randn(64, 128256, device=DEV)
    B = 64
    args = (torch.ones(B, device=DEV), torch.full((B,), 50, device=DEV, dtype=torch.int32), torch.full((B,), 0.9, device=DEV),
            torch.arange(B, device=DEV, dtype=torch.int64) + 1, torch.zeros(B, device=DEV, dtype=torch.int32),
            torch.zeros(B, device=DEV, dtype=torch.int32))
    for _ in range(2):
        native.sample(logits, *args)


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}


def time_cases(names):
    """CUDA-event timing (after warm-up); every case launches its kernel twice per call."""
    for n in names:
        fn = CASES[n]
        run = fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if callable(run):
            # the case handed back its launch closure: time the kernel alone (inputs stay resident; cases are
            # sized beyond L2 where DRAM traffic matters)
            reps = 10
            e0.record()
            for _ in range(reps):
                run()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            extra = ""
            if getattr(run, "flops", 0):
                extra += f", {run.flops / ms / 1e9:.1f} TFLOP/s"
            if getattr(run, "bytes", 0):
                extra += f", {run.bytes / ms / 1e6:.1f} GB/s of streamed bytes"
            print(f"{n}: {ms * 1000:.1f} us per launch{extra}")
            # clock record: the same launch repeated for about three quarters of a second while nvidia-smi samples
            # the SM clock and the throttle reasons (a burst of ten launches is over before the first sample)
            from ksanallm_b200.utils.clocks import ClockSampler
            sampler = ClockSampler(torch.cuda.current_device())
            sampler.start()
            loops = max(10, int(0.75 / max(ms * 1e-3, 1e-6)))
            e0.record()
            for _ in range(loops):
                run()
            e1.record()
            torch.cuda.synchronize()
            clocks = sampler.stop()
            print(f"{n}: sustained {e0.elapsed_time(e1) / loops * 1000:.1f} us per launch over {loops} launches; "
                  f"SM clock median {clocks.get('sm_mhz')} of {clocks.get('sm_max_mhz')} MHz, reasons {clocks.get('reasons')}")
            continue
        # inputs are re-created inside each case; time only the second half by differencing two call counts
        reps = 3
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        print(f"{n}: {e0.elapsed_time(e1) / reps:.3f} ms per case call (input creation included)")


def main(argv):
    unknown = [a for a in argv if a != "--time" and a not in CASES]
    if unknown:
        raise SystemExit(f"unknown case(s) {unknown}; cases: {' '.join(CASES)}")
    if argv and argv[0] == "--time":
        return time_cases(argv[1:] or list(CASES))
    names = argv or list(CASES)
    for n in names:
        CASES[n]()
        torch.cuda.synchronize()
        native.check_err_flag(DEV)
        print("ran", n)


if __name__ == "__main__":
    main(sys.argv[1:])
