// Epilogue of a row-parallel GEMM that sends its partial rows to other GPUs ("push" mode).
//
// After tcgen05.ld a thread holds one row of the tile (32 rows per warp, SEG columns of it at a time). Stored from
// there, every instruction would touch 32 rows with 16 bytes each, and over NVLink every such piece is a packet of
// its own. The warp therefore turns 2 KB at a time through shared memory - 8 rows x up to 128 columns, or 16 rows x
// 64 columns - and stores each row's SEG columns as one contiguous run (up to 256 bytes, 16 bytes per lane): the
// run of a row becomes one or two full-size link packets.
//
// Staging layout: row lr at lr * CP * 16 bytes, 16-byte chunk j at slot j ^ (lr & 7): both the row-wise writes
// (8 lanes x 16 bytes per shared-memory phase, one lane per row) and the chunk-wise reads (one lane per chunk) are
// free of bank conflicts.
//
// Row `grow` of the result belongs to rank `min(grow / push_rows, push_n - 1)` and lands at row
// `grow - owner * push_rows` of that rank's receive slot (`push[owner]`, leading dimension ldd, bf16).
// push_rows <= 0: broadcast - every rank receives every row (at row `grow` of `push[q]` for all q).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace ksana {

constexpr int kPushStageBytes = 2048;      // shared memory per epilogue warp

// r: SEG fp32 accumulators (as bits) of this lane's row, r[0] at global column `col`; grow_base: global row of lane 0.
template <int SEG>
__device__ __forceinline__ void push_rows_staged(uint8_t* stg, const uint32_t* r, const __nv_bfloat16* bias, int lane,
                                                 int grow_base, int col, int M, int N, __nv_bfloat16* const* push,
                                                 int push_n, int push_rows, int ldd) {
  static_assert(SEG % 8 == 0 && SEG <= 128, "segment: a multiple of 8 columns, at most 128");
  constexpr int C = SEG / 8;                      // 16-byte chunks per row
  constexpr int CP = C > 8 ? 16 : 8;              // chunk slots per staged row
  constexpr int ROWS = kPushStageBytes / (CP * 16);   // rows per round: 8 or 16
  constexpr int ROUNDS = 32 / ROWS;
  constexpr int RPI = 32 / CP;                    // rows per store instruction
#pragma unroll
  for (int ph = 0; ph < ROUNDS; ++ph) {
    if (lane / ROWS == ph) {
      const int lr = lane % ROWS;
#pragma unroll
      for (int j = 0; j < C; ++j) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[8 * j + i]);
        if (bias && col + 8 * j < N) {
          const uint4 bv = *reinterpret_cast<const uint4*>(bias + col + 8 * j);
          const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
          for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(b2[i]); o[2 * i] += f.x; o[2 * i + 1] += f.y; }
        }
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
        *reinterpret_cast<uint4*>(stg + lr * (CP * 16) + ((j ^ (lr & 7)) << 4)) = ov;
      }
    }
    __syncwarp();
    const int jc = lane % CP;
#pragma unroll
    for (int it = 0; it < ROWS / RPI; ++it) {
      const int rr = it * RPI + lane / CP;
      const int grow = grow_base + ph * ROWS + rr;
      const int gcol = col + 8 * jc;
      if (jc < C && grow < M && gcol < N) {
        const uint4 ov = *reinterpret_cast<const uint4*>(stg + rr * (CP * 16) + ((jc ^ (rr & 7)) << 4));
        if (push_rows > 0) {
          const int owner = min(grow / push_rows, push_n - 1);
          *reinterpret_cast<uint4*>(push[owner] + static_cast<size_t>(grow - owner * push_rows) * ldd + gcol) = ov;
        } else {
          // every rank reduces all rows itself (decode-sized batches): the row goes to this rank's slot in all of them
          for (int q = 0; q < push_n; ++q)
            *reinterpret_cast<uint4*>(push[q] + static_cast<size_t>(grow) * ldd + gcol) = ov;
        }
      }
    }
    __syncwarp();
  }
}

}  // namespace ksana
