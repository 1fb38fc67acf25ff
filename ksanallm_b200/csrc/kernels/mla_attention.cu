// Multi-head latent attention (DeepSeek-V2/V3 "absorbed" form) on the tcgen05 tensor cores, prefill and decode,
// over the paged latent cache. The reference has no MLA (its attention layers are flash-attention + vLLM paged
// attention over per-head K/V: src/ksana_llm/layers/nvidia/flash_attention_layer.cpp, paged_attention_layer.cpp);
// this file is new work for the DeepSeek family.
//
// Cache row (one per token and layer): 512 latent values c_kv followed by the 64 rotary key values k_pe, bf16.
// Query row (one per token and head): q_lat = q_nope W_uk (512) followed by the rotated q_pe (64).
//   S = Q K^T over all 576 columns, softmax, O = P V with V = the first 512 columns of the same cache rows,
// i.e. multi-query attention with one shared 576/512-wide "KV head".
//
// One CTA owns 128 packed query rows (row = (token, head), all G heads of this rank share every staged tile) and
// one half (256 columns) of the output. TMEM (512 columns): the O accumulator of the half (256), a double-buffered
// 64-token S/P tile (2 x 64) and the first 256 columns of Q as an A operand (128 columns of bf16 pairs). The
// sibling CTA of the other half recomputes S (the two run concurrently and share the tile reads through L2).
// Set-up: TMA brings the Q tile in (panels 0..3 into the not yet used KV stages), the softmax warps move those
// panels row by row into TMEM; the other five panels (latent 256..511 and the rotary part) stay in shared
// memory next to two 64-token KV stages. Per tile:
//   S = Q K^T      36 tcgen05.mma (9 panels of 64 columns, K = 16 each, N = 64): 16 with A from TMEM, 20 with A from
//                  shared memory; B = the staged tile, K-major (TMA, 128-byte swizzle). The 36 MMAs accumulate into
//                  one tile and are latency-bound as a chain, which is why the tile is 64 tokens wide and not 32
//                  (measured: same time per tile at either width).
//   softmax        4 warps, one thread per row (TMEM lane), online maximum with a lazy rescale of O
//   O += P V       P read from TMEM (bf16 pairs over S's columns), V = MN-major view of the same staged tile
// The MMA thread issues S of tile j+1 ahead of P V of tile j when it is ready first, so the softmax of one tile
// overlaps the tensor work of its neighbours. Warp roles: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner,
// warps 2..5 softmax + epilogue. Split-KV (decode): grid.x carries `nsplit` ranges of KV tiles whose unnormalised
// partial outputs (fp32 O, running maximum, row sum) are merged by mla_merge_kernel.
// Every wait is bounded; a timeout sets the error word and leaves the output untouched.
#include "sm100_ptx.cuh"
#include "guards.cuh"
#include <cuda_bf16.h>
#include <math_constants.h>

namespace ksana {

typedef __nv_bfloat16 bf16;
constexpr int kMlaThreads = 192;
constexpr int kMlaM = 128;                    // packed query rows per CTA
constexpr int kMlaTok = 64;                   // KV tokens per tile
constexpr int kMlaLora = 512, kMlaDk = 576;
constexpr int kMlaPanels = 9;                 // 64-column panels of a 576-wide row
constexpr int kMlaQPanelBytes = kMlaM * 128;
constexpr int kMlaQTmemPanels = 4;            // Q columns [0, 256) live in TMEM (128 columns of bf16 pairs)
constexpr int kMlaQSmemPanels = kMlaPanels - kMlaQTmemPanels;   // columns [384, 576) stay in shared memory
constexpr int kMlaQBytes = kMlaQSmemPanels * kMlaQPanelBytes;
constexpr int kMlaKvPanelBytes = kMlaTok * 128;
constexpr int kMlaKvBytes = kMlaPanels * kMlaKvPanelBytes;
constexpr int kMlaStages = 2;                 // KV tiles in flight
constexpr int kMlaSmemBytes = kMlaQBytes + kMlaStages * kMlaKvBytes + 1024 + 256;
constexpr uint32_t kMlaTmemCols = 512;        // O half [0,256), S/P buffers at 256 and 320, Q at [384, 512)
constexpr int kMlaMaxBoxes = kMlaTok / 8;      // TMA boxes per tile with the smallest (8-token) cache blocks
static_assert(kMlaQTmemPanels * kMlaQPanelBytes <= kMlaStages * kMlaKvBytes, "Q staging must fit in the KV stages");
constexpr float kMlaRescaleLog2 = 8.f;

struct MlaParams {
  bf16* out; long long out_tok_stride;        // [T, G, 512] bf16, elements between tokens
  float* part_o; float* part_ml;              // [nsplit, T, G, 512] / [nsplit, T, G, 2] when nsplit > 1
  const int* block_table; int table_stride;
  const int* cu_q; const int* kv_lens;
  int G, block_tokens, box_rows, nsplit, T;
  long long rows_per_block;                   // cache rows (576 elements each) between consecutive blocks
  int num_blocks;                             // blocks addressable from the layer base (block-table entries are checked)
  float scale_log2;
  int* err;
};

__device__ __forceinline__ float mla_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kMlaThreads, 1)
mla_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, const MlaParams p) {
  extern __shared__ uint8_t mla_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(mla_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + kMlaQBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kMlaQBytes + kMlaStages * kMlaKvBytes);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;      // [kMlaStages]
  uint64_t* kv_empty = bars + 5;     // [kMlaStages]
  uint64_t* s_full = bars + 9;       // [2]
  uint64_t* p_full = bars + 11;      // [2]
  uint64_t* pv_done = bars + 13;
  uint64_t* o_full = bars + 14;
  uint64_t* q_moved = bars + 15;     // the softmax warps have copied the TMEM part of Q out of the staging area
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.z, half = blockIdx.y;
  const int G = p.G;
  const int q0 = p.cu_q[s], q_len = p.cu_q[s + 1] - q0;
  const int kv_len = p.kv_lens[s];
  const int nqt = static_cast<int>(gridDim.x) / p.nsplit;
  const int split = static_cast<int>(blockIdx.x) % p.nsplit;
  const int qtile = nqt - 1 - static_cast<int>(blockIdx.x) / p.nsplit;      // longest rows first
  const int row0 = qtile * kMlaM;
  if (row0 >= q_len * G) return;
  // inconsistent sequence metadata: touch nothing (kv_len == 0 is the padding row of a captured decode graph: it
  // takes the empty-range path below)
  if (q0 < 0 || q_len < 0 || q0 + q_len > p.T || (kv_len != 0 && kv_len < q_len)) {
    if (threadIdx.x == 0) guard_report(p.err, kGuardQueryRow, q0 + q_len);
    return;
  }
  const int past = kv_len - q_len;
  const int last_row = min(row0 + kMlaM - 1, q_len * G - 1);
  const int kv_end = min(kv_len, past + last_row / G + 1);
  const int nt_all = (kv_end + kMlaTok - 1) / kMlaTok;
  const int per = (nt_all + p.nsplit - 1) / p.nsplit;
  const int tile_lo = split * per;
  const int ntiles = max(min(nt_all, tile_lo + per) - tile_lo, 0);
  const int* table = p.block_table + static_cast<size_t>(s) * p.table_stride;

  if (ntiles == 0) {
    // an empty KV range (more splits than tiles): publish "no contribution" for the merge and leave
    // (with a single split this only happens for kv_len == 0, e.g. padding rows of a captured decode graph:
    // their output rows are zeroed)
    if (warp >= 2) {
      const int vr = row0 + (warp & 3) * 32 + lane;
      if (vr < q_len * G) {
        if (p.nsplit > 1) {
          if (half == 0) {
            float* ml = p.part_ml + ((static_cast<size_t>(split) * p.T + q0 + vr / G) * G + vr % G) * 2;
            ml[0] = -CUDART_INF_F;
            ml[1] = 0.f;
          }
        } else {
          uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(q0 + vr / G) * p.out_tok_stride +
                                                (vr % G) * kMlaLora + half * 256);
          for (int i = 0; i < 32; ++i) dst[i] = make_uint4(0, 0, 0, 0);
        }
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kMlaStages; ++i) { mbar_init(kv_full + i, 1); mbar_init(kv_empty + i, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(s_full + i, 1); mbar_init(p_full + i, 4); }
    mbar_init(pv_done, 1); mbar_init(o_full, 1); mbar_init(q_moved, 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kMlaTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base, tmem_s = tmem_base + 256, tmem_q = tmem_base + 256 + 2 * kMlaTok;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&q_map);
      tma_prefetch_desc(&kv_map);
      // Q: panels 0..5 into the (still unused) KV stages as a staging area for their copy to TMEM, 6..8 to their home
      mbar_expect_tx(q_full, kMlaPanels * kMlaQPanelBytes);
      const int tok0 = q0 + row0 / G;
#pragma unroll
      for (int pn = 0; pn < kMlaPanels; ++pn) {
        uint8_t* dst = pn < kMlaQTmemPanels ? kv_s + pn * kMlaQPanelBytes : q_s + (pn - kMlaQTmemPanels) * kMlaQPanelBytes;
        tma_load_3d(dst, &q_map, q_full, pn * 64, 0, tok0);
      }
    }
    __syncwarp();
    {
      // KV tiles: the whole warp runs the loop; lane 0 owns the barrier traffic, lanes 0..8 each issue the boxes of
      // one 64-column panel (36 box copies per tile from a single thread were a microsecond of issue time)
      const int bt = p.block_tokens, br = p.box_rows;
      const int boxes = kMlaTok / br;                       // at most kMlaMaxBoxes (8-token blocks)
      // block-table entries of a tile are fetched one tile ahead, so that their global-memory latency is not part
      // of the chain "buffer freed -> TMA issued"
      int blk[kMlaMaxBoxes], blk_next[kMlaMaxBoxes];
      auto fetch = [&](int j, int (&dst)[kMlaMaxBoxes]) {
        const int t0 = (tile_lo + j) * kMlaTok;
#pragma unroll
        for (int bx = 0; bx < kMlaMaxBoxes; ++bx) {
          const int t = t0 + bx * br;
          int id = (bx < boxes && t < kv_len) ? __ldg(table + t / bt) : 0;
          if (id < 0 || id >= p.num_blocks) { guard_report(p.err, kGuardBlockId, id); id = 0; }
          dst[bx] = id;
        }
      };
      fetch(0, blk_next);
      bool ok = mbar_wait(q_moved, 0, abort_flag);           // the staging area is free
      for (int j = 0; j < ntiles; ++j) {
        const int b = j % kMlaStages;
        const int t0 = (tile_lo + j) * kMlaTok;
        const int nbox = min(boxes, (kv_len - t0 + br - 1) / br);
#pragma unroll
        for (int bx = 0; bx < kMlaMaxBoxes; ++bx) blk[bx] = blk_next[bx];
        if (j + 1 < ntiles) fetch(j + 1, blk_next);
        ok = ok && mbar_wait(kv_empty + b, ((j / kMlaStages) & 1) ^ 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) break;
        if (lane == 0) mbar_expect_tx(kv_full + b, static_cast<uint32_t>(nbox) * br * 128 * kMlaPanels);
        __syncwarp();
        if (lane < kMlaPanels) {
          uint8_t* dst = kv_s + b * kMlaKvBytes + lane * kMlaKvPanelBytes;
#pragma unroll
          for (int bx = 0; bx < kMlaMaxBoxes; ++bx) {
            if (bx < nbox) {
              const int t = t0 + bx * br;
              const long long r0 = static_cast<long long>(blk[bx]) * p.rows_per_block + (t % bt);
              tma_load_2d(dst + bx * br * 128, &kv_map, kv_full + b, lane * 64, static_cast<int>(r0));
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(128, kMlaTok, 1, 1);
      constexpr uint32_t idesc_pv = make_idesc(128, 256, 1, 1) | (1u << 16);     // B (= V) is MN-major
      bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(q_moved, 0, abort_flag);
      tc_fence_after();
      const uint32_t qb = smem_u32(q_s);
      // S of tile j+1 may be issued ahead of P V of tile j (it then overlaps the softmax of tile j), but whichever
      // of the two becomes ready first goes first: issuing P V as soon as P is ready frees the tile's buffer
      // early, which is what gives the next TMA load its lead time. The polls are test_wait (non-blocking): a
      // try_wait on the barrier that is not ready yet suspends the thread and hides the other one becoming ready.
      int s_next = 0, pv_next = 0;         // next tile whose S / P V has not been issued
      uint32_t idle = 0;
      while (ok && pv_next < ntiles) {
        bool progress = false;
        if (pv_next < s_next && mbar_test_wait(p_full + (pv_next & 1), (pv_next >> 1) & 1)) {
          const int j = pv_next, bb = j & 1, st = j % kMlaStages;
          tc_fence_after();
          const uint32_t vb = smem_u32(kv_s + st * kMlaKvBytes) + half * 4 * kMlaKvPanelBytes;
#pragma unroll
          for (int k = 0; k < kMlaTok / 16; ++k) {
            // 16 tokens per MMA: 8 TMEM columns of P (two bf16 each), 16 rows (2 KB per panel) of the tile
            const uint64_t bdesc = make_smem_desc_mn_sw128(vb + k * 2048, kMlaKvPanelBytes);
            mma_f16_ts(tmem_o, tmem_s + kMlaTok * bb + 8 * k, bdesc, idesc_pv, (j | k) != 0);
          }
          tc_commit(kv_empty + st);
          tc_commit(pv_done);
          if (j == ntiles - 1) tc_commit(o_full);
          ++pv_next;
          progress = true;
        } else if (s_next < ntiles && s_next <= pv_next + 1 &&
                   mbar_test_wait(kv_full + (s_next % kMlaStages), (s_next / kMlaStages) & 1)) {
          // (s_next <= pv_next + 1: the S/P buffer of tile s_next was last read by P V of tile s_next - 2)
          const int bb = s_next & 1;
          tc_fence_after();
          const uint32_t kb = smem_u32(kv_s + (s_next % kMlaStages) * kMlaKvBytes);
#pragma unroll
          for (int k = 0; k < 4 * kMlaPanels; ++k) {
            const int pn = k >> 2;
            const uint64_t bdesc = make_smem_desc_sw128(kb + pn * kMlaKvPanelBytes) + 2 * (k & 3);
            if (pn < kMlaQTmemPanels) {
              // A (16 Q columns = 8 TMEM columns of bf16 pairs) straight from TMEM: no shared-memory read of Q
              mma_f16_ts(tmem_s + kMlaTok * bb, tmem_q + 8 * k, bdesc, idesc_qk, k != 0);
            } else {
              const uint64_t adesc = make_smem_desc_sw128(qb + (pn - kMlaQTmemPanels) * kMlaQPanelBytes) + 2 * (k & 3);
              mma_f16(tmem_s + kMlaTok * bb, adesc, bdesc, idesc_qk, k != 0);
            }
          }
          tc_commit(s_full + bb);
          ++s_next;
          progress = true;
        }
        if (progress) {
          idle = 0;
        } else if (++idle >= kWaitPolls || ((idle & 63u) == 63u && *abort_flag)) {
          *abort_flag = 1;
          ok = false;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (one thread per row)
    const int qd = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const int vr = row0 + qd * 32 + lane;                  // packed row index inside the sequence
    const bool active = vr < q_len * G;
    const int tok = vr / G, head = vr % G;
    const int limit = active ? past + tok : -1;            // last visible KV position
    float m_used = -CUDART_INF_F, l = 0.f;
    bool ok = mbar_wait(q_full, 0, abort_flag);
    if (ok) {
      // this thread's Q row, columns [0, 384): staging area (128-byte-swizzled panels) -> registers -> TMEM, in the
      // layout the MMA reads an A operand from TMEM (row = lane, two consecutive bf16 per 32-bit column)
      const int rr = qd * 32 + lane;
#pragma unroll 1
      for (int pn = 0; pn < kMlaQTmemPanels; ++pn) {
        const uint8_t* src = kv_s + pn * kMlaQPanelBytes + rr * 128;
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 q4 = *reinterpret_cast<const uint4*>(src + ((c ^ (rr & 7)) << 4));
          v[4 * c] = q4.x; v[4 * c + 1] = q4.y; v[4 * c + 2] = q4.z; v[4 * c + 3] = q4.w;
        }
        tmem_st32(tmem_q + lane_off + pn * 32, v);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_moved);
    }
    for (int j = 0; ok && j < ntiles; ++j) {
      const int b = j & 1;
      const int t0 = (tile_lo + j) * kMlaTok;
      if (!mbar_wait(s_full + b, (j >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t r[kMlaTok];
#pragma unroll
      for (int c = 0; c < kMlaTok / 32; ++c)
        tmem_ld32(tmem_s + kMlaTok * b + lane_off + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
      tmem_ld_wait();
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int i = 0; i < kMlaTok; ++i) {
        const float v = (t0 + i <= limit) ? __uint_as_float(r[i]) * p.scale_log2 : -CUDART_INF_F;
        r[i] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
      // lazy rescale of O: keep the old reference maximum unless the row's maximum grew by more than 2^8
      float m_new = m_used;
      if (mx > m_used + kMlaRescaleLog2 || m_used == -CUDART_INF_F) m_new = (mx == -CUDART_INF_F) ? m_used : mx;
      const bool grow = m_new != m_used && m_used != -CUDART_INF_F;
      if (__any_sync(0xffffffffu, grow)) {
        // P V of the previous tile must have landed in O before O is rescaled (S of this tile was issued ahead of it)
        if (!mbar_wait(pv_done, (j - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const float f = grow ? exp2f(m_used - m_new) : 1.f;
        l *= f;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_o + lane_off + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tmem_st32(tmem_o + lane_off + c * 32, o);
        }
      }
      m_used = m_new;
      const float mref = (m_used == -CUDART_INF_F) ? 0.f : m_used;
#pragma unroll
      for (int i = 0; i < kMlaTok; i += 2) {
        const float p0 = mla_exp2(__uint_as_float(r[i]) - mref);
        const float p1 = mla_exp2(__uint_as_float(r[i + 1]) - mref);
        l += p0 + p1;
        __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        r[i >> 1] = *reinterpret_cast<uint32_t*>(&pb);          // in place: slot i/2 has already been consumed
      }
#pragma unroll
      for (int c = 0; c < kMlaTok / 32; ++c)
        tmem_st16(tmem_s + kMlaTok * b + lane_off + c * 16, *reinterpret_cast<uint32_t(*)[16]>(&r[c * 16]));
      tmem_st_wait();
      if (t0 + kMlaTok > kv_len) {
        // last tile of the sequence: rows past the sequence end hold stale shared memory or whatever the cache has
        // there; their probabilities are 0, but 0 x NaN would poison O. Zero them before the P V MMA reads them.
        const int first_bad = kv_len - t0;
        const int nchunks = (kMlaTok - first_bad) * (kMlaPanels * 8);      // 16-byte chunks
        uint8_t* buf = kv_s + (j % kMlaStages) * kMlaKvBytes;
        for (int i = threadIdx.x - 64; i < nchunks; i += 128) {
          const int rr = first_bad + i / (kMlaPanels * 8), c = i % (kMlaPanels * 8);
          *reinterpret_cast<uint4*>(buf + (c >> 3) * kMlaKvPanelBytes + rr * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        fence_async_smem();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + b);
    }
    if (ok && mbar_wait(o_full, 0, abort_flag)) {
      tc_fence_after();
      if (p.nsplit == 1) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* dst = p.out + static_cast<size_t>(q0 + tok) * p.out_tok_stride + head * kMlaLora + half * 256;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_o + lane_off + c * 32, o);
          tmem_ld_wait();
          if (active) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 ov;
              __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                o2[e] = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * e]) * inv, __uint_as_float(o[i + 2 * e + 1]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = ov;
            }
          }
        }
      } else {
        const size_t prow = (static_cast<size_t>(split) * p.T + q0 + tok) * G + head;
        float* dst = p.part_o + prow * kMlaLora + half * 256;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_o + lane_off + c * 32, o);
          tmem_ld_wait();
          if (active) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = make_uint4(o[i], o[i + 1], o[i + 2], o[i + 3]);
          }
        }
        if (active && half == 0) {
          p.part_ml[prow * 2] = m_used;
          p.part_ml[prow * 2 + 1] = l;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 8);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);       // let copies in flight land before the CTA retires
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kMlaTmemCols); }
}

// Merge of split-KV partials: out[row] = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s. One CTA per (token, head).
__global__ void mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                 long long out_tok_stride, int T, int G, int nsplit) {
  const int row = blockIdx.x, tok = row / G, head = row % G;
  const size_t rows = static_cast<size_t>(T) * G;
  float m = -CUDART_INF_F;
  for (int s = 0; s < nsplit; ++s) {
    const float* ml = part_ml + (s * rows + row) * 2;
    if (ml[1] > 0.f) m = fmaxf(m, ml[0]);
  }
  float denom = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < nsplit; ++s) {
    const float* ml = part_ml + (s * rows + row) * 2;
    if (!(ml[1] > 0.f)) continue;
    const float w = exp2f(ml[0] - m);
    denom += w * ml[1];
    const float4 o = *reinterpret_cast<const float4*>(part_o + (s * rows + row) * kMlaLora + threadIdx.x * 4);
    acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(out + static_cast<size_t>(tok) * out_tok_stride + head * kMlaLora + threadIdx.x * 4) = v;
}

// Per token: RMSNorm of the 512 latent values, rotation of the shared rotary key, append of both to the paged
// latent cache (slot < 0 skips the write), and rotation of every head's q_pe into the packed query rows.
//   q      [T, G, nope + 64] bf16 (q_b projection), q_stride elements between tokens
//   kv     [T, 576] bf16 (kv_a projection: raw latent | raw rotary key), kv_stride elements between tokens
//   qfull  [T, G, 576] bf16: columns [512, 576) are written here, [0, 512) by the q_nope W_uk product
// Rotation pairs are (2i, 2i+1) ("interleaved"); cos_sin: [max_pos][64] = cos(32) | sin(32).
__global__ void mla_rope_append_kernel(const bf16* __restrict__ q, long long q_stride, int nope, const bf16* __restrict__ kv,
                                       long long kv_stride, const bf16* __restrict__ norm_w, float eps,
                                       const int* __restrict__ positions, const int* __restrict__ slots,
                                       const float* __restrict__ cos_sin, bf16* __restrict__ qfull, bf16* __restrict__ cache,
                                       long long rows_per_block, int block_tokens, int G, int max_pos, long long num_slots,
                                       int* err) {
  __shared__ float red[4];
  const int t = blockIdx.x, tid = threadIdx.x;                 // 128 threads
  const bf16* row = kv + static_cast<size_t>(t) * kv_stride;
  int pos = positions[t];
  if (pos < 0 || pos >= max_pos) { if (tid == 0) guard_report(err, kGuardPosition, pos); pos = 0; }
  const float* cs = cos_sin + static_cast<size_t>(pos) * 64;
  int slot = slots[t];
  if (slot >= num_slots) { if (tid == 0) guard_report(err, kGuardSlot, slot); slot = -1; }
  bf16* crow = nullptr;
  if (slot >= 0 && cache != nullptr)
    crow = cache + (static_cast<size_t>(slot / block_tokens) * rows_per_block + slot % block_tokens) * kMlaDk;
  float v[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[i] = __bfloat162float(row[tid * 4 + i]); ss += v[i] * v[i]; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  const float inv = rsqrtf((red[0] + red[1] + red[2] + red[3]) * (1.f / kMlaLora) + eps);
  if (crow) {
#pragma unroll
    for (int i = 0; i < 4; ++i) crow[tid * 4 + i] = __float2bfloat16(v[i] * inv * __bfloat162float(norm_w[tid * 4 + i]));
    if (tid < 32) {
      const float x0 = __bfloat162float(row[kMlaLora + 2 * tid]), x1 = __bfloat162float(row[kMlaLora + 2 * tid + 1]);
      const float c = cs[tid], s = cs[32 + tid];
      crow[kMlaLora + 2 * tid] = __float2bfloat16(x0 * c - x1 * s);
      crow[kMlaLora + 2 * tid + 1] = __float2bfloat16(x1 * c + x0 * s);
    }
  }
  for (int i = tid; i < G * 32; i += 128) {
    const int h = i >> 5, j = i & 31;
    const bf16* qp = q + static_cast<size_t>(t) * q_stride + static_cast<size_t>(h) * (nope + 64) + nope;
    const float x0 = __bfloat162float(qp[2 * j]), x1 = __bfloat162float(qp[2 * j + 1]);
    const float c = cs[j], s = cs[32 + j];
    bf16* dst = qfull + (static_cast<size_t>(t) * G + h) * kMlaDk + kMlaLora;
    dst[2 * j] = __float2bfloat16(x0 * c - x1 * s);
    dst[2 * j + 1] = __float2bfloat16(x1 * c + x0 * s);
  }
}

typedef CUresult (*MlaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static MlaEncodeFn mla_encode_fn() {
  static MlaEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<MlaEncodeFn>(ptr);
  }
  return fn;
}

}  // namespace ksana

using namespace ksana;

// Absorbed MLA attention of this step's query rows against the paged latent cache.
//   q      [T, G, 576] bf16 contiguous (q_lat | rotated q_pe), T = rows addressable from q
//   out    [T, G, 512] bf16, out_tok_stride elements between tokens
//   cache  layer base of [block][block_tokens][576] bf16, blocks block_stride elements apart, cache_rows rows addressable
// Sequences: cu_q [B+1], kv_lens [B] (KV length including this step's rows), block_table [B][table_stride].
// nsplit > 1 needs part_o [nsplit*T*G*512] and part_ml [nsplit*T*G*2] fp32.
// Returns 0 when launched, -100 when the configuration is not covered (the caller uses its own fallback).
extern "C" int ksana_mla_attention(const void* q, long long T, void* out, long long out_tok_stride, const void* cache,
                                   long long block_stride, int block_tokens, const int* block_table, int table_stride,
                                   const int* cu_q, const int* kv_lens, int B, int max_q_len, int G, float scale,
                                   long long cache_rows, int nsplit, float* part_o, float* part_ml, int* err,
                                   cudaStream_t st) {
  if (B <= 0 || max_q_len <= 0) return 0;
  const int bt = block_tokens;
  if (G <= 0 || G > 128 || (G & (G - 1))) return -100;
  if (bt < 8 || (bt & (bt - 1)) || bt > 256) return -100;
  if (block_stride % kMlaDk || block_stride < static_cast<long long>(bt) * kMlaDk) return -100;
  if (cache_rows <= 0 || cache_rows >= (1LL << 31) || T <= 0 || T >= (1LL << 31)) return -100;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(out)) & 15) return -100;
  if (out_tok_stride % 8) return -100;
  if (nsplit < 1) nsplit = 1;
  if (nsplit > 1 && (!part_o || !part_ml)) return -10;
  MlaEncodeFn enc = mla_encode_fn();
  if (!enc) return -100;
  const int box_rows = bt < kMlaTok ? bt : kMlaTok;
  CUtensorMap q_map, kv_map;
  {
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(kMlaDk), static_cast<cuuint64_t>(G), static_cast<cuuint64_t>(T)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(kMlaDk) * 2, static_cast<cuuint64_t>(G) * kMlaDk * 2};
    cuuint32_t box[3] = {64, static_cast<cuuint32_t>(G), static_cast<cuuint32_t>(kMlaM / G)};
    cuuint32_t estr[3] = {1, 1, 1};
    if (enc(&q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -100;
  }
  {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(kMlaDk), static_cast<cuuint64_t>(cache_rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(kMlaDk) * 2};
    cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&kv_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -100;
  }
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(mla_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmemBytes) != cudaSuccess)
      return -3;
    set = true;
  }
  MlaParams p{};
  p.out = static_cast<bf16*>(out); p.out_tok_stride = out_tok_stride;
  p.part_o = part_o; p.part_ml = part_ml;
  p.block_table = block_table; p.table_stride = table_stride; p.cu_q = cu_q; p.kv_lens = kv_lens;
  p.G = G; p.block_tokens = bt; p.box_rows = box_rows; p.nsplit = nsplit; p.T = static_cast<int>(T);
  p.rows_per_block = block_stride / kMlaDk;
  p.num_blocks = static_cast<int>(cache_rows / p.rows_per_block);
  p.scale_log2 = scale * 1.44269504f;
  p.err = err;
  const int nqt = (max_q_len * G + kMlaM - 1) / kMlaM;
  dim3 grid(nqt * nsplit, 2, B);
  mla_tc_kernel<<<grid, kMlaThreads, kMlaSmemBytes, st>>>(q_map, kv_map, p);
  if (cudaGetLastError() != cudaSuccess) return -4;
  if (nsplit > 1) {
    mla_merge_kernel<<<static_cast<unsigned>(T) * G, 128, 0, st>>>(part_o, part_ml, static_cast<bf16*>(out), out_tok_stride,
                                                                 static_cast<int>(T), G, nsplit);
    if (cudaGetLastError() != cudaSuccess) return -4;
  }
  return 0;
}

extern "C" int ksana_mla_rope_append(const void* q, long long q_stride, int nope, const void* kv, long long kv_stride,
                                     const void* norm_w, float eps, const int* positions, const int* slots,
                                     const float* cos_sin, void* qfull, void* cache, long long block_stride,
                                     int block_tokens, int T, int G, int max_pos, long long num_slots, int* err,
                                     cudaStream_t st) {
  if (T <= 0) return 0;
  if (block_stride % kMlaDk) return -10;
  mla_rope_append_kernel<<<T, 128, 0, st>>>(static_cast<const bf16*>(q), q_stride, nope, static_cast<const bf16*>(kv),
                                            kv_stride, static_cast<const bf16*>(norm_w), eps, positions, slots, cos_sin,
                                            static_cast<bf16*>(qfull), static_cast<bf16*>(cache), block_stride / kMlaDk,
                                            block_tokens, G, max_pos, num_slots, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
