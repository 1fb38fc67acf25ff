// Paged attention for sm_100a: causal prefill (chunked-prefill and prefix-cache
// aware) and split-KV decode, both reading K/V in place from the paged cache
// through a block table.
//
// Grouped-query packing: the query heads that share one KV head are packed into
// the M dimension of the tensor-core tiles together with the query tokens, so a
// K/V tile staged in shared memory is used by the whole head group (8 heads for
// Llama-3 / Qwen2 70B) instead of being re-read per query head.
//
//   virtual row r of (sequence s, kv head g):  token = r / G,  head = g*G + r % G
//
// Prefill: 64 rows per CTA (4 warps x 16), K/V tiles of 64 tokens, online
// softmax in fp32 (exp2), only the NEW query rows are computed: the causal
// offset is kv_len - q_len, so cached prefixes cost no attention work.
// Decode: one CTA per (kv head, sequence, split); the 4 warps walk disjoint
// 16-token slices of each tile, partial (m, l, O) are merged in shared memory
// and, when the sequence was split, by a small reduce kernel.
//
// FP8 (e4m3) caches are dequantised with a per-layer scale while staging tiles.
//
// Functional counterpart of the reference's decode kernels
// (3rdparty/LLM_kernels/csrc/kernels/nvidia/paged_attention/paged_attention.cu:81-640)
// and of its FlashAttention-2 call (src/ksana_llm/kernels/nvidia/kernel_wrapper.cpp:437-588),
// without the reverse cache copy the latter needs.
#include "sm100_ptx.cuh"
#include "pdl.cuh"
#include "fp8_scale.cuh"
#include <cuda_fp8.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace ksana {

// K/V staging modes: plain cp.async (any block size), FP8 cache with conversion, or TMA: one elected thread
// issues a 2-D bulk tensor copy per (cache block, 64-column half) - the per-16-byte address arithmetic of
// the cp.async path made the decode kernel instruction-bound at a third of HBM bandwidth.
enum KvMode { kKvCpAsync = 0, kKvFp8 = 1, kKvTma = 2 };

typedef __nv_bfloat16 bf16;
constexpr int kTileTok = 64;     // KV tokens per shared-memory tile
constexpr int kAttnThreads = 128;
constexpr int kKvStages = 3;      // K/V tile ring: two tiles in flight while one is consumed

struct AttnParams {
  const bf16* q; long long q_stride;     // [T, q_stride] ; head h at column h*D
  bf16* out; long long out_stride;       // [T, out_stride]
  const void* cache;                     // layer base: [block][2][Hkv][block_tokens][D]
  long long block_stride;                // elements between blocks
  int block_tokens;
  const int* block_table; int table_stride;   // [B][table_stride]
  const int* cu_q;                       // [B+1] query row offsets (prefill) or null (decode: row = s)
  const int* kv_lens;                    // [B]
  const float* alibi;                    // [Hq] slopes or null
  int Hq, Hkv;
  float scale_log2;                      // softmax scale * log2(e)
  float k_scale, v_scale;                // fp8 cache dequant scales
  // decode split workspace
  float* part_o; float* part_ml; int num_splits;
  int* err;                              // device word set when a bounded wait gave up
  // decode, head dim 128: also emit the output as the FP8 operand of the next GEMM (e4m3 values [T][Hq*D] and one
  // power-of-two scale per row and head, [Hq][oscale_ld]), quantised from the bf16-rounded values exactly as the
  // stand-alone quantiser would
  uint8_t* outq; float* oscale; int oscale_ld;
};

// One head row of D = 128 outputs held one per thread of a 128-thread block: rounds to bf16, stores it (if `out`),
// and stores the row's e4m3 values and scale. Every thread of the block must call it.
__device__ __forceinline__ void store_head_row_q(const AttnParams& p, int s, int head, int d, float v, float* red4) {
  const __nv_bfloat16 b = __float2bfloat16(v);
  const float fb = __bfloat162float(b);
  if (p.out) p.out[static_cast<size_t>(s) * p.out_stride + head * 128 + d] = b;
  float am = fabsf(fb);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  __syncthreads();                                   // red4 may still be read from the previous row
  if ((threadIdx.x & 31) == 0) red4[threadIdx.x >> 5] = am;
  __syncthreads();
  am = fmaxf(fmaxf(red4[0], red4[1]), fmaxf(red4[2], red4[3]));
  const float sc = fp8_group_scale(am);
  const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(fb * (1.f / sc), __NV_SATFINITE, __NV_E4M3);
  p.outq[(static_cast<size_t>(s) * p.Hq + head) * 128 + d] = q;
  if (d == 0) p.oscale[static_cast<size_t>(head) * p.oscale_ld + s] = sc;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Shared tile of ROWS rows x D bf16, stored as D/64 panels of [ROWS][64] (128-byte rows); inside a panel the
// 16-byte chunk cc of row r lives at chunk (cc ^ (r & 7)): exactly what a TMA copy with the 128-byte swizzle
// writes, and conflict-free for ldmatrix.
template <int D, int ROWS>
__device__ __forceinline__ bf16* tile_ptr(bf16* base, int r, int chunk) {
  return base + (chunk >> 3) * (ROWS * 64) + r * 64 + (((chunk & 7) ^ (r & 7)) << 3);
}

// Stage one K or V tile (kTileTok tokens x D) of kv head g into shared memory.
template <int D, bool FP8>
__device__ __forceinline__ void load_kv_tile(bf16* dst, const AttnParams& p, const int* table, int g, int which,
                                             int tok0, int kv_len, float dq) {
  constexpr int CH = D / 8;
  for (int i = threadIdx.x; i < kTileTok * CH; i += kAttnThreads) {
    const int r = i / CH, c = i % CH;
    const int tok = tok0 + r;
    bf16* d = tile_ptr<D, kTileTok>(dst, r, c);
    if (tok < kv_len) {
      const int blk = table[tok / p.block_tokens];
      const size_t off = static_cast<size_t>(blk) * p.block_stride +
                         ((static_cast<size_t>(which) * p.Hkv + g) * p.block_tokens + tok % p.block_tokens) * D + c * 8;
      if (FP8) {
        const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(p.cache) + off);
        const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __half_raw h0 = __nv_cvt_fp8_to_halfraw(b[2 * e], __NV_E4M3);
          const __half_raw h1 = __nv_cvt_fp8_to_halfraw(b[2 * e + 1], __NV_E4M3);
          ow[e] = pack_bf16(__half2float(__half(h0)) * dq, __half2float(__half(h1)) * dq);
        }
        *reinterpret_cast<uint4*>(d) = o;
      } else {
        cp_async16(d, static_cast<const bf16*>(p.cache) + off);
      }
    } else {
      *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
  }
}

// TMA staging of one K + V tile (one thread): a box of [block_tokens rows x 64 columns] per cache block and
// 64-column panel. Tokens past kv_len inside the last block are loaded as they are (finite cache contents)
// and masked by the softmax; blocks past the sequence are not loaded at all.
template <int D>
__device__ __forceinline__ void tma_issue_kv(bf16* ks, bf16* vs, uint64_t* bar, const CUtensorMap* map, const AttnParams& p,
                                             const int* table, int g, int tok0, int kv_len, long long rows_per_block) {
  const int bt = p.block_tokens;
  const int nblk = min(kTileTok / bt, (kv_len - tok0 + bt - 1) / bt);
  constexpr int PANELS = D / 64;
  mbar_expect_tx(bar, static_cast<uint32_t>(nblk) * 2 * PANELS * bt * 128);
  for (int b = 0; b < nblk; ++b) {
    const long long row0 = static_cast<long long>(table[tok0 / bt + b]) * rows_per_block;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      bf16* dst = which ? vs : ks;
      const int y = static_cast<int>(row0 + (static_cast<long long>(which) * p.Hkv + g) * bt);
#pragma unroll
      for (int h = 0; h < PANELS; ++h) tma_load_2d(dst + h * (kTileTok * 64) + b * bt * 64, map, bar, h * 64, y);
    }
  }
}

// After a TMA-staged tile has landed: zero the V rows of tokens past the sequence end (rows of blocks that were
// not loaded hold stale shared memory, rows past kv_len inside the last block hold whatever the cache has there);
// their probabilities are exactly 0, but 0 x NaN would poison the output. K needs nothing: its scores are masked.
template <int D>
__device__ __forceinline__ void zero_v_tail(bf16* vs, int valid_rows) {
  if (valid_rows >= kTileTok) return;
  constexpr int CH = D / 8;
  const int n = (kTileTok - valid_rows) * CH;
  for (int i = threadIdx.x; i < n; i += kAttnThreads) {
    const int r = valid_rows + i / CH, c = i % CH;
    *reinterpret_cast<uint4*>(tile_ptr<D, kTileTok>(vs, r, c)) = make_uint4(0, 0, 0, 0);
  }
}

// One warp: S(16 x NT*8 tokens) = Q(16 x D) K^T over tokens [t0, t0 + NT*8) of the staged tile.
template <int D, int NT>
__device__ __forceinline__ void warp_qk(float (&s)[NT][4], const uint32_t (&qf)[D / 16][4], bf16* ks, int t0, int lane) {
#pragma unroll
  for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int jp = 0; jp < NT / 2; ++jp) {
      uint32_t b[4];
      const int r = t0 + jp * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int c = kk * 2 + ((lane >> 3) & 1);
      ldsm_x4(b, smem_addr(tile_ptr<D, kTileTok>(ks, r, c)));
      mma16816(s[2 * jp], qf[kk], b[0], b[1]);
      mma16816(s[2 * jp + 1], qf[kk], b[2], b[3]);
    }
  }
}

// One warp: O(16 x D) += P(16 x NT*8) V over tokens [t0, t0 + NT*8).
template <int D, int NT>
__device__ __forceinline__ void warp_pv(float (&o)[D / 8][4], const float (&s)[NT][4], bf16* vs, int t0, int lane) {
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      uint32_t b[4];
      const int r = t0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int c = np * 2 + (lane >> 4);
      ldsm_x4_t(b, smem_addr(tile_ptr<D, kTileTok>(vs, r, c)));
      mma16816(o[2 * np], a, b[0], b[1]);
      mma16816(o[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// Mask + online-softmax update for one warp's 16 x (NT*8) score tile.
// Rows lane/4 and lane/4+8; limit[i] = last visible kv position of that row (-1 = row inactive).
template <int D, int NT>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&o)[D / 8][4], float (&m)[2], float (&l)[2],
                                               const int (&limit)[2], const float (&slope)[2], int tok0, int lane,
                                               float scale_log2) {
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e >> 1;
      const int tok = tok0 + j * 8 + (lane & 3) * 2 + (e & 1);
      float v = s[j][e] * scale_log2;
      if (slope[i] != 0.f) v += slope[i] * 1.44269504f * static_cast<float>(tok - limit[i]);
      v = tok <= limit[i] ? v : -INFINITY;
      s[j][e] = v;
      mx[i] = fmaxf(mx[i], v);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
  }
  float corr[2], mnew[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mnew[i] = fmaxf(m[i], mx[i]);
    corr[i] = (mnew[i] == -INFINITY) ? 1.f : exp2f(m[i] - mnew[i]);
    m[i] = mnew[i];
    l[i] *= corr[i];
  }
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1]; }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e >> 1;
      const float pv = (mnew[i] == -INFINITY) ? 0.f : exp2f(s[j][e] - mnew[i]);
      s[j][e] = pv;
      l[i] += pv;   // per-thread partial; reduced over the 4 lanes of a row at the end
    }
  }
}

// ----------------------------------------------------------------------------- prefill
template <int D, int MODE>
__global__ void __launch_bounds__(kAttnThreads)
paged_prefill_kernel(const __grid_constant__ CUtensorMap kv_map, const AttnParams p, const long long rows_per_block) {
  constexpr bool FP8 = MODE == kKvFp8;
  extern __shared__ uint8_t smem_attn_raw[];
  uint8_t* smem_attn = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_attn_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[kKvStages];
  __shared__ uint32_t abort_word;
  bf16* qs = reinterpret_cast<bf16*>(smem_attn);            // 64 x D
  bf16* ks = qs + 64 * D;                                   // kKvStages x (64 x D)
  bf16* vs = ks + kKvStages * kTileTok * D;                 // kKvStages x (64 x D)

  const int s = blockIdx.z, g = blockIdx.y;
  const int G = p.Hq / p.Hkv;
  const int q0 = p.cu_q[s], q_len = p.cu_q[s + 1] - q0;
  const int kv_len = p.kv_lens[s];
  const int row0 = blockIdx.x * 64;
  if (row0 >= q_len * G) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* table = p.block_table + static_cast<size_t>(s) * p.table_stride;
  const int past = kv_len - q_len;   // tokens already in the cache before this chunk

  // stage Q rows (zero for rows beyond the sequence)
  constexpr int CH = D / 8;
  for (int i = threadIdx.x; i < 64 * CH; i += kAttnThreads) {
    const int r = i / CH, c = i % CH;
    const int vr = row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (vr < q_len * G) {
      const int tok = vr / G, head = g * G + vr % G;
      v = *reinterpret_cast<const uint4*>(p.q + static_cast<size_t>(q0 + tok) * p.q_stride + head * D + c * 8);
    }
    *reinterpret_cast<uint4*>(tile_ptr<D, 64>(qs, r, c)) = v;
  }
  // causal bound of this CTA's rows
  const int last_row = min(row0 + 63, q_len * G - 1);
  const int kv_end = min(kv_len, past + last_row / G + 1);
  const int ntiles = (kv_end + kTileTok - 1) / kTileTok;

  if (MODE == kKvTma && threadIdx.x == 0) {
    for (int i = 0; i < kKvStages; ++i) mbar_init(&full_bar[i], 1);
    abort_word = 0;
    mbar_fence_init();
  }
  __syncthreads();
  auto issue = [&](int t) {      // cp.async modes always commit a group so that the wait counts stay uniform
    const int st = t % kKvStages;
    if (MODE == kKvTma) {
      if (threadIdx.x == 0 && t < ntiles)
        tma_issue_kv<D>(ks + st * kTileTok * D, vs + st * kTileTok * D, &full_bar[st], &kv_map, p, table, g,
                        t * kTileTok, kv_len, rows_per_block);
      return;
    }
    if (t < ntiles) {
      load_kv_tile<D, FP8>(ks + st * kTileTok * D, p, table, g, 0, t * kTileTok, kv_len, p.k_scale);
      load_kv_tile<D, FP8>(vs + st * kTileTok * D, p, table, g, 1, t * kTileTok, kv_len, p.v_scale);
    }
    cp_commit();
  };
  issue(0);
  issue(1);
  __syncthreads();

  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int r = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
    const int c = kk * 2 + (lane >> 4);
    ldsm_x4(qf[kk], smem_addr(tile_ptr<D, 64>(qs, r, c)));
  }
  int limit[2]; float slope[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int vr = row0 + warp * 16 + (lane >> 2) + i * 8;
    limit[i] = vr < q_len * G ? past + vr / G : -1;
    slope[i] = (p.alibi && vr < q_len * G) ? p.alibi[g * G + vr % G] : 0.f;
  }
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  bool ok = true;
  for (int t = 0; t < ntiles; ++t) {
    const int buf = t % kKvStages;
    if (MODE == kKvTma) {
      if (!mbar_wait(&full_bar[buf], (t / kKvStages) & 1, &abort_word)) { ok = false; break; }
      zero_v_tail<D>(vs + buf * kTileTok * D, kv_len - t * kTileTok);
    } else {
      cp_wait<1>();               // tile t has landed (only the newest group may still be in flight)
    }
    __syncthreads();              // ... for every thread, and everyone is done with tile t-1
    issue(t + 2);                 // refill the stage tile t-1 used
    float sc[8][4];
    warp_qk<D, 8>(sc, qf, ks + buf * kTileTok * D, 0, lane);
    softmax_update<D, 8>(sc, o, m, l, limit, slope, t * kTileTok, lane, p.scale_log2);
    warp_pv<D, 8>(o, sc, vs + buf * kTileTok * D, 0, lane);
  }
  if (!ok) {                      // a bounded wait gave up: leave the output untouched, report through the error word
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 4);
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int vr = row0 + warp * 16 + (lane >> 2) + i * 8;
    if (vr >= q_len * G) continue;
    const int tok = vr / G, head = g * G + vr % G;
    const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
    bf16* dst = p.out + static_cast<size_t>(q0 + tok) * p.out_stride + head * D + (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------------------ decode
// grid (Hkv, B, splits). Rows = the G query heads of kv head g (G <= 16), one new token each.
template <int D, int MODE>
__global__ void __launch_bounds__(kAttnThreads)
paged_decode_kernel(const __grid_constant__ CUtensorMap kv_map, const AttnParams p, const long long rows_per_block) {
  constexpr bool FP8 = MODE == kKvFp8;
  extern __shared__ uint8_t smem_attn_raw[];
  uint8_t* smem_attn = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_attn_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[kKvStages];
  __shared__ uint32_t abort_word;
  __shared__ float red4[4];
  bf16* qs = reinterpret_cast<bf16*>(smem_attn);            // 16 x D
  bf16* ks = qs + 16 * D;                                   // kKvStages x (64 x D)
  bf16* vs = ks + kKvStages * kTileTok * D;
  float* merge = reinterpret_cast<float*>(ks);              // 4 warps x 16 rows x (D + 2), reuses the K ring after the loop

  pdl_trigger();
  pdl_wait();
  const int g = blockIdx.x, s = blockIdx.y, split = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int kv_len = p.kv_lens[s];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* table = p.block_table + static_cast<size_t>(s) * p.table_stride;
  const int total_tiles = (kv_len + kTileTok - 1) / kTileTok;
  const int tiles_per = (total_tiles + p.num_splits - 1) / p.num_splits;
  const int t_begin = split * tiles_per, t_end = min(total_tiles, t_begin + tiles_per);

  constexpr int CH = D / 8;
  for (int i = threadIdx.x; i < 16 * CH; i += kAttnThreads) {
    const int r = i / CH, c = i % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G) v = *reinterpret_cast<const uint4*>(p.q + static_cast<size_t>(s) * p.q_stride + (g * G + r) * D + c * 8);
    *reinterpret_cast<uint4*>(tile_ptr<D, 16>(qs, r, c)) = v;
  }
  if (MODE == kKvTma && threadIdx.x == 0) {
    for (int i = 0; i < kKvStages; ++i) mbar_init(&full_bar[i], 1);
    abort_word = 0;
    mbar_fence_init();
  }
  __syncthreads();
  auto issue = [&](int t) {
    const int st = (t - t_begin) % kKvStages;
    if (MODE == kKvTma) {
      if (threadIdx.x == 0 && t < t_end)
        tma_issue_kv<D>(ks + st * kTileTok * D, vs + st * kTileTok * D, &full_bar[st], &kv_map, p, table, g,
                        t * kTileTok, kv_len, rows_per_block);
      return;
    }
    if (t < t_end) {
      load_kv_tile<D, FP8>(ks + st * kTileTok * D, p, table, g, 0, t * kTileTok, kv_len, p.k_scale);
      load_kv_tile<D, FP8>(vs + st * kTileTok * D, p, table, g, 1, t * kTileTok, kv_len, p.v_scale);
    }
    cp_commit();
  };
  issue(t_begin);
  issue(t_begin + 1);
  __syncthreads();
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int r = (lane & 7) + (((lane >> 3) & 1) << 3);
    const int c = kk * 2 + (lane >> 4);
    ldsm_x4(qf[kk], smem_addr(tile_ptr<D, 16>(qs, r, c)));
  }
  int limit[2]; float slope[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = (lane >> 2) + i * 8;
    limit[i] = r < G ? kv_len - 1 : -1;
    slope[i] = (p.alibi && r < G) ? p.alibi[g * G + r] : 0.f;
  }
  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  bool ok = true;
  for (int t = t_begin; t < t_end; ++t) {
    const int buf = (t - t_begin) % kKvStages;
    if (MODE == kKvTma) {
      if (!mbar_wait(&full_bar[buf], ((t - t_begin) / kKvStages) & 1, &abort_word)) { ok = false; break; }
      zero_v_tail<D>(vs + buf * kTileTok * D, kv_len - t * kTileTok);
    } else {
      cp_wait<1>();
    }
    __syncthreads();
    issue(t + 2);
    float sc[2][4];
    warp_qk<D, 2>(sc, qf, ks + buf * kTileTok * D, warp * 16, lane);
    softmax_update<D, 2>(sc, o, m, l, limit, slope, t * kTileTok + warp * 16, lane, p.scale_log2);
    warp_pv<D, 2>(o, sc, vs + buf * kTileTok * D, warp * 16, lane);
  }
  cp_wait<0>();
  __syncthreads();                // the merge area aliases the K ring: every warp must be out of the loop
  if (!ok) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 4);
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  // merge the 4 warps' streams: stage (m, l, O) per warp, then every thread combines a slice
  constexpr int MS = D + 2;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = (lane >> 2) + i * 8;
    float* dst = merge + (warp * 16 + r) * MS;
    if ((lane & 3) == 0) { dst[D] = m[i]; dst[D + 1] = l[i]; }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      dst[n * 8 + (lane & 3) * 2] = o[n][2 * i];
      dst[n * 8 + (lane & 3) * 2 + 1] = o[n][2 * i + 1];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += kAttnThreads) {
    const int r = i / D, d = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, merge[(w * 16 + r) * MS + D]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* src = merge + (w * 16 + r) * MS;
      const float f = (src[D] == -INFINITY) ? 0.f : exp2f(src[D] - mm);
      acc += src[d] * f;
      ll += src[D + 1] * f;
    }
    const int head = g * G + r;
    if (p.num_splits == 1) {
      const float v = ll > 0.f ? acc / ll : 0.f;
      if constexpr (D == 128) {
        if (p.outq) { store_head_row_q(p, s, head, d, v, red4); continue; }   // (D == blockDim: r is uniform per pass)
      }
      p.out[static_cast<size_t>(s) * p.out_stride + head * D + d] = __float2bfloat16(v);
    } else {
      const size_t base = (static_cast<size_t>(s) * p.Hq + head) * p.num_splits + split;
      p.part_o[base * D + d] = acc;
      if (d == 0) { p.part_ml[base * 2] = mm; p.part_ml[base * 2 + 1] = ll; }
    }
  }
}

// grid (Hq, B): combine the per-split partials.
template <int D>
__global__ void decode_reduce_kernel(const AttnParams p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red4[4];
  const int head = blockIdx.x, s = blockIdx.y;
  const size_t base = (static_cast<size_t>(s) * p.Hq + head) * p.num_splits;
  float mm = -INFINITY;
  for (int k = 0; k < p.num_splits; ++k) mm = fmaxf(mm, p.part_ml[(base + k) * 2]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f, ll = 0.f;
    for (int k = 0; k < p.num_splits; ++k) {
      const float mk = p.part_ml[(base + k) * 2];
      const float f = (mk == -INFINITY) ? 0.f : exp2f(mk - mm);
      acc += p.part_o[(base + k) * D + d] * f;
      ll += p.part_ml[(base + k) * 2 + 1] * f;
    }
    const float v = ll > 0.f ? acc / ll : 0.f;
    if constexpr (D == 128) {
      if (p.outq) { store_head_row_q(p, s, head, d, v, red4); continue; }     // 128 threads: one pass, every thread in it
    }
    p.out[static_cast<size_t>(s) * p.out_stride + head * D + d] = __float2bfloat16(v);
  }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*AttnEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AttnEncodeFn attn_encode_fn() {
  static AttnEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<AttnEncodeFn>(ptr);
  }
  return fn;
}

// The layer's cache seen as rows of D bf16 (row = one token of one head of K or V of one block); box = one
// cache block's tokens x 64 columns, 128-byte swizzle.
static bool make_kv_map(CUtensorMap* map, const void* cache, long long rows, int D, int block_tokens) {
  AttnEncodeFn enc = attn_encode_fn();
  if (!enc || (reinterpret_cast<uintptr_t>(cache) & 15)) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(D) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(block_tokens)};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool tma_ok(const AttnParams& p, int D) {
  const int bt = p.block_tokens;
  return (bt == 8 || bt == 16 || bt == 32 || bt == 64) && p.block_stride % D == 0;
}

template <int D, int MODE>
static int launch_prefill(const AttnParams& p, const CUtensorMap& map, long long rows_per_block, int B, int max_q_len,
                          cudaStream_t st) {
  const int smem = (64 + 2 * kKvStages * kTileTok) * D * 2 + 1024;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(paged_prefill_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess) return -3;
    set = true;
  }
  const int G = p.Hq / p.Hkv;
  dim3 grid((max_q_len * G + 63) / 64, p.Hkv, B);
  paged_prefill_kernel<D, MODE><<<grid, kAttnThreads, smem, st>>>(map, p, rows_per_block);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <int D, int MODE>
static int launch_decode(const AttnParams& p, const CUtensorMap& map, long long rows_per_block, int B, cudaStream_t st) {
  const int smem = (16 + 2 * kKvStages * kTileTok) * D * 2 + 1024;   // the fp32 merge area fits inside the K ring
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(paged_decode_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess) return -3;
    set = true;
  }
  dim3 grid(p.Hkv, B, p.num_splits);
  if (launch_pdl(paged_decode_kernel<D, MODE>, grid, dim3(kAttnThreads), smem, st, map, p, rows_per_block) != cudaSuccess)
    return -4;
  if (p.num_splits > 1) {
    if (launch_pdl(decode_reduce_kernel<D>, dim3(p.Hq, B), dim3(D < 128 ? 64 : 128), 0, st, p) != cudaSuccess) return -5;
  }
  return 0;
}

template <int D>
static int dispatch_prefill(const AttnParams& p, int cache_fp8, long long cache_rows, int B, int max_q_len, cudaStream_t st) {
  CUtensorMap map{};
  const long long rpb = p.block_stride / D;
  if (cache_fp8) return launch_prefill<D, kKvFp8>(p, map, rpb, B, max_q_len, st);
  if (tma_ok(p, D) && cache_rows > 0 && make_kv_map(&map, p.cache, cache_rows, D, p.block_tokens))
    return launch_prefill<D, kKvTma>(p, map, rpb, B, max_q_len, st);
  return launch_prefill<D, kKvCpAsync>(p, map, rpb, B, max_q_len, st);
}

template <int D>
static int dispatch_decode(const AttnParams& p, int cache_fp8, long long cache_rows, int B, cudaStream_t st) {
  CUtensorMap map{};
  const long long rpb = p.block_stride / D;
  if (cache_fp8) return launch_decode<D, kKvFp8>(p, map, rpb, B, st);
  if (tma_ok(p, D) && cache_rows > 0 && make_kv_map(&map, p.cache, cache_rows, D, p.block_tokens))
    return launch_decode<D, kKvTma>(p, map, rpb, B, st);
  return launch_decode<D, kKvCpAsync>(p, map, rpb, B, st);
}

}  // namespace ksana

using namespace ksana;

// Causal attention of new query rows against the paged cache (which already holds their K/V).
// cache_rows: number of D-wide rows addressable from `cache` (blocks * block_stride / D); 0 disables the TMA path.
extern "C" int ksana_paged_prefill(const void* q, long long q_stride, void* out, long long out_stride,
                                   const void* cache, long long block_stride, int block_tokens, const int* block_table,
                                   int table_stride, const int* cu_q, const int* kv_lens, const float* alibi, int B,
                                   int max_q_len, int Hq, int Hkv, int D, float scale, int cache_fp8, float k_scale,
                                   float v_scale, long long cache_rows, int* err, cudaStream_t st) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (Hq % Hkv) return -10;
  AttnParams p{};
  p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out; p.out_stride = out_stride;
  p.cache = cache; p.block_stride = block_stride; p.block_tokens = block_tokens;
  p.block_table = block_table; p.table_stride = table_stride; p.cu_q = cu_q; p.kv_lens = kv_lens; p.alibi = alibi;
  p.Hq = Hq; p.Hkv = Hkv; p.scale_log2 = scale * 1.44269504f; p.k_scale = k_scale; p.v_scale = v_scale;
  p.num_splits = 1; p.err = err;
  if (D == 128) return dispatch_prefill<128>(p, cache_fp8, cache_rows, B, max_q_len, st);
  if (D == 64) return dispatch_prefill<64>(p, cache_fp8, cache_rows, B, max_q_len, st);
  return -11;
}

// One new token per sequence. workspace: part_o [B*Hq*splits*D] fp32, part_ml [B*Hq*splits*2] fp32 (splits > 1).
extern "C" int ksana_paged_decode(const void* q, long long q_stride, void* out, long long out_stride,
                                  const void* cache, long long block_stride, int block_tokens, const int* block_table,
                                  int table_stride, const int* kv_lens, const float* alibi, int B, int Hq, int Hkv,
                                  int D, float scale, int cache_fp8, float k_scale, float v_scale, int num_splits,
                                  float* part_o, float* part_ml, long long cache_rows, void* outq, float* oscale,
                                  int oscale_ld, int* err, cudaStream_t st) {
  if (B <= 0) return 0;
  if (outq && (D != 128 || !oscale)) return -13;
  if (Hq % Hkv || Hq / Hkv > 16) return -10;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (!part_o || !part_ml)) return -12;
  AttnParams p{};
  p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out; p.out_stride = out_stride;
  p.cache = cache; p.block_stride = block_stride; p.block_tokens = block_tokens;
  p.block_table = block_table; p.table_stride = table_stride; p.cu_q = nullptr; p.kv_lens = kv_lens; p.alibi = alibi;
  p.Hq = Hq; p.Hkv = Hkv; p.scale_log2 = scale * 1.44269504f; p.k_scale = k_scale; p.v_scale = v_scale;
  p.num_splits = num_splits; p.part_o = part_o; p.part_ml = part_ml; p.err = err;
  p.outq = static_cast<uint8_t*>(outq); p.oscale = oscale; p.oscale_ld = oscale_ld;
  if (D == 128) return dispatch_decode<128>(p, cache_fp8, cache_rows, B, st);
  if (D == 64) return dispatch_decode<64>(p, cache_fp8, cache_rows, B, st);
  return -11;
}
