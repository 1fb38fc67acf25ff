// Prefill (and chunked-prefill) attention on the tcgen05 tensor cores: causal attention of new query rows
// against the paged KV cache, head dimension 128, bf16 cache.
//
// One CTA owns 128 packed query rows of one KV head group: row = (token, head inside the group), so the G query
// heads that share a KV head reuse every staged K/V tile (G must divide 128). Per 128-token KV tile:
//   S = Q K^T      tcgen05.mma, both operands K-major in shared memory (TMA, 128-byte swizzle), S in TMEM
//   softmax        4 warps, one thread per row (TMEM lane): no cross-thread reductions; online max with a
//                  lazy rescale of O (only when a row's maximum grew by more than 2^8)
//   O += P V       tcgen05.mma with P read from TMEM (bf16 pairs written over S's columns by the softmax warps)
//                  and V as an MN-major shared-memory operand, O accumulating in TMEM
// Warp roles: warp 0 TMA producer (Q once; K and V tiles through the block table, one box per cache block and
// 64-column panel), warp 1 MMA issuer + TMEM owner, warps 2..5 softmax + epilogue. Two CTAs share an SM
// (96 KB of shared memory, 256 TMEM columns each), so one CTA's softmax overlaps the other's MMAs.
// Every wait is bounded; a timeout sets the error word and leaves the output untouched.
//
// Same operator as the reference's flash-attention prefill call plus its separate prefix-cache gather
// (src/ksana_llm/layers/flash_attention_layer.cpp, 3rdparty/LLM_kernels/csrc/kernels/nvidia/paged_attention):
// here K/V are read in place from the paged cache.
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>
#include <math_constants.h>
#include <stdio.h>

namespace ksana {

typedef __nv_bfloat16 bf16;
constexpr int kFaThreads = 192;
constexpr int kFaTile = 128;                 // query rows per CTA and KV tokens per tile
constexpr int kFaD = 128;
constexpr int kFaPanelBytes = kFaTile * 128; // one 64-column panel of a 128-row tile
constexpr int kFaTileBytes = 2 * kFaPanelBytes;
constexpr int kFaSmemBytes = 3 * kFaTileBytes + 1024 + 256;
constexpr uint32_t kFaTmemCols = 256;        // S / P at columns [0,128), O at [128,256)
constexpr float kFaRescaleLog2 = 8.f;        // O is rescaled only when a row maximum grew by more than this

struct FaParams {
  bf16* out; long long out_stride;
  const int* block_table; int table_stride;
  const int* cu_q; const int* kv_lens; const float* alibi;
  int Hq, Hkv, G, block_tokens;
  long long rows_per_block;                  // cache rows (of D elements) between consecutive blocks
  float scale_log2;
  int* err;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kFaThreads, 2)
prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map, const FaParams p) {
  extern __shared__ uint8_t fa_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = smem + kFaTileBytes;
  uint8_t* v_s = smem + 2 * kFaTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kFaTileBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* o_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.z, g = blockIdx.y;
  const int G = p.G;
  const int q0 = p.cu_q[s], q_len = p.cu_q[s + 1] - q0;
  const int kv_len = p.kv_lens[s];
  const int qtile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);   // longest rows first
  const int row0 = qtile * kFaTile;
  if (row0 >= q_len * G) return;
  const int past = kv_len - q_len;
  const int last_row = min(row0 + kFaTile - 1, q_len * G - 1);
  const int kv_end = min(kv_len, past + last_row / G + 1);
  const int ntiles = (kv_end + kFaTile - 1) / kFaTile;
  const int* table = p.block_table + static_cast<size_t>(s) * p.table_stride;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(k_full, 1); mbar_init(k_empty, 1); mbar_init(v_full, 1); mbar_init(v_empty, 1);
    mbar_init(s_full, 1); mbar_init(p_full, 4); mbar_init(o_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kFaTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&q_map);
      tma_prefetch_desc(&kv_map);
      mbar_expect_tx(q_full, kFaTileBytes);
      const int tok0 = q0 + row0 / G;
      tma_load_3d(q_s, &q_map, q_full, 0, g * G, tok0);
      tma_load_3d(q_s + kFaPanelBytes, &q_map, q_full, 64, g * G, tok0);
      const int bt = p.block_tokens;
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int t0 = j * kFaTile;
        const int nblk = min(kFaTile / bt, (kv_len - t0 + bt - 1) / bt);
        const uint32_t bytes = static_cast<uint32_t>(nblk) * 2 * bt * 128;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          uint64_t* full = which ? v_full : k_full;
          uint64_t* empty = which ? v_empty : k_empty;
          uint8_t* dst = which ? v_s : k_s;
          if (!mbar_wait(empty, (j & 1) ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full, bytes);
          for (int b = 0; b < nblk; ++b) {
            const long long r0 = static_cast<long long>(table[t0 / bt + b]) * p.rows_per_block +
                                 (static_cast<long long>(which) * p.Hkv + g) * bt;
            tma_load_2d(dst + b * bt * 128, &kv_map, full, 0, static_cast<int>(r0));
            tma_load_2d(dst + kFaPanelBytes + b * bt * 128, &kv_map, full, 64, static_cast<int>(r0));
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(128, 128, 1, 1);
      constexpr uint32_t idesc_pv = make_idesc(128, 128, 1, 1) | (1u << 16);     // B (= V) is MN-major
      bool ok = mbar_wait(q_full, 0, abort_flag);
      for (int j = 0; j < ntiles && ok; ++j) {
        const uint32_t par = j & 1;
        if (!mbar_wait(k_full, par, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kFaPanelBytes;
          const uint64_t adesc = make_smem_desc_sw128(smem_u32(q_s) + off) + 2 * (k & 3);
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(k_s) + off) + 2 * (k & 3);
          mma_f16(tmem_s, adesc, bdesc, idesc_qk, k != 0);
        }
        tc_commit(s_full);
        tc_commit(k_empty);
        if (!mbar_wait(v_full, par, abort_flag)) { ok = false; break; }
        if (!mbar_wait(p_full, par, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // 16 tokens per MMA: 8 TMEM columns of P (two bf16 each), 16 rows (2 KB) of the V tile
          const uint64_t bdesc = make_smem_desc_mn_sw128(smem_u32(v_s) + k * 2048, kFaPanelBytes);
          mma_f16_ts(tmem_o, tmem_s + 8 * k, bdesc, idesc_pv, (j | k) != 0);
        }
        tc_commit(v_empty);
        if (j == ntiles - 1) tc_commit(o_full);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (one thread per row)
    const int qd = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const int vr = row0 + qd * 32 + lane;                  // packed row index inside the sequence
    const bool active = vr < q_len * G;
    const int tok = vr / G, head = g * G + vr % G;
    const int limit = active ? past + tok : -1;            // last visible KV position
    const float slope2 = (p.alibi && active) ? p.alibi[head] * 1.44269504f : 0.f;
    float m_used = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const uint32_t par = j & 1;
      const int t0 = j * kFaTile;
      if (!mbar_wait(s_full, par, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (t0 + kFaTile - 1 > limit) || slope2 != 0.f || p.scale_log2 <= 0.f;
      // lazy rescale of O: keep the old reference maximum unless the row's maximum grew by more than 2^8
      auto update_reference = [&](float mx) {
        float m_new = m_used;
        if (mx > m_used + kFaRescaleLog2 || m_used == -CUDART_INF_F) m_new = (mx == -CUDART_INF_F) ? m_used : mx;
        const bool grow = j > 0 && m_new != m_used && m_used != -CUDART_INF_F;
        if (__any_sync(0xffffffffu, grow)) {
          const float f = grow ? exp2f(m_used - m_new) : 1.f;
          l *= f;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem_o + lane_off + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tmem_st32(tmem_o + lane_off + c * 32, o);
          }
        }
        m_used = m_new;
        return (m_used == -CUDART_INF_F) ? 0.f : m_used;
      };
      if (!__any_sync(0xffffffffu, need_mask)) {
        // interior tile: the whole row in registers with a single TMEM round trip
        uint32_t r[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s + lane_off + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
        tmem_ld_wait();
        float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int i = 0; i < 128; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i]));
        const float mref = update_reference(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2);
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 128; i += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, -mref));
          const float p1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -mref));
          l4[(i >> 1) & 3] += p0 + p1;
          __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
          r[i >> 1] = *reinterpret_cast<uint32_t*>(&pb);        // in place: slot i/2 has already been consumed
        }
        l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_st16(tmem_s + lane_off + c * 16, *reinterpret_cast<uint32_t(*)[16]>(&r[c * 16]));
      } else {
        // diagonal / last / ALiBi tile: masked two-pass form
        float mx = -CUDART_INF_F;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_s + lane_off + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int pos = t0 + c * 32 + i;
            const float v = __uint_as_float(r[i]) * p.scale_log2 + slope2 * static_cast<float>(pos - limit);
            mx = fmaxf(mx, pos <= limit ? v : -CUDART_INF_F);
          }
        }
        const float mref = update_reference(mx);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_s + lane_off + c * 32, r);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int pos = t0 + c * 32 + i;
            const float v0 = __uint_as_float(r[i]) * p.scale_log2 + slope2 * static_cast<float>(pos - limit) - mref;
            const float v1 = __uint_as_float(r[i + 1]) * p.scale_log2 + slope2 * static_cast<float>(pos + 1 - limit) - mref;
            const float p0 = pos <= limit ? fast_exp2(v0) : 0.f;
            const float p1 = pos + 1 <= limit ? fast_exp2(v1) : 0.f;
            l += p0 + p1;
            __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
            pk[i >> 1] = *reinterpret_cast<uint32_t*>(&pb);
          }
          tmem_st16(tmem_s + lane_off + c * 16, pk);
        }
      }
      tmem_st_wait();
      if (t0 + kFaTile > kv_len) {
        // last tile of the sequence: V rows past the sequence end hold stale shared memory or whatever the cache
        // has there; their probabilities are 0, but 0 x NaN would poison O. Zero them before the PV MMA reads.
        if (!mbar_wait(v_full, par, abort_flag)) { ok = false; break; }
        const int first_bad = kv_len - t0;
        const int nchunks = (kFaTile - first_bad) * 16;       // 16-byte chunks per row: 2 panels x 8
        for (int i = threadIdx.x - 64; i < nchunks; i += 128) {
          const int r = first_bad + (i >> 4), ch = i & 15;
          *reinterpret_cast<uint4*>(v_s + (ch >> 3) * kFaPanelBytes + r * 128 + (((ch & 7) ^ (r & 7)) << 4)) =
              make_uint4(0, 0, 0, 0);
        }
        fence_async_smem();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && mbar_wait(o_full, 0, abort_flag)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + static_cast<size_t>(q0 + tok) * p.out_stride + head * kFaD;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_o + lane_off + c * 32, r);
        tmem_ld_wait();
        if (active) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 ov;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              o2[e] = __floats2bfloat162_rn(__uint_as_float(r[i + 2 * e]) * inv, __uint_as_float(r[i + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = ov;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 7);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kFaTmemCols); }
}

typedef CUresult (*FaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static FaEncodeFn fa_encode_fn() {
  static FaEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<FaEncodeFn>(ptr);
  }
  return fn;
}

}  // namespace ksana

using namespace ksana;

// Returns 0 when launched, -100 when this kernel does not cover the configuration (the caller then uses the
// general kernel of attention.cu), other negatives on setup errors.
// q: [T, q_stride] bf16 with head h at column h*128 (T = rows addressable from q); cache: layer base of
// [block][2][Hkv][block_tokens][128] bf16, blocks block_stride elements apart, cache_rows rows of 128 elements
// addressable.
extern "C" int ksana_paged_prefill_tc(const void* q, long long q_stride, long long q_rows, void* out, long long out_stride,
                                      const void* cache, long long block_stride, int block_tokens,
                                      const int* block_table, int table_stride, const int* cu_q, const int* kv_lens,
                                      const float* alibi, int B, int max_q_len, int Hq, int Hkv, int D, float scale,
                                      long long cache_rows, int* err, cudaStream_t st) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (D != kFaD || Hkv <= 0 || Hq % Hkv) return -100;
  const int G = Hq / Hkv;
  const int bt = block_tokens;
  if (kFaTile % G || G > 128 || !(bt == 8 || bt == 16 || bt == 32 || bt == 64 || bt == 128)) return -100;
  if (block_stride % D || block_stride < 2LL * Hkv * bt * D || cache_rows <= 0 || q_rows <= 0) return -100;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache)) & 15 || (q_stride % 8)) return -100;
  FaEncodeFn enc = fa_encode_fn();
  if (!enc) return -100;
  CUtensorMap q_map, kv_map;
  {
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(Hq), static_cast<cuuint64_t>(q_rows)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(q_stride) * 2};
    cuuint32_t box[3] = {64, static_cast<cuuint32_t>(G), static_cast<cuuint32_t>(kFaTile / G)};
    cuuint32_t estr[3] = {1, 1, 1};
    if (enc(&q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -100;
  }
  {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(cache_rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(D) * 2};
    cuuint32_t box[2] = {64, static_cast<cuuint32_t>(bt)};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&kv_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -100;
  }
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFaSmemBytes) != cudaSuccess)
      return -3;
    set = true;
  }
  FaParams p{};
  p.out = static_cast<bf16*>(out); p.out_stride = out_stride;
  p.block_table = block_table; p.table_stride = table_stride; p.cu_q = cu_q; p.kv_lens = kv_lens; p.alibi = alibi;
  p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.block_tokens = bt;
  p.rows_per_block = block_stride / D;        // a block of one layer may sit inside a larger per-block record
  p.scale_log2 = scale * 1.44269504f;
  p.err = err;
  dim3 grid((max_q_len * G + kFaTile - 1) / kFaTile, Hkv, B);
  prefill_tc_kernel<<<grid, kFaThreads, kFaSmemBytes, st>>>(q_map, kv_map, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
