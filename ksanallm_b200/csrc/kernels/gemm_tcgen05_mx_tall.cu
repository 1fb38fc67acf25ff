// Hardware block-scaled FP8 GEMM with 256 x 224 output tiles per CTA (two 128-row MMAs share every W tile).
//
//   D[M,N] = (A_q * a_scale)[M,K] * (W_q * w_scale)[N,K]^T (+bias)(+residual)
//
// Operands and restrictions are those of gemm_tcgen05_mx.cu (e4m3 values, power-of-two scales: one per activation
// row and 128 K-elements stored [K/128][ld], one per 128 x 128 weight block). That kernel's 128 x 256 tile needs
// 48 KB of operands per 128-deep K block, and what an SM can take in per clock from L2 (about 60 bytes, measured:
// the producer's ring stays full while the MMA thread waits for data) then holds the tensor pipe below 60 %.
// A 256 x 224 tile needs 60 KB per K block for 1.75 times the MMA work (34 KB per 128 x 256 equivalent). It is
// the largest tile whose two fp32 accumulators (2 x 224 TMEM columns) leave room for the scale columns. No
// cluster, no multicast. Every wait is bounded.
//
// CTA layout (352 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warp 2 scale packer, warps 3..10
// epilogue (one warpgroup per accumulator, each drains its 224 columns in two passes of 112).
//
// Scale factors: per group of four K blocks the packer writes four 512-byte chunks (rows 0..127, rows 128..255,
// columns 0..127, columns 128..223 of the tile; layout of gemm_tcgen05_mx.cu) and tcgen05.cp puts them into 16
// TMEM columns. A 224-wide tile starts at a multiple of 32 columns, so every 32-column run of a W chunk lies in
// one 128 x 128 weight block.
//
// The reference has no counterpart (its FP8 GEMMs are cuBLASLt per-tensor or DeepGEMM on Hopper:
// src/ksana_llm/kernels/nvidia/kernel_wrapper.cpp:1014-1048).
#include "sm100_ptx.cuh"
#include "push_epilogue.cuh"
#include <cuda_bf16.h>
#include <stdio.h>

namespace ksana {

constexpr int kTlBM = 256;
constexpr int kTlBN = 224;
constexpr int kTlRowBytes = 128;
constexpr int kTlThreads = 96 + 256;
constexpr int kTlABytes = kTlBM * kTlRowBytes;
constexpr int kTlBBytes = kTlBN * kTlRowBytes;
constexpr int kTlStageBytes = kTlABytes + kTlBBytes;
constexpr int kTlStages = 3;
constexpr int kTlSfStages = 4;
constexpr int kTlSfStageBytes = 4 * 512;
constexpr int kTlSfCols = 16;                 // TMEM columns of one scale set: 2 x 4 (rows) + 2 x 4 (columns)
constexpr int kTlSfBase = 2 * kTlBN;          // first scale column
constexpr int kTlTmemCols = 512;
constexpr int kTlSmemBytes = kTlStages * kTlStageBytes + kTlSfStages * kTlSfStageBytes + 1024 + 512 + 8 * kPushStageBytes;
constexpr int kTlGroupM = 8;                  // 256-row tiles per raster group
constexpr int kTlPass = kTlBN / 2;            // columns per epilogue pass

struct TallParams {
  int M, N, K;
  __nv_bfloat16* D; float* out_f32; int ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual; int ldr;
  const float* a_scale; int a_scale_ld;
  const float* w_scale;
  int* err;
  __nv_bfloat16* push[8]; int push_n; int push_rows;
};

__device__ __forceinline__ void tl_tile_coords(int tile, int m_tiles, int n_tiles, int& m_blk, int& n_blk) {
  const int per_group = kTlGroupM * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * kTlGroupM;
  const int gsz = min(m_tiles - first_m, kTlGroupM);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

__global__ void __launch_bounds__(kTlThreads, 1)
gemm_mxfp8_tall_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                       const TallParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_smem = smem + kTlStages * kTlStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_smem + kTlSfStages * kTlSfStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = full_bar + kTlStages;
  uint64_t* sf_full = empty_bar + kTlStages;
  uint64_t* sf_empty = sf_full + kTlSfStages;
  uint64_t* tfull_bar = sf_empty + kTlSfStages;
  uint64_t* tempty_bar = tfull_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint8_t* epi_stage = reinterpret_cast<uint8_t*>(bars) + 512;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kTlBM - 1) / kTlBM;
  const int n_tiles = (p.N + kTlBN - 1) / kTlBN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = p.K / 128;
  const int num_groups = (num_kb + 3) / 4;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kTlStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < kTlSfStages; ++i) { mbar_init(&sf_full[i], 1); mbar_init(&sf_empty[i], 1); }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kTlTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        tl_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * kTlStageBytes;
          mbar_expect_tx(&full_bar[stage], kTlStageBytes);
          tma_load_2d(sa, &tma_a, &full_bar[stage], kb * 128, m_blk * kTlBM);
          tma_load_2d(sa + kTlABytes, &tma_b, &full_bar[stage], kb * 128, n_blk * kTlBN);
          if (++stage == kTlStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int sfs = 0; uint32_t sf_phase = 0;
      uint32_t acc_phase = 0;
      uint32_t set = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar, acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base, d1 = tmem_base + kTlBN;
        for (int g = 0; g < num_groups && ok; ++g) {
          if (!mbar_wait(&sf_full[sfs], sf_phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tsfa = tmem_base + kTlSfBase + set * kTlSfCols;
          const uint32_t tsfb = tsfa + 8;
          const uint32_t sf_addr = smem_u32(sf_smem + sfs * kTlSfStageBytes);
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_cp_sf(tsfa + 4 * c, make_sf_desc(sf_addr + 512 * c));
          for (int j = 0; j < 4; ++j) {
            const int kb = g * 4 + j;
            if (kb >= num_kb) break;
            if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * kTlStageBytes);
            const uint64_t adesc0 = make_smem_desc_sw128(sa);
            const uint64_t adesc1 = make_smem_desc_sw128(sa + 128 * kTlRowBytes);
            const uint64_t bdesc = make_smem_desc_sw128(sa + kTlABytes);
            const uint32_t idesc = make_idesc_mx(128, kTlBN, static_cast<uint32_t>(j));
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              mma_mxf8(d0, adesc0 + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0, tsfa, tsfb);
              mma_mxf8(d1, adesc1 + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0, tsfa + 4, tsfb);
            }
            tc_commit(&empty_bar[stage]);
            if (++stage == kTlStages) { stage = 0; phase ^= 1; }
          }
          tc_commit(&sf_empty[sfs]);
          if (++sfs == kTlSfStages) { sfs = 0; sf_phase ^= 1; }
          set ^= 1;
        }
        if (ok) {
          tc_commit(tfull_bar);
          acc_phase ^= 1;
        }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------- scale packer
    // The scale values of the next two groups are already on their way (plain loads whose results are not
    // touched until their turn) while the warp waits for the buffer of the current group. Three register sets
    // rotate by name, not by index, so that no load result is moved (a move would wait for it).
    int sfs = 0; uint32_t sf_phase = 0;
    const int n_blocks = (p.N + 127) / 128;
    struct Raw { float a[32]; float b[12]; int off; };
    auto fetch = [&](int tile, int g, Raw& r) {
      int m_blk, n_blk;
      tl_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
      const int m0 = m_blk * kTlBM;
#pragma unroll
      for (int r8 = 0; r8 < 8; ++r8) {
        const int row = min(m0 + r8 * 32 + lane, p.M - 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kb = min(g * 4 + j, num_kb - 1);
          r.a[r8 * 4 + j] = __ldg(p.a_scale + static_cast<size_t>(kb) * p.a_scale_ld + row);
        }
      }
      const int n0 = n_blk * kTlBN;
      r.off = n0 & 127;
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        const int nb = min(n0 / 128 + t, n_blocks - 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kb = min(g * 4 + j, num_kb - 1);
          r.b[t * 4 + j] = __ldg(p.w_scale + static_cast<size_t>(nb) * num_kb + kb);
        }
      }
    };
    // rows past M, column blocks past N and K blocks past the end repeat the last valid scale: what they scale
    // is zero-filled by TMA or never stored
    auto emit = [&](const Raw& r) -> bool {
      if (!mbar_wait(&sf_empty[sfs], sf_phase ^ 1, abort_flag)) return false;
      uint8_t* buf = sf_smem + sfs * kTlSfStageBytes;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t w[4];
#pragma unroll
        for (int r4 = 0; r4 < 4; ++r4) {
          uint32_t word = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) word |= ue8m0_of(r.a[(h * 4 + r4) * 4 + j]) << (8 * j);
          w[r4] = word;
        }
        *reinterpret_cast<uint4*>(buf + h * 512 + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      uint32_t bw[3];
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) word |= ue8m0_of(r.b[t * 4 + j]) << (8 * j);
        bw[t] = word;
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = (r.off + c * 128 + i * 32) >> 7;            // weight block of this 32-column run: 0..2
          w[i] = idx == 0 ? bw[0] : (idx == 1 ? bw[1] : bw[2]);
        }
        *reinterpret_cast<uint4*>(buf + 1024 + c * 512 + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_async_smem();          // the tensor core reads the chunks through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&sf_full[sfs]);
      if (++sfs == kTlSfStages) { sfs = 0; sf_phase ^= 1; }
      return true;
    };
    // (tile, group) sequence of this CTA; `ahead` runs two steps in front of `cur`
    int ct = static_cast<int>(blockIdx.x), cg = 0, at = ct, ag = 0;
    auto advance = [&](int& t, int& g) { if (++g == num_groups) { g = 0; t += static_cast<int>(gridDim.x); } };
    Raw r0, r1, r2;
    if (at < num_tiles) { fetch(at, ag, r0); advance(at, ag); }
    if (at < num_tiles) { fetch(at, ag, r1); advance(at, ag); }
    while (ct < num_tiles) {
      if (at < num_tiles) { fetch(at, ag, r2); advance(at, ag); }
      if (!emit(r0)) break;
      advance(ct, cg);
      if (ct >= num_tiles) break;
      if (at < num_tiles) { fetch(at, ag, r0); advance(at, ag); }
      if (!emit(r1)) break;
      advance(ct, cg);
      if (ct >= num_tiles) break;
      if (at < num_tiles) { fetch(at, ag, r1); advance(at, ag); }
      if (!emit(r2)) break;
      advance(ct, cg);
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int h = (warp - 3) >> 2;                    // accumulator (row half) of this warpgroup
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_blk, n_blk;
      tl_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
      const int row = m_blk * kTlBM + h * 128 + q * 32 + lane;
      const bool row_ok = row < p.M;
      if (!mbar_wait(tfull_bar, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      acc_phase ^= 1;
#pragma unroll 1
      for (int pass = 0; pass < 2; ++pass) {
        const int n0 = n_blk * kTlBN + pass * kTlPass;
        const uint32_t t0 = tmem_base + lane_base + h * kTlBN + pass * kTlPass;
        uint32_t r[kTlPass];
        tmem_ld32(t0, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld32(t0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_ld32(t0 + 64, *reinterpret_cast<uint32_t(*)[32]>(&r[64]));
        tmem_ld16(t0 + 96, *reinterpret_cast<uint32_t(*)[16]>(&r[96]));
        tmem_ld_wait();
        if (pass == 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar);       // the accumulator is in registers: the next tile may start
        }
        if (p.push_n && !p.out_f32) {
          // rows for the peers: one contiguous run of kTlPass columns (224 bytes) per row (see push_epilogue.cuh)
          push_rows_staged<kTlPass>(epi_stage + (warp - 3) * kPushStageBytes, r, p.bias, lane,
                                    m_blk * kTlBM + h * 128 + q * 32, n0, p.M, p.N, p.push, p.push_n, p.push_rows, p.ldd);
          continue;
        }
        if (!row_ok) continue;
#pragma unroll
        for (int c0 = 0; c0 < kTlPass; c0 += 8) {
          const int col = n0 + c0;
          if (col >= p.N) continue;
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[c0 + i]);
          if (p.bias) {
            const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(b2[i]); o[2 * i] += f.x; o[2 * i + 1] += f.y; }
          }
          if (p.residual) {
            const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(row) * p.ldr + col);
            const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(r2[i]); o[2 * i] += f.x; o[2 * i + 1] += f.y; }
          }
          if (p.out_f32) {
            float4* dst = reinterpret_cast<float4*>(p.out_f32 + static_cast<size_t>(row) * p.ldd + col);
            dst[0] = make_float4(o[0], o[1], o[2], o[3]);
            dst[1] = make_float4(o[4], o[5], o[6], o[7]);
          } else {
            uint4 ov;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
            for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
            *reinterpret_cast<uint4*>(p.D + static_cast<size_t>(row) * p.ldd + col) = ov;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 9);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kTlTmemCols); }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*TlEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TlEncodeFn tl_encode_fn() {
  static TlEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<TlEncodeFn>(ptr);
  }
  return fn;
}
static int tl_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  TlEncodeFn enc = tl_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
  cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

}  // namespace ksana

using namespace ksana;

// Same operands as ksana_gemm_mxfp8 (scales must be powers of two). K must be a multiple of 128, N of 8.
extern "C" int ksana_gemm_mxfp8_tall(const void* Aq, int lda, const float* a_scale, int a_scale_ld, const void* Wq, int ldw,
                                     const float* w_scale, void* D, void* out_f32, int ldd, const void* bias,
                                     const void* residual, int ldr, int M, int N, int K, int max_ctas,
                                     const unsigned long long* push_ptrs, int push_n, int push_rows, int* err_flag,
                                     cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (K % 128) || (lda % 16) || (ldw % 16) || (ldd % 8) || (residual && (ldr % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Wq)) & 15) return -11;
  CUtensorMap ma, mb;
  if (tl_map(&ma, Aq, M, K, lda, kTlBM)) return -12;
  if (tl_map(&mb, Wq, N, K, ldw, kTlBN)) return -13;
  TallParams p{};
  p.M = M; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.out_f32 = static_cast<float*>(out_f32); p.ldd = ldd;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.a_scale = a_scale; p.a_scale_ld = a_scale_ld; p.w_scale = w_scale;
  p.err = err_flag;
  for (int i = 0; i < push_n && i < 8; ++i) p.push[i] = reinterpret_cast<__nv_bfloat16*>(push_ptrs[i]);
  p.push_n = push_n; p.push_rows = push_rows;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(gemm_mxfp8_tall_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTlSmemBytes) !=
        cudaSuccess) return -3;
    set = true;
  }
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int tiles = ((M + kTlBM - 1) / kTlBM) * ((N + kTlBN - 1) / kTlBN);
  int grid = tiles < sms ? tiles : sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  gemm_mxfp8_tall_kernel<<<grid, kTlThreads, kTlSmemBytes, st>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
