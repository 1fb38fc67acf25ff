// NVFP4 GEMM on the block-scaled tensor-core path (tcgen05.mma kind::mxf4nvf4, 16-element blocks).
//
//   D[M,N] = alpha * (A_q * a_bs)[M,K] * (W_q * w_bs)[N,K]^T (+bias)(+residual),   alpha = a_ts * w_ts
//
// Both operands are e2m1 values, two per byte (even element in the low nibble), with one e4m3 scale per 16
// elements along K ([rows, K/16] bytes) and one fp32 scale per tensor. A 128-byte swizzled shared-memory row
// holds 256 elements = four MMAs of K = 64; each MMA consumes four scales per row, i.e. exactly one 32-bit
// TMEM word of the 512-byte scale chunk (see gemm_tcgen05_mx.cu for the chunk layout). Per K block of 256
// elements the scale warp reads 16 scale bytes per row and writes one chunk per MMA and 128-row group.
// Same warp roles, single 256-column accumulator and bounded waits as the FP8 hardware-scaled kernel.
//
// No counterpart in the reference (its low-bit paths are GPTQ/AWQ W4A16 through Marlin/Machete,
// 3rdparty/LLM_kernels/csrc/kernels/nvidia/mixture_of_experts and .../machete); the operator is specified by
// the fp32 statement in ops/reference.py (gemm_nvfp4).
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>
#include <stdio.h>

namespace ksana {

constexpr int kF4BM = 128;
constexpr int kF4RowBytes = 128;
constexpr int kF4SfStages = 4;
constexpr int kF4Threads = 96 + 256;

template <int BN>
struct F4Cfg {
  static constexpr int kABytes = kF4BM * kF4RowBytes;
  static constexpr int kBBytes = BN * kF4RowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kAccStages = BN == 256 ? 1 : 2;
  static constexpr int kBChunks = BN / 128;
  static constexpr int kSfStageBytes = 4 * (1 + kBChunks) * 512;   // per K block: one A chunk + kBChunks B chunks per MMA
  static constexpr int kSfCols = 4 * 4 * (1 + kBChunks);           // TMEM columns of one scale set (4 MMAs)
  static constexpr int kSfBase = kAccStages * BN;             // first scale column
  static constexpr int kTmemCols = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + kF4SfStages * kSfStageBytes + 1024 + 512;
  static constexpr int kEpiCols = BN / 2;
};

struct F4Params {
  int M, N, K;
  __nv_bfloat16* D; float* out_f32; int ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual; int ldr;
  const uint8_t* a_bs; int a_bs_ld;        // e4m3 block scales [M][K/16], row stride in bytes
  const uint8_t* w_bs; int w_bs_ld;        // [N][K/16]
  const float* a_ts; const float* w_ts;    // per-tensor scales (device scalars)
  int* err;
  __nv_bfloat16* push[8]; int push_n; int push_rows;
  // grouped (mixture-of-experts) mode: row tile i multiplies with expert tile_expert[i] (< 0: tile unused); W, w_bs
  // are the experts' matrices stacked along N (expert_rows rows each) and w_ts holds one tensor scale per expert
  const int* tile_expert; int expert_rows;
};

constexpr int kF4GroupM = 16;
__device__ __forceinline__ void f4_tile_coords(int tile, int m_tiles, int n_tiles, int& m_blk, int& n_blk) {
  const int per_group = kF4GroupM * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * kF4GroupM;
  const int gsz = min(m_tiles - first_m, kF4GroupM);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

template <int BN>
__global__ void __launch_bounds__(kF4Threads, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const F4Params p) {
  using Cfg = F4Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_smem = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_smem + kF4SfStages * Cfg::kSfStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* sf_full = empty_bar + Cfg::kStages;
  uint64_t* sf_empty = sf_full + kF4SfStages;
  uint64_t* tfull_bar = sf_empty + kF4SfStages;
  uint64_t* tempty_bar = tfull_bar + Cfg::kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + Cfg::kAccStages);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kF4BM - 1) / kF4BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = p.K / 256;            // 256 elements = one 128-byte row per stage

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < kF4SfStages; ++i) { mbar_init(&sf_full[i], 1); mbar_init(&sf_empty[i], 1); }
    for (int i = 0; i < Cfg::kAccStages; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], 8); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::kTmemCols); tmem_relinquish(); }
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
        f4_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
        int b_row = n_blk * BN;
        if (p.tile_expert) {
          const int e = p.tile_expert[m_blk];
          if (e < 0) continue;                 // every role skips the tiles of unused row blocks
          b_row += e * p.expert_rows;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_2d(sa, &tma_a, &full_bar[stage], kb * 128, m_blk * kF4BM);
          tma_load_2d(sa + Cfg::kABytes, &tma_b, &full_bar[stage], kb * 128, b_row);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int sfs = 0; uint32_t sf_phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      uint32_t set = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (p.tile_expert) {
          int m_blk, n_blk;
          f4_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
          if (p.tile_expert[m_blk] < 0) continue;
        }
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          if (!mbar_wait(&sf_full[sfs], sf_phase, abort_flag)) { ok = false; break; }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tsf = tmem_base + Cfg::kSfBase + set * Cfg::kSfCols;
          const uint32_t sf_addr = smem_u32(sf_smem + sfs * Cfg::kSfStageBytes);
          constexpr int kPerMma = 1 + Cfg::kBChunks;          // chunks per MMA: A, then the B halves
#pragma unroll
          for (int c = 0; c < 4 * kPerMma; ++c) tmem_cp_sf(tsf + 4 * c, make_sf_desc(sf_addr + 512 * c));
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + Cfg::kABytes);
          constexpr uint32_t idesc = make_idesc_nvf4(kF4BM, BN);
#pragma unroll
          for (int k = 0; k < 4; ++k)      // 64 elements (32 bytes) per MMA, four e4m3 scales per row and MMA
            mma_nvf4(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0, tsf + 4 * kPerMma * k,
                     tsf + 4 * kPerMma * k + 4);
          tc_commit(&empty_bar[stage]);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
          tc_commit(&sf_empty[sfs]);
          if (++sfs == kF4SfStages) { sfs = 0; sf_phase ^= 1; }
          set ^= 1;
        }
        if (ok) {
          tc_commit(&tfull_bar[acc]);
          if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------- scale packer
    int sfs = 0; uint32_t sf_phase = 0;
    bool ok = true;
    constexpr int kPerMma = 1 + Cfg::kBChunks;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_blk, n_blk;
      f4_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
      size_t w_row0 = 0;
      if (p.tile_expert) {
        const int e = p.tile_expert[m_blk];
        if (e < 0) continue;
        w_row0 = static_cast<size_t>(e) * p.expert_rows;
      }
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&sf_empty[sfs], sf_phase ^ 1, abort_flag)) { ok = false; break; }
        uint8_t* buf = sf_smem + sfs * Cfg::kSfStageBytes;
        // rows of A: 16 scale bytes per row and K block = one 32-bit word per MMA
        uint4 ra[4];
#pragma unroll
        for (int r4 = 0; r4 < 4; ++r4) {
          const int row = m_blk * kF4BM + r4 * 32 + lane;
          ra[r4] = row < p.M ? *reinterpret_cast<const uint4*>(p.a_bs + static_cast<size_t>(row) * p.a_bs_ld + kb * 16)
                             : make_uint4(0, 0, 0, 0);
        }
        uint4 rb[Cfg::kBChunks][4];
#pragma unroll
        for (int c = 0; c < Cfg::kBChunks; ++c) {
#pragma unroll
          for (int r4 = 0; r4 < 4; ++r4) {
            const int n = n_blk * BN + c * 128 + r4 * 32 + lane;
            rb[c][r4] = n < p.N ? *reinterpret_cast<const uint4*>(p.w_bs + (w_row0 + n) * p.w_bs_ld + kb * 16)
                                : make_uint4(0, 0, 0, 0);
          }
        }
        auto word = [](const uint4& v, int k) { return k == 0 ? v.x : (k == 1 ? v.y : (k == 2 ? v.z : v.w)); };
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          *reinterpret_cast<uint4*>(buf + (k * kPerMma) * 512 + lane * 16) =
              make_uint4(word(ra[0], k), word(ra[1], k), word(ra[2], k), word(ra[3], k));
#pragma unroll
          for (int c = 0; c < Cfg::kBChunks; ++c)
            *reinterpret_cast<uint4*>(buf + (k * kPerMma + 1 + c) * 512 + lane * 16) =
                make_uint4(word(rb[c][0], k), word(rb[c][1], k), word(rb[c][2], k), word(rb[c][3], k));
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sf_full[sfs]);
        if (++sfs == kF4SfStages) { sfs = 0; sf_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int wg = (warp - 3) >> 2;
    constexpr int EC = Cfg::kEpiCols;
    const int col_off = wg * EC;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_blk, n_blk;
      f4_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
      const int row = m_blk * kF4BM + q * 32 + lane;
      const int n0 = n_blk * BN + col_off;
      const bool row_ok = row < p.M;
      int expert = 0;
      if (p.tile_expert) {
        expert = p.tile_expert[m_blk];
        if (expert < 0) continue;
      }
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t r[EC];
#pragma unroll
      for (int c0 = 0; c0 < EC; c0 += 32) tmem_ld32(tmem_base + lane_base + acc * BN + col_off + c0, *reinterpret_cast<uint32_t(*)[32]>(&r[c0]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);     // the accumulator is in registers: the next tile may start
      if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
      if (!row_ok) continue;
      const float alpha = (p.a_ts ? *p.a_ts : 1.f) * (p.w_ts ? p.w_ts[expert] : 1.f);
#pragma unroll
      for (int c0 = 0; c0 < EC; c0 += 8) {
        const int col = n0 + c0;
        if (col >= p.N) continue;
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[c0 + i]) * alpha;
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
          if (p.push_n) {
            const int owner = min(row / p.push_rows, p.push_n - 1);
            *reinterpret_cast<uint4*>(p.push[owner] + static_cast<size_t>(row - owner * p.push_rows) * p.ldd + col) = ov;
          } else {
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
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 8);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, Cfg::kTmemCols); }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*F4EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static F4EncodeFn f4_encode_fn() {
  static F4EncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<F4EncodeFn>(ptr);
  }
  return fn;
}
static int f4_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  F4EncodeFn enc = f4_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
  cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

template <int BN>
static int launch_f4(const CUtensorMap& ma, const CUtensorMap& mb, const F4Params& p, int max_ctas, cudaStream_t st) {
  using Cfg = F4Cfg<BN>;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(gemm_nvfp4_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) !=
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
  const int tiles = ((p.M + kF4BM - 1) / kF4BM) * ((p.N + BN - 1) / BN);
  int grid = tiles < sms ? tiles : sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  gemm_nvfp4_kernel<BN><<<grid, kF4Threads, Cfg::kSmemBytes, st>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace ksana

using namespace ksana;

// A_q [M, K/2] packed e2m1 (row stride lda bytes), a_bs [M, K/16] e4m3 bytes (row stride a_bs_ld), a_ts device fp32
// scalar (null = 1); W likewise with N rows. K must be a multiple of 256, N of 8; strides multiples of 16 bytes.
// Output bf16 (D) or fp32 (out_f32). bn_hint: 128, 256 or 0 (automatic).
extern "C" int ksana_gemm_nvfp4(const void* Aq, int lda, const void* a_bs, int a_bs_ld, const float* a_ts, const void* Wq,
                                int ldw, const void* w_bs, int w_bs_ld, const float* w_ts, void* D, void* out_f32, int ldd,
                                const void* bias, const void* residual, int ldr, int M, int N, int K, int bn_hint,
                                int max_ctas, int* err_flag, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (K % 256) || (lda % 16) || (ldw % 16) || (a_bs_ld % 16) || (w_bs_ld % 16) || (ldd % 8) ||
      (residual && (ldr % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Wq) | reinterpret_cast<uintptr_t>(a_bs) |
       reinterpret_cast<uintptr_t>(w_bs)) & 15) return -11;
  int bn = bn_hint;
  if (bn != 128 && bn != 256) {
    const int m_tiles = (M + kF4BM - 1) / kF4BM;
    bn = (m_tiles * ((N + 255) / 256) >= 100) ? 256 : 128;
  }
  CUtensorMap ma, mb;
  if (f4_map(&ma, Aq, M, K / 2, lda, kF4BM)) return -12;
  if (f4_map(&mb, Wq, N, K / 2, ldw, bn)) return -13;
  F4Params p{};
  p.M = M; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.out_f32 = static_cast<float*>(out_f32); p.ldd = ldd;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.a_bs = static_cast<const uint8_t*>(a_bs); p.a_bs_ld = a_bs_ld;
  p.w_bs = static_cast<const uint8_t*>(w_bs); p.w_bs_ld = w_bs_ld;
  p.a_ts = a_ts; p.w_ts = w_ts;
  p.err = err_flag;
  return bn == 256 ? launch_f4<256>(ma, mb, p, max_ctas, st) : launch_f4<128>(ma, mb, p, max_ctas, st);
}

// Grouped (mixture-of-experts) form: A_q [cap, K/2] holds expert-major rows in 128-row tiles, tile_expert[cap / 128]
// names the expert of every tile (-1: unused, nothing is computed or stored for it). W_q [E * N, K/2], w_bs
// [E * N, K/16] are the experts' matrices stacked along N, w_ts [E] their tensor scales. N must be a multiple of 128.
extern "C" int ksana_gemm_grouped_nvfp4(const void* Aq, int lda, const void* a_bs, int a_bs_ld, const float* a_ts,
                                        const void* Wq, int ldw, const void* w_bs, int w_bs_ld, const float* w_ts,
                                        void* D, int ldd, int cap, int N, int K, int num_experts, const int* tile_expert,
                                        int bn_hint, int* err_flag, cudaStream_t st) {
  if (cap <= 0 || N <= 0 || K <= 0 || num_experts <= 0) return 0;
  if ((cap % 128) || (N % 128) || (K % 256) || (lda % 16) || (ldw % 16) || (a_bs_ld % 16) || (w_bs_ld % 16) || (ldd % 8) ||
      tile_expert == nullptr || w_ts == nullptr) return -10;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Wq) | reinterpret_cast<uintptr_t>(a_bs) |
       reinterpret_cast<uintptr_t>(w_bs)) & 15) return -11;
  // a weight tile must not reach into the next expert's rows
  int bn = (bn_hint == 128 || (N % 256)) ? 128 : 256;
  CUtensorMap ma, mb;
  if (f4_map(&ma, Aq, cap, K / 2, lda, kF4BM)) return -12;
  if (f4_map(&mb, Wq, num_experts * N, K / 2, ldw, bn)) return -13;
  F4Params p{};
  p.M = cap; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.a_bs = static_cast<const uint8_t*>(a_bs); p.a_bs_ld = a_bs_ld;
  p.w_bs = static_cast<const uint8_t*>(w_bs); p.w_bs_ld = w_bs_ld;
  p.a_ts = a_ts; p.w_ts = w_ts;
  p.err = err_flag;
  p.tile_expert = tile_expert; p.expert_rows = N;
  return bn == 256 ? launch_f4<256>(ma, mb, p, 0, st) : launch_f4<128>(ma, mb, p, 0, st);
}
