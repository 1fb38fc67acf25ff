// bf16 GEMM with 256 x 256 output tiles per CTA (two 128-row MMAs share every W tile).
//
//   D[M,N] = A[M,K] * W[N,K]^T (+bias)(+residual), bf16 operands, fp32 accumulation in TMEM
//
// The 128 x 256 tile of gemm_tcgen05.cu needs 48 KB of operands per 64-deep K block of 512 MMA clocks, more than an
// SM takes in from L2 in that time (about 60 bytes per clock, measured on the FP8 kernels). A 256 x 256 tile needs
// 64 KB for twice the MMA work. Its two fp32 accumulators fill all 512 TMEM columns, so the accumulator is not
// double-buffered: the epilogue drains it in two passes and hands it back before its second pass's stores.
// No cluster, no multicast. Every wait is bounded.
//
// CTA layout (320 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..9 epilogue (one
// warpgroup per accumulator). The reference's bf16 GEMMs are cuBLAS / cuBLASLt calls
// (src/ksana_llm/kernels/nvidia/kernel_wrapper.cpp:168-230).
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>
#include <stdio.h>

namespace ksana {

constexpr int kBtBM = 256;
constexpr int kBtBN = 256;
constexpr int kBtRowBytes = 128;
constexpr int kBtThreads = 64 + 256;
constexpr int kBtABytes = kBtBM * kBtRowBytes;
constexpr int kBtBBytes = kBtBN * kBtRowBytes;
constexpr int kBtStageBytes = kBtABytes + kBtBBytes;
constexpr int kBtStages = 3;
constexpr int kBtTmemCols = 512;
constexpr int kBtSmemBytes = kBtStages * kBtStageBytes + 1024 + 512;
constexpr int kBtGroupM = 8;                  // 256-row tiles per raster group
constexpr int kBtPass = kBtBN / 2;            // columns per epilogue pass

struct BtParams {
  int M, N, K;
  __nv_bfloat16* D; float* out_f32; int ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual; int ldr;
  int* err;
  __nv_bfloat16* push[8]; int push_n; int push_rows;
};

__device__ __forceinline__ void bt_tile_coords(int tile, int m_tiles, int n_tiles, int& m_blk, int& n_blk) {
  const int per_group = kBtGroupM * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * kBtGroupM;
  const int gsz = min(m_tiles - first_m, kBtGroupM);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

__global__ void __launch_bounds__(kBtThreads, 1)
gemm_bf16_tall_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const BtParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBtStages * kBtStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = full_bar + kBtStages;
  uint64_t* tfull_bar = empty_bar + kBtStages;
  uint64_t* tempty_bar = tfull_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kBtBM - 1) / kBtBM;
  const int n_tiles = (p.N + kBtBN - 1) / kBtBN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + 63) / 64;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kBtStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kBtTmemCols); tmem_relinquish(); }
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
        bt_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * kBtStageBytes;
          mbar_expect_tx(&full_bar[stage], kBtStageBytes);
          tma_load_2d(sa, &tma_a, &full_bar[stage], kb * 64, m_blk * kBtBM);
          tma_load_2d(sa + kBtABytes, &tma_b, &full_bar[stage], kb * 64, n_blk * kBtBN);
          if (++stage == kBtStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(128, kBtBN, 1, 1);
      int stage = 0; uint32_t phase = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar, acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base, d1 = tmem_base + kBtBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kBtStageBytes);
          const uint64_t adesc0 = make_smem_desc_sw128(sa);
          const uint64_t adesc1 = make_smem_desc_sw128(sa + 128 * kBtRowBytes);
          const uint64_t bdesc = make_smem_desc_sw128(sa + kBtABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            mma_f16(d0, adesc0 + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
            mma_f16(d1, adesc1 + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == kBtStages) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          tc_commit(tfull_bar);
          acc_phase ^= 1;
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int h = (warp - 2) >> 2;                    // accumulator (row half) of this warpgroup
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_blk, n_blk;
      bt_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
      const int row = m_blk * kBtBM + h * 128 + q * 32 + lane;
      const bool row_ok = row < p.M;
      if (!mbar_wait(tfull_bar, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      acc_phase ^= 1;
#pragma unroll 1
      for (int pass = 0; pass < 2; ++pass) {
        const int n0 = n_blk * kBtBN + pass * kBtPass;
        const uint32_t t0 = tmem_base + lane_base + h * kBtBN + pass * kBtPass;
        uint32_t r[kBtPass];
        tmem_ld32(t0, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld32(t0 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_ld32(t0 + 64, *reinterpret_cast<uint32_t(*)[32]>(&r[64]));
        tmem_ld32(t0 + 96, *reinterpret_cast<uint32_t(*)[32]>(&r[96]));
        tmem_ld_wait();
        if (pass == 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar);       // the accumulator is in registers: the next tile may start
        }
        if (!row_ok) continue;
#pragma unroll
        for (int c0 = 0; c0 < kBtPass; c0 += 8) {
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
  }


  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 10);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kBtTmemCols); }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*BtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static BtEncodeFn bt_encode_fn() {
  static BtEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<BtEncodeFn>(ptr);
  }
  return fn;
}
static int bt_map(CUtensorMap* map, const void* base, int rows, int cols, int ld) {
  BtEncodeFn enc = bt_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64, 256};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

}  // namespace ksana

using namespace ksana;

// A [M,K] bf16 (row stride lda), W [N,K] bf16. Output bf16 (D) or fp32 (out_f32). K must be a multiple of 8, N of 8.
extern "C" int ksana_gemm_bf16_tall(const void* A, int lda, const void* W, int ldw, void* D, void* out_f32, int ldd,
                                    const void* bias, const void* residual, int ldr, int M, int N, int K, int max_ctas,
                                    int* err_flag, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (K % 8) || (lda % 8) || (ldw % 8) || (ldd % 8) || (residual && (ldr % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -11;
  CUtensorMap ma, mb;
  if (bt_map(&ma, A, M, K, lda)) return -12;
  if (bt_map(&mb, W, N, K, ldw)) return -13;
  BtParams p{};
  p.M = M; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.out_f32 = static_cast<float*>(out_f32); p.ldd = ldd;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.err = err_flag;
  p.push_n = 0; p.push_rows = 1;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(gemm_bf16_tall_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBtSmemBytes) !=
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
  const int tiles = ((M + kBtBM - 1) / kBtBM) * ((N + kBtBN - 1) / kBtBN);
  int grid = tiles < sms ? tiles : sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  gemm_bf16_tall_kernel<<<grid, kBtThreads, kBtSmemBytes, st>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
