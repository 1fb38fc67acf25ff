// Dense GEMMs for sm_100a on the 5th-generation tensor cores.
//
//   D[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) (+ residual[M,N])
//
// Two operand kinds share one warp-specialised persistent kernel:
//   * bf16 x bf16 (tcgen05.mma kind::f16), the whole K loop accumulates in TMEM;
//   * fp8-e4m3 x fp8-e4m3 with fine-grained scales (kind::f8f6f4): activations
//     carry one fp32 scale per (row, 128-wide K group), weights one per
//     (128 x 128) block. Each 128-deep K block is multiplied into a fresh TMEM
//     accumulator and promoted into fp32 registers with its scale product, so
//     the scales stay exact fp32 (no power-of-two restriction).
//
// CTA layout (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA
// issuer (one elected lane), warps 2..5 = epilogue (each owns the 32 TMEM lanes
// its warp id modulo 4 selects). Operand tiles are 128-byte-swizzled rows
// written by TMA into a multi-stage shared-memory ring; accumulators are
// multi-buffered in TMEM so the epilogue of tile i overlaps the MMAs of tile
// i+1. No cluster multicast is used anywhere, so the kernel is safe in
// multi-GPU processes.
//
// Replaces the cuBLASLt wrapper of the reference
// (3rdparty/LLM_kernels/csrc/kernels/nvidia/gemm_wrapper/gemm_wrapper.cc:24-125)
// and its per-tensor FP8 path (src/ksana_llm/kernels/nvidia/kernel_wrapper.cpp:1014-1048).
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdio.h>

namespace ksana {

constexpr int kBM = 128;          // rows per tile = TMEM lanes
constexpr int kRowBytes = 128;    // one swizzled smem row: 64 bf16 or 128 fp8
constexpr int kSmemBudget = 200 * 1024;

enum GemmKind { kBf16 = 0, kFp8Block = 1 };

struct GemmParams {
  int M, N, K;
  __nv_bfloat16* D;       // bf16 output (may be null when out_f32 is set)
  float* out_f32;         // optional fp32 output
  int ldd;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  int ldr;
  const float* a_scale;   // fp8: [K/128][a_scale_ld]   (k-group major, contiguous over rows)
  int a_scale_ld;
  const float* w_scale;   // fp8: [ceil(N/128)][K/128]
  int* err;               // device word, set non-zero when a bounded wait gave up
  // grouped (mixture-of-experts) mode: row tile i multiplies with expert tile_expert[i] (< 0: tile unused);
  // W stacks the experts as [E * expert_rows, K] and w_scale as [E * scale_rows_per_expert][K/128].
  const int* tile_expert;
  int expert_rows;
  int scale_rows_per_expert;
  // push mode (tensor-parallel row-parallel linear): rows [r*push_rows, (r+1)*push_rows) of the partial
  // product are stored into rank r's receive slot for this rank (peer memory, plain P2P stores) instead of D.
  __nv_bfloat16* push[8];
  int push_n;
  int push_rows;
  // batched mode (bf16 only, batch > 0): `batch` independent products D_b = A_b W_b^T; the tensor maps are three-dimensional
  // (K, rows, batch), so a tile never reads another batch entry's rows, and D_b starts d_batch_stride elements
  // after D_{b-1} (any layout in which a row of D_b is contiguous: e.g. head-interleaved [rows, batch, N])
  int batch;
  long long d_batch_stride;
};

template <int BN, int KIND>
struct GemmCfg {
  static constexpr int kABytes = kBM * kRowBytes;
  static constexpr int kBBytes = BN * kRowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagesRaw = kSmemBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
  static constexpr int kAccStages = (KIND == kBf16) ? 2 : ((512 / BN) > 4 ? 4 : (512 / BN));
  // FP8 promotion costs one FMA per accumulator element per 128-deep K block; with 256-wide tiles two
  // epilogue warpgroups split the columns so that promotion keeps up with the tensor pipe.
  static constexpr int kEpiWG = (KIND == kFp8Block && BN == 256) ? 2 : 1;
  static constexpr int kThreads = 64 + 128 * kEpiWG;
  static constexpr int kEpiCols = BN / kEpiWG;
  static constexpr int kTmemCols = kAccStages * BN < 32 ? 32 : kAccStages * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 512 /*barriers*/;
  static constexpr int kElemsPerRow = (KIND == kBf16) ? 64 : 128;  // K elements per stage
  static constexpr int kMmaK = (KIND == kBf16) ? 16 : 32;
};

// Tile order: groups of kGroupM row-tiles sweep all column-tiles before the next group starts, so the
// CTAs running at any moment share a few A panels and W panels that stay resident in L2.
constexpr int kGroupM = 16;
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& m_blk, int& n_blk) {
  const int per_group = kGroupM * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * kGroupM;
  const int gsz = min(m_tiles - first_m, kGroupM);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

template <int BN, int KIND>
__global__ void __launch_bounds__(GemmCfg<BN, KIND>::kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const GemmParams p) {
  using Cfg = GemmCfg<BN, KIND>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::kStages;
  uint64_t* tfull_bar = bars + 2 * Cfg::kStages;
  uint64_t* tempty_bar = tfull_bar + Cfg::kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + Cfg::kAccStages);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kBM - 1) / kBM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int tiles_per_batch = m_tiles * n_tiles;
  const int num_tiles = tiles_per_batch * ((KIND == kBf16 && p.batch > 0) ? p.batch : 1);
  const int num_kb = (p.K + Cfg::kElemsPerRow - 1) / Cfg::kElemsPerRow;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < Cfg::kAccStages; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], 128 * Cfg::kEpiWG); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
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
        const int b = (KIND == kBf16) ? tile / tiles_per_batch : 0;
        tile_coords(tile - b * tiles_per_batch, m_tiles, n_tiles, m_blk, n_blk);
        const int m0 = m_blk * kBM;
        const int n0 = n_blk * BN;
        int w_row0 = n0;
        if (p.tile_expert) {
          const int e = p.tile_expert[m_blk];
          if (e < 0) continue;
          w_row0 = e * p.expert_rows + n0;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          if (KIND == kBf16 && p.batch > 0) {
            tma_load_3d(sa, &tma_a, &full_bar[stage], kb * Cfg::kElemsPerRow, m0, b);
            tma_load_3d(sb, &tma_b, &full_bar[stage], kb * Cfg::kElemsPerRow, n0, b);
          } else {
            tma_load_2d(sa, &tma_a, &full_bar[stage], kb * Cfg::kElemsPerRow, m0);
            tma_load_2d(sb, &tma_b, &full_bar[stage], kb * Cfg::kElemsPerRow, w_row0);
          }
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = (KIND == kBf16) ? make_idesc(kBM, BN, 1, 1) : make_idesc(kBM, BN, 0, 0);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (p.tile_expert) {
          int m_blk, n_blk;
          tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
          if (p.tile_expert[m_blk] < 0) continue;
        }
        if (KIND == kBf16) {
          if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (KIND == kFp8Block) {
            if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
          }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + Cfg::kABytes);
          const uint32_t d_tmem = tmem_base + acc * BN;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 32 bytes of K per MMA for both kinds (16 bf16 or 32 fp8): +2 in 16-byte units
            const uint32_t accum = (KIND == kBf16) ? ((kb | k) != 0) : (k != 0);
            if (KIND == kBf16) mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
            else mma_f8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
          if (KIND == kFp8Block) {
            tc_commit(&tfull_bar[acc]);
            if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
          }
        }
        if (KIND == kBf16 && ok) {
          tc_commit(&tfull_bar[acc]);
          if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;                     // TMEM lane quarter this warp may touch
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int wg = (warp - 2) >> 2;             // epilogue warpgroup -> column slice of the tile
    constexpr int EC = Cfg::kEpiCols;
    const int col_off = wg * EC;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_blk, n_blk;
      const int b = (KIND == kBf16) ? tile / tiles_per_batch : 0;
      tile_coords(tile - b * tiles_per_batch, m_tiles, n_tiles, m_blk, n_blk);
      const int m0 = m_blk * kBM;
      const int n0 = n_blk * BN + col_off;
      int expert = 0;
      if (p.tile_expert) {
        expert = p.tile_expert[m_blk];
        if (expert < 0) continue;
      }
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;

      auto store_chunk = [&](int c0, const float (&v)[32]) {
        if (!row_ok) return;
        const int col0 = n0 + c0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int col = col0 + g * 8;
          if (col >= p.N) continue;   // N is a multiple of 8 (checked on the host)
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = v[g * 8 + i];
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
              *reinterpret_cast<uint4*>(p.D + static_cast<size_t>(b) * p.d_batch_stride + static_cast<size_t>(row) * p.ldd + col) = ov;
            }
          }
        }
      };

      if (KIND == kBf16) {
        if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_base + acc * BN + c0, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          store_chunk(c0, v);
        }
        tc_fence_before();
        mbar_arrive(&tempty_bar[acc]);
        if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
      } else {
        float accv[EC];
#pragma unroll
        for (int i = 0; i < EC; ++i) accv[i] = 0.f;
        const int nkb_scale = (p.K + 127) / 128;
        const float* ws = p.w_scale + (static_cast<size_t>(expert) * p.scale_rows_per_expert + n0 / 128) * nkb_scale;
        for (int kb = 0; kb < num_kb; ++kb) {
          const float s = (row_ok ? p.a_scale[static_cast<size_t>(kb) * p.a_scale_ld + row] : 0.f) * ws[kb];
          if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < EC; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_base + lane_base + acc * BN + col_off + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) accv[c0 + i] = fmaf(s, __uint_as_float(r[i]), accv[c0 + i]);
          }
          tc_fence_before();
          mbar_arrive(&tempty_bar[acc]);
          if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
        }
        if (ok) {
#pragma unroll
          for (int c0 = 0; c0 < EC; c0 += 32) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = accv[c0 + i];
            store_chunk(c0, v);
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up: report, give copies/MMAs in flight a bounded time to land, then free TMEM.
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 1);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// Row-major [rows, cols] operand with `ld` elements between rows; box = 128 bytes x box_rows.
static int make_operand_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int elem_bytes,
                            int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kRowBytes / elem_bytes), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

static int g_num_sms = 0;
static int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN, int KIND>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int max_ctas,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<BN, KIND>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return -3;
    attr_set = true;
  }
  const int tiles = ((p.M + kBM - 1) / kBM) * ((p.N + BN - 1) / BN) * (p.batch > 0 ? p.batch : 1);
  int grid = tiles < num_sms() ? tiles : num_sms();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  gemm_tcgen05_kernel<BN, KIND><<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

static int pick_bn(int M, int N, int kind, int bn_hint) {
  if (bn_hint == 32 || bn_hint == 64 || bn_hint == 128 || bn_hint == 256) return bn_hint;
  const int sms = num_sms();
  const int m_tiles = (M + kBM - 1) / kBM;
  const int cands_bf16[4] = {256, 128, 64, 32};
  const int* c = cands_bf16;
  const int nc = 4;
  (void)kind;
  for (int i = 0; i < nc; ++i) {
    const int tiles = m_tiles * ((N + c[i] - 1) / c[i]);
    if (tiles >= sms) return c[i];   // at least one full wave with the widest tile that allows it
  }
  return c[nc - 1];
}

}  // namespace ksana

using namespace ksana;

// D = A[M,K](bf16, row stride lda) * W[N,K]^T (bf16) (+bias)(+residual); output bf16 or fp32.
// Returns 0 on launch success, negative on argument / setup errors.
static int gemm_bf16_impl(const void* A, int lda, const void* W, int ldw, void* D, void* out_f32, int ldd,
                          const void* bias, const void* residual, int ldr, int M, int N, int K, int bn_hint,
                          int max_ctas, int* err_flag, cudaStream_t stream, const unsigned long long* push_ptrs,
                          int push_n, int push_rows) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (K % 8) || (lda % 8) || (ldw % 8) || (ldd % 8) || (residual && (ldr % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -11;
  const int bn = pick_bn(M, N, kBf16, bn_hint);
  CUtensorMap ma, mb;
  if (make_operand_map(&ma, A, M, K, lda, 2, kBM)) return -12;
  if (make_operand_map(&mb, W, N, K, ldw, 2, bn)) return -13;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.out_f32 = static_cast<float*>(out_f32); p.ldd = ldd;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.err = err_flag;
  for (int i = 0; i < push_n && i < 8; ++i) p.push[i] = reinterpret_cast<__nv_bfloat16*>(push_ptrs[i]);
  p.push_n = push_n; p.push_rows = push_rows;
  switch (bn) {
    case 256: return launch_gemm<256, kBf16>(ma, mb, p, max_ctas, stream);
    case 128: return launch_gemm<128, kBf16>(ma, mb, p, max_ctas, stream);
    case 64: return launch_gemm<64, kBf16>(ma, mb, p, max_ctas, stream);
    default: return launch_gemm<32, kBf16>(ma, mb, p, max_ctas, stream);
  }
}

extern "C" int ksana_gemm_bf16(const void* A, int lda, const void* W, int ldw, void* D, void* out_f32, int ldd,
                               const void* bias, const void* residual, int ldr, int M, int N, int K, int bn_hint,
                               int max_ctas, int* err_flag, cudaStream_t stream) {
  return gemm_bf16_impl(A, lda, W, ldw, D, out_f32, ldd, bias, residual, ldr, M, N, K, bn_hint, max_ctas, err_flag,
                        stream, nullptr, 0, 0);
}

// Batched bf16 product: D_b[M, N] = A_b[M, K] W_b[N, K]^T for b < batch. Operand b starts a_batch / w_batch elements
// after operand b - 1 and its rows are lda / ldw elements apart (so A may be a head-interleaved [M, batch, K] tensor);
// D likewise with d_batch and ldd. All strides in elements, multiples of 8; K a multiple of 8. One launch, tiles of all
// batch entries in one persistent grid.
static int make_batched_map(CUtensorMap* map, const void* base, int rows, int cols, long long ld, long long batch_stride,
                            int batch, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(batch_stride) * 2};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kRowBytes / 2), static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

extern "C" int ksana_gemm_bf16_batched(const void* A, long long lda, long long a_batch, const void* W, long long ldw,
                                       long long w_batch, void* D, long long ldd, long long d_batch, int batch, int M,
                                       int N, int K, int* err_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if ((N % 8) || (K % 8) || (lda % 8) || (ldw % 8) || (ldd % 8) || (a_batch % 8) || (w_batch % 8) || (d_batch % 8) ||
      ldd > 0x7fffffffLL) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(D)) & 15) return -11;
  const int m_tiles = (M + kBM - 1) / kBM;
  int bn = 32;
  for (int c : {256, 128, 64, 32}) {
    if (c <= N || c == 32) { bn = c; if (batch * m_tiles * ((N + c - 1) / c) >= num_sms() / 2 || c == 32) break; }
  }
  CUtensorMap ma, mb;
  if (make_batched_map(&ma, A, M, K, lda, a_batch, batch, kBM)) return -12;
  if (make_batched_map(&mb, W, N, K, ldw, w_batch, batch, bn)) return -13;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.ldd = static_cast<int>(ldd);
  p.err = err_flag;
  p.batch = batch;
  p.d_batch_stride = d_batch;
  switch (bn) {
    case 256: return launch_gemm<256, kBf16>(ma, mb, p, 0, stream);
    case 128: return launch_gemm<128, kBf16>(ma, mb, p, 0, stream);
    case 64: return launch_gemm<64, kBf16>(ma, mb, p, 0, stream);
    default: return launch_gemm<32, kBf16>(ma, mb, p, 0, stream);
  }
}

// Push mode: partial rows go to the peers' receive slots (push_ptrs[r] = slot of this rank inside rank r's
// symmetric buffer; rows [r*push_rows, (r+1)*push_rows) belong to rank r). ldd is the slot's row stride.
extern "C" int ksana_gemm_bf16_push(const void* A, int lda, const void* W, int ldw, int ldd, const void* bias, int M,
                                    int N, int K, int bn_hint, const unsigned long long* push_ptrs, int push_n,
                                    int push_rows, int* err_flag, cudaStream_t stream) {
  return gemm_bf16_impl(A, lda, W, ldw, nullptr, nullptr, ldd, bias, nullptr, 0, M, N, K, bn_hint, 0, err_flag, stream,
                        push_ptrs, push_n, push_rows);
}

// Block-scaled FP8: A_q[M,K] e4m3 with a_scale[K/128][a_scale_ld] fp32, W_q[N,K] e4m3 with
// w_scale[ceil(N/128)][K/128] fp32. K must be a multiple of 128.
static int gemm_fp8_impl(const void* Aq, int lda, const float* a_scale, int a_scale_ld, const void* Wq,
                         int ldw, const float* w_scale, void* D, void* out_f32, int ldd, const void* bias,
                         const void* residual, int ldr, int M, int N, int K, int bn_hint, int max_ctas,
                         int* err_flag, cudaStream_t stream, const unsigned long long* push_ptrs, int push_n,
                         int push_rows) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (K % 128) || (lda % 16) || (ldw % 16) || (ldd % 8) || (residual && (ldr % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Wq)) & 15) return -11;
  const int bn = pick_bn(M, N, kFp8Block, bn_hint);
  CUtensorMap ma, mb;
  if (make_operand_map(&ma, Aq, M, K, lda, 1, kBM)) return -12;
  if (make_operand_map(&mb, Wq, N, K, ldw, 1, bn)) return -13;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.out_f32 = static_cast<float*>(out_f32); p.ldd = ldd;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.a_scale = a_scale; p.a_scale_ld = a_scale_ld; p.w_scale = w_scale;
  p.err = err_flag;
  for (int i = 0; i < push_n && i < 8; ++i) p.push[i] = reinterpret_cast<__nv_bfloat16*>(push_ptrs[i]);
  p.push_n = push_n; p.push_rows = push_rows;
  switch (bn) {
    case 256: return launch_gemm<256, kFp8Block>(ma, mb, p, max_ctas, stream);
    case 128: return launch_gemm<128, kFp8Block>(ma, mb, p, max_ctas, stream);
    case 64: return launch_gemm<64, kFp8Block>(ma, mb, p, max_ctas, stream);
    default: return launch_gemm<32, kFp8Block>(ma, mb, p, max_ctas, stream);
  }
}

extern "C" int ksana_gemm_fp8_block(const void* Aq, int lda, const float* a_scale, int a_scale_ld, const void* Wq,
                                    int ldw, const float* w_scale, void* D, void* out_f32, int ldd, const void* bias,
                                    const void* residual, int ldr, int M, int N, int K, int bn_hint, int max_ctas,
                                    int* err_flag, cudaStream_t stream) {
  return gemm_fp8_impl(Aq, lda, a_scale, a_scale_ld, Wq, ldw, w_scale, D, out_f32, ldd, bias, residual, ldr, M, N, K,
                       bn_hint, max_ctas, err_flag, stream, nullptr, 0, 0);
}

extern "C" int ksana_gemm_fp8_block_push(const void* Aq, int lda, const float* a_scale, int a_scale_ld, const void* Wq,
                                         int ldw, const float* w_scale, int ldd, const void* bias, int M, int N, int K,
                                         int bn_hint, const unsigned long long* push_ptrs, int push_n, int push_rows,
                                         int* err_flag, cudaStream_t stream) {
  return gemm_fp8_impl(Aq, lda, a_scale, a_scale_ld, Wq, ldw, w_scale, nullptr, nullptr, ldd, bias, nullptr, 0, M, N, K,
                       bn_hint, 0, err_flag, stream, push_ptrs, push_n, push_rows);
}

// Grouped GEMM for mixture-of-experts: rows of A are expert-major (each expert's segment padded to a
// multiple of 128 rows), tile_expert[m_tile] names the expert of every 128-row tile (-1 = unused).
// W: [E*N, K]; w_scale (fp8): [E * ceil(N/128)][K/128]. kind 0 = bf16, 1 = block-scaled fp8.
extern "C" int ksana_gemm_grouped(int kind, const void* A, int lda, const float* a_scale, int a_scale_ld, const void* W,
                                  int ldw, const float* w_scale, void* D, int ldd, int M_cap, int N, int K, int E,
                                  const int* tile_expert, int bn_hint, int* err_flag, cudaStream_t stream) {
  if (M_cap <= 0 || N <= 0 || K <= 0 || E <= 0) return 0;
  const int esz = kind == kBf16 ? 2 : 1;
  if ((N % 8) || (K % (kind == kBf16 ? 8 : 128)) || (lda % (16 / esz)) || (ldw % (16 / esz)) || (ldd % 8) || (M_cap % 128)) return -10;
  int bn = (bn_hint == 32 || bn_hint == 64 || bn_hint == 128 || bn_hint == 256) ? bn_hint : (N % 256 == 0 ? 256 : 128);
  if (kind == kFp8Block && N % 128) return -14;
  CUtensorMap ma, mb;
  if (make_operand_map(&ma, A, M_cap, K, lda, esz, kBM)) return -12;
  if (make_operand_map(&mb, W, E * N, K, ldw, esz, bn)) return -13;
  GemmParams p{};
  p.M = M_cap; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.a_scale = a_scale; p.a_scale_ld = a_scale_ld; p.w_scale = w_scale;
  p.err = err_flag;
  p.tile_expert = tile_expert; p.expert_rows = N; p.scale_rows_per_expert = (N + 127) / 128;
  if (kind == kBf16) {
    switch (bn) {
      case 256: return launch_gemm<256, kBf16>(ma, mb, p, 0, stream);
      case 128: return launch_gemm<128, kBf16>(ma, mb, p, 0, stream);
      case 64: return launch_gemm<64, kBf16>(ma, mb, p, 0, stream);
      default: return launch_gemm<32, kBf16>(ma, mb, p, 0, stream);
    }
  }
  switch (bn) {
    case 256: return launch_gemm<256, kFp8Block>(ma, mb, p, 0, stream);
    case 128: return launch_gemm<128, kFp8Block>(ma, mb, p, 0, stream);
    case 64: return launch_gemm<64, kFp8Block>(ma, mb, p, 0, stream);
    default: return launch_gemm<32, kFp8Block>(ma, mb, p, 0, stream);
  }
}
