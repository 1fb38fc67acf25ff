// FP8 GEMM with the block scaling done by the tensor cores (tcgen05.mma kind::mxf8f6f4.block_scale).
//
//   D[M,N] = (A_q * a_scale)[M,K] * (W_q * w_scale)[N,K]^T (+bias)(+residual)
//
// Same operands as the promoted-FP8 kernel in gemm_tcgen05.cu - e4m3 values, one activation scale per
// (row, 128 K-elements) stored [K/128][ld], one weight scale per 128 x 128 block - with one restriction:
// every scale is a power of two (UE8M0, what this engine's quantisers produce). The tensor core then applies
// the scales itself, the whole K loop accumulates in TMEM, and the epilogue runs once per tile instead of
// once per 128-deep K block: the TMEM -> register promotion chain of the exact-fp32-scale kernel held it at
// bf16 speed.
//
// Scale factors reach the tensor core through TMEM. Per group of four K blocks the scale warp packs the
// exponent bytes into the 512-byte chunk layout the hardware expects (128 rows x 4 scales: byte offset
// (row % 32) * 16 + (row / 32) * 4 + j), tcgen05.cp broadcasts a chunk into 4 TMEM columns, and each MMA
// names its byte j through the scale-factor id fields of the instruction descriptor.
//
// CTA layout (352 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warp 2 scale packer,
// warps 3..10 epilogue (two warpgroups split the columns). BN = 256 uses one 256-column accumulator (the
// epilogue drains it into registers and hands it back before storing); BN = 128 double-buffers.
// No cluster launch, no multicast. Every wait is bounded.
//
// The reference has no counterpart of the hardware-scaled path: its FP8 GEMMs are cuBLASLt per-tensor
// (src/ksana_llm/kernels/nvidia/kernel_wrapper.cpp:1014-1048) or DeepGEMM block-wise on Hopper.
#include "sm100_ptx.cuh"
#include "pdl.cuh"
#include "push_epilogue.cuh"
#include <cuda_bf16.h>
#include <stdio.h>

namespace ksana {

constexpr int kMxBM = 128;
constexpr int kMxRowBytes = 128;
constexpr int kMxSfStages = 4;
constexpr int kMxThreads = 96 + 256;

template <int BN>
struct MxCfg {
  static constexpr int kABytes = kMxBM * kMxRowBytes;
  static constexpr int kBBytes = BN * kMxRowBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kAccStages = BN == 256 ? 1 : 2;
  static constexpr int kBChunks = BN / 128;
  static constexpr int kSfStageBytes = (1 + kBChunks) * 512;
  static constexpr int kSfCols = 4 * (1 + kBChunks);          // TMEM columns of one scale set
  static constexpr int kSfBase = kAccStages * BN;             // first scale column
  static constexpr int kTmemCols = 512;
  static constexpr int kEpiStageBytes = 8 * kPushStageBytes;   // push epilogue: one transposition buffer per epilogue warp
  static constexpr int kSmemBytes = kStages * kStageBytes + kMxSfStages * kSfStageBytes + 1024 + 512 + kEpiStageBytes;
  static constexpr int kEpiCols = BN / 2;
};

struct MxParams {
  int M, N, K;
  __nv_bfloat16* D; float* out_f32; int ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual; int ldr;
  const float* a_scale; int a_scale_ld;
  const float* w_scale;
  int* err;
  __nv_bfloat16* push[8]; int push_n; int push_rows;
};

constexpr int kMxGroupM = 16;
__device__ __forceinline__ void mx_tile_coords(int tile, int m_tiles, int n_tiles, int& m_blk, int& n_blk) {
  const int per_group = kMxGroupM * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * kMxGroupM;
  const int gsz = min(m_tiles - first_m, kMxGroupM);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

template <int BN>
__global__ void __launch_bounds__(kMxThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const MxParams p) {
  pdl_trigger();
  using Cfg = MxCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_smem = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_smem + kMxSfStages * Cfg::kSfStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* sf_full = empty_bar + Cfg::kStages;
  uint64_t* sf_empty = sf_full + kMxSfStages;
  uint64_t* tfull_bar = sf_empty + kMxSfStages;
  uint64_t* tempty_bar = tfull_bar + Cfg::kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + Cfg::kAccStages);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint8_t* epi_stage = reinterpret_cast<uint8_t*>(bars) + 512;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kMxBM - 1) / kMxBM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = p.K / 128;
  const int num_groups = (num_kb + 3) / 4;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < kMxSfStages; ++i) { mbar_init(&sf_full[i], 1); mbar_init(&sf_empty[i], 1); }
    for (int i = 0; i < Cfg::kAccStages; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], 8); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Set-up overlapped the previous kernel (programmatic dependent launch); what that kernel produced is read only
  // after pdl_wait(), which every role calls first - except that the producer requests the weight tiles (B, never
  // written while the engine runs) of its first K blocks before it waits.

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      int pre = 0;
      if (static_cast<int>(blockIdx.x) < num_tiles) {
        int m_blk, n_blk;
        mx_tile_coords(blockIdx.x, m_tiles, n_tiles, m_blk, n_blk);
        for (; pre < Cfg::kStages && pre < num_kb; ++pre) {
          mbar_expect_tx(&full_bar[pre], Cfg::kStageBytes);
          tma_load_2d(smem + pre * Cfg::kStageBytes + Cfg::kABytes, &tma_b, &full_bar[pre], pre * 128, n_blk * BN);
        }
      }
      pdl_wait();
      int issued = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        mx_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
        for (int kb = 0; kb < num_kb; ++kb, ++issued) {
          if (issued < pre) {                 // first round of the ring: the weight tile was requested above
            tma_load_2d(smem + stage * Cfg::kStageBytes, &tma_a, &full_bar[stage], kb * 128, m_blk * kMxBM);
            if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
            continue;
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_2d(sa, &tma_a, &full_bar[stage], kb * 128, m_blk * kMxBM);
          tma_load_2d(sa + Cfg::kABytes, &tma_b, &full_bar[stage], kb * 128, n_blk * BN);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    pdl_wait();
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int sfs = 0; uint32_t sf_phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      uint32_t set = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int g = 0; g < num_groups && ok; ++g) {
          if (!mbar_wait(&sf_full[sfs], sf_phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tsfa = tmem_base + Cfg::kSfBase + set * Cfg::kSfCols;
          const uint32_t tsfb = tsfa + 4;
          const uint32_t sf_addr = smem_u32(sf_smem + sfs * Cfg::kSfStageBytes);
          tmem_cp_sf(tsfa, make_sf_desc(sf_addr));
#pragma unroll
          for (int c = 0; c < Cfg::kBChunks; ++c) tmem_cp_sf(tsfb + 4 * c, make_sf_desc(sf_addr + 512 * (1 + c)));
          for (int j = 0; j < 4; ++j) {
            const int kb = g * 4 + j;
            if (kb >= num_kb) break;
            if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
            const uint64_t adesc = make_smem_desc_sw128(sa);
            const uint64_t bdesc = make_smem_desc_sw128(sa + Cfg::kABytes);
            const uint32_t idesc = make_idesc_mx(kMxBM, BN, static_cast<uint32_t>(j));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_mxf8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0, tsfa, tsfb);
            tc_commit(&empty_bar[stage]);
            if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
          }
          tc_commit(&sf_empty[sfs]);
          if (++sfs == kMxSfStages) { sfs = 0; sf_phase ^= 1; }
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
    pdl_wait();
    // ------------------------------------------------------------- scale packer
    // The scale values of the next two groups are already on their way (plain loads whose results are not
    // touched until their turn) while the warp waits for the buffer of the current group: under the load of
    // the operand stream a group's loads take longer than its four K blocks of MMAs, so fetching on demand
    // starves the MMA thread. Three register sets rotate by name, not by index, so that no load result is
    // moved (a move would wait for it).
    int sfs = 0; uint32_t sf_phase = 0;
    const int n_blocks = (p.N + 127) / 128;
    constexpr int NB = Cfg::kBChunks;
    struct Raw { float a[16]; float b[NB * 4]; };
    auto fetch = [&](int tile, int g, Raw& r) {
      int m_blk, n_blk;
      mx_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
      const int m0 = m_blk * kMxBM;
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const int row = min(m0 + r4 * 32 + lane, p.M - 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kb = min(g * 4 + j, num_kb - 1);
          r.a[r4 * 4 + j] = __ldg(p.a_scale + static_cast<size_t>(kb) * p.a_scale_ld + row);
        }
      }
#pragma unroll
      for (int c = 0; c < NB; ++c) {
        const int nb = min(n_blk * NB + c, n_blocks - 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kb = min(g * 4 + j, num_kb - 1);
          r.b[c * 4 + j] = __ldg(p.w_scale + static_cast<size_t>(nb) * num_kb + kb);
        }
      }
    };
    // rows past M, column blocks past N and K blocks past the end repeat the last valid scale: what they scale
    // is zero-filled by TMA or never stored
    auto emit = [&](const Raw& r) -> bool {
      if (!mbar_wait(&sf_empty[sfs], sf_phase ^ 1, abort_flag)) return false;
      uint8_t* buf = sf_smem + sfs * Cfg::kSfStageBytes;
      uint32_t w[4];
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) word |= ue8m0_of(r.a[r4 * 4 + j]) << (8 * j);
        w[r4] = word;
      }
      *reinterpret_cast<uint4*>(buf + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
#pragma unroll
      for (int c = 0; c < NB; ++c) {
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) word |= ue8m0_of(r.b[c * 4 + j]) << (8 * j);
        *reinterpret_cast<uint4*>(buf + 512 * (1 + c) + lane * 16) = make_uint4(word, word, word, word);
      }
      fence_async_smem();          // the tensor core reads the chunk through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&sf_full[sfs]);
      if (++sfs == kMxSfStages) { sfs = 0; sf_phase ^= 1; }
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
    pdl_wait();                       // the residual / output may still be in use by the previous kernel
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int wg = (warp - 3) >> 2;
    constexpr int EC = Cfg::kEpiCols;
    const int col_off = wg * EC;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_blk, n_blk;
      mx_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
      const int row = m_blk * kMxBM + q * 32 + lane;
      const int n0 = n_blk * BN + col_off;
      const bool row_ok = row < p.M;
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
      if (p.push_n && !p.out_f32) {
        // rows for the peers: contiguous runs of EC columns per row (see push_epilogue.cuh)
        push_rows_staged<EC>(epi_stage + (warp - 3) * kPushStageBytes, r, p.bias, lane, m_blk * kMxBM + q * 32, n0, p.M,
                             p.N, p.push, p.push_n, p.push_rows, p.ldd);
        continue;
      }
      if (!row_ok) continue;
#pragma unroll
      for (int c0 = 0; c0 < EC; c0 += 8) {
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

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 6);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, Cfg::kTmemCols); }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*MxEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static MxEncodeFn mx_encode_fn() {
  static MxEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<MxEncodeFn>(ptr);
  }
  return fn;
}
static int mx_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  MxEncodeFn enc = mx_encode_fn();
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
static int launch_mx(const CUtensorMap& ma, const CUtensorMap& mb, const MxParams& p, int max_ctas, cudaStream_t st) {
  using Cfg = MxCfg<BN>;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(gemm_mxfp8_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) !=
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
  const int tiles = ((p.M + kMxBM - 1) / kMxBM) * ((p.N + BN - 1) / BN);
  int grid = tiles < sms ? tiles : sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  launch_pdl(gemm_mxfp8_kernel<BN>, dim3(grid), dim3(kMxThreads), Cfg::kSmemBytes, st, ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace ksana

using namespace ksana;

// A_q [M,K] e4m3 (row stride lda), a_scale [K/128][a_scale_ld] fp32 powers of two; W_q [N,K] e4m3, w_scale
// [ceil(N/128)][K/128] fp32 powers of two. Output bf16 (D) or fp32 (out_f32). bn_hint: 128, 256 or 0 (automatic).
// push_n > 0: rows go to the peers' receive slots (see gemm_tcgen05.cu). K must be a multiple of 128, N of 8.
extern "C" int ksana_gemm_mxfp8(const void* Aq, int lda, const float* a_scale, int a_scale_ld, const void* Wq, int ldw,
                                const float* w_scale, void* D, void* out_f32, int ldd, const void* bias,
                                const void* residual, int ldr, int M, int N, int K, int bn_hint, int max_ctas,
                                const unsigned long long* push_ptrs, int push_n, int push_rows, int* err_flag,
                                cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (K % 128) || (lda % 16) || (ldw % 16) || (ldd % 8) || (residual && (ldr % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Wq)) & 15) return -11;
  int bn = bn_hint;
  if (bn != 128 && bn != 256) {
    const int m_tiles = (M + kMxBM - 1) / kMxBM;
    bn = (m_tiles * ((N + 255) / 256) >= 148) ? 256 : 128;
  }
  CUtensorMap ma, mb;
  if (mx_map(&ma, Aq, M, K, lda, kMxBM)) return -12;
  if (mx_map(&mb, Wq, N, K, ldw, bn)) return -13;
  MxParams p{};
  p.M = M; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.out_f32 = static_cast<float*>(out_f32); p.ldd = ldd;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.a_scale = a_scale; p.a_scale_ld = a_scale_ld; p.w_scale = w_scale;
  p.err = err_flag;
  for (int i = 0; i < push_n && i < 8; ++i) p.push[i] = reinterpret_cast<__nv_bfloat16*>(push_ptrs[i]);
  p.push_n = push_n; p.push_rows = push_rows;
  return bn == 256 ? launch_mx<256>(ma, mb, p, max_ctas, st) : launch_mx<128>(ma, mb, p, max_ctas, st);
}
