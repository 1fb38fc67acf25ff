// CTA-pair GEMM for prefill-sized problems: two SMs cooperate on one 256 x 256 output tile with
// tcgen05.mma.cta_group::2.
//
//   D[M,N] = A[M,K] * W[N,K]^T (+bias)(+residual), bf16 x bf16 or block-scaled FP8 (see gemm_tcgen05.cu)
//
// Why pairs: the single-CTA kernel fills 48 KB of shared memory per 128x256x(128 B of K) block; at
// ~64-78 B/clk/SM from L2 that takes longer than the FP8 MMA itself (tensor pipe 35 % busy, measured).
// In a pair each CTA stages only its own 128 rows of A and HALF of the W tile (128 of the 256 rows):
// 32 KB per block for the same 128 x 256 output per CTA. The tensor cores of both SMs read both W
// halves through the pair's shared-memory window.
//
// Protocol (cluster of 2 CTAs, rank 0 = leader):
//   * each CTA's producer thread loads its A rows and its W half with TMA (cta_group::2 form, no
//     multicast); both CTAs' loads complete on the LEADER's "full" barrier (expect-tx = bytes of both);
//   * the leader's MMA thread issues the pair MMA; a commit per CTA releases the stage ("empty") in
//     each CTA and publishes accumulator stages ("tmem full") to each CTA's epilogue warps;
//   * epilogue warps of both CTAs read their own 128 TMEM lanes; FP8: promote each 128-deep K block
//     with the fp32 scale product; they arrive on the leader's "tmem empty" barrier (remote arrive);
//   * cluster barriers bracket the kernel so that no CTA leaves while its peer may still touch its
//     shared memory or TMEM. Every wait is bounded.
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>
#include <stdio.h>

namespace ksana {

constexpr int kPairBN = 256;
constexpr int kPairRowBytes = 128;
constexpr int kPairThreads = 64 + 256;     // producer warp, MMA warp, 8 epilogue warps
constexpr int kPairStageBytes = 128 * kPairRowBytes + 128 * kPairRowBytes;   // A rows + W half
constexpr int kPairStages = 6;
constexpr int kPairAccStages = 2;
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 512;
constexpr int kPairGroupM = 8;             // 256-row tiles per raster group

struct PairParams {
  int M, N, K;
  __nv_bfloat16* D; int ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual; int ldr;
  const float* a_scale; int a_scale_ld;
  const float* w_scale;
  int* err;
  __nv_bfloat16* push[8]; int push_n; int push_rows;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of this CTA's tile; completion is signalled on the barrier at cluster address `bar_cluster_addr`
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the barrier at `bar_cluster_addr` (any CTA of the pair) once the MMAs issued so far have completed
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void mma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                         bool fp8) {
  if (fp8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}

__device__ __forceinline__ void pair_tile_coords(int tile, int m_tiles, int n_tiles, int& m_blk, int& n_blk) {
  const int per_group = kPairGroupM * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * kPairGroupM;
  const int gsz = min(m_tiles - first_m, kPairGroupM);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

template <int KIND>   // 0 bf16, 1 fp8 block-scaled
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
  uint64_t* full_bar = bars;                       // used in the leader
  uint64_t* empty_bar = bars + kPairStages;        // one per CTA
  uint64_t* tfull_bar = bars + 2 * kPairStages;    // one per CTA
  uint64_t* tempty_bar = tfull_bar + kPairAccStages;   // used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + kPairAccStages);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  constexpr int kElems = KIND == 0 ? 64 : 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int m_tiles = (p.M + 255) / 256;
  const int n_tiles = (p.N + kPairBN - 1) / kPairBN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + kElems - 1) / kElems;
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kPairStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    // accumulator-empty: one arrive per epilogue warp of either CTA
    for (int i = 0; i < kPairAccStages; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], 2 * 8); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, kPairAccStages * kPairBN); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        int m_blk, n_blk;
        pair_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
        const int m0 = m_blk * 256 + static_cast<int>(rank) * 128;
        const int n0 = n_blk * kPairBN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * kPairStageBytes;
          const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kPairStageBytes);
          tma_load_2d_pair(sa, &tma_a, full_leader, kb * kElems, m0);
          tma_load_2d_pair(sa + 128 * kPairRowBytes, &tma_b, full_leader, kb * kElems, n0);
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = KIND == 0 ? make_idesc(256, kPairBN, 1, 1) : make_idesc(256, kPairBN, 0, 0);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        if (KIND == 0) {
          if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (KIND == 1) {
            if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
          }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kPairStageBytes);
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + 128 * kPairRowBytes);
          const uint32_t d_tmem = tmem_base + acc * kPairBN;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t accum = KIND == 0 ? ((kb | k) != 0) : (k != 0);
            mma_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum, KIND == 1);
          }
          // release this stage in both CTAs
          tc_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 0));
          tc_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 1));
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
          if (KIND == 1) {
            tc_commit_pair(map_to_cta(smem_u32(&tfull_bar[acc]), 0));
            tc_commit_pair(map_to_cta(smem_u32(&tfull_bar[acc]), 1));
            if (++acc == kPairAccStages) { acc = 0; acc_phase ^= 1; }
          }
        }
        if (KIND == 0 && ok) {
          tc_commit_pair(map_to_cta(smem_u32(&tfull_bar[acc]), 0));
          tc_commit_pair(map_to_cta(smem_u32(&tfull_bar[acc]), 1));
          if (++acc == kPairAccStages) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------- epilogue (both CTAs, 8 warps)
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int wg = (warp - 2) >> 2;
    const int col_off = wg * 128;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    const int nkb_scale = (p.K + 127) / 128;
    for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
      int m_blk, n_blk;
      pair_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
      const int row = m_blk * 256 + static_cast<int>(rank) * 128 + q * 32 + lane;
      const int n0 = n_blk * kPairBN + col_off;
      const bool row_ok = row < p.M;
      float accv[128];
      if (KIND == 1) {
#pragma unroll
        for (int i = 0; i < 128; ++i) accv[i] = 0.f;
      }
      auto store_chunk = [&](int c0, const float (&v)[32]) {
        if (!row_ok) return;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int col = n0 + c0 + g * 8;
          if (col >= p.N) continue;
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
      };
      const uint32_t tempty_leader_base = map_to_cta(smem_u32(&tempty_bar[0]), 0);
      if (KIND == 0) {
        if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_base + acc * kPairBN + col_off + c0, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          store_chunk(c0, v);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) remote_arrive(tempty_leader_base + acc * 8);
        if (++acc == kPairAccStages) { acc = 0; acc_phase ^= 1; }
      } else {
        const float* ws = p.w_scale + static_cast<size_t>(min(n0 / 128, (p.N + 127) / 128 - 1)) * nkb_scale;
        for (int kb = 0; kb < num_kb; ++kb) {
          const float s = (row_ok ? p.a_scale[static_cast<size_t>(kb) * p.a_scale_ld + row] : 0.f) * ws[kb];
          if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < 128; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_base + lane_base + acc * kPairBN + col_off + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) accv[c0 + i] = fmaf(s, __uint_as_float(r[i]), accv[c0 + i]);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) remote_arrive(tempty_leader_base + acc * 8);
          if (++acc == kPairAccStages) { acc = 0; acc_phase ^= 1; }
        }
        if (ok) {
#pragma unroll
          for (int c0 = 0; c0 < 128; c0 += 32) {
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
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 5);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();          // the peer is done with this CTA's shared memory and accumulators
  if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, kPairAccStages * kPairBN); }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*PairEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PairEncodeFn pair_encode_fn() {
  static PairEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<PairEncodeFn>(ptr);
  }
  return fn;
}
static int pair_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int esz) {
  PairEncodeFn enc = pair_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * esz};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kPairRowBytes / esz), 128};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
             const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

template <int KIND>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const PairParams& p, cudaStream_t st) {
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) !=
        cudaSuccess) return -3;
    set = true;
  }
  // Pairs that can be resident at once: GPCs with an odd number of usable SMs leave some SMs without a partner,
  // and a pair that starts only after another one finished would double the kernel's time.
  static int max_pairs = 0;
  if (!max_pairs) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74);
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<KIND>, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 64;
    }
    max_pairs = n;
  }
  const int tiles = ((p.M + 255) / 256) * ((p.N + kPairBN - 1) / kPairBN);
  int pairs = max_pairs;
  if (pairs > tiles) pairs = tiles;
  gemm_pair_kernel<KIND><<<pairs * 2, kPairThreads, kPairSmemBytes, st>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace ksana

using namespace ksana;

// kind 0: bf16 operands; kind 1: e4m3 operands with a_scale [K/128][a_scale_ld], w_scale [ceil(N/128)][K/128].
// push_n > 0: reduce-scatter push mode (see gemm_tcgen05.cu). N must be a multiple of 8, K of 8 (bf16) / 128 (fp8).
extern "C" int ksana_gemm_pair(int kind, const void* A, int lda, const float* a_scale, int a_scale_ld, const void* W,
                               int ldw, const float* w_scale, void* D, int ldd, const void* bias, const void* residual,
                               int ldr, int M, int N, int K, const unsigned long long* push_ptrs, int push_n,
                               int push_rows, int* err_flag, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int esz = kind == 0 ? 2 : 1;
  if ((N % 8) || (K % (kind == 0 ? 8 : 128)) || (lda % (16 / esz)) || (ldw % (16 / esz)) || (ldd % 8) ||
      (residual && (ldr % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -11;
  CUtensorMap ma, mb;
  if (pair_map(&ma, A, M, K, lda, esz)) return -12;
  if (pair_map(&mb, W, N, K, ldw, esz)) return -13;
  PairParams p{};
  p.M = M; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.ldd = ldd;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.a_scale = a_scale; p.a_scale_ld = a_scale_ld; p.w_scale = w_scale;
  p.err = err_flag;
  for (int i = 0; i < push_n && i < 8; ++i) p.push[i] = reinterpret_cast<__nv_bfloat16*>(push_ptrs[i]);
  p.push_n = push_n; p.push_rows = push_rows;
  return kind == 0 ? launch_pair<0>(ma, mb, p, st) : launch_pair<1>(ma, mb, p, st);
}
