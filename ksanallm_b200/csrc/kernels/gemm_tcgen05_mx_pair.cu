// Hardware block-scaled FP8 GEMM on CTA pairs: tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.
//
//   D[M,N] = (A_q * a_scale)[M,K] * (W_q * w_scale)[N,K]^T (+bias)(+residual)
//
// Operands and restrictions are those of gemm_tcgen05_mx.cu (e4m3 values, power-of-two scales: one per activation
// row and 128 K-elements stored [K/128][ld], one per 128 x 128 weight block). That kernel fills 48 KB of shared
// memory per 128 x 256 x 128 block, which takes longer than the block's MMAs (tensor pipe 58 % busy, measured).
// Here two CTAs of a cluster own one 256 x 256 output tile: each stages its own 128 rows of A and HALF of the W
// tile (32 KB per block for the same 128 x 256 output per CTA) and the tensor cores of both SMs read both W halves
// through the pair's shared-memory window.
//
// Protocol (rank 0 of the pair = leader):
//   * each CTA's producer thread loads its A rows and its W half with TMA (cta_group::2 form, no multicast); both
//     CTAs' loads complete on the LEADER's "full" barrier (expect-tx = bytes of both);
//   * each CTA's scale warp packs the exponent bytes of its own 128 rows and of all 256 columns into the chunk
//     layout of gemm_tcgen05_mx.cu in its OWN shared memory and arrives on the leader's "scales full" barrier;
//     the leader's tcgen05.cp.cta_group::2 then copies each CTA's chunks into that CTA's TMEM;
//   * the leader's MMA thread issues the pair MMAs; commits release the stage and the scale buffer in both CTAs
//     and publish the accumulator to both CTAs' epilogue warps;
//   * epilogue warps of both CTAs drain their own 128 TMEM lanes into registers and arrive on the leader's
//     "accumulator empty" barrier (remote arrive), then store;
//   * cluster barriers bracket the kernel so that no CTA leaves while its peer may still touch its shared memory
//     or TMEM. Every wait is bounded.
//
// The reference has no counterpart (its FP8 GEMMs are cuBLASLt per-tensor or DeepGEMM on Hopper:
// src/ksana_llm/kernels/nvidia/kernel_wrapper.cpp:1014-1048).
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>
#include <stdio.h>

namespace ksana {

constexpr int kMpBN = 256;
constexpr int kMpRowBytes = 128;
constexpr int kMpThreads = 96 + 256;       // producer, MMA issuer, scale packer, 8 epilogue warps
constexpr int kMpABytes = 128 * kMpRowBytes;
constexpr int kMpStageBytes = 2 * kMpABytes;           // own A rows + own half of W
constexpr int kMpStages = 6;
constexpr int kMpSfStages = 4;
constexpr int kMpSfStageBytes = 3 * 512;               // A chunk + two W chunks
constexpr int kMpSfCols = 12;                          // TMEM columns of one scale set
constexpr int kMpSfBase = kMpBN;                       // first scale column (one 256-column accumulator)
constexpr int kMpTmemCols = 512;
constexpr int kMpSmemBytes = kMpStages * kMpStageBytes + kMpSfStages * kMpSfStageBytes + 1024 + 512;
constexpr int kMpGroupM = 8;               // 256-row tiles per raster group

struct MxPairParams {
  int M, N, K;
  __nv_bfloat16* D; float* out_f32; int ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual; int ldr;
  const float* a_scale; int a_scale_ld;
  const float* w_scale;
  int* err;
  __nv_bfloat16* push[8]; int push_n; int push_rows;
};

__device__ __forceinline__ uint32_t mp_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mp_map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mp_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void mp_remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of this CTA's tile; completion is signalled on the barrier at cluster address `bar_cluster_addr`
__device__ __forceinline__ void mp_tma_load_2d(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void mp_tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mp_tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void mp_tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the barrier at `bar_cluster_addr` (either CTA of the pair) once the MMAs and copies issued so far are done
__device__ __forceinline__ void mp_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// scale chunk (128 rows x 4 bytes, 512 bytes) from each CTA's own shared memory into its own TMEM columns
__device__ __forceinline__ void mp_tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void mp_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                       uint32_t tsfa, uint32_t tsfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb) : "memory");
}

__device__ __forceinline__ void mp_tile_coords(int tile, int m_tiles, int n_tiles, int& m_blk, int& n_blk) {
  const int per_group = kMpGroupM * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * kMpGroupM;
  const int gsz = min(m_tiles - first_m, kMpGroupM);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMpThreads, 1)
gemm_mxfp8_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                       const MxPairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_smem = smem + kMpStages * kMpStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_smem + kMpSfStages * kMpSfStageBytes);
  uint64_t* full_bar = bars;                         // used in the leader
  uint64_t* empty_bar = full_bar + kMpStages;        // one per CTA
  uint64_t* sf_full = empty_bar + kMpStages;         // used in the leader (both packers arrive)
  uint64_t* sf_empty = sf_full + kMpSfStages;        // one per CTA
  uint64_t* tfull_bar = sf_empty + kMpSfStages;      // one per CTA
  uint64_t* tempty_bar = tfull_bar + 1;              // used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = mp_ctarank();
  const bool leader = rank == 0;
  const int m_tiles = (p.M + 255) / 256;
  const int n_tiles = (p.N + kMpBN - 1) / kMpBN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = p.K / 128;
  const int num_groups = (num_kb + 3) / 4;
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMpStages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < kMpSfStages; ++i) { mbar_init(&sf_full[i], 2); mbar_init(&sf_empty[i], 1); }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 2 * 8);            // one arrive per epilogue warp of either CTA
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { mp_tmem_alloc(tmem_slot, kMpTmemCols); mp_tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  mp_cluster_sync();           // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        int m_blk, n_blk;
        mp_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
        const int m0 = m_blk * 256 + static_cast<int>(rank) * 128;
        const int n0 = n_blk * kMpBN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * kMpStageBytes;
          const uint32_t full_leader = mp_map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kMpStageBytes);
          mp_tma_load_2d(sa, &tma_a, full_leader, kb * 128, m0);
          mp_tma_load_2d(sa + kMpABytes, &tma_b, full_leader, kb * 128, n0);
          if (++stage == kMpStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (leader only)
    if (leader && lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int sfs = 0; uint32_t sf_phase = 0;
      uint32_t acc_phase = 0;
      uint32_t set = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait(tempty_bar, acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base;
        for (int g = 0; g < num_groups && ok; ++g) {
          if (!mbar_wait(&sf_full[sfs], sf_phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tsfa = tmem_base + kMpSfBase + set * kMpSfCols;
          const uint32_t tsfb = tsfa + 4;
          const uint32_t sf_addr = smem_u32(sf_smem + sfs * kMpSfStageBytes);
          mp_tmem_cp_sf(tsfa, make_sf_desc(sf_addr));
          mp_tmem_cp_sf(tsfb, make_sf_desc(sf_addr + 512));
          mp_tmem_cp_sf(tsfb + 4, make_sf_desc(sf_addr + 1024));
          for (int j = 0; j < 4; ++j) {
            const int kb = g * 4 + j;
            if (kb >= num_kb) break;
            if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * kMpStageBytes);
            const uint64_t adesc = make_smem_desc_sw128(sa);
            const uint64_t bdesc = make_smem_desc_sw128(sa + kMpABytes);
            const uint32_t idesc = make_idesc_mx(256, kMpBN, static_cast<uint32_t>(j));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mp_mma(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0, tsfa, tsfb);
            // release this stage in both CTAs
            mp_commit(mp_map_to_cta(smem_u32(&empty_bar[stage]), 0));
            mp_commit(mp_map_to_cta(smem_u32(&empty_bar[stage]), 1));
            if (++stage == kMpStages) { stage = 0; phase ^= 1; }
          }
          mp_commit(mp_map_to_cta(smem_u32(&sf_empty[sfs]), 0));
          mp_commit(mp_map_to_cta(smem_u32(&sf_empty[sfs]), 1));
          if (++sfs == kMpSfStages) { sfs = 0; sf_phase ^= 1; }
          set ^= 1;
        }
        if (ok) {
          mp_commit(mp_map_to_cta(smem_u32(tfull_bar), 0));
          mp_commit(mp_map_to_cta(smem_u32(tfull_bar), 1));
          acc_phase ^= 1;
        }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------- scale packer (both CTAs)
    // The scale values of the next two groups are already on their way (plain loads whose results are not
    // touched until their turn) while the warp waits for the buffer of the current group: under the load of
    // the operand stream a group's loads take longer than its four K blocks of MMAs, so fetching on demand
    // starves the MMA thread. Three register sets rotate by name, not by index, so that no load result is
    // moved (a move would wait for it).
    int sfs = 0; uint32_t sf_phase = 0;
    const int n_blocks = (p.N + 127) / 128;
    constexpr int NB = 2;
    const uint32_t sf_full_leader = mp_map_to_cta(smem_u32(&sf_full[0]), 0);
    struct Raw { float a[16]; float b[NB * 4]; };
    auto fetch = [&](int tile, int g, Raw& r) {
      int m_blk, n_blk;
      mp_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
      const int m0 = m_blk * 256 + static_cast<int>(rank) * 128;
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
      uint8_t* buf = sf_smem + sfs * kMpSfStageBytes;
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
      if (lane == 0) mp_remote_arrive(sf_full_leader + sfs * 8);
      if (++sfs == kMpSfStages) { sfs = 0; sf_phase ^= 1; }
      return true;
    };
    // (tile, group) sequence of this CTA; `ahead` runs two steps in front of `cur`
    int ct = pair_id, cg = 0, at = ct, ag = 0;
    auto advance = [&](int& t, int& g) { if (++g == num_groups) { g = 0; t += num_pairs; } };
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
    // ---------------------------------------------------------------- epilogue (both CTAs, 8 warps)
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int wg = (warp - 3) >> 2;
    constexpr int EC = kMpBN / 2;
    const int col_off = wg * EC;
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t tempty_leader = mp_map_to_cta(smem_u32(tempty_bar), 0);
    for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
      int m_blk, n_blk;
      mp_tile_coords(tile, m_tiles, n_tiles, m_blk, n_blk);
      const int row = m_blk * 256 + static_cast<int>(rank) * 128 + q * 32 + lane;
      const int n0 = n_blk * kMpBN + col_off;
      const bool row_ok = row < p.M;
      if (!mbar_wait(tfull_bar, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t r[EC];
#pragma unroll
      for (int c0 = 0; c0 < EC; c0 += 32) tmem_ld32(tmem_base + lane_base + col_off + c0, *reinterpret_cast<uint32_t(*)[32]>(&r[c0]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mp_remote_arrive(tempty_leader);      // the accumulator is in registers: the next tile may start
      acc_phase ^= 1;
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
  mp_cluster_sync();           // the peer is done with this CTA's shared memory and accumulators
  if (warp == 1) { tc_fence_after(); mp_tmem_dealloc(tmem_base, kMpTmemCols); }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*MpEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static MpEncodeFn mp_encode_fn() {
  static MpEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<MpEncodeFn>(ptr);
  }
  return fn;
}
static int mp_map(CUtensorMap* map, const void* base, int rows, int cols, int ld) {
  MpEncodeFn enc = mp_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
  cuuint32_t box[2] = {128, 128};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

// Pairs that can be resident at once: a pair that starts only after another one finished would double the kernel's
// time, so the persistent grid is exactly the number of pairs the device can hold.
static int mx_pair_resident() {
  static int max_pairs = 0;
  if (!max_pairs) {
    cudaFuncSetAttribute(gemm_mxfp8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMpSmemBytes);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74);
    cfg.blockDim = dim3(kMpThreads);
    cfg.dynamicSmemBytes = kMpSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_mxfp8_pair_kernel, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 64;
    }
    max_pairs = n;
  }
  return max_pairs;
}

static int launch_mx_pair(const CUtensorMap& ma, const CUtensorMap& mb, const MxPairParams& p, cudaStream_t st) {
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(gemm_mxfp8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMpSmemBytes) !=
        cudaSuccess) return -3;
    set = true;
  }
  const int max_pairs = mx_pair_resident();
  const int tiles = ((p.M + 255) / 256) * ((p.N + kMpBN - 1) / kMpBN);
  int pairs = max_pairs;
  if (pairs > tiles) pairs = tiles;
  gemm_mxfp8_pair_kernel<<<pairs * 2, kMpThreads, kMpSmemBytes, st>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace ksana

using namespace ksana;

// Same operands as ksana_gemm_mxfp8 (scales must be powers of two). K must be a multiple of 128, N of 8.
extern "C" int ksana_gemm_mxfp8_pair(const void* Aq, int lda, const float* a_scale, int a_scale_ld, const void* Wq, int ldw,
                                     const float* w_scale, void* D, void* out_f32, int ldd, const void* bias,
                                     const void* residual, int ldr, int M, int N, int K,
                                     const unsigned long long* push_ptrs, int push_n, int push_rows, int* err_flag,
                                     cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) || (K % 128) || (lda % 16) || (ldw % 16) || (ldd % 8) || (residual && (ldr % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Wq)) & 15) return -11;
  CUtensorMap ma, mb;
  if (mp_map(&ma, Aq, M, K, lda)) return -12;
  if (mp_map(&mb, Wq, N, K, ldw)) return -13;
  MxPairParams p{};
  p.M = M; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.out_f32 = static_cast<float*>(out_f32); p.ldd = ldd;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.a_scale = a_scale; p.a_scale_ld = a_scale_ld; p.w_scale = w_scale;
  p.err = err_flag;
  for (int i = 0; i < push_n && i < 8; ++i) p.push[i] = reinterpret_cast<__nv_bfloat16*>(push_ptrs[i]);
  p.push_n = push_n; p.push_rows = push_rows;
  return launch_mx_pair(ma, mb, p, st);
}

// number of CTA pairs of the kernel above that the current device holds at once
extern "C" int ksana_mx_pair_resident() { return mx_pair_resident(); }
