// Skinny GEMM for decode steps (M <= 128 tokens) on tcgen05 tensor cores:
//
//   D[M,N] = X[M,K] * W[N,K]^T (+bias)(+residual)
//
// A decode GEMM is a weight stream: every byte of W is read once and the math is
// negligible, so the kernel is organised around keeping HBM busy.
//   * Operands are swapped: the 128-row MMA dimension carries weight rows (a full
//     128-byte-swizzled TMA tile of W per stage, all of it useful), the MMA N
//     dimension carries the (padded) tokens. TMEM lane = output feature, TMEM
//     column = token.
//   * K is split across CTAs so that small N still fills all SMs; partial tiles
//     go to a scratch buffer and the last CTA to arrive for an output tile sums
//     them in a fixed order (deterministic), adds bias/residual and writes bf16.
//     Counters are reset by that CTA, so the scratch needs no host-side clearing
//     between launches once it started zeroed.
//   * FP8 (e4m3 x e4m3, 1x128 activation scales, 128x128 weight scales): each
//     128-deep K block lands in a fresh TMEM accumulator and is promoted into
//     fp32 registers with its per-token scale.
//   * FP8 with power-of-two scales (kind 2): the tensor cores apply the scales themselves (block-scaled MMA,
//     scale chunks packed by one extra warp and copied into TMEM, see gemm_tcgen05_mx.cu), so a whole K
//     segment accumulates in TMEM and the epilogue runs once per segment, as for bf16.
// Same warp roles and bounded waits as gemm_tcgen05.cu. No cluster multicast.
#include "sm100_ptx.cuh"
#include "pdl.cuh"
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdio.h>
#include <atomic>
#include <mutex>
#include <type_traits>

namespace ksana {

constexpr int kSmThreads = 192;        // + one scale-packer warp (warp 6) for kind 2
constexpr int kSmSfStages = 4;        // scale-chunk buffers
constexpr int kSmRowBytes = 128;
constexpr int kSmSmemBudget = 226 * 1024;   // all shared memory of a CTA: operand ring + scale buffers + staging + barriers
constexpr int kSmXsKb = 256;          // kind 2: K blocks whose activation-scale exponents fit the shared-memory table

struct SmallMParams {
  int M, N, K;
  __nv_bfloat16* D; float* out_f32; int ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual; int ldr;
  const float* a_scale; int a_scale_ld;   // [K/128][ld]
  const float* w_scale;                   // [ceil(N/128)][K/128]
  int seg_cap;                            // scratch slots per output tile
  float* scratch;                         // [n_tiles][seg_cap][MP][128] fp32 partial tiles
  unsigned int* counters;                 // [2 * n_tiles] (pieces written, pieces reduced), zero before the first launch
  int vec_out;                            // D (and the residual) allow 16-byte row accesses
  int* err;
  // push mode: the (partial) result is stored into every rank's receive slot for this rank instead of D
  __nv_bfloat16* push[8];
  int push_n;
  // push mode, optional: once every CTA's pushes are out (system-wide), the last CTA raises this rank's "partial rows
  // delivered" flag at every peer (sig_flags[r], epoch = *sig_epoch + 1), so that the reduce kernel that follows only
  // has to wait for the peers' flags instead of exchanging them itself
  uint32_t* sig_flags[8];
  const uint32_t* sig_epoch;
  unsigned int* sig_done;
  int sig_n;
  // kind 3 (weight-only 4-bit): packed levels [N, K/2] (even k in the low nibble), fp16 scale and zero*scale [N, K/group]
  const uint8_t* w4; const __half* w4_scale; const __half* w4_zs; int w4_group;
  // optional cycle counters per CTA and role (16 words per CTA), see ksana_smallm_set_profile
  long long* prof;
};

__device__ __forceinline__ long long prof_clock() { return clock64(); }
// adds the cycles since t0 to counter k of this CTA when profiling is on
#define KSANA_PROF_ADD(k, t0) do { if (p.prof) p.prof[blockIdx.x * 16 + (k)] += prof_clock() - (t0); } while (0)

__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

constexpr int pow2_at_least(int x) { int p = 32; while (p < x) p *= 2; return p; }

template <int MP, int KIND>   // MP: padded token count (16..128); KIND 0 bf16, 1 fp8 fp32 scales, 2 fp8 UE8M0 scales,
                              // 3 bf16 activations x 4-bit weights expanded to bf16 tiles by eight extra warps
struct SmallMCfg {
  static constexpr int kThreads = KIND == 2 ? kSmThreads + 32 : (KIND == 3 ? kSmThreads + 256 : kSmThreads);
  static constexpr int kSfBytes = KIND == 2 ? kSmSfStages * 1024 : 0;     // per stage: weight chunk + token chunk
  // kind 2: exponent bytes of the activation scales of every K block ([kb][MP]), filled once per CTA so that the
  // scale packer never waits for a global load in the steady state
  static constexpr int kXsBytes = KIND == 2 ? kSmXsKb * MP : 0;
  static constexpr int kWBytes = 128 * kSmRowBytes;
  static constexpr int kXBytes = MP * kSmRowBytes;
  // kind 3: ring of packed 4-bit tiles, each 128 rows x 128 bytes = four K blocks (wide rows keep DRAM pages open)
  static constexpr int kPackedSlots = KIND == 3 ? 3 : 0;
  static constexpr int kPackedBytes = 128 * 128;
  static constexpr int kPackedRing = kPackedSlots * kPackedBytes;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  // epilogue staging tile [MP tokens][128 features] bf16: results leave (and residual rows enter) as 16-byte vectors
  static constexpr int kOutBytes = MP * 256;
  static constexpr int kStagesRaw = (kSmSmemBudget - kSfBytes - kXsBytes - kPackedRing - kOutBytes - 1536) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
  static constexpr int kAccStages = KIND != 1 ? 2 : ((512 / MP) > 4 ? 4 : (512 / MP));
  static constexpr int kSfBase = kAccStages * MP;                         // kind 2: two sets of 8 scale columns
  static constexpr int kTmemCols = pow2_at_least(kAccStages * MP + (KIND == 2 ? 16 : 0));
  static constexpr int kSmemBytes = kStages * kStageBytes + kPackedRing + kSfBytes + kXsBytes + kOutBytes + 1024 + 512;
  static constexpr int kElems = (KIND == 0 || KIND == 3) ? 64 : 128;
};

// Work decomposition ("stream-K"): the (tile, k-block) units of the whole GEMM are laid out in one
// line and cut into gridDim.x equal pieces, one per persistent CTA. A piece is a list of segments
// (tile, kb0, kb1); a tile cut across CTAs is finished by whichever CTA arrives last.
struct Segment { int tile, kb0, kb1; };

__device__ __forceinline__ long long cut(long long c, long long U, long long P) { return c * U / P; }

__device__ __forceinline__ bool next_segment(long long& u, long long end, int num_kb, Segment& s) {
  if (u >= end) return false;
  s.tile = static_cast<int>(u / num_kb);
  s.kb0 = static_cast<int>(u % num_kb);
  const long long room = end - u;
  s.kb1 = static_cast<int>(room < (num_kb - s.kb0) ? s.kb0 + room : num_kb);
  u += s.kb1 - s.kb0;
  return true;
}

// CTA that owns unit x
__device__ __forceinline__ int owner_of(long long x, long long U, long long P) {
  long long c = x * P / U;
  while (c + 1 < P && cut(c + 1, U, P) <= x) ++c;
  while (c > 0 && cut(c, U, P) > x) --c;
  return static_cast<int>(c);
}

// element i (0..7) of eight fp16 values held in a uint4, without indexing the registers dynamically
__device__ __forceinline__ float pick_half(const uint4& v, int i) {
  const uint32_t w = (i & 4) ? ((i & 2) ? v.w : v.z) : ((i & 2) ? v.y : v.x);
  return __half2float(__ushort_as_half(static_cast<unsigned short>((i & 1) ? (w >> 16) : (w & 0xffffu))));
}

// ---- epilogue output. A thread of the four epilogue warps owns one output feature (column tile * 128 + nrow) and
// holds NR consecutive token rows of it in registers (v[r] = row row0 + r); the output matrix is [token][feature].
// Staged form: the residual rows come in as 16-byte vectors, every thread adds its column in shared memory (one
// rounding of acc + bias + residual, as in the scalar form), and the rows leave as 16-byte vectors.
template <int NR>
__device__ __forceinline__ void store_rows_staged(const SmallMParams& p, uint8_t* out_stage, int tile, int nrow, int row0,
                                                  int nrows, const float (&v)[NR]) {
  const int t = static_cast<int>(threadIdx.x) - 64;
  const int n0 = tile * 128, n = n0 + nrow;
  uint4* st4 = reinterpret_cast<uint4*>(out_stage);
  __nv_bfloat16* stb = reinterpret_cast<__nv_bfloat16*>(out_stage);
  if (p.residual) {
    for (int i = t; i < nrows * 16; i += 128) {
      const int r = i >> 4, c = i & 15;
      const __nv_bfloat16* src = p.residual + static_cast<size_t>(row0 + r) * p.ldr + n0 + c * 8;
      if (n0 + c * 8 + 8 <= p.N) st4[i] = *reinterpret_cast<const uint4*>(src);
      else
        for (int e = 0; e < 8; ++e) stb[i * 8 + e] = (n0 + c * 8 + e < p.N) ? src[e] : __float2bfloat16(0.f);
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
  }
  const float b = (p.bias && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    if (r < nrows) {
      float o = v[r] + b;
      if (p.residual) o += __bfloat162float(stb[r * 128 + nrow]);
      stb[r * 128 + nrow] = __float2bfloat16(o);
    }
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (p.push_n) {
    // tensor-parallel push mode: the rows go to this rank's receive slot in every rank's memory (its own included),
    // 256 contiguous bytes per row and tile, written as 16-byte vectors by 16 neighbouring threads: posted stores
    // over NVLink that overlap with the tiles still being computed
    for (int i = t; i < nrows * 16; i += 128) {
      const int r = i >> 4, c = i & 15;
      const size_t off = static_cast<size_t>(row0 + r) * p.ldd + n0 + c * 8;
      const uint4 v = st4[i];
      if (n0 + c * 8 + 8 <= p.N) {
        for (int q = 0; q < p.push_n; ++q) *reinterpret_cast<uint4*>(p.push[q] + off) = v;
      } else {
        for (int q = 0; q < p.push_n; ++q)
          for (int e = 0; e < 8; ++e)
            if (n0 + c * 8 + e < p.N) p.push[q][off + e] = stb[i * 8 + e];
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    return;
  }
  for (int i = t; i < nrows * 16; i += 128) {
    const int r = i >> 4, c = i & 15;
    __nv_bfloat16* dst = p.D + static_cast<size_t>(row0 + r) * p.ldd + n0 + c * 8;
    if (n0 + c * 8 + 8 <= p.N) *reinterpret_cast<uint4*>(dst) = st4[i];
    else
      for (int e = 0; e < 8; ++e)
        if (n0 + c * 8 + e < p.N) dst[e] = stb[i * 8 + e];
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");      // the staging tile is reused by the next caller
}

// Scalar form (fp32 output, push mode, unaligned outputs): two-byte / four-byte accesses, eight rows at a time so
// that the residual loads of a batch are in flight together (the output may alias the residual).
template <int NR>
__device__ __forceinline__ void store_rows_scalar(const SmallMParams& p, int tile, int nrow, int row0, int nrows,
                                                  const float (&v)[NR]) {
  const int n = tile * 128 + nrow;
  if (n >= p.N) return;
  const float b = p.bias ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
  for (int r0 = 0; r0 < NR; r0 += 8) {
    if (r0 >= nrows) break;
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = r0 + i;
      o[i] = v[r < NR ? r : NR - 1] + b;
      if (p.residual && r < nrows) o[i] += __bfloat162float(p.residual[static_cast<size_t>(row0 + r) * p.ldr + n]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = r0 + i;
      if (r >= nrows) continue;
      const size_t m = static_cast<size_t>(row0 + r);
      if (p.push_n) {
        const __nv_bfloat16 ob = __float2bfloat16(o[i]);
        for (int q = 0; q < p.push_n; ++q) p.push[q][m * p.ldd + n] = ob;
      } else if (p.out_f32) p.out_f32[m * p.ldd + n] = o[i];
      else p.D[m * p.ldd + n] = __float2bfloat16(o[i]);
    }
  }
}

template <int NR>
__device__ __forceinline__ void store_rows(const SmallMParams& p, uint8_t* out_stage, int tile, int nrow, int row0,
                                           int nrows, const float (&v)[NR]) {
  if (nrows <= 0) return;
  if (p.vec_out && !p.out_f32) store_rows_staged<NR>(p, out_stage, tile, nrow, row0, nrows, v);
  else store_rows_scalar<NR>(p, tile, nrow, row0, nrows, v);
}

template <int MP, int KIND>
__global__ void __launch_bounds__(SmallMCfg<MP, KIND>::kThreads, 1)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                   const SmallMParams p) {
  using Cfg = SmallMCfg<MP, KIND>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* pk_smem = smem + Cfg::kStages * Cfg::kStageBytes;                  // kind 3: packed ring (1024-aligned)
  uint8_t* sf_smem = pk_smem + Cfg::kPackedRing;
  uint8_t* xs_tab = sf_smem + Cfg::kSfBytes;                                  // kind 2: [kb][MP] exponent bytes
  uint8_t* out_stage = xs_tab + Cfg::kXsBytes;                                // epilogue staging tile (16-byte aligned)
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + Cfg::kOutBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::kStages;
  uint64_t* tfull_bar = bars + 2 * Cfg::kStages;
  uint64_t* tempty_bar = tfull_bar + Cfg::kAccStages;
  uint64_t* sf_full = tempty_bar + Cfg::kAccStages;
  uint64_t* sf_empty = sf_full + kSmSfStages;
  uint64_t* pk_full = sf_empty + kSmSfStages;                                 // kind 3: packed tile landed / consumed
  uint64_t* pk_empty = pk_full + Cfg::kPackedSlots;
  uint64_t* xs_ready = pk_empty + Cfg::kPackedSlots;                          // kind 2: exponent table filled
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xs_ready + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint32_t* last_flag = tmem_slot + 2;

  pdl_trigger();                      // the next kernel of the stream may set itself up while this one runs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long prof_t0 = prof_clock();
  if (p.prof && threadIdx.x == 0) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));
    p.prof[blockIdx.x * 16 + 14] = static_cast<long long>(gt);
  }
  const int n_tiles = (p.N + 127) / 128;
  const int num_kb = (p.K + Cfg::kElems - 1) / Cfg::kElems;
  const long long U = static_cast<long long>(n_tiles) * num_kb, P = gridDim.x;
  const long long u_begin = cut(blockIdx.x, U, P), u_end = cut(blockIdx.x + 1, U, P);

  if (threadIdx.x == 0) {
    // kind 3: a stage is full when the activation tile has landed (TMA) and the four expansion warps have arrived
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&full_bar[i], KIND == 3 ? 9 : 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < Cfg::kPackedSlots; ++i) { mbar_init(&pk_full[i], 1); mbar_init(&pk_empty[i], 8); }
    for (int i = 0; i < Cfg::kAccStages; ++i) { mbar_init(&tfull_bar[i], 1); mbar_init(&tempty_bar[i], 128); }
    for (int i = 0; i < kSmSfStages; ++i) { mbar_init(&sf_full[i], 1); mbar_init(&sf_empty[i], 1); }
    mbar_init(xs_ready, 128);
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Barriers, TMEM and the launch itself overlapped the previous kernel's tail (programmatic dependent launch). What
  // the previous kernel produced - activations, their scales, the residual, the split-K counters - is read only
  // after pdl_wait(); every role calls it before its first such access. The weights are never written while the
  // engine runs, so the producer fills the ring with weight tiles before it waits: when the activations arrive
  // (for instance from the cross-GPU reduction that precedes this GEMM), the first MMAs find their weights loaded.

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tma_w);
      tma_prefetch_desc(&tma_x);
      int stage = 0; uint32_t phase = 0;
      [[maybe_unused]] int pslot = 0; [[maybe_unused]] uint32_t pphase = 0;       // kind 3: packed ring
      int pre = 0;                            // K blocks whose weight tile is already on its way
      if constexpr (KIND != 3) {
        long long u2 = u_begin; Segment s2;
        while (pre < Cfg::kStages && next_segment(u2, u_end, num_kb, s2)) {
          for (int kb = s2.kb0; kb < s2.kb1 && pre < Cfg::kStages; ++kb, ++pre) {
            mbar_expect_tx(&full_bar[pre], Cfg::kStageBytes);
            tma_load_2d(smem + pre * Cfg::kStageBytes, &tma_w, &full_bar[pre], kb * Cfg::kElems, s2.tile * 128);
          }
        }
      }
      pdl_wait();
      tma_prefetch_desc(&tma_x);
      int issued = 0;
      long long u = u_begin; Segment sg; bool ok = true;
      while (ok && next_segment(u, u_end, num_kb, sg)) {
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++issued) {
          if (issued < pre) {                 // first round of the ring: the weight tile was requested above
            tma_load_2d(smem + stage * Cfg::kStageBytes + Cfg::kWBytes, &tma_x, &full_bar[stage], kb * Cfg::kElems, 0);
            if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
            continue;
          }
          if constexpr (KIND == 3) {
            // every fourth K block of a segment: the packed tile of that block and the next three goes into the
            // packed ring; the expansion warps turn it into the bf16 tiles of the stages
            if (((kb - sg.kb0) & 3) == 0) {
              if (!mbar_wait(&pk_empty[pslot], pphase ^ 1, abort_flag)) { ok = false; break; }
              mbar_expect_tx(&pk_full[pslot], Cfg::kPackedBytes);
              tma_load_2d(pk_smem + pslot * Cfg::kPackedBytes, &tma_w, &pk_full[pslot], kb * 32, sg.tile * 128);
              if (++pslot == Cfg::kPackedSlots) { pslot = 0; pphase ^= 1; }
            }
          }
          { const long long pt_ = prof_clock(); if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; } KSANA_PROF_ADD(0, pt_); }
          uint8_t* sw = smem + stage * Cfg::kStageBytes;
          if constexpr (KIND == 3) {
            mbar_expect_tx(&full_bar[stage], Cfg::kXBytes);
          } else {
            mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
            tma_load_2d(sw, &tma_w, &full_bar[stage], kb * Cfg::kElems, sg.tile * 128);
          }
          tma_load_2d(sw + Cfg::kWBytes, &tma_x, &full_bar[stage], kb * Cfg::kElems, 0);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0) {
      constexpr bool kBf16 = KIND == 0 || KIND == 3;
      constexpr uint32_t idesc = kBf16 ? make_idesc(128, MP, 1, 1) : make_idesc(128, MP, 0, 0);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      long long u = u_begin; Segment sg; bool ok = true;
      int sfs = 0; uint32_t sf_phase = 0, set = 0;
      while (ok && next_segment(u, u_end, num_kb, sg)) {
        if (KIND != 1) {
          { const long long pt_ = prof_clock(); if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; } KSANA_PROF_ADD(1, pt_); }
          tc_fence_after();
        }
        if constexpr (KIND == 2) {
          // groups of up to four K blocks share one pair of scale chunks (byte j of a chunk = block kb0 + 4g + j)
          const uint32_t d_tmem = tmem_base + acc * MP;
          for (int g0 = sg.kb0; g0 < sg.kb1 && ok; g0 += 4) {
            { const long long pt_ = prof_clock(); if (!mbar_wait(&sf_full[sfs], sf_phase, abort_flag)) { ok = false; break; } KSANA_PROF_ADD(2, pt_); }
            tc_fence_after();
            const uint32_t tsfa = tmem_base + Cfg::kSfBase + set * 8;
            const uint32_t tsfb = tsfa + 4;
            const uint32_t sf_addr = smem_u32(sf_smem + sfs * 1024);
            tmem_cp_sf(tsfa, make_sf_desc(sf_addr));
            tmem_cp_sf(tsfb, make_sf_desc(sf_addr + 512));
            for (int j = 0; j < 4 && g0 + j < sg.kb1; ++j) {
              { const long long pt_ = prof_clock(); if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; } KSANA_PROF_ADD(3, pt_); }
              tc_fence_after();
              const uint32_t sw = smem_u32(smem + stage * Cfg::kStageBytes);
              const uint64_t wdesc = make_smem_desc_sw128(sw);
              const uint64_t xdesc = make_smem_desc_sw128(sw + Cfg::kWBytes);
              const uint32_t idesc = make_idesc_mx(128, MP, static_cast<uint32_t>(j));
#pragma unroll
              for (int k = 0; k < 4; ++k)
                mma_mxf8(d_tmem, wdesc + 2 * k, xdesc + 2 * k, idesc, (g0 + j != sg.kb0) || k != 0, tsfa, tsfb);
              tc_commit(&empty_bar[stage]);
              if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
            }
            tc_commit(&sf_empty[sfs]);
            if (++sfs == kSmSfStages) { sfs = 0; sf_phase ^= 1; }
            set ^= 1;
          }
          if (ok) {
            tc_commit(&tfull_bar[acc]);
            if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
          }
          continue;
        }
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (KIND == 1) {
            if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
          }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint64_t wdesc = make_smem_desc_sw128(sw);
          const uint64_t xdesc = make_smem_desc_sw128(sw + Cfg::kWBytes);
          const uint32_t d_tmem = tmem_base + acc * MP;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t accum = kBf16 ? ((kb != sg.kb0) || k != 0) : (k != 0);
            if (kBf16) mma_f16(d_tmem, wdesc + 2 * k, xdesc + 2 * k, idesc, accum);
            else mma_f8(d_tmem, wdesc + 2 * k, xdesc + 2 * k, idesc, accum);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
          if (KIND == 1) {
            tc_commit(&tfull_bar[acc]);
            if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
          }
        }
        if (kBf16 && ok) {
          tc_commit(&tfull_bar[acc]);
          if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    pdl_wait();
    if constexpr (KIND == 3) {
      // ---------------------------------------------------------- 4-bit weight expansion (kind 3), warps 6..13
      // Two threads share weight row r of the tile: per K block each reads 16 of its 32 packed bytes (32 levels) from the
      // packed ring (brought in by TMA four K blocks at a time, 128-byte swizzled), turns them into bf16
      // (level * scale - zero*scale in fp32, rounded once) and stores the 128-byte row into the stage in the
      // 128-byte-swizzled layout the MMA descriptor expects.
      const int r = ((warp - 6) & 3) * 32 + lane;           // eight warps: two per 32 rows, each half a row
      const int half = (warp - 6) >> 2;
      constexpr int kBatch = Cfg::kStages >= 8 ? 4 : 2;        // K blocks converted per round (at most half the ring)
      const int gblocks = p.w4_group / 64;                    // K blocks per group; a power of two in practice
      const int gshift = (gblocks & (gblocks - 1)) == 0 ? 31 - __clz(gblocks) : -1;
      int pslot = 0; uint32_t pphase = 0;
      const int ngroups = p.K / p.w4_group;
      const bool vec_scales = (ngroups & 7) == 0 && ((reinterpret_cast<uintptr_t>(p.w4_scale) |
                                                       reinterpret_cast<uintptr_t>(p.w4_zs)) & 15) == 0;
      int stage = 0; uint32_t phase = 0;
      long long u = u_begin; Segment sg; bool ok = true;
      while (ok && next_segment(u, u_end, num_kb, sg)) {
        const int n = min(sg.tile * 128 + r, p.N - 1);          // rows past N repeat the last row; never stored
        const __half* srow = p.w4_scale + static_cast<size_t>(n) * ngroups;
        const __half* zrow = p.w4_zs + static_cast<size_t>(n) * ngroups;
        // Scales and zero terms of eight groups at a time (one 16-byte load each), the next eight fetched when the
        // current eight are first used: a row's scales sit in a sector of their own, so a load per K block would
        // put a trip to memory on the path of every block.
        int cur_chunk = -1, cur_grp = -1;
        uint4 cs = make_uint4(0, 0, 0, 0), cz = cs, ns = cs, nz = cs;
        __nv_bfloat162 sc_hi, sc_lo, neg_zr, off;
        // Batches of kBatch K blocks: one wait per barrier, one proxy fence and one round of arrivals per batch,
        // and the conversions of the batch's blocks overlap each other's shared-memory latency.
        for (int kb = sg.kb0; kb < sg.kb1; kb += kBatch) {
          const int sub0 = (kb - sg.kb0) & 3;                                // first K block within the packed tile
          const int nb = min(kBatch, sg.kb1 - kb);
          if (sub0 == 0) if (!mbar_wait(&pk_full[pslot], pphase, abort_flag)) { ok = false; break; }
          {
            int st = stage; uint32_t ph = phase;
            for (int j = 0; j < nb; ++j) {                                    // the batch's bf16 tiles are no longer read
              if (!mbar_wait(&empty_bar[st], ph ^ 1, abort_flag)) { ok = false; break; }
              if (++st == Cfg::kStages) { st = 0; ph ^= 1; }
            }
            if (!ok) break;
          }
#pragma unroll
          for (int j = 0; j < kBatch; ++j) {
            if (j >= nb) break;
            const int grp = gshift >= 0 ? ((kb + j) >> gshift) : ((kb + j) * 64) / p.w4_group;
            if (grp != cur_grp) {
              cur_grp = grp;
              float sc, zz;
              if (vec_scales) {
                const int ch = grp >> 3;
                if (ch != cur_chunk) {
                  if (cur_chunk >= 0 && ch == cur_chunk + 1) { cs = ns; cz = nz; }
                  else { cs = __ldg(reinterpret_cast<const uint4*>(srow) + ch); cz = __ldg(reinterpret_cast<const uint4*>(zrow) + ch); }
                  cur_chunk = ch;
                  if ((ch + 1) * 8 < ngroups) {
                    ns = __ldg(reinterpret_cast<const uint4*>(srow) + ch + 1);
                    nz = __ldg(reinterpret_cast<const uint4*>(zrow) + ch + 1);
                  }
                }
                sc = pick_half(cs, grp & 7);
                zz = pick_half(cz, grp & 7);
              } else {
                sc = __half2float(srow[grp]);
                zz = __half2float(zrow[grp]);
              }
              // w = level * scale - zs in packed bf16 arithmetic (the fp32 -> bf16 pack instruction is too slow for
              // this path) without losing the fp16 scale's precision: with z0 the integer nearest zs / scale,
              // d = level - z0 is exact, the scale is split into two bf16 terms and the remainder zs - z0 * scale
              // is at most half a step, so t = d * scale_lo - remainder and w = d * scale_hi + t round only at
              // bf16's own resolution of w.
              float z0 = sc != 0.f ? rintf(zz / sc) : 0.f;
              z0 = fminf(fmaxf(z0, -64.f), 64.f);
              const __nv_bfloat16 sh = __float2bfloat16_rn(sc);
              sc_hi = __bfloat162bfloat162(sh);
              sc_lo = __float2bfloat162_rn(sc - __bfloat162float(sh));
              neg_zr = __float2bfloat162_rn(-(zz - z0 * sc));
              off = __float2bfloat162_rn(128.f + z0);                        // exact: an integer below 256
            }
            int st = stage + j;
            if (st >= Cfg::kStages) st -= Cfg::kStages;
            uint8_t* dst = smem + st * Cfg::kStageBytes + r * 128;
            const uint4 qa = *reinterpret_cast<const uint4*>(pk_smem + pslot * Cfg::kPackedBytes + r * 128 +
                                                             ((((sub0 + j) * 2 + half) ^ (r & 7)) << 4));
            const uint32_t words[4] = {qa.x, qa.y, qa.z, qa.w};
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              const int c = half * 4 + cc;
              const uint32_t w = words[cc];
              uint32_t pr[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                // 0x4300 | level is bf16(128 + level) exactly: levels q (low half) and q + 4 (high half)
                uint32_t v = ((w >> (4 * q)) & 0x000f000fu) | 0x43004300u;
                const __nv_bfloat162 d = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), off);     // exact
                __nv_bfloat162 t = __hfma2(d, sc_lo, neg_zr);
                t = __hfma2(d, sc_hi, t);
                pr[q] = *reinterpret_cast<uint32_t*>(&t);
              }
              uint4 o;                                         // back to K order: (0,1) (2,3) (4,5) (6,7)
              o.x = __byte_perm(pr[0], pr[1], 0x5410);
              o.y = __byte_perm(pr[2], pr[3], 0x5410);
              o.z = __byte_perm(pr[0], pr[1], 0x7632);
              o.w = __byte_perm(pr[2], pr[3], 0x7632);
              *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = o;
            }
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            for (int j = 0; j < nb; ++j) {
              int st = stage + j;
              if (st >= Cfg::kStages) st -= Cfg::kStages;
              mbar_arrive(&full_bar[st]);
            }
            if (sub0 + nb == 4 || kb + nb == sg.kb1) mbar_arrive(&pk_empty[pslot]);     // done with this packed tile
          }
          if (sub0 + nb == 4 || kb + nb == sg.kb1) {
            if (++pslot == Cfg::kPackedSlots) { pslot = 0; pphase ^= 1; }
          }
          stage += nb;
          if (stage >= Cfg::kStages) { stage -= Cfg::kStages; phase ^= 1; }
        }
      }
    }
    // ------------------------------------------------------------ scale packer (kind 2 only)
    if constexpr (KIND == 2) {
      // One group = up to four K blocks of one segment; the MMA issuer copies a group's two 512-byte chunks (weight
      // exponents, token exponents) into TMEM. Token exponents come from the shared-memory table the epilogue warps
      // fill once per CTA; weight exponents are fetched 32 K blocks at a time (one float per lane), so in the
      // steady state the packer waits for no global load. When K has more blocks than the table holds, the token
      // exponents are read from global memory per group instead.
      const bool tab = num_kb <= kSmXsKb;
      int sfs = 0; uint32_t sf_phase = 0;
      long long u = u_begin; Segment sg;
      bool ok = true;
      bool tab_ok = false;        // the first groups do not wait for the table: they read their scales themselves
      while (ok && next_segment(u, u_end, num_kb, sg)) {
        const float* ws = p.w_scale + static_cast<size_t>(sg.tile) * num_kb;
        uint32_t wexp = 127u;                   // exponent of block (wbase + lane)
        int wbase = -1000000;
        for (int g0 = sg.kb0; g0 < sg.kb1 && ok; g0 += 4) {
          if (tab && !tab_ok) tab_ok = mbar_test_wait(xs_ready, 0);
          if (g0 + 4 > wbase + 32) {
            wbase = g0;
            wexp = (g0 + lane < sg.kb1) ? ue8m0_of(ws[g0 + lane]) : 127u;
          }
          uint32_t w0 = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) w0 |= __shfl_sync(0xffffffffu, wexp, g0 - wbase + j) << (8 * j);
          uint32_t w[4];
#pragma unroll
          for (int r4 = 0; r4 < 4; ++r4) {
            const int tok = r4 * 32 + lane;
            uint32_t word = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t e = 127u;
              if (tok < MP && g0 + j < sg.kb1) {
                if (tab_ok) e = xs_tab[(g0 + j) * MP + tok];
                else if (tok < p.M) e = ue8m0_of(p.a_scale[static_cast<size_t>(g0 + j) * p.a_scale_ld + tok]);
              }
              word |= e << (8 * j);
            }
            w[r4] = word;
          }
          { const long long pt_ = prof_clock(); if (!mbar_wait(&sf_empty[sfs], sf_phase ^ 1, abort_flag)) { ok = false; break; } KSANA_PROF_ADD(4, pt_); }
          uint8_t* buf = sf_smem + sfs * 1024;
          *reinterpret_cast<uint4*>(buf + lane * 16) = make_uint4(w0, w0, w0, w0);
          *reinterpret_cast<uint4*>(buf + 512 + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sf_full[sfs]);
          if (++sfs == kSmSfStages) { sfs = 0; sf_phase ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    pdl_wait();
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int nrow = q * 32 + lane;          // output feature inside the tile
    int acc = 0; uint32_t acc_phase = 0;
    const int nkb_scale = (p.K + 127) / 128;
    if constexpr (KIND == 2) {
      // Exponent table for the scale packer: the K blocks this CTA's piece touches (all of them when the piece
      // spans more than one tile), tokens past M get the neutral exponent. The weight ring fills meanwhile.
      if (num_kb <= kSmXsKb) {
        int lo = 0, hi = num_kb;
        if (u_end > u_begin && u_begin / num_kb == (u_end - 1) / num_kb) {
          lo = static_cast<int>(u_begin % num_kb);
          hi = static_cast<int>((u_end - 1) % num_kb) + 1;
        }
        const int t = threadIdx.x - 64;                          // 0..127 over the four epilogue warps
        constexpr int Q = MP / 4;                                 // four tokens (one 16-byte load) per table word
        const bool vec = (reinterpret_cast<uintptr_t>(p.a_scale) & 15) == 0 && (p.a_scale_ld & 3) == 0;
        uint32_t* tab32 = reinterpret_cast<uint32_t*>(xs_tab);
#pragma unroll 4
        for (int i = lo * Q + t; i < hi * Q; i += 128) {
          const int kb = i / Q, tok = (i % Q) * 4;
          const float* src = p.a_scale + static_cast<size_t>(kb) * p.a_scale_ld + tok;
          float4 v = make_float4(1.f, 1.f, 1.f, 1.f);
          if (vec && tok + 3 < p.a_scale_ld) v = *reinterpret_cast<const float4*>(src);
          else {
            if (tok < p.M) v.x = src[0];
            if (tok + 1 < p.M) v.y = src[1];
            if (tok + 2 < p.M) v.z = src[2];
            if (tok + 3 < p.M) v.w = src[3];
          }
          const uint32_t e0 = tok < p.M ? ue8m0_of(v.x) : 127u, e1 = tok + 1 < p.M ? ue8m0_of(v.y) : 127u;
          const uint32_t e2 = tok + 2 < p.M ? ue8m0_of(v.z) : 127u, e3 = tok + 3 < p.M ? ue8m0_of(v.w) : 127u;
          tab32[i] = e0 | (e1 << 8) | (e2 << 16) | (e3 << 24);
        }
        mbar_arrive(xs_ready);
        if (threadIdx.x == 64) KSANA_PROF_ADD(6, prof_t0);
      }
    }
    long long u = u_begin; Segment sg; bool ok = true;
    int pend_tile[2], pend_nseg[2], pend_my[2], npend = 0;      // a piece starts and ends with at most one cut tile each
    while (ok && next_segment(u, u_end, num_kb, sg)) {
      const int n = sg.tile * 128 + nrow;
      float accv[MP];
#pragma unroll
      for (int i = 0; i < MP; ++i) accv[i] = 0.f;
      if (KIND != 1) {
        { const long long pt_ = prof_clock(); if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; } KSANA_PROF_ADD(5, pt_); }
        tc_fence_after();
        if constexpr (MP >= 32) {
#pragma unroll
          for (int c0 = 0; c0 < MP; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_base + lane_base + acc * MP + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) accv[c0 + i] = __uint_as_float(r[i]);
          }
        } else {
          uint32_t r[16];
          tmem_ld16(tmem_base + lane_base + acc * MP, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) accv[i] = __uint_as_float(r[i]);
        }
        tc_fence_before();
        mbar_arrive(&tempty_bar[acc]);
        if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
      } else {
        const float* ws = p.w_scale + static_cast<size_t>(sg.tile) * nkb_scale;
        // Activation scales of one k-block are MP consecutive floats: lane l keeps tokens l, l+32, ... and the
        // value for column i is broadcast with a shuffle. The next k-block's scales are fetched before waiting
        // for the current accumulator, so no load sits on the critical path.
        constexpr int NS = (MP + 31) / 32;
        float s_next[NS];
        auto fetch = [&](int kb, float (&dst)[NS]) {
          const float wsc = ws[kb];
          const float* as = p.a_scale + static_cast<size_t>(kb) * p.a_scale_ld;
#pragma unroll
          for (int j = 0; j < NS; ++j) {
            const int tok = j * 32 + lane;
            dst[j] = (tok < p.M) ? as[tok] * wsc : 0.f;
          }
        };
        fetch(sg.kb0, s_next);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          float s_cur[NS];
#pragma unroll
          for (int j = 0; j < NS; ++j) s_cur[j] = s_next[j];
          if (kb + 1 < sg.kb1) fetch(kb + 1, s_next);
          if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          if constexpr (MP >= 32) {
#pragma unroll
            for (int c0 = 0; c0 < MP; c0 += 32) {
              uint32_t r[32];
              tmem_ld32(tmem_base + lane_base + acc * MP + c0, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float sc = __shfl_sync(0xffffffffu, s_cur[c0 / 32], i);
                accv[c0 + i] = fmaf(sc, __uint_as_float(r[i]), accv[c0 + i]);
              }
            }
          } else {
            uint32_t r[16];
            tmem_ld16(tmem_base + lane_base + acc * MP, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float sc = __shfl_sync(0xffffffffu, s_cur[0], i);
              accv[i] = fmaf(sc, __uint_as_float(r[i]), accv[i]);
            }
          }
          tc_fence_before();
          mbar_arrive(&tempty_bar[acc]);
          if (++acc == Cfg::kAccStages) { acc = 0; acc_phase ^= 1; }
        }
        if (!ok) break;
      }

      if (sg.kb0 == 0 && sg.kb1 == num_kb) {
        const long long pt10 = prof_clock();
        store_rows<MP>(p, out_stage, sg.tile, nrow, 0, p.M < MP ? p.M : MP, accv);   // the whole K range of the tile
        if (threadIdx.x == 64) KSANA_PROF_ADD(10, pt10);
      } else {
        // A tile cut across CTAs: this piece goes to the scratch slot of its position; the sum is taken after the
        // last segment (below), when every CTA of the tile reduces its own share of the tokens.
        const long long t0 = static_cast<long long>(sg.tile) * num_kb;
        const int first = owner_of(t0, U, P), lastc = owner_of(t0 + num_kb - 1, U, P);
        const int my = static_cast<int>(blockIdx.x) - first;
        float* mine = p.scratch + (static_cast<size_t>(sg.tile) * p.seg_cap + my) * MP * 128;
        const long long pt7 = prof_clock();
#pragma unroll
        for (int m4 = 0; m4 < MP / 4; ++m4)       // [MP/4][128 features][4 tokens]: 16-byte stores, coalesced over lanes
          reinterpret_cast<float4*>(mine)[m4 * 128 + nrow] =
              make_float4(accv[4 * m4], accv[4 * m4 + 1], accv[4 * m4 + 2], accv[4 * m4 + 3]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) atomicAdd(&p.counters[sg.tile], 1u);
        if (npend < 2) { pend_tile[npend] = sg.tile; pend_nseg[npend] = lastc - first + 1; pend_my[npend] = my; ++npend; }
        if (threadIdx.x == 64) KSANA_PROF_ADD(7, pt7);
      }
    }

    // ---- tiles cut across CTAs: every CTA of such a tile sums a share of the tokens over all pieces (fixed order,
    // so the result does not depend on arrival order) once all pieces are written. The waits come after all of this
    // CTA's own pieces are published, so no CTA's progress depends on another CTA's wait; all CTAs of the grid are
    // resident together (one per SM), and the wait is bounded all the same.
    for (int i = 0; i < npend && ok; ++i) {
      const int tile = pend_tile[i], nseg = pend_nseg[i], my = pend_my[i];
      const long long pt9 = prof_clock();
      if (threadIdx.x == 64) {
        int it = 0;
        while (ld_acquire_gpu_u32(&p.counters[tile]) < static_cast<unsigned int>(nseg)) {
          if (++it > (1 << 22) || *abort_flag) { *abort_flag = 1; break; }
          __nanosleep(20);
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_flag) { ok = false; break; }
      constexpr int G = MP / 4;                         // token groups of four (one 16-byte word of a partial tile)
      constexpr int NG = G / 2;                         // a tile is cut at least in two: at most half the groups here
      const int g0 = my * G / nseg, g1 = (my + 1) * G / nseg;
      const int ng = g1 - g0;
      const float4* base = reinterpret_cast<const float4*>(p.scratch + static_cast<size_t>(tile) * p.seg_cap * MP * 128);
      float sum[4 * NG];
#pragma unroll
      for (int r = 0; r < 4 * NG; ++r) sum[r] = 0.f;
      // pieces in position order (the result does not depend on arrival order); the loads of up to eight pieces (few
      // groups) or two pieces (many groups) are in flight together. Written by other SMs: read through L2.
      auto add_pieces = [&](auto batch_tag) {
        constexpr int SB = decltype(batch_tag)::value;
        for (int s0 = 0; s0 < nseg; s0 += SB) {
          float4 buf[SB][NG];
#pragma unroll
          for (int q = 0; q < SB; ++q)
#pragma unroll
            for (int gi = 0; gi < NG; ++gi)
              if (s0 + q < nseg && gi < ng && (SB <= 2 || gi < 2))
                buf[q][gi] = __ldcg(base + static_cast<size_t>(s0 + q) * (MP * 32) + (g0 + gi) * 128 + nrow);
#pragma unroll
          for (int q = 0; q < SB; ++q)
#pragma unroll
            for (int gi = 0; gi < NG; ++gi)
              if (s0 + q < nseg && gi < ng && (SB <= 2 || gi < 2)) {
                sum[4 * gi] += buf[q][gi].x; sum[4 * gi + 1] += buf[q][gi].y;
                sum[4 * gi + 2] += buf[q][gi].z; sum[4 * gi + 3] += buf[q][gi].w;
              }
        }
      };
      if (ng <= 2) add_pieces(std::integral_constant<int, 8>{});
      else add_pieces(std::integral_constant<int, (NG >= 16 ? 1 : 2)>{});
      int nrows = 4 * ng;
      if (4 * g0 + nrows > p.M) nrows = p.M - 4 * g0;
      store_rows<4 * NG>(p, out_stage, tile, nrow, 4 * g0, nrows, sum);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        // the last CTA to finish reading leaves both counters of the tile at zero for the next launch
        const unsigned int prev = atomicAdd(&p.counters[n_tiles + tile], 1u);
        if (prev == static_cast<unsigned int>(nseg - 1)) { p.counters[tile] = 0; p.counters[n_tiles + tile] = 0; }
        KSANA_PROF_ADD(9, pt9);
      }
    }
    if (p.sig_n > 0) {
      // every store_rows call ended with a barrier of the four epilogue warps: all of this CTA's pushes precede it
      if (threadIdx.x == 64) {
        __threadfence_system();
        const unsigned int prev = atomicAdd(p.sig_done, 1u);
        if (prev == gridDim.x - 1) {
          *p.sig_done = 0;
          const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(p.sig_epoch) + 1;
          __threadfence_system();
          for (int r = 0; r < p.sig_n; ++r)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.sig_flags[r]), "r"(epoch) : "memory");
        }
      }
    }
  }

  if (p.prof && lane == 0 && (warp <= 2 || warp == 6)) p.prof[blockIdx.x * 16 + (warp == 6 ? 8 : 11 + warp)] += prof_clock() - prof_t0;
  tc_fence_before();
  __syncthreads();
  if (p.prof && threadIdx.x == 0) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));
    p.prof[blockIdx.x * 16 + 15] = static_cast<long long>(gt);
  }
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, 2);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, Cfg::kTmemCols); }
}

// ------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn2 encode_fn2() {
  static EncodeTiledFn2 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn2>(ptr);
  }
  return fn;
}
static int make_map2(CUtensorMap* map, const void* base, int rows, int cols, int ld, int esz, int box_rows) {
  EncodeTiledFn2 enc = encode_fn2();
  if (!enc) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * esz};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kSmRowBytes / esz), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
             const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

// 4-bit weights [rows, k / 2 bytes]: one box is 128 bytes x 128 rows (four K blocks), 128-byte swizzled
static int make_map_packed4(CUtensorMap* map, const void* base, int rows, int k) {
  EncodeTiledFn2 enc = encode_fn2();
  if (!enc) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k / 2), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(k / 2)};
  cuuint32_t box[2] = {128, 128};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

template <int MP, int KIND>
static int launch_smallm(const CUtensorMap& mw, const CUtensorMap& mx, const SmallMParams& p, int ctas,
                         cudaStream_t st) {
  using Cfg = SmallMCfg<MP, KIND>;
  // the opt-in to large dynamic shared memory is a per-device attribute of the function
  static std::atomic<bool> set[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -3;
  if (!set[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(gemm_smallm_kernel<MP, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes) != cudaSuccess) return -3;
    set[dev].store(true, std::memory_order_release);
  }
  return launch_pdl(gemm_smallm_kernel<MP, KIND>, dim3(ctas), dim3(Cfg::kThreads), Cfg::kSmemBytes, st, mw, mx, p) ==
                 cudaSuccess ? 0 : -4;
}

// How many persistent CTAs share the n_tiles x num_kb (tile, K block) units. Measured on 64-row FP8 problems (graphs
// of back-to-back launches): a launch costs about 9 us plus 0.5 us per unit of its longest CTA; when the even cut of
// the units leaves pieces that straddle tile boundaries, every CTA completes two cut tiles instead of one and the
// launch takes about 6.4 us longer; when no tile is cut at all, the partial-tile exchange disappears (about 3 us
// less). So beside the even cut over all SMs the candidates are cuts whose pieces end on tile boundaries: s equal
// pieces per tile (s divides num_kb, n_tiles * s CTAs) and j whole tiles per CTA (j divides n_tiles). Returns the CTA
// count; est_us (optional) receives the modelled time.
static long long smallm_pick_ctas(int n_tiles, int num_kb, int sms, int ctas_hint, double* est_us) {
  const long long U = static_cast<long long>(n_tiles) * num_kb;
  auto clamp_min_units = [&](long long P) {            // at least four K blocks per CTA
    if (P > sms) P = sms;
    if (P > U / 4) P = U / 4 > 0 ? U / 4 : 1;
    return P;
  };
  auto cost = [&](long long P, bool aligned, bool whole_tiles) {
    const double units = static_cast<double>((U + P - 1) / P);
    return 9.0 + 0.5 * units + (aligned ? 0.0 : 6.4) - (whole_tiles ? 3.0 : 0.0);
  };
  auto classify = [&](long long P, bool& aligned, bool& whole) {
    aligned = whole = false;
    if (U % P) return;
    const long long per = U / P;
    whole = per % num_kb == 0;
    aligned = whole || num_kb % per == 0;
  };
  if (ctas_hint > 0) {
    const long long P = clamp_min_units(ctas_hint);
    bool a, w;
    classify(P, a, w);
    if (est_us) *est_us = cost(P, a, w);
    return P;
  }
  long long best_p = clamp_min_units(sms);
  bool a, w;
  classify(best_p, a, w);
  double best = cost(best_p, a, w);
  // The tile-aligned cuts below win when launches of one GEMM are timed back to back (64 x 1280 x 8192: 13.4 against
  // 18.6 us, 64 x 8192 x 8192: 25.9 against 29.1 us), but whole decode steps did not get faster with them (one GPU,
  // 80 layers: 29.20 against 29.03 ms per step; two GPUs: 2240 against 2229 us for 8 layers), so the even cut over all
  // SMs stays the default and KSANA_SMALLM_ALIGNED_CUT=1 selects by the model.
  const char* al = std::getenv("KSANA_SMALLM_ALIGNED_CUT");
  if (!(al && al[0] == '1')) {
    if (est_us) *est_us = best;
    return best_p;
  }
  for (int sp = 1; sp <= num_kb && static_cast<long long>(n_tiles) * sp <= sms; ++sp) {
    if (num_kb % sp || (sp > 1 && num_kb / sp < 4)) continue;
    const long long P = static_cast<long long>(n_tiles) * sp;
    const double c = cost(P, true, sp == 1);
    if (c < best) { best = c; best_p = P; }
  }
  for (int j = 2; j <= 32; ++j) {
    if (n_tiles % j || n_tiles / j > sms) continue;
    const long long P = n_tiles / j;
    const double c = cost(P, true, true);
    if (c < best) { best = c; best_p = P; }
  }
  if (est_us) *est_us = best;
  return best_p;
}

static long long* g_smallm_prof = nullptr;

struct PushSignal {            // filled by ksana_gemm_smallm_push_signal for the launch it makes
  unsigned long long flags[8];
  const void* epoch;
  void* done;
  int n;
};

}  // namespace ksana

using namespace ksana;

// Profiling aid: with a device buffer of 16 x 148 64-bit words set here, every launch adds per-CTA cycle counts to it
// (waits of the producer / MMA / packer / epilogue roles, epilogue phases, role run times, start and end of the CTA
// on the global timer). nullptr switches it off (the default).
extern "C" void ksana_smallm_set_profile(void* buf) { g_smallm_prof = static_cast<long long*>(buf); }

// Scratch needed: n_tiles * seg_cap * MP * 128 * 4 bytes (seg_cap = pieces a tile can be cut into);
// counters: n_tiles words, zero before the first launch (the kernel leaves them zero).
// kind 0: X, W bf16. kind 1: e4m3 with fp32 scales. kind 2: e4m3 with power-of-two scales, applied by the tensor
// cores. ctas_hint > 0 fixes the number of persistent CTAs
// (1 = no K splitting at all when there is a single tile per CTA...). Returns 0 on success; -20 when M > 128.
static int smallm_impl(int kind, const void* X, int ldx, const float* a_scale, int a_scale_ld, const void* W,
                       int ldw, const float* w_scale, void* D, void* out_f32, int ldd, const void* bias,
                       const void* residual, int ldr, int M, int N, int K, int ctas_hint, void* scratch,
                       long long scratch_bytes, void* counters, int counters_len, int* err_flag,
                       cudaStream_t st, const unsigned long long* push_ptrs, int push_n, const void* w4_scale = nullptr,
                       const void* w4_zs = nullptr, int w4_group = 0, const PushSignal* sig = nullptr) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 128) return -20;
  if (kind < 0 || kind > 3) return -10;
  const bool w4 = kind == 3;
  const int esz = (kind == 0 || w4) ? 2 : 1;
  if (w4) {
    if ((K % 64) || w4_group < 64 || (w4_group % 64) || (K % w4_group) || (ldx % 8) || !w4_scale || !w4_zs ||
        (reinterpret_cast<uintptr_t>(W) & 15)) return -10;
  } else if ((K % (kind == 0 ? 8 : 128)) || (ldx % (16 / esz)) || (ldw % (16 / esz))) {
    return -10;
  }
  const int MP = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  const int n_tiles = (N + 127) / 128;
  const int num_kb = (K + (esz == 2 ? 64 : 128) - 1) / (esz == 2 ? 64 : 128);
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long U = static_cast<long long>(n_tiles) * num_kb;
  long long P = smallm_pick_ctas(n_tiles, num_kb, sms, ctas_hint, nullptr);
  // a tile may be cut only if scratch and counters can hold the pieces
  auto seg_cap_for = [&](long long ctas) {
    const long long per = U / ctas;               // smallest piece
    return static_cast<int>((num_kb + per - 1) / per + 1);
  };
  int seg_cap = seg_cap_for(P);
  const bool can_split = scratch != nullptr && counters != nullptr && counters_len >= 2 * n_tiles;
  while (P > 1 && (!can_split || static_cast<long long>(n_tiles) * seg_cap * MP * 128 * 4 > scratch_bytes)) {
    // fall back to whole tiles per CTA: pieces end on tile boundaries when P divides n_tiles evenly
    P = can_split ? P / 2 : 1;
    if (P < 1) P = 1;
    seg_cap = seg_cap_for(P);
    if (!can_split) break;
  }
  if (!can_split && P != 1) P = 1;
  CUtensorMap mw, mx;
  if (make_map2(&mx, X, M, K, ldx, esz, MP)) return -13;
  if (w4) {
    if (make_map_packed4(&mw, W, N, K)) return -12;
  } else if (make_map2(&mw, W, N, K, ldw, esz, 128)) return -12;
  SmallMParams p{};
  p.M = M; p.N = N; p.K = K;
  p.D = static_cast<__nv_bfloat16*>(D); p.out_f32 = static_cast<float*>(out_f32); p.ldd = ldd;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.a_scale = a_scale; p.a_scale_ld = a_scale_ld; p.w_scale = w_scale;
  p.seg_cap = seg_cap; p.scratch = static_cast<float*>(scratch); p.counters = static_cast<unsigned int*>(counters);
  p.err = err_flag;
  p.vec_out = D != nullptr && (reinterpret_cast<uintptr_t>(D) & 15) == 0 && (ldd % 8) == 0 &&
              (residual == nullptr || ((reinterpret_cast<uintptr_t>(residual) & 15) == 0 && (ldr % 8) == 0));
  if (push_n > 0) {
    p.vec_out = (ldd % 8) == 0 && residual == nullptr;
    for (int i = 0; i < push_n && i < 8; ++i) p.vec_out = p.vec_out && (push_ptrs[i] & 15) == 0;
  }
  p.prof = g_smallm_prof;
  for (int i = 0; i < push_n && i < 8; ++i) p.push[i] = reinterpret_cast<__nv_bfloat16*>(push_ptrs[i]);
  p.push_n = push_n;
  if (sig && sig->n > 0 && push_n > 0) {
    for (int i = 0; i < sig->n && i < 8; ++i) p.sig_flags[i] = reinterpret_cast<uint32_t*>(sig->flags[i]);
    p.sig_epoch = static_cast<const uint32_t*>(sig->epoch);
    p.sig_done = static_cast<unsigned int*>(sig->done);
    p.sig_n = sig->n;
  }
  if (w4) {
    p.w4 = static_cast<const uint8_t*>(W);
    p.w4_scale = static_cast<const __half*>(w4_scale);
    p.w4_zs = static_cast<const __half*>(w4_zs);
    p.w4_group = w4_group;
  }
  const int ctas = static_cast<int>(P);
#define KSANA_SM_DISPATCH(MPV)                                                                        \
  case MPV: return kind == 0 ? launch_smallm<MPV, 0>(mw, mx, p, ctas, st)                            \
                 : (kind == 1 ? launch_smallm<MPV, 1>(mw, mx, p, ctas, st)                            \
                 : (kind == 2 ? launch_smallm<MPV, 2>(mw, mx, p, ctas, st) : launch_smallm<MPV, 3>(mw, mx, p, ctas, st)));
  switch (MP) {
    KSANA_SM_DISPATCH(16)
    KSANA_SM_DISPATCH(32)
    KSANA_SM_DISPATCH(64)
    KSANA_SM_DISPATCH(128)
  }
#undef KSANA_SM_DISPATCH
  return -21;
}

// Modelled time of one launch in nanoseconds (see smallm_pick_ctas) and, through ctas_out, the CTA count it would
// use: what the dispatcher compares with the tiled kernel's model for 33..128 rows. No GPU work.
extern "C" int ksana_smallm_estimate(int kind, int M, int N, int K, int* ctas_out) {
  if (M <= 0 || N <= 0 || K <= 0 || M > 128) return -1;
  const int esz = (kind == 0 || kind == 3) ? 2 : 1;
  const int kelems = esz == 2 ? 64 : 128;
  const int n_tiles = (N + 127) / 128, num_kb = (K + kelems - 1) / kelems;
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  double us = 0.0;
  const long long P = smallm_pick_ctas(n_tiles, num_kb, sms, 0, &us);
  if (M > 64) us += 0.28 * static_cast<double>((static_cast<long long>(n_tiles) * num_kb + P - 1) / P);   // 128-row activation tiles
  if (ctas_out) *ctas_out = static_cast<int>(P);
  return static_cast<int>(us * 1000.0);
}

extern "C" int ksana_gemm_smallm(int kind, const void* X, int ldx, const float* a_scale, int a_scale_ld, const void* W,
                                 int ldw, const float* w_scale, void* D, void* out_f32, int ldd, const void* bias,
                                 const void* residual, int ldr, int M, int N, int K, int ctas_hint, void* scratch,
                                 long long scratch_bytes, void* counters, int counters_len, int* err_flag,
                                 cudaStream_t st) {
  return smallm_impl(kind, X, ldx, a_scale, a_scale_ld, W, ldw, w_scale, D, out_f32, ldd, bias, residual, ldr, M, N, K,
                     ctas_hint, scratch, scratch_bytes, counters, counters_len, err_flag, st, nullptr, 0);
}

// Weight-only 4-bit weights (kind 3): W = packed levels [N, K/2], fp16 scale and zero*scale [N, K/group], group a multiple
// of 64. bf16 activations and output; same stream-K decomposition, scratch and counters as the other kinds.
extern "C" int ksana_gemm_smallm_w4(const void* X, int ldx, const void* qw, const void* scale, const void* zs, int group,
                                    void* D, int ldd, const void* bias, const void* residual, int ldr, int M, int N, int K,
                                    void* scratch, long long scratch_bytes, void* counters, int counters_len,
                                    int* err_flag, cudaStream_t st) {
  return smallm_impl(3, X, ldx, nullptr, 0, qw, K / 2, nullptr, D, nullptr, ldd, bias, residual, ldr, M, N, K, 0, scratch,
                     scratch_bytes, counters, counters_len, err_flag, st, nullptr, 0, scale, zs, group);
}

// Push mode (tensor parallel, decode-sized batches): the partial product is stored into every rank's
// receive slot for this rank (push_ptrs[r], row stride ldd) with plain P2P stores from the epilogue.
extern "C" int ksana_gemm_smallm_push(int kind, const void* X, int ldx, const float* a_scale, int a_scale_ld,
                                      const void* W, int ldw, const float* w_scale, int ldd, const void* bias, int M,
                                      int N, int K, void* scratch, long long scratch_bytes, void* counters,
                                      int counters_len, const unsigned long long* push_ptrs, int push_n, int* err_flag,
                                      cudaStream_t st) {
  return smallm_impl(kind, X, ldx, a_scale, a_scale_ld, W, ldw, w_scale, nullptr, nullptr, ldd, bias, nullptr, 0, M, N,
                     K, 0, scratch, scratch_bytes, counters, counters_len, err_flag, st, push_ptrs, push_n);
}

// Push mode with the delivery flag raised by the GEMM itself: sig_flags[r] = address of this rank's flag word in rank
// r's flag pad, sig_epoch = the device counter of completed exchanges (the flag value is that counter + 1),
// sig_done = a zeroed device word counting finished CTAs (left at zero).
extern "C" int ksana_gemm_smallm_push_signal(int kind, const void* X, int ldx, const float* a_scale, int a_scale_ld,
                                             const void* W, int ldw, const float* w_scale, int ldd, const void* bias,
                                             int M, int N, int K, void* scratch, long long scratch_bytes, void* counters,
                                             int counters_len, const unsigned long long* push_ptrs, int push_n,
                                             const unsigned long long* sig_flags, const void* sig_epoch, void* sig_done,
                                             int* err_flag, cudaStream_t st) {
  PushSignal sig{};
  for (int i = 0; i < push_n && i < 8; ++i) sig.flags[i] = sig_flags[i];
  sig.epoch = sig_epoch; sig.done = sig_done; sig.n = push_n;
  return smallm_impl(kind, X, ldx, a_scale, a_scale_ld, W, ldw, w_scale, nullptr, nullptr, ldd, bias, nullptr, 0, M, N,
                     K, 0, scratch, scratch_bytes, counters, counters_len, err_flag, st, push_ptrs, push_n, nullptr,
                     nullptr, 0, &sig);
}

// ----------------------------------------------------------------------------------------------
// Entry point that allocates nothing (see ksana_noalloc.h). The scratch the split-K path needs is
// a device array inside this library image; host code only ever holds its device address, which
// it gets from cudaGetSymbolAddress once per device.
#include "ksana_noalloc.h"
#include <stdio.h>

static __device__ __align__(256) unsigned char g_noalloc_scratch[kKsanaNoAllocScratchBytes];
static __device__ __align__(256) unsigned int g_noalloc_counters[2 * kKsanaNoAllocMaxTiles];   // written + reduced, per tile

namespace {
constexpr int kMaxDevices = 64;
void* g_noalloc_scratch_addr[kMaxDevices];      // device addresses, filled on first use per device
void* g_noalloc_counter_addr[kMaxDevices];
cudaError_t g_noalloc_setup_err[kMaxDevices];
std::once_flag g_noalloc_once[kMaxDevices];
thread_local char g_noalloc_msg[256] = "";
}  // namespace

extern "C" const char* ksana_noalloc_last_error(void) { return g_noalloc_msg; }

extern "C" int ksana_gemm_smallm_noalloc(int kind, const void* X, int ldx, const float* a_scale, int a_scale_ld,
                                         const void* W, int ldw, const float* w_scale, void* D, int ldd,
                                         const void* bias, const void* residual, int ldr, int M, int N, int K,
                                         int* err_flag, cudaStream_t stream) {
  g_noalloc_msg[0] = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "ksana_gemm_smallm_noalloc: cannot query the current device");
    return KSANA_NOALLOC_SETUP_FAILED;
  }
  if (kind != 0 && kind != 1) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "ksana_gemm_smallm_noalloc: kind %d is not served here (0: bf16, 1: e4m3 "
             "with fp32 scales)", kind);
    return KSANA_NOALLOC_BAD_ARGUMENT;
  }
  // In host code the array names are host-side stand-ins, not device pointers: ask the runtime for the device
  // addresses, with this device current, exactly once per device (threads that arrive together wait for the one
  // that does it), and keep the outcome.
  std::call_once(g_noalloc_once[dev], [dev]() {
    void* s = nullptr;
    void* c = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&s, g_noalloc_scratch);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&c, g_noalloc_counters);
    if (e == cudaSuccess && (s == nullptr || c == nullptr)) e = cudaErrorInvalidSymbol;
    g_noalloc_scratch_addr[dev] = s;
    g_noalloc_counter_addr[dev] = c;
    g_noalloc_setup_err[dev] = e;
  });
  if (g_noalloc_setup_err[dev] != cudaSuccess) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "ksana_gemm_smallm_noalloc: cudaGetSymbolAddress failed on device %d: %s",
             dev, cudaGetErrorString(g_noalloc_setup_err[dev]));
    return KSANA_NOALLOC_SETUP_FAILED;
  }
  if (M <= 0 || N <= 0 || K <= 0) return KSANA_NOALLOC_OK;
  const int n_tiles = (N + 127) / 128;
  if (M > 128 || n_tiles > kKsanaNoAllocMaxTiles) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg),
             "ksana_gemm_smallm_noalloc: M=%d N=%d exceed the built-in limits (M <= 128, N <= %d)", M, N,
             128 * kKsanaNoAllocMaxTiles);
    return KSANA_NOALLOC_TOO_LARGE;
  }
  // The built-in scratch must hold the partial tiles of the split the kernel would choose; the shared
  // implementation shrinks the split to what fits, so only the no-split minimum can be too large.
  const int MP = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  const long long min_need = static_cast<long long>(n_tiles) * 2 * MP * 128 * 4;
  if (min_need > kKsanaNoAllocScratchBytes) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg),
             "ksana_gemm_smallm_noalloc: M=%d N=%d need %lld bytes of scratch, the built-in array has %d", M, N,
             min_need, static_cast<int>(kKsanaNoAllocScratchBytes));
    return KSANA_NOALLOC_TOO_LARGE;
  }
  // Counters must start at zero; an earlier call that gave up half-way may have left some behind.
  if (cudaMemsetAsync(g_noalloc_counter_addr[dev], 0, sizeof(unsigned int) * 2 * n_tiles, stream) != cudaSuccess) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "ksana_gemm_smallm_noalloc: clearing the tile counters failed");
    return KSANA_NOALLOC_SETUP_FAILED;
  }
  return smallm_impl(kind, X, ldx, a_scale, a_scale_ld, W, ldw, w_scale, D, nullptr, ldd, bias, residual, ldr, M, N, K,
                     0, g_noalloc_scratch_addr[dev], kKsanaNoAllocScratchBytes, g_noalloc_counter_addr[dev],
                     2 * kKsanaNoAllocMaxTiles, err_flag, stream, nullptr, 0);
}
