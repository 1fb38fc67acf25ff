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
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdio.h>

namespace ksana {

constexpr int kSmThreads = 192;        // + one scale-packer warp (warp 6) for kind 2
constexpr int kSmSfStages = 4;        // scale-chunk buffers
constexpr int kSmSfBatch = 1;
constexpr int kSmRowBytes = 128;
constexpr int kSmSmemBudget = 200 * 1024;

struct SmallMParams {
  int M, N, K;
  __nv_bfloat16* D; float* out_f32; int ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual; int ldr;
  const float* a_scale; int a_scale_ld;   // [K/128][ld]
  const float* w_scale;                   // [ceil(N/128)][K/128]
  int seg_cap;                            // scratch slots per output tile
  float* scratch;                         // [n_tiles][seg_cap][MP][128] fp32 partial tiles
  unsigned int* counters;                 // [n_tiles], zero before the first launch
  int* err;
  // push mode: the (partial) result is stored into every rank's receive slot for this rank instead of D
  __nv_bfloat16* push[8];
  int push_n;
  // kind 3 (weight-only 4-bit): packed levels [N, K/2] (even k in the low nibble), fp16 scale and zero*scale [N, K/group]
  const uint8_t* w4; const __half* w4_scale; const __half* w4_zs; int w4_group;
};

constexpr int pow2_at_least(int x) { int p = 32; while (p < x) p *= 2; return p; }

template <int MP, int KIND>   // MP: padded token count (16..128); KIND 0 bf16, 1 fp8 fp32 scales, 2 fp8 UE8M0 scales,
                              // 3 bf16 activations x 4-bit weights expanded to bf16 tiles by eight extra warps
struct SmallMCfg {
  static constexpr int kThreads = KIND == 2 ? kSmThreads + 32 : (KIND == 3 ? kSmThreads + 256 : kSmThreads);
  static constexpr int kSfBytes = KIND == 2 ? kSmSfStages * 1024 : 0;     // per stage: weight chunk + token chunk
  static constexpr int kWBytes = 128 * kSmRowBytes;
  static constexpr int kXBytes = MP * kSmRowBytes;
  // kind 3: ring of packed 4-bit tiles, each 128 rows x 128 bytes = four K blocks (wide rows keep DRAM pages open)
  static constexpr int kPackedSlots = KIND == 3 ? 3 : 0;
  static constexpr int kPackedBytes = 128 * 128;
  static constexpr int kPackedRing = kPackedSlots * kPackedBytes;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kStagesRaw = (kSmSmemBudget - kSfBytes - kPackedRing) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
  static constexpr int kAccStages = KIND != 1 ? 2 : ((512 / MP) > 4 ? 4 : (512 / MP));
  static constexpr int kSfBase = kAccStages * MP;                         // kind 2: two sets of 8 scale columns
  static constexpr int kTmemCols = pow2_at_least(kAccStages * MP + (KIND == 2 ? 16 : 0));
  static constexpr int kSmemBytes = kStages * kStageBytes + kPackedRing + kSfBytes + 1024 + 512;
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

template <int MP, int KIND>
__global__ void __launch_bounds__(SmallMCfg<MP, KIND>::kThreads, 1)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                   const SmallMParams p) {
  using Cfg = SmallMCfg<MP, KIND>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* pk_smem = smem + Cfg::kStages * Cfg::kStageBytes;                  // kind 3: packed ring (1024-aligned)
  uint8_t* sf_smem = pk_smem + Cfg::kPackedRing;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_smem + Cfg::kSfBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::kStages;
  uint64_t* tfull_bar = bars + 2 * Cfg::kStages;
  uint64_t* tempty_bar = tfull_bar + Cfg::kAccStages;
  uint64_t* sf_full = tempty_bar + Cfg::kAccStages;
  uint64_t* sf_empty = sf_full + kSmSfStages;
  uint64_t* pk_full = sf_empty + kSmSfStages;                                 // kind 3: packed tile landed / consumed
  uint64_t* pk_empty = pk_full + Cfg::kPackedSlots;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pk_empty + Cfg::kPackedSlots);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint32_t* last_flag = tmem_slot + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tma_w);
      tma_prefetch_desc(&tma_x);
      int stage = 0; uint32_t phase = 0;
      [[maybe_unused]] int pslot = 0; [[maybe_unused]] uint32_t pphase = 0;       // kind 3: packed ring
      long long u = u_begin; Segment sg; bool ok = true;
      while (ok && next_segment(u, u_end, num_kb, sg)) {
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
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
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
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
    if (lane == 0) {
      constexpr bool kBf16 = KIND == 0 || KIND == 3;
      constexpr uint32_t idesc = kBf16 ? make_idesc(128, MP, 1, 1) : make_idesc(128, MP, 0, 0);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      long long u = u_begin; Segment sg; bool ok = true;
      int sfs = 0; uint32_t sf_phase = 0, set = 0;
      while (ok && next_segment(u, u_end, num_kb, sg)) {
        if (KIND != 1) {
          if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        if constexpr (KIND == 2) {
          // groups of up to four K blocks share one pair of scale chunks (byte j of a chunk = block kb0 + 4g + j)
          const uint32_t d_tmem = tmem_base + acc * MP;
          for (int g0 = sg.kb0; g0 < sg.kb1 && ok; g0 += 4) {
            if (!mbar_wait(&sf_full[sfs], sf_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tsfa = tmem_base + Cfg::kSfBase + set * 8;
            const uint32_t tsfb = tsfa + 4;
            const uint32_t sf_addr = smem_u32(sf_smem + sfs * 1024);
            tmem_cp_sf(tsfa, make_sf_desc(sf_addr));
            tmem_cp_sf(tsfb, make_sf_desc(sf_addr + 512));
            for (int j = 0; j < 4 && g0 + j < sg.kb1; ++j) {
              if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
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
      // One group = up to four K blocks of one segment. The scales of the next group are fetched while the
      // current one waits for its buffer, so the L2 latency of the loads stays off the packer's critical path.
      struct GroupIter { long long u; Segment sg; int g0; bool valid; };
      auto next_group = [&](GroupIter& it) {
        if (it.valid && it.g0 + 4 < it.sg.kb1) { it.g0 += 4; return true; }
        it.valid = next_segment(it.u, u_end, num_kb, it.sg);
        it.g0 = it.sg.kb0;
        return it.valid;
      };
      auto load_group = [&](const GroupIter& it, uint32_t (&w)[5]) {   // w[0]: weight chunk word, w[1..4]: token words
        const float* ws = p.w_scale + static_cast<size_t>(it.sg.tile) * num_kb;
        w[0] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) w[0] |= (it.g0 + j < it.sg.kb1 ? ue8m0_of(ws[it.g0 + j]) : 127u) << (8 * j);
#pragma unroll
        for (int r4 = 0; r4 < 4; ++r4) {
          const int tok = r4 * 32 + lane;
          uint32_t word = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t e = 127u;
            if (tok < p.M && it.g0 + j < it.sg.kb1)
              e = ue8m0_of(p.a_scale[static_cast<size_t>(it.g0 + j) * p.a_scale_ld + tok]);
            word |= e << (8 * j);
          }
          w[1 + r4] = word;
        }
      };
      // Four groups per round (half of the buffers): their loads are all in flight together, so the packer exposes
      // one L2 round trip per four groups, and the MMA issuer works through the other half meanwhile.
      int sfs = 0; uint32_t sf_phase = 0;
      GroupIter it{u_begin, Segment{0, 0, 0}, 0, false};
      bool more = true, ok = true;
      while (more && ok) {
        uint32_t w[kSmSfBatch][5];
        bool have[kSmSfBatch];
#pragma unroll
        for (int i = 0; i < kSmSfBatch; ++i) {
          have[i] = more && next_group(it);
          more = have[i];
          if (have[i]) load_group(it, w[i]);
        }
#pragma unroll
        for (int i = 0; i < kSmSfBatch; ++i) {
          if (!have[i] || !ok) continue;
          if (!mbar_wait(&sf_empty[sfs], sf_phase ^ 1, abort_flag)) { ok = false; continue; }
          uint8_t* buf = sf_smem + sfs * 1024;
          *reinterpret_cast<uint4*>(buf + lane * 16) = make_uint4(w[i][0], w[i][0], w[i][0], w[i][0]);
          *reinterpret_cast<uint4*>(buf + 512 + lane * 16) = make_uint4(w[i][1], w[i][2], w[i][3], w[i][4]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sf_full[sfs]);
          if (++sfs == kSmSfStages) { sfs = 0; sf_phase ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int nrow = q * 32 + lane;          // output feature inside the tile
    int acc = 0; uint32_t acc_phase = 0;
    const int nkb_scale = (p.K + 127) / 128;
    long long u = u_begin; Segment sg; bool ok = true;
    while (ok && next_segment(u, u_end, num_kb, sg)) {
      const int n = sg.tile * 128 + nrow;
      float accv[MP];
#pragma unroll
      for (int i = 0; i < MP; ++i) accv[i] = 0.f;
      if (KIND != 1) {
        if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
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

      auto finish = [&](const float (&v)[MP]) {
        if (n >= p.N) return;
        const float b = p.bias ? __bfloat162float(p.bias[n]) : 0.f;
        // eight tokens at a time: the residual loads of a batch are issued together before its stores (the output
        // may alias the residual, so the compiler cannot move a load above an earlier store by itself)
#pragma unroll
        for (int m0 = 0; m0 < MP; m0 += 8) {
          if (m0 >= p.M) break;
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int m = m0 + i;
            o[i] = v[m] + b;
            if (p.residual && m < p.M) o[i] += __bfloat162float(p.residual[static_cast<size_t>(m) * p.ldr + n]);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int m = m0 + i;
            if (m >= p.M) continue;
            if (p.push_n) {
              const __nv_bfloat16 ob = __float2bfloat16(o[i]);
              for (int r = 0; r < p.push_n; ++r) p.push[r][static_cast<size_t>(m) * p.ldd + n] = ob;
            } else if (p.out_f32) p.out_f32[static_cast<size_t>(m) * p.ldd + n] = o[i];
            else p.D[static_cast<size_t>(m) * p.ldd + n] = __float2bfloat16(o[i]);
          }
        }
      };

      if (sg.kb0 == 0 && sg.kb1 == num_kb) {
        finish(accv);                        // this CTA covered the whole K range of the tile
      } else {
        const long long t0 = static_cast<long long>(sg.tile) * num_kb;
        const int first = owner_of(t0, U, P), lastc = owner_of(t0 + num_kb - 1, U, P);
        const int nseg = lastc - first + 1;
        const int my = static_cast<int>(blockIdx.x) - first;
        float* tile_scratch = p.scratch + static_cast<size_t>(sg.tile) * p.seg_cap * MP * 128;
        float* mine = tile_scratch + static_cast<size_t>(my) * MP * 128;
#pragma unroll
        for (int m4 = 0; m4 < MP / 4; ++m4)       // [MP/4][128 features][4 tokens]: 16-byte stores, coalesced over lanes
          reinterpret_cast<float4*>(mine)[m4 * 128 + nrow] =
              make_float4(accv[4 * m4], accv[4 * m4 + 1], accv[4 * m4 + 2], accv[4 * m4 + 3]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          const unsigned int prev = atomicAdd(&p.counters[sg.tile], 1u);
          const bool last = prev == static_cast<unsigned int>(nseg - 1);
          if (last) p.counters[sg.tile] = 0;   // ready for the next launch
          *last_flag = last ? 1u : 0u;
          __threadfence();
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*last_flag) {
          __threadfence();
          float sum[MP];
#pragma unroll
          for (int m = 0; m < MP; ++m) sum[m] = 0.f;
          for (int sgi = 0; sgi < nseg; ++sgi) {       // fixed order: deterministic sums
            // written by other SMs: read through L2 (ld.global.cg), never through this SM's L1
            const float4* src = reinterpret_cast<const float4*>(tile_scratch + static_cast<size_t>(sgi) * MP * 128);
#pragma unroll
            for (int m4 = 0; m4 < MP / 4; ++m4) {
              const float4 v = __ldcg(src + m4 * 128 + nrow);
              sum[4 * m4] += v.x; sum[4 * m4 + 1] += v.y; sum[4 * m4 + 2] += v.z; sum[4 * m4 + 3] += v.w;
            }
          }
          finish(sum);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // last_flag is reused by the next segment
      }
    }
  }

  tc_fence_before();
  __syncthreads();
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
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(gemm_smallm_kernel<MP, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes) != cudaSuccess) return -3;
    set = true;
  }
  gemm_smallm_kernel<MP, KIND><<<ctas, Cfg::kThreads, Cfg::kSmemBytes, st>>>(mw, mx, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace ksana

using namespace ksana;

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
                       const void* w4_zs = nullptr, int w4_group = 0) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 128) return -20;
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
  long long P = ctas_hint > 0 ? ctas_hint : sms;
  if (P > sms) P = sms;
  if (P > U / 4) P = U / 4 > 0 ? U / 4 : 1;      // at least four k-blocks per CTA
  // a tile may be cut only if scratch and counters can hold the pieces
  auto seg_cap_for = [&](long long ctas) {
    const long long per = U / ctas;               // smallest piece
    return static_cast<int>((num_kb + per - 1) / per + 1);
  };
  int seg_cap = seg_cap_for(P);
  const bool can_split = scratch != nullptr && counters != nullptr && counters_len >= n_tiles;
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
  for (int i = 0; i < push_n && i < 8; ++i) p.push[i] = reinterpret_cast<__nv_bfloat16*>(push_ptrs[i]);
  p.push_n = push_n;
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

// ----------------------------------------------------------------------------------------------
// Entry point that allocates nothing (see ksana_noalloc.h). The scratch the split-K path needs is
// a device array inside this library image; host code only ever holds its device address, which
// it gets from cudaGetSymbolAddress once per device.
#include "ksana_noalloc.h"
#include <stdio.h>

static __device__ __align__(256) unsigned char g_noalloc_scratch[kKsanaNoAllocScratchBytes];
static __device__ __align__(256) unsigned int g_noalloc_counters[kKsanaNoAllocMaxTiles];

namespace {
constexpr int kMaxDevices = 64;
void* g_noalloc_scratch_addr[kMaxDevices];      // device addresses, filled on first use per device
void* g_noalloc_counter_addr[kMaxDevices];
bool g_noalloc_ready[kMaxDevices];
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
  if (!g_noalloc_ready[dev]) {
    // In host code the array names are host-side stand-ins, not device pointers: ask the runtime for the
    // device addresses, with this device current, and check that it worked.
    void* s = nullptr;
    void* c = nullptr;
    const cudaError_t e1 = cudaGetSymbolAddress(&s, g_noalloc_scratch);
    const cudaError_t e2 = cudaGetSymbolAddress(&c, g_noalloc_counters);
    if (e1 != cudaSuccess || e2 != cudaSuccess || s == nullptr || c == nullptr) {
      snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "ksana_gemm_smallm_noalloc: cudaGetSymbolAddress failed on device %d: %s",
               dev, cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
      return KSANA_NOALLOC_SETUP_FAILED;
    }
    g_noalloc_scratch_addr[dev] = s;
    g_noalloc_counter_addr[dev] = c;
    g_noalloc_ready[dev] = true;
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
  if (cudaMemsetAsync(g_noalloc_counter_addr[dev], 0, sizeof(unsigned int) * n_tiles, stream) != cudaSuccess) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "ksana_gemm_smallm_noalloc: clearing the tile counters failed");
    return KSANA_NOALLOC_SETUP_FAILED;
  }
  return smallm_impl(kind, X, ldx, a_scale, a_scale_ld, W, ldw, w_scale, D, nullptr, ldd, bias, residual, ldr, M, N, K,
                     0, g_noalloc_scratch_addr[dev], kKsanaNoAllocScratchBytes, g_noalloc_counter_addr[dev],
                     kKsanaNoAllocMaxTiles, err_flag, stream, nullptr, 0);
}
