// Mixture-of-experts routing and token movement for sm_100a. The expert GEMMs themselves run on the
// grouped mode of the tcgen05 GEMM (gemm_tcgen05.cu: one expert per 128-row tile); these kernels
// produce what that mode consumes and fold the result back:
//
//   route    : router logits -> top-k expert ids + weights (softmax or sigmoid scoring, optional
//              correction bias, group-limited selection, renormalisation, scaling)
//   align    : per-expert token counts -> 128-row-aligned segment offsets, the tile->expert table
//              and the destination row of every (token, k) pair
//   permute  : activation rows -> expert-major padded buffer (bf16 copy)
//   combine  : out[token] (+)= sum_k weight * expert_out[row(token,k)]  (top-k weighted sum)
//
// Functional counterpart of the reference's routing / permutation kernels
// (3rdparty/LLM_kernels/csrc/kernels/nvidia/mixture_of_experts/moe_kernels.cu:209-433 topkGatingSoftmax,
//  :505-558 sort + offsets, :711 expandInputRows, :779 finalizeMoeRouting), without the radix sort:
// destination rows come from per-expert atomic counters.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "guards.cuh"

namespace ksana {

typedef __nv_bfloat16 bf16;
constexpr int kMaxExperts = 512;
constexpr int kMaxTopK = 16;

// One warp per token. scoring 0 = softmax over all experts, 1 = sigmoid. `bias` (may be null) is added
// for SELECTION only (DeepSeek-V3 e_score_correction_bias). n_group/topk_group: keep only the best
// topk_group groups (group score = sum of its two largest biased scores).
__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                 int* __restrict__ topk_ids, float* __restrict__ topk_w, int T, int E, int K,
                                 int scoring, int renorm, float scale, int n_group, int topk_group) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  __shared__ float s_score[8][kMaxExperts];     // 8 warps per block
  __shared__ float s_sel[8][kMaxExperts];
  float* score = s_score[(threadIdx.x >> 5)];
  float* sel = s_sel[(threadIdx.x >> 5)];
  const float* row = logits + static_cast<size_t>(warp) * E;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, row[e]);
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = scoring == 0 ? __expf(row[e] - mx) : 1.f / (1.f + __expf(-row[e]));
    score[e] = v;
    sum += v;
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  for (int e = lane; e < E; e += 32) {
    if (scoring == 0) score[e] /= sum;
    sel[e] = score[e] + (bias ? bias[e] : 0.f);
  }
  __syncwarp();
  if (n_group > 1 && topk_group < n_group) {
    const int gs = E / n_group;
    // lane g (< n_group <= 32) scores its group
    float gscore = -INFINITY;
    if (lane < n_group) {
      float a = -INFINITY, b = -INFINITY;
      for (int i = 0; i < gs; ++i) {
        const float v = sel[lane * gs + i];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gscore = a + b;
    }
    // keep the topk_group best groups: a group survives if fewer than topk_group groups beat it
    int better = 0;
    for (int g = 0; g < n_group; ++g) {
      const float og = __shfl_sync(0xffffffffu, gscore, g);
      if (og > gscore || (og == gscore && g < lane)) ++better;
    }
    const bool keep = lane < n_group && better < topk_group;
    const unsigned mask = __ballot_sync(0xffffffffu, keep);
    for (int e = lane; e < E; e += 32)
      if (!((mask >> (e / gs)) & 1u)) sel[e] = -INFINITY;
    __syncwarp();
  }
  float wsum = 0.f;
  for (int k = 0; k < K; ++k) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = sel[e];
      if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;
    const float w = score[bi];
    if (lane == 0) {
      topk_ids[static_cast<size_t>(warp) * K + k] = bi;
      topk_w[static_cast<size_t>(warp) * K + k] = w;
      sel[bi] = -INFINITY;
    }
    wsum += w;
    __syncwarp();
  }
  if (lane == 0) {
    const float f = (renorm ? 1.f / fmaxf(wsum, 1e-20f) : 1.f) * scale;
    for (int k = 0; k < K; ++k) topk_w[static_cast<size_t>(warp) * K + k] *= f;
  }
}

// Single CTA. counts -> padded offsets (multiples of 128) -> tile_expert[] (-1 for unused tiles) and
// dst_row[T*K]. `total_rows[0]` receives the padded row count.
__global__ void moe_align_kernel(const int* __restrict__ topk_ids, int* __restrict__ dst_row,
                                 int* __restrict__ tile_expert, int* __restrict__ expert_offsets,
                                 int* __restrict__ total_rows, int TK, int E, int max_tiles, int expert_lo,
                                 int expert_hi, int* err) {
  __shared__ int cnt[kMaxExperts];
  __shared__ int off[kMaxExperts + 1];
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < TK; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e == -1) continue;      // a choice that lives on another rank (all-to-all dispatch sends restricted choices)
    if (e < 0 || e >= E) { guard_report(err, kGuardExpert, e); continue; }
    if (e >= expert_lo && e < expert_hi) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      o += ((cnt[e] + 127) / 128) * 128;
    }
    off[E] = o;
    total_rows[0] = o;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) expert_offsets[e] = off[e];
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int r = t * 128;
    int e = -1;
    if (r < off[E]) {
      // binary search: largest e with off[e] <= r
      int lo = 0, hi = E - 1;
      while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (off[mid] <= r) lo = mid; else hi = mid - 1; }
      e = lo;
      if (r >= off[e] + ((cnt[e] + 127) / 128) * 128) e = -1;
    }
    tile_expert[t] = e;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < TK; i += blockDim.x) {
    const int e = topk_ids[i];
    dst_row[i] = (e >= 0 && e < E && e >= expert_lo && e < expert_hi) ? off[e] + atomicAdd(&cnt[e], 1) : -1;
  }
}

// perm[dst_row[t*K+k]] = x[t]; rows of padding stay as they are (their outputs are never read).
__global__ void moe_permute_kernel(const bf16* __restrict__ x, const int* __restrict__ dst_row, bf16* __restrict__ perm,
                                   int K, int H, int cap, int* err) {
  const int t = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H);
  for (int k = 0; k < K; ++k) {
    const int r = dst_row[t * K + k];
    if (r < 0) continue;
    if (r >= cap) { if (threadIdx.x == 0) guard_report(err, kGuardDstRow, r); continue; }
    uint4* dst = reinterpret_cast<uint4*>(perm + static_cast<size_t>(r) * H);
    for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = src[i];
  }
}

// out[t] = (accumulate ? out[t] : 0) + sum_k w[t,k] * y[dst_row[t,k]]
__global__ void moe_combine_kernel(const bf16* __restrict__ y, const int* __restrict__ dst_row,
                                   const float* __restrict__ topk_w, bf16* __restrict__ out, int K, int H,
                                   int accumulate, int cap, int* err) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
    float acc[8];
    if (accumulate) {
      const uint4 v = reinterpret_cast<const uint4*>(out + static_cast<size_t>(t) * H)[i];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p[e]); acc[2 * e] = f.x; acc[2 * e + 1] = f.y; }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    }
    for (int k = 0; k < K; ++k) {
      const int r = dst_row[t * K + k];
      if (r < 0) continue;
      if (r >= cap) { if (i == 0) guard_report(err, kGuardDstRow, r); continue; }
      const float w = topk_w[t * K + k];
      const uint4 v = reinterpret_cast<const uint4*>(y + static_cast<size_t>(r) * H)[i];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p[e]); acc[2 * e] += w * f.x; acc[2 * e + 1] += w * f.y; }
    }
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) op[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H)[i] = o;
  }
}

}  // namespace ksana

using namespace ksana;

extern "C" int ksana_moe_route(const float* logits, const float* bias, int* topk_ids, float* topk_w, int T, int E, int K,
                               int scoring, int renorm, float scale, int n_group, int topk_group, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > kMaxExperts || K > kMaxTopK || n_group > 32 || (n_group > 1 && E % n_group)) return -10;
  moe_route_kernel<<<(T + 7) / 8, 256, 0, st>>>(logits, bias, topk_ids, topk_w, T, E, K, scoring, renorm, scale,
                                                n_group, topk_group);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_moe_align(const int* topk_ids, int* dst_row, int* tile_expert, int* expert_offsets,
                               int* total_rows, int TK, int E, int max_tiles, int expert_lo, int expert_hi, int* err,
                               cudaStream_t st) {
  if (E > kMaxExperts) return -10;
  moe_align_kernel<<<1, 1024, 0, st>>>(topk_ids, dst_row, tile_expert, expert_offsets, total_rows, TK, E, max_tiles,
                                       expert_lo, expert_hi, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_moe_permute(const void* x, const int* dst_row, void* perm, int T, int K, int H, int cap, int* err,
                                 cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  moe_permute_kernel<<<T, 256, 0, st>>>((const bf16*)x, dst_row, (bf16*)perm, K, H, cap, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_moe_combine(const void* y, const int* dst_row, const float* topk_w, void* out, int T, int K, int H,
                                 int accumulate, int cap, int* err, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  moe_combine_kernel<<<T, 256, 0, st>>>((const bf16*)y, dst_row, topk_w, (bf16*)out, K, H, accumulate, cap, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
