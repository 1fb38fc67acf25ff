// Memory-bound fused ops for sm_100a. Each kernel moves 16-byte vectors, touches
// every activation byte once, and can emit the next GEMM's FP8 operand
// (e4m3 values + one fp32 scale per 128 consecutive elements) directly, so that
// no stand-alone quantisation pass reads the activation again.
//
// Covers the reference kernels
//   layernorm  : 3rdparty/LLM_kernels/csrc/kernels/nvidia/layernorm/layernorm.cu:378-587
//   add        : .../add/add.cu:55-90
//   activation : .../activation/activation.cu:205-232,497-507
//   embedding  : .../embedding/embedding.cu:20-75
//   assemble   : .../assemble_last_token/assemble_last_token.cu:14-42
//   rotary     : .../rotary_embedding/rotary_embedding.cu:70-197
//   cache copy : .../paged_attention/cache_copy.cu:21-254
//   fp8 quant  : 3rdparty/LLM_kernels/csrc/utils/nvidia/cuda_fp8_utils.cu:27-140
#include "guards.cuh"
#include "pdl.cuh"
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <stdint.h>
#include "fp8_scale.cuh"

namespace ksana {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
// 8 floats -> 8 e4m3 bytes (two 32-bit words)
__device__ __forceinline__ uint2 pack8_e4m3(const float (&f)[8], float inv_scale) {
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
        make_float2(f[4 * h] * inv_scale, f[4 * h + 1] * inv_scale), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
        make_float2(f[4 * h + 2] * inv_scale, f[4 * h + 3] * inv_scale), __NV_SATFINITE, __NV_E4M3);
    w[h] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
  }
  return make_uint2(w[0], w[1]);
}
// amax over the 16 lanes that share one 128-element group (8 elements per lane)
__device__ __forceinline__ float group16_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ----------------------------------------------------------------------------
// (residual +=) x ; y = norm(residual or x) * w (+ beta) ; optional fp8 copy of y.
// mode 0 = RMSNorm, 1 = LayerNorm. One CTA per row; up to kMaxVec vectors per thread.
constexpr int kMaxVec = 4;

template <int MODE>
__global__ void norm_kernel(const bf16* __restrict__ x, bf16* __restrict__ residual, const bf16* __restrict__ w,
                            const bf16* __restrict__ beta, bf16* __restrict__ y, uint8_t* __restrict__ yq,
                            float* __restrict__ yscale, int scale_ld, int H, float eps) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nvec = H >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + static_cast<size_t>(row) * H) : nullptr;
  float v[kMaxVec][8];
  float s = 0.f, s2 = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < nvec) {
      unpack8(xr[i], v[j]);
      if (rr) {
        float r[8];
        unpack8(rr[i], r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] += r[e];
        const uint4 packed = pack8(v[j]);
        rr[i] = packed;
        unpack8(packed, v[j]);   // normalise exactly what the residual stream now holds
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) { s += v[j][e]; s2 += v[j][e] * v[j][e]; }
    }
  }
  float mean = 0.f, rstd;
  if (MODE == 1) {
    mean = block_sum(s, red) / H;
    float var = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < nvec) {
#pragma unroll
        for (int e = 0; e < 8; ++e) { const float d = v[j][e] - mean; var += d * d; }
      }
    }
    rstd = rsqrtf(block_sum(var, red) / H + eps);
  } else {
    rstd = rsqrtf(block_sum(s2, red) / H + eps);
  }
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const uint4* br = beta ? reinterpret_cast<const uint4*>(beta) : nullptr;
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * blockDim.x;   // blockDim is a multiple of 32, so groups of 16 lanes stay aligned
    const bool on = i < nvec;
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = 0.f;
    if (on) {
      float wf[8];
      unpack8(wr[i], wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[j][e] - mean) * rstd * wf[e];
      if (br) {
        float bfv[8];
        unpack8(br[i], bfv);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += bfv[e];
      }
      // round to bf16 first so that the fp8 copy quantises the same values y holds
      const uint4 packed = pack8(o);
      if (y) reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H)[i] = packed;
      unpack8(packed, o);
    }
    if (yq) {
      float am = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) am = fmaxf(am, fabsf(o[e]));
      am = group16_max(am);
      const float scale = fp8_group_scale(am);
      if (on) {
        reinterpret_cast<uint2*>(yq + static_cast<size_t>(row) * H)[i] = pack8_e4m3(o, 1.f / scale);
        if ((i & 15) == 0) yscale[static_cast<size_t>(i >> 4) * scale_ld + row] = scale;
      }
    }
  }
}

// ----------------------------------------------------------------------------
// out[m, i] = act(gate_up[m, i]) * gate_up[m, I + i] ; optional fp8 copy. act: 0 silu 1 gelu(tanh) 2 relu
// When `gated` is 0 the input is [M, I] and out = act(in).
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float act_fn(float x, int act) {
  // silu(x) = x * sigmoid(x) = 0.5 x (1 + tanh(x / 2)): one special-function op per element instead of an
  // exponential and a division (the special-function unit, not memory, paced this kernel); the approximation's
  // error (about 2^-11) is below the bf16 rounding of the result
  if (act == 0) { const float hx = 0.5f * x; return fmaf(hx, tanh_fast(hx), hx); }
  if (act == 1) return 0.5f * x * (1.f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x)));
  return fmaxf(x, 0.f);
}

__global__ void act_mul_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, uint8_t* __restrict__ outq,
                               float* __restrict__ oscale, int scale_ld, int M, int I, int in_ld, int act, int gated) {
  pdl_trigger();
  pdl_wait();
  const int nvec = I >> 3;
  const long long total = static_cast<long long>(M) * nvec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       idx < ((total + 31) / 32) * 32; idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const bool on = idx < total;
    const int m = on ? static_cast<int>(idx / nvec) : 0;
    const int i = on ? static_cast<int>(idx % nvec) : 0;
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = 0.f;
    if (on) {
      const uint4* row = reinterpret_cast<const uint4*>(in + static_cast<size_t>(m) * in_ld);
      float g[8];
      unpack8(row[i], g);
      if (gated) {
        float u[8];
        unpack8(row[nvec + i], u);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = act_fn(g[e], act) * u[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = act_fn(g[e], act);
      }
      const uint4 packed = pack8(o);
      if (out) reinterpret_cast<uint4*>(out + static_cast<size_t>(m) * I)[i] = packed;
      unpack8(packed, o);
    }
    if (outq) {   // nvec is a multiple of 16 on this path, so 16 consecutive lanes share (m, group)
      float am = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) am = fmaxf(am, fabsf(o[e]));
      am = group16_max(am);
      const float scale = fp8_group_scale(am);
      if (on) {
        reinterpret_cast<uint2*>(outq + static_cast<size_t>(m) * I)[i] = pack8_e4m3(o, 1.f / scale);
        if ((i & 15) == 0) oscale[static_cast<size_t>(i >> 4) * scale_ld + m] = scale;
      }
    }
  }
}

// x[M,K] bf16 -> e4m3 + one scale per (row, 128 columns); scales stored [K/128][scale_ld].
__global__ void quant_fp8_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale,
                                 int scale_ld, int M, int K, int x_ld) {
  pdl_trigger();
  pdl_wait();
  const int nvec = K >> 3;                                    // a multiple of 16
  const long long total = static_cast<long long>(M) * nvec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       idx < ((total + 31) / 32) * 32; idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const bool on = idx < total;                              // whole warps stay in the loop for the shuffles
    const int m = on ? static_cast<int>(idx / nvec) : 0, i = on ? static_cast<int>(idx % nvec) : 0;
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = 0.f;
    if (on) unpack8(reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * x_ld)[i], f);
    float am = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) am = fmaxf(am, fabsf(f[e]));
    am = group16_max(am);
    const float sc = fp8_group_scale(am);
    if (on) {
      reinterpret_cast<uint2*>(q + static_cast<size_t>(m) * K)[i] = pack8_e4m3(f, 1.f / sc);
      if ((i & 15) == 0) scale[static_cast<size_t>(i >> 4) * scale_ld + m] = sc;
    }
  }
}

// ----------------------------------------------------------------------------
// Embedding gather with vocabulary-shard awareness; rows whose id falls outside
// [vocab_lo, vocab_hi) are zero-filled (the TP all-reduce then completes them).
// Optional learned position table add and scale (GPT-style models).
__global__ void embedding_kernel(const int* __restrict__ ids, const bf16* __restrict__ table,
                                 const int* __restrict__ positions, const bf16* __restrict__ pos_table,
                                 bf16* __restrict__ out, int H, int vocab_lo, int vocab_hi, float scale) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool mine = id >= vocab_lo && id < vocab_hi;
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(mine ? id - vocab_lo : 0) * H);
  const uint4* psrc = pos_table ? reinterpret_cast<const uint4*>(pos_table + static_cast<size_t>(positions[t]) * H)
                                : nullptr;
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
    float f[8];
    if (mine) {
      unpack8(src[i], f);
      if (scale != 1.f) {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= scale;
      }
      if (psrc) {
        float pf[8];
        unpack8(psrc[i], pf);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += pf[e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    dst[i] = pack8(f);
  }
}

// out[r, :] = in[idx[r], :]  (last-token assembly, logits gather)
__global__ void gather_rows_kernel(const bf16* __restrict__ in, const int* __restrict__ idx, bf16* __restrict__ out,
                                   int H, int in_rows, int* err) {
  pdl_trigger();
  pdl_wait();
  int r = idx[blockIdx.x];
  if (r < 0 || r >= in_rows) { if (threadIdx.x == 0) guard_report(err, kGuardGatherRow, r); r = 0; }
  const uint4* src = reinterpret_cast<const uint4*>(in + static_cast<size_t>(r) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(blockIdx.x) * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = src[i];
}

// rows[pos[r], :] = emb[r, :] (fp32 source): input-refit embeddings from plugins.
__global__ void refit_rows_kernel(bf16* __restrict__ hidden, const int* __restrict__ pos, const float* __restrict__ emb,
                                  int H) {
  const float* src = emb + static_cast<size_t>(blockIdx.x) * H;
  bf16* dst = hidden + static_cast<size_t>(pos[blockIdx.x]) * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __float2bfloat16(src[i]);
}

// ----------------------------------------------------------------------------
// RoPE on q and k of the packed qkv activations + append of k, v to the paged
// cache (optionally as fp8 with per-layer scales), one CTA per token.
// qkv row layout: [Hq*D | Hkv*D | Hkv*D]. cos_sin: [max_pos][rot_dim] = cos(rot/2) | sin(rot/2).
// Cache layout per layer: [block][2][Hkv][block_tokens][D] with `block_stride` elements between blocks.
// slot < 0 skips the cache write (padding rows). neox: rotate halves; otherwise rotate pairs.
// positions may carry 3 rows ([3][T]) for multimodal rotary sections (mrope_s0/s1 = section ends in pairs).
template <typename CacheT>
__global__ void rope_kv_append_kernel(bf16* __restrict__ qkv, const int* __restrict__ positions, int pos_stride,
                                      const int* __restrict__ slots, const float* __restrict__ cos_sin,
                                      CacheT* __restrict__ cache, long long block_stride, int block_tokens, int Hq,
                                      int Hkv, int D, int rot_dim, int neox, int mrope_s0, int mrope_s1,
                                      float k_scale_inv, float v_scale_inv, int apply_rope) {
  const int t = blockIdx.x;
  bf16* row = qkv + static_cast<size_t>(t) * (Hq + 2 * Hkv) * D;
  const int half = rot_dim >> 1;
  if (apply_rope) {
    const int nrot = (Hq + Hkv) * half;
    for (int i = threadIdx.x; i < nrot; i += blockDim.x) {
      const int h = i / half, j = i % half;
      int pos = positions[t];
      if (pos_stride) {   // multimodal: pair index selects the temporal / height / width position row
        const int sec = j < mrope_s0 ? 0 : (j < mrope_s1 ? 1 : 2);
        pos = positions[sec * pos_stride + t];
      }
      const float* cs = cos_sin + static_cast<size_t>(pos) * rot_dim;
      const float c = cs[j], s = cs[half + j];
      bf16* hp = row + static_cast<size_t>(h) * D;
      const int i0 = neox ? j : 2 * j, i1 = neox ? j + half : 2 * j + 1;
      const float x0 = __bfloat162float(hp[i0]), x1 = __bfloat162float(hp[i1]);
      hp[i0] = __float2bfloat16(x0 * c - x1 * s);
      hp[i1] = __float2bfloat16(x1 * c + x0 * s);
    }
    __syncthreads();
  }
  const int slot = slots[t];
  if (slot < 0 || cache == nullptr) return;
  const int blk = slot / block_tokens, off = slot % block_tokens;
  CacheT* kbase = cache + static_cast<size_t>(blk) * block_stride;
  const bf16* ksrc = row + static_cast<size_t>(Hq) * D;
  const int n = Hkv * D;
  for (int i = threadIdx.x; i < 2 * n; i += blockDim.x) {
    const int kv = i / n, r = i % n;
    const int h = r / D, d = r % D;
    const float val = __bfloat162float(ksrc[i]);
    const size_t dst = ((static_cast<size_t>(kv) * Hkv + h) * block_tokens + off) * D + d;
    if constexpr (sizeof(CacheT) == 1) {
      kbase[dst] = static_cast<CacheT>(
          __nv_cvt_float_to_fp8(val * (kv ? v_scale_inv : k_scale_inv), __NV_SATFINITE, __NV_E4M3));
    } else {
      kbase[dst] = ksrc[i];
    }
  }
}

// Vector form of the kernel above for the common case (rotate halves over the whole head, one position row):
// a thread rotates 8 pairs with two 16-byte loads / stores and copies 8 cache elements per 16-byte load.
template <typename CacheT>
__global__ void rope_kv_append_vec_kernel(bf16* __restrict__ qkv, const int* __restrict__ positions,
                                          const int* __restrict__ slots, const float* __restrict__ cos_sin,
                                          CacheT* __restrict__ cache, long long block_stride, int block_tokens, int Hq,
                                          int Hkv, int D, float k_scale_inv, float v_scale_inv, int apply_rope) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  bf16* row = qkv + static_cast<size_t>(t) * (Hq + 2 * Hkv) * D;
  const int half = D >> 1, hv = half >> 3;                   // 16-byte vectors per half head
  if (apply_rope) {
    const float* cs = cos_sin + static_cast<size_t>(positions[t]) * D;
    const int items = (Hq + Hkv) * hv;
    for (int i = threadIdx.x; i < items; i += blockDim.x) {
      const int h = i / hv, j0 = (i - h * hv) << 3;
      bf16* hp = row + static_cast<size_t>(h) * D;
      float x0[8], x1[8], c[8], sn[8], y0[8], y1[8];
      unpack8(*reinterpret_cast<const uint4*>(hp + j0), x0);
      unpack8(*reinterpret_cast<const uint4*>(hp + half + j0), x1);
      *reinterpret_cast<float4*>(&c[0]) = *reinterpret_cast<const float4*>(cs + j0);
      *reinterpret_cast<float4*>(&c[4]) = *reinterpret_cast<const float4*>(cs + j0 + 4);
      *reinterpret_cast<float4*>(&sn[0]) = *reinterpret_cast<const float4*>(cs + half + j0);
      *reinterpret_cast<float4*>(&sn[4]) = *reinterpret_cast<const float4*>(cs + half + j0 + 4);
#pragma unroll
      for (int e = 0; e < 8; ++e) { y0[e] = x0[e] * c[e] - x1[e] * sn[e]; y1[e] = x1[e] * c[e] + x0[e] * sn[e]; }
      *reinterpret_cast<uint4*>(hp + j0) = pack8(y0);
      *reinterpret_cast<uint4*>(hp + half + j0) = pack8(y1);
    }
    __syncthreads();
  }
  const int slot = slots[t];
  if (slot < 0 || cache == nullptr) return;
  const int blk = slot / block_tokens, off = slot % block_tokens;
  CacheT* kbase = cache + static_cast<size_t>(blk) * block_stride;
  const bf16* ksrc = row + static_cast<size_t>(Hq) * D;
  const int dv = D >> 3, n8 = Hkv * dv;
  for (int i = threadIdx.x; i < 2 * n8; i += blockDim.x) {
    const int kv = i / n8, r = i - kv * n8;
    const int h = r / dv, d = (r - h * dv) << 3;
    const uint4 v = *reinterpret_cast<const uint4*>(ksrc + (static_cast<size_t>(i) << 3));
    const size_t dst = ((static_cast<size_t>(kv) * Hkv + h) * block_tokens + off) * D + d;
    if constexpr (sizeof(CacheT) == 1) {
      float f[8];
      unpack8(v, f);
      *reinterpret_cast<uint2*>(kbase + dst) = pack8_e4m3(f, kv ? v_scale_inv : k_scale_inv);
    } else {
      *reinterpret_cast<uint4*>(kbase + dst) = v;
    }
  }
}

// Block-to-block copy inside the paged cache (beam fork, flexible cache, swap staging):
// pairs[2*i] = source block, pairs[2*i+1] = destination block; copies all layers of a block.
// A block id outside [0, num_blocks) is recorded in the error word and its copy is skipped.
__global__ void copy_blocks_kernel(uint4* __restrict__ cache, const int* __restrict__ pairs, long long block_vec,
                                   int num_blocks, int* err) {
  const int sb = pairs[2 * blockIdx.x], db = pairs[2 * blockIdx.x + 1];
  if (sb < 0 || sb >= num_blocks || db < 0 || db >= num_blocks) {
    if (threadIdx.x == 0 && blockIdx.y == 0) guard_report(err, kGuardBlockId, (sb < 0 || sb >= num_blocks) ? sb : db);
    return;
  }
  const uint4* src = cache + static_cast<size_t>(sb) * block_vec;
  uint4* dst = cache + static_cast<size_t>(db) * block_vec;
  for (long long i = blockIdx.y * static_cast<long long>(blockDim.x) + threadIdx.x; i < block_vec;
       i += static_cast<long long>(gridDim.y) * blockDim.x)
    dst[i] = src[i];
}

// Whole cache blocks between the device cache and a pool of host blocks in pinned (device-visible) host memory:
// pairs[2*i] = device block, pairs[2*i+1] = host block; dir 0: cache -> host pool, 1: host pool -> cache. One launch
// per swap list; the kernel moves the bytes over PCIe itself, so no staging copy and no host synchronisation is
// needed. Ids outside their pools are recorded in the error word and skipped.
__global__ void swap_blocks_kernel(uint4* __restrict__ cache, uint4* __restrict__ pool, const int* __restrict__ pairs,
                                   long long block_vec, int dir, int num_blocks, int num_pool_blocks, int* err) {
  const int b = pairs[2 * blockIdx.x], hb = pairs[2 * blockIdx.x + 1];
  if (b < 0 || b >= num_blocks || hb < 0 || hb >= num_pool_blocks) {
    if (threadIdx.x == 0 && blockIdx.y == 0) guard_report(err, kGuardBlockId, (b < 0 || b >= num_blocks) ? b : hb);
    return;
  }
  uint4* c = cache + static_cast<size_t>(b) * block_vec;
  uint4* s = pool + static_cast<size_t>(hb) * block_vec;
  for (long long i = blockIdx.y * static_cast<long long>(blockDim.x) + threadIdx.x; i < block_vec;
       i += static_cast<long long>(gridDim.y) * blockDim.x) {
    if (dir == 0) s[i] = c[i]; else c[i] = s[i];
  }
}

// Flexible-cache copies land at another position of the sequence: the K rows of the destination block are rotated by
// the position delta (rotary rotations add, so one rotation by |delta| with the sign on the sine does it), in place,
// for every layer and KV head of the block. triples[3*i] = source block (unused here), [3*i+1] = destination block,
// [3*i+2] = position delta. Cache layout [blocks][layers][2][kv heads][block tokens][head dim], K panel first;
// cos_sin [max_pos][rot_dim] = cos | sin (fp32). FP8 caches are rotated on their raw values (the tensor scale is
// a common factor). Bad block ids and deltas beyond the table are recorded in the error word and skipped.
template <typename T>
__device__ __forceinline__ float kv_to_float(T v);
template <> __device__ __forceinline__ float kv_to_float<bf16>(bf16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float kv_to_float<uint8_t>(uint8_t v) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(v, __NV_E4M3)));
}
template <typename T>
__device__ __forceinline__ T kv_from_float(float v);
template <> __device__ __forceinline__ bf16 kv_from_float<bf16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ uint8_t kv_from_float<uint8_t>(float v) {
  return __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

template <typename T>
__global__ void rerotate_blocks_kernel(T* __restrict__ cache, const int* __restrict__ triples, const float* __restrict__ cos_sin,
                                       int max_pos, int layers, int hkv, int bt, int D, int rot_dim, int neox,
                                       int num_blocks, int* err) {
  const int db = triples[3 * blockIdx.x + 1], delta = triples[3 * blockIdx.x + 2];
  if (delta == 0) return;
  const int ad = delta < 0 ? -delta : delta;
  if (db < 0 || db >= num_blocks || ad >= max_pos) {
    if (threadIdx.x == 0 && blockIdx.y == 0) guard_report(err, db < 0 || db >= num_blocks ? kGuardBlockId : kGuardPosition,
                                                          db < 0 || db >= num_blocks ? db : ad);
    return;
  }
  const int half = rot_dim >> 1;
  const float* cs = cos_sin + static_cast<size_t>(ad) * rot_dim;
  const float sgn = delta > 0 ? 1.f : -1.f;
  const long long panel = static_cast<long long>(bt) * D;                 // one head's K panel
  const long long layer_stride = 2LL * hkv * panel, block_stride = layers * layer_stride;
  T* blk = cache + static_cast<size_t>(db) * block_stride;
  const long long pairs = static_cast<long long>(layers) * hkv * bt * half;
  for (long long i = blockIdx.y * static_cast<long long>(blockDim.x) + threadIdx.x; i < pairs;
       i += static_cast<long long>(gridDim.y) * blockDim.x) {
    const int j = static_cast<int>(i % half);
    long long t = i / half;
    const int tok = static_cast<int>(t % bt); t /= bt;
    const int head = static_cast<int>(t % hkv);
    const int layer = static_cast<int>(t / hkv);
    T* row = blk + layer * layer_stride + head * panel + static_cast<long long>(tok) * D;
    const int i0 = neox ? j : 2 * j, i1 = neox ? j + half : 2 * j + 1;
    const float c = cs[j], sn = cs[half + j] * sgn;
    const float x0 = kv_to_float<T>(row[i0]), x1 = kv_to_float<T>(row[i1]);
    row[i0] = kv_from_float<T>(x0 * c - x1 * sn);
    row[i1] = kv_from_float<T>(x1 * c + x0 * sn);
  }
}

// Largest magnitude of a bf16 matrix as a quantisation scale on the device: scale = max(|x|) / divisor (at least
// `floor`), without a host round trip and without a widened copy of x. `acc` is a zeroed 32-bit word; magnitudes are
// non-negative, so their bit patterns order like integers and atomicMax works on them. The finishing kernel writes the
// scale and leaves `acc` at zero for the next call.
__global__ void absmax_kernel(const bf16* __restrict__ x, int rows, int cols, long long ldx, unsigned int* acc) {
  __shared__ float red[32];
  const int vec_per_row = cols >> 3;
  const long long nvec = static_cast<long long>(rows) * vec_per_row;
  float m = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row);
    const uint4 v = *reinterpret_cast<const uint4*>(x + r * ldx + c * 8);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(p[k]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (threadIdx.x == 0 && m > 0.f && m == m) atomicMax(acc, __float_as_uint(m));
  }
}
__global__ void absmax_finish_kernel(unsigned int* acc, float* scale, float inv_divisor, float floor_value) {
  *scale = fmaxf(__uint_as_float(*acc) * inv_divisor, floor_value);
  *acc = 0u;
}

// ids[rows[i]] = prev_tokens[src[i]]: a pipelined step takes the input ids of its decode rows straight from the
// previous step's sampler output on the device (the host has not read those tokens yet).
__global__ void patch_ids_kernel(int* __restrict__ ids, const int* __restrict__ rows, const int* __restrict__ src,
                                 const int* __restrict__ prev_tokens, int n, int n_ids, int n_prev, int* err) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = rows[i], sidx = src[i];
  if (r < 0 || r >= n_ids || sidx < 0 || sidx >= n_prev) { guard_report(err, kGuardGatherRow, r < 0 || r >= n_ids ? r : sidx); return; }
  ids[r] = prev_tokens[sidx];
}

// out = a + b (+ bias), bf16 (used for unfused residual paths and the baseline backend)
__global__ void add_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, const bf16* __restrict__ bias,
                           bf16* __restrict__ out, long long nvec_total, int nvec_row) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec_total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float x[8], y[8];
    unpack8(reinterpret_cast<const uint4*>(a)[i], x);
    if (b) {
      unpack8(reinterpret_cast<const uint4*>(b)[i], y);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] += y[e];
    }
    if (bias) {
      unpack8(reinterpret_cast<const uint4*>(bias)[i % nvec_row], y);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] += y[e];
    }
    reinterpret_cast<uint4*>(out)[i] = pack8(x);
  }
}

// bf16 -> fp32 cast of selected rows (logits for the sampler when the GEMM wrote bf16)
__global__ void cast_f32_kernel(const bf16* __restrict__ in, float* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = __bfloat162float(in[i]);
}

static inline int grid_for(long long work, int threads, int cap = 148 * 8) {
  long long g = (work + threads - 1) / threads;
  if (g < 1) g = 1;
  return static_cast<int>(g > cap ? cap : g);
}
static inline int norm_threads(int H) {
  int t = ((H >> 3) + kMaxVec - 1) / kMaxVec;
  t = ((t + 31) / 32) * 32;
  if (t < 32) t = 32;
  return t > 1024 ? 1024 : t;
}

// ----------------------------------------------------------------------------
// NVFP4 quantisation of GEMM inputs: 16-element blocks along K, e2m1 values (two per byte, even element in the
// low nibble), one e4m3 scale per block, one fp32 scale per tensor (given): x ~= e2m1 * block_scale * tensor_scale.
__global__ void quant_nvfp4_kernel(const bf16* __restrict__ x, int ldx, uint8_t* __restrict__ q, int ldq,
                                   uint8_t* __restrict__ bs, int ldbs, const float* __restrict__ ts, int M, int K) {
  const int nb = K >> 4;
  const long long total = static_cast<long long>(M) * nb;
  const float inv_ts = 1.f / (ts ? *ts : 1.f);
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(idx / nb), b = static_cast<int>(idx % nb);
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ldx + b * 16);
    float f[16];
    unpack8(src[0], *reinterpret_cast<float(*)[8]>(&f[0]));
    unpack8(src[1], *reinterpret_cast<float(*)[8]>(&f[8]));
    float am = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) { f[i] *= inv_ts; am = fmaxf(am, fabsf(f[i])); }
    const __nv_fp8_storage_t sc8 = __nv_cvt_float_to_fp8(fminf(am / 6.f, 448.f), __NV_SATFINITE, __NV_E4M3);
    const float scf = fmaxf(__half2float(__half(__nv_cvt_fp8_to_halfraw(sc8, __NV_E4M3))), 1.f / 512.f);
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __nv_fp4x2_storage_t v = __nv_cvt_float2_to_fp4x2(make_float2(f[2 * i] / scf, f[2 * i + 1] / scf), __NV_E2M1,
                                                              cudaRoundNearest);
      w[i >> 2] |= static_cast<uint32_t>(v) << (8 * (i & 3));
    }
    *reinterpret_cast<uint2*>(q + static_cast<size_t>(row) * ldq + b * 8) = make_uint2(w[0], w[1]);
    bs[static_cast<size_t>(row) * ldbs + b] = sc8;
  }
}

}  // namespace ksana

using namespace ksana;

extern "C" int ksana_norm(const void* x, void* residual, const void* w, const void* beta, void* y, void* yq,
                          float* yscale, int scale_ld, int M, int H, float eps, int layernorm, cudaStream_t st) {
  if (M <= 0) return 0;
  if (H % 8 || H > 8 * kMaxVec * 1024) return -10;
  if (yq && (H % 128)) return -11;
  const int threads = norm_threads(H);
  if (layernorm)
    launch_pdl(norm_kernel<1>, dim3(M), dim3(threads), 0, st, (const bf16*)x, (bf16*)residual, (const bf16*)w, (const bf16*)beta, (bf16*)y,
                                          (uint8_t*)yq, yscale, scale_ld, H, eps);
  else
    launch_pdl(norm_kernel<0>, dim3(M), dim3(threads), 0, st, (const bf16*)x, (bf16*)residual, (const bf16*)w, (const bf16*)beta, (bf16*)y,
                                          (uint8_t*)yq, yscale, scale_ld, H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_act_mul(const void* in, void* out, void* outq, float* oscale, int scale_ld, int M, int I,
                             int in_ld, int act, int gated, cudaStream_t st) {
  if (M <= 0) return 0;
  if (I % 8 || in_ld % 8) return -10;
  if (outq && (I % 128)) return -11;
  const long long total = static_cast<long long>(M) * (I >> 3);
  launch_pdl(act_mul_kernel, dim3(grid_for(total, 256)), dim3(256), 0, st, (const bf16*)in, (bf16*)out, (uint8_t*)outq, oscale, scale_ld, M,
                                                       I, in_ld, act, gated);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_quant_fp8(const void* x, void* q, float* scale, int scale_ld, int M, int K, int x_ld,
                               cudaStream_t st) {
  if (M <= 0) return 0;
  if (K % 128 || x_ld % 8) return -10;
  const long long total = static_cast<long long>(M) * (K >> 3);
  launch_pdl(quant_fp8_kernel, dim3(grid_for(total, 256)), dim3(256), 0, st, (const bf16*)x, (uint8_t*)q, scale, scale_ld, M, K, x_ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// x [M, K] bf16 -> q [M, K/2] packed e2m1, bs [M, K/16] e4m3 block scales; ts: device fp32 tensor scale (null = 1).
extern "C" int ksana_quant_nvfp4(const void* x, int x_ld, void* q, int q_ld, void* bs, int bs_ld, const float* ts, int M,
                                 int K, cudaStream_t st) {
  if (M <= 0) return 0;
  if (K % 16 || x_ld % 8 || q_ld % 8) return -10;
  const long long total = static_cast<long long>(M) * (K >> 4);
  quant_nvfp4_kernel<<<grid_for(total, 256), 256, 0, st>>>((const bf16*)x, x_ld, (uint8_t*)q, q_ld, (uint8_t*)bs, bs_ld,
                                                           ts, M, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_embedding(const int* ids, const void* table, const int* positions, const void* pos_table,
                               void* out, int T, int H, int vocab_lo, int vocab_hi, float scale, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  launch_pdl(embedding_kernel, dim3(T), dim3(256), 0, st, ids, (const bf16*)table, positions, (const bf16*)pos_table, (bf16*)out, H,
                                      vocab_lo, vocab_hi, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_gather_rows(const void* in, const int* idx, void* out, int R, int H, int in_rows, int* err,
                                 cudaStream_t st) {
  if (R <= 0) return 0;
  if (H % 8 || in_rows <= 0) return -10;
  launch_pdl(gather_rows_kernel, dim3(R), dim3(256), 0, st, (const bf16*)in, idx, (bf16*)out, H, in_rows, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_refit_rows(void* hidden, const int* pos, const float* emb, int R, int H, cudaStream_t st) {
  if (R <= 0) return 0;
  refit_rows_kernel<<<R, 256, 0, st>>>((bf16*)hidden, pos, emb, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_rope_kv_append(void* qkv, const int* positions, int pos_stride, const int* slots,
                                    const float* cos_sin, void* cache, long long block_stride, int block_tokens, int T,
                                    int Hq, int Hkv, int D, int rot_dim, int neox, int mrope_s0, int mrope_s1,
                                    int cache_fp8, float k_scale, float v_scale, int apply_rope, cudaStream_t st) {
  if (T <= 0) return 0;
  if (neox && rot_dim == D && (D % 16) == 0 && pos_stride == 0 && (block_stride % 16) == 0 &&
      (reinterpret_cast<uintptr_t>(qkv) % 16) == 0 && (reinterpret_cast<uintptr_t>(cache) % 16) == 0 &&
      (reinterpret_cast<uintptr_t>(cos_sin) % 16) == 0) {
    if (cache_fp8)
      launch_pdl(rope_kv_append_vec_kernel<uint8_t>, dim3(T), dim3(256), 0, st, (bf16*)qkv, positions, slots, cos_sin, (uint8_t*)cache,
                                                            block_stride, block_tokens, Hq, Hkv, D, 1.f / k_scale,
                                                            1.f / v_scale, apply_rope);
    else
      launch_pdl(rope_kv_append_vec_kernel<bf16>, dim3(T), dim3(256), 0, st, (bf16*)qkv, positions, slots, cos_sin, (bf16*)cache,
                                                         block_stride, block_tokens, Hq, Hkv, D, 1.f, 1.f, apply_rope);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  if (cache_fp8)
    rope_kv_append_kernel<uint8_t><<<T, 256, 0, st>>>((bf16*)qkv, positions, pos_stride, slots, cos_sin,
                                                      (uint8_t*)cache, block_stride, block_tokens, Hq, Hkv, D, rot_dim,
                                                      neox, mrope_s0, mrope_s1, 1.f / k_scale, 1.f / v_scale,
                                                      apply_rope);
  else
    rope_kv_append_kernel<bf16><<<T, 256, 0, st>>>((bf16*)qkv, positions, pos_stride, slots, cos_sin, (bf16*)cache,
                                                   block_stride, block_tokens, Hq, Hkv, D, rot_dim, neox, mrope_s0,
                                                   mrope_s1, 1.f, 1.f, apply_rope);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_copy_blocks(void* cache, const int* pairs, int npairs, long long block_bytes, int num_blocks,
                                 int* err, cudaStream_t st) {
  if (npairs <= 0) return 0;
  if (block_bytes % 16) return -10;
  copy_blocks_kernel<<<dim3(npairs, 16), 256, 0, st>>>((uint4*)cache, pairs, block_bytes / 16, num_blocks, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_swap_blocks(void* cache, void* pool, const int* pairs, int n, long long block_bytes, int dir,
                                 int num_blocks, int num_pool_blocks, int* err, cudaStream_t st) {
  if (n <= 0) return 0;
  if (block_bytes % 16) return -10;
  swap_blocks_kernel<<<dim3(n, 16), 256, 0, st>>>((uint4*)cache, (uint4*)pool, pairs, block_bytes / 16, dir, num_blocks,
                                                  num_pool_blocks, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// kv_bytes: 2 (bf16 cache) or 1 (e4m3 cache).
extern "C" int ksana_rerotate_blocks(void* cache, const int* triples, int n, const float* cos_sin, int max_pos, int layers,
                                     int hkv, int bt, int D, int rot_dim, int neox, int kv_bytes, int num_blocks,
                                     int* err, cudaStream_t st) {
  if (n <= 0) return 0;
  if (rot_dim <= 0 || rot_dim > D || (rot_dim & 1) || (kv_bytes != 1 && kv_bytes != 2)) return -10;
  if (kv_bytes == 2)
    rerotate_blocks_kernel<bf16><<<dim3(n, 8), 256, 0, st>>>((bf16*)cache, triples, cos_sin, max_pos, layers, hkv, bt, D,
                                                            rot_dim, neox, num_blocks, err);
  else
    rerotate_blocks_kernel<uint8_t><<<dim3(n, 8), 256, 0, st>>>((uint8_t*)cache, triples, cos_sin, max_pos, layers, hkv,
                                                                bt, D, rot_dim, neox, num_blocks, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// scale[0] = max(max |x| / divisor, floor) for x [rows, cols] bf16 (row stride ldx, cols a multiple of 8); acc: one
// zeroed 32-bit word of device scratch that the call leaves zeroed.
extern "C" int ksana_absmax_scale(const void* x, int rows, int cols, long long ldx, float divisor, float floor_value,
                                  void* acc, float* scale, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols % 8) || (ldx % 8) || divisor <= 0.f || (reinterpret_cast<uintptr_t>(x) & 15)) return -10;
  const long long nvec = static_cast<long long>(rows) * (cols >> 3);
  absmax_kernel<<<grid_for(nvec, 256), 256, 0, st>>>((const bf16*)x, rows, cols, ldx, (unsigned int*)acc);
  absmax_finish_kernel<<<1, 1, 0, st>>>((unsigned int*)acc, scale, 1.f / divisor, floor_value);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_patch_ids(int* ids, const int* rows, const int* src, const int* prev_tokens, int n, int n_ids,
                               int n_prev, int* err, cudaStream_t st) {
  if (n <= 0) return 0;
  return launch_pdl(patch_ids_kernel, dim3((n + 127) / 128), dim3(128), 0, st, ids, rows, src, prev_tokens, n, n_ids,
                    n_prev, err) == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_add(const void* a, const void* b, const void* bias, void* out, long long M, int H,
                         cudaStream_t st) {
  if (M <= 0) return 0;
  if (H % 8) return -10;
  const long long nvec = M * (H >> 3);
  add_kernel<<<grid_for(nvec, 256), 256, 0, st>>>((const bf16*)a, (const bf16*)b, (const bf16*)bias, (bf16*)out, nvec,
                                                  H >> 3);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_cast_f32(const void* in, float* out, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  cast_f32_kernel<<<grid_for(n, 256), 256, 0, st>>>((const bf16*)in, out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
