// Weight-only 4-bit linear layers (GPTQ / AWQ style group quantisation, bf16 activations).
//
// Storage (one format for both checkpoint families, produced by the loader):
//   qw    [N, K/2] uint8   two weights per byte along K: low nibble = even k, high nibble = odd k, values 0..15
//   scale [N, K/g] fp16    group scale (the checkpoints' own precision)
//   zs    [N, K/g] fp16    zero point times scale, so w[n,k] = q * scale - zs
// Decode steps (M <= 8 rows per pass) are weight streams at half a byte per weight: a CUDA-core kernel where every
// warp owns four output features, unpacks 32 weights per lane and step and keeps the M x 4 accumulators in
// registers (the activations come through L1 and are shared by the four features). Larger batches are compute
// bound: the weights are expanded to bf16 once per call into a scratch matrix that the tcgen05 bf16 GEMM consumes.
// Counterpart of the reference's CUTLASS fpA_intB / Marlin / batched-GEMV trio
// (3rdparty/LLM_kernels/csrc/kernels/nvidia/asymmetric_gemm/fpA_intB_gemm, gptq_marlin, weight_only_batched_gemv).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ksana {

typedef __nv_bfloat16 bf16;
constexpr int kW4Feat = 4;          // output features per warp
constexpr int kW4Warps = 8;

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// y[m, n] = sum_k x[m, k] * (q[n, k] * scale[n, k/g] - zs[n, k/g]) (+ bias[n]) (+ residual[m, n])
// K % 32 == 0, g % 32 == 0 (a lane's 32 weights never straddle a group).
template <int M>
__global__ void __launch_bounds__(kW4Warps * 32)
w4_gemv_kernel(const bf16* __restrict__ x, long long ldx, const uint8_t* __restrict__ qw, const __half* __restrict__ scale,
               const __half* __restrict__ zs, const bf16* __restrict__ bias, const bf16* __restrict__ residual, long long ldr,
               bf16* __restrict__ y, long long ldy, int N, int K, int g) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * kW4Warps + warp) * kW4Feat;
  if (n0 >= N) return;
  const int ngroups = K / g;
  float acc[M][kW4Feat];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int f = 0; f < kW4Feat; ++f) acc[m][f] = 0.f;

  for (int k0 = lane * 32; k0 < K; k0 += 32 * 32) {
    const int grp = k0 / g;
    uint4 wq[kW4Feat];
    float sc[kW4Feat], z[kW4Feat];
#pragma unroll
    for (int f = 0; f < kW4Feat; ++f) {
      const int n = min(n0 + f, N - 1);
      wq[f] = __ldg(reinterpret_cast<const uint4*>(qw + static_cast<size_t>(n) * (K >> 1) + (k0 >> 1)));
      sc[f] = __half2float(scale[static_cast<size_t>(n) * ngroups + grp]);
      z[f] = __half2float(zs[static_cast<size_t>(n) * ngroups + grp]);
    }
    float xs[M], dot[M][kW4Feat];
#pragma unroll
    for (int m = 0; m < M; ++m) {
      xs[m] = 0.f;
#pragma unroll
      for (int f = 0; f < kW4Feat; ++f) dot[m][f] = 0.f;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {             // 8 weights per 32-bit word = one uint4 of activations per row
      uint4 xv[M];
#pragma unroll
      for (int m = 0; m < M; ++m) xv[m] = __ldg(reinterpret_cast<const uint4*>(x + m * ldx + k0) + c);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x0[M], x1[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint32_t xw = reinterpret_cast<const uint32_t*>(&xv[m])[e];
          x0[m] = bf16_lo(xw);
          x1[m] = bf16_hi(xw);
          xs[m] += x0[m] + x1[m];
        }
#pragma unroll
        for (int f = 0; f < kW4Feat; ++f) {
          const uint32_t w = reinterpret_cast<const uint32_t*>(&wq[f])[c];
          const float q0 = static_cast<float>((w >> (8 * e)) & 15u), q1 = static_cast<float>((w >> (8 * e + 4)) & 15u);
#pragma unroll
          for (int m = 0; m < M; ++m) dot[m][f] = fmaf(q1, x1[m], fmaf(q0, x0[m], dot[m][f]));
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int f = 0; f < kW4Feat; ++f) acc[m][f] += dot[m][f] * sc[f] - xs[m] * z[f];
  }
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int f = 0; f < kW4Feat; ++f) {
      float v = acc[m][f];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[m][f] = v;
    }
  if (lane < M * kW4Feat) {
    const int m = lane / kW4Feat, f = lane % kW4Feat;
    float v = 0.f;
#pragma unroll
    for (int mm = 0; mm < M; ++mm)
#pragma unroll
      for (int ff = 0; ff < kW4Feat; ++ff)
        if (mm == m && ff == f) v = acc[mm][ff];
    const int n = n0 + f;
    if (n < N) {
      if (bias) v += __bfloat162float(bias[n]);
      if (residual) v += __bfloat162float(residual[m * ldr + n]);
      y[m * ldy + n] = __float2bfloat16(v);
    }
  }
}

// Expansion to bf16 [N, K] (row stride ldw) for the compute-bound path: one thread per 8 weights.
__global__ void w4_dequant_kernel(const uint8_t* __restrict__ qw, const __half* __restrict__ scale, const __half* __restrict__ zs,
                                  bf16* __restrict__ w, long long ldw, int N, int K, int g) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const int kv = K >> 3;
  if (i >= static_cast<long long>(N) * kv) return;
  const int n = static_cast<int>(i / kv), k0 = static_cast<int>(i % kv) * 8;
  const uint32_t q = *reinterpret_cast<const uint32_t*>(qw + static_cast<size_t>(n) * (K >> 1) + (k0 >> 1));
  const int ngroups = K / g;
  const float sc = __half2float(scale[static_cast<size_t>(n) * ngroups + k0 / g]);
  const float z = __half2float(zs[static_cast<size_t>(n) * ngroups + k0 / g]);
  uint4 out;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int e = 0; e < 4; ++e)
    o2[e] = __floats2bfloat162_rn(static_cast<float>((q >> (8 * e)) & 15u) * sc - z,
                                  static_cast<float>((q >> (8 * e + 4)) & 15u) * sc - z);
  *reinterpret_cast<uint4*>(w + static_cast<size_t>(n) * ldw + k0) = out;
}

template <int M>
static void launch_gemv(const bf16* x, long long ldx, const uint8_t* qw, const __half* scale, const __half* zs, const bf16* bias,
                        const bf16* residual, long long ldr, bf16* y, long long ldy, int N, int K, int g, cudaStream_t st) {
  const int per_block = kW4Warps * kW4Feat;
  w4_gemv_kernel<M><<<(N + per_block - 1) / per_block, kW4Warps * 32, 0, st>>>(x, ldx, qw, scale, zs, bias, residual, ldr, y,
                                                                              ldy, N, K, g);
}

}  // namespace ksana

using namespace ksana;

// y [M, N] = x [M, K] W^T for 4-bit group-quantised W, M rows in passes of at most 8. Returns -10 on unsupported shapes.
extern "C" int ksana_w4_gemv(const void* x, long long ldx, const void* qw, const void* scale, const void* zs,
                             const void* bias, const void* residual, long long ldr, void* y, long long ldy, int M, int N,
                             int K, int g, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 32 || g % 32 || K % g || (ldx % 8) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(qw) & 15))
    return -10;
  const bf16* xp = static_cast<const bf16*>(x);
  const bf16* rp = static_cast<const bf16*>(residual);
  bf16* yp = static_cast<bf16*>(y);
  for (int m0 = 0; m0 < M; m0 += 8) {
    const int m = M - m0 < 8 ? M - m0 : 8;
    const bf16* xr = xp + m0 * ldx;
    const bf16* rr = rp ? rp + m0 * ldr : nullptr;
    bf16* yr = yp + m0 * ldy;
#define KSANA_W4_CASE(MM)                                                                                              \
  case MM:                                                                                                             \
    launch_gemv<MM>(xr, ldx, static_cast<const uint8_t*>(qw), static_cast<const __half*>(scale), static_cast<const __half*>(zs), \
                    static_cast<const bf16*>(bias), rr, ldr, yr, ldy, N, K, g, st);                                    \
    break;
    switch (m) {
      KSANA_W4_CASE(1) KSANA_W4_CASE(2) KSANA_W4_CASE(3) KSANA_W4_CASE(4)
      KSANA_W4_CASE(5) KSANA_W4_CASE(6) KSANA_W4_CASE(7) KSANA_W4_CASE(8)
    }
#undef KSANA_W4_CASE
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_w4_dequant(const void* qw, const void* scale, const void* zs, void* w, long long ldw, int N, int K,
                                int g, cudaStream_t st) {
  if (N <= 0) return 0;
  if (K % 8 || g % 8 || K % g || (ldw % 8)) return -10;
  const long long n = static_cast<long long>(N) * (K >> 3);
  w4_dequant_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
      static_cast<const uint8_t*>(qw), static_cast<const __half*>(scale), static_cast<const __half*>(zs), static_cast<bf16*>(w),
      ldw, N, K, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
