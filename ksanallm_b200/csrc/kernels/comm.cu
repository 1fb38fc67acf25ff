// Tensor-parallel collectives over NVLink peer memory, fused with the memory-bound work that
// follows them. One process per GPU; every rank maps every peer's symmetric buffer, so kernels
// address peers with plain pointers (P2P loads / stores through NVSwitch).
//
// Row-parallel linear (o_proj, down_proj) in two kernels:
//   1. the GEMM kernels (gemm_tcgen05.cu / gemm_smallm.cu) run in "push" mode: their epilogue stores
//      each partial tile straight into the receive slot of the rank that will reduce those rows
//      (posted P2P stores, so the reduce-scatter traffic overlaps the remaining tiles' math);
//   2. reduce_norm_kernel (here): waits - bounded - until every peer's pushes for this epoch are
//      flagged, sums the partial slots in rank order (identical bits on every rank), adds the
//      residual, applies RMSNorm / LayerNorm, optionally quantises to FP8 (1x128 scales) for the next
//      GEMM, and (large batches) pushes its row slice of the results to every peer (all-gather).
// This replaces NCCL all-reduce + add + norm (+ quant) of the reference op sequence
// (src/ksana_llm/models/common/common_model.cpp:498-527,549-569,586-615) and its custom all-reduce
// (3rdparty/LLM_kernels/csrc/kernels/nvidia/all_reduce/custom_all_reduce.cu:116-400), whose flag
// spins are unbounded.
//
// Flags: each rank owns a pad of 32-bit words in its symmetric memory. Word [kind*16 + r] holds the
// last epoch for which rank r signalled `kind` to this rank. Epochs only grow, so flags are never reset.
// The epoch of a call is read from a device counter (ctrs[kind]) and advanced by the last block of the
// call, so a launch captured in a CUDA graph gets a fresh epoch on every replay. All ranks issue the same
// sequence of collective calls, which keeps their counters in step.
// A wait that exceeds its budget sets the error word and the kernel skips the dependent work.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include "fp8_scale.cuh"
#include "pdl.cuh"
#include <cstdlib>

namespace ksana {

typedef __nv_bfloat16 bf16;
constexpr int kMaxRanks = 8;
constexpr int kFlagStride = 16;

struct CommPeers {
  void* data[kMaxRanks];          // peers' symmetric data buffers (same layout on every rank)
  uint32_t* flags[kMaxRanks];     // peers' flag pads
  int rank, size;
  int spin_limit;                 // polls a wait on a peer's flag may take before it gives up (see kSpinLimit)
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Budget of a peer wait: kSpinLimit polls with a short sleep each (about a second in total).
constexpr int kSpinLimit = 1 << 20;

// Signal `kind` for `epoch` to every peer (one thread per peer of block 0), then every block waits until
// all peers have signalled the same. Returns false on timeout (err word set).
__device__ __forceinline__ bool signal_and_wait(const CommPeers& c, int kind, uint32_t epoch, int* err, bool do_signal) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (do_signal && blockIdx.x == 0 && threadIdx.x < c.size) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + kind * kFlagStride + c.rank, epoch);
  }
  if (threadIdx.x < c.size) {
    const uint32_t* f = c.flags[c.rank] + kind * kFlagStride + threadIdx.x;
    int it = 0;
    // signed distance handles wrap-around of the 32-bit epoch
    while (static_cast<int32_t>(ld_acquire_sys(f) - epoch) < 0) {
      if (++it > c.spin_limit) { s_ok = 0; if (err) atomicExch(err, 3); break; }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return s_ok != 0;
}

__device__ __forceinline__ void unpack8c(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8c(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
__device__ __forceinline__ uint2 pack8_e4m3c(const float (&f)[8], float inv_scale) {
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

// Epoch bookkeeping in local device memory: ctrs[kind] = last completed epoch, ctrs[8 + kind] = blocks done.
__device__ __forceinline__ uint32_t begin_epoch(const uint32_t* ctrs, int kind) {
  return *reinterpret_cast<const volatile uint32_t*>(ctrs + kind) + 1;
}
// Returns true (to every thread of the block) in the last block of the grid to get here. `sys`: the block's stores
// to peers are made visible system-wide before it is counted, so that the last block may tell the peers about them.
__device__ __forceinline__ bool end_epoch(uint32_t* ctrs, int kind, uint32_t epoch, bool sys = false) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (sys) __threadfence_system(); else __threadfence();
    const bool last = atomicAdd(ctrs + 8 + kind, 1u) == gridDim.x - 1;
    if (last) {
      ctrs[8 + kind] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(ctrs + kind) = epoch;
    }
    s_last = last ? 1 : 0;
  }
  __syncthreads();
  return s_last != 0;
}

// "My rows are delivered": the last block of a kernel that pushed rows to the peers raises flag `kind` at every
// peer with the next epoch of that kind; the consumer's wait (the last block of gather_finish_kernel)
// reads the same counter after this kernel has finished.
__device__ __forceinline__ void signal_delivered(const CommPeers& c, uint32_t* ctrs, int kind) {
  const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(ctrs + kind) + 1;
  if (threadIdx.x < c.size) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + kind * kFlagStride + c.rank, epoch);
  }
  __syncthreads();
  if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(ctrs + kind) = epoch;
}

struct ReduceNormParams {
  CommPeers peers;
  uint32_t* ctrs;
  // receive slots in the local symmetric buffer: slot r at slots_off + r * slot_stride (bytes), each
  // [rows_local, H] bf16 where rows_local = rows this rank reduces
  long long slots_off, slot_stride;
  int row_begin, row_count;       // rows of the full [M, H] problem this rank reduces (all rows in one-shot mode)
  int M, H;
  bf16* h;                        // residual stream [M, H] (local, full); rows reduced here are updated in place
  const bf16* norm_w; const bf16* norm_b; float eps; int layernorm;   // norm_w null: no norm (plain all-reduce + residual)
  bf16* y;                        // normalised output [M, H] (local) or null
  uint8_t* yq; float* yscale; int scale_ld;   // fp8 operand of y or null
  int gather;                     // bit 0: push this rank's rows of y / yq to every peer, then wait for theirs;
                                  // bit 1: push its rows of h too; bit 2: pull mode - every rank's partial
                                  // product [M, H] sits at slots_off in its own buffer and the row owner reads
                                  // its rows from all peers (coalesced peer loads) instead of receiving pushes
  long long h_sym_off, y_sym_off, yq_sym_off, ys_sym_off;   // offsets of h / y / yq / yscale inside the symmetric buffer (gather mode: those tensors live there)
  // NVLS: multicast address of the symmetric buffer (null: plain peer loads / stores). With it, pull mode takes the
  // sum over all ranks' partial rows from the switch (one multimem.ld_reduce per 16 bytes instead of one load per
  // rank) and the gather pushes go out once (multimem.st, replicated by the switch, own copy included).
  uint8_t* mc;
  int* err;
};

__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const uint8_t* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st16(uint8_t* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               :: "l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void multimem_st8(uint8_t* mc_addr, const uint2& v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" :: "l"(mc_addr), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void multimem_st4(uint8_t* mc_addr, float v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" :: "l"(mc_addr), "f"(v) : "memory");
}

constexpr int kRnMaxVec = 4;

// grid = row_count blocks; block handles one row (up to NV * blockDim vectors of 8). NV = 1 runs 1024 threads per row
// (decode-sized batches: all of a row's peer loads are in flight at once), NV = kRnMaxVec 256 threads.
template <int NV>
__device__ __forceinline__ void reduce_norm_body(const ReduceNormParams& p) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const CommPeers& c = p.peers;
  const uint32_t epoch = begin_epoch(p.ctrs, 0);
  // gather bit 4: the GEMM that pushed the partial rows already raised this rank's flag at the peers (its last CTA,
  // after a system-wide fence): only wait for theirs
  if (!signal_and_wait(c, 0, epoch, p.err, (p.gather & 16) == 0)) return;
  const int lrow = blockIdx.x;                  // row inside this rank's slice
  if (lrow >= p.row_count) {          // a rank without rows only exchanges flags
    end_epoch(p.ctrs, 0, epoch);
    return;
  }
  const int row = p.row_begin + lrow;
  const int nvec = p.H >> 3;
  const uint8_t* base = static_cast<const uint8_t*>(c.data[c.rank]) + p.slots_off;
  float v[NV][8];
  float s = 0.f, s2 = 0.f;
  const bool in_switch = p.mc != nullptr && (p.gather & 4);
  // in-switch sums of all of this thread's vectors are requested up front: one round trip through the switch for
  // the row instead of one per vector (the requests are what keeps the links busy)
  uint4 sw[NV];
  if (in_switch) {
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < nvec)
        sw[j] = multimem_ld_reduce_bf16x8(p.mc + p.slots_off + (static_cast<size_t>(row) * p.H + static_cast<size_t>(i) * 8) * 2);
    }
  }
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < nvec) {
      float acc[8];
      if (p.h) unpack8c(reinterpret_cast<const uint4*>(p.h + static_cast<size_t>(row) * p.H)[i], acc);
      else {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      }
      // all loads first (peer loads in pull mode: one NVLink round trip, not one per rank), then a fixed summation
      // order so that every rank produces the same bits
      if (in_switch) {
        // every rank's partial row sits at the same offset of its symmetric buffer: the switch returned their sum
        // (fp32 accumulation, rounded to bf16 once)
        float f[8];
        unpack8c(sw[j], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += f[e];
      }
      uint4 pv[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < c.size && !in_switch) {
          const uint8_t* src = (p.gather & 4)
              ? static_cast<const uint8_t*>(c.data[r]) + p.slots_off + (static_cast<size_t>(row) * p.H) * 2
              : base + r * p.slot_stride + (static_cast<size_t>(lrow) * p.H) * 2;
          pv[r] = reinterpret_cast<const uint4*>(src)[i];
        }
      }
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < c.size && !in_switch) {
          float f[8];
          unpack8c(pv[r], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += f[e];
        }
      }
      const uint4 packed = pack8c(acc);
      if (p.h) reinterpret_cast<uint4*>(p.h + static_cast<size_t>(row) * p.H)[i] = packed;
      if ((p.gather & 2) && p.h && p.mc) {
        multimem_st16(p.mc + p.h_sym_off + (static_cast<size_t>(row) * p.H + static_cast<size_t>(i) * 8) * 2, packed);
      } else if ((p.gather & 2) && p.h) {
        for (int r = 0; r < c.size; ++r) {
          if (r == c.rank) continue;
          bf16* ph = reinterpret_cast<bf16*>(static_cast<uint8_t*>(c.data[r]) + p.h_sym_off);
          reinterpret_cast<uint4*>(ph + static_cast<size_t>(row) * p.H)[i] = packed;
        }
      }
      unpack8c(packed, v[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) { s += v[j][e]; s2 += v[j][e] * v[j][e]; }
    }
  }
  if (p.norm_w) {
    // block reductions
    auto block_sum = [&](float x) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
      const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
      if (l == 0) red[w] = x;
      __syncthreads();
      float t = l < nw ? red[l] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      __syncthreads();
      return t;
    };
    float mean = 0.f, rstd;
    if (p.layernorm) {
      mean = block_sum(s) / p.H;
      float var = 0.f;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nvec) {
#pragma unroll
          for (int e = 0; e < 8; ++e) { const float d = v[j][e] - mean; var += d * d; }
        }
      }
      rstd = rsqrtf(block_sum(var) / p.H + p.eps);
    } else {
      rstd = rsqrtf(block_sum(s2) / p.H + p.eps);
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      const bool on = i < nvec;
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = 0.f;
      if (on) {
        float wf[8];
        unpack8c(reinterpret_cast<const uint4*>(p.norm_w)[i], wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (v[j][e] - mean) * rstd * wf[e];
        if (p.norm_b) {
          float bfv[8];
          unpack8c(reinterpret_cast<const uint4*>(p.norm_b)[i], bfv);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += bfv[e];
        }
        const uint4 packed = pack8c(o);
        if (p.y) {
          reinterpret_cast<uint4*>(p.y + static_cast<size_t>(row) * p.H)[i] = packed;
          if ((p.gather & 1) && p.mc) {
            multimem_st16(p.mc + p.y_sym_off + (static_cast<size_t>(row) * p.H + static_cast<size_t>(i) * 8) * 2, packed);
          } else if (p.gather & 1) {
            for (int r = 0; r < c.size; ++r) {
              if (r == c.rank) continue;
              bf16* py = reinterpret_cast<bf16*>(static_cast<uint8_t*>(c.data[r]) + p.y_sym_off);
              reinterpret_cast<uint4*>(py + static_cast<size_t>(row) * p.H)[i] = packed;
            }
          }
        }
        unpack8c(packed, o);
      }
      if (p.yq) {
        float am = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) am = fmaxf(am, fabsf(o[e]));
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, off));
        const float scale = fp8_group_scale(am);
        // two neighbouring threads' eight bytes leave as one 16-byte store (local copy and peers alike); the scales
        // stay local here: a scale per row and K block is four bytes in a column of its own, and pushed one by one
        // they cost a link packet each - the finishing kernel sends this rank's slice of every scale row in one piece
        uint2 q = make_uint2(0u, 0u);
        if (on) q = pack8_e4m3c(o, 1.f / scale);
        const uint32_t nx = __shfl_down_sync(0xffffffffu, q.x, 1), ny = __shfl_down_sync(0xffffffffu, q.y, 1);
        if (on) {
          if ((i & 15) == 0) p.yscale[static_cast<size_t>(i >> 4) * p.scale_ld + row] = scale;
          if ((threadIdx.x & 1) == 0) {
            const uint4 qq = make_uint4(q.x, q.y, nx, ny);
            const size_t at = static_cast<size_t>(row) * p.H + static_cast<size_t>(i) * 8;
            *reinterpret_cast<uint4*>(p.yq + at) = qq;
            if ((p.gather & 1) && p.mc) {
              multimem_st16(p.mc + p.yq_sym_off + at, qq);
            } else if (p.gather & 1) {
              for (int r = 0; r < c.size; ++r) {
                if (r == c.rank) continue;
                *reinterpret_cast<uint4*>(static_cast<uint8_t*>(c.data[r]) + p.yq_sym_off + at) = qq;
              }
            }
          }
        }
      }
    }
  }
  // gather mode: gather_finish_kernel, next in the stream, tells the peers that this rank's slice is there
  end_epoch(p.ctrs, 0, epoch);
}

__global__ void __launch_bounds__(1024) reduce_norm_kernel_v1(const ReduceNormParams p) { reduce_norm_body<1>(p); }
__global__ void reduce_norm_kernel_v4(const ReduceNormParams p) { reduce_norm_body<kRnMaxVec>(p); }
// (Variants limited to 78 and 64 registers, three and four blocks per SM instead of two, were timed on 4 GPUs with 4096
// rows per rank: 489 and 496 us against 487 us. The requests in flight are not what limits this kernel.)

// Second half of the gather mode, stream-ordered after reduce_norm_kernel. (1) The FP8 scales of this rank's rows go
// to the peers: scale row kb holds one float per token, so this rank's slice [row_begin, row_begin + row_count) is
// contiguous and leaves as 16-byte stores (one multimem.st each with a multicast binding). (2) Once every block's
// stores are out (system-wide fence, block count in ctrs[9]), the last block raises this rank's "slice delivered"
// flag (kind 1) at every peer - the reduce kernel's pushes are covered by the same release, since that kernel has
// finished - and (3) waits, bounded, until every peer has raised its own.
__global__ void gather_finish_kernel(const CommPeers c, uint32_t* ctrs, const float* ys_local, long long ys_sym_off,
                                     uint8_t* mc, int scale_ld, int row_begin, int row_count, int nkb, int* err) {
  __shared__ int s_last;
  pdl_trigger();
  pdl_wait();
  if (ys_local != nullptr && row_count > 0) {
    for (int kb = blockIdx.x; kb < nkb; kb += gridDim.x) {
      const size_t first = static_cast<size_t>(kb) * scale_ld + row_begin;       // in floats
      const float* src = ys_local + first;
      const int head = min(row_count, static_cast<int>((4 - (first & 3)) & 3));     // floats before a 16-byte boundary
      const int nvec = (row_count - head) >> 2;
      const int tail0 = head + nvec * 4;
      auto put4 = [&](size_t elem, float v) {
        if (mc) { multimem_st4(mc + ys_sym_off + elem * 4, v); return; }
        for (int r = 0; r < c.size; ++r)
          if (r != c.rank) reinterpret_cast<float*>(static_cast<uint8_t*>(c.data[r]) + ys_sym_off)[elem] = v;
      };
      for (int t = threadIdx.x; t < head; t += blockDim.x) put4(first + t, src[t]);
      for (int t = tail0 + threadIdx.x; t < row_count; t += blockDim.x) put4(first + t, src[t]);
      for (int t = threadIdx.x; t < nvec; t += blockDim.x) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + head + static_cast<size_t>(t) * 4);
        const size_t at = (first + head + static_cast<size_t>(t) * 4) * 4;
        if (mc) { multimem_st16(mc + ys_sym_off + at, v); continue; }
        for (int r = 0; r < c.size; ++r)
          if (r != c.rank) *reinterpret_cast<uint4*>(static_cast<uint8_t*>(c.data[r]) + ys_sym_off + at) = v;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const bool last = atomicAdd(ctrs + 9, 1u) == gridDim.x - 1;
    if (last) ctrs[9] = 0;
    s_last = last ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  signal_delivered(c, ctrs, 1);
  __syncthreads();
  const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(ctrs + 1);
  signal_and_wait(c, 1, epoch, err, false);
}

// Plain barrier across ranks (bounded).
__global__ void barrier_kernel(const CommPeers c, uint32_t* ctrs, int* err) {
  const uint32_t epoch = begin_epoch(ctrs, 2);
  if (signal_and_wait(c, 2, epoch, err, true)) end_epoch(ctrs, 2, epoch);
}

// One-shot pull all-reduce of a buffer every rank holds at the same symmetric offset: out = sum_r peer_r[off..]
// (+ residual). For small tensors (router outputs, embeddings, MoE sums).
__global__ void allreduce_pull_kernel(const CommPeers c, uint32_t* ctrs, long long off, bf16* out, const bf16* residual,
                                      long long nvec, int* err) {
  const uint32_t epoch = begin_epoch(ctrs, 3);
  if (!signal_and_wait(c, 3, epoch, err, true)) return;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
    if (residual) unpack8c(reinterpret_cast<const uint4*>(residual)[i], acc);
    else {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    }
    for (int r = 0; r < c.size; ++r) {
      float f[8];
      unpack8c(reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(c.data[r]) + off)[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    reinterpret_cast<uint4*>(out)[i] = pack8c(acc);
  }
  end_epoch(ctrs, 3, epoch);
}

// All-gather along the last dimension by pulling: every rank staged its [rows, src_ld] fp32 shard at the same
// symmetric offset; out[row, r * cols + c] = shard_r[row, c] for c < cols.
__global__ void allgather_pull_kernel(const CommPeers c, uint32_t* ctrs, long long off, float* out, int rows, int cols,
                                      int src_ld, int dst_ld, int* err) {
  const uint32_t epoch = begin_epoch(ctrs, 3);
  if (!signal_and_wait(c, 3, epoch, err, true)) return;
  const long long per_rank = static_cast<long long>(rows) * cols;
  const long long total = per_rank * c.size;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / per_rank);
    const long long j = i - r * per_rank;
    const int row = static_cast<int>(j / cols), col = static_cast<int>(j % cols);
    const float* src = reinterpret_cast<const float*>(static_cast<const uint8_t*>(c.data[r]) + off);
    out[static_cast<long long>(row) * dst_ld + static_cast<long long>(r) * cols + col] = src[static_cast<long long>(row) * src_ld + col];
  }
  end_epoch(ctrs, 3, epoch);
}

static int g_spin_limit = kSpinLimit;

static CommPeers make_peers(const unsigned long long* data_ptrs, const unsigned long long* flag_ptrs, int rank, int size) {
  CommPeers c{};
  c.spin_limit = g_spin_limit;
  for (int i = 0; i < size && i < kMaxRanks; ++i) {
    c.data[i] = reinterpret_cast<void*>(data_ptrs[i]);
    c.flags[i] = reinterpret_cast<uint32_t*>(flag_ptrs[i]);
  }
  c.rank = rank;
  c.size = size;
  return c;
}

}  // namespace ksana

using namespace ksana;

// Budget of every wait on a peer's flag, in polls of about 0.1 us each (default 2^20, about a second; <= 0 restores
// the default). A wait that runs out sets the device error word to 3 and the kernel returns without touching the
// data that depended on the peer; the context stays usable. Failure-detection tests use a budget of a millisecond.
extern "C" void ksana_comm_set_spin_limit(int polls) { g_spin_limit = polls > 0 ? polls : kSpinLimit; }

// Reduce the partial slots that the peers' GEMM epilogues pushed, add the residual, normalise, optionally
// quantise and all-gather. See ReduceNormParams. Launches 1 kernel (2 in gather mode).
extern "C" int ksana_reduce_norm(const unsigned long long* data_ptrs, const unsigned long long* flag_ptrs, int rank,
                                 int size, void* ctrs, long long slots_off, long long slot_stride,
                                 int row_begin, int row_count, int M, int H, void* h, const void* norm_w,
                                 const void* norm_b, float eps, int layernorm, void* y, void* yq, float* yscale,
                                 int scale_ld, int gather, long long h_sym_off, long long y_sym_off,
                                 long long yq_sym_off, long long ys_sym_off, unsigned long long mc_base, int* err,
                                 cudaStream_t st) {
  if (size > kMaxRanks || H % 8 || H > 8 * kRnMaxVec * 1024) return -10;
  if (mc_base && ((slots_off | h_sym_off | y_sym_off | yq_sym_off | ys_sym_off) & 15)) return -12;
  if (yq && H % 128) return -11;
  ReduceNormParams p{};
  p.peers = make_peers(data_ptrs, flag_ptrs, rank, size);
  p.ctrs = static_cast<uint32_t*>(ctrs); p.slots_off = slots_off; p.slot_stride = slot_stride;
  p.row_begin = row_begin; p.row_count = row_count; p.M = M; p.H = H;
  p.h = static_cast<bf16*>(h);
  p.norm_w = static_cast<const bf16*>(norm_w); p.norm_b = static_cast<const bf16*>(norm_b);
  p.eps = eps; p.layernorm = layernorm;
  p.y = static_cast<bf16*>(y); p.yq = static_cast<uint8_t*>(yq); p.yscale = yscale; p.scale_ld = scale_ld;
  p.gather = gather; p.h_sym_off = h_sym_off; p.y_sym_off = y_sym_off; p.yq_sym_off = yq_sym_off; p.ys_sym_off = ys_sym_off;
  p.mc = reinterpret_cast<uint8_t*>(mc_base);
  p.err = err;
  // few rows (decode): one 16-byte vector per thread, so that a row's loads from all peers are in flight together;
  // many rows: up to kRnMaxVec vectors per thread
  const int per_thread = (row_count <= 64 && H <= 8192) ? 1 : kRnMaxVec;
  int threads = (((H >> 3) + per_thread - 1) / per_thread + 31) / 32 * 32;
  if (threads < 32) threads = 32;
  if (threads > 1024) threads = 1024;
  // a rank with no rows still takes part in the flag exchange
  const dim3 grid(row_count > 0 ? row_count : 1);
  const cudaError_t e = per_thread == 1 ? launch_pdl(reduce_norm_kernel_v1, grid, dim3(threads), 0, st, p)
                                        : launch_pdl(reduce_norm_kernel_v4, grid, dim3(threads), 0, st, p);
  if (e != cudaSuccess) return -4;
  if (gather & 1) {
    const int nkb = yq ? H / 128 : 0;
    if (launch_pdl(gather_finish_kernel, dim3(nkb > 0 ? (nkb < 64 ? nkb : 64) : 1), dim3(256), 0, st, p.peers, p.ctrs,
                   static_cast<const float*>(yq ? yscale : nullptr), ys_sym_off, p.mc, scale_ld, row_begin, row_count,
                   nkb, err) != cudaSuccess) return -5;
  }
  return 0;
}
// The same all-reduce with the sum taken inside the NVSwitch (NVLS): `mc` is the multicast address of the symmetric
// buffer (every rank's copy of the staged tensor bound to one address); one multimem.ld_reduce returns the sum over
// all ranks' copies, so a rank receives n bytes instead of size x n. Summation order is the switch's, the result is
// rounded to bf16 once before the residual is added.
__global__ void allreduce_nvls_kernel(const CommPeers c, uint32_t* ctrs, const uint8_t* mc, long long off, bf16* out,
                                      const bf16* residual, long long nvec, int* err) {
  const uint32_t epoch = begin_epoch(ctrs, 3);
  if (!signal_and_wait(c, 3, epoch, err, true)) return;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc + off + i * 16)
                 : "memory");
    if (residual) {
      float a[8], b[8];
      unpack8c(v, a);
      unpack8c(reinterpret_cast<const uint4*>(residual)[i], b);
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] += b[e];
      v = pack8c(a);
    }
    reinterpret_cast<uint4*>(out)[i] = v;
  }
  end_epoch(ctrs, 3, epoch);
}


extern "C" int ksana_comm_barrier(const unsigned long long* data_ptrs, const unsigned long long* flag_ptrs, int rank,
                                  int size, void* ctrs, int* err, cudaStream_t st) {
  barrier_kernel<<<1, 32, 0, st>>>(make_peers(data_ptrs, flag_ptrs, rank, size), static_cast<uint32_t*>(ctrs), err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_allreduce_pull(const unsigned long long* data_ptrs, const unsigned long long* flag_ptrs, int rank,
                                    int size, void* ctrs, long long off, void* out, const void* residual,
                                    long long n_elems, int* err, cudaStream_t st) {
  if (n_elems % 8) return -10;
  const long long nvec = n_elems / 8;
  long long g = (nvec + 255) / 256;
  if (g > 148 * 4) g = 148 * 4;
  if (g < 1) g = 1;
  allreduce_pull_kernel<<<static_cast<int>(g), 256, 0, st>>>(make_peers(data_ptrs, flag_ptrs, rank, size),
                                                             static_cast<uint32_t*>(ctrs), off,
                                                             static_cast<bf16*>(out),
                                                             static_cast<const bf16*>(residual), nvec, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_allgather_pull(const unsigned long long* data_ptrs, const unsigned long long* flag_ptrs, int rank,
                                    int size, void* ctrs, long long off, float* out, int rows, int cols, int src_ld,
                                    int dst_ld, int* err, cudaStream_t st) {
  const long long total = static_cast<long long>(rows) * cols * size;
  long long g = (total + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  if (g < 1) g = 1;
  allgather_pull_kernel<<<static_cast<int>(g), 256, 0, st>>>(make_peers(data_ptrs, flag_ptrs, rank, size),
                                                             static_cast<uint32_t*>(ctrs), off, out, rows, cols,
                                                             src_ld, dst_ld, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// mc_base: multicast address of the symmetric buffer (0: not available -> -10).
extern "C" int ksana_allreduce_nvls(const unsigned long long* data_ptrs, const unsigned long long* flag_ptrs, int rank,
                                    int size, void* ctrs, unsigned long long mc_base, long long off, void* out,
                                    const void* residual, long long n_elems, int* err, cudaStream_t st) {
  if (n_elems % 8 || mc_base == 0 || (off & 15)) return -10;
  const long long nvec = n_elems / 8;
  long long g = (nvec + 255) / 256;
  if (g > 148 * 4) g = 148 * 4;
  if (g < 1) g = 1;
  allreduce_nvls_kernel<<<static_cast<int>(g), 256, 0, st>>>(make_peers(data_ptrs, flag_ptrs, rank, size),
                                                             static_cast<uint32_t*>(ctrs),
                                                             reinterpret_cast<const uint8_t*>(mc_base), off,
                                                             static_cast<bf16*>(out),
                                                             static_cast<const bf16*>(residual), nvec, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
