// Fused sampler for sm_100a: one CTA per request row does, in one launch,
//   temperature -> top-k (k <= 1024, exact radix select over the vocabulary)
//   -> top-p -> multinomial draw (counter-based Philox, no RNG state arrays)
//   -> optional top-N log-probabilities,
// with an argmax fast path when the row is greedy and wants no log-probs.
// Penalty / banning kernels edit the fp32 logits in place beforehand.
//
// Semantics follow the reference sampler (src/ksana_llm/samplers/sampler.cpp:82-400,
// src/ksana_llm/samplers/topk/topk_sampling.cpp:55-110): repetition penalty multiplies the
// logits of seen tokens by 1/penalty; top-N log-probs are a log-softmax over the N largest
// temperature-scaled logits only; top-k rows with k == 1 are greedy.
// Replaces 3rdparty/LLM_kernels/csrc/kernels/nvidia/samplers/{greedy.cu:23-56,
// samplingTopKKernels.cu:55-300, decodingCommon.cu:95-207, repetition_penalty.cu:19}.
#include <cuda_runtime.h>
#include <stdint.h>
#include "pdl.cuh"

namespace ksana {

constexpr int kSampThreads = 1024;
constexpr int kMaxK = 1024;

__device__ __forceinline__ uint32_t f2ord(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Philox4x32-10 keyed by (seed), counter (row, step): one uniform in [0,1).
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint32_t row, uint32_t step) {
  uint32_t c0 = row, c1 = step, c2 = 0x9E3779B9u, c3 = 0xBB67AE85u;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n1 = static_cast<uint32_t>(p1);
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
    const uint32_t n3 = static_cast<uint32_t>(p0);
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return (c0 >> 8) * (1.0f / 16777216.0f);
}

struct SampleParams {
  const float* logits; long long ld;   // [rows][ld]
  const int* row_idx;                  // logits row of request b (null: b)
  const float* temperature;            // [B]
  const int* top_k;                    // [B]
  const float* top_p;                  // [B]
  const unsigned long long* seeds;     // [B]
  const int* steps;                    // [B] per-request draw counter
  int* out_tokens;                     // [B]
  int num_logprobs;                    // N (0 = none), same for the launch
  int* lp_ids; float* lp_vals;         // [B][N]
  int vocab;
  // Vocabulary-sharded sampling (tensor parallel). Candidate mode (cand_val != null): nothing is drawn; the row's
  // cand_k largest logits (sorted: value descending, index ascending) are written to cand_val / cand_idx
  // [B][cand_k] with idx_offset added to the indices (this shard's first token id); short rows are padded with
  // -inf. Merge mode (col_ids != null): `logits` rows are candidate lists gathered from all shards and
  // col_ids [rows][col_ld] holds the token id of every column; drawn tokens and log-prob ids are mapped through it.
  float* cand_val; int* cand_idx; int cand_k; int idx_offset;
  const int* col_ids; long long col_ld;
};

__global__ void __launch_bounds__(kSampThreads)
sample_kernel(const SampleParams p) {
  __shared__ uint32_t hist[256];
  __shared__ float cand_val[kMaxK];
  __shared__ int cand_idx[kMaxK];
  __shared__ float red_val[32];
  __shared__ int red_idx[32];
  __shared__ uint32_t sh_prefix, sh_remaining, sh_count, sh_ties;

  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  const long long src_row = p.row_idx ? p.row_idx[b] : b;
  const float* row = p.logits + src_row * p.ld;
  const int* ids = p.col_ids ? p.col_ids + src_row * p.col_ld : nullptr;
  const int V = p.vocab;
  const bool cand_mode = p.cand_val != nullptr;
  const int k_req = cand_mode ? max(1, min(p.cand_k, kMaxK)) : max(1, min(p.top_k[b], kMaxK));
  const int N = cand_mode ? 0 : p.num_logprobs;
  const int tid = threadIdx.x;

  if (k_req == 1 && N == 0) {
    // ---- greedy: (max value, lowest index)
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = tid; i < V; i += kSampThreads) {
      const float v = row[i];
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { red_val[tid >> 5] = bv; red_idx[tid >> 5] = bi; }
    __syncthreads();
    if (tid < 32) {
      bv = red_val[tid]; bi = red_idx[tid];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (tid == 0) {
        if (cand_mode) {
          p.cand_val[b] = bv;
          p.cand_idx[b] = bi == 0x7fffffff ? 0x7fffffff : bi + p.idx_offset;
        } else {
          const int pick = bi == 0x7fffffff ? 0 : bi;
          p.out_tokens[b] = ids ? ids[pick] : pick;
        }
      }
    }
    return;
  }

  // ---- exact K-th largest by 4-pass radix select on order-preserving keys
  const int K = min(V, max(k_req, N));
  if (tid == 0) { sh_prefix = 0; sh_remaining = K; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = sh_prefix;
    const uint32_t mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < V; i += kSampThreads) {
      const uint32_t key = f2ord(row[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t rem = sh_remaining;
      int bin = 255;
      for (; bin > 0; --bin) {
        if (hist[bin] >= rem) break;
        rem -= hist[bin];
      }
      sh_prefix = prefix | (static_cast<uint32_t>(bin) << shift);
      sh_remaining = rem;   // how many elements equal to the final key still belong to the top K
    }
    __syncthreads();
  }
  const uint32_t kth = sh_prefix;
  const uint32_t ties_allowed = sh_remaining;
  if (tid == 0) { sh_count = 0; sh_ties = 0; }
  for (int i = tid; i < kMaxK; i += kSampThreads) { cand_val[i] = -INFINITY; cand_idx[i] = 0x7fffffff; }
  __syncthreads();
  for (int i = tid; i < V; i += kSampThreads) {
    const float v = row[i];
    const uint32_t key = f2ord(v);
    bool take = key > kth;
    if (key == kth) take = atomicAdd(&sh_ties, 1u) < ties_allowed;
    if (take) {
      const uint32_t slot = atomicAdd(&sh_count, 1u);
      if (slot < kMaxK) { cand_val[slot] = v; cand_idx[slot] = i; }
    }
  }
  __syncthreads();
  // ---- bitonic sort, descending by value then ascending by index (1024 slots, one per thread)
  for (int size = 2; size <= kMaxK; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int partner = tid ^ stride;
      if (partner > tid) {
        const bool desc = (tid & size) == 0;
        const float a = cand_val[tid], c = cand_val[partner];
        const int ai = cand_idx[tid], ci = cand_idx[partner];
        const bool a_first = a > c || (a == c && ai < ci);
        if (desc ? !a_first : a_first) {
          cand_val[tid] = c; cand_val[partner] = a;
          cand_idx[tid] = ci; cand_idx[partner] = ai;
        }
      }
      __syncthreads();
    }
  }
  if (cand_mode) {
    for (int i = tid; i < p.cand_k; i += kSampThreads) {
      const bool has = i < K && cand_idx[i] != 0x7fffffff;
      p.cand_val[static_cast<long long>(b) * p.cand_k + i] = has ? cand_val[i] : -INFINITY;
      p.cand_idx[static_cast<long long>(b) * p.cand_k + i] = has ? cand_idx[i] + p.idx_offset : 0x7fffffff;
    }
    return;
  }
  const float temp = p.temperature[b] > 0.f ? p.temperature[b] : 1.f;
  const float inv_t = 1.f / temp;

  if (N > 0 && tid == 0) {
    // log-softmax over the N largest temperature-scaled logits
    const int n = min(N, K);
    const float mx = cand_val[0] * inv_t;
    float sum = 0.f;
    for (int i = 0; i < n; ++i) sum += __expf(cand_val[i] * inv_t - mx);
    const float lse = mx + __logf(sum);
    for (int i = 0; i < N; ++i) {
      p.lp_ids[static_cast<long long>(b) * N + i] = i < n ? (ids ? ids[cand_idx[i]] : cand_idx[i]) : -1;
      p.lp_vals[static_cast<long long>(b) * N + i] = i < n ? cand_val[i] * inv_t - lse : -INFINITY;
    }
  }
  if (tid == 0) {
    const int k = min(k_req, K);
    int choice = cand_idx[0];
    if (k > 1) {
      const float mx = cand_val[0] * inv_t;
      float total = 0.f;
      for (int i = 0; i < k; ++i) total += __expf(cand_val[i] * inv_t - mx);
      const float top_p = (p.top_p[b] > 0.f && p.top_p[b] < 1.f) ? p.top_p[b] : 1.f;
      // nucleus: shortest prefix whose mass reaches top_p
      float mass = 0.f; int keep = k;
      if (top_p < 1.f) {
        for (int i = 0; i < k; ++i) {
          mass += __expf(cand_val[i] * inv_t - mx);
          if (mass >= top_p * total) { keep = i + 1; break; }
        }
      } else {
        mass = total;
      }
      const float u = philox_uniform(p.seeds[b], static_cast<uint32_t>(b), static_cast<uint32_t>(p.steps[b])) * mass;
      float acc = 0.f;
      choice = cand_idx[keep - 1];
      for (int i = 0; i < keep; ++i) {
        acc += __expf(cand_val[i] * inv_t - mx);
        if (u < acc) { choice = cand_idx[i]; break; }
      }
    }
    p.out_tokens[b] = ids ? ids[choice] : choice;
  }
}

// logits[row, id] *= 1/penalty for every id in that row's token list (CSR: offsets[B+1], ids[]).
__global__ void repetition_penalty_kernel(float* logits, long long ld, const int* row_idx, const int* offsets,
                                          const int* ids, const float* penalty, int vocab) {
  const int b = blockIdx.x;
  const float pen = penalty[b];
  if (pen == 1.f) return;
  float* row = logits + static_cast<long long>(row_idx ? row_idx[b] : b) * ld;
  // the host passes each distinct id once per row (a repeated id would be penalised twice)
  for (int i = offsets[b] + threadIdx.x; i < offsets[b + 1]; i += blockDim.x) {
    const int id = ids[i];
    if (id >= 0 && id < vocab) row[id] *= 1.f / pen;
  }
}

// logits[row, id] = -inf for banned ids (CSR per row): no-repeat-ngram / encoder-no-repeat-ngram / FSM masks.
__global__ void ban_tokens_kernel(float* logits, long long ld, const int* row_idx, const int* offsets, const int* ids,
                                  int vocab) {
  const int b = blockIdx.x;
  float* row = logits + static_cast<long long>(row_idx ? row_idx[b] : b) * ld;
  for (int i = offsets[b] + threadIdx.x; i < offsets[b + 1]; i += blockDim.x) {
    const int id = ids[i];
    if (id >= 0 && id < vocab) row[id] = -INFINITY;
  }
}

}  // namespace ksana

using namespace ksana;

extern "C" int ksana_sample(const float* logits, long long ld, const int* row_idx, const float* temperature,
                            const int* top_k, const float* top_p, const unsigned long long* seeds, const int* steps,
                            int* out_tokens, int num_logprobs, int* lp_ids, float* lp_vals, int B, int vocab,
                            cudaStream_t st) {
  if (B <= 0) return 0;
  if (num_logprobs > kMaxK) return -10;
  SampleParams p{logits, ld, row_idx, temperature, top_k, top_p, seeds, steps, out_tokens, num_logprobs, lp_ids,
                 lp_vals, vocab, nullptr, nullptr, 0, 0, nullptr, 0};
  return launch_pdl(sample_kernel, dim3(B), dim3(kSampThreads), 0, st, p) == cudaSuccess ? 0 : -4;
}

// Sampling over candidate lists gathered from the vocabulary shards: logits [rows][ld] holds `ncols` candidate
// values per row and col_ids [rows][col_ld] their token ids; everything else as ksana_sample.
extern "C" int ksana_sample_merged(const float* logits, long long ld, const int* col_ids, long long col_ld,
                                   const int* row_idx, const float* temperature, const int* top_k, const float* top_p,
                                   const unsigned long long* seeds, const int* steps, int* out_tokens, int num_logprobs,
                                   int* lp_ids, float* lp_vals, int B, int ncols, cudaStream_t st) {
  if (B <= 0) return 0;
  if (num_logprobs > kMaxK || !col_ids) return -10;
  SampleParams p{logits, ld, row_idx, temperature, top_k, top_p, seeds, steps, out_tokens, num_logprobs, lp_ids,
                 lp_vals, ncols, nullptr, nullptr, 0, 0, col_ids, col_ld};
  return launch_pdl(sample_kernel, dim3(B), dim3(kSampThreads), 0, st, p) == cudaSuccess ? 0 : -4;
}

// This shard's k largest logits per row (value descending, index ascending) with their token ids
// (column + idx_offset): cand_val / cand_idx [B][k]. k <= 1024.
extern "C" int ksana_shard_topk(const float* logits, long long ld, const int* row_idx, int B, int vocab, int k,
                                int idx_offset, float* cand_val, int* cand_idx, cudaStream_t st) {
  if (B <= 0) return 0;
  if (k < 1 || k > kMaxK || !cand_val || !cand_idx) return -10;
  SampleParams p{logits, ld, row_idx, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, vocab,
                 cand_val, cand_idx, k, idx_offset, nullptr, 0};
  return launch_pdl(sample_kernel, dim3(B), dim3(kSampThreads), 0, st, p) == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_repetition_penalty(float* logits, long long ld, const int* row_idx, const int* offsets,
                                        const int* ids, const float* penalty, int B, int vocab, cudaStream_t st) {
  if (B <= 0) return 0;
  repetition_penalty_kernel<<<B, 256, 0, st>>>(logits, ld, row_idx, offsets, ids, penalty, vocab);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int ksana_ban_tokens(float* logits, long long ld, const int* row_idx, const int* offsets, const int* ids,
                                int B, int vocab, cudaStream_t st) {
  if (B <= 0) return 0;
  ban_tokens_kernel<<<B, 256, 0, st>>>(logits, ld, row_idx, offsets, ids, vocab);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
