// Top-k sampling of the next token on the device: the reference's selectTopK -> cpuSoftmax ->
// sampleFromDistribution chain (globals.js:47-74, called at model.js:81-83) without reading the logits back.
// The reference draws Math.random() inside sampleFromDistribution; here the caller supplies one uniform
// number per (step, sequence), so a run is reproducible and can be compared token for token with a CPU run
// that uses the same numbers.
//
// One CTA of 1024 threads per sequence:
//   1. every thread folds its strided share of the logits into one 64-bit key (order-preserving float bits in
//      the high word, ~index in the low word, so larger key = earlier in the reference's stable descending sort);
//   2. a bitonic sort of the 1024 per-thread maxima gives tau, the top_k-th largest of them: a lower bound of
//      the true top_k-th key, reached by exactly top_k threads;
//   3. those threads rescan their share and append every key >= tau to a candidate list
//      (at most top_k * ceil(V / 1024) entries); a rank sort of the candidates yields the top_k keys in order;
//   4. exp((v - max) / temperature) in double precision, a left-to-right sum and running sum as in the
//      reference, and the first index whose running sum exceeds the uniform number is the pick.
// The kernel then writes the token and advances the session like argmax_kernel.
#pragma once
#include "common.cuh"

namespace wgpt {

constexpr int kSampleThreads = 1024;
constexpr int kMaxTopK = 128;

__device__ __forceinline__ unsigned long long sample_key(float v, int idx) {
  uint32_t u = __float_as_uint(v);
  if (u == 0x80000000u) u = 0u;  // -0 and +0 compare equal in the reference's sort
  uint32_t k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)k << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)idx);
}

__device__ __forceinline__ int sample_key_index(unsigned long long c) {
  return (int)(0xFFFFFFFFu - (uint32_t)(c & 0xFFFFFFFFull));
}

// Dynamic shared memory: (1024 + cap) 64-bit keys, cap = top_k * ceil(V / 1024).
// uniforms: [steps][gridDim.x] doubles in [0,1), indexed by the session's step counter.
// done_counter must be zero on entry and is left zero.
__global__ void __launch_bounds__(kSampleThreads)
sample_topk_kernel(const float *__restrict__ logits, int V, int top_k, double temperature,
                   const double *__restrict__ uniforms, int cap, uint32_t *__restrict__ next_ids,
                   uint32_t *__restrict__ out_ids, int out_stride, int *__restrict__ pos, int *__restrict__ step,
                   int n_tok, unsigned int *__restrict__ done_counter) {
  extern __shared__ __align__(16) unsigned long long skeys[];
  unsigned long long *srt = skeys;
  unsigned long long *cand = skeys + kSampleThreads;
  __shared__ unsigned long long top[kMaxTopK];
  __shared__ double ev[kMaxTopK];
  __shared__ double s_sum;
  __shared__ int s_cnt;
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, tid = threadIdx.x;
  const int my_step = __ldcg(step);
  const float *x = logits + (size_t)seq * V;

  unsigned long long best = 0ull;  // below every real key (their low word is never zero for idx < 2^32 - 1)
  {
    int i = tid;  // 16 loads in flight per thread: one CTA scans the row, so latency is what bounds it
    for (; i + 15 * kSampleThreads < V; i += 16 * kSampleThreads) {
      float f[16];
#pragma unroll
      for (int u = 0; u < 16; u++) f[u] = __ldcg(x + i + u * kSampleThreads);
#pragma unroll
      for (int u = 0; u < 16; u++) {
        unsigned long long c = sample_key(f[u], i + u * kSampleThreads);
        best = c > best ? c : best;
      }
    }
    for (; i + 3 * kSampleThreads < V; i += 4 * kSampleThreads) {
      float f[4];
#pragma unroll
      for (int u = 0; u < 4; u++) f[u] = __ldcg(x + i + u * kSampleThreads);
#pragma unroll
      for (int u = 0; u < 4; u++) {
        unsigned long long c = sample_key(f[u], i + u * kSampleThreads);
        best = c > best ? c : best;
      }
    }
    for (; i < V; i += kSampleThreads) {
      unsigned long long c = sample_key(__ldcg(x + i), i);
      best = c > best ? c : best;
    }
  }
  srt[tid] = best;
  if (tid == 0) s_cnt = 0;
  __syncthreads();
  // bitonic sort, descending
  for (int k2 = 2; k2 <= kSampleThreads; k2 <<= 1) {
    for (int j = k2 >> 1; j > 0; j >>= 1) {
      int other = tid ^ j;
      if (other > tid) {
        unsigned long long a = srt[tid], b = srt[other];
        bool desc = (tid & k2) == 0;
        if (desc ? (a < b) : (a > b)) { srt[tid] = b; srt[other] = a; }
      }
      __syncthreads();
    }
  }
  const unsigned long long tau = srt[top_k - 1];
  if (best >= tau && best != 0ull) {  // at most top_k threads: their share again, 16 loads at a time
    int i = tid;
    for (; i + 15 * kSampleThreads < V; i += 16 * kSampleThreads) {
      float f[16];
#pragma unroll
      for (int u = 0; u < 16; u++) f[u] = __ldcg(x + i + u * kSampleThreads);
#pragma unroll
      for (int u = 0; u < 16; u++) {
        unsigned long long c = sample_key(f[u], i + u * kSampleThreads);
        if (c >= tau) {
          int slot = atomicAdd(&s_cnt, 1);
          if (slot < cap) cand[slot] = c;
        }
      }
    }
    for (; i < V; i += kSampleThreads) {
      unsigned long long c = sample_key(__ldcg(x + i), i);
      if (c >= tau) {
        int slot = atomicAdd(&s_cnt, 1);
        if (slot < cap) cand[slot] = c;
      }
    }
  }
  __syncthreads();
  const int C = s_cnt < cap ? s_cnt : cap;
  for (int i = tid; i < C; i += kSampleThreads) {
    unsigned long long ci = cand[i];
    int rank = 0;
    for (int j = 0; j < C; j++) rank += cand[j] > ci ? 1 : 0;
    if (rank < top_k) top[rank] = ci;
  }
  __syncthreads();
  // softmax over the kept logits in double precision (JS numbers), globals.js:59-64
  const double vmax = (double)__ldcg(x + sample_key_index(top[0]));
  if (tid < top_k) ev[tid] = exp(((double)__ldcg(x + sample_key_index(top[tid])) - vmax) / temperature);
  __syncthreads();
  if (tid == 0) {
    double s = 0.0;
    for (int j = 0; j < top_k; j++) s += ev[j];
    s_sum = s;
  }
  __syncthreads();
  if (tid < top_k) ev[tid] = ev[tid] / s_sum;
  __syncthreads();
  if (tid == 0) {
    const double u = __ldcg(uniforms + (size_t)my_step * gridDim.x + seq);
    int pick = top_k - 1;
    double cum = 0.0;
    for (int j = 0; j < top_k; j++) {
      cum += ev[j];
      if (u < cum) { pick = j; break; }
    }
    uint32_t id = (uint32_t)sample_key_index(top[pick]);
    next_ids[seq] = id;
    if (out_ids) out_ids[(size_t)seq * out_stride + my_step] = id;
    __threadfence();
    unsigned int prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *pos = __ldcg(pos) + n_tok;
      *step = my_step + 1;
      *done_counter = 0u;
    }
  }
}

}  // namespace wgpt
