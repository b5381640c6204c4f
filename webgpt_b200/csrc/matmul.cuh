// FP32 matrix products on the CUDA cores.
//  - gemv_nk_kernel : up to 8 activation rows against a weight stored [N,K] (K contiguous). One warp per
//                     output column (group), 128-bit streaming loads, warp-shuffle reduction, optional fused
//                     LayerNorm on the input rows, fused bias/GELU/residual/KV-scatter on the way out.
//                     HBM-bound: bytes = 4*N*K per launch.
//  - gemv_kn_*      : the same product for a weight in the reference's [K,N] layout (fastMatMul,
//                     instructions.js:179-319), split along K across CTAs with a deterministic two-stage sum.
//  - gemm_simt_kernel: general M; 64x64x16 tiles, 4x4 register tile per thread. The FP32 reference mode for
//                     the tensor-core path and the executor of the per-operator API.
#pragma once
#include "attention.cuh"
#include "common.cuh"

namespace wgpt {

// ------------------------------------------------------------------------------------------------
// Optional tail of gemv_nk_kernel for the de-embedding: greedy pick fused into the producing kernel.
// Every CTA reduces its columns to one (value, index) candidate per row; the last CTA to finish reduces the
// candidates (lowest index wins ties, globals.js:66-74 with top_k = 1), writes the next input id and the output
// list entry, and advances the session's position and step counters. pval == nullptr disables it.
struct GreedyPick {
  float *pval;            // [M][gridDim.x] candidates
  int *pidx;
  unsigned int *counter;  // zero on entry, left zero
  uint32_t *next_ids;     // [M]
  uint32_t *out_ids;      // [M][out_stride] or nullptr
  int out_stride;
  int *pos, *step;
  int n_tok;
  // gemv_loop_kernel only: one 64-bit (value, index) key per row, zero on entry and left zero, and a weight block
  // the kernel asks for in L2 when its own work is done (the next kernel's; may be null)
  unsigned long long *keys;
  const char *next_w;
  unsigned int next_w_bytes;
};

// Second half of the greedy pick: thread m < M of every CTA brings the CTA's best (value, index) of row m; the
// last CTA to arrive reduces the candidates of all CTAs (lowest index wins ties), writes the next input id and the
// output list entry, and advances the position and step counters. All 256 threads of the CTA must call it.
template <int M>
__device__ __forceinline__ void greedy_pick_finish(const GreedyPick &gp, float bv, int bn) {
  __shared__ float fin_v[8];
  __shared__ int fin_n[8];
  __shared__ unsigned int is_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < M) {
    gp.pval[(size_t)tid * gridDim.x + blockIdx.x] = bv;
    gp.pidx[(size_t)tid * gridDim.x + blockIdx.x] = bn;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = (atomicAdd(gp.counter, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int my_step = __ldcg(gp.step);
  for (int m = 0; m < M; m++) {
    bv = -INFINITY;
    bn = 0x7fffffff;
    for (int j = tid; j < (int)gridDim.x; j += 256) {
      float v = __ldcg(gp.pval + (size_t)m * gridDim.x + j);
      int n = __ldcg(gp.pidx + (size_t)m * gridDim.x + j);
      if (v > bv || (v == bv && n < bn)) { bv = v; bn = n; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int on = __shfl_xor_sync(0xffffffffu, bn, o);
      if (ov > bv || (ov == bv && on < bn)) { bv = ov; bn = on; }
    }
    __syncthreads();  // fin_* are re-used from one row to the next
    if (lane == 0) { fin_v[warp] = bv; fin_n[warp] = bn; }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < 8; w++)
        if (fin_v[w] > bv || (fin_v[w] == bv && fin_n[w] < bn)) { bv = fin_v[w]; bn = fin_n[w]; }
      if (bn == 0x7fffffff) bn = 0;  // a row of NaNs compares false everywhere: report index 0
      gp.next_ids[m] = (uint32_t)bn;
      if (gp.out_ids) gp.out_ids[(size_t)m * gp.out_stride + my_step] = (uint32_t)bn;
    }
  }
  if (tid == 0) {
    *gp.pos = __ldcg(gp.pos) + gp.n_tok;
    *gp.step = my_step + 1;
    *gp.counter = 0u;
  }
}

// x: [M, K] rows at stride ldx; Wt: [N, K]. CTA = 8 warps = (8/WK) column groups x WK slices of K.
// Each warp accumulates CPW columns over its K slice for all M rows.
// Order of work: (1) allow the next kernel to launch and put this warp's first weights in flight (weights are
// written by no kernel, so this may run while the previous kernel is still executing); (2) wait for the previous
// kernel; (3) all threads stage the M input rows in shared memory, one warp per row applies the LayerNorm
// (instructions.js:451-550); (4) multiply; (5) fixed-order sum of the K slices, epilogue, optional greedy pick.
// Dynamic shared memory: M*K floats + 8*CPW*M partial sums.
template <int M, int WK, int CPW>
__global__ void __launch_bounds__(256)
gemv_nk_kernel(const float *__restrict__ x, size_t ldx, const float *__restrict__ gamma,
               const float *__restrict__ beta, const float *__restrict__ Wt, int K, int N, Epilogue epi,
               int prefetch, GreedyPick gp) {
  extern __shared__ __align__(128) float smem[];
  float *xs = smem;
  float *red = smem + (size_t)M * K;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K4 = K >> 2;
  constexpr int WC = 8 / WK;
  constexpr int PRE = CPW == 1 ? 8 : (CPW == 2 ? 4 : 2);  // float4 per lane and column in flight before the wait
  const int wc = warp / WK, wk = warp % WK;
  const int col0 = (blockIdx.x * WC + wc) * CPW;
  const int beg = (int)(((long long)K4 * wk) / WK), end = (int)(((long long)K4 * (wk + 1)) / WK);
  const float4 *w4[CPW];
#pragma unroll
  for (int c = 0; c < CPW; c++) {
    int col = col0 + c < N ? col0 + c : N - 1;  // clamp: out-of-range columns read a valid row, never stored
    w4[c] = reinterpret_cast<const float4 *>(Wt + (size_t)col * K);
  }

  // (1)
  TRACE_BEGIN(1);
  trace(1, 0);
  pdl_launch_dependents();
  float4 wpre[CPW][PRE];
#pragma unroll
  for (int j = 0; j < PRE; j++) {
    const int i = beg + lane + 32 * j;
#pragma unroll
    for (int c = 0; c < CPW; c++)
      wpre[c][j] = i < end ? ldg_stream4(w4[c] + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (prefetch && lane == 0 && end > beg + 32 * PRE) {
#pragma unroll
    for (int c = 0; c < CPW; c++) prefetch_l2(w4[c] + beg + 32 * PRE, (uint32_t)(end - beg - 32 * PRE) * 16u);
  }
  // (2)
  pdl_wait();
  trace(1, 1);

  // (3)
  {
    float4 *xs4w = reinterpret_cast<float4 *>(xs);
    const size_t ldx4 = ldx >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    for (int idx = tid; idx < M * K4; idx += 256) {
      int m = idx / K4, i = idx - m * K4;
      xs4w[idx] = __ldcg(x4 + (size_t)m * ldx4 + i);
    }
  }
  __syncthreads();
  if (gamma != nullptr) {
    for (int m = warp; m < M; m += 8) {
      float4 *row = reinterpret_cast<float4 *>(xs + (size_t)m * K);
      float s = 0.f;
      for (int i = lane; i < K4; i += 32) {
        float4 v = row[i];
        s += (v.x + v.y) + (v.z + v.w);
      }
      float mean = warp_sum(s) / (float)K;
      float q = 0.f;
      for (int i = lane; i < K4; i += 32) {
        float4 v = row[i];
        float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
        q += (a * a + b * b) + (c * c + d * d);
      }
      float sd = sqrtf(warp_sum(q) / (float)K + 1e-5f);
      const float4 *g4 = reinterpret_cast<const float4 *>(gamma);
      const float4 *b4 = reinterpret_cast<const float4 *>(beta);
      for (int i = lane; i < K4; i += 32) {
        float4 v = row[i], g = g4[i], b = b4[i];
        row[i] = make_float4(g.x * ((v.x - mean) / sd) + b.x, g.y * ((v.y - mean) / sd) + b.y,
                             g.z * ((v.z - mean) / sd) + b.z, g.w * ((v.w - mean) / sd) + b.w);
      }
    }
    __syncthreads();
  }

  trace(1, 2);
  // (4)
  float acc[CPW][M];
#pragma unroll
  for (int c = 0; c < CPW; c++)
#pragma unroll
    for (int m = 0; m < M; m++) acc[c][m] = 0.f;
  const float4 *xs4 = reinterpret_cast<const float4 *>(xs);
#pragma unroll
  for (int j = 0; j < PRE; j++) {
    const int i = beg + lane + 32 * j;
    if (i < end) {
#pragma unroll
      for (int m = 0; m < M; m++) {
        float4 xv = xs4[(size_t)m * K4 + i];
#pragma unroll
        for (int c = 0; c < CPW; c++) acc[c][m] += dot4(wpre[c][j], xv);
      }
    }
  }
#pragma unroll 4
  for (int i = beg + lane + 32 * PRE; i < end; i += 32) {
    float4 w[CPW];
#pragma unroll
    for (int c = 0; c < CPW; c++) w[c] = ldg_stream4(w4[c] + i);
#pragma unroll
    for (int m = 0; m < M; m++) {
      float4 xv = xs4[(size_t)m * K4 + i];
#pragma unroll
      for (int c = 0; c < CPW; c++) acc[c][m] += dot4(w[c], xv);
    }
  }
#pragma unroll
  for (int c = 0; c < CPW; c++)
#pragma unroll
    for (int m = 0; m < M; m++) {
      float v = warp_sum(acc[c][m]);
      if (lane == 0) red[((wc * WK + wk) * CPW + c) * M + m] = v;
    }
  __syncthreads();
  // (5) sum the K slices in a fixed order, apply the epilogue
  float outv = -INFINITY;
  int outn = 0x7fffffff;
  if (tid < WC * CPW * M) {
    int m = tid % M, c = (tid / M) % CPW, g = tid / (M * CPW);
    int n = (blockIdx.x * WC + g) * CPW + c;
    if (n < N) {
      float v = 0.f;
#pragma unroll
      for (int k = 0; k < WK; k++) v += red[((g * WK + k) * CPW + c) * M + m];
      v = epi_apply(epi, v, m, n);
      *epi_addr(epi, m, n) = v;
      outv = v;
      outn = n;
    }
  }
  trace(1, 3);
  if (gp.pval == nullptr) return;

  // ---- greedy pick ----
  constexpr int NC = WC * CPW * M;
  __shared__ float cand_v[NC];
  __shared__ int cand_n[NC];
  if (tid < NC) { cand_v[tid] = outv; cand_n[tid] = outn; }
  __syncthreads();
  float bv = -INFINITY;
  int bn = 0x7fffffff;
  if (tid < M) {  // candidates of row m sit at tid + M*j; columns ascend with j, so ">" keeps the lowest index
    for (int j = 0; j < WC * CPW; j++) {
      float v = cand_v[tid + M * j];
      int n = cand_n[tid + M * j];
      if (v > bv || (v == bv && n < bn)) { bv = v; bn = n; }
    }
  }
  greedy_pick_finish<M>(gp, bv, bn);
}

// ------------------------------------------------------------------------------------------------
// gemv_loop_kernel: the product of gemv_nk_kernel for a matrix larger than L2 (the tied de-embedding,
// model.js:224-229: 50257 x n_embd floats per token). A few CTAs per SM stay resident and every warp walks a
// contiguous range of columns, CPW at a time, so the input rows are staged and normalised once per CTA instead of
// once per 32 columns, and the warps never meet at a barrier inside the loop: their loads stay spread over time and
// the stream has no per-CTA start and tail. Optional greedy pick as in gemv_nk_kernel.
// Dynamic shared memory: M*K floats. HBM-bound: bytes = 4*N*K per launch.
template <int M, int CPW>
__global__ void __maxnreg__(96)
gemv_loop_kernel(const float *__restrict__ x, size_t ldx, const float *__restrict__ gamma,
                 const float *__restrict__ beta, const float *__restrict__ Wt, int K, int N, Epilogue epi,
                 GreedyPick gp, unsigned int *__restrict__ work) {
  extern __shared__ __align__(128) float smem[];
  float *xs = smem;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K4 = K >> 2;
  // Work is handed out CPW columns at a time: the first chunk of every warp is fixed (so its first loads can be
  // issued ahead of the dependency wait), the rest comes from a counter, because SMs do not all get the same share
  // of the memory bandwidth and equal shares of the columns left the slowest ones 6 us behind. work[0] counts the
  // chunks handed out beyond the fixed ones, work[1] the CTAs that are done; the last CTA leaves both zero.
  const int gw = blockIdx.x * 8 + warp, tw = gridDim.x * 8;
  const int c_beg = gw * CPW;
  TRACE_BEGIN(5);
  trace(5, 0);
  // first loads of this warp's first columns: weights are written by no kernel, so they may be requested while the
  // previous kernel is still running
  constexpr int PRE = 2;
  float4 wpre[CPW][PRE];
#pragma unroll
  for (int c = 0; c < CPW; c++) {
    const int col = min(c_beg + c, N - 1);
#pragma unroll
    for (int j = 0; j < PRE; j++) {
      const int i = lane + 32 * j;
      wpre[c][j] = i < K4 ? ldg_stream4(reinterpret_cast<const float4 *>(Wt + (size_t)col * K) + i)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  // gamma and beta are weights too
  const bool one_pass = M == 1 && K4 <= 256;  // the whole row fits one float4 per thread: block-wide LayerNorm
  float4 g_first = make_float4(1.f, 1.f, 1.f, 1.f), b_first = make_float4(0.f, 0.f, 0.f, 0.f);
  if (one_pass && gamma != nullptr && tid < K4) {
    g_first = reinterpret_cast<const float4 *>(gamma)[tid];
    b_first = reinterpret_cast<const float4 *>(beta)[tid];
  }
  pdl_wait();
  trace(5, 1);
  if (one_pass) {
    __shared__ float ln_red[16];
    const bool has = tid < K4;
    float4 v = has ? __ldcg(reinterpret_cast<const float4 *>(x) + tid) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (gamma != nullptr) v = block_layernorm4<256>(v, has, K, g_first, b_first, ln_red);
    if (has) reinterpret_cast<float4 *>(xs)[tid] = v;
    __syncthreads();
    pdl_launch_dependents();
  } else {
    {
      float4 *xs4w = reinterpret_cast<float4 *>(xs);
      const size_t ldx4 = ldx >> 2;
      const float4 *x4 = reinterpret_cast<const float4 *>(x);
      for (int idx = tid; idx < M * K4; idx += 256) {
        int m = idx / K4, i = idx - m * K4;
        xs4w[idx] = __ldcg(x4 + (size_t)m * ldx4 + i);
      }
    }
    __syncthreads();
    pdl_launch_dependents();
    if (gamma != nullptr) {  // LayerNorm (instructions.js:451-550), one warp per row, two passes over the row
      for (int m = warp; m < M; m += 8) {
        float4 *row = reinterpret_cast<float4 *>(xs + (size_t)m * K);
        float s = 0.f;
        for (int i = lane; i < K4; i += 32) {
          float4 v = row[i];
          s += (v.x + v.y) + (v.z + v.w);
        }
        float mean = warp_sum(s) / (float)K;
        float q = 0.f;
        for (int i = lane; i < K4; i += 32) {
          float4 v = row[i];
          float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
          q += (a * a + b * b) + (c * c + d * d);
        }
        float sd = sqrtf(warp_sum(q) / (float)K + 1e-5f);
        const float4 *g4 = reinterpret_cast<const float4 *>(gamma);
        const float4 *b4 = reinterpret_cast<const float4 *>(beta);
        for (int i = lane; i < K4; i += 32) {
          float4 v = row[i], g = g4[i], b = b4[i];
          row[i] = make_float4(g.x * ((v.x - mean) / sd) + b.x, g.y * ((v.y - mean) / sd) + b.y,
                               g.z * ((v.z - mean) / sd) + b.z, g.w * ((v.w - mean) / sd) + b.w);
        }
      }
      __syncthreads();
    }
  }
  trace(5, 2);

  const float4 *xs4 = reinterpret_cast<const float4 *>(xs);
  float bv[M];
  int bn[M];
#pragma unroll
  for (int m = 0; m < M; m++) { bv[m] = -INFINITY; bn[m] = 0x7fffffff; }
  unsigned int grabbed = 0;  // lane 0: the request for the chunk after the current one, issued one chunk ahead
  if (lane == 0) grabbed = atomicAdd(&work[0], 1u);
  int c0 = c_beg;
  while (c0 < N) {
    const int c_end = min(c0 + CPW, N);
    const float4 *w4[CPW];
#pragma unroll
    for (int c = 0; c < CPW; c++) w4[c] = reinterpret_cast<const float4 *>(Wt + (size_t)min(c0 + c, N - 1) * K);
    float acc[CPW][M];
#pragma unroll
    for (int c = 0; c < CPW; c++)
#pragma unroll
      for (int m = 0; m < M; m++) acc[c][m] = 0.f;
    int i0 = lane;
    if (c0 == c_beg) {  // the loads issued ahead of the dependency wait
#pragma unroll
      for (int j = 0; j < PRE; j++) {
        const int i = lane + 32 * j;
        if (i < K4) {
#pragma unroll
          for (int m = 0; m < M; m++) {
            const float4 xv = xs4[(size_t)m * K4 + i];
#pragma unroll
            for (int c = 0; c < CPW; c++) acc[c][m] += dot4(wpre[c][j], xv);
          }
        }
      }
      i0 = lane + 32 * PRE;
    }
#pragma unroll 4
    for (int i = i0; i < K4; i += 32) {
      float4 w[CPW];
#pragma unroll
      for (int c = 0; c < CPW; c++) w[c] = ldg_stream4(w4[c] + i);
#pragma unroll
      for (int m = 0; m < M; m++) {
        const float4 xv = xs4[(size_t)m * K4 + i];
#pragma unroll
        for (int c = 0; c < CPW; c++) acc[c][m] += dot4(w[c], xv);
      }
    }
    // every lane ends up with every sum; lane c*M + m stores column c0+c of row m
    float mine = 0.f;
#pragma unroll
    for (int c = 0; c < CPW; c++)
#pragma unroll
      for (int m = 0; m < M; m++) {
        const int n = c0 + c;
        float v = warp_sum(acc[c][m]);
        if (n < c_end) {  // same for the whole warp
          v = epi_apply(epi, v, m, n);
          if (lane == c * M + m) mine = v;
          if (v > bv[m]) { bv[m] = v; bn[m] = n; }  // columns ascend: the lowest index of equal values is kept
        }
      }
    if (lane < CPW * M) {
      const int c = lane / M, m = lane - c * M;
      if (c0 + c < c_end) *epi_addr(epi, m, c0 + c) = mine;
    }
    const long long nxt = ((long long)tw + (long long)__shfl_sync(0xffffffffu, grabbed, 0)) * CPW;
    if (nxt >= N) break;
    c0 = (int)nxt;
    if (lane == 0) grabbed = atomicAdd(&work[0], 1u);
  }
  trace(5, 3);
  // ---- greedy pick: every warp folds its best (value, index) of each row into one 64-bit key per row with an
  // atomic maximum (value in sortable form in the high word, 2^32-1 - index in the low word, so the lowest index
  // wins ties; a row of NaNs leaves the key zero and reports index 0); the last CTA to finish reads the keys.
  if (gp.keys != nullptr && lane == 0) {
#pragma unroll
    for (int m = 0; m < M; m++) {
      if (bn[m] != 0x7fffffff) {
        const unsigned int b = __float_as_uint(bv[m]);
        const unsigned int ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
        atomicMax(&gp.keys[m], ((unsigned long long)ord << 32) | (unsigned long long)(0xffffffffu - (unsigned int)bn[m]));
      }
    }
  }
  if (gp.next_w != nullptr && tid == 32) {  // this CTA's share of the next kernel's weights, towards L2
    const unsigned int n16 = gp.next_w_bytes >> 4;
    const unsigned int beg = (unsigned int)(((unsigned long long)n16 * blockIdx.x) / gridDim.x);
    const unsigned int end = (unsigned int)(((unsigned long long)n16 * (blockIdx.x + 1)) / gridDim.x);
    for (unsigned int o = beg; o < end; o += 1024u)
      prefetch_l2(gp.next_w + ((size_t)o << 4), min(end - o, 1024u) << 4);
  }
  __shared__ unsigned int is_last;
  __syncthreads();  // every warp of this CTA has made its last request and its last update of the keys
  if (tid == 0) {
    __threadfence();
    is_last = (atomicAdd(&work[1], 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  int my_step = 0;
  if (gp.keys != nullptr && tid < M) {
    const unsigned long long key = atomicExch(&gp.keys[tid], 0ull);
    const unsigned int idx = key ? 0xffffffffu - (unsigned int)(key & 0xffffffffull) : 0u;
    my_step = __ldcg(gp.step);
    gp.next_ids[tid] = idx;
    if (gp.out_ids) gp.out_ids[(size_t)tid * gp.out_stride + my_step] = idx;
  }
  __syncthreads();  // every row has read the step counter
  if (tid == 0) {
    work[0] = 0u;
    work[1] = 0u;
    if (gp.keys != nullptr) {
      *gp.pos = __ldcg(gp.pos) + gp.n_tok;
      *gp.step = my_step + 1;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// LayerNorm of M rows of K floats held in shared memory (normStats + norm, instructions.js:451-550).
// Every warp computes the two-pass statistics of every row itself (the row is only K floats, and this needs no
// block-wide barrier); the threads of the CTA then share the writes of the normalised rows into a second buffer.
// Ends with one __syncthreads(). gamma and beta are weights: the caller loads element tid of each before
// waiting on the previous kernel, so their memory latency is off the critical path.
template <int M>
__device__ __forceinline__ void cta_layernorm_rows(const float *raw, float *normed, int K,
                                                   const float *__restrict__ gamma, const float *__restrict__ beta,
                                                   float4 g_first, float4 b_first, int rs4) {
  // rs4: row stride of raw and normed in float4 (K/4, or more when the rows are padded against bank conflicts)
  const int tid = threadIdx.x, lane = tid & 31;
  const int K4 = K >> 2;
  const float4 *x4 = reinterpret_cast<const float4 *>(raw);
  float4 *o4 = reinterpret_cast<float4 *>(normed);
  const float4 *g4 = reinterpret_cast<const float4 *>(gamma);
  const float4 *b4 = reinterpret_cast<const float4 *>(beta);
  if (M > 1) {
    // Several rows: the warps share them (warp w takes rows w, w + warps, ...), each computing the statistics of
    // its row once and writing the normalised row itself. With every warp doing every row the cost grew with M
    // (28 us against 7 us for an eight-row QKV product).
    const int warp = tid >> 5, nw = (int)blockDim.x >> 5;
    // gamma and beta of this lane's first eight positions, requested before the statistics so that their L2
    // latency overlaps them (loaded one by one inside the last loop they cost a round trip per position)
    constexpr int GP = 8;
    float4 gpre[GP], bpre[GP];
    if (warp < M) {
#pragma unroll
      for (int j = 0; j < GP; j++) {
        const int i = lane + 32 * j;
        gpre[j] = i < K4 ? __ldg(g4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        bpre[j] = i < K4 ? __ldg(b4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    for (int m = warp; m < M; m += nw) {
      float s = 0.f;
#pragma unroll 4
      for (int i = lane; i < K4; i += 32) {
        float4 v = x4[(size_t)m * rs4 + i];
        s += (v.x + v.y) + (v.z + v.w);
      }
      const float mean = warp_sum(s) / (float)K;
      float q = 0.f;
#pragma unroll 4
      for (int i = lane; i < K4; i += 32) {
        float4 v = x4[(size_t)m * rs4 + i];
        float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
        q += (a * a + b * b) + (c * c + d * d);
      }
      const float rsd = 1.0f / sqrtf(warp_sum(q) / (float)K + 1e-5f);
#pragma unroll
      for (int j = 0; j < GP; j++) {
        const int i = lane + 32 * j;
        if (i < K4) {
          const float4 v = x4[(size_t)m * rs4 + i], g = gpre[j], b = bpre[j];
          o4[(size_t)m * rs4 + i] = make_float4(g.x * ((v.x - mean) * rsd) + b.x, g.y * ((v.y - mean) * rsd) + b.y,
                                               g.z * ((v.z - mean) * rsd) + b.z, g.w * ((v.w - mean) * rsd) + b.w);
        }
      }
      for (int i = lane + 32 * GP; i < K4; i += 32) {
        const float4 v = x4[(size_t)m * rs4 + i], g = __ldg(g4 + i), b = __ldg(b4 + i);
        o4[(size_t)m * rs4 + i] = make_float4(g.x * ((v.x - mean) * rsd) + b.x, g.y * ((v.y - mean) * rsd) + b.y,
                                             g.z * ((v.z - mean) * rsd) + b.z, g.w * ((v.w - mean) * rsd) + b.w);
      }
    }
    __syncthreads();
    return;
  }
#pragma unroll
  for (int m = 0; m < M; m++) {
    float s = 0.f;
#pragma unroll 4
    for (int i = lane; i < K4; i += 32) {
      float4 v = x4[(size_t)m * rs4 + i];
      s += (v.x + v.y) + (v.z + v.w);
    }
    const float mean = warp_sum(s) / (float)K;
    float q = 0.f;
#pragma unroll 4
    for (int i = lane; i < K4; i += 32) {
      float4 v = x4[(size_t)m * rs4 + i];
      float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
      q += (a * a + b * b) + (c * c + d * d);
    }
    // one division per row; the shader divides every element by sd (instructions.js:544), which differs from
    // multiplying by 1/sd by at most one unit in the last place
    const float rsd = 1.0f / sqrtf(warp_sum(q) / (float)K + 1e-5f);
    for (int i = tid; i < K4; i += (int)blockDim.x) {
      float4 v = x4[(size_t)m * rs4 + i], g = i == tid ? g_first : g4[i], b = i == tid ? b_first : b4[i];
      o4[(size_t)m * rs4 + i] = make_float4(g.x * ((v.x - mean) * rsd) + b.x, g.y * ((v.y - mean) * rsd) + b.y,
                                           g.z * ((v.z - mean) * rsd) + b.z, g.w * ((v.w - mean) * rsd) + b.w);
    }
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------------
// The layer GEMVs of a decode step (N up to a few thousand columns, 2-10 MB of weights): one CTA per SM owns
// `cols` consecutive output columns, i.e. one contiguous block of Wt, and fetches the whole block into shared
// memory with bulk asynchronous copies issued before the dependency wait, so the HBM stream of this kernel runs
// while the previous kernel is still executing. After the wait: stage + normalise the input rows, wait for the
// copies (bounded), multiply out of shared memory. Work items are (column, K slice), wk in {1,2,4,8}; a warp
// keeps the same K slice for all its items and handles three columns at a time; the K slices of a column are
// summed in a fixed order.
// Dynamic shared memory: [cols*K] weights, [M*K] input rows (twice with LayerNorm), [max(cols*wk, 16)*M]
// partial sums, one mbarrier.
// *err is set (and nothing stored) if the copies do not land within the poll limit.
constexpr int kBlockGemvThreads = 512;

template <int M>
__global__ void __launch_bounds__(kBlockGemvThreads)
gemv_block_kernel(const float *__restrict__ x, size_t ldx, const float *__restrict__ gamma,
                  const float *__restrict__ beta, const float *__restrict__ Wt, int K, int N, int cols, int wk,
                  Epilogue epi, int *err, AttnPartials ap) {
  extern __shared__ __align__(128) float smem[];
  // Rows-in-lanes form (more than four rows, see below): eight lanes read the same float4 position of eight
  // rows at once, so the rows are padded by one float4 to fall into different banks.
  constexpr bool kRowsInLanes = M > 4;
  const int RS4 = (K >> 2) + (kRowsInLanes ? 1 : 0);                      // row stride of xs / xn in float4
  float *wbuf = smem;
  float *xs = wbuf + (size_t)cols * K;                                    // input rows as staged
  float *xn = gamma != nullptr ? xs + (size_t)M * RS4 * 4 : xs;          // normalised rows (LayerNorm only)
  float *red = xn + (size_t)M * RS4 * 4;
  constexpr int NT = kBlockGemvThreads, NW = NT / 32;
  const int red_floats = ((kRowsInLanes ? NW * cols : max(cols * wk, NW)) * M + 3) & ~3;
  uint64_t *bar = reinterpret_cast<uint64_t *>(red + red_floats);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K4 = K >> 2;
  const int col0 = blockIdx.x * cols;
  const int ncol = min(cols, N - col0);

  TRACE_BEGIN(2);
  trace(2, 0);
  if (tid == 0) {
    mbar_init(bar, 1);
    const uint32_t row_bytes = (uint32_t)K * 4u;
    mbar_expect_tx(bar, row_bytes * (uint32_t)ncol);
    // a few rows per copy keeps each request modest and lets several be in flight
    const int rows_per_copy = max(1, (int)(16384u / row_bytes));
    for (int r = 0; r < ncol; r += rows_per_copy) {
      int nr = min(rows_per_copy, ncol - r);
      bulk_g2s(wbuf + (size_t)r * K, Wt + (size_t)(col0 + r) * K, row_bytes * (uint32_t)nr, bar);
    }
  }
  // The output this thread will finish in the epilogue: fetch its bias now (a weight: readable before the wait).
  const bool has_out = tid < ncol * M;
  const int oc = has_out ? tid / M : 0, om = has_out ? tid - oc * M : 0;
  float bias_v = 0.f, scale_v = 1.f;
  if (has_out && epi.bias) bias_v = epi.bias[col0 + oc];
  if (has_out && epi.colscale) scale_v = epi.colscale[col0 + oc];
  // All index arithmetic happens here, ahead of the wait (integer division is slow enough to matter after it).
  const int wk_log2 = 31 - __clz(wk);          // wk is a power of two
  const int ks = warp & (wk - 1);              // NW % wk == 0: every item of this warp has the same K slice
  const int beg = (int)(((unsigned)K4 * (unsigned)ks) >> wk_log2);
  const int end = (int)(((unsigned)K4 * (unsigned)(ks + 1)) >> wk_log2);
  const int items = ncol << wk_log2;
  float4 g_first = make_float4(0.f, 0.f, 0.f, 0.f), b_first = g_first;
  if (gamma != nullptr && tid < K4) {
    g_first = reinterpret_cast<const float4 *>(gamma)[tid];
    b_first = reinterpret_cast<const float4 *>(beta)[tid];
  }
  pdl_launch_dependents();
  pdl_wait();
  trace(2, 1);
  float res_v = 0.f;
  if (has_out && epi.residual) res_v = __ldcg(epi.residual + (size_t)om * epi.ld + col0 + oc);
  {
    float4 *xs4w = reinterpret_cast<float4 *>(xs);
    const size_t ldx4 = ldx >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    if (ap.part != nullptr) {  // the input rows are attention outputs still split into position slices
#pragma unroll
      for (int m = 0; m < M; m++)
        for (int i = tid; i < K4; i += NT) xs4w[(size_t)m * RS4 + i] = attn_merged_value4(ap, m, 4 * i);
    } else if (M > 1) {
      // Every CTA reads the same rows at the same time; starting each CTA at a different offset spreads the
      // requests over L2 instead of having all SMs ask for the same lines at once.
      const int total = M * K4;
      const int rot = (int)(((unsigned)blockIdx.x * 32u * 13u) % (unsigned)total);
      for (int j = tid; j < total; j += NT) {
        int idx = j + rot;
        if (idx >= total) idx -= total;
        const int m = idx / K4, i = idx - m * K4;
        xs4w[(size_t)m * RS4 + i] = __ldcg(x4 + (size_t)m * ldx4 + i);
      }
    } else {
#pragma unroll
      for (int m = 0; m < M; m++)
#pragma unroll 4
        for (int i = tid; i < K4; i += NT) xs4w[(size_t)m * RS4 + i] = __ldcg(x4 + (size_t)m * ldx4 + i);
    }
  }
  __syncthreads();  // also makes the mbarrier initialisation visible to every thread
  trace(2, 2);
  if (gamma != nullptr) cta_layernorm_rows<M>(xs, xn, K, gamma, beta, g_first, b_first, RS4);

  // Bounded wait for the weights. On expiry: flag the error, give the copies one more bounded chance to land
  // (shared memory must not be released under them), and leave without storing.
  trace(2, 3);
  const int landed = __syncthreads_and(mbar_wait(bar, 0, 1u << 20) ? 1 : 0);  // one decision for the whole CTA
  if (!landed) {
    if (tid == 0) atomicExch(err, 2);
    mbar_wait(bar, 0, 1u << 22);
    return;
  }

  trace(2, 4);
  const float4 *w4 = reinterpret_cast<const float4 *>(wbuf);
  const float4 *xs4 = reinterpret_cast<const float4 *>(xn);
  if (kRowsInLanes) {
    // More than four rows: a lane is (row slot = lane % 8, one of four K sub-slices = lane / 8) and every warp takes one
    // K chunk for all of the CTA's columns, eight columns at a time. A weight float4 is then read once per warp
    // (the eight row lanes share the address) and an input float4 once per column pass; with the K-in-lanes form
    // used for one row every warp re-read all M rows for every three columns (245 KB of shared-memory reads per
    // CTA for an eight-row QKV product, 4 us).
    constexpr int CB = 8;
    const int mrow = lane & 7, ksl = lane >> 3;
    const int mm = mrow < M ? mrow : M - 1;
    const int cbeg = (int)(((unsigned)K4 * (unsigned)warp) / NW), cend = (int)(((unsigned)K4 * (unsigned)(warp + 1)) / NW);
    for (int c0 = 0; c0 < ncol; c0 += CB) {
      float acc[CB];
#pragma unroll
      for (int cc = 0; cc < CB; cc++) acc[cc] = 0.f;
      for (int i = cbeg + ksl; i < cend; i += 4) {
        const float4 xv = xs4[(size_t)mm * RS4 + i];
#pragma unroll
        for (int cc = 0; cc < CB; cc++) {
          const int c = c0 + cc < ncol ? c0 + cc : ncol - 1;
          acc[cc] += dot4(w4[(size_t)c * K4 + i], xv);
        }
      }
#pragma unroll
      for (int cc = 0; cc < CB; cc++) {
        float v = acc[cc];
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if (ksl == 0 && mrow < M && c0 + cc < ncol) red[((size_t)warp * cols + c0 + cc) * M + mrow] = v;
      }
    }
    trace(2, 5);
    __syncthreads();
    for (int o = tid; o < ncol * M; o += NT) {  // the K chunks of an output in warp order
      const int cc = o / M, m = o - cc * M;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < NW; w++) v += red[((size_t)w * cols + cc) * M + m];
      epi_store(epi, v, m, col0 + cc);
    }
    trace(2, 6);
    return;
  }
  constexpr int NB = 3;
  for (int it0 = warp; it0 < items; it0 += NW * NB) {
    int c[NB];
    bool valid[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) {
      int it = it0 + NW * b;
      valid[b] = it < items;
      c[b] = valid[b] ? (it >> wk_log2) : 0;
    }
    float acc[NB][M];
#pragma unroll
    for (int b = 0; b < NB; b++)
#pragma unroll
      for (int m = 0; m < M; m++) acc[b][m] = 0.f;
#pragma unroll 4
    for (int i = beg + lane; i < end; i += 32) {
      float4 xv[M];
#pragma unroll
      for (int m = 0; m < M; m++) xv[m] = xs4[(size_t)m * RS4 + i];
#pragma unroll
      for (int b = 0; b < NB; b++) {
        if (valid[b]) {
          float4 w = w4[(size_t)c[b] * K4 + i];
#pragma unroll
          for (int m = 0; m < M; m++) acc[b][m] += dot4(w, xv[m]);
        }
      }
    }
    trace(2, 7);
#pragma unroll
    for (int b = 0; b < NB; b++)
#pragma unroll
      for (int m = 0; m < M; m++) {
        float v = warp_sum(acc[b][m]);
        if (lane == 0 && valid[b]) red[(c[b] * wk + ks) * M + m] = v;
      }
  }
  trace(2, 5);
  __syncthreads();
  if (has_out) {  // first NT outputs: bias / residual were fetched ahead
    float v = 0.f;
    for (int k = 0; k < wk; k++) v += red[(oc * wk + k) * M + om];
    v = v * scale_v + bias_v;
    if (epi.act == 1) v = gelu_f(v);
    if (epi.residual) v += res_v;
    *epi_addr(epi, om, col0 + oc) = v;
  }
  for (int o = tid + NT; o < ncol * M; o += NT) {
    const int cc = o / M, m = o - cc * M;
    float v = 0.f;
    for (int k = 0; k < wk; k++) v += red[(cc * wk + k) * M + m];
    epi_store(epi, v, m, col0 + cc);
  }
  trace(2, 6);
}

// ------------------------------------------------------------------------------------------------
// Weight in the reference layout W[K,N]. Thread owns 4 consecutive columns; a warp covers 128 columns of one
// k row per load (512 contiguous bytes); the CTA's 8 warps and gridDim.y CTAs split K.
// part receives [gridDim.y][M][N] partial sums (scratch); gemv_kn_reduce_kernel adds them in order.
template <int M>
__global__ void __launch_bounds__(256)
gemv_kn_partial_kernel(const float *__restrict__ x, const float *__restrict__ W, int K, int N,
                       float *__restrict__ part) {
  extern __shared__ __align__(128) float smem[];  // xs[M][kslice] + red[8][M][128]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ksplit = gridDim.y;
  const int kbeg = (int)(((long long)(K / 4) * blockIdx.y) / ksplit) * 4;
  const int kend = (int)(((long long)(K / 4) * (blockIdx.y + 1)) / ksplit) * 4;
  const int klen = kend - kbeg;
  float *xs = smem;
  float4 *red = reinterpret_cast<float4 *>(smem + (size_t)M * ((klen + 3) & ~3));
  for (int i = tid; i < M * klen; i += 256) {
    int m = i / klen, k = i - m * klen;
    xs[m * klen + k] = x[(size_t)m * K + kbeg + k];
  }
  __syncthreads();
  const int n = blockIdx.x * 128 + lane * 4;
  float4 acc[M];
#pragma unroll
  for (int m = 0; m < M; m++) acc[m] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (n < N) {
    const float *wp = W + (size_t)kbeg * N + n;
#pragma unroll 8
    for (int k = warp; k < klen; k += 8) {
      float4 w = ldg_stream4(reinterpret_cast<const float4 *>(wp + (size_t)k * N));
#pragma unroll
      for (int m = 0; m < M; m++) {
        float a = xs[m * klen + k];
        acc[m].x += a * w.x; acc[m].y += a * w.y; acc[m].z += a * w.z; acc[m].w += a * w.w;
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; m++) red[(warp * M + m) * 32 + lane] = acc[m];
  __syncthreads();
  for (int i = tid; i < M * 32; i += 256) {
    int m = i / 32, l = i % 32;
    int nn = blockIdx.x * 128 + l * 4;
    if (nn >= N) continue;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 8; w++) {
      float4 v = red[(w * M + m) * 32 + l];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    *reinterpret_cast<float4 *>(part + ((size_t)blockIdx.y * M + m) * N + nn) = s;
  }
}

// part: [ksplit][N / tw column tiles][M][tw] (tw = N: plain [ksplit][M][N]); tw % 4 == 0.
__global__ void gemv_kn_reduce_kernel(const float *__restrict__ part, int ksplit, int M, int N, Epilogue epi, int tw) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;  // float4 index over [M, N/4]
  int N4 = N >> 2;
  TRACE_BEGIN(6);
  trace(6, 0);
  const bool live = i < M * N4;
  const int m = live ? i / N4 : 0, n = live ? (i - m * N4) * 4 : 0;
  float4 bias_pre = make_float4(0.f, 0.f, 0.f, 0.f), res_pre = bias_pre;
  if (live && epi.bias) bias_pre = *reinterpret_cast<const float4 *>(epi.bias + n);  // a weight: ahead of the wait
  pdl_launch_dependents();
  pdl_wait();  // the partial sums come from the previous kernel
  trace(6, 1);
  if (!live) return;
  if (epi.residual) res_pre = __ldcg(reinterpret_cast<const float4 *>(epi.residual + (size_t)m * epi.ld + n));
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  const int n_tiles = (N + tw - 1) / tw, nt = n / tw;
  const float *p0 = part + ((size_t)nt * M + m) * tw + (n - nt * tw);
  const size_t zstride = (size_t)n_tiles * M * tw;
#pragma unroll 8
  for (int k = 0; k < ksplit; k++) {
    float4 v = __ldcg(reinterpret_cast<const float4 *>(p0 + (size_t)k * zstride));
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  *reinterpret_cast<float4 *>(epi_addr(epi, m, n)) = epi_apply4_pre(epi, s, bias_pre, res_pre, n);
  trace(6, 2);
}

// Second stage of a split-K product whose consumer is a LayerNorm (the residual stream feeding the next block):
// one CTA per row adds the slices in order (layout as in gemv_kn_reduce_kernel), applies the epilogue (bias, residual) into epi.out, and normalises the
// finished row, still in registers, into ln_out[M, N] (mean and variance over N as in layernorm_kernel). Saves the
// separate LayerNorm pass and its read of the row. N <= 4096 (four float4 per thread).
constexpr int kReduceLnVec = 4;
__global__ void __launch_bounds__(256)
splitk_reduce_ln_kernel(const float *__restrict__ part, int ksplit, int M, int N, Epilogue epi,
                        const float *__restrict__ gamma, const float *__restrict__ beta,
                        float *__restrict__ ln_out, int tw) {
  __shared__ float red[2][8];
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N4 = N >> 2;
  TRACE_BEGIN(7);
  trace(7, 0);
  // weights (LayerNorm scale and shift, bias) ahead of the dependency wait; the residual with the partial sums
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 g_pre[kReduceLnVec], b_pre[kReduceLnVec], bias_pre[kReduceLnVec], res_pre[kReduceLnVec];
#pragma unroll
  for (int r = 0; r < kReduceLnVec; r++) {
    const int i = tid + 256 * r;
    g_pre[r] = b_pre[r] = bias_pre[r] = res_pre[r] = zero4;
    if (i < N4) {
      g_pre[r] = *reinterpret_cast<const float4 *>(gamma + 4 * i);
      b_pre[r] = *reinterpret_cast<const float4 *>(beta + 4 * i);
      if (epi.bias) bias_pre[r] = *reinterpret_cast<const float4 *>(epi.bias + 4 * i);
    }
  }
  pdl_launch_dependents();
  pdl_wait();  // the partial sums come from the previous kernel
  trace(7, 1);
  if (epi.residual) {
#pragma unroll
    for (int r = 0; r < kReduceLnVec; r++) {
      const int i = tid + 256 * r;
      if (i < N4) res_pre[r] = __ldcg(reinterpret_cast<const float4 *>(epi.residual + (size_t)m * epi.ld + 4 * i));
    }
  }
  float4 v[kReduceLnVec];
  float s = 0.f;
#pragma unroll
  for (int r = 0; r < kReduceLnVec; r++) {
    const int i = tid + 256 * r;
    v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < N4) {
      const int n = i * 4;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      const int n_tiles = (N + tw - 1) / tw, nt = n / tw;
      const float *p0 = part + ((size_t)nt * M + m) * tw + (n - nt * tw);
      const size_t zstride = (size_t)n_tiles * M * tw;
      // eight slices in flight per thread: the row is short and few CTAs run, so the loop is bound by latency
      int k = 0;
      for (; k + 12 <= ksplit; k += 12) {
        float4 t[12];
#pragma unroll
        for (int u = 0; u < 12; u++) t[u] = __ldcg(reinterpret_cast<const float4 *>(p0 + (size_t)(k + u) * zstride));
#pragma unroll
        for (int u = 0; u < 12; u++) { a.x += t[u].x; a.y += t[u].y; a.z += t[u].z; a.w += t[u].w; }
      }
      for (; k + 4 <= ksplit; k += 4) {
        float4 t[4];
#pragma unroll
        for (int u = 0; u < 4; u++) t[u] = __ldcg(reinterpret_cast<const float4 *>(p0 + (size_t)(k + u) * zstride));
#pragma unroll
        for (int u = 0; u < 4; u++) { a.x += t[u].x; a.y += t[u].y; a.z += t[u].z; a.w += t[u].w; }
      }
      for (; k < ksplit; k++) {
        float4 t = __ldcg(reinterpret_cast<const float4 *>(p0 + (size_t)k * zstride));
        a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
      }
      a = epi_apply4_pre(epi, a, bias_pre[r], res_pre[r], n);
      *reinterpret_cast<float4 *>(epi_addr(epi, m, n)) = a;
      v[r] = a;
      s += (a.x + a.y) + (a.z + a.w);
    }
  }
  s = warp_sum(s);
  if (lane == 0) red[0][warp] = s;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; w++) tot += red[0][w];
  const float mean = tot / (float)N;
  float q = 0.f;
#pragma unroll
  for (int r = 0; r < kReduceLnVec; r++) {
    if (tid + 256 * r < N4) {
      float a = v[r].x - mean, b = v[r].y - mean, c = v[r].z - mean, d = v[r].w - mean;
      q += (a * a + b * b) + (c * c + d * d);
    }
  }
  q = warp_sum(q);
  if (lane == 0) red[1][warp] = q;
  __syncthreads();
  float qt = 0.f;
#pragma unroll
  for (int w = 0; w < 8; w++) qt += red[1][w];
  const float sd = sqrtf(qt / (float)N + 1e-5f);
#pragma unroll
  for (int r = 0; r < kReduceLnVec; r++) {
    const int i = tid + 256 * r;
    if (i < N4) {
      const float4 g = g_pre[r], b = b_pre[r];
      *reinterpret_cast<float4 *>(ln_out + (size_t)m * N + 4 * i) =
          make_float4(g.x * ((v[r].x - mean) / sd) + b.x, g.y * ((v[r].y - mean) / sd) + b.y,
                      g.z * ((v[r].z - mean) / sd) + b.z, g.w * ((v[r].w - mean) / sd) + b.w);
    }
  }
  trace(7, 2);
}

// ------------------------------------------------------------------------------------------------
// C[M,N] = A[M,K] . B (+ epilogue). A rows at stride lda. B is [K,N] (B_NK = false, the reference layout)
// or [N,K] (B_NK = true). K % 4 == 0, N % 4 == 0. 256 threads, 64x64 tile, 16-deep K step.
template <bool B_NK>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const float *__restrict__ A, size_t lda, const float *__restrict__ B, int M, int K, int N,
                 Epilogue epi) {
  __shared__ __align__(16) float As[16][64 + 4];
  __shared__ __align__(16) float Bs[16][64 + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each 4 rows x 4 cols
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  const int a_row = tid >> 2, a_k4 = (tid & 3) * 4;  // A tile: 64 rows x 16 k
  const int bkn_k = tid >> 4, bkn_n4 = (tid & 15) * 4;  // B[K,N] tile: 16 k x 64 n
  const int bnk_n = tid >> 2, bnk_k4 = (tid & 3) * 4;   // B[N,K] tile: 64 n x 16 k

  for (int k0 = 0; k0 < K; k0 += 16) {
    {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m0 + a_row < M && k0 + a_k4 < K)
        v = *reinterpret_cast<const float4 *>(A + (size_t)(m0 + a_row) * lda + k0 + a_k4);
      As[a_k4 + 0][a_row] = v.x; As[a_k4 + 1][a_row] = v.y; As[a_k4 + 2][a_row] = v.z; As[a_k4 + 3][a_row] = v.w;
    }
    if (B_NK) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (n0 + bnk_n < N && k0 + bnk_k4 < K)
        v = *reinterpret_cast<const float4 *>(B + (size_t)(n0 + bnk_n) * K + k0 + bnk_k4);
      Bs[bnk_k4 + 0][bnk_n] = v.x; Bs[bnk_k4 + 1][bnk_n] = v.y; Bs[bnk_k4 + 2][bnk_n] = v.z; Bs[bnk_k4 + 3][bnk_n] = v.w;
    } else {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k0 + bkn_k < K && n0 + bkn_n4 < N)
        v = *reinterpret_cast<const float4 *>(B + (size_t)(k0 + bkn_k) * N + n0 + bkn_n4);
      *reinterpret_cast<float4 *>(&Bs[bkn_k][bkn_n4]) = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; k++) {
      float4 a = *reinterpret_cast<const float4 *>(&As[k][ty * 4]);
      float4 b = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4]);
      float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }
  const bool vec_ok = ((N | epi.ld) & 3) == 0;  // e.g. vocab-sized outputs are not a multiple of 4
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int m = m0 + ty * 4 + i, n = n0 + tx * 4;
    if (m >= M || n >= N) continue;
    if (vec_ok) {
      epi_store4(epi, make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]), m, n);
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (n + j < N) epi_store(epi, acc[i][j], m, n + j);
    }
  }
}

}  // namespace wgpt
