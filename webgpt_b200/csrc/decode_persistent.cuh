// Whole-token decode kernel for one sequence: a single cooperative launch runs n_steps greedy decode steps.
//
// One 512-thread CTA per SM stays resident; the five dependent stages of every layer (LN1+QKV, attention,
// projection+residual, LN2+FC+GELU, down-projection+residual) and the ln_f + de-embedding + greedy pick are
// separated by grid-wide barriers instead of kernel boundaries. Every CTA owns the same consecutive block of
// output columns of each weight matrix for the whole run and fetches block j+1 into the second of two shared-
// memory buffers (untiled TMA bulk copies, one mbarrier per buffer) while stage j computes, so the HBM stream
// does not stop at stage boundaries. The de-embedding table (larger than shared memory) is streamed through
// registers. Activations cross CTAs through global memory: writers fence before arriving at the barrier,
// readers use L2 loads (ld.global.cg).
//
// Status: correct (it passes the same parity tests as the kernel chain) but slower on B200 - 0.349 ms/token
// against 0.274 for the CUDA-graph chain with programmatic dependent launch on GPT-2 117M. A device-side trace
// shows why: a software barrier through L2 costs ~1.8 us (148 same-address atomics plus a poll) and the first
// read of data another SM just wrote costs another 0.9-1.9 us, while the hardware's kernel-to-kernel hand-off
// costs ~0.65 us and the input rows arrive in ~0.55 us. It is therefore opt-in (WGPT_PERSISTENT=1) and kept as
// the base for a version with fewer barriers per layer.
//
// Barrier: one 64-bit counter, monotonically increasing; barrier k of a launch is passed when the counter
// reaches base + (k+1)*gridDim.x (base is a launch argument kept by the host). The spin is bounded: on expiry,
// or when another CTA raised the abort word, the CTA flags *err = 4 and the whole grid leaves.
#pragma once
#include "attention.cuh"
#include "common.cuh"
#include "gemm_tc.cuh"
#include "matmul.cuh"

namespace wgpt {

struct LayerPtrs {
  const float *ln1_g, *ln1_b, *wqkv, *bqkv, *wo, *bo, *ln2_g, *ln2_b, *wfc, *bfc, *wpr, *bpr;
};

struct DecodeParams {
  const LayerPtrs *layers;
  int n_layer, E, H, n_ctx, V;
  const float *wte, *wpe, *lnf_g, *lnf_b;
  float *x, *q, *f, *logits;   // [E], [E], [4E], [V]
  float *kc, *vc;              // layer l at + l*kv_layer_stride, rows of E floats
  size_t kv_layer_stride;
  float *attn_part;            // [H][nsl][hs+4]
  float *cand_val;             // [gridDim.x] per-CTA arg-max candidates
  int *cand_idx;
  uint32_t *next_id, *out_ids;
  int *pos, *step;
  int n_steps;
  unsigned long long *bar_counter;
  unsigned long long bar_base;
  int *err;                    // device error word
  int *abort_word;             // zero on entry; any CTA that gives up sets it
  float scale;
  int cols_qkv, cols_proj, cols_fc, cols_down;  // columns per CTA
  int wk_qkv, wk_proj, wk_fc, wk_down;          // K slices per column (power of two <= 16)
  int rows_deembed;                             // vocabulary rows per CTA
  int nsl;                                      // position slices per head in the attention stage (<= 8)
  int wbuf_floats;                              // capacity of one weight buffer
};

constexpr int kDecodeThreads = 512;

// Development aid (-DWGPT_TRACE): thread 0 of CTA 0 stamps globaltimer at every stage boundary.
#ifdef WGPT_TRACE
#define PK_TRACE(id)                                                                  \
  do {                                                                                \
    if (threadIdx.x == 0 && blockIdx.x == 0 && pk_tr < (1 << 16)) {                   \
      unsigned long long t_;                                                          \
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));                           \
      g_trace_buf[2 * pk_tr] = t_;                                                    \
      g_trace_buf[2 * pk_tr + 1] = ((unsigned long long)5 << 16) | ((unsigned long long)(id) << 8); \
      pk_tr++;                                                                        \
    }                                                                                 \
  } while (0)
#else
#define PK_TRACE(id) ((void)0)
#endif
constexpr unsigned kBarrierPolls = 1u << 22;

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Grid-wide barrier; returns false (for every thread of the CTA) if the grid is being abandoned.
__device__ __forceinline__ bool grid_barrier(const DecodeParams &p, unsigned long long &target) {
  target += gridDim.x;
  __syncthreads();
  int ok = 1;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(p.bar_counter, 1ULL);
    unsigned n = 0;
    while (ld_acquire_u64(p.bar_counter) < target) {
      if (++n > kBarrierPolls || *reinterpret_cast<volatile int *>(p.abort_word) != 0) {
        ok = 0;
        break;
      }
    }
    if (!ok) {
      atomicExch(p.abort_word, 1);
      atomicExch(p.err, 4);
    }
    __threadfence();
  }
  return __syncthreads_and(ok) != 0;
}

// Thread 0 starts the copy of this CTA's rows [col0, col0+ncol) of Wt[N,K] into wbuf and arms `bar`.
__device__ __forceinline__ void issue_weight_block(float *wbuf, uint64_t *bar, const float *Wt, int N, int K, int cols) {
  const int col0 = blockIdx.x * cols;
  if (col0 >= N) {  // this CTA owns no column of the matrix: complete the barrier phase so that parities stay in step
    mbar_arrive(bar);
    return;
  }
  const int ncol = min(cols, N - col0);
  const uint32_t row_bytes = (uint32_t)K * 4u;
  fence_async_smem();
  mbar_expect_tx(bar, row_bytes * (uint32_t)ncol);
  const int rows_per_copy = max(1, (int)(16384u / row_bytes));
  for (int r = 0; r < ncol; r += rows_per_copy) {
    int nr = min(rows_per_copy, ncol - r);
    bulk_g2s(wbuf + (size_t)r * K, Wt + (size_t)(col0 + r) * K, row_bytes * (uint32_t)nr, bar);
  }
}

// y[c] = sum_k w[c][k] * xin[k] for this CTA's ncol columns held in shared memory; items = (column, K slice),
// three columns per warp pass, K slices summed in order; result handed to emit(c_local, value) by thread c_local.
template <typename Emit>
__device__ __forceinline__ void cta_block_gemv(const float *wbuf, const float *xin, int K, int ncol, int wk, float *red,
                                               Emit emit) {
  constexpr int NW = kDecodeThreads / 32, NB = 3;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K4 = K >> 2;
  const int wk_log2 = 31 - __clz(wk);
  const int ks = warp & (wk - 1);
  const int beg = (int)(((unsigned)K4 * (unsigned)ks) >> wk_log2);
  const int end = (int)(((unsigned)K4 * (unsigned)(ks + 1)) >> wk_log2);
  const int items = ncol << wk_log2;
  const float4 *w4 = reinterpret_cast<const float4 *>(wbuf);
  const float4 *x4 = reinterpret_cast<const float4 *>(xin);
  for (int it0 = warp; it0 < items; it0 += NW * NB) {
    int c[NB];
    bool valid[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) {
      int it = it0 + NW * b;
      valid[b] = it < items;
      c[b] = valid[b] ? (it >> wk_log2) : 0;
    }
    float acc[NB] = {0.f, 0.f, 0.f};
#pragma unroll 4
    for (int i = beg + lane; i < end; i += 32) {
      const float4 xv = x4[i];
#pragma unroll
      for (int b = 0; b < NB; b++)
        if (valid[b]) acc[b] += dot4(w4[(size_t)c[b] * K4 + i], xv);
    }
#pragma unroll
    for (int b = 0; b < NB; b++) {
      float v = warp_sum(acc[b]);
      if (lane == 0 && valid[b]) red[c[b] * wk + ks] = v;
    }
  }
  __syncthreads();
  if (tid < ncol) {
    float v = 0.f;
    for (int k = 0; k < wk; k++) v += red[tid * wk + k];
    emit(tid, v);
  }
  __syncthreads();
}

// Two-pass LayerNorm of one row of K floats in shared memory into `out` (instructions.js:451-550): every warp
// computes the statistics itself, the threads share the writes. Ends with __syncthreads().
__device__ __forceinline__ void cta_layernorm_row(const float *raw, float *out, int K, const float *__restrict__ gamma,
                                                  const float *__restrict__ beta) {
  const int tid = threadIdx.x, lane = tid & 31, K4 = K >> 2;
  const float4 *x4 = reinterpret_cast<const float4 *>(raw);
  float s = 0.f;
  for (int i = lane; i < K4; i += 32) {
    float4 v = x4[i];
    s += (v.x + v.y) + (v.z + v.w);
  }
  const float mean = warp_sum(s) / (float)K;
  float q = 0.f;
  for (int i = lane; i < K4; i += 32) {
    float4 v = x4[i];
    float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
    q += (a * a + b * b) + (c * c + d * d);
  }
  const float rsd = 1.0f / sqrtf(warp_sum(q) / (float)K + 1e-5f);
  const float4 *g4 = reinterpret_cast<const float4 *>(gamma), *b4 = reinterpret_cast<const float4 *>(beta);
  float4 *o4 = reinterpret_cast<float4 *>(out);
  for (int i = tid; i < K4; i += kDecodeThreads) {
    float4 v = x4[i], g = g4[i], b = b4[i];
    o4[i] = make_float4(g.x * ((v.x - mean) * rsd) + b.x, g.y * ((v.y - mean) * rsd) + b.y,
                        g.z * ((v.z - mean) * rsd) + b.z, g.w * ((v.w - mean) * rsd) + b.w);
  }
  __syncthreads();
}


// Shared memory: two weight buffers, xs (4E floats: staged input), xn (E floats: normalised input), red, small.
template <int HS>
__global__ void __launch_bounds__(kDecodeThreads, 1) decode_persistent_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(128) float dsm[];
  float *wbuf0 = dsm, *wbuf1 = dsm + p.wbuf_floats;
  float *xs = wbuf1 + p.wbuf_floats;        // 4E
  float *xn = xs + 4 * p.E;                 // E
  float *red = xn + p.E;                    // max(cols*wk) <= 1024
  uint64_t *bars = reinterpret_cast<uint64_t *>(red + 1024);
  __shared__ float sm_m[16], sm_l[16];
  __shared__ __align__(16) float sm_acc[16][HS];
  __shared__ float cand_v[16];
  __shared__ int cand_n[16];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int E = p.E, F = 4 * p.E, E4 = p.E >> 2, H = p.H;
  unsigned long long target = p.bar_base;
  int blk = 0;  // weight blocks consumed so far: block j lives in buffer j&1, its mbarrier phase is (j>>1)&1

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    fence_async_smem();
  }
  __syncthreads();
  int issued = 0;  // weight blocks issued so far (thread 0 only uses it)
  auto issue = [&](const float *Wt, int N, int K, int cols) {
    if (tid == 0) issue_weight_block((issued & 1) ? wbuf1 : wbuf0, &bars[issued & 1], Wt, N, K, cols);
    issued++;
  };
  // Waits for block `blk`; false (for the whole CTA) = timed out.
  auto wait_block = [&]() -> bool {
    const bool ok = mbar_wait(&bars[blk & 1], (blk >> 1) & 1, 1u << 20);
    return __syncthreads_and(ok ? 1 : 0) != 0;
  };
  bool alive = true;
#ifdef WGPT_TRACE
  unsigned int pk_tr = 0;
#endif
  auto give_up = [&]() {
    if (tid == 0) {
      atomicExch(p.abort_word, 1);
      atomicExch(p.err, 4);
    }
    alive = false;
  };

  issue(p.layers[0].wqkv, 3 * E, E, p.cols_qkv);

  for (int st = 0; st < p.n_steps && alive; st++) {
    const int pos = __ldcg(p.pos);
    const uint32_t id = __ldcg(p.next_id);
    // ---- embedding (EmbedBlock, instructions.js:790-827): every CTA builds x itself, CTA 0 publishes it ----
    {
      const float4 *a = reinterpret_cast<const float4 *>(p.wte + (size_t)id * E);
      const float4 *b = reinterpret_cast<const float4 *>(p.wpe + (size_t)pos * E);
      for (int i = tid; i < E4; i += kDecodeThreads) {
        float4 u = a[i], v = b[i];
        float4 r = make_float4(u.x + v.x, u.y + v.y, u.z + v.z, u.w + v.w);
        reinterpret_cast<float4 *>(xs)[i] = r;
        if (blockIdx.x == 0) reinterpret_cast<float4 *>(p.x)[i] = r;
      }
      __syncthreads();
    }
    for (int l = 0; l < p.n_layer && alive; l++) {
      const LayerPtrs L = p.layers[l];
      float *kc = p.kc + (size_t)l * p.kv_layer_stride, *vc = p.vc + (size_t)l * p.kv_layer_stride;
      // ================= stage 1: LN1 + QKV, K and V rows straight into the cache =================
      if (l > 0) {
        for (int i = tid; i < E4; i += kDecodeThreads)
          reinterpret_cast<float4 *>(xs)[i] = __ldcg(reinterpret_cast<const float4 *>(p.x) + i);
        __syncthreads();
      }
      issue(L.wo, E, E, p.cols_proj);
      // this CTA's slice of the cache for the attention stage, towards L2 (rows 0..pos-1 never change)
      if (blockIdx.x < H * p.nsl) {
        const int h = blockIdx.x / p.nsl, sl = blockIdx.x % p.nsl;
        const int chunk = (pos + 1 + p.nsl - 1) / p.nsl;
        const int b0 = sl * chunk, e0 = min(pos, b0 + chunk);
        for (int r = b0 + (tid >> 1); r < e0; r += kDecodeThreads / 2)
          prefetch_l2(((tid & 1) ? vc : kc) + (size_t)r * E + h * HS, HS * 4);
      }
      PK_TRACE(1);
      cta_layernorm_row(xs, xn, E, L.ln1_g, L.ln1_b);
      PK_TRACE(2);
      if (!wait_block()) { give_up(); break; }
      PK_TRACE(3);
      {
        const int col0 = blockIdx.x * p.cols_qkv, ncol = max(0, min(p.cols_qkv, 3 * E - col0));
        cta_block_gemv((blk & 1) ? wbuf1 : wbuf0, xn, E, ncol, p.wk_qkv, red, [&](int c, float v) {
          const int n = col0 + c;
          v += L.bqkv[n];
          if (n < E) p.q[n] = v;
          else if (n < 2 * E) kc[(size_t)pos * E + (n - E)] = v;
          else vc[(size_t)pos * E + (n - 2 * E)] = v;
        });
      }
      blk++;
      PK_TRACE(4);
      if (!grid_barrier(p, target)) { alive = false; break; }
      PK_TRACE(5);
      // ================= stage 2: attention over the cache, one (head, position slice) per CTA =================
      if (blockIdx.x < H * p.nsl) {
        constexpr int LPP = HS / 4, G = 32 / LPP, NW = kDecodeThreads / 32;
        const int h = blockIdx.x / p.nsl, sl = blockIdx.x % p.nsl;
        const int g = lane / LPP, lig = lane % LPP;
        const int Lk = pos + 1, chunk = (Lk + p.nsl - 1) / p.nsl;
        const int beg = sl * chunk, end = min(Lk, beg + chunk);
        const float4 q4 = __ldcg(reinterpret_cast<const float4 *>(p.q + h * HS + lig * 4));
        const float *kb = kc + h * HS + lig * 4, *vb = vc + h * HS + lig * 4;
        float m = -INFINITY, lsum = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
        for (int j0 = beg + warp * G; j0 < end; j0 += NW * G) {  // warp-uniform trip count
          const int j = j0 + g;
          const bool valid = j < end;
          const int jj = valid ? j : end - 1;
          float4 k4 = __ldcg(reinterpret_cast<const float4 *>(kb + (size_t)jj * E));
          float4 v4 = __ldcg(reinterpret_cast<const float4 *>(vb + (size_t)jj * E));
          float sc = dot4(q4, k4);
#pragma unroll
          for (int o = LPP / 2; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
          if (valid) {
            sc *= p.scale;
            float mn = fmaxf(m, sc);
            float corr = expf(m - mn), pr = expf(sc - mn);
            lsum = lsum * corr + pr;
            acc.x = acc.x * corr + pr * v4.x; acc.y = acc.y * corr + pr * v4.y;
            acc.z = acc.z * corr + pr * v4.z; acc.w = acc.w * corr + pr * v4.w;
            m = mn;
          }
        }
        __syncwarp();
#pragma unroll
        for (int o = LPP; o < 32; o <<= 1) {
          float mo = __shfl_xor_sync(0xffffffffu, m, o), lo = __shfl_xor_sync(0xffffffffu, lsum, o);
          float4 ao;
          ao.x = __shfl_xor_sync(0xffffffffu, acc.x, o); ao.y = __shfl_xor_sync(0xffffffffu, acc.y, o);
          ao.z = __shfl_xor_sync(0xffffffffu, acc.z, o); ao.w = __shfl_xor_sync(0xffffffffu, acc.w, o);
          float mn = fmaxf(m, mo);
          float c0 = (m == -INFINITY) ? 0.f : expf(m - mn), c1 = (mo == -INFINITY) ? 0.f : expf(mo - mn);
          lsum = lsum * c0 + lo * c1;
          acc.x = acc.x * c0 + ao.x * c1; acc.y = acc.y * c0 + ao.y * c1;
          acc.z = acc.z * c0 + ao.z * c1; acc.w = acc.w * c0 + ao.w * c1;
          m = mn;
        }
        if (g == 0) {
          *reinterpret_cast<float4 *>(&sm_acc[warp][lig * 4]) = acc;
          if (lig == 0) { sm_m[warp] = m; sm_l[warp] = lsum; }
        }
        __syncthreads();
        if (tid < HS) {
          float mm = sm_m[0];
#pragma unroll
          for (int w = 1; w < NW; w++) mm = fmaxf(mm, sm_m[w]);
          float ll = 0.f, a = 0.f;
#pragma unroll
          for (int w = 0; w < NW; w++) {
            float c = (sm_m[w] == -INFINITY) ? 0.f : expf(sm_m[w] - mm);
            ll += sm_l[w] * c;
            a += sm_acc[w][tid] * c;
          }
          float *my = p.attn_part + ((size_t)h * p.nsl + sl) * (HS + 4);
          my[tid] = a;
          if (tid == 0) { my[HS] = mm; my[HS + 1] = ll; }
        }
      }
      PK_TRACE(6);
      if (!grid_barrier(p, target)) { alive = false; break; }
      PK_TRACE(7);
      // ================= stage 3: merge the slices, output projection + residual =================
      issue(L.wfc, F, E, p.cols_fc);
      {
        AttnPartials ap;
        ap.part = p.attn_part; ap.n_split = p.nsl; ap.H = H; ap.hs = HS;
        for (int i = tid; i < E4; i += kDecodeThreads) reinterpret_cast<float4 *>(xs)[i] = attn_merged_value4(ap, 0, 4 * i);
        __syncthreads();
      }
      PK_TRACE(8);
      if (!wait_block()) { give_up(); break; }
      PK_TRACE(9);
      {
        const int col0 = blockIdx.x * p.cols_proj, ncol = max(0, min(p.cols_proj, E - col0));
        cta_block_gemv((blk & 1) ? wbuf1 : wbuf0, xs, E, ncol, p.wk_proj, red, [&](int c, float v) {
          const int n = col0 + c;
          p.x[n] = v + L.bo[n] + __ldcg(p.x + n);
        });
      }
      blk++;
      PK_TRACE(10);
      if (!grid_barrier(p, target)) { alive = false; break; }
      PK_TRACE(11);
      // ================= stage 4: LN2 + FC + GELU =================
      issue(L.wpr, E, F, p.cols_down);
      for (int i = tid; i < E4; i += kDecodeThreads)
        reinterpret_cast<float4 *>(xs)[i] = __ldcg(reinterpret_cast<const float4 *>(p.x) + i);
      __syncthreads();
      PK_TRACE(12);
      cta_layernorm_row(xs, xn, E, L.ln2_g, L.ln2_b);
      PK_TRACE(13);
      if (!wait_block()) { give_up(); break; }
      PK_TRACE(14);
      {
        const int col0 = blockIdx.x * p.cols_fc, ncol = max(0, min(p.cols_fc, F - col0));
        cta_block_gemv((blk & 1) ? wbuf1 : wbuf0, xn, E, ncol, p.wk_fc, red, [&](int c, float v) {
          const int n = col0 + c;
          p.f[n] = gelu_f(v + L.bfc[n]);
        });
      }
      blk++;
      PK_TRACE(15);
      if (!grid_barrier(p, target)) { alive = false; break; }
      PK_TRACE(16);
      // ================= stage 5: down projection + residual =================
      if (l + 1 < p.n_layer) issue(p.layers[l + 1].wqkv, 3 * E, E, p.cols_qkv);
      else if (st + 1 < p.n_steps) issue(p.layers[0].wqkv, 3 * E, E, p.cols_qkv);
      for (int i = tid; i < E; i += kDecodeThreads)  // 4E floats = E float4
        reinterpret_cast<float4 *>(xs)[i] = __ldcg(reinterpret_cast<const float4 *>(p.f) + i);
      __syncthreads();
      PK_TRACE(17);
      if (!wait_block()) { give_up(); break; }
      PK_TRACE(18);
      {
        const int col0 = blockIdx.x * p.cols_down, ncol = max(0, min(p.cols_down, E - col0));
        cta_block_gemv((blk & 1) ? wbuf1 : wbuf0, xs, F, ncol, p.wk_down, red, [&](int c, float v) {
          const int n = col0 + c;
          p.x[n] = v + L.bpr[n] + __ldcg(p.x + n);
        });
      }
      blk++;
      PK_TRACE(19);
      if (!grid_barrier(p, target)) { alive = false; break; }
      PK_TRACE(20);
    }
    if (!alive) break;
    // ================= ln_f + tied de-embedding (register-streamed) + greedy pick =================
    for (int i = tid; i < E4; i += kDecodeThreads)
      reinterpret_cast<float4 *>(xs)[i] = __ldcg(reinterpret_cast<const float4 *>(p.x) + i);
    __syncthreads();
    cta_layernorm_row(xs, xn, E, p.lnf_g, p.lnf_b);
    {
      constexpr int NW = kDecodeThreads / 32;
      const int r0 = blockIdx.x * p.rows_deembed, r1 = min(p.V, r0 + p.rows_deembed);
      const float4 *x4 = reinterpret_cast<const float4 *>(xn);
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int r = r0 + 2 * warp; r < r1; r += 2 * NW) {  // two vocabulary rows per warp pass
        const bool two = r + 1 < r1;
        const float4 *wa = reinterpret_cast<const float4 *>(p.wte + (size_t)r * E);
        const float4 *wb = reinterpret_cast<const float4 *>(p.wte + (size_t)(two ? r + 1 : r) * E);
        float sa = 0.f, sb = 0.f;
#pragma unroll 6
        for (int i = lane; i < E4; i += 32) {
          float4 xv = x4[i];
          sa += dot4(ldg_stream4(wa + i), xv);
          sb += dot4(ldg_stream4(wb + i), xv);
        }
        sa = warp_sum(sa);
        sb = warp_sum(sb);
        if (lane == 0) {
          p.logits[r] = sa;
          if (sa > best) { best = sa; bi = r; }
          if (two) {
            p.logits[r + 1] = sb;
            if (sb > best) { best = sb; bi = r + 1; }
          }
        }
      }
      if (lane == 0) { cand_v[warp] = best; cand_n[warp] = bi; }
      __syncthreads();
      if (tid == 0) {
        for (int w = 1; w < NW; w++)
          if (cand_v[w] > best || (cand_v[w] == best && cand_n[w] < bi)) { best = cand_v[w]; bi = cand_n[w]; }
        p.cand_val[blockIdx.x] = best;
        p.cand_idx[blockIdx.x] = bi;
      }
    }
    PK_TRACE(21);
    if (!grid_barrier(p, target)) { alive = false; break; }
    PK_TRACE(22);
    if (blockIdx.x == 0 && warp == 0) {  // lowest index wins ties (globals.js:66-74 with top_k = 1)
      float bv = -INFINITY;
      int bn = 0x7fffffff;
      for (int j = lane; j < (int)gridDim.x; j += 32) {
        float v = __ldcg(p.cand_val + j);
        int n = __ldcg(p.cand_idx + j);
        if (v > bv || (v == bv && n < bn)) { bv = v; bn = n; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int on = __shfl_xor_sync(0xffffffffu, bn, o);
        if (ov > bv || (ov == bv && on < bn)) { bv = ov; bn = on; }
      }
      if (lane == 0) {
        if (bn == 0x7fffffff) bn = 0;
        const int my_step = __ldcg(p.step);
        *p.next_id = (uint32_t)bn;
        if (p.out_ids) p.out_ids[my_step] = (uint32_t)bn;
        *p.pos = pos + 1;
        *p.step = my_step + 1;
      }
    }
    if (!grid_barrier(p, target)) { alive = false; break; }  // everyone sees the new id and position
    PK_TRACE(23);
  }
  // Leave no copy in flight into shared memory that is about to be released.
  if (tid == 0 && issued > blk) mbar_wait(&bars[blk & 1], (blk >> 1) & 1, 1u << 20);
}

}  // namespace wgpt
