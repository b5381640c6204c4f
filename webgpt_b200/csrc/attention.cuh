// Causal attention over a KV cache, replacing the reference's formatQ + fusedWeights + softmax +
// attentionValues chain (instructions.js:1101-1214, :593-666) without materialising the [H*T, T] score and
// probability matrices. Masked scores are -1e9 in the reference (:1176) and exp(-1e9 - max) is exactly 0 in
// f32, so skipping masked keys gives the same probabilities.
//
// Layout: Q rows [rows, ldq] with head h in columns [h*HS, (h+1)*HS); K and V rows for sequence s, position
// j at base + (s*kv_seq_stride + j)*ldkv, same column convention (the reference's [T, E] K/V buffers).
#pragma once
#include "common.cuh"

namespace wgpt {

// ------------------------------------------------------------------------------------------------
// Decode: one query row per sequence at position *pos (keys 0..*pos). grid = (H, n_seq, n_split): the CTAs along
// z share one (sequence, head) and each takes a slice of the positions. A CTA (8 warps) runs an online softmax
// over its slice. With n_split == 1 it writes the head's output; otherwise it writes an un-normalised partial
// (acc[HS], max, sum, 2 pad) to scratch, part[((seq*H + h)*n_split + split)*(HS+4)], and the consumer merges the
// slices in slice order while it stages its input (attn_merged_value below): no atomics, no extra pass.
// HBM-bound: reads 2*HS*4 bytes per position per head. Before the dependency wait the CTA asks for its slice of
// the cache in L2, computed from the position counter as it stands then (possibly one step old: the rows of
// earlier positions never change, so a stale bound only misses the newest row).
// Split-K partial tiles of the QKV product that feeds a decode attention (batched decode on the tensor cores):
// [slice][feature tile of 128][row = sequence][128], feature n of [0, 3E) = q | k | v. With FROM_QKV_PART the
// attention CTA is that product's second stage for its own (sequence, head): it adds the slices in order, adds the
// bias, keeps q, and writes the k and v rows of the newest position into the cache before it reads the cache.
struct QkvPartials {
  const float *part;
  const float *bias;  // [3E]
  int splits, n_rows, E;
};

template <int HS, bool FROM_QKV_PART = false>
__global__ void __launch_bounds__(256)
attn_decode_kernel(const float *__restrict__ q, int ldq, const float *__restrict__ kc, const float *__restrict__ vc,
                   int ldkv, size_t kv_seq_stride, float *__restrict__ out, int ldo, const int *__restrict__ pos,
                   float scale, float *__restrict__ part, QkvPartials qp = QkvPartials()) {
  constexpr int LPP = HS / 4;      // lanes per position (one float4 each)
  constexpr int G = 32 / LPP;      // positions per warp iteration
  constexpr int NW = 8;
  const int h = blockIdx.x, seq = blockIdx.y, split = blockIdx.z, n_split = gridDim.z, H = gridDim.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane / LPP, lig = lane % LPP;
  const float *kb = kc + (size_t)seq * kv_seq_stride * ldkv + h * HS;
  const float *vb = vc + (size_t)seq * kv_seq_stride * ldkv + h * HS;
  TRACE_BEGIN(3);
  trace(3, 0);
  pdl_launch_dependents();
  {
    const int Ls = __ldcg(pos) + 1;
    const int chunk_s = (Ls + n_split - 1) / n_split;
    const int beg_s = split * chunk_s, end_s = min(Ls, beg_s + chunk_s);
    constexpr int LPR = HS * 4 >= 128 ? HS * 4 / 128 : 1;  // 128-byte lines per row slice
    const int total = max(end_s - beg_s, 0) * 2 * LPR;
    for (int i = tid; i < total; i += 256) {
      const int r = beg_s + i / (2 * LPR), w = i % (2 * LPR);
      prefetch_line_l2((w < LPR ? kb : vb) + (size_t)r * ldkv + (w % LPR) * 32);
    }
  }
  pdl_wait();  // q, the cache row of this step and *pos come from earlier kernels
  trace(3, 1);
  const int L = __ldcg(pos) + 1;
  const int chunk = (L + n_split - 1) / n_split;
  const int beg = split * chunk, end = min(L, beg + chunk);
  float4 q4;
  if (FROM_QKV_PART) {
    __shared__ __align__(16) float s_q[HS];
    if (tid < 3 * HS) {
      const int sec = tid / HS, d = tid - sec * HS;
      const int n = sec * qp.E + h * HS + d;
      const int n_tiles = (3 * qp.E + 127) >> 7, nt = n >> 7;
      const float *p0 = qp.part + ((size_t)nt * qp.n_rows + seq) * 128 + (n & 127);
      const size_t zstride = (size_t)n_tiles * qp.n_rows * 128;
      float a = 0.f;
#pragma unroll 8
      for (int z = 0; z < qp.splits; z++) a += __ldcg(p0 + (size_t)z * zstride);
      a += qp.bias[n];
      if (sec == 0) s_q[d] = a;
      // the newest position's row; kc/vc are written here and read below by this same CTA only
      else if (sec == 1) const_cast<float *>(kb)[(size_t)(L - 1) * ldkv + d] = a;
      else const_cast<float *>(vb)[(size_t)(L - 1) * ldkv + d] = a;
    }
    __syncthreads();
    q4 = *reinterpret_cast<const float4 *>(&s_q[lig * 4]);
  } else {
    q4 = __ldcg(reinterpret_cast<const float4 *>(q + (size_t)seq * ldq + h * HS + lig * 4));
  }
  kb += lig * 4;
  vb += lig * 4;

  float m = -INFINITY, l = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  // The trip count is the same for every lane of the warp (the shuffles below name all 32 lanes); a group whose
  // position falls past the end of the slice runs the iteration with `valid` false and contributes nothing.
#pragma unroll 2
  for (int j0 = beg + warp * G; j0 < end; j0 += NW * G) {
    const int j = j0 + g;
    const bool valid = j < end;
    const int jj = valid ? j : end - 1;  // in-bounds address for the idle group
    float4 k4 = __ldcg(reinterpret_cast<const float4 *>(kb + (size_t)jj * ldkv));
    float4 v4 = __ldcg(reinterpret_cast<const float4 *>(vb + (size_t)jj * ldkv));
    float s = dot4(q4, k4);
#pragma unroll
    for (int o = LPP / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (valid) {
      s *= scale;
      float mn = fmaxf(m, s);
      float corr = expf(m - mn), p = expf(s - mn);  // m = -inf on the first key: corr = 0
      l = l * corr + p;
      acc.x = acc.x * corr + p * v4.x; acc.y = acc.y * corr + p * v4.y;
      acc.z = acc.z * corr + p * v4.z; acc.w = acc.w * corr + p * v4.w;
      m = mn;
    }
  }
  __syncwarp();
  // merge the G groups of the warp
#pragma unroll
  for (int o = LPP; o < 32; o <<= 1) {
    float mo = __shfl_xor_sync(0xffffffffu, m, o), lo = __shfl_xor_sync(0xffffffffu, l, o);
    float4 ao;
    ao.x = __shfl_xor_sync(0xffffffffu, acc.x, o); ao.y = __shfl_xor_sync(0xffffffffu, acc.y, o);
    ao.z = __shfl_xor_sync(0xffffffffu, acc.z, o); ao.w = __shfl_xor_sync(0xffffffffu, acc.w, o);
    float mn = fmaxf(m, mo);
    float c0 = (m == -INFINITY) ? 0.f : expf(m - mn), c1 = (mo == -INFINITY) ? 0.f : expf(mo - mn);
    l = l * c0 + lo * c1;
    acc.x = acc.x * c0 + ao.x * c1; acc.y = acc.y * c0 + ao.y * c1;
    acc.z = acc.z * c0 + ao.z * c1; acc.w = acc.w * c0 + ao.w * c1;
    m = mn;
  }
  trace(3, 2);
  __shared__ float sm_m[NW], sm_l[NW];
  __shared__ __align__(16) float sm_acc[NW][HS];
  if (g == 0) {
    *reinterpret_cast<float4 *>(&sm_acc[warp][lig * 4]) = acc;
    if (lig == 0) { sm_m[warp] = m; sm_l[warp] = l; }
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
    if (n_split == 1) {
      out[(size_t)seq * ldo + h * HS + tid] = a / ll;
    } else {
      float *my = part + ((size_t)(seq * H + h) * n_split + split) * (HS + 4);
      my[tid] = a;
      if (tid == 0) { my[HS] = mm; my[HS + 1] = ll; }
    }
  }
  trace(3, 4);
}

// Description of attention partials left by attn_decode_kernel with n_split > 1, for consumers that merge them
// while staging their input. part == nullptr: no merge, the input is read as is.
struct AttnPartials {
  const float *part;
  int n_split, H, hs;
};

// Elements c..c+3 (c % 4 == 0, all in one head) of the attention output of sequence `seq`: the slices'
// partials combined in slice order.
__device__ __forceinline__ float4 attn_merged_value4(const AttnPartials &ap, int seq, int c) {
  const int h = c / ap.hs, d = c - h * ap.hs;
  const int stride = ap.hs + 4;
  const float *p0 = ap.part + (size_t)(seq * ap.H + h) * ap.n_split * stride;
  float pm[8], pl[8];
  float4 pa[8];
#pragma unroll
  for (int r = 0; r < 8; r++) {
    if (r < ap.n_split) {
      const float *pr = p0 + (size_t)r * stride;
      pa[r] = __ldcg(reinterpret_cast<const float4 *>(pr + d));
      float2 ml = __ldcg(reinterpret_cast<const float2 *>(pr + ap.hs));
      pm[r] = ml.x;
      pl[r] = ml.y;
    } else {
      pm[r] = -INFINITY; pl[r] = 0.f; pa[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  float mm = pm[0];
#pragma unroll
  for (int r = 1; r < 8; r++) mm = fmaxf(mm, pm[r]);
  float ll = 0.f;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < 8; r++) {
    float c2 = (pm[r] == -INFINITY) ? 0.f : expf(pm[r] - mm);
    ll += pl[r] * c2;
    a.x += pa[r].x * c2; a.y += pa[r].y * c2; a.z += pa[r].z * c2; a.w += pa[r].w * c2;
  }
  return make_float4(a.x / ll, a.y / ll, a.z / ll, a.w / ll);
}

// Stand-alone merge for consumers that cannot merge on the fly: out[seq, c] for c in [0, H*hs).
__global__ void attn_merge_kernel(AttnPartials ap, float *__restrict__ out, int ldo) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.y, c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c < ap.H * ap.hs) *reinterpret_cast<float4 *>(out + (size_t)seq * ldo + c) = attn_merged_value4(ap, seq, c);
}

// ------------------------------------------------------------------------------------------------
// Prefill: n_tok new query rows per sequence at positions *pos .. *pos+n_tok-1, keys 0..position.
// grid = (ceil(n_tok/32), H, n_seq), 128 threads: a 32-query tile against 32-key tiles held in shared
// memory, online softmax per query row. Thread (qi = tid/4, sub = tid%4) owns keys sub, sub+4, ... of the
// tile for the scores and dims sub, sub+4, ... of the output.
constexpr size_t attn_prefill_smem_bytes(int hs) { return (size_t)(96 * (hs + 1) + 32 * 33) * sizeof(float); }

template <int HS>
__global__ void __launch_bounds__(128)
attn_prefill_kernel(const float *__restrict__ q, int ldq, const float *__restrict__ kc, const float *__restrict__ vc,
                    int ldkv, size_t kv_seq_stride, float *__restrict__ out, int ldo, int n_tok,
                    const int *__restrict__ pos, float scale) {
  constexpr int TQ = 32, TK = 32, LD = HS + 1, DPT = HS / 4;
  extern __shared__ float attn_smem[];  // attn_prefill_smem_bytes(HS): above 48 KB for HS = 128
  float (*Qs)[LD] = reinterpret_cast<float (*)[LD]>(attn_smem);
  float (*Ks)[LD] = reinterpret_cast<float (*)[LD]>(attn_smem + TQ * LD);
  float (*Vs)[LD] = reinterpret_cast<float (*)[LD]>(attn_smem + (TQ + TK) * LD);
  float (*Ps)[TK + 1] = reinterpret_cast<float (*)[TK + 1]>(attn_smem + (TQ + 2 * TK) * LD);
  const int h = blockIdx.y, seq = blockIdx.z, t0 = blockIdx.x * TQ;
  const int tid = threadIdx.x, qi = tid >> 2, sub = tid & 3;
  const int pos0 = pos ? *pos : 0;
  const int nq = min(TQ, n_tok - t0);
  const int my_t = t0 + min(qi, nq - 1);       // out-of-range query threads shadow the last valid row
  const int my_pos = pos0 + my_t;
  const int last_key = pos0 + t0 + nq - 1;     // newest key any query of this tile may see

  for (int i = tid; i < TQ * (HS / 4); i += 128) {
    int r = i / (HS / 4), c4 = (i % (HS / 4)) * 4;
    int t = t0 + min(r, nq - 1);
    float4 v = *reinterpret_cast<const float4 *>(q + ((size_t)seq * n_tok + t) * ldq + h * HS + c4);
    Qs[r][c4] = v.x; Qs[r][c4 + 1] = v.y; Qs[r][c4 + 2] = v.z; Qs[r][c4 + 3] = v.w;
  }
  const float *kb = kc + (size_t)seq * kv_seq_stride * ldkv + h * HS;
  const float *vb = vc + (size_t)seq * kv_seq_stride * ldkv + h * HS;

  float m = -INFINITY, l = 0.f, o[DPT];
#pragma unroll
  for (int d = 0; d < DPT; d++) o[d] = 0.f;

  for (int j0 = 0; j0 <= last_key; j0 += TK) {
    __syncthreads();
    for (int i = tid; i < TK * (HS / 4); i += 128) {
      int r = i / (HS / 4), c4 = (i % (HS / 4)) * 4;
      int j = min(j0 + r, last_key);
      float4 kv = *reinterpret_cast<const float4 *>(kb + (size_t)j * ldkv + c4);
      float4 vv = *reinterpret_cast<const float4 *>(vb + (size_t)j * ldkv + c4);
      Ks[r][c4] = kv.x; Ks[r][c4 + 1] = kv.y; Ks[r][c4 + 2] = kv.z; Ks[r][c4 + 3] = kv.w;
      Vs[r][c4] = vv.x; Vs[r][c4 + 1] = vv.y; Vs[r][c4 + 2] = vv.z; Vs[r][c4 + 3] = vv.w;
    }
    __syncthreads();
    float s[TK / 4];
#pragma unroll
    for (int kk = 0; kk < TK / 4; kk++) s[kk] = 0.f;
    for (int d = 0; d < HS; d++) {
      float qv = Qs[qi][d];
#pragma unroll
      for (int kk = 0; kk < TK / 4; kk++) s[kk] += qv * Ks[sub + 4 * kk][d];
    }
    float tmax = -INFINITY;
#pragma unroll
    for (int kk = 0; kk < TK / 4; kk++) {
      int j = j0 + sub + 4 * kk;
      s[kk] = (j <= my_pos) ? s[kk] * scale : -INFINITY;
      tmax = fmaxf(tmax, s[kk]);
    }
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    float mn = fmaxf(m, tmax);  // key j0 <= my_pos is visible in every processed tile? no: guard below
    float corr = (m == -INFINITY) ? 0.f : expf(m - mn);
    float psum = 0.f;
#pragma unroll
    for (int kk = 0; kk < TK / 4; kk++) {
      float p = (s[kk] == -INFINITY) ? 0.f : expf(s[kk] - mn);
      Ps[qi][sub + 4 * kk] = p;
      psum += p;
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    if (mn != -INFINITY) {
      l = l * corr + psum;
      m = mn;
    }
    __syncwarp();
#pragma unroll
    for (int d = 0; d < DPT; d++) o[d] *= corr;
    for (int k = 0; k < TK; k++) {
      float p = Ps[qi][k];
#pragma unroll
      for (int d = 0; d < DPT; d++) o[d] += p * Vs[k][sub + 4 * d];
    }
  }
  if (qi < nq) {
    float *op = out + ((size_t)seq * n_tok + t0 + qi) * ldo + h * HS;
    float inv = 1.f / l;
#pragma unroll
    for (int d = 0; d < DPT; d++) op[sub + 4 * d] = o[d] * inv;
  }
}

// ------------------------------------------------------------------------------------------------
// Prefill for head size 64 (every GPT-2 size and the char model), register-tiled: a CTA of 256 threads takes 64
// query rows against key tiles of 64, thread (ty, tx) of a 16 x 16 grid owns queries ty, ty+16, ty+32, ty+48 and
// keys tx, tx+16, tx+32, tx+48 of the tile for the scores, and the same queries with output dims 4tx..4tx+3 for
// the values. Q, K, V and the probabilities sit in shared memory in their natural row layout with rows padded to
// 68 floats; every inner step is 128-bit loads (the four keys of a lane are 16 rows apart, so a quarter-warp's
// eight addresses fall into different banks): 64 multiply-adds per eight loads, against one per load in the
// 32 x 32 kernel above. Online softmax per query row across tiles; the 16 lanes that share a row combine their
// maxima and sums with shuffles. Same mathematics as the chain it replaces (formatQ, fusedWeights with the causal
// mask, softmax, attentionValues: instructions.js:1101-1214, :593-666); masked keys contribute exactly zero.
constexpr int kAttn64Tile = 64, kAttn64Ld = 68;
constexpr size_t attn_prefill64_smem_bytes() { return (size_t)4 * kAttn64Tile * kAttn64Ld * sizeof(float); }

__global__ void __launch_bounds__(256)
attn_prefill64_kernel(const float *__restrict__ q, int ldq, const float *__restrict__ kc, const float *__restrict__ vc,
                      int ldkv, size_t kv_seq_stride, float *__restrict__ out, int ldo, int n_tok,
                      const int *__restrict__ pos, float scale) {
  constexpr int HS = 64, T = kAttn64Tile, LD = kAttn64Ld;
  extern __shared__ __align__(16) float attn_smem[];
  float *Qs = attn_smem, *Ks = Qs + T * LD, *Vs = Ks + T * LD, *Ps = Vs + T * LD;
  const int h = blockIdx.y, seq = blockIdx.z, t0 = blockIdx.x * T;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int pos0 = pos ? *pos : 0;
  const int nq = min(T, n_tok - t0);
  const int last_key = pos0 + t0 + nq - 1;  // newest key any query of this tile may see
  int my_pos[4];
#pragma unroll
  for (int i = 0; i < 4; i++) my_pos[i] = pos0 + t0 + min(ty + 16 * i, nq - 1);  // rows past the end shadow the last one

  for (int idx = tid; idx < T * (HS / 4); idx += 256) {
    const int r = idx >> 4, c4 = (idx & 15) * 4;
    const int t = t0 + min(r, nq - 1);
    *reinterpret_cast<float4 *>(Qs + r * LD + c4) =
        *reinterpret_cast<const float4 *>(q + ((size_t)seq * n_tok + t) * ldq + h * HS + c4);
  }
  const float *kb = kc + (size_t)seq * kv_seq_stride * ldkv + h * HS;
  const float *vb = vc + (size_t)seq * kv_seq_stride * ldkv + h * HS;

  float m[4], l[4], o[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int d = 0; d < 4; d++) o[i][d] = 0.f;
  }

  for (int j0 = 0; j0 <= last_key; j0 += T) {
    __syncthreads();  // the previous tile's K, V and P are no longer read
    for (int idx = tid; idx < T * (HS / 4); idx += 256) {
      const int r = idx >> 4, c4 = (idx & 15) * 4;
      const int j = min(j0 + r, last_key);
      *reinterpret_cast<float4 *>(Ks + r * LD + c4) = *reinterpret_cast<const float4 *>(kb + (size_t)j * ldkv + c4);
      *reinterpret_cast<float4 *>(Vs + r * LD + c4) = *reinterpret_cast<const float4 *>(vb + (size_t)j * ldkv + c4);
    }
    __syncthreads();
    // ---- scores of 4 queries x 4 keys
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int k = 0; k < 4; k++) s[i][k] = 0.f;
#pragma unroll 4
    for (int d = 0; d < HS; d += 4) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) qv[i] = *reinterpret_cast<const float4 *>(Qs + (ty + 16 * i) * LD + d);
#pragma unroll
      for (int k = 0; k < 4; k++) kv[k] = *reinterpret_cast<const float4 *>(Ks + (tx + 16 * k) * LD + d);
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int k = 0; k < 4; k++) s[i][k] += dot4(qv[i], kv[k]);
    }
    // ---- online softmax per query row (the 16 lanes with this ty share the row)
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float tmax = -INFINITY;
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const int j = j0 + tx + 16 * k;
        s[i][k] = (j <= my_pos[i]) ? s[i][k] * scale : -INFINITY;
        tmax = fmaxf(tmax, s[i][k]);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
      const float mn = fmaxf(m[i], tmax);
      const float corr = (m[i] == -INFINITY) ? 0.f : expf(m[i] - mn);
      float psum = 0.f;
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const float p = (s[i][k] == -INFINITY) ? 0.f : expf(s[i][k] - mn);
        Ps[(ty + 16 * i) * LD + tx + 16 * k] = p;
        psum += p;
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
      if (mn != -INFINITY) {
        l[i] = l[i] * corr + psum;
        m[i] = mn;
      }
#pragma unroll
      for (int d = 0; d < 4; d++) o[i][d] *= corr;
    }
    __syncthreads();  // the probabilities of the tile are complete
    // ---- values: 4 queries x 4 output dims
#pragma unroll 4
    for (int k = 0; k < T; k += 4) {
      float4 pv[4], vv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) pv[i] = *reinterpret_cast<const float4 *>(Ps + (ty + 16 * i) * LD + k);
#pragma unroll
      for (int kk = 0; kk < 4; kk++) vv[kk] = *reinterpret_cast<const float4 *>(Vs + (k + kk) * LD + 4 * tx);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        o[i][0] += pv[i].x * vv[0].x + pv[i].y * vv[1].x + pv[i].z * vv[2].x + pv[i].w * vv[3].x;
        o[i][1] += pv[i].x * vv[0].y + pv[i].y * vv[1].y + pv[i].z * vv[2].y + pv[i].w * vv[3].y;
        o[i][2] += pv[i].x * vv[0].z + pv[i].y * vv[1].z + pv[i].z * vv[2].z + pv[i].w * vv[3].z;
        o[i][3] += pv[i].x * vv[0].w + pv[i].y * vv[1].w + pv[i].z * vv[2].w + pv[i].w * vv[3].w;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int r = ty + 16 * i;
    if (r < nq) {
      const float inv = 1.f / l[i];
      *reinterpret_cast<float4 *>(out + ((size_t)seq * n_tok + t0 + r) * ldo + h * HS + 4 * tx) =
          make_float4(o[i][0] * inv, o[i][1] * inv, o[i][2] * inv, o[i][3] * inv);
    }
  }
}

}  // namespace wgpt

namespace wgpt {

// ------------------------------------------------------------------------------------------------
// Prefill for head size 64 on the tensor cores (warp-level mma.sync.m16n8k8, TF32 inputs, FP32 accumulation), used
// when the device computes products in TF32 or 3xTF32; the FP32 mode keeps attn_prefill64_kernel. A CTA of four
// warps takes 64 query rows (16 per warp) against key tiles of 64 held in shared memory; scores, online softmax and
// the probabilities never leave registers (the accumulator fragment of the score product is re-arranged into the
// A fragment of the value product with shuffles inside each quad of lanes). X3: every operand is split into
// hi = its top 19 bits and lo = x - hi, and each product is hi*hi + hi*lo + lo*hi, as in the GEMM kernels.
// Same mathematics as attn_prefill64_kernel (instructions.js:1101-1214, :593-666); masked keys contribute zero.
constexpr int kAttnMmaKLd = 68, kAttnMmaVLd = 72;  // row strides (floats) that keep the fragment loads conflict-free

__device__ __forceinline__ void mma_tf32_16x8x8(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t tf32_hi_bits(float x) { return __float_as_uint(x) & 0xFFFFE000u; }
__device__ __forceinline__ uint32_t tf32_lo_bits(float x) {
  return __float_as_uint(x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u));
}

template <bool X3>
__global__ void __launch_bounds__(128)
attn_prefill64_mma_kernel(const float *__restrict__ q, int ldq, const float *__restrict__ kc,
                          const float *__restrict__ vc, int ldkv, size_t kv_seq_stride, float *__restrict__ out,
                          int ldo, int n_tok, const int *__restrict__ pos, float scale) {
  constexpr int HS = 64, T = 64, KLD = kAttnMmaKLd, VLD = kAttnMmaVLd;
  __shared__ __align__(16) float Ks[T * KLD];
  __shared__ __align__(16) float Vs[T * VLD];
  const int h = blockIdx.y, seq = blockIdx.z, t0 = blockIdx.x * T;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int pos0 = pos ? *pos : 0;
  const int nq = min(T, n_tok - t0);
  const int last_key = pos0 + t0 + nq - 1;  // newest key any query of this tile may see
  const int r0 = 16 * warp + g, r1 = r0 + 8;  // this lane's two query rows inside the tile
  const int p0 = pos0 + t0 + min(r0, nq - 1), p1 = pos0 + t0 + min(r1, nq - 1);  // rows past the end shadow the last
  const int warp_last = pos0 + t0 + min(16 * warp + 15, nq - 1);

  // ---- Q fragments (A operand of the score product), staged through the K buffer
  for (int idx = tid; idx < T * (HS / 4); idx += 128) {
    const int r = idx >> 4, c4 = (idx & 15) * 4;
    const int tq = t0 + min(r, nq - 1);
    *reinterpret_cast<float4 *>(Ks + r * KLD + c4) =
        *reinterpret_cast<const float4 *>(q + ((size_t)seq * n_tok + tq) * ldq + h * HS + c4);
  }
  __syncthreads();
  uint32_t qh[8][4], ql[X3 ? 8 : 1][4];
#pragma unroll
  for (int ks = 0; ks < 8; ks++) {
    const float x0 = Ks[r0 * KLD + 8 * ks + t], x1 = Ks[r1 * KLD + 8 * ks + t];
    const float x2 = Ks[r0 * KLD + 8 * ks + t + 4], x3 = Ks[r1 * KLD + 8 * ks + t + 4];
    qh[ks][0] = tf32_hi_bits(x0); qh[ks][1] = tf32_hi_bits(x1); qh[ks][2] = tf32_hi_bits(x2); qh[ks][3] = tf32_hi_bits(x3);
    if (X3) {
      ql[ks][0] = tf32_lo_bits(x0); ql[ks][1] = tf32_lo_bits(x1); ql[ks][2] = tf32_lo_bits(x2); ql[ks][3] = tf32_lo_bits(x3);
    }
  }
  const float *kb = kc + (size_t)seq * kv_seq_stride * ldkv + h * HS;
  const float *vb = vc + (size_t)seq * kv_seq_stride * ldkv + h * HS;

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; j++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[j][e] = 0.f;

  for (int j0 = 0; j0 <= last_key; j0 += T) {
    __syncthreads();  // the previous tile (or the staged Q) is no longer read
    for (int idx = tid; idx < T * (HS / 4); idx += 128) {
      const int r = idx >> 4, c4 = (idx & 15) * 4;
      const int j = min(j0 + r, last_key);
      *reinterpret_cast<float4 *>(Ks + r * KLD + c4) = *reinterpret_cast<const float4 *>(kb + (size_t)j * ldkv + c4);
      *reinterpret_cast<float4 *>(Vs + r * VLD + c4) = *reinterpret_cast<const float4 *>(vb + (size_t)j * ldkv + c4);
    }
    __syncthreads();
    if (j0 > warp_last) continue;  // every key of the tile is masked for this warp's rows (same for the whole warp)

    // ---- scores: 16 rows x 64 keys as eight 16x8 accumulators
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++) {
#pragma unroll
      for (int e = 0; e < 4; e++) s[j][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ks++) {
        const float k0 = Ks[(8 * j + g) * KLD + 8 * ks + t], k1 = Ks[(8 * j + g) * KLD + 8 * ks + t + 4];
        const uint32_t kh0 = tf32_hi_bits(k0), kh1 = tf32_hi_bits(k1);
        mma_tf32_16x8x8(s[j], qh[ks], kh0, kh1);
        if (X3) {
          mma_tf32_16x8x8(s[j], qh[ks], tf32_lo_bits(k0), tf32_lo_bits(k1));
          mma_tf32_16x8x8(s[j], ql[ks], kh0, kh1);
        }
      }
    }
    // ---- online softmax of rows r0 (elements 0, 1) and r1 (elements 2, 3); key of element e: j0 + 8j + 2t + (e & 1)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; j++) {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int key = j0 + 8 * j + 2 * t + (e & 1);
        const int pq = e < 2 ? p0 : p1;
        s[j][e] = key <= pq ? s[j][e] * scale : -INFINITY;
      }
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float c0 = (m0 == -INFINITY) ? 0.f : expf(m0 - mn0), c1 = (m1 == -INFINITY) ? 0.f : expf(m1 - mn1);
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      s[j][0] = (s[j][0] == -INFINITY) ? 0.f : expf(s[j][0] - mn0);
      s[j][1] = (s[j][1] == -INFINITY) ? 0.f : expf(s[j][1] - mn0);
      s[j][2] = (s[j][2] == -INFINITY) ? 0.f : expf(s[j][2] - mn1);
      s[j][3] = (s[j][3] == -INFINITY) ? 0.f : expf(s[j][3] - mn1);
      ps0 += s[j][0] + s[j][1];
      ps1 += s[j][2] + s[j][3];
    }
    if (mn0 != -INFINITY) { l0 = l0 * c0 + ps0; m0 = mn0; }  // l holds this lane's share of the row sum
    if (mn1 != -INFINITY) { l1 = l1 * c1 + ps1; m1 = mn1; }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1;
    }
    // ---- values: the probabilities of keys 8ks..8ks+7 become the A fragment of k-step ks
    const int src_lo = (lane & ~3) | (t >> 1), src_hi = src_lo + 2;
    const bool odd = (t & 1) != 0;
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
      // element (row, key 8ks + c) sits in the lane of the quad with 2*tig == c & ~1, as element c & 1 (row r0) / 2 + (c & 1) (row r1)
      const float e0a = __shfl_sync(0xffffffffu, s[ks][0], src_lo), e1a = __shfl_sync(0xffffffffu, s[ks][1], src_lo);
      const float e2a = __shfl_sync(0xffffffffu, s[ks][2], src_lo), e3a = __shfl_sync(0xffffffffu, s[ks][3], src_lo);
      const float e0b = __shfl_sync(0xffffffffu, s[ks][0], src_hi), e1b = __shfl_sync(0xffffffffu, s[ks][1], src_hi);
      const float e2b = __shfl_sync(0xffffffffu, s[ks][2], src_hi), e3b = __shfl_sync(0xffffffffu, s[ks][3], src_hi);
      const float a0 = odd ? e1a : e0a, a1 = odd ? e3a : e2a;  // keys 8ks + t of rows r0, r1
      const float a2 = odd ? e1b : e0b, a3 = odd ? e3b : e2b;  // keys 8ks + t + 4
      uint32_t ph[4] = {tf32_hi_bits(a0), tf32_hi_bits(a1), tf32_hi_bits(a2), tf32_hi_bits(a3)};
      uint32_t pl[4] = {0u, 0u, 0u, 0u};
      if (X3) { pl[0] = tf32_lo_bits(a0); pl[1] = tf32_lo_bits(a1); pl[2] = tf32_lo_bits(a2); pl[3] = tf32_lo_bits(a3); }
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const float v0 = Vs[(8 * ks + t) * VLD + 8 * j + g], v1 = Vs[(8 * ks + t + 4) * VLD + 8 * j + g];
        const uint32_t vh0 = tf32_hi_bits(v0), vh1 = tf32_hi_bits(v1);
        mma_tf32_16x8x8(o[j], ph, vh0, vh1);
        if (X3) {
          mma_tf32_16x8x8(o[j], ph, tf32_lo_bits(v0), tf32_lo_bits(v1));
          mma_tf32_16x8x8(o[j], pl, vh0, vh1);
        }
      }
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = 1.f / l0, i1 = 1.f / l1;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    if (r0 < nq)
      *reinterpret_cast<float2 *>(out + ((size_t)seq * n_tok + t0 + r0) * ldo + h * HS + 8 * j + 2 * t) =
          make_float2(o[j][0] * i0, o[j][1] * i0);
    if (r1 < nq)
      *reinterpret_cast<float2 *>(out + ((size_t)seq * n_tok + t0 + r1) * ldo + h * HS + 8 * j + 2 * t) =
          make_float2(o[j][2] * i1, o[j][3] * i1);
  }
}

}  // namespace wgpt
