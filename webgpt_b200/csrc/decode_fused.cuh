// Single-sequence decode with two kernels per transformer block instead of five.
//
// The reference runs a block as LayerNorm, three projections, the attention chain, the output projection, a
// residual add, LayerNorm, two MLP products with a GELU between them and another residual add
// (model.js:123-210), each its own pass. At one row per pass the arithmetic is nothing and the cost of a pass is
// its dependency hand-off, so the block is cut where the data flow forces a grid-wide exchange and nowhere else:
//
//  attn_block_kernel  : one cluster of CS CTAs per head. Each CTA first sums its share of the columns of the
//                       previous block's partial results into the residual stream and hands it to the others
//                       through distributed shared memory; then LayerNorm, the head's q/k/v columns (each CTA
//                       HS/CS of each), exchange of q and the new k, v rows, attention over the cache (the CS
//                       CTAs split the positions), merge, and this head's share of the output projection as a
//                       partial result [H][E] over heads.
//  mlp_block_kernel   : sums the H partial results (+ bias + residual), LayerNorm, and for this CTA's slice of
//                       the 4E hidden units: up-projection, GELU and immediately those units' rows of the
//                       down-projection, as a partial result [CTAs][E].
//  finish_row_kernel  : after the last block, sums the MLP partial results into the residual stream for ln_f.
//
// Every sum of partial results runs in a fixed order (no float atomics), so results are reproducible. Weights
// arrive in shared memory by bulk asynchronous copies issued before the dependency wait, i.e. while the previous
// kernel is still running; the attention kernel re-uses its q/k/v weight buffer for its slice of the output
// projection, fetched while the attention itself runs. Every copy has one destination CTA; remote shared memory
// is only ever written with plain st.shared::cluster stores between cluster barriers.
#pragma once
#include "common.cuh"
#include "matmul.cuh"

namespace wgpt {

// Cluster barrier (hardware; threads that have exited count as arrived). release/acquire order the
// st.shared::cluster stores before it against the reads after it.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Address of this CTA's shared-memory location p in CTA `cta` of the cluster.
__device__ __forceinline__ uint32_t dsmem_addr(const void *p, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr(p)), "r"(cta));
  return r;
}
__device__ __forceinline__ void dsmem_st(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void dsmem_st4(uint32_t addr, float4 v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
// Orders this thread's earlier generic-proxy accesses to shared memory before later asynchronous-proxy (bulk
// copy) writes to it.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

// Sums over the rows of a row-major float4 matrix the previous kernel wrote (partial results, one row per
// producer). Two things decide what this costs. A round trip to L2 for lines another SM has just written takes
// more than a microsecond, so a thread issues every load it will need in one batch before the first add. And a
// warp-wide load is served one cache line at a time, so the lanes of a warp read neighbouring columns of the same
// row. Rows are added in a fixed order everywhere, so results are reproducible.
//
// warp_rows_partial: lane = column (< ncols <= 32), warp w of NW holds rows w, w+NW, ... (at most MAXR of them);
// returns this warp's sum for the lane's column. The caller adds the NW warps' results in warp order.
// L2 load whose position in the instruction stream the compiler keeps (it would otherwise sink each load of a
// batch down to its add to save registers, which serialises the round trips).
__device__ __forceinline__ float4 ldcg_pinned(const float4 *p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
// Requires the four values to be in registers here, i.e. the loads that produce them to have been issued.
__device__ __forceinline__ void pin4(const float4 &a) {
  asm volatile("" ::"f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w));
}

template <int NW, int MAXR>
__device__ __forceinline__ float4 warp_rows_partial(const float4 *__restrict__ base, int ncols, size_t stride4,
                                                    int n_rows, int warp, int lane) {
  float4 v[MAXR];
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  if (n_rows <= 0) return a;  // same for the whole CTA
  const int cc = lane < ncols ? lane : 0;
#pragma unroll
  for (int k = 0; k < MAXR; k++) {  // out-of-range slots read row 0 and are dropped below: no branch between loads
    const int r = warp + NW * k;
    v[k] = ldcg_pinned(base + (size_t)(r < n_rows ? r : 0) * stride4 + cc);
  }
#pragma unroll
  for (int k = 0; k < MAXR; k++) pin4(v[k]);
#pragma unroll
  for (int k = 0; k < MAXR; k++)
    if (lane < ncols && warp + NW * k < n_rows) a = add4(a, v[k]);
  return a;
}
// halfwarp_rows_sum: lanes 0..15 and 16..31 of a warp are the same 16 columns (col16 = lane & 15) and take the even
// and the odd rows (at most MAXR each); the two halves are combined with one shuffle. Every lane of the warp must
// call it; returns the sum of all rows for the lane's column (the same value in both halves).
// `between` runs once the loads have been issued and before the first of them is waited for.
template <int MAXR, typename Between>
__device__ __forceinline__ float4 halfwarp_rows_sum(const float4 *__restrict__ base, int ncols, size_t stride4,
                                                    int n_rows, int lane, Between between) {
  const int c = lane & 15, half = lane >> 4;
  float4 v[MAXR];
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  if (n_rows > 0 && ncols > 0) {  // same for the whole warp
    const int cc = c < ncols ? c : 0;
#pragma unroll
    for (int k = 0; k < MAXR; k++) {  // out-of-range slots read row 0 and are dropped below
      const int r = half + 2 * k;
      v[k] = ldcg_pinned(base + (size_t)(r < n_rows ? r : 0) * stride4 + cc);
    }
    between();
#pragma unroll
    for (int k = 0; k < MAXR; k++) pin4(v[k]);
#pragma unroll
    for (int k = 0; k < MAXR; k++)
      if (c < ncols && half + 2 * k < n_rows) a = add4(a, v[k]);
  } else {
    between();
  }
  a.x += __shfl_xor_sync(0xffffffffu, a.x, 16);
  a.y += __shfl_xor_sync(0xffffffffu, a.y, 16);
  a.z += __shfl_xor_sync(0xffffffffu, a.z, 16);
  a.w += __shfl_xor_sync(0xffffffffu, a.w, 16);
  return a;
}
constexpr int kAttnSumRows = 10;  // attn_block_kernel / finish_row_kernel: partial rows <= 10 * 8 warps
constexpr int kMlpSumRows = 8;    // mlp_block_kernel: partial rows (heads) <= 2 * 8

// Asks for a contiguous block in L2, in pieces of at most 16 KB.
__device__ __forceinline__ void prefetch_l2_block(const void *src, uint32_t bytes) {
  for (uint32_t off = 0; off < bytes; off += 16384u)
    prefetch_l2(reinterpret_cast<const char *>(src) + off, min(16384u, bytes - off));
}
// Bulk copy of a contiguous block into shared memory in pieces of at most 16 KB, all counted on one mbarrier.
__device__ __forceinline__ void bulk_g2s_block(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  for (uint32_t off = 0; off < bytes; off += 16384u)
    bulk_g2s(reinterpret_cast<char *>(dst) + off, reinterpret_cast<const char *>(src) + off, min(16384u, bytes - off), bar);
}

constexpr int kAttnBlockThreads = 256;
constexpr int kMlpBlockThreads = 512;
constexpr uint32_t kFusedPolls = 1u << 20;

// Device layout of one (head, cluster rank) weight block of attn_block_kernel, contiguous:
//   3*HS/CS rows of E floats: the rank's q columns, then k, then v (rows of the [3E, E] transposed c_attn weight)
//   HS rows of E/CS floats  : rows h*HS .. h*HS+HS-1, columns rank*E/CS .. of the [E, E] c_proj weight in the
//                             reference's [K, N] orientation
// fused_attn_relayout_kernel fills it once at load.
__global__ void fused_attn_relayout_kernel(const float *__restrict__ wqkv_t, const float *__restrict__ wo_t,
                                           float *__restrict__ blk, int E, int H, int HS, int CS) {
  const int nq = HS / CS, ncolA = E / CS;
  const size_t blk_floats = (size_t)3 * nq * E + (size_t)HS * ncolA;
  const size_t total = blk_floats * H * CS;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t b = i / blk_floats, o = i - b * blk_floats;
    const int h = (int)(b / CS), r = (int)(b % CS);
    float v;
    if (o < (size_t)3 * nq * E) {
      const int row = (int)(o / E), k = (int)(o % E);
      const int sec = row / nq, j = row % nq;
      v = wqkv_t[((size_t)sec * E + h * HS + r * nq + j) * E + k];
    } else {
      const size_t o2 = o - (size_t)3 * nq * E;
      const int d = (int)(o2 / ncolA), n = (int)(o2 % ncolA);
      v = wo_t[((size_t)r * ncolA + n) * E + h * HS + d];
    }
    blk[i] = v;
  }
}

struct AttnBlockParams {
  // residual stream entering the block: x = xin + bias_in + sum of part_in rows, or (ids != nullptr) the
  // embedding wte[ids[0]] + wpe[pos] (instructions.js:790-827)
  const float *xin;
  const float *part_in;  // [n_part][E]
  const float *bias_in;  // [E] or nullptr
  int n_part;
  const uint32_t *ids;
  const float *wte, *wpe;
  int vocab;
  float *x_out;          // [E]: x as computed here, for the MLP kernel's residual
  const float *gamma, *beta;
  const float *wblk;     // [H][CS][blk_floats]
  size_t blk_floats;
  const float *bqkv;     // [3E]
  float *kc, *vc;        // this block's cache rows [n_ctx][E]
  float *part_out;       // [H][E]
  const int *pos;
  int E, H;
  float scale;
  int proj_parts;        // slices of the head dimension in the projection step
  int red_floats;        // scratch floats (multiple of 4)
  const char *pf_a, *pf_b;  // for the clusters beyond the heads: the next kernel's two weight arrays (pf_bytes each)
  unsigned int pf_bytes;
  int *err;
};

template <int HS, int CS>
constexpr size_t attn_block_smem_floats(int E, int red_floats) {
  return (size_t)3 * (HS / CS) * E + (size_t)E + red_floats + 3 * HS + CS * (HS + 4) + HS + 8;
}

template <int HS, int CS>
__global__ void __launch_bounds__(kAttnBlockThreads)
attn_block_kernel(AttnBlockParams p) {
  constexpr int NT = kAttnBlockThreads, NW = NT / 32;
  constexpr int NQ = HS / CS;   // q columns (and k, and v) this CTA computes
  constexpr int NC = 3 * NQ;    // weight rows staged
  constexpr int NB = (NC + NW - 1) / NW;  // columns per warp
  constexpr int LPP = HS / 4;   // lanes per cache position (one float4 each)
  constexpr int G = 32 / LPP;   // positions per warp iteration
  constexpr int MS = HS + 4;    // stride of a merge record: acc[HS], max, sum, pad
  extern __shared__ __align__(128) float smem[];
  const int E = p.E, E4 = E >> 2;
  const int ncolA = E / CS, ncol4 = ncolA >> 2;
  float *wbuf = smem;                       // q/k/v weight rows, later the projection slice [HS][ncolA]
  float *xs = wbuf + (size_t)NC * E;        // residual stream (filled by all CTAs of the cluster), then normalised
  float *hn = xs;                           // in place: every thread holds its elements in registers in between
  float *red = xs + E;
  float *qfull = red + p.red_floats;        // filled by all CTAs of the cluster
  float *knew = qfull + HS, *vnew = knew + HS;
  float *mrg = vnew + HS;                   // [CS][MS], filled by all CTAs of the cluster
  float *osm = mrg + CS * MS;               // attention output of the head
  uint64_t *bars = reinterpret_cast<uint64_t *>(osm + HS);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int h = blockIdx.x / CS;
  if (h >= p.H) {
    // Clusters beyond the heads (the heads' clusters leave a third of the SMs idle) do nothing but ask for the next
    // kernel's weights in L2 once the previous kernel has completed: this kernel's own weights have landed by then
    // and everything it still reads comes from L2, so HBM is otherwise idle while it runs, and the MLP kernel's bulk
    // copies then find their 19 MB in L2. Two clusters measured best (-4.4 us per token); one is too few threads to
    // issue the requests quickly and holds the kernel up (+50 us), four or six gain less.
    pdl_wait();
    const unsigned int n_ext = gridDim.x - (unsigned int)p.H * CS, e = blockIdx.x - (unsigned int)p.H * CS;
    const unsigned int per16 = (p.pf_bytes >> 4);
    for (int arr = 0; arr < 2; arr++) {
      const char *base = arr == 0 ? p.pf_a : p.pf_b;
      if (base == nullptr) continue;
      const unsigned int beg = (unsigned int)(((unsigned long long)per16 * e) / n_ext);
      const unsigned int end = (unsigned int)(((unsigned long long)per16 * (e + 1)) / n_ext);
      for (unsigned int o = beg + 1024u * tid; o < end; o += 1024u * NT)
        prefetch_l2(base + ((size_t)o << 4), min(end - o, 1024u) << 4);
    }
    return;
  }
  const float *blk = p.wblk + ((size_t)h * CS + rank) * p.blk_floats;
  const int col0 = (int)rank * ncolA;       // first residual/projection column of this CTA
  TRACE_BEGIN(8);
  trace(8, 0);

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_expect_tx(&bars[0], (uint32_t)NC * (uint32_t)E * 4u);
  }
  // constants of the model, fetched ahead of the dependency wait
  float bias_c[NB];
#pragma unroll
  for (int b = 0; b < NB; b++) {
    const int c = warp + NW * b;
    bias_c[b] = 0.f;
    if (c < NC) bias_c[b] = p.bqkv[(c / NQ) * E + h * HS + (int)rank * NQ + (c % NQ)];
  }
  float4 g_first = make_float4(0.f, 0.f, 0.f, 0.f), b_first = g_first;
  if (tid < E4) {
    g_first = reinterpret_cast<const float4 *>(p.gamma)[tid];
    b_first = reinterpret_cast<const float4 *>(p.beta)[tid];
  }
  const float *kb = p.kc + h * HS, *vb = p.vc + h * HS;
  {  // ask for this CTA's slice of the cache in L2, from the position as it stands now (possibly one step old)
    const int Ls = __ldcg(p.pos) + 1;
    const int chunk_s = (Ls + CS - 1) / CS;
    const int beg_s = (int)rank * chunk_s, end_s = min(Ls, beg_s + chunk_s);
    constexpr int LPR = HS * 4 >= 128 ? HS * 4 / 128 : 1;  // 128-byte lines per row slice
    const int total = max(end_s - beg_s, 0) * 2 * LPR;
    for (int i = tid; i < total; i += NT) {
      const int r = beg_s + i / (2 * LPR), w = i % (2 * LPR);
      prefetch_line_l2((w < LPR ? kb : vb) + (size_t)r * E + (w % LPR) * 32);
    }
  }
  cluster_arrive();  // pairs with the wait below: every CTA of the cluster is running before any remote store
  if (tid == 0) {  // the q/k/v weights into shared memory, the projection slice towards L2
    bulk_g2s_block(wbuf, blk, (uint32_t)NC * (uint32_t)E * 4u, &bars[0]);
    prefetch_l2_block(blk + (size_t)NC * E, (uint32_t)HS * (uint32_t)ncolA * 4u);
  }
  pdl_wait();
  const int pos = __ldcg(p.pos);
  trace(8, 1);

  // Global stores are held back until after the last cluster barrier: a releasing barrier arrival waits for the
  // acknowledgement of every store issued before it, and with the next kernel's weight burst in flight towards the
  // same SM such an acknowledgement took about 3 us.
  float4 x_keep = make_float4(0.f, 0.f, 0.f, 0.f);
  // ---- the residual stream: this CTA sums columns [col0, col0 + ncolA) and hands them to the whole cluster.
  //      One group of 16 lanes per float4 column; lane 0 of the group adds the row the partial results belong to.
  {
    const float4 part = warp_rows_partial<NW, kAttnSumRows>(reinterpret_cast<const float4 *>(p.part_in + col0), ncol4,
                                                            (size_t)E4, p.n_part, warp, lane);
    float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (tid < ncol4) {
      if (p.ids != nullptr) {
        const uint32_t id = __ldcg(p.ids);
        if (id >= (uint32_t)p.vocab) {
          if (tid == 0 && blockIdx.x == 0) atomicExch(p.err, 1);  // the row stays zero, as in embed_kernel
        } else {
          x0 = add4(reinterpret_cast<const float4 *>(p.wte + (size_t)id * E + col0)[tid],
                    reinterpret_cast<const float4 *>(p.wpe + (size_t)pos * E + col0)[tid]);
        }
      } else {
        x0 = __ldcg(reinterpret_cast<const float4 *>(p.xin + col0) + tid);
      }
      if (p.bias_in) x0 = add4(x0, reinterpret_cast<const float4 *>(p.bias_in + col0)[tid]);
    }
    if (lane < ncol4) reinterpret_cast<float4 *>(red)[warp * 32 + lane] = part;
    __syncthreads();
    cluster_wait();
    if (tid < ncol4) {
      float4 x = x0;
#pragma unroll
      for (int w = 0; w < NW; w++) x = add4(x, reinterpret_cast<const float4 *>(red)[w * 32 + tid]);
#pragma unroll
      for (int cc = 0; cc < CS; cc++) dsmem_st4(dsmem_addr(xs + col0 + 4 * tid, (uint32_t)cc), x);
      x_keep = x;
    }
  }
  trace(8, 2);
  cluster_arrive();
  cluster_wait();
  trace(8, 3);

  // ---- LayerNorm (normStats + norm, instructions.js:451-550): thread t holds elements 4t..4t+3
  {
    const bool has = tid < E4;
    const float4 v = has ? reinterpret_cast<const float4 *>(xs)[tid] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 y = block_layernorm4<NT>(v, has, E, g_first, b_first, red);
    if (has) reinterpret_cast<float4 *>(hn)[tid] = y;
    __syncthreads();
  }
  trace(8, 4);

  // ---- q, k, v columns of this CTA
  trace(8, 4);
  {
    const int landed = __syncthreads_and(mbar_wait(&bars[0], 0, kFusedPolls) ? 1 : 0);
    if (!landed) {  // flag it, give the copies one more bounded chance, carry on (the result is void)
      if (tid == 0) atomicExch(p.err, 2);
      mbar_wait(&bars[0], 0, kFusedPolls << 2);
    }
  }
  float kv_keep[NB];  // the new k and v values, written to the cache at the end of the kernel
  {
    const float4 *w4 = reinterpret_cast<const float4 *>(wbuf);
    const float4 *h4 = reinterpret_cast<const float4 *>(hn);
    float acc[NB];
    trace(8, 5);
#pragma unroll
    for (int b = 0; b < NB; b++) acc[b] = 0.f;
#pragma unroll 2
    for (int i = lane; i < E4; i += 32) {
      const float4 xv = h4[i];
#pragma unroll
      for (int b = 0; b < NB; b++) {
        const int c = warp + NW * b;
        if (c < NC) acc[b] += dot4(w4[(size_t)c * E4 + i], xv);
      }
    }
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const int c = warp + NW * b;
      const float v = warp_sum(acc[b]) + bias_c[b];
      kv_keep[b] = v;
      if (c < NC) {
        const int sec = c / NQ, d = (int)rank * NQ + (c % NQ);
        float *dst = sec == 0 ? qfull : (sec == 1 ? knew : vnew);
        if (lane < CS) dsmem_st(dsmem_addr(dst + d, (uint32_t)lane), v);
      }
    }
  }
  __syncthreads();  // every warp is done with the q/k/v weights
  trace(8, 11);
  cluster_arrive();
  if (tid == 0) {   // fetch the projection slice into their place while the cluster barrier completes
    fence_proxy_async();
    const uint32_t bytes = (uint32_t)HS * (uint32_t)ncolA * 4u;
    mbar_expect_tx(&bars[1], bytes);
    const char *src = reinterpret_cast<const char *>(blk + (size_t)NC * E);
    for (uint32_t off = 0; off < bytes; off += 16384u)
      bulk_g2s(reinterpret_cast<char *>(wbuf) + off, src + off, min(16384u, bytes - off), &bars[1]);
  }
  cluster_wait();  // q and the new k, v rows are complete in every CTA
  trace(8, 6);

  // ---- attention of the head over positions 0..pos, this CTA's slice (online softmax; masked keys of the
  //      reference, instructions.js:1176, are simply not visited)
  {
    const int L = pos + 1;
    const int chunk = (L + CS - 1) / CS;
    const int beg = (int)rank * chunk, end = min(L, beg + chunk);
    const int g = lane / LPP, lig = lane % LPP;
    const float4 q4 = *reinterpret_cast<const float4 *>(qfull + lig * 4);
    const float4 kn4 = *reinterpret_cast<const float4 *>(knew + lig * 4);
    const float4 vn4 = *reinterpret_cast<const float4 *>(vnew + lig * 4);
    const float *kbl = kb + lig * 4, *vbl = vb + lig * 4;
    float m = -INFINITY, l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
    for (int j0 = beg + warp * G; j0 < end; j0 += NW * G) {  // same trip count for every lane of the warp
      const int j = j0 + g;
      const bool valid = j < end;
      const int jj = valid ? j : end - 1;
      float4 k4, v4;
      if (jj == pos) {
        k4 = kn4;
        v4 = vn4;
      } else {
        k4 = __ldcg(reinterpret_cast<const float4 *>(kbl + (size_t)jj * E));
        v4 = __ldcg(reinterpret_cast<const float4 *>(vbl + (size_t)jj * E));
      }
      float s = dot4(q4, k4);
#pragma unroll
      for (int o = LPP / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (valid) {
        s *= p.scale;
        const float mn = fmaxf(m, s);
        const float corr = expf(m - mn), pr = expf(s - mn);
        l = l * corr + pr;
        acc.x = acc.x * corr + pr * v4.x; acc.y = acc.y * corr + pr * v4.y;
        acc.z = acc.z * corr + pr * v4.z; acc.w = acc.w * corr + pr * v4.w;
        m = mn;
      }
    }
    __syncwarp();
#pragma unroll
    for (int o = LPP; o < 32; o <<= 1) {  // merge the G groups of the warp
      const float mo = __shfl_xor_sync(0xffffffffu, m, o), lo = __shfl_xor_sync(0xffffffffu, l, o);
      float4 ao;
      ao.x = __shfl_xor_sync(0xffffffffu, acc.x, o); ao.y = __shfl_xor_sync(0xffffffffu, acc.y, o);
      ao.z = __shfl_xor_sync(0xffffffffu, acc.z, o); ao.w = __shfl_xor_sync(0xffffffffu, acc.w, o);
      const float mn = fmaxf(m, mo);
      const float c0 = (m == -INFINITY) ? 0.f : expf(m - mn), c1 = (mo == -INFINITY) ? 0.f : expf(mo - mn);
      l = l * c0 + lo * c1;
      acc.x = acc.x * c0 + ao.x * c1; acc.y = acc.y * c0 + ao.y * c1;
      acc.z = acc.z * c0 + ao.z * c1; acc.w = acc.w * c0 + ao.w * c1;
      m = mn;
    }
    float *wm = red;  // [NW][MS]
    if (g == 0) {
      *reinterpret_cast<float4 *>(wm + warp * MS + lig * 4) = acc;
      if (lig == 0) { wm[warp * MS + HS] = m; wm[warp * MS + HS + 1] = l; }
    }
    __syncthreads();
    if (tid < HS + 2) {  // merge the warps, hand the CTA's record to every CTA of the cluster
      float mm = wm[HS];
#pragma unroll
      for (int w = 1; w < NW; w++) mm = fmaxf(mm, wm[w * MS + HS]);
      float ll = 0.f, a = 0.f;
#pragma unroll
      for (int w = 0; w < NW; w++) {
        const float wmx = wm[w * MS + HS];
        const float c = (wmx == -INFINITY) ? 0.f : expf(wmx - mm);
        ll += wm[w * MS + HS + 1] * c;
        if (tid < HS) a += wm[w * MS + tid] * c;
      }
      const float v = tid < HS ? a : (tid == HS ? mm : ll);
#pragma unroll
      for (int c = 0; c < CS; c++) dsmem_st(dsmem_addr(mrg + (int)rank * MS + tid, (uint32_t)c), v);
    }
  }
  trace(8, 7);
  // Only now may the next kernel start. Its CTAs fetch 19 MB of weights the moment they start, and while such a
  // burst is on its way to the SMs this kernel's small latency-critical transfers wait behind it: measured 4.7 us
  // instead of 1.3 us for the loads of the partial results, 3.1 us instead of 0.6 us for the cluster barrier after
  // the q/k/v exchange. What is left from here on (merge, projection out of shared memory) is short; of five release
  // points this one gave the shortest decode step.
  pdl_launch_dependents();
  cluster_arrive();
  cluster_wait();
  trace(8, 8);
  if (tid < HS) {  // the CS slices in slice order: identical in every CTA of the cluster
    float mm = mrg[HS];
#pragma unroll
    for (int r = 1; r < CS; r++) mm = fmaxf(mm, mrg[r * MS + HS]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int r = 0; r < CS; r++) {
      const float rm = mrg[r * MS + HS];
      const float c = (rm == -INFINITY) ? 0.f : expf(rm - mm);
      ll += mrg[r * MS + HS + 1] * c;
      a += mrg[r * MS + tid] * c;
    }
    osm[tid] = a / ll;
  }
  {
    const int landed = __syncthreads_and(mbar_wait(&bars[1], 0, kFusedPolls) ? 1 : 0);
    if (!landed) {
      if (tid == 0) atomicExch(p.err, 2);
      mbar_wait(&bars[1], 0, kFusedPolls << 2);
    }
  }
  // ---- this head's share of the output projection for columns [col0, col0 + ncolA): a partial result over heads
  trace(8, 9);
  {
    const int n = tid % ncolA, part = tid / ncolA;
    if (part < p.proj_parts) {
      const int dbeg = (HS * part) / p.proj_parts, dend = (HS * (part + 1)) / p.proj_parts;
      float s = 0.f;
#pragma unroll 8
      for (int d = dbeg; d < dend; d++) s += osm[d] * wbuf[d * ncolA + n];
      red[part * ncolA + n] = s;
    }
    __syncthreads();
    if (tid < ncolA) {
      float s = red[tid];
      for (int q = 1; q < p.proj_parts; q++) s += red[q * ncolA + tid];
      p.part_out[(size_t)h * E + col0 + tid] = s;
    }
  }
  // ---- the held-back stores: the residual stream for the MLP kernel, and the new k, v rows for later steps (this
  //      step read them from shared memory)
  if (h == 0 && tid < ncol4) reinterpret_cast<float4 *>(p.x_out + col0)[tid] = x_keep;
  if (lane == 0) {
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const int c = warp + NW * b;
      if (c < NC && c >= NQ) {
        const int sec = c / NQ, d = (int)rank * NQ + (c % NQ);
        (sec == 1 ? p.kc : p.vc)[(size_t)pos * E + h * HS + d] = kv_keep[b];
      }
    }
  }
  trace(8, 10);
}

constexpr int kMlpCluster = 2;  // CTAs per cluster of mlp_block_kernel (33 clusters of 4 fit on a B200 at once, 74 of 2)

struct MlpBlockParams {
  const float *xin;      // [E] residual stream before the attention block's contribution
  const float *part_in;  // [n_part][E] per-head partial results of the output projection
  const float *bias_in;  // [E] output-projection bias
  int n_part;
  float *x_out;          // [E]: xin + bias + partial results, for the next kernel's residual
  const float *gamma, *beta;
  const float *wfc_t;    // [F][E]
  const float *bfc;      // [F]
  const float *wpr_kn;   // [F][E]: the down-projection in the reference's [K, N] orientation
  float *part_out;       // [gridDim.x / kMlpCluster][E]: one row per cluster
  int E, F, units;       // units: most hidden units any CTA owns (sizes the shared-memory layout)
  int wk;                // K slices of the up-projection inside the CTA (power of two)
  int down_parts;        // unit slices of the down-projection step
  int red_floats;
  int *err;
};

__host__ __device__ inline size_t mlp_block_smem_floats(int E, int units, int red_floats) {
  return (size_t)2 * units * E + (size_t)E + (size_t)E /* exchange buffer: kMlpCluster x E/kMlpCluster */ +
         ((units + 3) & ~3) + red_floats + 8;
}

// grid = kMlpCluster * clusters; CTA c owns hidden units [F*c/grid, F*(c+1)/grid). Inside a cluster each CTA sums
// its share of the residual stream's columns and hands it to the others, and the cluster's partial results of the
// down-projection are added (in rank order) by the CTA that owns the columns, so the next kernel reads one row per
// cluster.
__global__ void __launch_bounds__(kMlpBlockThreads)
mlp_block_kernel(MlpBlockParams p) {
  constexpr int NT = kMlpBlockThreads, NW = NT / 32, CS = kMlpCluster;
  extern __shared__ __align__(128) float smem[];
  const int E = p.E, E4 = E >> 2, U = p.units;
  const int nq4 = E4 / CS;                 // float4 columns of the residual stream this CTA sums and owns
  float *wfc = smem;                       // [U][E]; re-used for the down-projection's slice sums
  float *wdn = wfc + (size_t)U * E;        // [U][E]
  float *xs = wdn + (size_t)U * E;         // residual stream (filled by all CTAs of the cluster), then normalised
  float *xch = xs + E;                     // [CS][E/CS]: the cluster's partial results for this CTA's columns
  float *gs = xch + E;                     // GELU outputs of this CTA's units
  float *red = gs + ((U + 3) & ~3);
  uint64_t *bars = reinterpret_cast<uint64_t *>(red + p.red_floats);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int j0 = (int)(((long long)p.F * blockIdx.x) / gridDim.x);
  const int nu = (int)(((long long)p.F * (blockIdx.x + 1)) / gridDim.x) - j0;
  TRACE_BEGIN(9);
  trace(9, 0);

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_expect_tx(&bars[0], (uint32_t)nu * (uint32_t)E * 4u);
    mbar_expect_tx(&bars[1], (uint32_t)nu * (uint32_t)E * 4u);
  }
  const int wk_log2 = 31 - __clz(p.wk);
  const int ks = warp & (p.wk - 1);
  const int kbeg = (int)(((unsigned)E4 * (unsigned)ks) >> wk_log2);
  const int kend = (int)(((unsigned)E4 * (unsigned)(ks + 1)) >> wk_log2);
  const int items = nu << wk_log2;
  float bias_u = 0.f;
  if (tid < nu) bias_u = p.bfc[j0 + tid];
  float4 g_first = make_float4(0.f, 0.f, 0.f, 0.f), b_first = g_first;
  if (tid < E4) {
    g_first = reinterpret_cast<const float4 *>(p.gamma)[tid];
    b_first = reinterpret_cast<const float4 *>(p.beta)[tid];
  }
  cluster_arrive();  // pairs with the wait below: every CTA of the cluster is running before any remote store
  if (tid == 0) {
    bulk_g2s_block(wfc, p.wfc_t + (size_t)j0 * E, (uint32_t)nu * (uint32_t)E * 4u, &bars[0]);
  }
  pdl_wait();
  trace(9, 1);

  // ---- residual stream: xin + bias + the per-head partial results for this CTA's share of the columns
  float4 x_keep = make_float4(0.f, 0.f, 0.f, 0.f);
  int x_col = -1;
  {
    const int cbase = (int)rank * nq4;
    const int c = warp * 16 + (lane & 15);  // one warp per 16 columns, its two halves take alternate rows
    const bool mine = c < nq4 && lane < 16;
    // The second weight block is requested only here, behind this kernel's own loads of the partial results: requested
    // ahead of the wait together with the first, its 9.4 MB were still arriving when these loads were issued, and they
    // waited behind it (2.9 us instead of 1.6 us from the wait to the exchange).
    const float4 sum = halfwarp_rows_sum<kMlpSumRows>(
        reinterpret_cast<const float4 *>(p.part_in) + cbase + warp * 16, min(16, max(nq4 - warp * 16, 0)), (size_t)E4,
        p.n_part, lane, [&] {
          if (tid == 0)
            bulk_g2s_block(wdn, p.wpr_kn + (size_t)j0 * E, (uint32_t)nu * (uint32_t)E * 4u, &bars[1]);
        });
    float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f);
    x_col = cbase + c;
    if (mine)
      x0 = add4(__ldcg(reinterpret_cast<const float4 *>(p.xin) + cbase + c),
                reinterpret_cast<const float4 *>(p.bias_in)[cbase + c]);
    cluster_wait();
    if (mine) {
      const float4 x = add4(x0, sum);
#pragma unroll
      for (int cc = 0; cc < CS; cc++) dsmem_st4(dsmem_addr(xs + 4 * (cbase + c), (uint32_t)cc), x);
      if (blockIdx.x < CS) x_keep = x;  // stored after the last cluster barrier (see attn_block_kernel)
      else x_col = -1;
    } else {
      x_col = -1;
    }
  }
  cluster_arrive();
  cluster_wait();
  trace(9, 2);
  {
    const bool has = tid < E4;
    const float4 v = has ? reinterpret_cast<const float4 *>(xs)[tid] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 y = block_layernorm4<NT>(v, has, E, g_first, b_first, red);
    if (has) reinterpret_cast<float4 *>(xs)[tid] = y;  // in place: v was read before the barriers inside
  }
  trace(9, 3);

  // ---- up-projection + bias + GELU for this CTA's hidden units
  {
    const int landed = __syncthreads_and(mbar_wait(&bars[0], 0, kFusedPolls) ? 1 : 0);  // also publishes xs
    if (!landed) {
      if (tid == 0) atomicExch(p.err, 2);
      mbar_wait(&bars[0], 0, kFusedPolls << 2);
    }
  }
  trace(9, 4);
  {
    const float4 *w4 = reinterpret_cast<const float4 *>(wfc);
    const float4 *h4 = reinterpret_cast<const float4 *>(xs);
    constexpr int NBI = 3;
    for (int it0 = warp; it0 < items; it0 += NW * NBI) {
      int c[NBI];
      bool valid[NBI];
      float acc[NBI];
#pragma unroll
      for (int b = 0; b < NBI; b++) {
        const int it = it0 + NW * b;
        valid[b] = it < items;
        c[b] = valid[b] ? (it >> wk_log2) : 0;
        acc[b] = 0.f;
      }
#pragma unroll 3
      for (int i = kbeg + lane; i < kend; i += 32) {
        const float4 xv = h4[i];
#pragma unroll
        for (int b = 0; b < NBI; b++) acc[b] += dot4(w4[(size_t)c[b] * E4 + i], xv);
      }
#pragma unroll
      for (int b = 0; b < NBI; b++) {
        const float v = warp_sum(acc[b]);
        if (lane == 0 && valid[b]) red[c[b] * p.wk + ks] = v;
      }
    }
  }
  __syncthreads();
  if (tid < nu) {
    float v = 0.f;
    for (int k = 0; k < p.wk; k++) v += red[tid * p.wk + k];
    gs[tid] = gelu_f(v + bias_u);
  }
  // Only now may the next kernel start fetching its weights (see attn_block_kernel): after the partial results have
  // been read and the hidden units computed; the down-projection below works out of shared memory.
  pdl_launch_dependents();
  trace(9, 5);
  {
    const int landed = __syncthreads_and(mbar_wait(&bars[1], 0, kFusedPolls) ? 1 : 0);
    if (!landed) {
      if (tid == 0) atomicExch(p.err, 2);
      mbar_wait(&bars[1], 0, kFusedPolls << 2);
    }
  }
  // ---- these units' rows of the down-projection, then the cluster's results added by the column owner
  trace(9, 6);
  {
    const int c4 = tid % E4, part = tid / E4;
    float4 *dsum = reinterpret_cast<float4 *>(wfc);  // the up-projection weights are no longer needed
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (part < p.down_parts) {
      const int ub = (nu * part) / p.down_parts, ue = (nu * (part + 1)) / p.down_parts;
      const float4 *w4 = reinterpret_cast<const float4 *>(wdn) + c4;
#pragma unroll 4
      for (int u = ub; u < ue; u++) {
        const float gv = gs[u];
        const float4 w = w4[(size_t)u * E4];
        a.x += gv * w.x; a.y += gv * w.y; a.z += gv * w.z; a.w += gv * w.w;
      }
      if (part > 0) dsum[(part - 1) * E4 + c4] = a;
    }
    __syncthreads();
    if (part == 0) {
      for (int q = 1; q < p.down_parts; q++) a = add4(a, dsum[(q - 1) * E4 + c4]);
      const int owner = c4 / nq4, cc = c4 - owner * nq4;
      dsmem_st4(dsmem_addr(xch + 4 * ((int)rank * nq4 + cc), (uint32_t)owner), a);
    }
  }
  cluster_arrive();
  cluster_wait();
  if (tid < nq4) {
    const float4 *x4 = reinterpret_cast<const float4 *>(xch);
    float4 a = x4[tid];
#pragma unroll
    for (int r = 1; r < CS; r++) a = add4(a, x4[r * nq4 + tid]);
    reinterpret_cast<float4 *>(p.part_out + (size_t)(blockIdx.x / CS) * E)[(int)rank * nq4 + tid] = a;
  }
  if (x_col >= 0) reinterpret_cast<float4 *>(p.x_out)[x_col] = x_keep;
  trace(9, 7);
}

// x_out = xin + bias + sum of the n_part partial rows (at most 8 * kAttnSumRows). grid = ceil(E/4 / 32), 256
// threads: lane = float4 column, the 8 warps share the rows.
__global__ void __launch_bounds__(256)
finish_row_kernel(const float *__restrict__ xin, const float *__restrict__ bias, const float *__restrict__ part,
                  int n_part, int E, float *__restrict__ x_out) {
  __shared__ float4 red[8][32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int E4 = E >> 2, c0 = blockIdx.x * 32;
  const int ncols = min(32, E4 - c0);
  float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (tid < ncols) x0 = reinterpret_cast<const float4 *>(bias)[c0 + tid];
  pdl_wait();
  red[warp][lane] = warp_rows_partial<8, kAttnSumRows>(reinterpret_cast<const float4 *>(part) + c0, ncols, (size_t)E4,
                                                       n_part, warp, lane);
  if (tid < ncols) x0 = add4(x0, __ldcg(reinterpret_cast<const float4 *>(xin) + c0 + tid));
  __syncthreads();
  pdl_launch_dependents();
  if (tid < ncols) {
#pragma unroll
    for (int w = 0; w < 8; w++) x0 = add4(x0, red[w][tid]);
    reinterpret_cast<float4 *>(x_out)[c0 + tid] = x0;
  }
}

}  // namespace wgpt
