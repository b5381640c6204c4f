// Shared device helpers for the sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace wgpt {

constexpr int kWarp = 32;

// Where a matmul result goes and what is applied to it on the way out.
// Fuses the reference's separate bias add (instructions.js:304-314), GELU pass (:705-748) and
// residual pass (:358-384) into the producing kernel, and lets the QKV projection write K and V
// rows straight into the KV cache.
struct Epilogue {
  const float *colscale;  // [N] or nullptr: multiplies the raw product (int8 per-column dequant scale)
  const float *bias;      // [N] or nullptr
  const float *residual;  // [M, ld] or nullptr; may alias out
  float *out;             // [M, ld]
  int ld;
  int act;                // 1 = GELU
  // KV scatter (kc != nullptr): columns [E,2E) go to kc, [2E,3E) to vc; row m = seq*n_tok + t
  // lands in cache row seq*n_ctx + *pos + t.
  float *kc, *vc;
  int E, n_tok, n_ctx;
  const int *pos;  // device position counter; a kernel that stores many elements reads it once into pos_base
  int pos_base;    // used when pos == nullptr
};

__device__ __forceinline__ float gelu_f(float x) {
  // instructions.js:711-727
  float x3 = x * x * x;
  float r = x * (0.5f * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x3))));
  r = x < -10.0f ? 0.0f : r;
  return x > 10.0f ? x : r;
}

// Address of element (m, n) of the epilogue's destination. n..n+3 stay in one section when E % 4 == 0.
__device__ __forceinline__ float *epi_addr(const Epilogue &e, int m, int n) {
  if (e.kc == nullptr || n < e.E) return e.out + (size_t)m * e.ld + n;
  int sec = n >= 2 * e.E ? 2 : 1;
  int c = n - sec * e.E;
  int seq = m / e.n_tok, t = m - seq * e.n_tok;
  size_t row = (size_t)seq * e.n_ctx + (size_t)(e.pos ? __ldcg(e.pos) : e.pos_base) + t;
  return (sec == 1 ? e.kc : e.vc) + row * e.E + c;
}

__device__ __forceinline__ float epi_apply(const Epilogue &e, float v, int m, int n) {
  if (e.colscale) v *= e.colscale[n];
  if (e.bias) v += e.bias[n];
  if (e.act == 1) v = gelu_f(v);
  if (e.residual) v += __ldcg(e.residual + (size_t)m * e.ld + n);
  return v;
}

__device__ __forceinline__ void epi_store(const Epilogue &e, float v, int m, int n) {
  *epi_addr(e, m, n) = epi_apply(e, v, m, n);
}

__device__ __forceinline__ float4 epi_apply4(const Epilogue &e, float4 v, int m, int n) {
  if (e.colscale) {
    float4 c = *reinterpret_cast<const float4 *>(e.colscale + n);
    v.x *= c.x; v.y *= c.y; v.z *= c.z; v.w *= c.w;
  }
  if (e.bias) {
    float4 b = *reinterpret_cast<const float4 *>(e.bias + n);
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
  }
  if (e.act == 1) { v.x = gelu_f(v.x); v.y = gelu_f(v.y); v.z = gelu_f(v.z); v.w = gelu_f(v.w); }
  if (e.residual) {
    float4 r = __ldcg(reinterpret_cast<const float4 *>(e.residual + (size_t)m * e.ld + n));
    v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
  }
  return v;
}

// epi_apply4 with the bias and the residual already in registers (zero where the epilogue has none): a second stage
// fetches the bias ahead of its dependency wait and requests the residual together with its partial sums instead
// of one memory round trip later.
__device__ __forceinline__ float4 epi_apply4_pre(const Epilogue &e, float4 v, float4 bias, float4 res, int n) {
  if (e.colscale) {
    float4 c = *reinterpret_cast<const float4 *>(e.colscale + n);
    v.x *= c.x; v.y *= c.y; v.z *= c.z; v.w *= c.w;
  }
  v.x += bias.x; v.y += bias.y; v.z += bias.z; v.w += bias.w;
  if (e.act == 1) { v.x = gelu_f(v.x); v.y = gelu_f(v.y); v.z = gelu_f(v.z); v.w = gelu_f(v.w); }
  v.x += res.x; v.y += res.y; v.z += res.z; v.w += res.w;
  return v;
}

__device__ __forceinline__ void epi_store4(const Epilogue &e, float4 v, int m, int n) {
  *reinterpret_cast<float4 *>(epi_addr(e, m, n)) = epi_apply4(e, v, m, n);
}

// 128-bit read-only load that does not allocate in L1 (weights are streamed once per pass).
__device__ __forceinline__ float4 ldg_stream4(const float4 *p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_stream4u(const uint4 *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Development aid, compiled in only with -DWGPT_TRACE: thread 0 of the first and last CTA of a kernel append
// (globaltimer, kernel id, phase) records to a device buffer that a debug entry point reads back.
#ifdef WGPT_TRACE
__device__ unsigned long long g_trace_buf[1 << 17];
__device__ unsigned int g_trace_n;
// One atomic per kernel (at entry, ahead of the dependency wait) reserves 32 record slots; later phases only read
// the timer and store, so they do not stall the traced thread.
__device__ __forceinline__ unsigned int trace_begin(int kid) {
  unsigned int base = 0xffffffffu;
  if (threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) {
    base = atomicAdd(&g_trace_n, 32u);
    if (base + 32 > (1u << 16)) base = 0xffffffffu;
  }
  return base;
}
__device__ __forceinline__ void trace_at(unsigned int base, int kid, int phase) {
  if (base != 0xffffffffu) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    g_trace_buf[2 * (base + phase)] = t;
    g_trace_buf[2 * (base + phase) + 1] =
        ((unsigned long long)kid << 16) | ((unsigned long long)phase << 8) | (blockIdx.x == 0 ? 0u : 1u);
  }
}
#define TRACE_BEGIN(kid) const unsigned int trace_base_ = trace_begin(kid)
#define trace(kid, phase) trace_at(trace_base_, kid, phase)
#else
#define TRACE_BEGIN(kid) ((void)0)
#define trace(kid, phase) ((void)0)
#endif

// Activations written by an earlier kernel are read with __ldcg (L2, bypassing L1) in every kernel that can be
// launched programmatically: such a kernel becomes resident, and has its SM's L1 invalidated, while its
// predecessor is still running, so a line another CTA of the predecessor pulled into that L1 afterwards (for
// instance around an in-place residual update) would otherwise be read stale after the wait.
//
// Programmatic dependent launch. A kernel launched with the programmatic-serialisation attribute may start
// while its predecessor in the stream is still running; everything it does before pdl_wait() must therefore
// touch only data no earlier kernel writes (here: weights). pdl_wait() returns once every earlier kernel has
// completed and its writes are visible; without the attribute both calls are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Asks the memory system to bring [p, p+bytes) into L2 (p 16-byte aligned, bytes a multiple of 16).
__device__ __forceinline__ void prefetch_l2(const void *p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Asks for the 128-byte line that holds p in L2 through the load/store unit. Used where many small strided pieces
// are wanted (rows of the K/V cache): hundreds of bulk prefetch requests from one CTA, issued while another CTA of
// the same SM had bulk copies in flight, coincided with launch failures, so the bulk-copy engine is kept for few,
// large requests.
__device__ __forceinline__ void prefetch_line_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// ---- bulk asynchronous copy (TMA, untiled form) global -> shared, completion counted on an mbarrier ----
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// dst (shared) and src (global) 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
// Bounded wait for the given phase parity: returns false if the copy has not landed after max_polls polls
// (each poll may itself block for a hardware-defined short time).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t max_polls) {
  uint32_t done = 0;
  for (uint32_t i = 0; i < max_polls && !done; i++) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
  }
  return done != 0;
}

// Rank of this CTA inside its thread-block cluster.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

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

__device__ __forceinline__ float dot4(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }

// LayerNorm of one row of E floats (normStats + norm, instructions.js:451-550) by a whole CTA of NT threads:
// thread t < E/4 holds elements 4t..4t+3 in v. Two block-wide sums (mean, then the squared deviations from it),
// each a warp butterfly plus a fixed-order sum of the warps' results; sred needs 2*NT/32 floats. Returns the
// normalised elements; multiplies by 1/sd where the shader divides (at most one unit in the last place apart).
template <int NT>
__device__ __forceinline__ float4 block_layernorm4(float4 v, bool has, int E, float4 g, float4 b, float *sred) {
  constexpr int NW = NT / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float s = has ? (v.x + v.y) + (v.z + v.w) : 0.f;
  s = warp_sum(s);
  if (lane == 0) sred[warp] = s;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < NW; w++) tot += sred[w];
  const float mean = tot / (float)E;
  const float dx = v.x - mean, dy = v.y - mean, dz = v.z - mean, dw = v.w - mean;
  float q = has ? (dx * dx + dy * dy) + (dz * dz + dw * dw) : 0.f;
  q = warp_sum(q);
  if (lane == 0) sred[NW + warp] = q;
  __syncthreads();
  float qt = 0.f;
#pragma unroll
  for (int w = 0; w < NW; w++) qt += sred[NW + w];
  const float rsd = 1.0f / sqrtf(qt / (float)E + 1e-5f);
  return make_float4(g.x * (dx * rsd) + b.x, g.y * (dy * rsd) + b.y, g.z * (dz * rsd) + b.z, g.w * (dw * rsd) + b.w);
}


}  // namespace wgpt
