// Memory-bound row/elementwise kernels: residual add, GELU, LayerNorm, softmax, embedding gather,
// arg-max, transposition. All are 128-bit vectorised where the shape allows.
#pragma once
#include "common.cuh"

namespace wgpt {

// out = a + b (elementWiseAddition, instructions.js:358-384), n4 float4 elements.
__global__ void residual_kernel(const float4 *__restrict__ a, const float4 *__restrict__ b, float4 *__restrict__ out,
                                size_t n4) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n4; i += stride) {
    float4 x = a[i], y = b[i];
    out[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
  }
}

// GELU (instructions.js:705-748).
__global__ void gelu_kernel(const float4 *__restrict__ in, float4 *__restrict__ out, size_t n4) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n4; i += stride) {
    float4 x = in[i];
    out[i] = make_float4(gelu_f(x.x), gelu_f(x.y), gelu_f(x.z), gelu_f(x.w));
  }
}

// LayerNorm, one warp per row (normStats + norm, instructions.js:451-550):
// mean = sum/N, var = sum((x-mean)^2)/N, y = gamma*((x-mean)/sqrt(var+1e-5))+beta.
// Row r of the input starts at in + r*ld_in (lets the caller normalise only the last row of each sequence).
__global__ void layernorm_kernel(const float *__restrict__ in, size_t ld_in, const float *__restrict__ gamma,
                                 const float *__restrict__ beta, float *__restrict__ out, size_t ld_out, int rows,
                                 int N) {
  int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();  // the rows come from the previous kernel (read through L2, see common.cuh)
  if (row >= rows) return;
  const float4 *x = reinterpret_cast<const float4 *>(in + (size_t)row * ld_in);
  int n4 = N >> 2;
  float s = 0.f;
  for (int i = lane; i < n4; i += 32) {
    float4 v = __ldcg(x + i);
    s += (v.x + v.y) + (v.z + v.w);
  }
  float mean = warp_sum(s) / (float)N;
  float q = 0.f;
  for (int i = lane; i < n4; i += 32) {
    float4 v = __ldcg(x + i);
    float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
    q += (a * a + b * b) + (c * c + d * d);
  }
  float sd = sqrtf(warp_sum(q) / (float)N + 1e-5f);
  const float4 *g4 = reinterpret_cast<const float4 *>(gamma);
  const float4 *b4 = reinterpret_cast<const float4 *>(beta);
  float4 *o = reinterpret_cast<float4 *>(out + (size_t)row * ld_out);
  for (int i = lane; i < n4; i += 32) {
    float4 v = __ldcg(x + i), g = g4[i], b = b4[i];
    o[i] = make_float4(g.x * ((v.x - mean) / sd) + b.x, g.y * ((v.y - mean) / sd) + b.y,
                       g.z * ((v.z - mean) / sd) + b.z, g.w * ((v.w - mean) / sd) + b.w);
  }
}

// Row softmax, one warp per row (instructions.js:593-666). Scalar accesses: cols is arbitrary.
__global__ void softmax_kernel(const float *__restrict__ in, float *__restrict__ out, int rows, int cols) {
  int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float *x = in + (size_t)row * cols;
  float m = -3.402823e+38f;
  for (int i = lane; i < cols; i += 32) m = fmaxf(m, x[i]);
  m = warp_max(m);
  float s = 0.f;
  for (int i = lane; i < cols; i += 32) s += expf(x[i] - m);
  s = warp_sum(s);
  float *o = out + (size_t)row * cols;
  for (int i = lane; i < cols; i += 32) o[i] = expf(x[i] - m) / s;
}

// Embedding gather + positional add (EmbedBlock, instructions.js:790-827) with ids on the device.
// Row m = seq*n_tok + t reads wte[idx[m]] and wpe[*pos + t]. An id >= vocab sets *err and leaves zeros.
__global__ void embed_kernel(const uint32_t *__restrict__ idx, const float *__restrict__ wte,
                             const float *__restrict__ wpe, float *__restrict__ out, int rows, int n_tok, int E,
                             int vocab, const int *__restrict__ pos, int *err) {
  int m = blockIdx.x;
  if (m >= rows) return;
  TRACE_BEGIN(4);
  trace(4, 0);
  pdl_launch_dependents();
  pdl_wait();  // idx and *pos are written by the previous step's arg-max
  uint32_t id = __ldcg(idx + m);
  int t = m % n_tok;
  int p = (pos ? __ldcg(pos) : 0) + t;
  float4 *o = reinterpret_cast<float4 *>(out + (size_t)m * E);
  if (id >= (uint32_t)vocab) {
    if (threadIdx.x == 0) atomicExch(err, 1);
    for (int i = threadIdx.x; i < E / 4; i += blockDim.x) o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    return;
  }
  const float4 *a = reinterpret_cast<const float4 *>(wte + (size_t)id * E);
  const float4 *b = reinterpret_cast<const float4 *>(wpe + (size_t)p * E);
  for (int i = threadIdx.x; i < E / 4; i += blockDim.x) {
    float4 x = a[i], y = b[i];
    o[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
  }
}

// Greedy pick per sequence: arg-max of logits[seq, 0..V), lowest index on ties (globals.js:66-74
// with top_k = 1). Writes the id as the next input token and into the output list at *step. The last block to
// finish then advances the session's position by n_tok and its step counter by one (every block has read
// *step before it can be counted as finished). done_counter must be zero on entry and is left zero.
__global__ void argmax_kernel(const float *__restrict__ logits, int V, uint32_t *__restrict__ next_ids,
                              uint32_t *__restrict__ out_ids, int out_stride, int *__restrict__ pos,
                              int *__restrict__ step, int n_tok, unsigned int *__restrict__ done_counter) {
  pdl_launch_dependents();
  pdl_wait();
  int seq = blockIdx.x;
  const int my_step = __ldcg(step);
  const float *x = logits + (size_t)seq * V;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  // eight loads in flight per thread (few CTAs run: the row scan is bound by latency, not bandwidth); a thread's
  // indices ascend, so a strict > keeps its lowest index among equal values
  int i = threadIdx.x;
  const int stride = blockDim.x;
  for (; i + 7 * stride < V; i += 8 * stride) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; u++) v[u] = __ldcg(x + i + u * stride);
#pragma unroll
    for (int u = 0; u < 8; u++)
      if (v[u] > best) { best = v[u]; bi = i + u * stride; }
  }
  for (; i < V; i += stride) {
    float v = __ldcg(x + i);
    if (v > best) { best = v; bi = i; }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      if (bi == 0x7fffffff) bi = 0;  // a row of NaNs compares false everywhere: report index 0
      next_ids[seq] = (uint32_t)bi;
      if (out_ids) out_ids[(size_t)seq * out_stride + my_step] = (uint32_t)bi;
      __threadfence();
      unsigned int prev = atomicAdd(done_counter, 1u);
      if (prev == gridDim.x - 1) {
        *pos = __ldcg(pos) + n_tok;
        *step = my_step + 1;
        *done_counter = 0u;
      }
    }
  }
}

// lo = w - tf32(w): what a TF32 tensor-core product drops from each weight (it reads the top 19 bits of an FP32
// operand), kept as a second matrix so that the 3xTF32 GEMM can fetch it by TMA. Load time only.
__global__ void tf32_lo_kernel(const float4 *__restrict__ w, float4 *__restrict__ lo, size_t n4) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n4; i += stride) {
    float4 x = w[i], l;
    l.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
    l.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
    l.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
    l.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
    lo[i] = l;
  }
}

// Advances the session's device-side position and step counters after a decode step.
__global__ void advance_kernel(int *pos, int *step, int n_tok) {
  pdl_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    *pos = __ldcg(pos) + n_tok;
    *step = __ldcg(step) + 1;
  }
}

// out[c][r] = in[r][c] for an [R, C] matrix; 32x32 tiles through shared memory. Used once per weight at
// load time (the reference transposes on the host, globals.js:80-94).
__global__ void transpose_kernel(const float *__restrict__ in, float *__restrict__ out, int R, int C) {
  __shared__ float tile[32][33];
  int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = r0 + j, c = c0 + threadIdx.x;
    if (r < R && c < C) tile[j][threadIdx.x] = in[(size_t)r * C + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int c = c0 + j, r = r0 + threadIdx.x;
    if (r < R && c < C) out[(size_t)c * R + r] = tile[threadIdx.x][j];
  }
}


// Heat map of the residual stream, the fragment shader of the reference's visualiser (visuals.js:104-135) run
// headless: pixel (x, y) of an n_embd x n_ctx image shows v = 0.1 * buf[y*n_embd + x]; negative values go to
// blue (plus green beyond -1), positive to red (plus green beyond +1), green capped at 0.7, alpha left at 0 as
// in the shader. Output is RGBA8 (unorm: clamp to [0,1], round to nearest), 4 bytes per pixel, row-major.
__global__ void heatmap_kernel(const float *__restrict__ buf, uchar4 *__restrict__ rgba, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float v = buf[i] * 0.1f;
    float r = 0.f, g = 0.f, b = 0.f;
    if (v < 0.f) {
      b = -v;
      if (v < -1.0f) g = -v - 1.0f;
    } else {
      r = v;
      if (v > 1.0f) g = v - 1.0f;
    }
    g = fminf(g, 0.7f);
    uchar4 px;
    px.x = (unsigned char)floorf(fminf(fmaxf(r, 0.f), 1.f) * 255.f + 0.5f);
    px.y = (unsigned char)floorf(fminf(fmaxf(g, 0.f), 1.f) * 255.f + 0.5f);
    px.z = (unsigned char)floorf(fminf(fmaxf(b, 0.f), 1.f) * 255.f + 0.5f);
    px.w = 0;
    rgba[i] = px;
  }
}

// Diagnostic: drives the bounded mbarrier wait the bulk-copy kernels use to its limit, safely. The barrier is armed
// for 32 bytes but only 16 are copied at first, so its phase cannot complete and mbar_wait gives up after `polls`
// polls; the kernel then does what the product kernels do on expiry: it sets the device error word to 2, lets the
// outstanding copy finish (here by supplying the missing 16 bytes, after which a second bounded wait succeeds) and
// returns. Nothing spins without a limit and nothing faults; the context stays usable.
__global__ void wait_expiry_probe_kernel(const float *__restrict__ src16, int *err, uint32_t polls, int *observed) {
  __shared__ __align__(16) float buf[8];
  __shared__ uint64_t bar;
  if (threadIdx.x != 0) return;
  mbar_init(&bar, 1);
  mbar_expect_tx(&bar, 32);
  bulk_g2s(buf, src16, 16, &bar);
  const bool first = mbar_wait(&bar, 0, polls);
  if (!first) atomicExch(err, 2);
  bulk_g2s(buf + 4, src16, 16, &bar);                 // the rest of the bytes the barrier was armed for
  const bool second = mbar_wait(&bar, 0, 1u << 22);   // drain: bounded as well
  observed[0] = first ? 1 : 0;
  observed[1] = second ? 1 : 0;
}

}  // namespace wgpt
