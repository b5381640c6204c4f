// int8 weight-only dequant matmul, the kernel prototyped in other/int8-gemm.js:117-229.
// Bq is [K, N/4] 32-bit words, byte j of word w in row k = column 4w+j (other/int8-gemm.js:36-42).
// Integers are recovered exactly as the prototype does, (int32(word) << (24-8j)) >> 24 (:126-131); they are
// exact in f32, the products accumulate in FP32, and the per-column scale multiplies the finished sum.
// HBM-bound for small M: bytes = K*N (weights) + 4*M*K + 4*M*N + 4*N.
#pragma once
#include "common.cuh"

namespace wgpt {

__device__ __forceinline__ void unpack_int8x4(uint32_t word, float (&f)[4]) {
  int32_t v = (int32_t)word;
  f[0] = (float)((v << 24) >> 24);
  f[1] = (float)((v << 16) >> 24);
  f[2] = (float)((v << 8) >> 24);
  f[3] = (float)(v >> 24);
}

// The same four integers as unpack_int8x4, as floats, without integer-to-float conversions (a quarter-rate
// instruction): byte b as an unsigned u = b ^ 0x80 is dropped into the mantissa of 2^23 (bits 0x4B000000 | u =
// 2^23 + u exactly) and 2^23 + 128 is subtracted, which leaves u - 128 = the signed code, exactly.
__device__ __forceinline__ float4 unpack_int8x4_fast(uint32_t word) {
  const uint32_t u = word ^ 0x80808080u;
  const float bias = 8388736.0f;  // 2^23 + 128
  return make_float4(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - bias,
                     __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - bias,
                     __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - bias,
                     __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - bias);
}

// quantizeMatrix, other/int8-gemm.js:25-46, on the device. Pass 1: |w| maxima per output column of the row-major
// [K, N] matrix (the prototype's header asks for vector-wise scales, :4), one thread per column per k slice,
// partial maxima [gridDim.y][N]. The maximum is order-independent, so no fixed order is needed for exactness.
__global__ void int8_absmax_kernel(const float *__restrict__ w, int K, int N, float *__restrict__ part) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const int kb = (int)(((long long)K * blockIdx.y) / gridDim.y), ke = (int)(((long long)K * (blockIdx.y + 1)) / gridDim.y);
  float a = 0.f;
  for (int k = kb; k < ke; k++) a = fmaxf(a, fabsf(w[(size_t)k * N + n]));
  part[(size_t)blockIdx.y * N + n] = a;
}
// Pass 2: column maxima from the partial maxima (per_column == 0: one maximum for the whole matrix, the
// prototype's own rule :29-33), scale[n] = absmax_n / 127 in double rounded to f32.
__global__ void int8_scale_kernel(const float *__restrict__ part, int slices, int N, int per_column,
                                  float *__restrict__ absmax, float *__restrict__ scale) {
  __shared__ float red[256];
  const int tid = threadIdx.x;
  float g = 0.f;
  for (int n = tid; n < N; n += 256) {
    float a = 0.f;
    for (int s = 0; s < slices; s++) a = fmaxf(a, part[(size_t)s * N + n]);
    absmax[n] = a;
    g = fmaxf(g, a);
  }
  red[tid] = g;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) red[tid] = fmaxf(red[tid], red[tid + o]);
    __syncthreads();
  }
  g = red[0];
  for (int n = tid; n < N; n += 256) {
    const float a = per_column ? absmax[n] : g;
    absmax[n] = a;
    scale[n] = (float)((double)a / 127.0);
  }
}
// Pass 3: word w of row k packs columns 4w..4w+3: byte j = round(x / absmax * 127) & 0xff with the arithmetic of
// the JavaScript expression: double precision, Math.round = floor(x + 0.5) (:36-42). A zero column packs zeros.
__global__ void int8_pack_kernel(const float *__restrict__ w, const float *__restrict__ absmax, int K, int N,
                                 uint32_t *__restrict__ packed) {
  const size_t total = (size_t)K * (N >> 2);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t k = i / (N >> 2);
    const int n = (int)(i - k * (N >> 2)) * 4;
    const float4 x = *reinterpret_cast<const float4 *>(w + k * N + n);
    const float4 a = *reinterpret_cast<const float4 *>(absmax + n);
    const float xv[4] = {x.x, x.y, x.z, x.w}, av[4] = {a.x, a.y, a.z, a.w};
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int q = 0;
      if (av[j] > 0.f) q = (int)floor(__dmul_rn(__ddiv_rn((double)xv[j], (double)av[j]), 127.0) + 0.5);
      word |= ((uint32_t)q & 0xffu) << (8 * j);
    }
    packed[i] = word;
  }
}

// M <= 16 rows. Lane owns 4*VEC consecutive columns (VEC 32-bit words per load: VEC = 4 is a 128-bit load);
// a warp covers 128*VEC columns of one k row; 8 warps x gridDim.y CTAs split K.
// part: [gridDim.y][M][N] partial sums, summed (and scaled) by gemv_kn_reduce_kernel.
template <int M, int VEC>
__global__ void __launch_bounds__(256)
int8_gemv_partial_kernel(const float *__restrict__ x, const uint32_t *__restrict__ Bq, int K, int N,
                         float *__restrict__ part) {
  extern __shared__ __align__(128) float smem[];
  constexpr int CPL = 4 * VEC;  // columns per lane
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ksplit = gridDim.y;
  const int kbeg = (int)(((long long)(K / 4) * blockIdx.y) / ksplit) * 4;
  const int kend = (int)(((long long)(K / 4) * (blockIdx.y + 1)) / ksplit) * 4;
  const int klen = kend - kbeg;
  float *xs = smem;
  float *red = smem + (size_t)M * klen;  // [8 warps][M][32 lanes][CPL]
  for (int i = tid; i < M * klen; i += 256) {
    int m = i / klen, k = i - m * klen;
    xs[m * klen + k] = x[(size_t)m * K + kbeg + k];
  }
  __syncthreads();
  const int n = (blockIdx.x * 32 + lane) * CPL;
  const int ND4 = N >> 2;
  float acc[M][CPL];
#pragma unroll
  for (int m = 0; m < M; m++)
#pragma unroll
    for (int c = 0; c < CPL; c++) acc[m][c] = 0.f;
  if (n < N) {
    const uint32_t *bp = Bq + (size_t)kbeg * ND4 + (n >> 2);
#pragma unroll 4
    for (int k = warp; k < klen; k += 8) {
      uint32_t w[VEC];
      if (VEC == 4) {
        uint4 t = ldg_stream4u(reinterpret_cast<const uint4 *>(bp + (size_t)k * ND4));
        w[0] = t.x; w[VEC > 1 ? 1 : 0] = t.y; w[VEC > 2 ? 2 : 0] = t.z; w[VEC > 3 ? 3 : 0] = t.w;
      } else {
#pragma unroll
        for (int v = 0; v < VEC; v++) w[v] = __ldg(bp + (size_t)k * ND4 + v);
      }
      float b[CPL];
#pragma unroll
      for (int v = 0; v < VEC; v++) {
        float f[4];
        unpack_int8x4(w[v], f);
        b[4 * v] = f[0]; b[4 * v + 1] = f[1]; b[4 * v + 2] = f[2]; b[4 * v + 3] = f[3];
      }
#pragma unroll
      for (int m = 0; m < M; m++) {
        float a = xs[m * klen + k];
#pragma unroll
        for (int c = 0; c < CPL; c++) acc[m][c] += a * b[c];
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; m++)
#pragma unroll
    for (int c = 0; c < CPL; c++) red[((warp * M + m) * 32 + lane) * CPL + c] = acc[m][c];
  __syncthreads();
  for (int i = tid; i < M * 32 * CPL; i += 256) {
    int c = i % CPL, l = (i / CPL) % 32, m = i / (CPL * 32);
    int nn = (blockIdx.x * 32 + l) * CPL + c;
    if (nn >= N) continue;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) s += red[((w * M + m) * 32 + l) * CPL + c];
    part[((size_t)blockIdx.y * M + m) * N + nn] = s;
  }
}

// General M: the 64x64x16 SIMT tile of gemm_simt_kernel with the B tile dequantised while it is staged.
__global__ void __launch_bounds__(256)
int8_gemm_simt_kernel(const float *__restrict__ A, const uint32_t *__restrict__ Bq, int M, int K, int N,
                      Epilogue epi) {
  __shared__ __align__(16) float As[16][64 + 4];
  __shared__ __align__(16) float Bs[16][64 + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64, ND4 = N >> 2;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  const int a_row = tid >> 2, a_k4 = (tid & 3) * 4;
  const int b_k = tid >> 4, b_w = tid & 15;  // 16 k x 16 words (64 columns)
  for (int k0 = 0; k0 < K; k0 += 16) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (m0 + a_row < M && k0 + a_k4 < K) v = *reinterpret_cast<const float4 *>(A + (size_t)(m0 + a_row) * K + k0 + a_k4);
    As[a_k4 + 0][a_row] = v.x; As[a_k4 + 1][a_row] = v.y; As[a_k4 + 2][a_row] = v.z; As[a_k4 + 3][a_row] = v.w;
    float f[4] = {0.f, 0.f, 0.f, 0.f};
    if (k0 + b_k < K && n0 + b_w * 4 < N) unpack_int8x4(__ldg(Bq + (size_t)(k0 + b_k) * ND4 + (n0 >> 2) + b_w), f);
    *reinterpret_cast<float4 *>(&Bs[b_k][b_w * 4]) = make_float4(f[0], f[1], f[2], f[3]);
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
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int m = m0 + ty * 4 + i, n = n0 + tx * 4;
    if (m < M && n < N) epi_store4(epi, make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]), m, n);
  }
}

// Large M on the tensor cores: the packed words are expanded once per call to an FP32 weight in the [N,K] layout
// the tcgen05 GEMM reads (K contiguous). The integers are exact in TF32, so the product keeps the accuracy of the
// activation split alone. 32 k x 128 columns per CTA, transposed through shared memory so that both the word reads
// (along N) and the float writes (along K) are coalesced.
__global__ void __launch_bounds__(256)
int8_expand_nk_kernel(const uint32_t *__restrict__ Bq, int K, int N, float *__restrict__ Wt) {
  __shared__ float t[32][129];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int k0 = blockIdx.y * 32, w0 = blockIdx.x * 32, ND4 = N >> 2;
#pragma unroll
  for (int r = 0; r < 4; r++) {
    int k = warp + 8 * r;
    float f[4] = {0.f, 0.f, 0.f, 0.f};
    if (k0 + k < K && w0 + lane < ND4) unpack_int8x4(__ldg(Bq + (size_t)(k0 + k) * ND4 + w0 + lane), f);
    t[k][4 * lane + 0] = f[0]; t[k][4 * lane + 1] = f[1]; t[k][4 * lane + 2] = f[2]; t[k][4 * lane + 3] = f[3];
  }
  __syncthreads();
  for (int i = warp; i < 128; i += 8) {
    int n = w0 * 4 + i;
    if (n < N && k0 + lane < K) Wt[(size_t)n * K + k0 + lane] = t[lane][i];
  }
}

// ------------------------------------------------------------------------------------------------
// Load-time re-layout for a weight that is used many times: the prototype's words [K, N/4] (four columns of one k
// per word, other/int8-gemm.js:36-42) become bytes [N, K], K contiguous, so that one output column's codes are a
// contiguous run that 128-bit loads and bulk copies can stream (16 codes per load). 32 k x 128 columns per CTA.
__global__ void __launch_bounds__(256)
int8_relayout_nk_kernel(const uint32_t *__restrict__ Bq, int K, int N, uint8_t *__restrict__ out) {
  __shared__ uint32_t t[32][33];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int k0 = blockIdx.y * 32, w0 = blockIdx.x * 32, ND4 = N >> 2;
#pragma unroll
  for (int r = 0; r < 4; r++) {
    const int k = warp + 8 * r;
    t[k][lane] = (k0 + k < K && w0 + lane < ND4) ? __ldg(Bq + (size_t)(k0 + k) * ND4 + w0 + lane) : 0u;
  }
  __syncthreads();
  for (int i = tid; i < 128 * 8; i += 256) {
    const int nl = i >> 3, kq = i & 7;          // column within the tile, group of four k
    const int n = w0 * 4 + nl, k = k0 + 4 * kq;
    if (n >= N || k >= K) continue;             // K % 4 == 0: a group is whole or absent
    const int sh = 8 * (nl & 3);
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) word |= ((t[4 * kq + j][nl >> 2] >> sh) & 0xffu) << (8 * j);
    *reinterpret_cast<uint32_t *>(out + (size_t)n * K + k) = word;
  }
}

// Bytes [N, K] -> FP32 [N, K] (exact), for the tensor-core product of many rows.
__global__ void int8_expand_bytes_kernel(const uint8_t *__restrict__ q, size_t n16, float *__restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 w = ldg_stream4u(reinterpret_cast<const uint4 *>(q) + i);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
    float4 *o = reinterpret_cast<float4 *>(out) + 4 * i;
#pragma unroll
    for (int v = 0; v < 4; v++) {
      float f[4];
      unpack_int8x4(ws[v], f);
      o[v] = make_float4(f[0], f[1], f[2], f[3]);
    }
  }
}

// Up to four activation rows against a re-laid-out weight (bytes [N, K]): the int8 counterpart of
// gemv_block_kernel. One CTA per SM owns `cols` consecutive columns, i.e. one contiguous run of cols*K bytes,
// fetched into shared memory by bulk copies issued before the dependency wait. Work items are (column, K slice);
// a lane takes 16 codes per step (one 128-bit load), unpacks them exactly as the prototype does
// ((int32(word) << (24-8j)) >> 24, other/int8-gemm.js:126-131) and multiplies with the matching 16 activations;
// slices are summed in a fixed order and the per-column scale multiplies the finished sum.
// HBM-bound: bytes = K*N + 4*N + 4*M*(K+N). K % 16 == 0.
constexpr int kInt8BlockThreads = 512;
template <int M>
__global__ void __launch_bounds__(kInt8BlockThreads)
int8_block_gemv_kernel(const float *__restrict__ x, const uint8_t *__restrict__ Wq, const float *__restrict__ scale,
                       int K, int N, int cols, int wk, float *__restrict__ out, int *err) {
  extern __shared__ __align__(128) float smem[];
  constexpr int NT = kInt8BlockThreads, NW = NT / 32;
  uint8_t *wbuf = reinterpret_cast<uint8_t *>(smem);                     // [cols][K] bytes
  float *xs = smem + ((size_t)cols * K) / 4;                             // [M][K]
  float *red = xs + (size_t)M * K;
  const int red_floats = (max(cols * wk, NW) * M + 3) & ~3;
  uint64_t *bar = reinterpret_cast<uint64_t *>(red + red_floats);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int col0 = blockIdx.x * cols;
  const int ncol = min(cols, N - col0);
  if (tid == 0) {
    mbar_init(bar, 1);
    const uint32_t bytes = (uint32_t)ncol * (uint32_t)K;
    mbar_expect_tx(bar, bytes);
    for (uint32_t off = 0; off < bytes; off += 16384u)
      bulk_g2s(wbuf + off, Wq + (size_t)col0 * K + off, min(16384u, bytes - off), bar);
  }
  const int wk_log2 = 31 - __clz(wk);
  const int ks = warp & (wk - 1);
  const int K16 = K >> 4;
  const int beg = (int)(((unsigned)K16 * (unsigned)ks) >> wk_log2), end = (int)(((unsigned)K16 * (unsigned)(ks + 1)) >> wk_log2);
  pdl_launch_dependents();
  pdl_wait();
  {
    // A lane's 16 codes meet activations 16i..16i+15, four float4; stored as they come, the lanes of a warp would
    // read float4 number 4i+v at a stride of 64 bytes (four-way bank conflicts). Row m is therefore staged as four
    // planes, plane v holding float4 number 4i+v at position i, so that consecutive lanes read consecutive float4.
    const int K4 = K >> 2;
    for (int j = tid; j < M * K4; j += NT) {
      const int m = j / K4, idx = j - m * K4;
      reinterpret_cast<float4 *>(xs)[(size_t)m * K4 + (idx & 3) * K16 + (idx >> 2)] =
          __ldcg(reinterpret_cast<const float4 *>(x) + j);
    }
  }
  __syncthreads();
  const int landed = __syncthreads_and(mbar_wait(bar, 0, 1u << 20) ? 1 : 0);
  if (!landed) {
    if (tid == 0) atomicExch(err, 2);
    mbar_wait(bar, 0, 1u << 22);
    return;
  }
  const float4 *x4 = reinterpret_cast<const float4 *>(xs);
  constexpr int CG = M == 1 ? 4 : 2;  // columns per work item: they share the activation loads
  const int groups = (ncol + CG - 1) / CG;
  for (int it = warp; it < (groups << wk_log2); it += NW) {
    const int g = it >> wk_log2;
    const uint4 *w16[CG];
#pragma unroll
    for (int q = 0; q < CG; q++) w16[q] = reinterpret_cast<const uint4 *>(wbuf + (size_t)min(g * CG + q, ncol - 1) * K);
    float acc[CG][M];
#pragma unroll
    for (int q = 0; q < CG; q++)
#pragma unroll
      for (int m = 0; m < M; m++) acc[q][m] = 0.f;
#pragma unroll 2
    for (int i = beg + lane; i < end; i += 32) {
      float4 xv[M][4];
#pragma unroll
      for (int m = 0; m < M; m++)
#pragma unroll
        for (int v = 0; v < 4; v++) xv[m][v] = x4[(size_t)m * (K >> 2) + v * K16 + i];
#pragma unroll
      for (int q = 0; q < CG; q++) {
        const uint4 w = w16[q][i];
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int v = 0; v < 4; v++) {
          const float4 wf = unpack_int8x4_fast(ws[v]);
#pragma unroll
          for (int m = 0; m < M; m++) acc[q][m] += dot4(wf, xv[m][v]);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < CG; q++)
#pragma unroll
      for (int m = 0; m < M; m++) {
        const float v = warp_sum(acc[q][m]);
        if (lane == 0 && g * CG + q < ncol) red[((g * CG + q) * wk + ks) * M + m] = v;
      }
  }
  __syncthreads();
  for (int o = tid; o < ncol * M; o += NT) {
    const int c = o / M, m = o - c * M;
    float v = 0.f;
    for (int k = 0; k < wk; k++) v += red[(c * wk + k) * M + m];
    out[(size_t)m * N + col0 + c] = v * scale[col0 + c];
  }
}

}  // namespace wgpt
