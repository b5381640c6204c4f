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
#include "common.cuh"

namespace wgpt {

// ------------------------------------------------------------------------------------------------
// x: [M, K] rows at stride ldx; Wt: [N, K]. CTA = 8 warps = (8/WK) column groups x WK slices of K.
// Each warp accumulates CPW columns over its K slice for all M rows.
// Dynamic shared memory: M*K floats (staged, optionally normalised, input rows) + 8*CPW*M partial sums.
template <int M, int WK, int CPW>
__global__ void __launch_bounds__(256)
gemv_nk_kernel(const float *__restrict__ x, size_t ldx, const float *__restrict__ gamma,
               const float *__restrict__ beta, const float *__restrict__ Wt, int K, int N, Epilogue epi,
               int prefetch) {
  extern __shared__ __align__(16) float smem[];
  float *xs = smem;
  float *red = smem + (size_t)M * K;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K4 = K >> 2;
  constexpr int WC = 8 / WK;
  const int wc = warp / WK, wk = warp % WK;
  const int col0 = (blockIdx.x * WC + wc) * CPW;
  const int beg = (int)(((long long)K4 * wk) / WK), end = (int)(((long long)K4 * (wk + 1)) / WK);
  const float4 *w4[CPW];
#pragma unroll
  for (int c = 0; c < CPW; c++) {
    int col = col0 + c < N ? col0 + c : N - 1;  // clamp: out-of-range columns read a valid row, never stored
    w4[c] = reinterpret_cast<const float4 *>(Wt + (size_t)col * K);
  }
  // ---- before the dependency wait: let the next kernel start, and pull this warp's weight slice (which no
  // kernel writes) towards L2 so that the HBM stream does not stop at the kernel boundary ----
  pdl_launch_dependents();
  if (prefetch && lane == 0 && end > beg) {
#pragma unroll
    for (int c = 0; c < CPW; c++) prefetch_l2(w4[c] + beg, (uint32_t)(end - beg) * 16u);
  }
  pdl_wait();

  // ---- stage the input rows; one warp per row does the LayerNorm (instructions.js:451-550) ----
  for (int m = warp; m < M; m += 8) {
    const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)m * ldx);
    float4 *dst = reinterpret_cast<float4 *>(xs + (size_t)m * K);
    if (gamma == nullptr) {
      for (int i = lane; i < K4; i += 32) dst[i] = __ldcg(src + i);
    } else {
      float s = 0.f;
      for (int i = lane; i < K4; i += 32) {
        float4 v = __ldcg(src + i);
        dst[i] = v;
        s += (v.x + v.y) + (v.z + v.w);
      }
      float mean = warp_sum(s) / (float)K;
      float q = 0.f;
      for (int i = lane; i < K4; i += 32) {
        float4 v = dst[i];
        float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
        q += (a * a + b * b) + (c * c + d * d);
      }
      float sd = sqrtf(warp_sum(q) / (float)K + 1e-5f);
      const float4 *g4 = reinterpret_cast<const float4 *>(gamma);
      const float4 *b4 = reinterpret_cast<const float4 *>(beta);
      for (int i = lane; i < K4; i += 32) {
        float4 v = dst[i], g = g4[i], b = b4[i];
        dst[i] = make_float4(g.x * ((v.x - mean) / sd) + b.x, g.y * ((v.y - mean) / sd) + b.y,
                             g.z * ((v.z - mean) / sd) + b.z, g.w * ((v.w - mean) / sd) + b.w);
      }
    }
  }
  __syncthreads();

  // ---- stream the weight rows ----
  float acc[CPW][M];
#pragma unroll
  for (int c = 0; c < CPW; c++)
#pragma unroll
    for (int m = 0; m < M; m++) acc[c][m] = 0.f;

  const float4 *xs4 = reinterpret_cast<const float4 *>(xs);
#pragma unroll 4
  for (int i = beg + lane; i < end; i += 32) {
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
  // ---- sum the K slices in a fixed order, apply the epilogue ----
  if (tid < WC * CPW * M) {
    int m = tid % M, c = (tid / M) % CPW, g = tid / (M * CPW);
    int n = (blockIdx.x * WC + g) * CPW + c;
    if (n < N) {
      float v = 0.f;
#pragma unroll
      for (int k = 0; k < WK; k++) v += red[((g * WK + k) * CPW + c) * M + m];
      epi_store(epi, v, m, n);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Weight in the reference layout W[K,N]. Thread owns 4 consecutive columns; a warp covers 128 columns of one
// k row per load (512 contiguous bytes); the CTA's 8 warps and gridDim.y CTAs split K.
// part receives [gridDim.y][M][N] partial sums (scratch); gemv_kn_reduce_kernel adds them in order.
template <int M>
__global__ void __launch_bounds__(256)
gemv_kn_partial_kernel(const float *__restrict__ x, const float *__restrict__ W, int K, int N,
                       float *__restrict__ part) {
  extern __shared__ __align__(16) float smem[];  // xs[M][kslice] + red[8][M][128]
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

__global__ void gemv_kn_reduce_kernel(const float *__restrict__ part, int ksplit, int M, int N, Epilogue epi) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;  // float4 index over [M, N/4]
  int N4 = N >> 2;
  if (i >= M * N4) return;
  int m = i / N4, n = (i - m * N4) * 4;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k = 0; k < ksplit; k++) {
    float4 v = *reinterpret_cast<const float4 *>(part + ((size_t)k * M + m) * N + n);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  epi_store4(epi, s, m, n);
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
