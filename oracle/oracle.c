/*
 * CPU oracle: a plain-C restatement of the WGSL kernels and the forward pass of
 * 0hq/WebGPT, used ONLY as test infrastructure (parity checker and timed CPU
 * baseline). Nothing in the shipped library links, loads or calls this file.
 *
 * Parity pinning: the reference's own validation fixtures and weights are
 * Git-LFS stubs and its JavaScript cannot run without a browser, so this
 * restatement is "parity unpinned" against reference-generated artefacts.
 * It is pinned instead against (1) the known-answer patterns the reference's
 * manual harnesses construct (other/test.js:370-388, other/int8-gemm.js:25-62)
 * and (2) an independent implementation of the same mathematics
 * (HuggingFace GPT2LMHeadModel on identical weights) through committed
 * golden vectors.
 *
 * Every function cites the reference file:line it follows. All arrays are
 * row-major f32 unless stated. Summation orders follow the shaders (sequential
 * ascending-k multiply-add for the matmuls, strided partial sums followed by a
 * binary tree for the workgroup reductions).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ K1 ---- */
/* fastMatMul, instructions.js:179-319: C[m][n] = (sum_{k ascending} A[m][k]*B[k][n]) + bias[n],
 * accumulators start at zero (:239-246), one multiply-add per k (:256-301), the bias is added
 * after the loop (:304-314). B is [K,N]. bias may be NULL (the int8 prototype and the de-embed
 * have none). */
ORC_API void orc_matmul(const float *A, const float *B, const float *bias, float *C, int M, int K, int N) {
  const int NB = M < 8 ? 64 : 256; /* column block: an accumulator strip in L1; narrower when few rows must feed all threads */
#pragma omp parallel for collapse(2) schedule(static)
  for (int m = 0; m < M; m++) {
    for (int n0 = 0; n0 < N; n0 += NB) {
      int nb = N - n0 < NB ? N - n0 : NB;
      float acc[256];
      for (int j = 0; j < nb; j++) acc[j] = 0.0f;
      const float *a = A + (size_t)m * K;
      for (int k = 0; k < K; k++) {
        float av = a[k];
        const float *b = B + (size_t)k * N + n0;
        for (int j = 0; j < nb; j++) acc[j] = av * b[j] + acc[j];
      }
      float *c = C + (size_t)m * N + n0;
      if (bias)
        for (int j = 0; j < nb; j++) c[j] = acc[j] + bias[n0 + j];
      else
        for (int j = 0; j < nb; j++) c[j] = acc[j];
    }
  }
}

/* ------------------------------------------------------------------ K2 ---- */
/* elementWiseAddition, instructions.js:358-384. */
ORC_API void orc_residual(const float *a, const float *b, float *out, int M, int N) {
  size_t n = (size_t)M * N;
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; i++) out[i] = a[i] + b[i];
}

/* ---------------------------------------------------------------- K3/K4 --- */
/* Workgroup tree reduction used by normStats and softmax (instructions.js:481-486, :649-654):
 * op[col] += op[col+i] for i = wg/2, wg/4, ... 1. */
static float tree_sum(float *op, int wg) {
  for (int i = wg >> 1; i > 0; i >>= 1)
    for (int c = 0; c < i; c++) op[c] = op[c] + op[c + i];
  return op[0];
}

/* normStats (instructions.js:451-515) then norm (:517-550).
 * wg_size = 256 if N > 4096 else 64 (:412). mean = sum/N (:489); the variance sums
 * pow(x-mean,2) per thread and divides each thread's partial by N before the tree (:496-498);
 * stdev = sqrt(var + 1e-5) (:508); y = gamma*((x-mean)/stdev)+beta (:544-548).
 * stats (optional) receives [mean, stdev] per row (:511-512). */
ORC_API void orc_layernorm(const float *x, const float *gamma, const float *beta, float *out, float *stats, int M,
                           int N) {
  int wg = N > 4096 ? 256 : 64;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < M; r++) {
    float op[256];
    const float *row = x + (size_t)r * N;
    for (int c = 0; c < wg; c++) {
      float s = 0.0f;
      for (int i = c; i < N; i += wg) s = s + row[i];
      op[c] = s;
    }
    float mean = tree_sum(op, wg) / (float)N;
    for (int c = 0; c < wg; c++) {
      float s = 0.0f;
      for (int i = c; i < N; i += wg) {
        float d = row[i] - mean;
        s = s + d * d;
      }
      op[c] = s / (float)N;
    }
    float sd = sqrtf(tree_sum(op, wg) + 1e-5f);
    if (stats) {
      stats[2 * r] = mean;
      stats[2 * r + 1] = sd;
    }
    float *o = out + (size_t)r * N;
    for (int i = 0; i < N; i++) o[i] = gamma[i] * ((row[i] - mean) / sd) + beta[i];
  }
}

/* ------------------------------------------------------------------ K5 ---- */
/* softmax fusedShader, instructions.js:593-666. wg_size = 256 if cols > 4096 else 64 (:568).
 * max: per-thread strided max from -3.402823e38 (:601,:619-622), then the odd-size-safe
 * reduction of :629-636; sum of exp(x-max): strided partials + binary tree (:642-654);
 * y = exp(x-max)/sum (:661-663). */
ORC_API void orc_softmax(const float *x, float *out, int rows, int cols) {
  int wg = cols > 4096 ? 256 : 64;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; r++) {
    float op[256] = {0};
    const float *row = x + (size_t)r * cols;
    for (int c = 0; c < wg; c++) {
      float m = -3.402823e+38f;
      for (int i = c; i < cols; i += wg) m = fmaxf(m, row[i]);
      if (c < cols) op[c] = m;
    }
    int red = cols < wg ? cols : wg;
    for (int i = red >> 1; i > 0; i = red >> 1) {
      red = i + (red & 1);
      for (int c = 0; c < i; c++) op[c] = fmaxf(op[c], op[c + red]);
    }
    float mx = op[0];
    for (int c = 0; c < wg; c++) {
      float s = 0.0f;
      for (int i = c; i < cols; i += wg) s = s + expf(row[i] - mx);
      op[c] = s;
    }
    float sum = tree_sum(op, wg);
    float *o = out + (size_t)r * cols;
    for (int i = 0; i < cols; i++) o[i] = expf(row[i] - mx) / sum;
  }
}

/* ------------------------------------------------------------------ K6 ---- */
/* GELUShader, instructions.js:705-748: 0.5*(1+tanh(0.7978845608*(x+0.044715*x^3))) * x with
 * x < -10 -> 0 and x > 10 -> x (:711-727). pow(x,3) is taken as x*x*x (C semantics for a
 * negative base with an integral exponent). */
ORC_API float orc_gelu1(float x) {
  float x3 = x * x * x;
  float cdf = 0.5f * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x3)));
  float r = x * cdf;
  if (x < -10.0f) r = 0.0f;
  if (x > 10.0f) r = x;
  return r;
}
ORC_API void orc_gelu(const float *x, float *out, int M, int N) {
  size_t n = (size_t)M * N;
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; i++) out[i] = orc_gelu1(x[i]);
}

/* ------------------------------------------------------------------ K7 ---- */
/* EmbedBlock.newInstance, instructions.js:790-827: row i of the output is a copy of wte row
 * idx[i] (:795-809) added (K2, :821) to a copy of wpe rows 0..T-1 (:812-819). */
ORC_API void orc_embed(const uint32_t *idx, int T, int E, const float *wte, const float *wpe, float *out) {
  for (int t = 0; t < T; t++)
    for (int e = 0; e < E; e++) out[(size_t)t * E + e] = wte[(size_t)idx[t] * E + e] + wpe[(size_t)t * E + e];
}

/* ------------------------------------------------------------------ K8 ---- */
/* deEmbed, instructions.js:890-952 on the transposed wte chunks built at model.js:362:
 * logits[v] = sum_{k ascending} x_last[k] * wte[v][k], no bias. x_last is the last row of the
 * input (:849-856). Chunking only splits the v range (:858-882) and does not change values. */
ORC_API void orc_deembed(const float *x_last, int E, int V, const float *wte, float *logits) {
#pragma omp parallel for schedule(static)
  for (int v = 0; v < V; v++) {
    const float *w = wte + (size_t)v * E;
    float s = 0.0f;
    for (int k = 0; k < E; k++) s = x_last[k] * w[k] + s;
    logits[v] = s;
  }
}

/* ------------------------------------------------------------------ K9 ---- */
/* formatQShader, instructions.js:1101-1138: out[(c/hs)*hs*T + r*hs + c%hs] = Q[r][c]. */
ORC_API void orc_format_q(const float *Q, float *out, int T, int E, int hs) {
  for (int r = 0; r < T; r++)
    for (int c = 0; c < E; c++) out[(size_t)(c / hs) * hs * T + (size_t)r * hs + c % hs] = Q[(size_t)r * E + c];
}

/* ----------------------------------------------------------------- K10 ---- */
/* fusedWeightsShader, instructions.js:1141-1178. Qf is [H*T, hs]; Kmat is [T, E].
 * S[row][col] = (col <= row%T) ? scale * sum_i dot4(Qf[row][4i..], K[col][head*hs+4i..]) : -1e9.
 * The dot of each vec4 is formed first, then added to the running sum (:1168-1171);
 * the scale multiplies the finished sum (:1176). */
ORC_API void orc_attn_weights(const float *Qf, const float *Kmat, float *S, int T, int E, int H, float scale) {
  int hs = E / H;
#pragma omp parallel for schedule(static)
  for (int row = 0; row < H * T; row++) {
    int head = row / T, rm = row % T;
    const float *q = Qf + (size_t)row * hs;
    for (int col = 0; col < T; col++) {
      const float *k = Kmat + (size_t)col * E + head * hs;
      float sum = 0.0f;
      for (int i = 0; i < hs; i += 4) {
        float d = q[i] * k[i] + q[i + 1] * k[i + 1] + q[i + 2] * k[i + 2] + q[i + 3] * k[i + 3];
        sum = sum + d;
      }
      S[(size_t)row * T + col] = (col <= rm) ? sum * scale : -1e9f;
    }
  }
}

/* ----------------------------------------------------------------- K11 ---- */
/* newAttentionValuesShader, instructions.js:1180-1214: P is [H*T, T], V is [T, E];
 * O[t][c] = sum_{i=0..T-1 ascending} V[i][c] * P[(c/hs)*T*T + t*T + i]  (:1205-1212). */
ORC_API void orc_attn_values(const float *P, const float *V, float *O, int T, int E, int H) {
  int hs = E / H;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; t++) {
    for (int c = 0; c < E; c++) {
      int head = c / hs;
      const float *p = P + (size_t)head * T * T + (size_t)t * T;
      float s = 0.0f;
      for (int i = 0; i < T; i++) s = s + V[(size_t)i * E + c] * p[i];
      O[(size_t)t * E + c] = s;
    }
  }
}

/* AttentionBlock.newFusedInstance, instructions.js:985-1099: Q,K,V projections (K1 x3), formatQ,
 * fused weights, softmax over [H*T, T], values, output projection (K1). scratch sizes are
 * allocated here. out is [T,E]. */
ORC_API void orc_attention(const float *x, int T, int E, int H, float scale, const float *wq, const float *bq,
                           const float *wk, const float *bk, const float *wv, const float *bv, const float *wo,
                           const float *bo, float *out) {
  int hs = E / H;
  size_t te = (size_t)T * E, htt = (size_t)H * T * T;
  float *q = malloc(te * 4), *k = malloc(te * 4), *v = malloc(te * 4), *qf = malloc(te * 4);
  float *s = malloc(htt * 4), *p = malloc(htt * 4), *o = malloc(te * 4);
  orc_matmul(x, wq, bq, q, T, E, E);
  orc_matmul(x, wk, bk, k, T, E, E);
  orc_matmul(x, wv, bv, v, T, E, E);
  orc_format_q(q, qf, T, E, hs);
  orc_attn_weights(qf, k, s, T, E, H, scale);
  orc_softmax(s, p, H * T, T);
  orc_attn_values(p, v, o, T, E, H);
  orc_matmul(o, wo, bo, out, T, E, E);
  free(q); free(k); free(v); free(qf); free(s); free(p); free(o);
}

/* ----------------------------------------------------------------- K12 ---- */
/* int8 prototype, other/int8-gemm.js.
 * JS Math.round rounds halves toward +infinity: floor(x + 0.5). */
static double js_round(double x) { return floor(x + 0.5); }
/* Math.round((x / absmax) * 127): three separately rounded double operations, as JavaScript evaluates them;
 * the volatile keeps a compiler from contracting the multiply and the + 0.5 into one fused operation. */
static double js_quant(double x, double absmax) {
  volatile double t = x / absmax;
  t = t * 127.0;
  return js_round(t);
}

/* quantizeMatrix, other/int8-gemm.js:25-46: word w packs elements 4w..4w+3 of the flattened
 * row-major matrix, byte j = round(x/absmax*127) & 0xff. count must be a multiple of 4.
 * The arithmetic is JS double precision on f32 inputs. */
ORC_API void orc_int8_quantize(const float *x, size_t count, double absmax, int32_t *packed) {
  for (size_t i = 0; i < count; i += 4) {
    uint32_t w = 0;
    for (int j = 0; j < 4; j++) {
      int32_t q = (int32_t)js_quant((double)x[i + j], absmax);
      w |= ((uint32_t)q & 0xffu) << (8 * j);
    }
    packed[i / 4] = (int32_t)w;
  }
}

/* quantizeMatrix with the vector-wise scales its header asks for (other/int8-gemm.js:4): the same expression
 * round(x / absmax * 127) & 0xff (:36-42), packed four per word along N, but with absmax taken per output column n
 * of the row-major [K, N] matrix (:29-33 take it over the whole matrix). scale[n] = absmax_n / 127 as f32 is the
 * factor the dequant-GEMM multiplies by. A column of zeros quantises to zeros with scale 0 (the JS expression gives
 * NaN & 0xff = 0 there). per_column == 0 reproduces the prototype: one absmax for the matrix. N % 4 == 0. */
ORC_API void orc_int8_quantize_matrix(const float *w, int K, int N, int per_column, int32_t *packed, float *scale) {
  double *amax = calloc((size_t)N, sizeof(double));
  for (int k = 0; k < K; k++)
    for (int n = 0; n < N; n++) {
      double a = fabs((double)w[(size_t)k * N + n]);
      if (a > amax[n]) amax[n] = a;
    }
  if (!per_column) {
    double g = 0.0;
    for (int n = 0; n < N; n++) if (amax[n] > g) g = amax[n];
    for (int n = 0; n < N; n++) amax[n] = g;
  }
  for (int n = 0; n < N; n++) scale[n] = (float)(amax[n] / 127.0);
  for (int k = 0; k < K; k++)
    for (int n = 0; n < N; n += 4) {
      uint32_t word = 0;
      for (int j = 0; j < 4; j++) {
        double a = amax[n + j];
        int32_t q = a > 0.0 ? (int32_t)js_quant((double)w[(size_t)k * N + n + j], a) : 0;
        word |= ((uint32_t)q & 0xffu) << (8 * j);
      }
      packed[((size_t)k * N + n) / 4] = (int32_t)word;
    }
  free(amax);
}

/* The integer half of unpackInt8x4, other/int8-gemm.js:126-132: lane j = (v << (24-8j)) >> 24
 * with an arithmetic right shift. */
ORC_API void orc_int8_unpack(const int32_t *packed, size_t words, int8_t *out) {
  for (size_t w = 0; w < words; w++) {
    int32_t v = packed[w];
    for (int j = 0; j < 4; j++) out[4 * w + j] = (int8_t)(((int32_t)((uint32_t)v << (24 - 8 * j))) >> 24);
  }
}

/* int8 dequant-GEMM, other/int8-gemm.js:117-229: K1 without bias where each B element is
 * f32(q)/127.0*absmax (:127-130). Here the scale is per output column: the file's own header
 * asks for vector-wise scales (:4); scale[n] plays the role of absmax/127, i.e. the reference
 * expression with absmax_n = 127*scale[n] reduces to f32(q)*scale[n] up to one rounding.
 * literal != 0 evaluates the reference's literal form f32(q)/127.0f*absmax_n instead.
 * Bq is [K, N/4] words; byte j of word w in row k is column 4w+j. */
ORC_API void orc_int8_matmul(const float *A, const int32_t *Bq, const float *scale, float *C, int M, int K, int N,
                             int literal) {
  int ND4 = N / 4;
#pragma omp parallel for collapse(2) schedule(static)
  for (int m = 0; m < M; m++) {
    for (int w0 = 0; w0 < ND4; w0 += 64) {
      int wb = ND4 - w0 < 64 ? ND4 - w0 : 64;
      float acc[256];
      for (int j = 0; j < 4 * wb; j++) acc[j] = 0.0f;
      for (int k = 0; k < K; k++) {
        float av = A[(size_t)m * K + k];
        const int32_t *b = Bq + (size_t)k * ND4 + w0;
        for (int w = 0; w < wb; w++) {
          int32_t v = b[w];
          for (int j = 0; j < 4; j++) {
            int32_t q = ((int32_t)((uint32_t)v << (24 - 8 * j))) >> 24;
            int n = 4 * (w0 + w) + j;
            float bw = literal ? (float)q / 127.0f * (127.0f * scale[n]) : (float)q * scale[n];
            acc[4 * w + j] = av * bw + acc[4 * w + j];
          }
        }
      }
      for (int j = 0; j < 4 * wb; j++) C[(size_t)m * N + 4 * w0 + j] = acc[j];
    }
  }
}

/* --------------------------------------------------------------- model ---- */
/* Weight set in the on-disk convention of model.js:341,371,382-383,409-420: tensors[] holds
 * wte [V,E], wpe [n_ctx,E], ln_f.weight, ln_f.bias, then per layer
 * ln_1.w, ln_1.b, c_attn.w [E,3E], c_attn.b [3E], attn.c_proj.w [E,E], attn.c_proj.b,
 * ln_2.w, ln_2.b, c_fc.w [E,4E], c_fc.b, mlp.c_proj.w [4E,E], mlp.c_proj.b. */
typedef struct {
  int n_layer, n_head, n_embd, n_ctx, vocab;
  const float **tensors; /* 4 + 12*n_layer entries, owned by the caller */
  float **wq, **wk, **wv; /* split copies, [E,E] each (model.js:456-468) */
} orc_model;

/* fetchAndSplitQKVWeightTensors, model.js:456-468: transpose [E,3E] to [3E,E], slice three
 * [E,E] blocks, transpose each back. Net effect: W_x[k][n] = c_attn[k][x*E + n]. */
static float *split_qkv(const float *cattn, int E, int which) {
  float *w = malloc((size_t)E * E * 4);
  for (int k = 0; k < E; k++) memcpy(w + (size_t)k * E, cattn + (size_t)k * 3 * E + (size_t)which * E, (size_t)E * 4);
  return w;
}

ORC_API orc_model *orc_model_create(int n_layer, int n_head, int n_embd, int n_ctx, int vocab, const float **tensors) {
  /* loadParameters checks, model.js:294-297 */
  if (n_embd % 4 || n_embd % n_head || (n_embd / n_head) % 4) return NULL;
  orc_model *m = calloc(1, sizeof *m);
  m->n_layer = n_layer; m->n_head = n_head; m->n_embd = n_embd; m->n_ctx = n_ctx; m->vocab = vocab;
  m->tensors = malloc(sizeof(float *) * (4 + 12 * (size_t)n_layer));
  memcpy(m->tensors, tensors, sizeof(float *) * (4 + 12 * (size_t)n_layer));
  m->wq = malloc(sizeof(float *) * n_layer); m->wk = malloc(sizeof(float *) * n_layer);
  m->wv = malloc(sizeof(float *) * n_layer);
  for (int l = 0; l < n_layer; l++) {
    const float *ca = tensors[4 + 12 * l + 2];
    m->wq[l] = split_qkv(ca, n_embd, 0); m->wk[l] = split_qkv(ca, n_embd, 1); m->wv[l] = split_qkv(ca, n_embd, 2);
  }
  return m;
}

ORC_API void orc_model_destroy(orc_model *m) {
  if (!m) return;
  for (int l = 0; l < m->n_layer; l++) { free(m->wq[l]); free(m->wk[l]); free(m->wv[l]); }
  free(m->wq); free(m->wk); free(m->wv); free((void *)m->tensors); free(m);
}

/* Number of [T,E] activation taps orc_model_run can record: tok_pos_emb, then per block
 * ln1, attn, r1, ln2, mlp, r2 (other/validation/validation.js:113-134), then ln_f. */
ORC_API int orc_model_num_taps(const orc_model *m) { return 2 + 6 * m->n_layer; }

/* GPT.run, model.js:104-268: one forward pass over the whole window idx[0..T-1]; writes the
 * vocab logits of the last position. taps (optional) receives num_taps blocks of [T,E]. */
ORC_API int orc_model_run(const orc_model *m, const uint32_t *idx, int T, float *logits, float *taps) {
  int E = m->n_embd, H = m->n_head, F = 4 * E;
  if (T < 1 || T > m->n_ctx) return -1;
  for (int t = 0; t < T; t++) if (idx[t] >= (uint32_t)m->vocab) return -2;
  float scale = (float)(1.0 / sqrt((double)(E / H))); /* model.js:321 f64, stored f32 at instructions.js:1038 */
  size_t te = (size_t)T * E;
  float *x = malloc(te * 4), *h = malloc(te * 4), *a = malloc(te * 4), *f = malloc((size_t)T * F * 4),
        *g = malloc((size_t)T * F * 4);
  int tap = 0;
#define TAP(buf) do { if (taps) memcpy(taps + (size_t)(tap++) * te, (buf), te * 4); } while (0)
  orc_embed(idx, T, E, m->tensors[0], m->tensors[1], x); /* model.js:118 */
  TAP(x);
  for (int l = 0; l < m->n_layer; l++) {
    const float **w = m->tensors + 4 + 12 * l;
    orc_layernorm(x, w[0], w[1], h, NULL, T, E); /* model.js:126 */
    TAP(h);
    orc_attention(h, T, E, H, scale, m->wq[l], w[3], m->wk[l], w[3] + E, m->wv[l], w[3] + 2 * E, w[4], w[5],
                  a); /* model.js:137; bias split model.js:470-482 */
    TAP(a);
    orc_residual(a, x, x, T, E); /* model.js:159 */
    TAP(x);
    orc_layernorm(x, w[6], w[7], h, NULL, T, E); /* model.js:165 */
    TAP(h);
    orc_matmul(h, w[8], w[9], f, T, E, F); /* model.js:176 */
    orc_gelu(f, g, T, F); /* model.js:188 */
    orc_matmul(g, w[10], w[11], a, T, F, E); /* model.js:193 */
    TAP(a);
    orc_residual(a, x, x, T, E); /* model.js:205 */
    TAP(x);
  }
  orc_layernorm(x, m->tensors[2], m->tensors[3], h, NULL, T, E); /* model.js:224 (all T rows) */
  TAP(h);
  orc_deembed(h + (size_t)(T - 1) * E, E, m->vocab, m->tensors[0], logits); /* model.js:229 */
#undef TAP
  free(x); free(h); free(a); free(f); free(g);
  return 0;
}

/* Greedy pick = selectTopK(logits, 1) -> cpuSoftmax of one value -> index 0
 * (globals.js:47-74): the arg-max, lowest index on exact ties (stable descending sort). */
ORC_API uint32_t orc_argmax(const float *logits, int V) {
  int best = 0;
  for (int v = 1; v < V; v++) if (logits[v] > logits[best]) best = v;
  return (uint32_t)best;
}

/* GPT.generate with top_k = 1, model.js:53-102: every new token re-runs the whole window
 * history.slice(-n_ctx) (:69,:73; the useAttCache flag of :70 is ignored by run).
 * history_out receives n_prompt + n_new ids. logits_trace (optional) receives the vocab logits
 * of each step. Returns 0 on success. */
ORC_API int orc_generate_greedy(const orc_model *m, const uint32_t *prompt, int n_prompt, int n_new,
                                uint32_t *history_out, float *logits_trace) {
  int V = m->vocab;
  float *logits = malloc((size_t)V * 4);
  memcpy(history_out, prompt, (size_t)n_prompt * 4);
  int len = n_prompt;
  for (int i = 0; i < n_new; i++) {
    int T = len < m->n_ctx ? len : m->n_ctx;
    int rc = orc_model_run(m, history_out + (len - T), T, logits, NULL);
    if (rc) { free(logits); return rc; }
    if (logits_trace) memcpy(logits_trace + (size_t)i * V, logits, (size_t)V * 4);
    history_out[len++] = orc_argmax(logits, V);
  }
  free(logits);
  return 0;
}

/* ------------------------------------------------- KV-cached CPU decode ---- */
/* Same mathematics as orc_model_run restricted to the newest row, with the K and V rows of
 * earlier positions kept from earlier steps (causal attention makes them independent of later
 * tokens). Only valid while the window does not slide (history <= n_ctx, the condition of
 * model.js:70). Used for the timed CPU baseline and to check cached == recomputed. */
typedef struct {
  const orc_model *m;
  int len;
  float *k, *v; /* [n_layer][n_ctx][E] */
} orc_kv;

ORC_API orc_kv *orc_kv_create(const orc_model *m) {
  orc_kv *s = calloc(1, sizeof *s);
  size_t n = (size_t)m->n_layer * m->n_ctx * m->n_embd;
  s->m = m; s->k = malloc(n * 4); s->v = malloc(n * 4);
  return s;
}
ORC_API void orc_kv_destroy(orc_kv *s) { if (s) { free(s->k); free(s->v); free(s); } }
ORC_API void orc_kv_reset(orc_kv *s) { s->len = 0; }

/* Feeds one token at position s->len; writes the vocab logits for that position. */
ORC_API int orc_kv_step(orc_kv *s, uint32_t id, float *logits) {
  const orc_model *m = s->m;
  int E = m->n_embd, H = m->n_head, F = 4 * E, hs = E / H, pos = s->len;
  if (pos >= m->n_ctx || id >= (uint32_t)m->vocab) return -1;
  float scale = (float)(1.0 / sqrt((double)hs));
  float *x = malloc((size_t)E * 4), *h = malloc((size_t)E * 4), *q = malloc((size_t)E * 4),
        *o = malloc((size_t)E * 4), *a = malloc((size_t)E * 4), *f = malloc((size_t)F * 4),
        *g = malloc((size_t)F * 4), *sc = malloc((size_t)(pos + 1) * 4), *p = malloc((size_t)(pos + 1) * 4);
  for (int e = 0; e < E; e++) x[e] = m->tensors[0][(size_t)id * E + e] + m->tensors[1][(size_t)pos * E + e];
  for (int l = 0; l < m->n_layer; l++) {
    const float **w = m->tensors + 4 + 12 * l;
    float *kc = s->k + ((size_t)l * m->n_ctx) * E, *vc = s->v + ((size_t)l * m->n_ctx) * E;
    orc_layernorm(x, w[0], w[1], h, NULL, 1, E);
    orc_matmul(h, m->wq[l], w[3], q, 1, E, E);
    orc_matmul(h, m->wk[l], w[3] + E, kc + (size_t)pos * E, 1, E, E);
    orc_matmul(h, m->wv[l], w[3] + 2 * E, vc + (size_t)pos * E, 1, E, E);
    for (int hd = 0; hd < H; hd++) {
      for (int j = 0; j <= pos; j++) {
        const float *kk = kc + (size_t)j * E + hd * hs, *qq = q + hd * hs;
        float sum = 0.0f;
        for (int i = 0; i < hs; i += 4)
          sum = sum + (qq[i] * kk[i] + qq[i + 1] * kk[i + 1] + qq[i + 2] * kk[i + 2] + qq[i + 3] * kk[i + 3]);
        sc[j] = sum * scale;
      }
      orc_softmax(sc, p, 1, pos + 1);
      for (int c = 0; c < hs; c++) {
        float sum = 0.0f;
        for (int j = 0; j <= pos; j++) sum = sum + vc[(size_t)j * E + hd * hs + c] * p[j];
        o[hd * hs + c] = sum;
      }
    }
    orc_matmul(o, w[4], w[5], a, 1, E, E);
    orc_residual(a, x, x, 1, E);
    orc_layernorm(x, w[6], w[7], h, NULL, 1, E);
    orc_matmul(h, w[8], w[9], f, 1, E, F);
    orc_gelu(f, g, 1, F);
    orc_matmul(g, w[10], w[11], a, 1, F, E);
    orc_residual(a, x, x, 1, E);
  }
  orc_layernorm(x, m->tensors[2], m->tensors[3], h, NULL, 1, E);
  if (logits) orc_deembed(h, E, m->vocab, m->tensors[0], logits);
  s->len = pos + 1;
  free(x); free(h); free(q); free(o); free(a); free(f); free(g); free(sc); free(p);
  return 0;
}

/* Greedy generation through the KV cache: prompt tokens are fed one by one, then n_new
 * arg-max tokens. Requires n_prompt + n_new <= n_ctx. */
ORC_API int orc_kv_generate_greedy(orc_kv *s, const uint32_t *prompt, int n_prompt, int n_new, uint32_t *new_ids) {
  int V = s->m->vocab;
  if (n_prompt + n_new > s->m->n_ctx) return -1;
  float *logits = malloc((size_t)V * 4);
  orc_kv_reset(s);
  for (int i = 0; i < n_prompt; i++)
    if (orc_kv_step(s, prompt[i], i == n_prompt - 1 ? logits : NULL)) { free(logits); return -2; }
  for (int i = 0; i < n_new; i++) {
    new_ids[i] = orc_argmax(logits, V);
    if (i + 1 < n_new && orc_kv_step(s, new_ids[i], logits)) { free(logits); return -3; }
  }
  free(logits);
  return 0;
}

/* ------------------------------------------------- top-k sampling ---- */
/* One sampling step of GPT.generate, model.js:81-83, with the uniform random number supplied by the caller
 * (the reference draws Math.random() inside sampleFromDistribution, globals.js:48):
 *   selectTopK (globals.js:66-74): indices sorted by descending logit with a stable sort, so equal values keep
 *     ascending index order (-0 and +0 compare equal there); the first top_k are kept;
 *   cpuSoftmax (globals.js:59-64): exp((v - max) / temperature) in double precision, summed left to right;
 *   sampleFromDistribution (globals.js:47-57): the first i whose running sum exceeds u, else the last.
 * Returns the chosen vocabulary index; the selected indices are written to top_idx (top_k entries) when not NULL. */
ORC_API uint32_t orc_sample_topk(const float *logits, int V, int top_k, double temperature, double u,
                                 uint32_t *top_idx) {
  if (top_k > V) top_k = V;
  if (top_k < 1) top_k = 1;
  uint32_t *sel = malloc((size_t)top_k * 4);
  /* insertion into a descending list; a later index never displaces an equal earlier one */
  int n = 0;
  for (int v = 0; v < V; v++) {
    float x = logits[v];
    if (n == top_k && !(x > logits[sel[n - 1]])) continue;
    int j = n < top_k ? n : top_k - 1;
    while (j > 0 && x > logits[sel[j - 1]]) { sel[j] = sel[j - 1]; j--; }
    sel[j] = (uint32_t)v;
    if (n < top_k) n++;
  }
  double *e = malloc((size_t)top_k * sizeof(double));
  double maxv = (double)logits[sel[0]];
  for (int j = 1; j < top_k; j++) if ((double)logits[sel[j]] > maxv) maxv = (double)logits[sel[j]];
  double sum = 0.0;
  for (int j = 0; j < top_k; j++) { e[j] = exp(((double)logits[sel[j]] - maxv) / temperature); sum += e[j]; }
  int pick = top_k - 1;
  double cum = 0.0;
  for (int j = 0; j < top_k; j++) {
    cum += e[j] / sum;
    if (u < cum) { pick = j; break; }
  }
  uint32_t id = sel[pick];
  if (top_idx) memcpy(top_idx, sel, (size_t)top_k * 4);
  free(e);
  free(sel);
  return id;
}

/* Sampled generation through the KV cache: like orc_kv_generate_greedy with orc_sample_topk as the pick;
 * uniforms holds one number per new token. Requires n_prompt + n_new <= n_ctx. */
ORC_API int orc_kv_generate_sample(orc_kv *s, const uint32_t *prompt, int n_prompt, int n_new, int top_k,
                                   double temperature, const double *uniforms, uint32_t *new_ids) {
  int V = s->m->vocab;
  if (n_prompt + n_new > s->m->n_ctx) return -1;
  float *logits = malloc((size_t)V * 4);
  orc_kv_reset(s);
  for (int i = 0; i < n_prompt; i++)
    if (orc_kv_step(s, prompt[i], i == n_prompt - 1 ? logits : NULL)) { free(logits); return -2; }
  for (int i = 0; i < n_new; i++) {
    new_ids[i] = orc_sample_topk(logits, V, top_k, temperature, uniforms[i], NULL);
    if (i + 1 < n_new && orc_kv_step(s, new_ids[i], logits)) { free(logits); return -3; }
  }
  free(logits);
  return 0;
}

/* Sampled generation by full-window recompute, the reference's own loop (model.js:53-102). */
ORC_API int orc_generate_sample(const orc_model *m, const uint32_t *prompt, int n_prompt, int n_new, int top_k,
                                double temperature, const double *uniforms, uint32_t *history_out) {
  int V = m->vocab;
  float *logits = malloc((size_t)V * 4);
  memcpy(history_out, prompt, (size_t)n_prompt * 4);
  int len = n_prompt;
  for (int i = 0; i < n_new; i++) {
    int T = len < m->n_ctx ? len : m->n_ctx;
    int rc = orc_model_run(m, history_out + (len - T), T, logits, NULL);
    if (rc) { free(logits); return rc; }
    history_out[len++] = orc_sample_topk(logits, V, top_k, temperature, uniforms[i], NULL);
  }
  free(logits);
  return 0;
}

/* Visualiser fragment shader, visuals.js:104-135: pixel (x,y) reads buf[y*n_embd + x] (the canvas is n_embd x
 * n_ctx pixels and fragCoord is the pixel centre, :105-110), v = 0.1*value (:115); hdrColorMapping with threshold 1
 * (:120-135): v<0 -> b=-v, and g=-v-1 below -1; else r=v, and g=v-1 above 1; g=min(g,0.7). The vec4 starts at
 * zero, so alpha stays 0. The 8-bit unorm target clamps to [0,1] and rounds to nearest. out: n*4 bytes RGBA. */
ORC_API void orc_heatmap(const float *buf, size_t n, uint8_t *out) {
  for (size_t i = 0; i < n; i++) {
    float v = buf[i] * 0.1f, r = 0.f, g = 0.f, b = 0.f;
    if (v < 0.f) { b = -v; if (v < -1.0f) g = -v - 1.0f; }
    else { r = v; if (v > 1.0f) g = v - 1.0f; }
    g = fminf(g, 0.7f);
    float c[3] = {r, g, b};
    for (int k = 0; k < 3; k++) out[4 * i + k] = (uint8_t)floorf(fminf(fmaxf(c[k], 0.f), 1.f) * 255.f + 0.5f);
    out[4 * i + 3] = 0;
  }
}

/* Caps the OpenMP team. A container may see every core of the host while being allowed only a few. */
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
