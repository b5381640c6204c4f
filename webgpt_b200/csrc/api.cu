// C ABI of webgpt_b200 (declared in include/webgpt_b200.h): device/buffer management, the per-operator entry
// points mirroring the reference's instruction classes, and the model/session level that mirrors class GPT.
#include "../../include/webgpt_b200.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "attention.cuh"
#include "common.cuh"
#include "decode_fused.cuh"
#include "elementwise.cuh"
#include "gemm_tc.cuh"
#include "gemm_tc2.cuh"
#include "int8.cuh"
#include "sampling.cuh"
#include "matmul.cuh"

using namespace wgpt;

#define WGPT_EXPORT extern "C" __attribute__((visibility("default")))

// ------------------------------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";

static int32_t fail(int32_t code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
  return code;
}

#define CK(call)                                                                                   \
  do {                                                                                             \
    cudaError_t e__ = (call);                                                                      \
    if (e__ != cudaSuccess)                                                                        \
      return fail(e__ == cudaErrorMemoryAllocation ? WGPT_ERR_OOM : WGPT_ERR_CUDA, "%s: %s", #call, \
                  cudaGetErrorString(e__));                                                        \
  } while (0)

#define TRY(call)                 \
  do {                            \
    int32_t rc__ = (call);        \
    if (rc__ != WGPT_OK) return rc__; \
  } while (0)

#define REQUIRE(cond, code, ...) \
  do {                           \
    if (!(cond)) return fail((code), __VA_ARGS__); \
  } while (0)

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------------------------------------ device
struct wgpt_device {
  int ordinal;
  cudaStream_t stream;
  int precision;
  uint64_t launches;
  int sm_count;
  size_t smem_optin;
  void *scratch;  // library-owned workspace (split-K partial sums, temporaries of wgpt_attention)
  size_t scratch_cap;
  uint64_t scratch_gen;  // bumped whenever the workspace moves: recorded pass lists hold its old address
  int *d_err;     // device-side error word (out-of-range token id)
  float *tc_scratch;  // split-K partial tiles of the tensor-core GEMM (fixed size)
  size_t tc_scratch_bytes;
  bool pdl;       // launch the decode-chain kernels with programmatic dependent launch (WGPT_PDL=0 turns it off)
  bool graphs;    // replay decode steps as a CUDA graph (WGPT_GRAPH=0 turns it off)
  bool capturing;   // between wgpt_graph_begin and wgpt_graph_end
  uint64_t capture_launch0;
  bool block_gemv;  // layer GEMVs through gemv_block_kernel (WGPT_BLOCK_GEMV=0: register-streaming kernel)
  int deembed_tc_min_rows;   // fewest sequences whose de-embedding runs on the tensor-core GEMM (WGPT_DEEMBED_TC_ROWS)
  int gemv_stream_max_rows;  // most rows the register-streaming GEMV takes for a layer product (WGPT_GEMV_MAX_ROWS)
  unsigned int *d_work;  // two counters of gemv_loop_kernel (left zero by every launch)
  bool loop_gemv;     // products against matrices larger than L2 through gemv_loop_kernel (WGPT_LOOP_GEMV=0: off)
  bool fused_decode;  // single-sequence decode with two kernels per block (WGPT_FUSED_DECODE=0 turns it off)
};

#define LAUNCH(dev, kernel, grid, block, smem, ...)                       \
  do {                                                                    \
    kernel<<<(grid), (block), (smem), (dev)->stream>>>(__VA_ARGS__);      \
    (dev)->launches++;                                                    \
    CK(cudaGetLastError());                                               \
  } while (0)

// Launch for kernels that call pdl_wait() before touching anything an earlier kernel wrote: with dev->pdl they
// carry the programmatic-serialisation attribute and may start while their predecessor is still running.
template <typename... KArgs, typename... Args>
static cudaError_t launch_ex(bool pdl, int cluster_z, cudaStream_t stream, void (*kernel)(KArgs...), dim3 grid,
                             dim3 block, size_t smem, Args... args);

// Launch with thread-block clusters of cluster_x CTAs along x (and programmatic dependent launch if pdl).
template <typename P>
static cudaError_t launch_cluster_x(bool pdl, int cluster_x, cudaStream_t stream, void (*kernel)(P), dim3 grid,
                                    dim3 block, size_t smem, const P &arg) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
  }
  attr[n].id = cudaLaunchAttributeClusterDimension;
  attr[n].val.clusterDim.x = (unsigned)cluster_x;
  attr[n].val.clusterDim.y = 1;
  attr[n].val.clusterDim.z = 1;
  n++;
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, arg);
}

template <typename... KArgs, typename... Args>
static cudaError_t launch_ex(bool pdl, int cluster_z, cudaStream_t stream, void (*kernel)(KArgs...), dim3 grid,
                             dim3 block, size_t smem, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
  }
  if (cluster_z > 1) {  // thread-block clusters along z
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = (unsigned)cluster_z;
    n++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define LAUNCH_PDL(dev, kernel, grid, block, smem, ...)                                          \
  do {                                                                                           \
    CK(launch_ex((dev)->pdl, 0, (dev)->stream, kernel, dim3(grid), dim3(block), (smem), __VA_ARGS__)); \
    (dev)->launches++;                                                                           \
  } while (0)

static int32_t use(wgpt_device *dev) {
  REQUIRE(dev != nullptr, WGPT_ERR_ARG, "device handle is null");
  CK(cudaSetDevice(dev->ordinal));
  return WGPT_OK;
}

// Grows the workspace. Work already enqueued may still be using the old block, so drain first.
static int32_t scratch_reserve(wgpt_device *dev, size_t bytes) {
  if (bytes <= dev->scratch_cap) return WGPT_OK;
  REQUIRE(!dev->capturing, WGPT_ERR_STATE,
          "the workspace would have to grow while a pass list is being recorded: run the pass list once first");
  CK(cudaStreamSynchronize(dev->stream));
  if (dev->scratch) CK(cudaFree(dev->scratch));
  dev->scratch = nullptr;
  dev->scratch_cap = 0;
  size_t cap = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
  CK(cudaMalloc(&dev->scratch, cap));
  dev->scratch_cap = cap;
  dev->scratch_gen++;
  return WGPT_OK;
}

// Calls that synchronise the stream (or free memory a recording may name) are not valid while a pass list is
// being recorded: a synchronise on a capturing stream would invalidate the capture.
#define NOT_RECORDING(dev, what)                                                                       \
  REQUIRE(!(dev)->capturing, WGPT_ERR_STATE, "%s is not valid between wgpt_graph_begin and wgpt_graph_end", what)

WGPT_EXPORT int32_t wgpt_abi_version(void) { return WGPT_ABI_VERSION; }
WGPT_EXPORT const char *wgpt_last_error(void) { return g_err; }

WGPT_EXPORT int32_t wgpt_device_create(int32_t ordinal, wgpt_device **out) {
  REQUIRE(out != nullptr, WGPT_ERR_ARG, "out is null");
  *out = nullptr;
  int count = 0;
  CK(cudaGetDeviceCount(&count));
  REQUIRE(ordinal >= 0 && ordinal < count, WGPT_ERR_ARG, "device ordinal %d out of range (%d devices)", ordinal, count);
  CK(cudaSetDevice(ordinal));
  cudaDeviceProp prop;
  CK(cudaGetDeviceProperties(&prop, ordinal));
  // These kernels are built for sm_100a only; there is no other code path.
  REQUIRE(prop.major == 10, WGPT_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library contains sm_100a code only",
          ordinal, prop.major, prop.minor);
  wgpt_device *dev = new wgpt_device();
  dev->ordinal = ordinal;
  dev->precision = WGPT_PRECISION_TF32X3;  // FP32-class accuracy on the tensor cores; see wgpt_device_set_precision
  dev->launches = 0;
  dev->sm_count = prop.multiProcessorCount;
  dev->smem_optin = prop.sharedMemPerBlockOptin;
  dev->scratch = nullptr;
  dev->scratch_cap = 0;
  dev->scratch_gen = 0;
  dev->d_err = nullptr;
  dev->d_work = nullptr;
  const char *ev = getenv("WGPT_PDL");
  dev->pdl = !(ev && ev[0] == '0');
  ev = getenv("WGPT_GRAPH");
  dev->graphs = !(ev && ev[0] == '0');
  ev = getenv("WGPT_BLOCK_GEMV");
  dev->block_gemv = !(ev && ev[0] == '0');
  ev = getenv("WGPT_DEEMBED_TC_ROWS");
  dev->deembed_tc_min_rows = ev ? atoi(ev) : 6;
  ev = getenv("WGPT_GEMV_MAX_ROWS");
  dev->gemv_stream_max_rows = ev ? atoi(ev) : 5;
  ev = getenv("WGPT_FUSED_DECODE");
  dev->fused_decode = !(ev && ev[0] == '0');
  ev = getenv("WGPT_LOOP_GEMV");
  dev->loop_gemv = !(ev && ev[0] == '0');
  dev->capturing = false;
  dev->capture_launch0 = 0;
  cudaError_t e = cudaStreamCreateWithFlags(&dev->stream, cudaStreamNonBlocking);
  dev->tc_scratch = nullptr;
  dev->tc_scratch_bytes = size_t(64) << 20;
  if (e == cudaSuccess) e = cudaMalloc(&dev->d_err, sizeof(int));
  if (e == cudaSuccess) e = cudaMalloc(&dev->d_work, 2 * sizeof(unsigned int));
  if (e == cudaSuccess) e = cudaMemsetAsync(dev->d_work, 0, 2 * sizeof(unsigned int), dev->stream);
  if (e == cudaSuccess) e = cudaMalloc(&dev->tc_scratch, dev->tc_scratch_bytes);
  if (e == cudaSuccess) e = cudaMemsetAsync(dev->d_err, 0, sizeof(int), dev->stream);
  if (e != cudaSuccess) {
    delete dev;
    return fail(WGPT_ERR_CUDA, "device setup: %s", cudaGetErrorString(e));
  }
  *out = dev;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_device_destroy(wgpt_device *dev) {
  TRY(use(dev));
  cudaStreamSynchronize(dev->stream);
  if (dev->scratch) cudaFree(dev->scratch);
  if (dev->d_err) cudaFree(dev->d_err);
  if (dev->d_work) cudaFree(dev->d_work);
  if (dev->tc_scratch) cudaFree(dev->tc_scratch);
  cudaStreamDestroy(dev->stream);
  delete dev;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_device_synchronize(wgpt_device *dev) {
  TRY(use(dev));
  NOT_RECORDING(dev, "wgpt_device_synchronize");
  CK(cudaStreamSynchronize(dev->stream));
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_device_set_precision(wgpt_device *dev, int32_t mode) {
  TRY(use(dev));
  REQUIRE(mode >= WGPT_PRECISION_FP32 && mode <= WGPT_PRECISION_TF32, WGPT_ERR_ARG, "unknown precision mode %d", mode);
  dev->precision = mode;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_device_mem_info(wgpt_device *dev, uint64_t *free_bytes, uint64_t *total_bytes) {
  TRY(use(dev));
  REQUIRE(free_bytes && total_bytes, WGPT_ERR_ARG, "null argument");
  size_t f = 0, t = 0;
  CK(cudaMemGetInfo(&f, &t));
  *free_bytes = f;
  *total_bytes = t;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_device_launch_count(wgpt_device *dev, uint64_t *count) {
  REQUIRE(dev && count, WGPT_ERR_ARG, "null argument");
  *count = dev->launches;
  return WGPT_OK;
}

// ------------------------------------------------------------------------------------------ buffers
WGPT_EXPORT int32_t wgpt_buffer_create(wgpt_device *dev, uint64_t bytes, void **dptr) {
  TRY(use(dev));
  REQUIRE(dptr != nullptr, WGPT_ERR_ARG, "dptr is null");
  *dptr = nullptr;
  CK(cudaMalloc(dptr, bytes ? bytes : 16));
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_buffer_destroy(wgpt_device *dev, void *dptr) {
  TRY(use(dev));
  if (!dptr) return WGPT_OK;
  NOT_RECORDING(dev, "wgpt_buffer_destroy");
  CK(cudaStreamSynchronize(dev->stream));
  CK(cudaFree(dptr));
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_buffer_write(wgpt_device *dev, void *dst, uint64_t off, const void *src_host, uint64_t bytes) {
  TRY(use(dev));
  REQUIRE(dst && (src_host || !bytes), WGPT_ERR_ARG, "null pointer");
  NOT_RECORDING(dev, "wgpt_buffer_write");
  if (!bytes) return WGPT_OK;
  CK(cudaMemcpyAsync(static_cast<char *>(dst) + off, src_host, bytes, cudaMemcpyHostToDevice, dev->stream));
  // The source may be pageable and reused by the caller right away.
  CK(cudaStreamSynchronize(dev->stream));
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_buffer_read(wgpt_device *dev, const void *src, uint64_t off, void *dst_host, uint64_t bytes) {
  TRY(use(dev));
  REQUIRE(src && (dst_host || !bytes), WGPT_ERR_ARG, "null pointer");
  NOT_RECORDING(dev, "wgpt_buffer_read");
  if (bytes) CK(cudaMemcpyAsync(dst_host, static_cast<const char *>(src) + off, bytes, cudaMemcpyDeviceToHost, dev->stream));
  CK(cudaStreamSynchronize(dev->stream));
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_buffer_copy(wgpt_device *dev, const void *src, uint64_t soff, void *dst, uint64_t doff,
                                     uint64_t bytes) {
  TRY(use(dev));
  REQUIRE(src && dst, WGPT_ERR_ARG, "null pointer");
  if (bytes)
    CK(cudaMemcpyAsync(static_cast<char *>(dst) + doff, static_cast<const char *>(src) + soff, bytes,
                       cudaMemcpyDeviceToDevice, dev->stream));
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_host_alloc(uint64_t bytes, void **p) {
  REQUIRE(p != nullptr, WGPT_ERR_ARG, "ptr is null");
  *p = nullptr;
  CK(cudaMallocHost(p, bytes ? bytes : 16));
  return WGPT_OK;
}
WGPT_EXPORT int32_t wgpt_host_free(void *p) {
  if (p) CK(cudaFreeHost(p));
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_event_create(wgpt_device *dev, void **event) {
  TRY(use(dev));
  REQUIRE(event != nullptr, WGPT_ERR_ARG, "event is null");
  cudaEvent_t ev;
  CK(cudaEventCreate(&ev));
  *event = ev;
  return WGPT_OK;
}
WGPT_EXPORT int32_t wgpt_event_record(wgpt_device *dev, void *event) {
  TRY(use(dev));
  CK(cudaEventRecord(static_cast<cudaEvent_t>(event), dev->stream));
  return WGPT_OK;
}
WGPT_EXPORT int32_t wgpt_event_elapsed_ms(wgpt_device *dev, void *start, void *stop, float *ms) {
  TRY(use(dev));
  REQUIRE(ms != nullptr, WGPT_ERR_ARG, "ms is null");
  CK(cudaEventSynchronize(static_cast<cudaEvent_t>(stop)));
  CK(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  return WGPT_OK;
}
WGPT_EXPORT int32_t wgpt_event_destroy(wgpt_device *dev, void *event) {
  TRY(use(dev));
  if (event) CK(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return WGPT_OK;
}

// ------------------------------------------------------------------------------------------ pass-list graphs
struct wgpt_graph {
  cudaGraphExec_t exec;
  uint64_t launches;
  uint64_t scratch_gen;  // generation of the device workspace whose address the recording may hold
};

WGPT_EXPORT int32_t wgpt_graph_begin(wgpt_device *dev) {
  TRY(use(dev));
  REQUIRE(!dev->capturing, WGPT_ERR_STATE, "a pass list is already being recorded on this device");
  CK(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeRelaxed));
  dev->capturing = true;
  dev->capture_launch0 = dev->launches;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_graph_end(wgpt_device *dev, wgpt_graph **out) {
  TRY(use(dev));
  REQUIRE(out != nullptr, WGPT_ERR_ARG, "out is null");
  *out = nullptr;
  REQUIRE(dev->capturing, WGPT_ERR_STATE, "no pass list is being recorded on this device");
  dev->capturing = false;
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(dev->stream, &g);
  uint64_t n = dev->launches - dev->capture_launch0;
  dev->launches = dev->capture_launch0;  // recording enqueued nothing
  if (e != cudaSuccess) return fail(WGPT_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
  cudaGraphExec_t ex = nullptr;
  e = cudaGraphInstantiate(&ex, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return fail(WGPT_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
  wgpt_graph *gr = new wgpt_graph();
  gr->exec = ex;
  gr->launches = n;
  gr->scratch_gen = dev->scratch_gen;
  *out = gr;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_graph_launch(wgpt_device *dev, wgpt_graph *graph) {
  TRY(use(dev));
  REQUIRE(graph != nullptr, WGPT_ERR_ARG, "graph handle is null");
  NOT_RECORDING(dev, "wgpt_graph_launch");
  REQUIRE(graph->scratch_gen == dev->scratch_gen, WGPT_ERR_STATE,
          "the device workspace was re-allocated after this pass list was recorded (a later call needed a larger "
          "one): the recording names freed memory and must be recorded again");
  CK(cudaGraphLaunch(graph->exec, dev->stream));
  dev->launches += graph->launches;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_graph_destroy(wgpt_device *dev, wgpt_graph *graph) {
  TRY(use(dev));
  if (!graph) return WGPT_OK;
  NOT_RECORDING(dev, "wgpt_graph_destroy");
  CK(cudaStreamSynchronize(dev->stream));
  cudaGraphExecDestroy(graph->exec);
  delete graph;
  return WGPT_OK;
}

// ------------------------------------------------------------------------------------------ launch helpers
static Epilogue plain_epi(float *out, int ld, const float *bias) {
  Epilogue e;
  memset(&e, 0, sizeof e);
  e.out = out;
  e.ld = ld;
  e.bias = bias;
  return e;
}

// Largest row count the staged-input GEMV handles for a given K (input rows live in shared memory).
static bool gemv_nk_fits(const wgpt_device *dev, int M, int K) {
  return M >= 1 && M <= 8 && (size_t)M * K * 4 + 8 * 4 * 8 * 4 <= dev->smem_optin - 1024;
}

template <int M, int WK, int CPW>
static int32_t launch_gemv_nk_t(wgpt_device *dev, const float *x, size_t ldx, const float *gamma, const float *beta,
                                const float *Wt, int K, int N, const Epilogue &epi, const GreedyPick &gp) {
  constexpr int WC = 8 / WK;
  size_t smem = (size_t)M * K * 4 + (size_t)8 * CPW * M * 4;
  auto kern = gemv_nk_kernel<M, WK, CPW>;
  if (smem > 48 * 1024) CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = (N + WC * CPW - 1) / (WC * CPW);
  // Weight slices are pulled towards L2 ahead of the dependency wait unless the matrix would flush L2 (the
  // de-embedding table is larger than L2 and is long enough to be bandwidth-bound on its own).
  int prefetch = (size_t)N * K * 4 <= (size_t(32) << 20) ? 1 : 0;
  LAUNCH_PDL(dev, kern, grid, 256, smem, x, ldx, gamma, beta, Wt, K, N, epi, prefetch, gp);
  return WGPT_OK;
}

// Matrices larger than L2 (the de-embedding): resident CTAs that loop over the columns (gemv_loop_kernel).
template <int M>
static int32_t launch_gemv_loop_t(wgpt_device *dev, const float *x, size_t ldx, const float *gamma, const float *beta,
                                  const float *Wt, int K, int N, const Epilogue &epi, const GreedyPick &gp) {
  constexpr int CPW = M <= 4 ? 4 : 2;
  size_t smem = (size_t)M * K * 4;
  auto kern = gemv_loop_kernel<M, CPW>;
  if (smem > 48 * 1024) CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  LAUNCH_PDL(dev, kern, 2 * dev->sm_count, 256, smem, x, ldx, gamma, beta, Wt, K, N, epi, gp, dev->d_work);
  return WGPT_OK;
}

template <int M>
static int32_t launch_gemv_nk_m(wgpt_device *dev, const float *x, size_t ldx, const float *gamma, const float *beta,
                                const float *Wt, int K, int N, const Epilogue &epi, const GreedyPick &gp) {
  if (dev->loop_gemv && (size_t)N * K * 4 >= (size_t(64) << 20) && N >= 64 * dev->sm_count &&
      (size_t)M * K * 4 <= 96 * 1024)
    return launch_gemv_loop_t<M>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
  // Enough warps to cover the machine several times over: split K across the warps of a CTA when N is small.
  int wk = 1;
  while (wk < 8 && (long long)N * wk < 3000 && K / (wk * 2) >= 256) wk *= 2;
  if (N >= 16384) return launch_gemv_nk_t<M, 1, 4>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
  switch (wk) {
    case 1: return launch_gemv_nk_t<M, 1, 1>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
    case 2: return launch_gemv_nk_t<M, 2, 1>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
    case 4: return launch_gemv_nk_t<M, 4, 1>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
    default: return launch_gemv_nk_t<M, 8, 1>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
  }
}

static GreedyPick no_pick() {
  GreedyPick gp;
  memset(&gp, 0, sizeof gp);
  return gp;
}

// Plan for gemv_block_kernel: one CTA per SM, each owning `cols` consecutive columns whose weights fit in shared
// memory together with the input rows. Returns false when the block does not fit (the register-streaming kernel
// is used instead).
static bool gemv_block_plan(const wgpt_device *dev, int M, int K, int N, bool layernorm, int *cols, int *wk,
                            size_t *smem) {
  if (N >= 16384 || K % 4 != 0) return false;
  int c = (N + dev->sm_count - 1) / dev->sm_count;
  const int nw0 = kBlockGemvThreads / 32;
  int w = 1;
  while (c * w < 2 * nw0 && w < 8 && (K / 4) / (w * 2) >= 32) w *= 2;
  const int nw = kBlockGemvThreads / 32;
  size_t red = M > 4 ? (size_t)nw * c * M : (size_t)(c * w > nw ? c * w : nw) * M;
  const size_t row = (size_t)K + (M > 4 ? 4 : 0);  // input rows are padded by one float4 in the rows-in-lanes form
  size_t bytes = ((size_t)c * K + (size_t)M * row * (layernorm ? 2 : 1) + ((red + 3) & ~size_t(3))) * 4 + 16;
  if (bytes > dev->smem_optin - 2048) return false;
  *cols = c;
  *wk = w;
  *smem = bytes;
  return true;
}

template <int M>
static int32_t launch_gemv_block_t(wgpt_device *dev, const float *x, size_t ldx, const float *gamma, const float *beta,
                                   const float *Wt, int K, int N, int cols, int wk, size_t smem, const Epilogue &epi,
                                   const AttnPartials &ap) {
  auto kern = gemv_block_kernel<M>;
  if (smem > 48 * 1024) CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = (N + cols - 1) / cols;
  LAUNCH_PDL(dev, kern, grid, kBlockGemvThreads, smem, x, ldx, gamma, beta, Wt, K, N, cols, wk, epi, dev->d_err, ap);
  return WGPT_OK;
}

static int32_t launch_gemv_nk(wgpt_device *dev, int M, const float *x, size_t ldx, const float *gamma,
                              const float *beta, const float *Wt, int K, int N, const Epilogue &epi,
                              const GreedyPick &gp = no_pick(), const AttnPartials *partials = nullptr) {
  AttnPartials ap;
  memset(&ap, 0, sizeof ap);
  if (partials) ap = *partials;
  int cols = 0, wk = 0;
  size_t smem = 0;
  if (gp.pval == nullptr && dev->block_gemv && gemv_block_plan(dev, M, K, N, gamma != nullptr, &cols, &wk, &smem)) {
    switch (M) {
      case 1: return launch_gemv_block_t<1>(dev, x, ldx, gamma, beta, Wt, K, N, cols, wk, smem, epi, ap);
      case 2: return launch_gemv_block_t<2>(dev, x, ldx, gamma, beta, Wt, K, N, cols, wk, smem, epi, ap);
      case 3: return launch_gemv_block_t<3>(dev, x, ldx, gamma, beta, Wt, K, N, cols, wk, smem, epi, ap);
      case 4: return launch_gemv_block_t<4>(dev, x, ldx, gamma, beta, Wt, K, N, cols, wk, smem, epi, ap);
      case 5: return launch_gemv_block_t<5>(dev, x, ldx, gamma, beta, Wt, K, N, cols, wk, smem, epi, ap);
      case 6: return launch_gemv_block_t<6>(dev, x, ldx, gamma, beta, Wt, K, N, cols, wk, smem, epi, ap);
      case 7: return launch_gemv_block_t<7>(dev, x, ldx, gamma, beta, Wt, K, N, cols, wk, smem, epi, ap);
      case 8: return launch_gemv_block_t<8>(dev, x, ldx, gamma, beta, Wt, K, N, cols, wk, smem, epi, ap);
    }
  }
  if (ap.part != nullptr) {  // the register-streaming kernel reads merged rows: merge into x first
    dim3 mg((ap.H * ap.hs / 4 + 127) / 128, M);
    LAUNCH_PDL(dev, attn_merge_kernel, mg, 128, 0, ap, const_cast<float *>(x), (int)ldx);
  }
  switch (M) {
    case 1: return launch_gemv_nk_m<1>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
    case 2: return launch_gemv_nk_m<2>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
    case 3: return launch_gemv_nk_m<3>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
    case 4: return launch_gemv_nk_m<4>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
    case 5: return launch_gemv_nk_m<5>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
    case 6: return launch_gemv_nk_m<6>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
    case 7: return launch_gemv_nk_m<7>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
    case 8: return launch_gemv_nk_m<8>(dev, x, ldx, gamma, beta, Wt, K, N, epi, gp);
  }
  return fail(WGPT_ERR_SHAPE, "gemv rows %d out of range", M);
}

static int32_t launch_gemm_simt(wgpt_device *dev, bool b_nk, const float *A, size_t lda, const float *B, int M, int K,
                                int N, const Epilogue &epi) {
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  if (b_nk)
    LAUNCH(dev, gemm_simt_kernel<true>, grid, 256, 0, A, lda, B, M, K, N, epi);
  else
    LAUNCH(dev, gemm_simt_kernel<false>, grid, 256, 0, A, lda, B, M, K, N, epi);
  return WGPT_OK;
}

// ---- tensor-core GEMM launch ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Tensor map of a row-major FP32 matrix [rows, cols] with row stride ld (floats), boxes of 32 x 128 elements,
// 128-byte swizzle, zero fill outside the matrix.
static int32_t make_tile_map(CUtensorMap *map, const float *base, uint64_t rows, uint64_t cols, uint64_t ld,
                             int box_rows = TC_BM) {
  EncodeTiledFn fn = encode_tiled_fn();
  REQUIRE(fn != nullptr, WGPT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 4};
  cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  REQUIRE(r == CUDA_SUCCESS, WGPT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return WGPT_OK;
}

// A LayerNorm that consumes a product's output (the next block's input): when the product runs split-K, its
// second stage normalises the finished rows as it writes them (splitk_reduce_ln_kernel) and sets `done`.
struct LnAfter {
  const float *gamma, *beta;
  float *out;  // [M, N]
  bool done;
};

// A consumer that adds the split-K slices itself (the decode attention for the QKV product): when the product
// runs split-K in the exchanged form its second stage is not launched and the slices are handed over.
struct SplitHandoff {
  const float *part = nullptr;
  int splits = 0;
  bool taken = false;
};

// C = A[M,K] (row stride lda) . Wt[N,K]^T on the tensor cores; x3 selects 3 x TF32.
static int32_t launch_gemm_tc(wgpt_device *dev, bool x3, const float *A, size_t lda, const float *Wt, int M, int K,
                              int N, const Epilogue &epi, LnAfter *ln = nullptr, bool b_static = true,
                              const float *Wt_lo = nullptr, SplitHandoff *handoff = nullptr, bool b_exact = false) {
  REQUIRE(aligned16(A) && aligned16(Wt) && (lda % 4) == 0 && (K % 4) == 0, WGPT_ERR_ALIGN,
          "tensor-core GEMM operands must be 16-byte aligned with row strides that are multiples of 16 bytes");
  CUtensorMap ma, mb;
  TRY(make_tile_map(&ma, A, (uint64_t)M, (uint64_t)K, lda));
  TRY(make_tile_map(&mb, Wt, (uint64_t)N, (uint64_t)K, (uint64_t)K));
  // Too few 128x128 tiles to occupy the machine (skinny M): split the K loop over CTAs.
  const int tiles = ((N + TC_BN - 1) / TC_BN) * ((M + TC_BM - 1) / TC_BM);
  const int total_kb = (K + TC_BK - 1) / TC_BK;
  int splits = 1, kb_per_split = total_kb;
  float *split_out = nullptr;
  if (tiles * 2 <= dev->sm_count && total_kb > 1 && dev->tc_scratch != nullptr) {
    int want = (dev->sm_count + tiles - 1) / tiles;
    if (want > total_kb / 2) want = total_kb / 2;  // at least two k-blocks per slice: fewer slices to add up
    if (want < 1) want = 1;
    {
      static const int max_splits = [] { const char *ev = getenv("WGPT_MAX_SPLITS"); return ev ? atoi(ev) : 0; }();
      if (max_splits > 0 && want > max_splits) want = max_splits;
    }
    kb_per_split = (total_kb + want - 1) / want;
    splits = (total_kb + kb_per_split - 1) / kb_per_split;
    const size_t n_pad = (size_t)((N + TC_BM - 1) / TC_BM) * TC_BM;  // the exchanged form stores whole feature tiles
    if (splits > 1 && (size_t)splits * M * n_pad * 4 <= dev->tc_scratch_bytes && (N % 4) == 0) {
      split_out = dev->tc_scratch;
    } else {
      splits = 1;
      kb_per_split = total_kb;
    }
  }
  // Skinny split-K products run with the operands exchanged: the kernel sees C^T[N,M] = Wt[N,K] . A[M,K]^T, so the
  // accumulator's 128 lanes are output features (all live) and its columns the few activation rows; the partial
  // tiles are written feature-tile-major, which the second stage reads with tile width 128.
  // Without split-K (a very wide product such as the de-embedding of up to 64 sequences) the exchanged form
  // finishes the values itself; it carries no activation or cache scatter.
  const bool exchanged = M <= 64 && (split_out != nullptr || (epi.act == 0 && epi.kc == nullptr));
  // The exchanged form issues its instruction only as wide as the activation rows need (a multiple of 16) and
  // fetches only those rows of the activation tile.
  if (exchanged) TRY(make_tile_map(&ma, A, (uint64_t)M, (uint64_t)K, lda, M + 15 < TC_BN ? (M + 15) & ~15 : TC_BN));
  const int tw = exchanged ? TC_BM : N;
  const int n_work = tiles * splits;
  dim3 grid(n_work < dev->sm_count ? n_work : dev->sm_count);
  const CUtensorMap &m_first = exchanged ? mb : ma, &m_second = exchanged ? ma : mb;
  const int km = exchanged ? N : M, kn = exchanged ? M : N;
  const int static_op = b_static ? (exchanged ? 2 : 1) : 0;
  // Compute-bound 3xTF32 products read the weight's precomputed low part (x - tf32(x), same layout) by TMA
  // instead of deriving it in shared memory; skinny products are HBM-bound on the weights and keep deriving it.
  const bool lo_tma = x3 && Wt_lo != nullptr && !exchanged && b_static;
  CUtensorMap mlo = mb;
  if (lo_tma) TRY(make_tile_map(&mlo, Wt_lo, (uint64_t)N, (uint64_t)K, (uint64_t)K));
  // Large 3xTF32 products without split-K and without a precomputed low part of the weight (the per-operator
  // entry points) run on the CTA-pair kernel (256 x 256 tile per two SMs) when its tiles fill the pairs evenly
  // enough. Measured back to back: 8192x768x2304 226-232 against 171-182 TFLOP/s; with 96 tiles on 74 pairs it is
  // no faster than the 128 x 128 tiles, in plain TF32 it is slower (302 against 330-360), and inside the model's
  // prefill the one-CTA kernel with the low part fetched by TMA measured the same or better (10.9 against 11.1 ms),
  // so the model path keeps that. WGPT_PAIR_GEMM=0 turns the pair kernel off, 2 uses it wherever it fits.
  static const int pair_mode = [] { const char *ev = getenv("WGPT_PAIR_GEMM"); return ev ? atoi(ev) : 1; }();
  const int work2 = ((M + 255) / 256) * ((N + TC2_BN - 1) / TC2_BN);
  int pairs = dev->sm_count / 2;
  const int rounds2 = (work2 + pairs - 1) / pairs;
  const bool pair_fits = work2 * 5 >= rounds2 * pairs * 4;  // at least 80 % of the pair slots do useful work
  if (pair_mode > 0 && ((x3 && !lo_tma) || pair_mode == 2) && split_out == nullptr && !exchanged && M >= 512 &&
      N >= 256 && pair_fits) {
    if (pairs > work2) pairs = work2;
    dim3 grid2(2 * pairs);
    if (x3) {
      auto kern = gemm_tc2_kernel<true>;
      CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcPlan<true>::kSmemBytes));
      LAUNCH_PDL(dev, kern, grid2, TcPlan<true>::kThreads, TcPlan<true>::kSmemBytes, ma, mb, mlo, M, K, N, epi,
                 dev->d_err, lo_tma ? 1 : 0);
    } else {
      auto kern = gemm_tc2_kernel<false>;
      CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcPlan<false>::kSmemBytes));
      LAUNCH_PDL(dev, kern, grid2, TcPlan<false>::kThreads, TcPlan<false>::kSmemBytes, ma, mb, mlo, M, K, N, epi,
                 dev->d_err, 0);
    }
    return WGPT_OK;
  }
  if (x3) {
    auto kern = gemm_tc_kernel<true>;
    CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcPlan<true>::kSmemBytes));
    LAUNCH_PDL(dev, kern, grid, TcPlan<true>::kThreads, TcPlan<true>::kSmemBytes, m_first, m_second, mlo, km, K, kn,
               epi, dev->d_err, kb_per_split, splits, split_out, static_op, exchanged ? 1 : 0,
               lo_tma ? 1 : (b_exact && !exchanged ? 2 : 0));
  } else {
    auto kern = gemm_tc_kernel<false>;
    CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcPlan<false>::kSmemBytes));
    LAUNCH_PDL(dev, kern, grid, TcPlan<false>::kThreads, TcPlan<false>::kSmemBytes, m_first, m_second, mlo, km, K, kn,
               epi, dev->d_err, kb_per_split, splits, split_out, static_op, exchanged ? 1 : 0, 0);
  }
  if (split_out != nullptr && handoff != nullptr && exchanged) {
    handoff->part = split_out;
    handoff->splits = splits;
    handoff->taken = true;
    return WGPT_OK;
  }
  if (split_out != nullptr) {
    if (ln != nullptr && N / 4 <= 256 * kReduceLnVec && epi.kc == nullptr) {
      LAUNCH_PDL(dev, splitk_reduce_ln_kernel, M, 256, 0, (const float *)split_out, splits, M, N, epi, ln->gamma,
                 ln->beta, ln->out, tw);
      ln->done = true;
    } else {
      int n4 = M * (N / 4);
      LAUNCH_PDL(dev, gemv_kn_reduce_kernel, (n4 + 255) / 256, 256, 0, (const float *)split_out, splits, M, N, epi, tw);
    }
  }
  return WGPT_OK;
}

// Matrix product for more than 8 rows against a weight stored [N,K]: tensor cores or CUDA cores per dev->precision.
static int32_t launch_gemm_nk(wgpt_device *dev, const float *A, size_t lda, const float *Wt, int M, int K, int N,
                              const Epilogue &epi, LnAfter *ln = nullptr, const float *Wt_lo = nullptr,
                              SplitHandoff *handoff = nullptr) {
  if (dev->precision == WGPT_PRECISION_FP32) return launch_gemm_simt(dev, true, A, lda, Wt, M, K, N, epi);
  return launch_gemm_tc(dev, dev->precision == WGPT_PRECISION_TF32X3, A, lda, Wt, M, K, N, epi, ln, true, Wt_lo,
                        handoff);
}

static int32_t launch_layernorm(wgpt_device *dev, const float *in, size_t ld_in, const float *gamma, const float *beta,
                                float *out, size_t ld_out, int rows, int N) {
  LAUNCH_PDL(dev, layernorm_kernel, (rows + 3) / 4, 128, 0, in, ld_in, gamma, beta, out, ld_out, rows, N);
  return WGPT_OK;
}

// K split for the [K,N]-layout GEMV: enough CTAs for about two per SM, at least 32 k rows per CTA.
// Each CTA stages its K slice of all M input rows in shared memory, so the split is also at least what makes
// that slice fit (M * K/ksplit floats beside the 8 KB-per-row reduction buffer).
static int kn_ksplit(const wgpt_device *dev, int M, int K, int col_groups, size_t red_bytes_per_row = 8 * 32 * 16) {
  int want = (2 * dev->sm_count + col_groups - 1) / col_groups;
  int maxs = K / 32 > 0 ? K / 32 : 1;
  int s = want < maxs ? want : maxs;
  if (s < 1) s = 1;
  const size_t room = dev->smem_optin - 2048 - (size_t)M * red_bytes_per_row;
  const size_t klen_fit = room / ((size_t)M * 4) - 8;
  const int need = (int)(((size_t)K + klen_fit - 1) / klen_fit);
  return s > need ? s : need;
}

template <int M>
static int32_t launch_gemv_kn_t(wgpt_device *dev, const float *x, const float *W, int K, int N, int ksplit,
                                float *part) {
  int klen_max = ((K / 4 + ksplit - 1) / ksplit + 1) * 4;
  size_t smem = (size_t)M * klen_max * 4 + (size_t)8 * M * 32 * 16;
  auto kern = gemv_kn_partial_kernel<M>;
  if (smem > 48 * 1024) CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((N + 127) / 128, ksplit);
  LAUNCH(dev, kern, grid, 256, smem, x, W, K, N, part);
  return WGPT_OK;
}

// out = x[M,K] . W[K,N] (+ epilogue) for M <= 8, split-K with the partial sums in `part`
// ([ksplit][M][N] floats, caller-provided).
static int32_t gemv_kn_with_scratch(wgpt_device *dev, int M, const float *x, const float *W, int K, int N, int ksplit,
                                    float *part, const Epilogue &epi) {
  switch (M) {
    case 1: TRY(launch_gemv_kn_t<1>(dev, x, W, K, N, ksplit, part)); break;
    case 2: TRY(launch_gemv_kn_t<2>(dev, x, W, K, N, ksplit, part)); break;
    case 3: TRY(launch_gemv_kn_t<3>(dev, x, W, K, N, ksplit, part)); break;
    case 4: TRY(launch_gemv_kn_t<4>(dev, x, W, K, N, ksplit, part)); break;
    case 5: TRY(launch_gemv_kn_t<5>(dev, x, W, K, N, ksplit, part)); break;
    case 6: TRY(launch_gemv_kn_t<6>(dev, x, W, K, N, ksplit, part)); break;
    case 7: TRY(launch_gemv_kn_t<7>(dev, x, W, K, N, ksplit, part)); break;
    case 8: TRY(launch_gemv_kn_t<8>(dev, x, W, K, N, ksplit, part)); break;
    default: return fail(WGPT_ERR_SHAPE, "gemv rows %d out of range", M);
  }
  int n4 = M * (N / 4);
  LAUNCH_PDL(dev, gemv_kn_reduce_kernel, (n4 + 255) / 256, 256, 0, part, ksplit, M, N, epi, N);
  return WGPT_OK;
}

// out = A[M,K] . W[K,N] on the tensor cores: wt (K*N floats of workspace) receives W transposed to [N,K].
static int32_t gemm_kn_via_transpose(wgpt_device *dev, const float *A, size_t lda, const float *W, int M, int K, int N,
                                     const Epilogue &epi, float *wt) {
  dim3 tg((unsigned)((N + 31) / 32), (unsigned)((K + 31) / 32));
  LAUNCH(dev, transpose_kernel, tg, dim3(32, 8), 0, W, wt, K, N);
  // the transposed copy was written by the kernel just before: no reads of it ahead of the dependency wait
  return launch_gemm_tc(dev, dev->precision == WGPT_PRECISION_TF32X3, A, lda, wt, M, K, N, epi, nullptr, false);
}

// The reference-layout matmul used by the per-operator API: W is [K,N].
static int32_t matmul_kn(wgpt_device *dev, int M, int K, int N, const float *in, const float *W, const Epilogue &epi) {
  if (M <= 8) {
    int ksplit = kn_ksplit(dev, M, K, (N + 127) / 128);
    TRY(scratch_reserve(dev, (size_t)ksplit * M * N * 4));
    return gemv_kn_with_scratch(dev, M, in, W, K, N, ksplit, static_cast<float *>(dev->scratch), epi);
  }
  if (dev->precision != WGPT_PRECISION_FP32 && M >= 32) {
    // Tensor cores behind the reference layout: W[K,N] is transposed into the workspace (one pass over the weight,
    // a few microseconds against a product of more than a hundred) and the [N,K] kernel runs on the copy.
    TRY(scratch_reserve(dev, (size_t)K * N * 4));
    return gemm_kn_via_transpose(dev, in, (size_t)K, W, M, K, N, epi, static_cast<float *>(dev->scratch));
  }
  return launch_gemm_simt(dev, false, in, (size_t)K, W, M, K, N, epi);
}

template <int HS>
static int32_t launch_attn_prefill_t(wgpt_device *dev, const float *q, int ldq, const float *kc, const float *vc,
                                     int ldkv, size_t kv_seq_stride, float *out, int ldo, int n_tok, int n_seq, int H,
                                     const int *pos, float scale) {
  size_t smem = attn_prefill_smem_bytes(HS);
  auto kern = attn_prefill_kernel<HS>;
  if (smem > 48 * 1024) CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((n_tok + 31) / 32, H, n_seq);
  LAUNCH(dev, kern, grid, 128, smem, q, ldq, kc, vc, ldkv, kv_seq_stride, out, ldo, n_tok, pos, scale);
  return WGPT_OK;
}

static int32_t launch_attn_prefill(wgpt_device *dev, int hs, const float *q, int ldq, const float *kc, const float *vc,
                                   int ldkv, size_t kv_seq_stride, float *out, int ldo, int n_tok, int n_seq, int H,
                                   const int *pos, float scale) {
  static const bool tiled64 = [] { const char *ev = getenv("WGPT_ATTN_PREFILL64"); return !(ev && ev[0] == '0'); }();
  static const bool mma64 = [] { const char *ev = getenv("WGPT_ATTN_PREFILL_MMA"); return !(ev && ev[0] == '0'); }();
  if (hs == 64 && mma64 && dev->precision != WGPT_PRECISION_FP32 && n_tok >= 16 && (ldq % 4) == 0 && (ldkv % 4) == 0 &&
      (ldo % 2) == 0) {
    // products in TF32 / 3xTF32: the warp-level tensor-core kernel; FP32 mode keeps the CUDA-core kernels below
    dim3 grid((n_tok + 63) / 64, H, n_seq);
    if (dev->precision == WGPT_PRECISION_TF32X3)
      LAUNCH(dev, attn_prefill64_mma_kernel<true>, grid, 128, 0, q, ldq, kc, vc, ldkv, kv_seq_stride, out, ldo, n_tok, pos,
             scale);
    else
      LAUNCH(dev, attn_prefill64_mma_kernel<false>, grid, 128, 0, q, ldq, kc, vc, ldkv, kv_seq_stride, out, ldo, n_tok,
             pos, scale);
    return WGPT_OK;
  }
  if (hs == 64 && tiled64 && n_tok >= 16 && (ldq % 4) == 0 && (ldkv % 4) == 0 && (ldo % 4) == 0) {
    const size_t smem = attn_prefill64_smem_bytes();
    CK(cudaFuncSetAttribute(attn_prefill64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((n_tok + kAttn64Tile - 1) / kAttn64Tile, H, n_seq);
    LAUNCH(dev, attn_prefill64_kernel, grid, 256, smem, q, ldq, kc, vc, ldkv, kv_seq_stride, out, ldo, n_tok, pos, scale);
    return WGPT_OK;
  }
#define CASE(HSV) \
  case HSV: return launch_attn_prefill_t<HSV>(dev, q, ldq, kc, vc, ldkv, kv_seq_stride, out, ldo, n_tok, n_seq, H, pos, scale);
  switch (hs) {
    CASE(4) CASE(8) CASE(16) CASE(32) CASE(64) CASE(128)
  }
#undef CASE
  return fail(WGPT_ERR_UNSUPPORTED, "head_size %d: supported sizes are 4, 8, 16, 32, 64, 128", hs);
}

static int32_t launch_attn_decode(wgpt_device *dev, int hs, const float *q, int ldq, const float *kc, const float *vc,
                                  int ldkv, size_t kv_seq_stride, float *out, int ldo, int n_seq, int H, int n_split,
                                  const int *pos, float scale, float *part, const QkvPartials *qp = nullptr) {
  dim3 grid(H, n_seq, n_split);
  if (qp != nullptr) {  // the attention CTAs are the QKV product's second stage (one position slice, 3*hs <= 256)
    switch (hs) {
#define CASE_Q(HSV)                                                                                                  \
  case HSV:                                                                                                          \
    LAUNCH_PDL(dev, (attn_decode_kernel<HSV, true>), grid, 256, 0, q, ldq, kc, vc, ldkv, kv_seq_stride, out, ldo, pos, \
               scale, part, *qp);                                                                                    \
    return WGPT_OK;
      CASE_Q(4) CASE_Q(8) CASE_Q(16) CASE_Q(32) CASE_Q(64)
#undef CASE_Q
    }
    return fail(WGPT_ERR_UNSUPPORTED, "head_size %d with fused QKV second stage", hs);
  }
#define CASE(HSV)                                                                                                   \
  case HSV:                                                                                                         \
    LAUNCH_PDL(dev, attn_decode_kernel<HSV>, grid, 256, 0, q, ldq, kc, vc, ldkv, kv_seq_stride, out, ldo, pos, scale, \
               part, QkvPartials());                                                                                \
    return WGPT_OK;
  switch (hs) {
    CASE(4) CASE(8) CASE(16) CASE(32) CASE(64) CASE(128)
  }
#undef CASE
  return fail(WGPT_ERR_UNSUPPORTED, "head_size %d: supported sizes are 4, 8, 16, 32, 64, 128", hs);
}

static int grid_for(size_t n, int block, int sm_count) {
  size_t g = (n + block - 1) / block;
  size_t cap = (size_t)sm_count * 16;
  return (int)(g < cap ? (g ? g : 1) : cap);
}

// ------------------------------------------------------------------------------------------ per-operator API
WGPT_EXPORT int32_t wgpt_matmul(wgpt_device *dev, int32_t rows, int32_t cols, int32_t shared, const float *in,
                                const float *W, const float *bias, float *out) {
  TRY(use(dev));
  REQUIRE(in && W && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(rows >= 1 && cols >= 1 && shared >= 1, WGPT_ERR_SHAPE, "empty matmul %dx%dx%d", rows, cols, shared);
  REQUIRE(cols % 8 == 0, WGPT_ERR_SHAPE, "Cols must be divisible by 16.");  // message of instructions.js:158
  REQUIRE(shared % 4 == 0, WGPT_ERR_SHAPE, "shared dimension %d must be divisible by 4", shared);
  REQUIRE(aligned16(in) && aligned16(W) && aligned16(out) && aligned16(bias), WGPT_ERR_ALIGN,
          "buffers must be 16-byte aligned");
  return matmul_kn(dev, rows, shared, cols, in, W, plain_epi(out, cols, bias));
}

static int32_t check_err_word(wgpt_device *dev, const char *what);

WGPT_EXPORT int32_t wgpt_matmul_nk(wgpt_device *dev, int32_t rows, int32_t cols, int32_t shared, const float *in,
                                   const float *Wt, const float *bias, float *out) {
  TRY(use(dev));
  REQUIRE(in && Wt && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(rows >= 1 && cols >= 1 && shared >= 1, WGPT_ERR_SHAPE, "empty matmul %dx%dx%d", rows, cols, shared);
  REQUIRE(cols % 8 == 0, WGPT_ERR_SHAPE, "Cols must be divisible by 16.");
  REQUIRE(shared % 4 == 0, WGPT_ERR_SHAPE, "shared dimension %d must be divisible by 4", shared);
  REQUIRE(aligned16(in) && aligned16(Wt) && aligned16(out) && aligned16(bias), WGPT_ERR_ALIGN,
          "buffers must be 16-byte aligned");
  Epilogue e = plain_epi(out, cols, bias);
  if (gemv_nk_fits(dev, rows, shared)) return launch_gemv_nk(dev, rows, in, (size_t)shared, nullptr, nullptr, Wt, shared, cols, e);
  return launch_gemm_nk(dev, in, (size_t)shared, Wt, rows, shared, cols, e);
}

WGPT_EXPORT int32_t wgpt_device_check(wgpt_device *dev) {
  TRY(use(dev));
  NOT_RECORDING(dev, "wgpt_device_check");
  return check_err_word(dev, "wgpt_device_check");
}

WGPT_EXPORT int32_t wgpt_device_probe_wait_expiry(wgpt_device *dev, uint32_t polls, int32_t *first_wait_completed,
                                                  int32_t *drain_wait_completed) {
  TRY(use(dev));
  NOT_RECORDING(dev, "wgpt_device_probe_wait_expiry");
  REQUIRE(first_wait_completed && drain_wait_completed, WGPT_ERR_ARG, "null argument");
  REQUIRE(polls >= 1 && polls <= 1024, WGPT_ERR_ARG, "polls must be in 1..1024");
  TRY(scratch_reserve(dev, 256));
  float *src = static_cast<float *>(dev->scratch);
  int *obs = reinterpret_cast<int *>(src + 16);
  CK(cudaMemsetAsync(src, 0, 128, dev->stream));
  LAUNCH(dev, wait_expiry_probe_kernel, 1, 32, 0, (const float *)src, dev->d_err, polls, obs);
  int h[2] = {-1, -1};
  CK(cudaMemcpyAsync(h, obs, sizeof h, cudaMemcpyDeviceToHost, dev->stream));
  CK(cudaStreamSynchronize(dev->stream));
  *first_wait_completed = h[0];
  *drain_wait_completed = h[1];
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_residual(wgpt_device *dev, int32_t rows, int32_t cols, const float *a, const float *b,
                                  float *out) {
  TRY(use(dev));
  REQUIRE(a && b && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(rows >= 1 && cols >= 1, WGPT_ERR_SHAPE, "empty residual %dx%d", rows, cols);
  REQUIRE(cols % 4 == 0, WGPT_ERR_SHAPE, "Cols must be divisible by 4.");  // instructions.js:337
  REQUIRE(aligned16(a) && aligned16(b) && aligned16(out), WGPT_ERR_ALIGN, "buffers must be 16-byte aligned");
  size_t n4 = (size_t)rows * cols / 4;
  LAUNCH(dev, residual_kernel, grid_for(n4, 256, dev->sm_count), 256, 0, reinterpret_cast<const float4 *>(a),
         reinterpret_cast<const float4 *>(b), reinterpret_cast<float4 *>(out), n4);
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_gelu(wgpt_device *dev, int32_t rows, int32_t cols, const float *in, float *out) {
  TRY(use(dev));
  REQUIRE(in && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(rows >= 1 && cols >= 1, WGPT_ERR_SHAPE, "empty gelu %dx%d", rows, cols);
  REQUIRE(cols % 4 == 0, WGPT_ERR_SHAPE, "Cols must be divisible by 4.");  // instructions.js:684
  REQUIRE(aligned16(in) && aligned16(out), WGPT_ERR_ALIGN, "buffers must be 16-byte aligned");
  size_t n4 = (size_t)rows * cols / 4;
  LAUNCH(dev, gelu_kernel, grid_for(n4, 256, dev->sm_count), 256, 0, reinterpret_cast<const float4 *>(in),
         reinterpret_cast<float4 *>(out), n4);
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_layernorm(wgpt_device *dev, int32_t rows, int32_t cols, const float *in, const float *gamma,
                                   const float *beta, float *out) {
  TRY(use(dev));
  REQUIRE(in && gamma && beta && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(rows >= 1 && cols >= 1, WGPT_ERR_SHAPE, "empty layernorm %dx%d", rows, cols);
  REQUIRE(cols % 4 == 0, WGPT_ERR_SHAPE, "Cols must be divisible by 4.");  // instructions.js:410
  REQUIRE(aligned16(in) && aligned16(gamma) && aligned16(beta) && aligned16(out), WGPT_ERR_ALIGN,
          "buffers must be 16-byte aligned");
  return launch_layernorm(dev, in, (size_t)cols, gamma, beta, out, (size_t)cols, rows, cols);
}

WGPT_EXPORT int32_t wgpt_softmax(wgpt_device *dev, int32_t rows, int32_t cols, const float *in, float *out) {
  TRY(use(dev));
  REQUIRE(in && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(rows >= 1 && cols >= 1, WGPT_ERR_SHAPE, "empty softmax %dx%d", rows, cols);
  LAUNCH(dev, softmax_kernel, (rows + 3) / 4, 128, 0, in, out, rows, cols);
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_visuals_render(wgpt_device *dev, const float *embeddings, int32_t n_ctx, int32_t n_embd,
                                        uint8_t *rgba_out) {
  TRY(use(dev));
  REQUIRE(embeddings && rgba_out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(n_ctx >= 1 && n_embd >= 1, WGPT_ERR_SHAPE, "empty image %dx%d", n_embd, n_ctx);
  REQUIRE((reinterpret_cast<uintptr_t>(rgba_out) & 3u) == 0, WGPT_ERR_ALIGN, "rgba_out must be 4-byte aligned");
  size_t n = (size_t)n_ctx * n_embd;
  LAUNCH(dev, heatmap_kernel, grid_for(n, 256, dev->sm_count), 256, 0, embeddings, reinterpret_cast<uchar4 *>(rgba_out), n);
  return WGPT_OK;
}

static int32_t check_err_word(wgpt_device *dev, const char *what) {
  int h = 0;
  CK(cudaMemcpyAsync(&h, dev->d_err, sizeof h, cudaMemcpyDeviceToHost, dev->stream));
  CK(cudaStreamSynchronize(dev->stream));
  if (h) {
    CK(cudaMemsetAsync(dev->d_err, 0, sizeof(int), dev->stream));
    if (h == 4) return fail(WGPT_ERR_TIMEOUT, "%s: the whole-token decode kernel gave up at a grid barrier", what);
    if (h == 2) return fail(WGPT_ERR_TIMEOUT, "%s: a bulk copy into shared memory did not complete in time", what);
    if (h == 3) return fail(WGPT_ERR_TIMEOUT, "%s: the tensor-core GEMM pipeline gave up waiting on a barrier", what);
    return fail(WGPT_ERR_ARG, "%s: token id out of range", what);
  }
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_embed(wgpt_device *dev, const uint32_t *idx, int32_t seq_length, int32_t n_embd,
                               int32_t vocab_size, const float *wte, const float *wpe, float *out) {
  TRY(use(dev));
  REQUIRE(idx && wte && wpe && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(seq_length >= 1 && vocab_size >= 1, WGPT_ERR_SHAPE, "empty embed");
  REQUIRE(n_embd >= 4 && n_embd % 4 == 0, WGPT_ERR_SHAPE, "n_embd must be divisible by 4.");
  REQUIRE(aligned16(wte) && aligned16(wpe) && aligned16(out), WGPT_ERR_ALIGN, "buffers must be 16-byte aligned");
  LAUNCH_PDL(dev, embed_kernel, seq_length, 128, 0, idx, wte, wpe, out, seq_length, seq_length, n_embd, vocab_size,
             (const int *)nullptr, dev->d_err);
  // While a pass list is being recorded nothing runs yet: an id out of range then surfaces at the next
  // wgpt_device_check after a replay.
  if (dev->capturing) return WGPT_OK;
  return check_err_word(dev, "wgpt_embed");
}

WGPT_EXPORT int32_t wgpt_deembed(wgpt_device *dev, int32_t n_embd, int32_t vocab_size, int32_t seq_length,
                                 const float *x, const float *wte, float *logits) {
  TRY(use(dev));
  REQUIRE(x && wte && logits, WGPT_ERR_ARG, "null pointer");
  REQUIRE(seq_length >= 1 && vocab_size >= 1, WGPT_ERR_SHAPE, "empty deembed");
  REQUIRE(n_embd >= 4 && n_embd % 4 == 0, WGPT_ERR_SHAPE, "n_embd must be divisible by 4.");
  REQUIRE(aligned16(x) && aligned16(wte), WGPT_ERR_ALIGN, "buffers must be 16-byte aligned");
  REQUIRE(gemv_nk_fits(dev, 1, n_embd), WGPT_ERR_UNSUPPORTED, "n_embd %d too large", n_embd);
  const float *x_last = x + (size_t)(seq_length - 1) * n_embd;  // slice copy of instructions.js:849-856
  return launch_gemv_nk(dev, 1, x_last, (size_t)n_embd, nullptr, nullptr, wte, n_embd, vocab_size,
                        plain_epi(logits, vocab_size, nullptr));
}

WGPT_EXPORT int32_t wgpt_attention(wgpt_device *dev, int32_t T, int32_t E, float scale, int32_t H, int32_t hs,
                                   const float *in, const float *qW, const float *qB, const float *kW, const float *kB,
                                   const float *vW, const float *vB, const float *linW, const float *linB, float *out) {
  TRY(use(dev));
  REQUIRE(in && qW && kW && vW && linW && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(T >= 1 && E >= 8 && H >= 1, WGPT_ERR_SHAPE, "empty attention");
  REQUIRE(E % 8 == 0, WGPT_ERR_SHAPE, "Cols must be divisible by 16.");
  REQUIRE(H * hs == E, WGPT_ERR_SHAPE, "n_head * head_size (%d * %d) != n_embd (%d)", H, hs, E);
  REQUIRE(aligned16(in) && aligned16(qW) && aligned16(kW) && aligned16(vW) && aligned16(linW) && aligned16(out) &&
              aligned16(qB) && aligned16(kB) && aligned16(vB) && aligned16(linB),
          WGPT_ERR_ALIGN, "buffers must be 16-byte aligned");
  // workspace: q, k, v, o [T,E] + split-K partials
  size_t te = (size_t)T * E;
  int ksplit = T <= 8 ? kn_ksplit(dev, T, E, (E + 127) / 128) : 0;
  const bool tc = dev->precision != WGPT_PRECISION_FP32 && T >= 32;
  size_t part_floats = tc ? (size_t)E * E : (size_t)ksplit * T * E;  // split-K partials, or a transposed weight
  TRY(scratch_reserve(dev, (4 * te + part_floats) * 4));
  float *q = static_cast<float *>(dev->scratch), *k = q + te, *v = k + te, *o = v + te, *part = o + te;
  auto mm = [&](const float *a, const float *W, const float *b, float *dst) -> int32_t {
    Epilogue e = plain_epi(dst, E, b);
    if (T <= 8) return gemv_kn_with_scratch(dev, T, a, W, E, E, ksplit, part, e);
    if (tc) return gemm_kn_via_transpose(dev, a, (size_t)E, W, T, E, E, e, part);
    return launch_gemm_simt(dev, false, a, (size_t)E, W, T, E, E, e);
  };
  TRY(mm(in, qW, qB, q));
  TRY(mm(in, kW, kB, k));
  TRY(mm(in, vW, vB, v));
  TRY(launch_attn_prefill(dev, hs, q, E, k, v, E, 0, o, E, T, 1, H, nullptr, scale));
  return mm(o, linW, linB, out);
}

WGPT_EXPORT int32_t wgpt_int8_quantize(wgpt_device *dev, int32_t K, int32_t N, int32_t per_column, const float *W,
                                       uint32_t *Bq_out, float *scale_out) {
  TRY(use(dev));
  REQUIRE(W && Bq_out && scale_out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(K >= 1 && N >= 4 && N % 4 == 0, WGPT_ERR_SHAPE, "quantise needs K >= 1 and N a positive multiple of 4");
  REQUIRE(aligned16(W) && aligned16(Bq_out) && aligned16(scale_out), WGPT_ERR_ALIGN, "buffers must be 16-byte aligned");
  int slices = K / 64 > 0 ? K / 64 : 1;
  if (slices > 64) slices = 64;
  TRY(scratch_reserve(dev, ((size_t)slices + 1) * N * 4));
  float *part = static_cast<float *>(dev->scratch), *absmax = part + (size_t)slices * N;
  LAUNCH(dev, int8_absmax_kernel, dim3((N + 127) / 128, slices), 128, 0, W, K, N, part);
  LAUNCH(dev, int8_scale_kernel, 1, 256, 0, (const float *)part, slices, N, per_column ? 1 : 0, absmax, scale_out);
  LAUNCH(dev, int8_pack_kernel, grid_for((size_t)K * (N / 4), 256, dev->sm_count), 256, 0, W, (const float *)absmax,
         K, N, Bq_out);
  return WGPT_OK;
}

template <int M, int VEC>
static int32_t launch_int8_gemv_t(wgpt_device *dev, const float *x, const uint32_t *Bq, int K, int N, int ksplit,
                                  float *part) {
  int klen_max = ((K / 4 + ksplit - 1) / ksplit + 1) * 4;
  size_t smem = (size_t)M * klen_max * 4 + (size_t)8 * M * 32 * 4 * VEC * 4;
  auto kern = int8_gemv_partial_kernel<M, VEC>;
  if (smem > 48 * 1024) CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((N + 128 * VEC - 1) / (128 * VEC), ksplit);
  LAUNCH(dev, kern, grid, 256, smem, x, Bq, K, N, part);
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_int8_matmul(wgpt_device *dev, int32_t M, int32_t K, int32_t N, const float *A,
                                     const uint32_t *Bq, const float *scale, float *out) {
  TRY(use(dev));
  REQUIRE(A && Bq && scale && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(M >= 1 && K >= 4 && N >= 8, WGPT_ERR_SHAPE, "empty int8 matmul");
  REQUIRE(N % 8 == 0 && K % 4 == 0, WGPT_ERR_SHAPE, "N must be divisible by 8 and K by 4");
  REQUIRE(aligned16(A) && aligned16(Bq) && aligned16(scale) && aligned16(out), WGPT_ERR_ALIGN,
          "buffers must be 16-byte aligned");
  Epilogue e = plain_epi(out, N, nullptr);
  e.colscale = scale;
  if (M > 16) {
    if (dev->precision != WGPT_PRECISION_FP32) {
      // expand the words to an FP32 [N,K] weight in scratch, then the tcgen05 GEMM with the scales in its epilogue
      TRY(scratch_reserve(dev, (size_t)N * K * 4));
      float *wt = static_cast<float *>(dev->scratch);
      dim3 xgrid((N / 4 + 31) / 32, (K + 31) / 32);
      LAUNCH(dev, int8_expand_nk_kernel, xgrid, 256, 0, Bq, K, N, wt);
      // the expanded weight was written by the kernel just before: no reads of it ahead of the dependency wait
      // the expanded codes are integers: exact in TF32, no low part
      return launch_gemm_tc(dev, dev->precision == WGPT_PRECISION_TF32X3, A, (size_t)K, wt, M, K, N, e, nullptr, false,
                            nullptr, nullptr, true);
    }
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    LAUNCH(dev, int8_gemm_simt_kernel, grid, 256, 0, A, Bq, M, K, N, e);
    return WGPT_OK;
  }
  bool wide = (N % 16 == 0) && M <= 4;
  int col_groups = wide ? (N + 511) / 512 : (N + 127) / 128;
  int ksplit = kn_ksplit(dev, M, K, col_groups, (size_t)8 * 32 * 4 * (wide ? 4 : 1) * 4);
  TRY(scratch_reserve(dev, (size_t)ksplit * M * N * 4));
  float *part = static_cast<float *>(dev->scratch);
#define CASE_W(MV) case MV: TRY((launch_int8_gemv_t<MV, 4>(dev, A, Bq, K, N, ksplit, part))); break;
#define CASE_N(MV) case MV: TRY((launch_int8_gemv_t<MV, 1>(dev, A, Bq, K, N, ksplit, part))); break;
  if (wide) {
    switch (M) { CASE_W(1) CASE_W(2) CASE_W(3) CASE_W(4) }
  } else {
    switch (M) {
      CASE_N(1) CASE_N(2) CASE_N(3) CASE_N(4) CASE_N(5) CASE_N(6) CASE_N(7) CASE_N(8)
      CASE_N(9) CASE_N(10) CASE_N(11) CASE_N(12) CASE_N(13) CASE_N(14) CASE_N(15) CASE_N(16)
    }
  }
#undef CASE_W
#undef CASE_N
  int n4 = M * (N / 4);
  LAUNCH_PDL(dev, gemv_kn_reduce_kernel, (n4 + 255) / 256, 256, 0, part, ksplit, M, N, e, N);
  return WGPT_OK;
}

// ---- int8 weight handle: the load step of the prototype (it creates a buffer for the packed matrix and uploads it
// once, other/int8-gemm.js:101-113, then dispatches against it). The handle owns a re-laid-out copy.
struct wgpt_int8_weight {
  wgpt_device *dev;
  int K, N;
  uint32_t *words;   // [K, N/4], the prototype's packing (copy)
  uint8_t *bytes;    // [N, K], K contiguous; nullptr when K % 16 != 0
  float *scale;      // [N]
};

WGPT_EXPORT int32_t wgpt_int8_weight_create(wgpt_device *dev, int32_t K, int32_t N, const uint32_t *Bq,
                                            const float *scale, wgpt_int8_weight **out) {
  TRY(use(dev));
  REQUIRE(Bq && scale && out, WGPT_ERR_ARG, "null pointer");
  *out = nullptr;
  NOT_RECORDING(dev, "wgpt_int8_weight_create");
  REQUIRE(K >= 4 && N >= 8 && N % 8 == 0 && K % 4 == 0, WGPT_ERR_SHAPE, "N must be divisible by 8 and K by 4");
  REQUIRE(aligned16(Bq) && aligned16(scale), WGPT_ERR_ALIGN, "buffers must be 16-byte aligned");
  wgpt_int8_weight *w = new wgpt_int8_weight();
  w->dev = dev; w->K = K; w->N = N; w->words = nullptr; w->bytes = nullptr; w->scale = nullptr;
  const size_t nbytes = (size_t)K * N;
  cudaError_t e = cudaMalloc(&w->words, nbytes);
  if (e == cudaSuccess) e = cudaMalloc(&w->scale, (size_t)N * 4);
  if (e == cudaSuccess && K % 16 == 0) e = cudaMalloc(&w->bytes, nbytes);
  if (e == cudaSuccess) e = cudaMemcpyAsync(w->words, Bq, nbytes, cudaMemcpyDeviceToDevice, dev->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(w->scale, scale, (size_t)N * 4, cudaMemcpyDeviceToDevice, dev->stream);
  if (e != cudaSuccess) {
    cudaFree(w->words); cudaFree(w->scale); cudaFree(w->bytes);
    delete w;
    return fail(e == cudaErrorMemoryAllocation ? WGPT_ERR_OOM : WGPT_ERR_CUDA, "int8 weight: %s", cudaGetErrorString(e));
  }
  if (w->bytes) {
    dim3 grid((N / 4 + 31) / 32, (K + 31) / 32);
    LAUNCH(dev, int8_relayout_nk_kernel, grid, 256, 0, (const uint32_t *)w->words, K, N, w->bytes);
  }
  CK(cudaStreamSynchronize(dev->stream));
  *out = w;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_int8_weight_destroy(wgpt_int8_weight *w) {
  if (!w) return WGPT_OK;
  TRY(use(w->dev));
  NOT_RECORDING(w->dev, "wgpt_int8_weight_destroy");
  CK(cudaStreamSynchronize(w->dev->stream));
  cudaFree(w->words); cudaFree(w->scale); cudaFree(w->bytes);
  delete w;
  return WGPT_OK;
}

template <int M>
static int32_t launch_int8_block_t(wgpt_device *dev, const wgpt_int8_weight *w, const float *A, float *out) {
  const int K = w->K, N = w->N, nw = kInt8BlockThreads / 32;
  const int cols = (N + dev->sm_count - 1) / dev->sm_count;
  int wk = 1;
  while (cols * wk < 2 * nw && wk < 8 && (K / 16) / (wk * 2) >= 32) wk *= 2;
  const size_t red = (size_t)(cols * wk > nw ? cols * wk : nw) * M;
  const size_t smem = (size_t)cols * K + ((size_t)M * K + ((red + 3) & ~size_t(3))) * 4 + 16;
  if (smem > dev->smem_optin - 2048) return WGPT_ERR_UNSUPPORTED;  // caller falls back (no message: not an error)
  auto kern = int8_block_gemv_kernel<M>;
  if (smem > 48 * 1024) CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  // the whole carveout, so that the next launch's CTA fits beside this one and fetches its codes early
  CK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
  LAUNCH_PDL(dev, kern, (N + cols - 1) / cols, kInt8BlockThreads, smem, A, (const uint8_t *)w->bytes,
             (const float *)w->scale, K, N, cols, wk, out, dev->d_err);
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_int8_matmul_w(wgpt_device *dev, int32_t M, const wgpt_int8_weight *w, const float *A,
                                       float *out) {
  TRY(use(dev));
  REQUIRE(w && A && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(w->dev == dev, WGPT_ERR_ARG, "the weight belongs to another device handle");
  REQUIRE(M >= 1, WGPT_ERR_SHAPE, "empty int8 matmul");
  REQUIRE(aligned16(A) && aligned16(out), WGPT_ERR_ALIGN, "buffers must be 16-byte aligned");
  const int K = w->K, N = w->N;
  if (w->bytes != nullptr && M <= 4) {
    int32_t rc = WGPT_ERR_UNSUPPORTED;
    switch (M) {
      case 1: rc = launch_int8_block_t<1>(dev, w, A, out); break;
      case 2: rc = launch_int8_block_t<2>(dev, w, A, out); break;
      case 3: rc = launch_int8_block_t<3>(dev, w, A, out); break;
      case 4: rc = launch_int8_block_t<4>(dev, w, A, out); break;
    }
    if (rc != WGPT_ERR_UNSUPPORTED) return rc;
  }
  if (w->bytes != nullptr && M > 16 && dev->precision != WGPT_PRECISION_FP32) {
    // many rows: the codes are expanded to an FP32 [N,K] weight in the workspace (exact; one coalesced pass) and the
    // tcgen05 product runs on it with the scales in its epilogue
    TRY(scratch_reserve(dev, (size_t)N * K * 4));
    float *wt = static_cast<float *>(dev->scratch);
    const size_t n16 = (size_t)N * K / 16;
    LAUNCH(dev, int8_expand_bytes_kernel, grid_for(n16, 256, dev->sm_count), 256, 0, (const uint8_t *)w->bytes, n16, wt);
    Epilogue e = plain_epi(out, N, nullptr);
    e.colscale = w->scale;
    return launch_gemm_tc(dev, dev->precision == WGPT_PRECISION_TF32X3, A, (size_t)K, wt, M, K, N, e, nullptr, false,
                          nullptr, nullptr, true);
  }
  return wgpt_int8_matmul(dev, M, K, N, A, w->words, w->scale, out);
}

// ------------------------------------------------------------------------------------------ model
struct LayerWeights {
  float *ln1_g, *ln1_b, *wqkv_t, *bqkv, *wo_t, *bo, *ln2_g, *ln2_b, *wfc_t, *bfc, *wpr_t, *bpr;
  // low parts of the four matrices for 3xTF32 (w - tf32(w), same [N,K] layout), filled by wgpt_model_finalize
  float *wqkv_lo = nullptr, *wo_lo = nullptr, *wfc_lo = nullptr, *wpr_lo = nullptr;
  // single-sequence fused decode (decode_fused.cuh): per-(head, cluster rank) blocks of the attention weights and
  // the MLP down-projection in the [K,N] orientation, filled by wgpt_model_finalize when the plan applies
  float *attn_blk = nullptr, *wpr_kn = nullptr;
};

// Launch plan of the two-kernels-per-block decode for one model on one device; ok == false keeps the kernel chain.
struct FusedPlan {
  bool ok = false;
  int cs = 0;              // cluster size of attn_block_kernel
  size_t blk_floats = 0;
  int proj_parts = 0, red_a = 0;
  size_t smem_a = 0;
  int units = 0, n_mlp = 0 /* CTAs */, n_mlp_rows = 0 /* clusters = partial rows */, wk = 0, down_parts = 0, red_b = 0;
  size_t smem_b = 0;
  int attn_extra = 0;      // clusters of attn_block_kernel beyond the heads that prefetch the MLP kernel's weights
};

struct wgpt_model {
  wgpt_device *dev;
  wgpt_params p;
  int hs;
  float scale;
  float *wte, *wpe, *lnf_g, *lnf_b;
  std::vector<LayerWeights> layers;
  std::vector<char> have;  // per tensor slot
  bool finalized;
  std::vector<void *> allocs;
  FusedPlan fused;
};

static int32_t model_alloc(wgpt_model *m, float **p, size_t floats) {
  CK(cudaMalloc(reinterpret_cast<void **>(p), floats * 4));
  m->allocs.push_back(*p);
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_model_create(wgpt_device *dev, const wgpt_params *params, wgpt_model **out) {
  TRY(use(dev));
  REQUIRE(params && out, WGPT_ERR_ARG, "null argument");
  *out = nullptr;
  const wgpt_params &p = *params;
  REQUIRE(p.n_layer >= 1 && p.n_head >= 1 && p.n_embd >= 1 && p.n_ctx >= 1 && p.vocab_size >= 1, WGPT_ERR_SHAPE,
          "Model load failed: parameters must be positive.");
  // messages of model.js:294-297
  REQUIRE(p.n_embd % 4 == 0, WGPT_ERR_SHAPE, "Model load failed: n_embd must be divisible by 4.");
  REQUIRE(p.n_embd % p.n_head == 0, WGPT_ERR_SHAPE, "Model load failed: n_embd must be divisible by n_head.");
  REQUIRE((p.n_embd / p.n_head) % 4 == 0, WGPT_ERR_SHAPE, "Model load failed: n_embd / n_head must be divisible by 4.");
  int hs = p.n_embd / p.n_head;
  REQUIRE(hs == 4 || hs == 8 || hs == 16 || hs == 32 || hs == 64 || hs == 128, WGPT_ERR_UNSUPPORTED,
          "head_size %d: supported sizes are 4, 8, 16, 32, 64, 128", hs);
  wgpt_model *m = new wgpt_model();
  m->dev = dev;
  m->p = p;
  m->hs = hs;
  m->scale = (float)(1.0 / std::sqrt((double)hs));  // model.js:321, stored as f32 at instructions.js:1038
  m->finalized = false;
  m->layers.resize(p.n_layer);
  m->have.assign(4 + 12 * (size_t)p.n_layer, 0);
  size_t E = p.n_embd, F = 4 * E;
  int32_t rc = WGPT_OK;
  auto A = [&](float **ptr, size_t n) { if (rc == WGPT_OK) rc = model_alloc(m, ptr, n); };
  A(&m->wte, (size_t)p.vocab_size * E);
  A(&m->wpe, (size_t)p.n_ctx * E);
  A(&m->lnf_g, E);
  A(&m->lnf_b, E);
  for (auto &L : m->layers) {
    A(&L.ln1_g, E); A(&L.ln1_b, E); A(&L.wqkv_t, 3 * E * E); A(&L.bqkv, 3 * E); A(&L.wo_t, E * E); A(&L.bo, E);
    A(&L.ln2_g, E); A(&L.ln2_b, E); A(&L.wfc_t, F * E); A(&L.bfc, F); A(&L.wpr_t, E * F); A(&L.bpr, E);
  }
  if (rc != WGPT_OK) {
    for (void *q : m->allocs) cudaFree(q);
    delete m;
    return rc;
  }
  *out = m;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_model_destroy(wgpt_model *m) {
  REQUIRE(m != nullptr, WGPT_ERR_ARG, "model handle is null");
  TRY(use(m->dev));
  NOT_RECORDING(m->dev, "wgpt_model_destroy");
  cudaStreamSynchronize(m->dev->stream);
  for (void *q : m->allocs) cudaFree(q);
  delete m;
  return WGPT_OK;
}

// Uploads a tensor; matmul weights arrive as [in,out] = [K,N] and are stored transposed as [N,K] so that
// each output column's weights are contiguous (the reference also re-lays-out at load: model.js:362,456-468).
static int32_t upload(wgpt_model *m, float *dst, const float *src_host, size_t rows, size_t cols, bool transpose) {
  wgpt_device *dev = m->dev;
  size_t n = rows * cols;
  if (!transpose) {
    CK(cudaMemcpyAsync(dst, src_host, n * 4, cudaMemcpyHostToDevice, dev->stream));
    CK(cudaStreamSynchronize(dev->stream));
    return WGPT_OK;
  }
  TRY(scratch_reserve(dev, n * 4));
  CK(cudaMemcpyAsync(dev->scratch, src_host, n * 4, cudaMemcpyHostToDevice, dev->stream));
  dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
  LAUNCH(dev, transpose_kernel, grid, dim3(32, 8), 0, static_cast<const float *>(dev->scratch), dst, (int)rows,
         (int)cols);
  CK(cudaStreamSynchronize(dev->stream));
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_model_set_tensor(wgpt_model *m, const char *name, const float *data, uint64_t count) {
  REQUIRE(m && name && data, WGPT_ERR_ARG, "null argument");
  TRY(use(m->dev));
  NOT_RECORDING(m->dev, "wgpt_model_set_tensor");
  REQUIRE(!m->finalized, WGPT_ERR_STATE, "Model already loaded");
  size_t E = m->p.n_embd, F = 4 * E, V = m->p.vocab_size, C = m->p.n_ctx;
  std::string s(name);
  float *dst = nullptr;
  size_t rows = 1, cols = 0;
  bool tr = false;
  int slot = -1;
  if (s == "transformer.wte.weight") { dst = m->wte; rows = V; cols = E; slot = 0; }
  else if (s == "transformer.wpe.weight") { dst = m->wpe; rows = C; cols = E; slot = 1; }
  else if (s == "transformer.ln_f.weight") { dst = m->lnf_g; cols = E; slot = 2; }
  else if (s == "transformer.ln_f.bias") { dst = m->lnf_b; cols = E; slot = 3; }
  else if (s.rfind("transformer.h.", 0) == 0) {
    size_t dot = s.find('.', 14);
    REQUIRE(dot != std::string::npos, WGPT_ERR_ARG, "unknown tensor name '%s'", name);
    int l = atoi(s.substr(14, dot - 14).c_str());
    REQUIRE(l >= 0 && l < m->p.n_layer, WGPT_ERR_ARG, "layer index out of range in '%s'", name);
    std::string k = s.substr(dot + 1);
    LayerWeights &L = m->layers[l];
    int j = -1;
    if (k == "ln_1.weight") { dst = L.ln1_g; cols = E; j = 0; }
    else if (k == "ln_1.bias") { dst = L.ln1_b; cols = E; j = 1; }
    else if (k == "attn.c_attn.weight") { dst = L.wqkv_t; rows = E; cols = 3 * E; tr = true; j = 2; }
    else if (k == "attn.c_attn.bias") { dst = L.bqkv; cols = 3 * E; j = 3; }
    else if (k == "attn.c_proj.weight") { dst = L.wo_t; rows = E; cols = E; tr = true; j = 4; }
    else if (k == "attn.c_proj.bias") { dst = L.bo; cols = E; j = 5; }
    else if (k == "ln_2.weight") { dst = L.ln2_g; cols = E; j = 6; }
    else if (k == "ln_2.bias") { dst = L.ln2_b; cols = E; j = 7; }
    else if (k == "mlp.c_fc.weight") { dst = L.wfc_t; rows = E; cols = F; tr = true; j = 8; }
    else if (k == "mlp.c_fc.bias") { dst = L.bfc; cols = F; j = 9; }
    else if (k == "mlp.c_proj.weight") { dst = L.wpr_t; rows = F; cols = E; tr = true; j = 10; }
    else if (k == "mlp.c_proj.bias") { dst = L.bpr; cols = E; j = 11; }
    REQUIRE(j >= 0, WGPT_ERR_ARG, "unknown tensor name '%s'", name);
    slot = 4 + 12 * l + j;
  }
  REQUIRE(slot >= 0, WGPT_ERR_ARG, "unknown tensor name '%s'", name);
  REQUIRE(count == rows * cols, WGPT_ERR_SHAPE, "tensor '%s' has %llu values, expected %llu", name,
          (unsigned long long)count, (unsigned long long)(rows * cols));
  TRY(upload(m, dst, data, rows, cols, tr));
  m->have[slot] = 1;
  return WGPT_OK;
}


// ------------------------------------------------------------------------------------------ fused decode plan
template <int HS, int CS>
static int32_t attn_block_launch_t(wgpt_device *dev, const FusedPlan &fp, int H, const AttnBlockParams &a,
                                   int *max_clusters) {
  auto kern = attn_block_kernel<HS, CS>;
  CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp.smem_a));
  // the whole shared-memory carveout: the next kernel's CTA must fit on the SM beside this one to fetch its
  // weights while this one runs
  CK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
  if (max_clusters != nullptr) {  // planning: how many clusters of this shape can be resident at once
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(H * CS);
    cfg.blockDim = dim3(kAttnBlockThreads);
    cfg.dynamicSmemBytes = fp.smem_a;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CK(cudaOccupancyMaxActiveClusters(max_clusters, kern, &cfg));
    return WGPT_OK;
  }
  const int extra = a.pf_a != nullptr ? fp.attn_extra : 0;  // clusters that only prefetch for the next kernel
  CK(launch_cluster_x(dev->pdl, CS, dev->stream, kern, dim3((H + extra) * CS), dim3(kAttnBlockThreads), fp.smem_a, a));
  dev->launches++;
  return WGPT_OK;
}

// Dispatch on (head size, cluster size). With max_clusters != nullptr nothing is launched (occupancy query).
static int32_t attn_block_launch(wgpt_device *dev, const FusedPlan &fp, int hs, int H, const AttnBlockParams &a,
                                 int *max_clusters = nullptr) {
#define CASE_A(HSV, CSV) \
  if (hs == HSV && fp.cs == CSV) return attn_block_launch_t<HSV, CSV>(dev, fp, H, a, max_clusters);
  CASE_A(128, 8) CASE_A(64, 8) CASE_A(32, 8) CASE_A(16, 8) CASE_A(8, 8)
  CASE_A(128, 4) CASE_A(64, 4) CASE_A(32, 4) CASE_A(16, 4) CASE_A(8, 4) CASE_A(4, 4)
#undef CASE_A
  return fail(WGPT_ERR_UNSUPPORTED, "no fused attention kernel for head_size %d with clusters of %d", hs, fp.cs);
}

template <int HS, int CS>
static size_t attn_block_smem_t(int E, int red) { return attn_block_smem_floats<HS, CS>(E, red) * 4; }

static size_t attn_block_smem(int hs, int cs, int E, int red) {
  // attn_block_smem_floats for run-time hs, cs
  return ((size_t)3 * (hs / cs) * E + (size_t)E + red + 3 * hs + (size_t)cs * (hs + 4) + hs + 8) * 4;
}

// Decides whether single-sequence decode of this model can run as two kernels per block on this device: both
// kernels' weight slices must fit in one SM's shared memory side by side (each prefetches its weights while the
// other is still running), and one cluster per head must be resident at once.
static int32_t fused_plan(wgpt_model *m) {
  wgpt_device *dev = m->dev;
  FusedPlan &fp = m->fused;
  fp = FusedPlan();
  const int E = m->p.n_embd, H = m->p.n_head, hs = m->hs, F = 4 * E;
  if (!dev->fused_decode || E % 32 != 0) return WGPT_OK;
  // MLP kernel: clusters of kMlpCluster CTAs, as many as can be resident at once (at most one CTA per SM), each
  // CTA a contiguous slice of the hidden units
  if ((E / 4) % kMlpCluster != 0 || E / 4 > kAttnBlockThreads) return WGPT_OK;
  auto mlp = mlp_block_kernel;
  int clusters = dev->sm_count / kMlpCluster;
  for (int attempt = 0; attempt < 2; attempt++) {
    fp.n_mlp = clusters * kMlpCluster;
    if (fp.n_mlp > F) fp.n_mlp = (F / kMlpCluster) * kMlpCluster;
    if (fp.n_mlp < kMlpCluster) return WGPT_OK;
    fp.n_mlp_rows = fp.n_mlp / kMlpCluster;
    fp.units = (F + fp.n_mlp - 1) / fp.n_mlp;
    fp.wk = 1;
    while (fp.units * fp.wk < 2 * (kMlpBlockThreads / 32) && fp.wk < 8 && (E / 4) / (fp.wk * 2) >= 32) fp.wk *= 2;
    fp.down_parts = kMlpBlockThreads / (E / 4);
    if (fp.down_parts > fp.units) fp.down_parts = fp.units;
    if (fp.down_parts < 1) return WGPT_OK;
    int red = fp.units * fp.wk;
    if (red < 2 * (kMlpBlockThreads / 32)) red = 2 * (kMlpBlockThreads / 32);
    fp.red_b = (red + 3) & ~3;
    fp.smem_b = mlp_block_smem_floats(E, fp.units, fp.red_b) * 4;
    if (fp.smem_b > (size_t)dev->smem_optin) return WGPT_OK;
    // limits of the batched row sums (warp_rows_partial / halfwarp_rows_sum in decode_fused.cuh)
    if (fp.n_mlp_rows > (kAttnBlockThreads / 32) * kAttnSumRows || H > 2 * kMlpSumRows ||
        (E / 4) / kMlpCluster > 16 * (kMlpBlockThreads / 32))
      return WGPT_OK;
    CK(cudaFuncSetAttribute(mlp, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp.smem_b));
    CK(cudaFuncSetAttribute(mlp, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(fp.n_mlp);
    cfg.blockDim = dim3(kMlpBlockThreads);
    cfg.dynamicSmemBytes = fp.smem_b;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kMlpCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int max_clusters = 0;
    CK(cudaOccupancyMaxActiveClusters(&max_clusters, mlp, &cfg));
    if (getenv("WGPT_DEBUG_PLAN"))
      fprintf(stderr, "[wgpt plan] mlp: grid %d units %d smem %zu -> max active clusters of %d: %d\n", fp.n_mlp, fp.units,
              fp.smem_b, kMlpCluster, max_clusters);
    if (max_clusters >= fp.n_mlp_rows) break;
    if (attempt == 1 || max_clusters < 1) return WGPT_OK;
    clusters = max_clusters;  // fewer clusters fit side by side than SMs / 4: size the grid to what is resident
  }
  for (int cs : {8, 4}) {
    if (hs % cs != 0 || E % (4 * cs) != 0 || (cs == 8 && hs < 8)) continue;
    const int ncolA = E / cs, ncol4 = ncolA / 4;
    if (ncolA > kAttnBlockThreads || ncol4 > 32) continue;
    fp.cs = cs;
    (void)ncol4;
    fp.proj_parts = kAttnBlockThreads / ncolA < hs ? kAttnBlockThreads / ncolA : hs;
    int red = (kAttnBlockThreads / 32) * (hs + 4);
    if (red < (kAttnBlockThreads / 32) * 32 * 4) red = (kAttnBlockThreads / 32) * 32 * 4;  // [warps][32] float4 row sums
    if (fp.proj_parts * ncolA > red) red = fp.proj_parts * ncolA;
    fp.red_a = (red + 3) & ~3;
    fp.blk_floats = (size_t)3 * (hs / cs) * E + (size_t)hs * ncolA;
    fp.smem_a = attn_block_smem(hs, cs, E, fp.red_a);
    // side by side on one SM, 1 KB reserved per resident CTA
    if (getenv("WGPT_DEBUG_PLAN"))
      fprintf(stderr, "[wgpt plan] attn cluster %d: smem %zu + mlp %zu (limit %zu)\n", cs, fp.smem_a, fp.smem_b,
              (size_t)dev->smem_optin + 1024 - 2048);
    if (fp.smem_a + fp.smem_b + 2048 > (size_t)dev->smem_optin + 1024) continue;
    int max_clusters = 0;
    AttnBlockParams dummy;
    memset(&dummy, 0, sizeof dummy);
    if (attn_block_launch(dev, fp, hs, H, dummy, &max_clusters) != WGPT_OK) continue;
    if (getenv("WGPT_DEBUG_PLAN"))
      fprintf(stderr, "[wgpt plan] attn: cluster %d smem %zu -> max active clusters %d (need %d)\n", cs, fp.smem_a,
              max_clusters, H);
    if (max_clusters < H) continue;
    fp.ok = true;
    {  // two more clusters when they are resident together with the heads' and SMs are left over for them
      const char *ev = getenv("WGPT_ATTN_EXTRA");
      const int want = ev ? atoi(ev) : 2;
      fp.attn_extra = (max_clusters >= H + want && (H + want) * cs <= dev->sm_count && want >= 2) ? want : 0;
    }
    break;
  }
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_model_finalize(wgpt_model *m) {
  REQUIRE(m != nullptr, WGPT_ERR_ARG, "model handle is null");
  for (size_t i = 0; i < m->have.size(); i++)
    REQUIRE(m->have[i], WGPT_ERR_STATE, "tensor slot %zu was never set (4 + 12*layer + index)", i);
  TRY(use(m->dev));
  {
    const size_t E = m->p.n_embd, F = 4 * E;
    for (auto &L : m->layers) {
      struct { const float *src; float **dst; size_t n; } jobs[4] = {
          {L.wqkv_t, &L.wqkv_lo, 3 * E * E}, {L.wo_t, &L.wo_lo, E * E}, {L.wfc_t, &L.wfc_lo, F * E}, {L.wpr_t, &L.wpr_lo, E * F}};
      for (auto &j : jobs) {
        if (*j.dst == nullptr) TRY(model_alloc(m, j.dst, j.n));
        size_t n4 = j.n / 4;
        LAUNCH(m->dev, tf32_lo_kernel, grid_for(n4, 256, m->dev->sm_count), 256, 0,
               reinterpret_cast<const float4 *>(j.src), reinterpret_cast<float4 *>(*j.dst), n4);
      }
    }
  }
  TRY(fused_plan(m));
  if (m->fused.ok) {
    const int E = m->p.n_embd, F = 4 * E, H = m->p.n_head;
    const size_t blk_total = m->fused.blk_floats * H * m->fused.cs;
    for (auto &L : m->layers) {
      if (L.attn_blk == nullptr) TRY(model_alloc(m, &L.attn_blk, blk_total));
      if (L.wpr_kn == nullptr) TRY(model_alloc(m, &L.wpr_kn, (size_t)F * E));
      LAUNCH(m->dev, fused_attn_relayout_kernel, grid_for(blk_total, 256, m->dev->sm_count), 256, 0,
             (const float *)L.wqkv_t, (const float *)L.wo_t, L.attn_blk, E, H, m->hs, m->fused.cs);
      // wpr_t is [E, F] (N rows of K); its transpose is the reference's [K, N] orientation
      dim3 tg((unsigned)((F + 31) / 32), (unsigned)((E + 31) / 32));
      LAUNCH(m->dev, transpose_kernel, tg, dim3(32, 8), 0, (const float *)L.wpr_t, L.wpr_kn, E, F);
    }
  }
  CK(cudaStreamSynchronize(m->dev->stream));
  m->finalized = true;
  return WGPT_OK;
}

// ------------------------------------------------------------------------------------------ session
struct wgpt_session {
  wgpt_model *m = nullptr;
  int n_seq = 0;
  int len;       // tokens held per sequence (host mirror of *d_pos)
  int cap_tok;   // tokens per forward the activation buffers are sized for
  int out_cap;   // capacity (per sequence) of d_out_ids
  int last_rows; // rows of the most recent forward (for the tap)
  int n_split;        // position slices of the decode attention (attn_split_for), fixed while a step graph lives
  bool split_forced;  // set by WGPT_ATTN_SPLIT
  float *x, *h, *q, *o, *f, *logits;
  float *kc, *vc;  // [n_layer][n_seq][n_ctx][E]
  float *fx_a = nullptr, *fx_b = nullptr;     // fused decode: residual stream entering the attention / MLP kernel
  float *fpart_a = nullptr, *fpart_b = nullptr;  // fused decode: partial results [n_head][E] and [mlp CTAs][E]
  float *attn_part;  // decode-attention partials, [n_seq][n_head][n_split][hs + 4]
  unsigned int *attn_cnt;
  uint32_t *ids, *next_ids, *out_ids;
  float *pick_val;  // [n_seq][vocab] per-CTA arg-max candidates of the fused greedy pick
  int *pick_idx;
  unsigned long long *pick_keys;  // [8] (value, index) keys of gemv_loop_kernel's greedy pick, zero between launches
  int *d_pos, *d_step;
  std::vector<uint32_t> prompts;  // host copy, [n_seq][n_prompt]
  int n_prompt, n_generated;
  bool ids_dirty;  // s->ids no longer holds the prompt window
  // top-k sampling (0 = greedy pick): parameters and the per-(step, sequence) uniform numbers on the device
  int sample_k = 0;
  double sample_temp = 1.0;
  double *d_uniform = nullptr;
  size_t uniform_cap = 0;  // doubles
  cudaGraphExec_t step_graph;  // one captured decode step (pointers of this session baked in)
  uint64_t step_graph_launches;
  bool step_warm;
};

static void drop_step_graph(wgpt_session *s);

static void session_free_act(wgpt_session *s) {
  cudaFree(s->x); cudaFree(s->h); cudaFree(s->q); cudaFree(s->o); cudaFree(s->f); cudaFree(s->ids);
  s->x = s->h = s->q = s->o = s->f = nullptr;
  s->ids = nullptr;
}

static int32_t session_reserve(wgpt_session *s, int n_tok) {
  if (n_tok <= s->cap_tok) return WGPT_OK;
  wgpt_device *dev = s->m->dev;
  CK(cudaStreamSynchronize(dev->stream));
  drop_step_graph(s);  // the captured step holds the old buffer addresses
  session_free_act(s);
  s->cap_tok = 0;
  size_t M = (size_t)s->n_seq * n_tok, E = s->m->p.n_embd;
  CK(cudaMalloc(&s->x, M * E * 4)); CK(cudaMalloc(&s->h, M * E * 4)); CK(cudaMalloc(&s->q, M * E * 4));
  CK(cudaMalloc(&s->o, M * E * 4)); CK(cudaMalloc(&s->f, M * 4 * E * 4)); CK(cudaMalloc(&s->ids, M * 4));
  s->cap_tok = n_tok;
  return WGPT_OK;
}

// Position slices per (sequence, head) of the decode attention: 1, 2, 4 or 8 CTAs share a head's cache rows.
// Doubled while the grid stays within a CTA budget: about two CTAs per SM for up to eight sequences with a short
// context (the projection that follows merges the slices of every row in every CTA, so slices are not free
// there), about five per SM for more sequences or a long context, where the attention itself is what costs.
// Measured per decode pass, chosen / other: GPT-2 117M 16 rows 0.606 (4) / 0.645 (1), 32 rows 0.683 (2) / 0.711 (1),
// 64 rows 0.791 (1) / 0.820 (2), 8 rows 0.574 (2) / 0.584 (8); GPT-2 XL at 768+ positions 8 sequences 6.57 (4) /
// 7.46 (1), 16 sequences 6.70 (2) / 7.66 (1), 32 sequences 8.23 (1) / 8.28 (4) ms.
constexpr int kMaxAttnSplit = 8;
static int attn_split_for(const wgpt_device *dev, int n_head, int n_seq, int context_len) {
  const int budget = (n_seq > 8 || context_len >= 512) ? (11 * dev->sm_count) / 2 : 2 * dev->sm_count;
  int split = 1;
  while (split < kMaxAttnSplit && n_head * n_seq * split * 2 <= budget) split *= 2;
  return split;
}

WGPT_EXPORT int32_t wgpt_session_create(wgpt_model *m, int32_t n_seq, wgpt_session **out) {
  REQUIRE(m && out, WGPT_ERR_ARG, "null argument");
  *out = nullptr;
  TRY(use(m->dev));
  REQUIRE(m->finalized, WGPT_ERR_STATE, "Model not loaded yet");
  NOT_RECORDING(m->dev, "wgpt_session_create");
  REQUIRE(n_seq >= 1, WGPT_ERR_SHAPE, "n_seq must be at least 1");
  wgpt_session *s = new wgpt_session();
  s->m = m;
  s->n_seq = n_seq;
  const wgpt_params &p = m->p;
  size_t kv = (size_t)p.n_layer * n_seq * p.n_ctx * p.n_embd;
  s->split_forced = false;
  if (const char *ev = getenv("WGPT_ATTN_SPLIT")) {  // tuning override: 1, 2, 4 or 8
    int v = atoi(ev);
    if (v == 1 || v == 2 || v == 4 || v == 8) {
      s->n_split = v;
      s->split_forced = true;
    }
  }
  if (!s->split_forced) s->n_split = attn_split_for(m->dev, p.n_head, n_seq, 0);
  cudaError_t e = cudaMalloc(&s->kc, kv * 4);
  if (e == cudaSuccess) e = cudaMalloc(&s->vc, kv * 4);
  if (e == cudaSuccess) e = cudaMalloc(&s->logits, (size_t)n_seq * p.vocab_size * 4);
  if (e == cudaSuccess) e = cudaMalloc(&s->attn_part, (size_t)n_seq * p.n_head * kMaxAttnSplit * (m->hs + 4) * 4);
  if (e == cudaSuccess) e = cudaMalloc(&s->attn_cnt, ((size_t)n_seq * p.n_head + 1) * 4);  // + arg-max done counter
  if (e == cudaSuccess) e = cudaMalloc(&s->next_ids, (size_t)n_seq * 4);
  if (e == cudaSuccess) e = cudaMalloc(&s->pick_val, (size_t)n_seq * p.vocab_size * 4);
  if (e == cudaSuccess) e = cudaMalloc(&s->pick_idx, (size_t)n_seq * p.vocab_size * 4);
  if (e == cudaSuccess) e = cudaMalloc(&s->pick_keys, 8 * sizeof(unsigned long long));
  if (e == cudaSuccess) e = cudaMemsetAsync(s->pick_keys, 0, 8 * sizeof(unsigned long long), m->dev->stream);
  if (e == cudaSuccess) e = cudaMalloc(&s->d_pos, 2 * sizeof(int));
  if (e == cudaSuccess && m->fused.ok && n_seq == 1) {
    const size_t E = p.n_embd;
    e = cudaMalloc(&s->fx_a, E * 4);
    if (e == cudaSuccess) e = cudaMalloc(&s->fx_b, E * 4);
    if (e == cudaSuccess) e = cudaMalloc(&s->fpart_a, (size_t)p.n_head * E * 4);
    if (e == cudaSuccess) e = cudaMalloc(&s->fpart_b, (size_t)m->fused.n_mlp * E * 4);
  }
  if (e == cudaSuccess) e = cudaMemsetAsync(s->attn_cnt, 0, ((size_t)n_seq * p.n_head + 1) * 4, m->dev->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(s->d_pos, 0, 2 * sizeof(int), m->dev->stream);
  if (e != cudaSuccess) {
    cudaFree(s->kc); cudaFree(s->vc); cudaFree(s->logits); cudaFree(s->attn_part); cudaFree(s->attn_cnt);
    cudaFree(s->next_ids); cudaFree(s->d_pos); cudaFree(s->pick_val); cudaFree(s->pick_idx); cudaFree(s->pick_keys);
    cudaFree(s->fx_a); cudaFree(s->fx_b); cudaFree(s->fpart_a); cudaFree(s->fpart_b);
    delete s;
    return fail(e == cudaErrorMemoryAllocation ? WGPT_ERR_OOM : WGPT_ERR_CUDA, "session allocation: %s",
                cudaGetErrorString(e));
  }
  s->d_step = s->d_pos + 1;
  *out = s;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_session_destroy(wgpt_session *s) {
  REQUIRE(s != nullptr, WGPT_ERR_ARG, "session handle is null");
  TRY(use(s->m->dev));
  NOT_RECORDING(s->m->dev, "wgpt_session_destroy");
  cudaStreamSynchronize(s->m->dev->stream);
  drop_step_graph(s);
  session_free_act(s);
  cudaFree(s->kc); cudaFree(s->vc); cudaFree(s->logits); cudaFree(s->attn_part); cudaFree(s->attn_cnt);
  cudaFree(s->next_ids); cudaFree(s->out_ids); cudaFree(s->d_pos); cudaFree(s->pick_val); cudaFree(s->pick_idx); cudaFree(s->pick_keys);
  cudaFree(s->d_uniform);
  cudaFree(s->fx_a); cudaFree(s->fx_b); cudaFree(s->fpart_a); cudaFree(s->fpart_b);
  delete s;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_session_reset(wgpt_session *s) {
  REQUIRE(s != nullptr, WGPT_ERR_ARG, "session handle is null");
  TRY(use(s->m->dev));
  CK(cudaMemsetAsync(s->d_pos, 0, 2 * sizeof(int), s->m->dev->stream));
  s->len = 0;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_session_length(wgpt_session *s, int32_t *length) {
  REQUIRE(s && length, WGPT_ERR_ARG, "null argument");
  *length = s->len;
  return WGPT_OK;
}

// One forward pass over n_tok new tokens per sequence whose ids are already in `ids` (device, [n_seq*n_tok]).
// Leaves the logits of each sequence's newest position in s->logits. Does not advance the position.
static int32_t pick_and_advance(wgpt_session *s, int n_tok);


// The transformer blocks of a single-sequence decode step as two kernels per block (decode_fused.cuh); leaves the
// residual stream before ln_f in s->x.
static int32_t forward_blocks_fused(wgpt_session *s, const uint32_t *ids) {
  wgpt_model *m = s->m;
  wgpt_device *dev = m->dev;
  const wgpt_params &p = m->p;
  const FusedPlan &fp = m->fused;
  const int E = p.n_embd, F = 4 * E, H = p.n_head;
  const size_t kv_layer = (size_t)p.n_ctx * E;
  auto mlp = mlp_block_kernel;
  if (fp.smem_b > 48 * 1024) CK(cudaFuncSetAttribute(mlp, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp.smem_b));
  CK(cudaFuncSetAttribute(mlp, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
  for (int l = 0; l < p.n_layer; l++) {
    const LayerWeights &L = m->layers[l];
    AttnBlockParams a;
    memset(&a, 0, sizeof a);
    if (l == 0) {
      a.ids = ids; a.wte = m->wte; a.wpe = m->wpe; a.vocab = p.vocab_size;
    } else {
      a.xin = s->fx_b; a.part_in = s->fpart_b; a.bias_in = m->layers[l - 1].bpr; a.n_part = fp.n_mlp_rows;
    }
    a.x_out = s->fx_a;
    a.gamma = L.ln1_g; a.beta = L.ln1_b;
    a.wblk = L.attn_blk; a.blk_floats = fp.blk_floats; a.bqkv = L.bqkv;
    a.kc = s->kc + (size_t)l * kv_layer; a.vc = s->vc + (size_t)l * kv_layer;
    a.part_out = s->fpart_a;
    a.pos = s->d_pos;
    a.E = E; a.H = H; a.scale = m->scale;
    a.proj_parts = fp.proj_parts; a.red_floats = fp.red_a;
    a.err = dev->d_err;
    if (fp.attn_extra > 0) {  // the MLP kernel's weights, for the clusters beyond the heads
      a.pf_a = reinterpret_cast<const char *>(L.wfc_t); a.pf_b = reinterpret_cast<const char *>(L.wpr_kn);
      a.pf_bytes = (unsigned int)((size_t)F * E * 4);
    }
    TRY(attn_block_launch(dev, fp, m->hs, H, a));
    MlpBlockParams b;
    memset(&b, 0, sizeof b);
    b.xin = s->fx_a; b.part_in = s->fpart_a; b.bias_in = L.bo; b.n_part = H;
    b.x_out = s->fx_b;
    b.gamma = L.ln2_g; b.beta = L.ln2_b;
    b.wfc_t = L.wfc_t; b.bfc = L.bfc; b.wpr_kn = L.wpr_kn;
    b.part_out = s->fpart_b;
    b.E = E; b.F = F; b.units = fp.units; b.wk = fp.wk; b.down_parts = fp.down_parts; b.red_floats = fp.red_b;
    b.err = dev->d_err;
    CK(launch_cluster_x(dev->pdl, kMlpCluster, dev->stream, mlp, dim3(fp.n_mlp), dim3(kMlpBlockThreads), fp.smem_b, b));
    dev->launches++;
  }
  LAUNCH_PDL(dev, finish_row_kernel, (E / 4 + 31) / 32, 256, 0, (const float *)s->fx_b,
             (const float *)m->layers[p.n_layer - 1].bpr, (const float *)s->fpart_b, fp.n_mlp_rows, E, s->x);
  return WGPT_OK;
}

// With pick, the greedy choice of every sequence is also made (next_ids, out_ids) and the position advanced.
static int32_t forward(wgpt_session *s, const uint32_t *ids, int n_tok, bool pick = false) {
  wgpt_model *m = s->m;
  wgpt_device *dev = m->dev;
  const wgpt_params &p = m->p;
  const int E = p.n_embd, F = 4 * E, H = p.n_head, hs = m->hs, M = s->n_seq * n_tok;
  const size_t kv_layer = (size_t)s->n_seq * p.n_ctx * E;

  const bool fused = n_tok == 1 && s->n_seq == 1 && m->fused.ok && s->fx_a != nullptr;
  if (!fused)
    LAUNCH_PDL(dev, embed_kernel, M, 128, 0, ids, m->wte, m->wpe, s->x, M, n_tok, E, p.vocab_size,
               (const int *)s->d_pos, dev->d_err);

  // s->h already holds the LayerNorm of s->x that the next product wants (left there by the split-K second
  // stage of the product that wrote s->x)
  bool h_ready = false;
  auto mm = [&](const float *a, const float *gamma, const float *beta, const float *Wt, const float *Wt_lo, int K,
                int N, const Epilogue &e, const float *next_gamma = nullptr, const float *next_beta = nullptr,
                SplitHandoff *handoff = nullptr) -> int32_t {
    // a: [M,K] contiguous. Small M: weight-streaming GEMV with the LayerNorm fused in; otherwise a LayerNorm pass
    // into s->h (separate, or riding on the previous product's second stage) and a tiled GEMM. next_gamma/beta:
    // the LayerNorm that will consume this product's output rows e.out[M,N].
    if (gemv_nk_fits(dev, M, K)) {
      // Many rows of a long K leave the register-streaming kernel few warps per SM (the rows fill shared memory):
      // unless the shared-memory block form takes the product, the tiled GEMM in its exchanged form is faster from
      // six rows on (GPT-2 XL decode pass: 5.89 against 6.60 ms at eight rows, 5.50 against 5.16 ms at four). FP32
      // mode keeps the GEMV: its GEMM runs on the CUDA cores.
      int bc = 0, bw = 0;
      size_t bs = 0;
      const bool block_form = dev->block_gemv && gemv_block_plan(dev, M, K, N, gamma != nullptr, &bc, &bw, &bs);
      if (block_form || M <= dev->gemv_stream_max_rows || dev->precision == WGPT_PRECISION_FP32)
        return launch_gemv_nk(dev, M, a, (size_t)K, gamma, beta, Wt, K, N, e);
    }
    const float *src = a;
    if (gamma) {
      if (!h_ready) TRY(launch_layernorm(dev, a, (size_t)K, gamma, beta, s->h, (size_t)K, M, K));
      h_ready = false;
      src = s->h;
    }
    LnAfter ln = {next_gamma, next_beta, s->h, false};
    // the product must not read s->h itself while its second stage rewrites it
    bool can_fuse = next_gamma != nullptr && src != s->h;
    TRY(launch_gemm_nk(dev, src, (size_t)K, Wt, M, K, N, e, can_fuse ? &ln : nullptr, Wt_lo, handoff));
    h_ready = ln.done;
    return WGPT_OK;
  };

  if (fused) TRY(forward_blocks_fused(s, ids));
  for (int l = 0; l < (fused ? 0 : p.n_layer); l++) {
    const LayerWeights &L = m->layers[l];
    float *kc = s->kc + (size_t)l * kv_layer, *vc = s->vc + (size_t)l * kv_layer;
    SplitHandoff qkv_slices;
    {  // LN1 + QKV projection; K and V rows go straight into the cache
      Epilogue e = plain_epi(s->q, E, L.bqkv);
      e.kc = kc; e.vc = vc; e.E = E; e.n_tok = n_tok; e.n_ctx = p.n_ctx; e.pos = s->d_pos;
      // one query per sequence and one position slice: the attention CTAs can add the product's slices themselves
      const bool consumer_sums = n_tok == 1 && s->n_split == 1 && 3 * hs <= 256;
      TRY(mm(s->x, L.ln1_g, L.ln1_b, L.wqkv_t, L.wqkv_lo, E, 3 * E, e, nullptr, nullptr,
             consumer_sums ? &qkv_slices : nullptr));
    }
    if (n_tok == 1 && qkv_slices.taken) {
      QkvPartials qp{qkv_slices.part, L.bqkv, qkv_slices.splits, M, E};
      TRY(launch_attn_decode(dev, hs, s->q, E, kc, vc, E, (size_t)p.n_ctx, s->o, E, s->n_seq, H, s->n_split, s->d_pos,
                             m->scale, s->attn_part, &qp));
    } else if (n_tok == 1)
      TRY(launch_attn_decode(dev, hs, s->q, E, kc, vc, E, (size_t)p.n_ctx, s->o, E, s->n_seq, H, s->n_split, s->d_pos,
                             m->scale, s->attn_part));
    else
      TRY(launch_attn_prefill(dev, hs, s->q, E, kc, vc, E, (size_t)p.n_ctx, s->o, E, n_tok, s->n_seq, H, s->d_pos,
                              m->scale));
    {  // attention output projection + residual
      Epilogue e = plain_epi(s->x, E, L.bo);
      e.residual = s->x;
      if (n_tok == 1 && s->n_split > 1) {
        // the decode attention left per-slice partials; the projection merges them while staging its input
        AttnPartials ap;
        ap.part = s->attn_part; ap.n_split = s->n_split; ap.H = H; ap.hs = hs;
        if (gemv_nk_fits(dev, M, E)) {
          TRY(launch_gemv_nk(dev, M, s->o, (size_t)E, nullptr, nullptr, L.wo_t, E, E, e, no_pick(), &ap));
        } else {
          dim3 mg((E / 4 + 127) / 128, M);
          LAUNCH_PDL(dev, attn_merge_kernel, mg, 128, 0, ap, s->o, E);
          TRY(mm(s->o, nullptr, nullptr, L.wo_t, L.wo_lo, E, E, e, L.ln2_g, L.ln2_b));
        }
      } else {
        TRY(mm(s->o, nullptr, nullptr, L.wo_t, L.wo_lo, E, E, e, L.ln2_g, L.ln2_b));
      }
    }
    {  // LN2 + MLP up-projection + GELU
      Epilogue e = plain_epi(s->f, F, L.bfc);
      e.act = 1;
      TRY(mm(s->x, L.ln2_g, L.ln2_b, L.wfc_t, L.wfc_lo, E, F, e));
    }
    {  // MLP down-projection + residual
      Epilogue e = plain_epi(s->x, E, L.bpr);
      e.residual = s->x;
      const bool last = l + 1 == p.n_layer;
      // the next consumer of s->x: the following block's ln_1, or ln_f when every row is a newest row
      const float *ng = last ? (n_tok == 1 ? m->lnf_g : nullptr) : m->layers[l + 1].ln1_g;
      const float *nb = last ? (n_tok == 1 ? m->lnf_b : nullptr) : m->layers[l + 1].ln1_b;
      TRY(mm(s->f, nullptr, nullptr, L.wpr_t, L.wpr_lo, F, E, e, ng, nb));
    }
  }
  // ln_f + tied de-embedding on the newest row of each sequence only (the reference normalises all rows and
  // then slices the last one, model.js:224-229 / instructions.js:849-856).
  const float *x_last = s->x + (size_t)(n_tok - 1) * E;
  size_t ld_last = (size_t)n_tok * E;
  Epilogue e = plain_epi(s->logits, p.vocab_size, nullptr);
  s->last_rows = M;
  // Six or more sequences: the de-embedding streams faster through the tensor-core GEMM's exchanged form plus the
  // arg-max kernel than through the looping GEMV with its fused pick (decode pass of GPT-2 117M 0.548 against
  // 0.573 ms at eight rows, 0.503 / 0.518 at six, 0.427 / 0.419 at four). Not in FP32 mode, whose GEMM runs on
  // the CUDA cores.
  const bool deembed_tc = dev->precision != WGPT_PRECISION_FP32 && s->n_seq >= dev->deembed_tc_min_rows;
  if (gemv_nk_fits(dev, s->n_seq, E) && !deembed_tc) {
    GreedyPick gp = no_pick();
    if (pick && s->sample_k == 0) {  // arg-max and position advance ride on the de-embedding kernel
      gp.pval = s->pick_val; gp.pidx = s->pick_idx; gp.counter = s->attn_cnt + (size_t)s->n_seq * H;
      gp.next_ids = s->next_ids; gp.out_ids = s->out_ids; gp.out_stride = s->out_cap;
      gp.pos = s->d_pos; gp.step = s->d_step; gp.n_tok = n_tok;
      gp.keys = s->pick_keys;
      if (s->n_seq == 1 && m->fused.ok && s->fx_a != nullptr) {  // the next step's first kernel finds its weights in L2
        gp.next_w = reinterpret_cast<const char *>(m->layers[0].attn_blk);
        gp.next_w_bytes = (unsigned int)((size_t)H * m->fused.cs * m->fused.blk_floats * 4);
      }
    }
    TRY(launch_gemv_nk(dev, s->n_seq, x_last, ld_last, m->lnf_g, m->lnf_b, m->wte, E, p.vocab_size, e, gp));
    if (pick && s->sample_k > 0) return pick_and_advance(s, n_tok);
    if (pick) s->len += n_tok;
    return WGPT_OK;
  }
  if (!h_ready) TRY(launch_layernorm(dev, x_last, ld_last, m->lnf_g, m->lnf_b, s->h, (size_t)E, s->n_seq, E));
  TRY(launch_gemm_nk(dev, s->h, (size_t)E, m->wte, s->n_seq, E, p.vocab_size, e));
  if (pick) TRY(pick_and_advance(s, n_tok));
  return WGPT_OK;
}

static int32_t advance(wgpt_session *s, int n_tok) {
  LAUNCH_PDL(s->m->dev, advance_kernel, 1, 32, 0, s->d_pos, s->d_step, n_tok);
  s->len += n_tok;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_session_forward(wgpt_session *s, const uint32_t *ids_host, int32_t n_tok, float *logits_host) {
  REQUIRE(s && ids_host, WGPT_ERR_ARG, "null argument");
  wgpt_device *dev = s->m->dev;
  TRY(use(dev));
  NOT_RECORDING(dev, "wgpt_session_forward");
  REQUIRE(n_tok >= 1, WGPT_ERR_SHAPE, "n_tok must be at least 1");
  REQUIRE(s->len + n_tok <= s->m->p.n_ctx, WGPT_ERR_SHAPE, "sequence length %d + %d exceeds n_ctx %d", s->len, n_tok,
          s->m->p.n_ctx);
  TRY(session_reserve(s, n_tok));
  size_t M = (size_t)s->n_seq * n_tok;
  CK(cudaMemcpyAsync(s->ids, ids_host, M * 4, cudaMemcpyHostToDevice, dev->stream));
  s->ids_dirty = true;
  TRY(forward(s, s->ids, n_tok));
  TRY(advance(s, n_tok));
  if (logits_host)
    CK(cudaMemcpyAsync(logits_host, s->logits, (size_t)s->n_seq * s->m->p.vocab_size * 4, cudaMemcpyDeviceToHost,
                       dev->stream));
  int32_t rc = check_err_word(dev, "wgpt_session_forward");  // also waits for the copies
  if (rc != WGPT_OK) {
    wgpt_session_reset(s);  // the cache now holds a row computed from a bad id
    return rc;
  }
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_model_run(wgpt_session *s, const uint32_t *idx_host, int32_t n, float *logits_host) {
  REQUIRE(s && idx_host && logits_host, WGPT_ERR_ARG, "null argument");
  REQUIRE(s->n_seq == 1, WGPT_ERR_STATE, "wgpt_model_run needs a session with one sequence");
  REQUIRE(n >= 1 && n <= s->m->p.n_ctx, WGPT_ERR_SHAPE, "window length %d outside 1..n_ctx (%d)", n, s->m->p.n_ctx);
  TRY(wgpt_session_reset(s));
  return wgpt_session_forward(s, idx_host, n, logits_host);
}

static int32_t reserve_out_ids(wgpt_session *s, int n_new) {
  if (n_new <= s->out_cap) return WGPT_OK;
  CK(cudaStreamSynchronize(s->m->dev->stream));
  drop_step_graph(s);  // out_ids and its stride are baked into the captured step
  cudaFree(s->out_ids);
  s->out_ids = nullptr;
  s->out_cap = 0;
  CK(cudaMalloc(&s->out_ids, (size_t)s->n_seq * n_new * 4));
  s->out_cap = n_new;
  return WGPT_OK;
}

// Arg-max of the newest logits of every sequence -> next input ids and output list; the same kernel then advances
// the session's position by n_tok and its step counter by one.
static int32_t launch_sample_topk(wgpt_device *dev, const float *logits, int n_rows, int V, int top_k,
                                  double temperature, const double *uniforms, uint32_t *next_ids, uint32_t *out_ids,
                                  int out_stride, int *pos, int *step, int n_tok, unsigned int *counter) {
  const int per_thread = (V + kSampleThreads - 1) / kSampleThreads;
  const size_t cap = (size_t)top_k * per_thread;
  const size_t smem = (kSampleThreads + cap) * sizeof(unsigned long long);
  REQUIRE(smem <= size_t(200) << 10, WGPT_ERR_SHAPE,
          "top_k %d with a vocabulary of %d needs %zu bytes of shared memory for the candidate list", top_k, V, smem);
  if (smem > 40 * 1024)  // the kernel's static arrays count against the 48 KB default as well
    CK(cudaFuncSetAttribute(sample_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  LAUNCH_PDL(dev, sample_topk_kernel, n_rows, kSampleThreads, smem, logits, V, top_k, temperature, uniforms, (int)cap,
             next_ids, out_ids, out_stride, pos, step, n_tok, counter);
  return WGPT_OK;
}

static int32_t pick_and_advance(wgpt_session *s, int n_tok) {
  if (s->sample_k > 0) {
    TRY(launch_sample_topk(s->m->dev, s->logits, s->n_seq, s->m->p.vocab_size, s->sample_k, s->sample_temp,
                           s->d_uniform, s->next_ids, s->out_ids, s->out_cap, s->d_pos, s->d_step, n_tok,
                           s->attn_cnt + (size_t)s->n_seq * s->m->p.n_head));
    s->len += n_tok;
    return WGPT_OK;
  }
  LAUNCH_PDL(s->m->dev, argmax_kernel, s->n_seq, 1024, 0, (const float *)s->logits, s->m->p.vocab_size, s->next_ids,
             s->out_ids, s->out_cap, s->d_pos, s->d_step, n_tok, s->attn_cnt + (size_t)s->n_seq * s->m->p.n_head);
  s->len += n_tok;
  return WGPT_OK;
}

// One decode step (newest token of every sequence -> next token), replayed as a CUDA graph: all position- and
// step-dependent values are read from device memory, so one captured step serves every position.
static int32_t decode_step(wgpt_session *s) {
  wgpt_device *dev = s->m->dev;
  // the slice count follows the context length as it is when the step is (re)captured
  if (!s->split_forced && (!dev->graphs || s->step_graph == nullptr))
    s->n_split = attn_split_for(dev, s->m->p.n_head, s->n_seq, s->len);
  if (!dev->graphs) {
    return forward(s, s->next_ids, 1, true);
  }
  if (s->step_graph == nullptr) {
    // The first step runs eagerly (it also sets every kernel's shared-memory attribute); the second is captured.
    if (!s->step_warm) {
      s->step_warm = true;
      return forward(s, s->next_ids, 1, true);
    }
    uint64_t before = dev->launches;
    int len_before = s->len;
    cudaGraph_t graph = nullptr;
    CK(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeRelaxed));
    int32_t rc = forward(s, s->next_ids, 1, true);
    cudaError_t e = cudaStreamEndCapture(dev->stream, &graph);
    s->len = len_before;  // capturing enqueued nothing
    s->step_graph_launches = dev->launches - before;
    dev->launches = before;
    if (rc != WGPT_OK) {
      if (graph) cudaGraphDestroy(graph);
      return rc;
    }
    if (e != cudaSuccess) return fail(WGPT_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&s->step_graph, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
      s->step_graph = nullptr;
      return fail(WGPT_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    }
  }
  CK(cudaGraphLaunch(s->step_graph, dev->stream));
  dev->launches += s->step_graph_launches;
  s->len += 1;
  return WGPT_OK;
}

static void drop_step_graph(wgpt_session *s) {
  if (s->step_graph) cudaGraphExecDestroy(s->step_graph);
  s->step_graph = nullptr;
  s->step_warm = false;
}

// Host copy of the prompts (needed again only if the window slides) and their device copy.
static int32_t set_prompts(wgpt_session *s, const uint32_t *prompts_host, int n_prompt) {
  wgpt_device *dev = s->m->dev;
  const int n_ctx = s->m->p.n_ctx, n_seq = s->n_seq;
  // The newest n_ctx prompt tokens form the first window (history.slice(-n_ctx), model.js:69).
  int first = n_prompt <= n_ctx ? n_prompt : n_ctx;
  TRY(session_reserve(s, first));
  TRY(wgpt_session_reset(s));
  s->prompts.assign(prompts_host, prompts_host + (size_t)n_seq * n_prompt);
  s->n_prompt = n_prompt;
  for (int q = 0; q < n_seq; q++)
    CK(cudaMemcpyAsync(s->ids + (size_t)q * first, prompts_host + (size_t)q * n_prompt + (n_prompt - first),
                       (size_t)first * 4, cudaMemcpyHostToDevice, dev->stream));
  // prompts_host may be pageable and is the caller's to reuse as soon as this returns
  CK(cudaStreamSynchronize(dev->stream));
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_session_set_prompts(wgpt_session *s, const uint32_t *prompts_host, int32_t n_prompt) {
  REQUIRE(s && prompts_host, WGPT_ERR_ARG, "null argument");
  TRY(use(s->m->dev));
  REQUIRE(n_prompt >= 1, WGPT_ERR_SHAPE, "n_prompt must be at least 1");
  NOT_RECORDING(s->m->dev, "wgpt_session_set_prompts");
  return set_prompts(s, prompts_host, n_prompt);
}

// Switches the session between the greedy pick (top_k = 0) and top-k sampling; the captured decode step holds
// the pick kernel and its arguments, so a change drops it.
static void set_pick_mode(wgpt_session *s, int top_k, double temperature) {
  if (s->sample_k != top_k || (top_k > 0 && s->sample_temp != temperature)) drop_step_graph(s);
  s->sample_k = top_k;
  s->sample_temp = temperature;
}

static int32_t generate(wgpt_session *s, int32_t n_new);

WGPT_EXPORT int32_t wgpt_session_generate(wgpt_session *s, int32_t n_new) {
  REQUIRE(s != nullptr, WGPT_ERR_ARG, "session handle is null");
  TRY(use(s->m->dev));
  NOT_RECORDING(s->m->dev, "wgpt_session_generate");
  set_pick_mode(s, 0, 1.0);
  return generate(s, n_new);
}

WGPT_EXPORT int32_t wgpt_session_generate_sample(wgpt_session *s, int32_t n_new, int32_t top_k, double temperature,
                                                 const double *uniforms_host) {
  REQUIRE(s && uniforms_host, WGPT_ERR_ARG, "null argument");
  wgpt_device *dev = s->m->dev;
  TRY(use(dev));
  NOT_RECORDING(dev, "wgpt_session_generate_sample");
  REQUIRE(n_new >= 1, WGPT_ERR_SHAPE, "n_new must be at least 1");
  REQUIRE(top_k >= 1 && top_k <= kMaxTopK && top_k <= s->m->p.vocab_size, WGPT_ERR_SHAPE,
          "top_k %d outside 1..%d", top_k, kMaxTopK < s->m->p.vocab_size ? kMaxTopK : s->m->p.vocab_size);
  REQUIRE(temperature > 0.0, WGPT_ERR_ARG, "temperature must be positive");
  size_t n_u = (size_t)n_new * s->n_seq;
  if (n_u > s->uniform_cap) {
    CK(cudaStreamSynchronize(dev->stream));
    drop_step_graph(s);  // the captured step holds the old address
    cudaFree(s->d_uniform);
    s->d_uniform = nullptr;
    s->uniform_cap = 0;
    CK(cudaMalloc(&s->d_uniform, n_u * sizeof(double)));
    s->uniform_cap = n_u;
  }
  CK(cudaMemcpyAsync(s->d_uniform, uniforms_host, n_u * sizeof(double), cudaMemcpyHostToDevice, dev->stream));
  CK(cudaStreamSynchronize(dev->stream));  // uniforms_host may be pageable and is the caller's again on return
  set_pick_mode(s, top_k, temperature);
  return generate(s, n_new);
}

static int32_t generate(wgpt_session *s, int32_t n_new) {
  wgpt_device *dev = s->m->dev;
  const int n_ctx = s->m->p.n_ctx, n_seq = s->n_seq, n_prompt = s->n_prompt;
  REQUIRE(n_prompt >= 1, WGPT_ERR_STATE, "no prompts set");
  REQUIRE(n_new >= 1, WGPT_ERR_SHAPE, "n_new must be at least 1");
  TRY(reserve_out_ids(s, n_new));
  int first = n_prompt <= n_ctx ? n_prompt : n_ctx;
  // (Re)start from the prompt window held in s->ids by set_prompts; a repeated call regenerates from the prompt.
  CK(cudaMemsetAsync(s->d_pos, 0, 2 * sizeof(int), dev->stream));
  s->len = 0;
  if (s->ids_dirty) {
    for (int q = 0; q < n_seq; q++)
      CK(cudaMemcpyAsync(s->ids + (size_t)q * first, s->prompts.data() + (size_t)q * n_prompt + (n_prompt - first),
                         (size_t)first * 4, cudaMemcpyHostToDevice, dev->stream));
    CK(cudaStreamSynchronize(dev->stream));
    s->ids_dirty = false;
  }
  TRY(forward(s, s->ids, first, true));
  const int i_start = 1;
  for (int i = i_start; i < n_new; i++) {
    if (s->len + 1 <= n_ctx) {
      TRY(decode_step(s));
      continue;
    }
    // Window slides: every position index shifts, so the cache is void; recompute the newest n_ctx tokens
    // from scratch as the reference does for every token (model.js:69-73). The ids produced so far come back
    // to the host to build the window, one round trip per token like the reference's own loop.
    std::vector<uint32_t> got((size_t)n_seq * s->out_cap);
    CK(cudaMemcpyAsync(got.data(), s->out_ids, got.size() * 4, cudaMemcpyDeviceToHost, dev->stream));
    CK(cudaStreamSynchronize(dev->stream));
    TRY(session_reserve(s, n_ctx));
    std::vector<uint32_t> window((size_t)n_seq * n_ctx);
    for (int q = 0; q < n_seq; q++) {
      std::vector<uint32_t> hist(s->prompts.begin() + (size_t)q * n_prompt, s->prompts.begin() + (size_t)(q + 1) * n_prompt);
      hist.insert(hist.end(), got.begin() + (size_t)q * s->out_cap, got.begin() + (size_t)q * s->out_cap + i);
      memcpy(window.data() + (size_t)q * n_ctx, hist.data() + (hist.size() - n_ctx), (size_t)n_ctx * 4);
    }
    CK(cudaMemsetAsync(s->d_pos, 0, sizeof(int), dev->stream));  // position only; the step counter keeps counting
    s->len = 0;
    CK(cudaMemcpyAsync(s->ids, window.data(), window.size() * 4, cudaMemcpyHostToDevice, dev->stream));
    s->ids_dirty = true;
    TRY(forward(s, s->ids, n_ctx, true));
    CK(cudaStreamSynchronize(dev->stream));  // `window` is pageable host memory about to go out of scope
  }
  s->n_generated = n_new;
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_session_get_new_ids(wgpt_session *s, int32_t n_new, uint32_t *new_ids_host) {
  REQUIRE(s && new_ids_host, WGPT_ERR_ARG, "null argument");
  wgpt_device *dev = s->m->dev;
  TRY(use(dev));
  NOT_RECORDING(dev, "wgpt_session_get_new_ids");
  REQUIRE(n_new >= 1 && n_new <= s->n_generated, WGPT_ERR_STATE, "only %d tokens have been generated", s->n_generated);
  for (int q = 0; q < s->n_seq; q++)
    CK(cudaMemcpyAsync(new_ids_host + (size_t)q * n_new, s->out_ids + (size_t)q * s->out_cap, (size_t)n_new * 4,
                       cudaMemcpyDeviceToHost, dev->stream));
  int32_t rc = check_err_word(dev, "generate");  // also waits for the copies
  if (rc != WGPT_OK) wgpt_session_reset(s);
  return rc;
}

WGPT_EXPORT int32_t wgpt_generate_greedy(wgpt_session *s, const uint32_t *prompts_host, int32_t n_prompt,
                                         int32_t n_new, uint32_t *new_ids_host) {
  REQUIRE(s && prompts_host && new_ids_host, WGPT_ERR_ARG, "null argument");
  TRY(use(s->m->dev));
  REQUIRE(n_prompt >= 1 && n_new >= 1, WGPT_ERR_SHAPE, "n_prompt and n_new must be at least 1");
  TRY(set_prompts(s, prompts_host, n_prompt));
  TRY(wgpt_session_generate(s, n_new));
  return wgpt_session_get_new_ids(s, n_new, new_ids_host);
}

WGPT_EXPORT int32_t wgpt_generate_sample(wgpt_session *s, const uint32_t *prompts_host, int32_t n_prompt,
                                         int32_t n_new, int32_t top_k, double temperature,
                                         const double *uniforms_host, uint32_t *new_ids_host) {
  REQUIRE(s && prompts_host && new_ids_host && uniforms_host, WGPT_ERR_ARG, "null argument");
  TRY(use(s->m->dev));
  REQUIRE(n_prompt >= 1 && n_new >= 1, WGPT_ERR_SHAPE, "n_prompt and n_new must be at least 1");
  TRY(set_prompts(s, prompts_host, n_prompt));
  TRY(wgpt_session_generate_sample(s, n_new, top_k, temperature, uniforms_host));
  return wgpt_session_get_new_ids(s, n_new, new_ids_host);
}

// Sequence sharding inside the library: sessions[i] holds n_seq_i sequences on its own device (weights are
// replicated, one model per device); prompts_host is [sum n_seq_i, n_prompt] in session order and new_ids_host
// [sum n_seq_i, n_new] likewise. One host thread per session runs wgpt_generate_greedy on its block; all are joined
// before the call returns. No data crosses between devices: the path has no exchange step.
WGPT_EXPORT int32_t wgpt_generate_greedy_sharded(wgpt_session **sessions, int32_t n_sessions,
                                                 const uint32_t *prompts_host, int32_t n_prompt, int32_t n_new,
                                                 uint32_t *new_ids_host) {
  REQUIRE(sessions && prompts_host && new_ids_host, WGPT_ERR_ARG, "null argument");
  REQUIRE(n_sessions >= 1, WGPT_ERR_SHAPE, "n_sessions must be at least 1");
  REQUIRE(n_prompt >= 1 && n_new >= 1, WGPT_ERR_SHAPE, "n_prompt and n_new must be at least 1");
  for (int i = 0; i < n_sessions; i++) {
    REQUIRE(sessions[i] != nullptr, WGPT_ERR_ARG, "session %d is null", i);
    for (int j = 0; j < i; j++)
      REQUIRE(sessions[j]->m->dev != sessions[i]->m->dev, WGPT_ERR_ARG,
              "sessions %d and %d share a device handle: a device handle may be driven by one thread at a time", j, i);
  }
  std::vector<int32_t> rc(n_sessions, WGPT_OK);
  std::vector<std::string> msg(n_sessions);
  std::vector<std::thread> workers;
  size_t row = 0;
  for (int i = 0; i < n_sessions; i++) {
    wgpt_session *s = sessions[i];
    const uint32_t *p = prompts_host + row * (size_t)n_prompt;
    uint32_t *o = new_ids_host + row * (size_t)n_new;
    row += (size_t)s->n_seq;
    workers.emplace_back([=, &rc, &msg] {
      rc[i] = wgpt_generate_greedy(s, p, n_prompt, n_new, o);
      if (rc[i] != WGPT_OK) msg[i] = g_err;  // g_err is per thread: carry the message back
    });
  }
  for (auto &t : workers) t.join();
  for (int i = 0; i < n_sessions; i++)
    if (rc[i] != WGPT_OK) return fail(rc[i], "session %d: %s", i, msg[i].c_str());
  return WGPT_OK;
}

// Per-operator form of the sampling step: one pick per row of logits[n_rows, V] (all device pointers).
WGPT_EXPORT int32_t wgpt_sample_topk(wgpt_device *dev, const float *logits, int32_t n_rows, int32_t V, int32_t top_k,
                                     double temperature, const double *uniforms, uint32_t *ids_out) {
  TRY(use(dev));
  REQUIRE(logits && uniforms && ids_out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(n_rows >= 1 && V >= 1, WGPT_ERR_SHAPE, "empty logits");
  REQUIRE(top_k >= 1 && top_k <= kMaxTopK && top_k <= V, WGPT_ERR_SHAPE, "top_k %d outside 1..%d", top_k,
          kMaxTopK < V ? kMaxTopK : V);
  REQUIRE(temperature > 0.0, WGPT_ERR_ARG, "temperature must be positive");
  // position, step and done counters of the kernel's advance step live in the workspace, zeroed per call
  TRY(scratch_reserve(dev, 256));
  int *ctr = static_cast<int *>(dev->scratch);
  CK(cudaMemsetAsync(ctr, 0, 16, dev->stream));
  return launch_sample_topk(dev, logits, n_rows, V, top_k, temperature, uniforms, ids_out, nullptr, 0, ctr, ctr + 1, 1,
                            reinterpret_cast<unsigned int *>(ctr + 2));
}

WGPT_EXPORT int32_t wgpt_session_tap(wgpt_session *s, float *dst, uint64_t max_floats, uint64_t *floats_written) {
  REQUIRE(s && dst, WGPT_ERR_ARG, "null argument");
  TRY(use(s->m->dev));
  REQUIRE(s->last_rows > 0, WGPT_ERR_STATE, "no forward pass has run in this session");
  uint64_t n = (uint64_t)s->last_rows * s->m->p.n_embd;
  REQUIRE(n <= max_floats, WGPT_ERR_SHAPE, "tap needs room for %llu floats", (unsigned long long)n);
  CK(cudaMemcpyAsync(dst, s->x, n * 4, cudaMemcpyDeviceToDevice, s->m->dev->stream));
  if (floats_written) *floats_written = n;
  return WGPT_OK;
}

// ------------------------------------------------------------------------------------------ matmul without allocation
// Split-K partial sums of wgpt_matmul_static live here instead of in the device workspace that wgpt_matmul
// grows with cudaMalloc. The array is part of the loaded module: every GPU that loads this library holds these
// 8 MiB until the process exits. In host code the name below is only a handle for the runtime's symbol table,
// never a device address; the address is looked up once per device with cudaGetSymbolAddress and that pointer is
// what the kernels receive.
static __device__ __align__(256) float g_static_scratch[WGPT_STATIC_SCRATCH_FLOATS];
static std::mutex g_static_mu;
static float *g_static_scratch_ptr[64];  // per device ordinal, filled on first use

static int32_t static_scratch_for(wgpt_device *dev, float **out) {
  std::lock_guard<std::mutex> lock(g_static_mu);
  REQUIRE(dev->ordinal >= 0 && dev->ordinal < 64, WGPT_ERR_UNSUPPORTED, "device ordinal %d not supported", dev->ordinal);
  if (g_static_scratch_ptr[dev->ordinal] == nullptr) {
    float *p = nullptr;
    CK(cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_scratch));  // dev is the current device
    REQUIRE(p != nullptr, WGPT_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_static_scratch_ptr[dev->ordinal] = p;
  }
  *out = g_static_scratch_ptr[dev->ordinal];
  return WGPT_OK;
}

WGPT_EXPORT int32_t wgpt_matmul_static(wgpt_device *dev, int32_t rows, int32_t cols, int32_t shared, const float *in,
                                       const float *W, const float *bias, float *out) {
  TRY(use(dev));
  REQUIRE(in && W && out, WGPT_ERR_ARG, "null pointer");
  REQUIRE(rows >= 1 && cols >= 1 && shared >= 1, WGPT_ERR_SHAPE, "empty matmul %dx%dx%d", rows, cols, shared);
  REQUIRE(cols % 8 == 0, WGPT_ERR_SHAPE, "Cols must be divisible by 16.");
  REQUIRE(shared % 4 == 0, WGPT_ERR_SHAPE, "shared dimension %d must be divisible by 4", shared);
  REQUIRE(aligned16(in) && aligned16(W) && aligned16(out) && aligned16(bias), WGPT_ERR_ALIGN,
          "buffers must be 16-byte aligned");
  REQUIRE(rows <= 8, WGPT_ERR_SHAPE, "wgpt_matmul_static handles at most 8 rows, got %d", rows);
  const size_t per_slice = (size_t)rows * cols;
  REQUIRE(per_slice <= WGPT_STATIC_SCRATCH_FLOATS, WGPT_ERR_SHAPE,
          "rows*cols = %zu exceeds the built-in scratch of %u floats; use wgpt_matmul", per_slice,
          (unsigned)WGPT_STATIC_SCRATCH_FLOATS);
  const int ksplit = kn_ksplit(dev, rows, shared, (cols + 127) / 128);
  REQUIRE((size_t)ksplit * per_slice <= WGPT_STATIC_SCRATCH_FLOATS, WGPT_ERR_SHAPE,
          "the %d K slices of a %dx%dx%d product need %zu floats, the built-in scratch holds %u; use wgpt_matmul",
          ksplit, rows, cols, shared, (size_t)ksplit * per_slice, (unsigned)WGPT_STATIC_SCRATCH_FLOATS);
  float *part = nullptr;
  TRY(static_scratch_for(dev, &part));
  // Every element of the [ksplit][rows][cols] partial block is written by the first kernel before the second
  // reads it, so nothing left over from an earlier call is ever read and nothing needs clearing.
  return gemv_kn_with_scratch(dev, rows, in, W, shared, cols, ksplit, part, plain_epi(out, cols, bias));
}

#ifdef WGPT_TRACE
// Development build only: copies the trace records (pairs of 64-bit words) to the host and clears the buffer.
WGPT_EXPORT int32_t wgpt_debug_trace_read(wgpt_device *dev, unsigned long long *out_host, uint32_t max_records,
                                          uint32_t *n_records) {
  TRY(use(dev));
  CK(cudaStreamSynchronize(dev->stream));
  unsigned int n = 0;
  CK(cudaMemcpyFromSymbol(&n, g_trace_n, sizeof n));
  n = 1u << 16;  // some kernels write their records without the counter; the reader drops empty slots
  if (n > max_records) n = max_records;
  if (n) CK(cudaMemcpyFromSymbol(out_host, g_trace_buf, (size_t)n * 16));
  unsigned int zero = 0;
  CK(cudaMemcpyToSymbol(g_trace_n, &zero, sizeof zero));
  void *tb = nullptr;
  CK(cudaGetSymbolAddress(&tb, g_trace_buf));
  CK(cudaMemset(tb, 0, sizeof(unsigned long long) << 17));
  *n_records = n;
  return WGPT_OK;
}
#endif
