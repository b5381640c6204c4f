// Tensor-core GEMM for sm_100a: C[M,N] = A[M,K] . Wt[N,K]^T (+ epilogue), FP32 in and out.
//
// Persistent CTAs (one per SM) each compute a sequence of 128 x 128 tiles. TMA (cp.async.bulk.tensor, 128-byte swizzle) stages 128 x 32 FP32 tiles of
// A and of Wt into a ring in shared memory; one thread issues tcgen05.mma kind::tf32 into a 128-lane x
// 128-column FP32 accumulator in tensor memory (two of them alternate, so a tile's epilogue overlaps the next
// tile's main loop); four warps read it back with tcgen05.ld and apply the fused
// epilogue (bias / GELU / residual / KV scatter).
//
// Precision modes:
//   1 x TF32  - the tensor core reads the FP32 tiles as they are (it uses the top 19 bits of each value).
//   3 x TF32  - with hi = x truncated to TF32 (what the tensor core sees when it reads x) four extra warps write
//               lo = x - hi (exact in FP32) next to every staged tile, and three products are accumulated:
//               hi*hi + hi*lo + lo*hi. The dropped lo*lo term and the truncation of lo are ~2^-21 relative.
//
// Roles (warp index): 0 TMA producer, 1 MMA issuer (also owns the tensor-memory allocation), 2-5 epilogue
// (warp w reads accumulator lanes 32*(w%4)..+31), 6-9 hi/lo split (3 x TF32 only).
// With few output tiles the K loop is split over gridDim.z CTAs (deterministic two-stage sum).
// Every mbarrier wait is bounded; on expiry the CTA raises a shared abort flag, sets *err = 3, drains and exits.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace wgpt {

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 32;  // BK * 4 bytes = one 128-byte swizzle row
constexpr int TC_TILE_BYTES = TC_BM * TC_BK * 4;      // 16 KiB, A and B tiles alike
constexpr uint32_t TC_POLLS = 1u << 18;

// ---- tcgen05 / TMA wrappers ----
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_addr(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_addr(bar))
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Executed by one whole warp: allocates ncols (power of two >= 32) tensor-memory columns, address -> *slot (smem).
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], issued by one thread.
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread = lane, register j = column j).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
}

// 128-bit accesses in the shared state space by 32-bit address (a pointer derived from the dynamic shared-memory
// base by integer arithmetic would otherwise be accessed generically).
__device__ __forceinline__ float4 lds128(uint32_t saddr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t saddr, float4 v) {
  asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(saddr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// Shared-memory matrix descriptor for a K-major tile stored as rows of 128 bytes with the 128-byte swizzle
// (what TMA writes for a {32 floats, rows} box): start address, stride between 8-row groups = 1024 bytes,
// descriptor version 1, swizzle mode 2 (128 B). The tile base must be 1024-byte aligned; advancing by k*32
// bytes inside the swizzle row selects the k-th group of 8 TF32 values.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);       // bits 0-13: start address >> 4
  d |= (uint64_t)(1024u >> 4) << 32;              // bits 32-45: stride byte offset >> 4
  d |= (uint64_t)1 << 46;                         // bits 46-47: descriptor version
  d |= (uint64_t)2 << 61;                         // bits 61-63: 128-byte swizzle
  return d;
}
// Instruction descriptor: FP32 accumulate, TF32 A and B, both K-major, N = TC_BN, M = TC_BM.
constexpr uint32_t TC_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TC_BN >> 3) << 17) |
                              ((uint32_t)(TC_BM >> 4) << 24);


// Shared-memory plan: [stages][A tile | B tile | (X3: A lo | B lo)] (1024-byte aligned), then the barriers.
template <bool X3>
struct TcPlan {
  static constexpr int kStages = X3 ? 3 : 6;
  static constexpr int kStageBytes = (X3 ? 4 : 2) * TC_TILE_BYTES;
  static constexpr int kThreads = X3 ? 320 : 192;
  // dynamic part: alignment slack + stages + barriers and flags (512 bytes)
  static constexpr size_t kSmemBytes = 1024 + (size_t)kStages * kStageBytes + 512;
};

// Work item w of a launch: output tile (m_tile, n_tile) and K slice z, tiles of one K slice enumerated with the
// M tile fastest so that CTAs working side by side share the weight tile.
struct TcWork {
  int m0, n0, kb0, num_kb, z;
};
__device__ __forceinline__ TcWork tc_work(int w, int m_tiles, int n_tiles, int kb_per_split, int total_kb) {
  TcWork t;
  const int per_z = m_tiles * n_tiles;
  t.z = w / per_z;
  const int r = w - t.z * per_z;
  const int nt = r / m_tiles, mt = r - nt * m_tiles;
  t.m0 = mt * TC_BM;
  t.n0 = nt * TC_BN;
  t.kb0 = t.z * kb_per_split;
  t.num_kb = min(kb_per_split, total_kb - t.kb0);
  return t;
}

// Persistent: gridDim.x CTAs (one per SM) walk the work items w = blockIdx.x, blockIdx.x + gridDim.x, ...
// Two accumulators in tensor memory alternate, so the epilogue of one tile overlaps the main loop of the next.
template <bool X3>
__global__ void __launch_bounds__(TcPlan<X3>::kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_b_lo, int M, int K, int N, Epilogue epi, int *err,
               int kb_per_split, int splits, float *split_out, int static_op, int transposed, int b_lo_tma) {
  using Plan = TcPlan<X3>;
  constexpr int S = Plan::kStages;
  extern __shared__ uint8_t tc_smem_raw[];
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t *bars = reinterpret_cast<uint64_t *>(tiles + (size_t)S * Plan::kStageBytes);
  uint64_t *full = bars, *empty = bars + S, *ready = bars + 2 * S;
  uint64_t *acc_full = bars + 3 * S, *acc_empty = bars + 3 * S + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * S + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // transposition pads of the epilogue warps: a static array, so that the compiler addresses it as shared memory
  __shared__ float epi_pad[4 * 32 * 33];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (K + TC_BK - 1) / TC_BK;
  const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + TC_BN - 1) / TC_BN;
  const int n_work = m_tiles * n_tiles * splits;
  // 3xTF32 with the weight operand's low part precomputed in HBM (map_b_lo): TMA brings it into the stage's B-lo
  // slot and the split warps only treat the A tile. Requires B to be the static operand or no early loads.
  // b_lo_tma == 2: the weight operand is exact in TF32 (small integers, the int8 codes): it has no low part, so its
  // tile is not split and the a_hi x b_lo product is not issued (two MMAs per k-step instead of three).
  const bool lo_tma = X3 && b_lo_tma == 1;
  const bool b_exact = X3 && b_lo_tma == 2;
  // Exchanged operands: the second operand's live rows are the few activation rows, so the instruction is issued
  // only as wide as they need (a multiple of 16 columns) and only that part of the tile is split into hi and lo.
  const int n_mma = transposed ? min(TC_BN, (N + 15) & ~15) : TC_BN;
  const uint32_t idesc = (TC_IDESC & ~(0x3Fu << 17)) | ((uint32_t)(n_mma >> 3) << 17);
  // ... and the tensor map of that operand has a box of n_mma rows: bytes one stage receives
  const uint32_t stage_tx = (uint32_t)TC_TILE_BYTES + (uint32_t)n_mma * (TC_BK * 4) + (lo_tma ? (uint32_t)TC_TILE_BYTES : 0u);
#ifdef WGPT_TRACE
  __shared__ unsigned int tc_trace_base;  // the roles below are different threads: they share thread 0's record
  {
    TRACE_BEGIN(5);
    trace(5, 0);
    if (threadIdx.x == 0) tc_trace_base = trace_base_;
  }
#define TC_TRACE(phase) do { if (lane == 0) trace_at(tc_trace_base, 5, phase); } while (0)
#else
#define TC_TRACE(phase) ((void)0)
#endif

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; i++) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
      mbar_init(&ready[i], 128);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
    }
    *abort_flag = 0;
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * TC_BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) TC_TRACE(1);
  pdl_launch_dependents();
  // static_op names the operand that does not depend on the previous kernel (model weights, written long before):
  // 1 = B, 2 = A, 0 = neither. The producer requests that operand's tiles of its first work item's first k-blocks
  // (one per pipeline stage) before the dependency wait, so that their HBM latency overlaps the tail of the
  // previous kernel. The other operand's tiles follow after the wait.
  int pre = 0;
  if (static_op != 0 && warp == 0 && lane == 0 && (int)blockIdx.x < n_work) {
    const TcWork t = tc_work(blockIdx.x, m_tiles, n_tiles, kb_per_split, total_kb);
    pre = t.num_kb < S ? t.num_kb : S;
    for (int kb = 0; kb < pre; kb++) {
      uint8_t *st = tiles + (size_t)kb * Plan::kStageBytes;
      mbar_expect_tx(&full[kb], stage_tx);
      if (static_op == 1) {
        tma_load_2d(st + TC_TILE_BYTES, &map_b, (t.kb0 + kb) * TC_BK, t.n0, &full[kb]);
        if (lo_tma) tma_load_2d(st + 3 * TC_TILE_BYTES, &map_b_lo, (t.kb0 + kb) * TC_BK, t.n0, &full[kb]);
      } else
        tma_load_2d(st, &map_a, (t.kb0 + kb) * TC_BK, t.m0, &full[kb]);
    }
  }
  pdl_wait();  // A (activations) comes from the previous kernel
  if (warp == 0) TC_TRACE(2);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int kc = 0;  // k-blocks issued so far by this CTA: stage = kc % S, use = kc / S
      for (int w = blockIdx.x; w < n_work && !*abort_flag; w += gridDim.x) {
        const TcWork t = tc_work(w, m_tiles, n_tiles, kb_per_split, total_kb);
        for (int kb = 0; kb < t.num_kb; kb++, kc++) {
          const int s = kc % S, it = kc / S;
          uint8_t *st = tiles + (size_t)s * Plan::kStageBytes;
          if (kc < pre) {  // first use of the stage; the static operand's tile is already on the way
            if (static_op == 1)
              tma_load_2d(st, &map_a, (t.kb0 + kb) * TC_BK, t.m0, &full[s]);
            else
              tma_load_2d(st + TC_TILE_BYTES, &map_b, (t.kb0 + kb) * TC_BK, t.n0, &full[s]);
            continue;
          }
          if (*abort_flag || !mbar_wait(&empty[s], (it & 1) ^ 1, TC_POLLS)) { *abort_flag = 1; break; }
          mbar_expect_tx(&full[s], stage_tx);
          tma_load_2d(st, &map_a, (t.kb0 + kb) * TC_BK, t.m0, &full[s]);
          tma_load_2d(st + TC_TILE_BYTES, &map_b, (t.kb0 + kb) * TC_BK, t.n0, &full[s]);
          if (lo_tma) tma_load_2d(st + 3 * TC_TILE_BYTES, &map_b_lo, (t.kb0 + kb) * TC_BK, t.n0, &full[s]);
        }
        if (w == blockIdx.x) TC_TRACE(3);
      }
      TC_TRACE(14);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int kc = 0, i = 0;  // i: work items done by this CTA; accumulator = i & 1, its use count = i >> 1
      for (int w = blockIdx.x; w < n_work && !*abort_flag; w += gridDim.x, i++) {
        const TcWork t = tc_work(w, m_tiles, n_tiles, kb_per_split, total_kb);
        const int buf = i & 1, use = i >> 1;
        if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, TC_POLLS << 4)) { *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * TC_BN);
        for (int kb = 0; kb < t.num_kb; kb++, kc++) {
          const int s = kc % S, it = kc / S;
          uint64_t *go = X3 ? &ready[s] : &full[s];
          if (*abort_flag || !mbar_wait(go, it & 1, TC_POLLS)) { *abort_flag = 1; break; }
          tc_fence_after();
          if (kc == 0) TC_TRACE(4);
          const uint32_t a_hi = smem_addr(tiles + (size_t)s * Plan::kStageBytes);
          const uint32_t b_hi = a_hi + TC_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < TC_BK / 8; k++) {
            const uint64_t da = umma_desc_sw128(a_hi + k * 32), db = umma_desc_sw128(b_hi + k * 32);
            umma_tf32(tmem_acc, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            if (X3) {
              const uint64_t dal = umma_desc_sw128(a_hi + 2 * TC_TILE_BYTES + k * 32);
              const uint64_t dbl = umma_desc_sw128(b_hi + 2 * TC_TILE_BYTES + k * 32);
              if (!b_exact) umma_tf32(tmem_acc, da, dbl, idesc, 1u);
              umma_tf32(tmem_acc, dal, db, idesc, 1u);
            }
          }
          umma_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
        }
        umma_commit(&acc_full[buf]);  // this tile's accumulator is complete (also reached after an abort)
        if (i == 0) TC_TRACE(5);
      }
      TC_TRACE(13);
    }
  } else if (warp < 6) {
    // ---------------- epilogue: accumulator lanes 32*(warp%4).. ----------------
    const int quad = warp & 3;
    int i = 0;
    for (int w = blockIdx.x; w < n_work; w += gridDim.x, i++) {
      const TcWork t = tc_work(w, m_tiles, n_tiles, kb_per_split, total_kb);
      const int buf = i & 1, use = i >> 1;
      const bool ok = mbar_wait(&acc_full[buf], use & 1, TC_POLLS << 4) && !*abort_flag;
      if (!ok) { *abort_flag = 1; break; }
      tc_fence_after();
      if (i == 0 && warp == 2) TC_TRACE(6);
      Epilogue e = epi;
      if (e.kc != nullptr && e.pos != nullptr) {  // one read of the position counter instead of one per store
        e.pos_base = __ldcg(e.pos);
        e.pos = nullptr;
      }
      if (split_out != nullptr) {  // raw partial tile of K slice z; a second kernel sums the slices in order
        e.colscale = nullptr; e.bias = nullptr; e.residual = nullptr; e.kc = nullptr; e.vc = nullptr;
        e.act = 0;
        e.out = split_out + (size_t)t.z * M * N;
        e.ld = N;
      }
      const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * TC_BN);
      if (transposed) {
        // Skinny products run with the operands exchanged (kernel rows = output features, kernel columns = the
        // few activation rows): all four warps hold live lanes, only ceil(N/32) column chunks are live, and for a
        // fixed activation row the 32 lanes are 32 consecutive features, so every store is 128 contiguous bytes
        // without a transposition. Split-K: raw partials, layout [z][feature tile][activation row][128].
        // Otherwise the finished value with scale, bias and residual (no activation or cache scatter in this form).
        const int feat = t.m0 + quad * 32 + lane;
        float *tile_out = split_out != nullptr
                              ? split_out + ((size_t)t.z * m_tiles + t.m0 / TC_BM) * (size_t)N * TC_BM + quad * 32 + lane
                              : nullptr;
        const bool feat_ok = feat < M;
        const float cs = (tile_out == nullptr && epi.colscale && feat_ok) ? epi.colscale[feat] : 1.f;
        const float bs = (tile_out == nullptr && epi.bias && feat_ok) ? epi.bias[feat] : 0.f;
#pragma unroll 1
        for (int c = 0; c < TC_BN / 32; c++) {
          const int nb = c * 32;
          float v[32];
          if (nb < N) tmem_ld_32x32(tmem_acc + ((uint32_t)(quad * 32) << 16) + (uint32_t)nb, v);
          if (c == TC_BN / 32 - 1) {
            tc_fence_before();
            mbar_arrive(&acc_empty[buf]);
          }
          if (nb >= N) continue;
          if (tile_out != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; j++)
              if (nb + j < N) tile_out[(size_t)(nb + j) * TC_BM] = v[j];
          } else if (feat_ok) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              if (nb + j < N) {
                const size_t at = (size_t)(nb + j) * epi.ld + feat;
                float x = v[j] * cs + bs;
                if (epi.residual) x += __ldcg(epi.residual + at);
                epi.out[at] = x;
              }
            }
          }
        }
        continue;
      }
      // A lane of the accumulator is an output row, so the values a thread reads back lie along one row while
      // the 32 lanes of the warp are 32 different rows. Storing from there would scatter every warp-wide store
      // over 32 rows; each 32 x 32 block is transposed through a padded shared-memory tile instead, after which a
      // warp-wide float4 store covers four rows x 128 contiguous bytes (and the residual reads coalesce too).
      float *pad = epi_pad + (warp - 2) * (32 * 33);
      const int row0 = t.m0 + quad * 32;
      const bool rows_live = row0 < M;  // a tile hanging over the last row: nothing to store from these lanes
      const bool vec_ok = ((N | e.ld) & 3) == 0;
      const int sub_r = lane >> 3, col4 = (lane & 7) * 4;
#pragma unroll 1
      for (int c = 0; c < TC_BN / 32; c++) {
        float v[32];
        if (rows_live) tmem_ld_32x32(tmem_acc + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32), v);
        if (c == TC_BN / 32 - 1) {  // everything is in registers: hand the accumulator back before storing
          tc_fence_before();
          mbar_arrive(&acc_empty[buf]);
        }
        const int nb = t.n0 + c * 32;
        if (!rows_live || nb >= N) continue;
#pragma unroll
        for (int j = 0; j < 32; j++) pad[lane * 33 + j] = v[j];
        __syncwarp();
#pragma unroll 1
        for (int it = 0; it < 8; it++) {
          const int r = it * 4 + sub_r;
          const int m = row0 + r, n = nb + col4;
          const float *src = pad + r * 33 + col4;
          const float4 x = make_float4(src[0], src[1], src[2], src[3]);
          if (m < M && n < N) {
            if (vec_ok) {
              epi_store4(e, x, m, n);
            } else {
              epi_store(e, x.x, m, n);
              if (n + 1 < N) epi_store(e, x.y, m, n + 1);
              if (n + 2 < N) epi_store(e, x.z, m, n + 2);
              if (n + 3 < N) epi_store(e, x.w, m, n + 3);
            }
          }
        }
        __syncwarp();
      }
    }
    if (warp == 2) TC_TRACE(7);
    if (warp == 4) TC_TRACE(10);
    if (warp == 5) TC_TRACE(11);
    tc_fence_before();
  } else if (X3) {
    // ---------------- hi/lo split (warps 6-9) ----------------
    const int tix = threadIdx.x - 6 * 32;  // 0..127
    int kc = 0;
    // 2 KiB pieces (16 tile rows) to split: the whole first tile, and of the second tile nothing when its low part
    // came by TMA or is zero, otherwise the rows the instruction reads.
    constexpr int kTilePieces = TC_TILE_BYTES / (16 * 128);
    const int q_end = kTilePieces + ((lo_tma || b_exact) ? 0 : n_mma / 16);
    for (int w = blockIdx.x; w < n_work && !*abort_flag; w += gridDim.x) {
      const TcWork t = tc_work(w, m_tiles, n_tiles, kb_per_split, total_kb);
      for (int kb = 0; kb < t.num_kb; kb++, kc++) {
        const int s = kc % S, it = kc / S;
        if (*abort_flag || !mbar_wait(&full[s], it & 1, TC_POLLS)) { *abort_flag = 1; break; }
        // A and B tiles are adjacent (32 KiB); the lo copies sit 32 KiB further. Element order does not matter.
        const uint32_t hi = smem_addr(tiles + (size_t)s * Plan::kStageBytes) + (uint32_t)tix * 16u;
        const uint32_t lo = hi + 2 * TC_TILE_BYTES;
#pragma unroll 8
        for (int q = 0; q < q_end; q++) {
          // kind::tf32 reads the top 19 bits of each FP32 operand and ignores the rest (checked on B200: clearing
          // the low 13 bits first gives bit-identical products), so the staged tile itself serves as `hi`.
          float4 x = lds128(hi + (uint32_t)q * 2048u), l;
          l.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
          l.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
          l.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
          l.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
          sts128(lo + (uint32_t)q * 2048u, l);
        }
        fence_async_smem();  // make these generic-proxy writes visible to the tensor core's reads
        mbar_arrive(&ready[s]);
      }
    }
    if (warp == 6) TC_TRACE(12);
  }

  __syncthreads();
  if (warp == 0) TC_TRACE(8);
  if (threadIdx.x == 0 && *abort_flag) atomicExch(err, 3);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * TC_BN);
    TC_TRACE(9);
  }
}

}  // namespace wgpt
