// CTA-pair form of the tensor-core GEMM for large products: C[M,N] = A[M,K] . Wt[N,K]^T (+ epilogue).
//
// Two CTAs of a cluster (two SMs) share one 256 x 256 output tile through tcgen05 cta_group::2: each CTA stages
// its own 128 rows of A and its own 128 of the tile's 256 rows of Wt per k-block (32 KB, as in the one-CTA
// kernel), the pair's tensor cores read both halves of Wt, and each CTA accumulates its 128 rows x 256 columns
// in its own tensor memory. Bytes staged per MMA cycle halve against the 128 x 128 tile, which is what bounds the
// one-CTA kernel (operand fill per SM).
//
// Roles per CTA (warp index) are those of gemm_tc_kernel: 0 TMA producer, 1 MMA issuer in the leader CTA (cluster
// rank 0) and relay in the other, 2-5 epilogue, 6-9 hi/lo split (3 x TF32). Signals between the two CTAs:
//   * relay threads of the other CTA (one lane per pipeline stage) wait for their stage to be ready (tiles landed,
//     low parts written) and arrive on the leader's peer_ready barrier; one more lane reports the other CTA's free
//     accumulator buffers (peer_acc_empty);
//   * the leader's tcgen05.commit arrives on the empty / acc_full barriers of both CTAs (one commit per CTA,
//     the second through the other CTA's shared-memory address).
// Every load and every commit names exactly one destination CTA. Every wait is bounded; on expiry the CTA sets *err = 3, drains and exits.
#pragma once
#include "gemm_tc.cuh"

namespace wgpt {

constexpr int TC2_BN = 256;  // tile columns of the pair; each CTA stages 128 of the 256 Wt rows
// Instruction descriptor: FP32 accumulate, TF32 A and B, both K-major, N = 256, M = 256 (128 rows per CTA).
constexpr uint32_t TC2_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TC2_BN >> 3) << 17) |
                               ((uint32_t)(256 >> 4) << 24);

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in the CTA of the given cluster rank.
__device__ __forceinline__ uint32_t peer_smem_addr(const void *p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t *slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier at the given shared::cluster address once this thread's earlier MMAs have completed.
__device__ __forceinline__ void umma2_commit(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

// TMA tile load whose completion is counted on an mbarrier given by shared::cluster address, which may belong to
// the other CTA of the pair (cta_group::2 form, one destination); the tile itself lands in this CTA's shared memory.
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, int x, int y, uint32_t bar_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_addr(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar_addr)
      : "memory");
}

// gridDim.x = 2 x pairs, cluster (2,1,1). Pair p walks the 256 x 256 tiles p, p + pairs, ... (row tile fastest).
template <bool X3>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TcPlan<X3>::kThreads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_b_lo, int M, int K, int N, Epilogue epi, int *err,
                int b_lo_tma) {
  using Plan = TcPlan<X3>;
  constexpr int S = Plan::kStages;
  extern __shared__ uint8_t tc_smem_raw[];
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t *bars = reinterpret_cast<uint64_t *>(tiles + (size_t)S * Plan::kStageBytes);
  uint64_t *full = bars, *empty = bars + S, *ready = bars + 2 * S, *peer_ready = bars + 3 * S;
  uint64_t *acc_full = bars + 4 * S, *acc_empty = bars + 4 * S + 2, *peer_acc_empty = bars + 4 * S + 4;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 4 * S + 6);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  __shared__ float epi_pad[4 * 32 * 33];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int total_kb = (K + TC_BK - 1) / TC_BK;
  const int m_tiles = (M + 255) / 256, n_tiles = (N + TC2_BN - 1) / TC2_BN;
  const int n_work = m_tiles * n_tiles;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const bool lo_tma = X3 && b_lo_tma != 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; i++) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
      mbar_init(&ready[i], 128);
      mbar_init(&peer_ready[i], 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
      mbar_init(&peer_acc_empty[i], 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc2(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_launch_dependents();
  pdl_wait();  // A (activations) comes from the previous kernel

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's 128 rows of A and 128 of the tile's 256 rows of Wt ----------------
    if (lane == 0) {
      int kc = 0;
      for (int w = pair; w < n_work && !*abort_flag; w += pairs) {
        const int nt = w / m_tiles, mt = w - nt * m_tiles;
        const int m0 = mt * 256 + (int)rank * 128, nb0 = nt * TC2_BN + (int)rank * 128;
        for (int kb = 0; kb < total_kb; kb++, kc++) {
          const int s = kc % S, it = kc / S;
          uint8_t *st = tiles + (size_t)s * Plan::kStageBytes;
          if (*abort_flag || !mbar_wait(&empty[s], (it & 1) ^ 1, TC_POLLS)) { *abort_flag = 1; break; }
          if (!X3) {
            // plain TF32: nothing in this CTA looks at the staged tiles, so both CTAs' loads are counted on the
            // leader's barrier (which expects the bytes of both) and no relay is needed
            const uint32_t lead_full = peer_smem_addr(&full[s], 0);
            if (leader) mbar_expect_tx(&full[s], 4 * TC_TILE_BYTES);
            tma_load_2d_pair(st, &map_a, kb * TC_BK, m0, lead_full);
            tma_load_2d_pair(st + TC_TILE_BYTES, &map_b, kb * TC_BK, nb0, lead_full);
            continue;
          }
          mbar_expect_tx(&full[s], (lo_tma ? 3 : 2) * TC_TILE_BYTES);
          tma_load_2d(st, &map_a, kb * TC_BK, m0, &full[s]);
          tma_load_2d(st + TC_TILE_BYTES, &map_b, kb * TC_BK, nb0, &full[s]);
          if (lo_tma) tma_load_2d(st + 3 * TC_TILE_BYTES, &map_b_lo, kb * TC_BK, nb0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------- MMA issuer (leader CTA) ----------------
      int kc = 0, i = 0;
      for (int w = pair; w < n_work && !*abort_flag; w += pairs, i++) {
        const int buf = i & 1, use = i >> 1;
        if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, TC_POLLS << 4) ||
            !mbar_wait(&peer_acc_empty[buf], (use & 1) ^ 1, TC_POLLS << 4)) { *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * TC2_BN);
        for (int kb = 0; kb < total_kb; kb++, kc++) {
          const int s = kc % S, it = kc / S;
          uint64_t *go = X3 ? &ready[s] : &full[s];
          if (*abort_flag || !mbar_wait(go, it & 1, TC_POLLS) ||
              (X3 && !mbar_wait(&peer_ready[s], it & 1, TC_POLLS))) {
            *abort_flag = 1;
            break;
          }
          tc_fence_after();
          const uint32_t a_hi = smem_addr(tiles + (size_t)s * Plan::kStageBytes);
          const uint32_t b_hi = a_hi + TC_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < TC_BK / 8; k++) {
            const uint64_t da = umma_desc_sw128(a_hi + k * 32), db = umma_desc_sw128(b_hi + k * 32);
            umma2_tf32(tmem_acc, da, db, TC2_IDESC, (kb > 0 || k > 0) ? 1u : 0u);
            if (X3) {
              const uint64_t dal = umma_desc_sw128(a_hi + 2 * TC_TILE_BYTES + k * 32);
              const uint64_t dbl = umma_desc_sw128(b_hi + 2 * TC_TILE_BYTES + k * 32);
              umma2_tf32(tmem_acc, da, dbl, TC2_IDESC, 1u);
              umma2_tf32(tmem_acc, dal, db, TC2_IDESC, 1u);
            }
          }
          umma2_commit(smem_addr(&empty[s]));  // both CTAs may refill the stage once these MMAs have read it
          umma2_commit(peer_smem_addr(&empty[s], 1));
        }
        umma2_commit(smem_addr(&acc_full[buf]));  // (also reached after an abort)
        umma2_commit(peer_smem_addr(&acc_full[buf], 1));
      }
    } else if (X3 && !leader && lane < S) {
      // ---------------- stage relays (the other CTA): lane s tells the leader each time stage s of this CTA is
      // ready (tiles landed; in 3 x TF32 also the low parts written). A remote arrive occupies its thread for about
      // a microsecond, so one lane per stage keeps S of them in flight ----------------
      const int s = lane;
      const int my_tiles = pair < n_work ? (n_work - pair + pairs - 1) / pairs : 0;
      const int total_kc = my_tiles * total_kb;
      const uint32_t dst = peer_smem_addr(&peer_ready[s], 0);
      uint64_t *go = X3 ? &ready[s] : &full[s];
      for (int kc = s; kc < total_kc && !*abort_flag; kc += S) {
        if (!mbar_wait(go, (kc / S) & 1, TC_POLLS << 4)) { *abort_flag = 1; break; }
        mbar_arrive_cluster(dst);
      }
    } else if (!leader && lane == 8) {
      // ---------------- accumulator relay (the other CTA): a buffer of this CTA has been read back ----------------
      int i = 0;
      for (int w = pair; w < n_work && !*abort_flag; w += pairs, i++) {
        const int buf = i & 1, use = i >> 1;
        if (use == 0) continue;  // the leader's first wait on each buffer passes on a fresh barrier
        if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, TC_POLLS << 4)) { *abort_flag = 1; break; }
        mbar_arrive_cluster(peer_smem_addr(&peer_acc_empty[buf], 0));
      }
    }
  } else if (warp < 6) {
    // ---------------- epilogue: this CTA's 128 rows x 256 columns ----------------
    const int quad = warp & 3;
    float *pad = epi_pad + (warp - 2) * (32 * 33);
    const int sub_r = lane >> 3, col4 = (lane & 7) * 4;
    Epilogue e = epi;
    if (e.kc != nullptr && e.pos != nullptr) {  // one read of the position counter instead of one per store
      e.pos_base = __ldcg(e.pos);
      e.pos = nullptr;
    }
    int i = 0;
    for (int w = pair; w < n_work; w += pairs, i++) {
      const int nt = w / m_tiles, mt = w - nt * m_tiles;
      const int m0 = mt * 256 + (int)rank * 128, n0 = nt * TC2_BN;
      const int buf = i & 1, use = i >> 1;
      const bool ok = mbar_wait(&acc_full[buf], use & 1, TC_POLLS << 4) && !*abort_flag;
      if (!ok) { *abort_flag = 1; break; }
      tc_fence_after();
      const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * TC2_BN);
      const int row0 = m0 + quad * 32;
      const bool rows_live = row0 < M;
      const bool vec_ok = ((N | e.ld) & 3) == 0;
#pragma unroll 1
      for (int c = 0; c < TC2_BN / 32; c++) {
        float v[32];
        const int nb = n0 + c * 32;
        const bool live = rows_live && nb < N;
        if (live) tmem_ld_32x32(tmem_acc + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32), v);
        if (c == TC2_BN / 32 - 1) {  // everything is in registers: hand the accumulator back before storing
          tc_fence_before();
          mbar_arrive(&acc_empty[buf]);
        }
        if (!live) continue;
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
    tc_fence_before();
  } else if (X3) {
    // ---------------- hi/lo split of this CTA's staged tiles (warps 6-9) ----------------
    const int tix = threadIdx.x - 6 * 32;
    int kc = 0;
    for (int w = pair; w < n_work && !*abort_flag; w += pairs) {
      for (int kb = 0; kb < total_kb; kb++, kc++) {
        const int s = kc % S, it = kc / S;
        if (*abort_flag || !mbar_wait(&full[s], it & 1, TC_POLLS)) { *abort_flag = 1; break; }
        const uint32_t hi = smem_addr(tiles + (size_t)s * Plan::kStageBytes) + (uint32_t)tix * 16u;
        const uint32_t lo = hi + 2 * TC_TILE_BYTES;
#pragma unroll 8
        for (int q = 0; q < (2 * TC_TILE_BYTES) / (16 * 128); q++) {
          if (lo_tma && q == TC_TILE_BYTES / (16 * 128)) break;  // the Wt tile's low part came by TMA
          float4 x = lds128(hi + (uint32_t)q * 2048u), l;
          l.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
          l.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
          l.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
          l.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
          sts128(lo + (uint32_t)q * 2048u, l);
        }
        fence_async_smem();
        mbar_arrive(&ready[s]);
      }
    }
  }

  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(err, 3);
  cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

}  // namespace wgpt
