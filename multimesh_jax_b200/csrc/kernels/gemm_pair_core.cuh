// bf16 GEMM main loop on CTA pairs: tcgen05.mma.cta_group::2 with a 256x256 tile per pair.
//
// Two CTAs of a cluster (two neighbouring SMs) work on one 256x256 output tile. Each CTA loads
// its own 128 rows of A and its own 128 of the tile's 256 rows of B; the pair's tensor cores read
// both B halves, so every SM fetches only half of B from shared memory and from L2 per MMA. The
// accumulator of CTA r (128 lanes x 256 fp32 columns of its TMEM) holds rows [128r, 128r+128) of
// the tile. Roles per CTA:
//
//   warp 0     : TMA producer. Loads signal the full barrier of the pair's leader (CTA rank 0);
//                the leader's producer posts the expected byte count of both CTAs.
//   warp 1     : TMEM allocation in both CTAs; in the leader one lane issues the MMAs for the
//                pair and commits to the empty / accumulator-full barriers of both CTAs.
//   warps 2..5 : epilogue of the CTA's own accumulator half through the same `TileHook` interface
//                as the single-CTA kernel (a hook sees 128-row blocks); arrivals go to the leader's
//                accumulator-empty barrier (8 arrivals per tile: 4 warps of each CTA).
//   warps 6..  : the hook's helper warps, if it has any.
//
// Loads carry no multicast qualifier. Every mbarrier wait is bounded; the cluster barriers at the
// start and the end are reached by every thread on every path, so an expired wait unwinds both
// CTAs (TMEM freed) instead of leaving one of them waiting.
#pragma once
#include <cstdio>

#include "gemm_core.cuh"
#include "host_common.h"

namespace mm {

constexpr int G2_BM = 128;          // rows of A per CTA (256 per pair)
constexpr int G2_BN = 256;          // tile columns (128 rows of B per CTA)
constexpr int G2_BNH = G2_BN / 2;
constexpr int G2_BK = 64;
constexpr int G2_STAGES = 6;
constexpr int G2_A_STAGE = G2_BM * G2_BK * 2;    // 16 KiB
constexpr int G2_B_STAGE = G2_BNH * G2_BK * 2;   // 16 KiB
constexpr int G2_STAGE_BYTES = G2_A_STAGE + G2_B_STAGE;
constexpr int G2_THREADS = 192;
constexpr int G2_SMEM_BYTES = G2_STAGES * G2_STAGE_BYTES + 256 + 1024;   // plus Hook::kStageBytes
static_assert(G2_BM == GEMM_BM && G2_BN == GEMM_BN, "hooks index 128-row blocks and 256-column blocks");

// ---- cluster-scope PTX used only here
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (an address in this CTA's shared memory) inside CTA `rank`
__device__ __forceinline__ uint32_t mapa_u32(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled load into this CTA's shared memory; completion bytes go to the mbarrier at the
// shared::cluster address `bar_cluster_addr` (the leader's barrier). No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at the same shared-memory offset in every CTA of `mask` once all MMAs
// issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}

template <bool A_MN, bool B_MN, class Hook>
__global__ void __launch_bounds__(G2_THREADS + 32 * Hook::kAuxWarps, 1)
    gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      GemmShape shape, const __grid_constant__ Hook hook, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  // the pair's descriptors name the same offsets in both CTAs: align on the shared-window offset
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* sA = smem;
  uint8_t* sB = smem + G2_STAGES * G2_A_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + G2_STAGES * G2_STAGE_BYTES);
  uint64_t* full = bars;                   // [STAGES]  used in the leader only
  uint64_t* empty = bars + G2_STAGES;      // [STAGES]  one set per CTA
  uint64_t* tfull = bars + 2 * G2_STAGES;  // [2]       one set per CTA
  uint64_t* tempty = tfull + 2;            // [2]       used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  uint8_t* epi_stage = smem + G2_STAGES * G2_STAGE_BYTES + 256;   // Hook::kStageBytes

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int K = shape.depth(), N = shape.N;
  const int M = K > 0 ? shape.rows() : 0;     // nothing to contract: no tile is visited, the output is left alone
  const int num_m = (M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int num_n = (N + G2_BN - 1) / G2_BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + G2_BK - 1) / G2_BK;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < G2_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 8);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m_blk, n_blk;
        gemm_tile_coords(tile, num_m, num_n, m_blk, n_blk);
        const int m128 = hook.map_m(m_blk * 2 + static_cast<int>(rank));   // this CTA's 128-row block
        if (!hook.before_tile_loads(m128, n_blk, err)) { ok = false; break; }
        const int a_row0 = hook.a_row(m128);
        const CUtensorMap* mapA = hook.a_map(m128, &tmA);
        const int b_row0 = n_blk * G2_BN + static_cast<int>(rank) * G2_BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, err, MM_ERR_WAIT_EMPTY)) { ok = false; break; }
          if (leader) mbar_expect_tx(&full[stage], 2 * G2_STAGE_BYTES);
          const uint32_t bar = mapa_u32(&full[stage], 0);
          uint8_t* a_dst = sA + stage * G2_A_STAGE;
          uint8_t* b_dst = sB + stage * G2_B_STAGE;
          if (!A_MN) {
            tma_load_2d_pair(a_dst, mapA, bar, kb * G2_BK, a_row0);
          } else {
#pragma unroll
            for (int i = 0; i < G2_BM / 64; ++i)
              tma_load_2d_pair(a_dst + i * (G2_BK * 128), mapA, bar, a_row0 + i * 64, kb * G2_BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(b_dst, &tmB, bar, kb * G2_BK, b_row0);
          } else {
#pragma unroll
            for (int i = 0; i < G2_BNH / 64; ++i)
              tma_load_2d_pair(b_dst + i * (G2_BK * 128), &tmB, bar, b_row0 + i * 64, kb * G2_BK);
          }
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // give copies that are still in flight time to land before the pair leaves
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * G2_BM, G2_BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, err, MM_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * G2_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, err, MM_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + stage * G2_A_STAGE);
          const uint32_t b_base = smem_u32(sB + stage * G2_B_STAGE);
#pragma unroll
          for (int k = 0; k < G2_BK / 16; ++k) {
            const uint64_t da = A_MN ? umma_desc_sw128(a_base + k * 2048, G2_BK * 128, 1024)
                                     : umma_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_desc_sw128(b_base + k * 2048, G2_BK * 128, 1024)
                                     : umma_desc_sw128(b_base + k * 32, 16, 1024);
            umma_bf16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage], 3);   // frees the stage in both CTAs
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tfull[acc], 3);       // both halves of the accumulator are complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else if (warp >= 6) {
    hook.aux(warp - 6, lane, M, K, err);
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    typename Hook::State hstate{};
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      int m_blk, n_blk;
      gemm_tile_coords(tile, num_m, num_n, m_blk, n_blk);
      const int m128 = hook.map_m(m_blk * 2 + static_cast<int>(rank));
      if (!mbar_wait(&tfull[acc], acc_phase, err, MM_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const uint32_t t_base = tmem_base + acc * G2_BN + (static_cast<uint32_t>(q * 32) << 16);
      // the hook arrives on the leader's accumulator-empty barrier once it has drained its rows
      const TmemRelease rel{mapa_u32(&tempty[acc], 0), true};
      hook.epilogue(t_base, m128, n_blk, q, lane, M, N, err, epi_stage, hstate, rel);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    hook.finish(hstate, epi_stage, q, lane, M, N, err);
  }

  // nobody leaves, and no TMEM is freed, while the partner may still signal this CTA's barriers
  // or run MMAs on its tensor memory
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// Number of CTA pairs the kernel runs for an M x N problem on the current device: one per output
// tile, but never more than can be resident at the same time (hooks whose CTAs wait for one
// another - the all-gather prologue, the peers of a fused collective - rely on every launched
// pair running). The residency limit comes from the occupancy query for clusters of two and is
// cached per device. Returns 0 on failure.
template <bool A_MN, bool B_MN, class Hook>
static int pair_kernel_pairs(int M, int N, int sm_count) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, Hook>;
  constexpr int smem_bytes = G2_SMEM_BYTES + Hook::kStageBytes;
  static_assert(smem_bytes <= 232448, "shared memory of the paired GEMM exceeds the CTA limit");
  static int resident[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 0;
  if (resident[dev] == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return 0;
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(2 * (sm_count / 2), 1, 1);
    q.blockDim = dim3(G2_THREADS + 32 * Hook::kAuxWarps, 1, 1);
    q.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2;
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    q.attrs = qa;
    q.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &q) != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      clusters = sm_count / 2;      // the query is advisory: fall back to one pair per two SMs
    }
    resident[dev] = clusters < sm_count / 2 ? clusters : sm_count / 2;
  }
  const int num_tiles = ((M + 2 * G2_BM - 1) / (2 * G2_BM)) * ((N + G2_BN - 1) / G2_BN);
  return num_tiles < resident[dev] ? num_tiles : resident[dev];
}

// Launches the pair kernel: clusters of two CTAs, at most as many as are resident together.
template <bool A_MN, bool B_MN, class Hook>
static int launch_pair_kernel(const CUtensorMap& tmA, const CUtensorMap& tmB, const Hook& hook, int M, int N, int K,
                              int sm_count, int* status, cudaStream_t stream, const int* m_dev = nullptr,
                              const int* k_dev = nullptr) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, Hook>;
  constexpr int smem_bytes = G2_SMEM_BYTES + Hook::kStageBytes;
  const int pairs = pair_kernel_pairs<A_MN, B_MN, Hook>(M, N, sm_count);
  if (pairs < 1) return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(G2_THREADS + 32 * Hook::kAuxWarps, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GemmShape shape{M, N, K, m_dev, k_dev};
  if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, shape, hook, status) != cudaSuccess) {
    fprintf(stderr, "[mm_kernels] paired GEMM launch failed: %s\n", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  return 0;
}

// Tensor maps of the pair kernel: A as in the single-CTA kernel, B with 128-row boxes.
static inline int make_pair_tmaps(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, int a_mn, int64_t lda,
                                  const void* B, int b_mn, int64_t ldb, int M, int N, int K) {
  int rc;
  if (!a_mn)
    rc = encode_tmap_2d_bf16(tmA, A, K, M, lda * 2, G2_BK, G2_BM);
  else
    rc = encode_tmap_2d_bf16(tmA, A, M, K, lda * 2, 64, G2_BK);
  if (rc) return rc;
  if (!b_mn)
    rc = encode_tmap_2d_bf16(tmB, B, K, N, ldb * 2, G2_BK, G2_BNH);
  else
    rc = encode_tmap_2d_bf16(tmB, B, N, K, ldb * 2, 64, G2_BK);
  return rc;
}

}  // namespace mm
