// Persistent, warp-specialised bf16 GEMM main loop for sm_100a.
//
//   warp 0      : TMA producer (one elected lane) - fills a 4-stage ring of
//                 128B-swizzled A (128x64) and B (256x64) tiles in shared memory
//   warp 1      : allocates TMEM, issues tcgen05.mma (one lane), commits stages
//   warps 2..5  : epilogue - tcgen05.ld the 128x256 fp32 accumulator from TMEM,
//                 convert and hand 32-column row chunks to an epilogue functor
//
// Two 256-column accumulators live in TMEM (all 512 columns), so the epilogue
// of tile i overlaps the main loop of tile i+1. Operands may be K-major
// (row = M/N index, 64 K-elements contiguous) or MN-major (row = K index, 64
// M/N-elements contiguous); both use the same TMA swizzle and differ only in
// the UMMA descriptor. No TMA multicast is used anywhere.
//
// The kernel is a template over a `TileHook` that lets fused compute+collective
// variants (all-gather -> GEMM, GEMM -> reduce-scatter) wait on peer flags
// before a tile's loads and redirect the epilogue's stores to peer memory.
#pragma once
#include "ptx.cuh"

namespace mm {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BN = 256;
constexpr int GEMM_BK = 64;
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_A_STAGE = GEMM_BM * GEMM_BK * 2;  // 16 KiB
constexpr int GEMM_B_STAGE = GEMM_BN * GEMM_BK * 2;  // 32 KiB
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_GROUP_M = 16;
constexpr int GEMM_SMEM_BYTES =
    GEMM_STAGES * (GEMM_A_STAGE + GEMM_B_STAGE) + 256 /*barriers*/ + 1024 /*alignment slack*/;
// a hook that stages epilogue tiles in shared memory adds Hook::kStageBytes to this

enum GemmOut : int {
  OUT_BF16 = 0,      // C(bf16)  = acc
  OUT_F32 = 1,       // C(fp32)  = acc
  OUT_F32_ACC = 2,   // C(fp32) += acc
  OUT_BF16_ACC = 3,  // C(bf16) += acc
};

struct GemmShape {
  int M, N, K;
  // Optional run-time extents in device memory (null: the static ones). The kernel computes
  // min(M, *m_dev) row and min(K, *k_dev) contraction elements: the tensor maps and the grid are
  // made for the static upper bounds, the roles only walk the tiles that exist. This is how the
  // expert GEMMs of a mixture-of-experts layer run on however many rows were routed to the expert
  // without the host ever reading the count. An extent of zero makes the launch a no-op.
  const int* m_dev = nullptr;
  const int* k_dev = nullptr;
  __device__ __forceinline__ int rows() const {
    if (!m_dev) return M;
    const int v = *m_dev;
    return v < 0 ? 0 : (v < M ? v : M);
  }
  __device__ __forceinline__ int depth() const {
    if (!k_dev) return K;
    const int v = *k_dev;
    return v < 0 ? 0 : (v < K ? v : K);
  }
};

__device__ __forceinline__ void gemm_tile_coords(int tile, int num_m, int num_n, int& m_blk,
                                                 int& n_blk) {
  const int group_size = GEMM_GROUP_M * num_n;
  const int group_id = tile / group_size;
  const int first_m = group_id * GEMM_GROUP_M;
  const int gsz = min(num_m - first_m, GEMM_GROUP_M);
  const int in_group = tile - group_id * group_size;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

// Writes one 32-column chunk of one accumulator row to C.
template <int OUT>
__device__ __forceinline__ void gemm_store_chunk(void* C, int64_t ldc, int row, int col0, int N,
                                                 const uint32_t (&r)[32], bool vec_ok) {
  const int ncols = min(32, N - col0);
  if (OUT == OUT_BF16 || OUT == OUT_BF16_ACC) {
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(C) + static_cast<int64_t>(row) * ldc + col0;
    if (vec_ok && ncols == 32) {
      uint4* p4 = reinterpret_cast<uint4*>(p);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[i * 8 + j]);
        if (OUT == OUT_BF16_ACC) {
          uint4 old = p4[i];
          float2 a = unpack_bf16(old.x), b = unpack_bf16(old.y), c = unpack_bf16(old.z),
                 d = unpack_bf16(old.w);
          f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y;
          f[4] += c.x; f[5] += c.y; f[6] += d.x; f[7] += d.y;
        }
        uint4 o;
        o.x = pack_bf16(f[0], f[1]);
        o.y = pack_bf16(f[2], f[3]);
        o.z = pack_bf16(f[4], f[5]);
        o.w = pack_bf16(f[6], f[7]);
        p4[i] = o;
      }
    } else {
      for (int j = 0; j < ncols; ++j) {
        float v = __uint_as_float(r[j]);
        if (OUT == OUT_BF16_ACC) v += __bfloat162float(p[j]);
        p[j] = __float2bfloat16(v);
      }
    }
  } else {
    float* p = reinterpret_cast<float*>(C) + static_cast<int64_t>(row) * ldc + col0;
    if (vec_ok && ncols == 32) {
      float4* p4 = reinterpret_cast<float4*>(p);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 o = make_float4(__uint_as_float(r[i * 4]), __uint_as_float(r[i * 4 + 1]),
                               __uint_as_float(r[i * 4 + 2]), __uint_as_float(r[i * 4 + 3]));
        if (OUT == OUT_F32_ACC) {
          float4 old = p4[i];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        p4[i] = o;
      }
    } else {
      for (int j = 0; j < ncols; ++j) {
        float v = __uint_as_float(r[j]);
        if (OUT == OUT_F32_ACC) v += p[j];
        p[j] = v;
      }
    }
  }
}

// How an epilogue warp hands a drained accumulator back to the MMA lane: an arrival on the
// accumulator-empty barrier of its own CTA, or - in a CTA pair - of the pair's leader.
struct TmemRelease {
  uint32_t addr;   // shared::cta address (own CTA) or shared::cluster address (leader CTA)
  bool remote;
  __device__ __forceinline__ void arrive() const {
    if (remote)
      asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
    else
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");
  }
};

// Default hook: plain GEMM writing to local memory.
template <int OUT>
struct PlainHook {
  void* C;
  int64_t ldc;
  bool vec_ok;
  // Called by the producer lane before issuing the loads of tile (m_blk, n_blk).
  __device__ __forceinline__ bool before_tile_loads(int, int, int*) const { return true; }
  // Row of A (in the tensor map's coordinates) where tile row-block m_blk starts.
  __device__ __forceinline__ int a_row(int m_blk) const { return m_blk * GEMM_BM; }
  // Tensor map the rows of block m_blk are loaded through (hooks whose A lives in two buffers
  // carry a second map; the kernel's own one is the default).
  __device__ __forceinline__ const CUtensorMap* a_map(int, const CUtensorMap* dflt) const { return dflt; }
  // Drains one 128x256 accumulator: warp `q` owns TMEM lanes [32q, 32q+32), i.e. rows
  // m_blk*128 + 32q + lane. `t_base` already points at that lane quarter.
  static constexpr int kStageBytes = 0;  // no shared-memory staging in the epilogue
  static constexpr int kAuxWarps = 0;    // no helper warps besides producer, MMA and epilogue
  // Row block of A / C that the scheduler's m index stands for (hooks may permute the order).
  __device__ __forceinline__ int map_m(int m_blk) const { return m_blk; }
  __device__ __forceinline__ void aux(int, int, int, int, int*) const {}
  struct State {};
  __device__ __forceinline__ void finish(State&, uint8_t*, int, int, int, int, int*) const {}
  __device__ __forceinline__ void epilogue(uint32_t t_base, int m_blk, int n_blk, int q, int lane, int M, int N,
                                           int* err, uint8_t* stage, State& st, const TmemRelease& rel) const {
    (void)err; (void)stage; (void)st;
    const int row = m_blk * GEMM_BM + q * 32 + lane;
#pragma unroll 1
    for (int c = 0; c < GEMM_BN / 32; ++c) {
      const int col0 = n_blk * GEMM_BN + c * 32;
      if (col0 >= N) break;
      uint32_t r[32];
      tmem_ld_32x32(t_base + c * 32, r);
      tmem_ld_wait();
      if (row < M) gemm_store_chunk<OUT>(C, ldc, row, col0, N, r, vec_ok);
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) rel.arrive();
  }
};

template <bool A_MN, bool B_MN, class Hook>
__global__ void __launch_bounds__(GEMM_THREADS + 32 * Hook::kAuxWarps, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     GemmShape shape, const __grid_constant__ Hook hook, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + GEMM_STAGES * GEMM_A_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GEMM_STAGES * (GEMM_A_STAGE + GEMM_B_STAGE));
  uint64_t* full = bars;                    // [STAGES]
  uint64_t* empty = bars + GEMM_STAGES;     // [STAGES]
  uint64_t* tfull = bars + 2 * GEMM_STAGES; // [2]
  uint64_t* tempty = tfull + 2;             // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  uint8_t* epi_stage = smem + GEMM_STAGES * (GEMM_A_STAGE + GEMM_B_STAGE) + 256;  // Hook::kStageBytes

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int K = shape.depth(), N = shape.N;
  const int M = K > 0 ? shape.rows() : 0;     // nothing to contract: no tile is visited, the output is left alone
  const int num_m = (M + GEMM_BM - 1) / GEMM_BM;
  const int num_n = (N + GEMM_BN - 1) / GEMM_BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < GEMM_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        gemm_tile_coords(tile, num_m, num_n, m_blk, n_blk);
        m_blk = hook.map_m(m_blk);
        if (!hook.before_tile_loads(m_blk, n_blk, err)) { ok = false; break; }
        const int a_row0 = hook.a_row(m_blk);
        const CUtensorMap* mapA = hook.a_map(m_blk, &tmA);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, err, MM_ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&full[stage], GEMM_A_STAGE + GEMM_B_STAGE);
          uint8_t* a_dst = sA + stage * GEMM_A_STAGE;
          uint8_t* b_dst = sB + stage * GEMM_B_STAGE;
          if (!A_MN) {
            tma_load_2d(a_dst, mapA, &full[stage], kb * GEMM_BK, a_row0);
          } else {
#pragma unroll
            for (int i = 0; i < GEMM_BM / 64; ++i)
              tma_load_2d(a_dst + i * (GEMM_BK * 128), mapA, &full[stage], a_row0 + i * 64,
                          kb * GEMM_BK);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &tmB, &full[stage], kb * GEMM_BK, n_blk * GEMM_BN);
          } else {
#pragma unroll
            for (int i = 0; i < GEMM_BN / 64; ++i)
              tma_load_2d(b_dst + i * (GEMM_BK * 128), &tmB, &full[stage], n_blk * GEMM_BN + i * 64,
                          kb * GEMM_BK);
          }
          if (++stage == GEMM_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Give copies that are still in flight time to land before the CTA exits.
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(GEMM_BM, GEMM_BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, err, MM_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * GEMM_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, err, MM_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + stage * GEMM_A_STAGE);
          const uint32_t b_base = smem_u32(sB + stage * GEMM_B_STAGE);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t da = A_MN ? umma_desc_sw128(a_base + k * 2048, GEMM_BK * 128, 1024)
                                     : umma_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_desc_sw128(b_base + k * 2048, GEMM_BK * 128, 1024)
                                     : umma_desc_sw128(b_base + k * 32, 16, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == GEMM_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
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
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int m_blk, n_blk;
      gemm_tile_coords(tile, num_m, num_n, m_blk, n_blk);
      m_blk = hook.map_m(m_blk);
      if (!mbar_wait(&tfull[acc], acc_phase, err, MM_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const uint32_t t_base = tmem_base + acc * GEMM_BN + (static_cast<uint32_t>(q * 32) << 16);
      // the hook arrives on tempty[acc] itself as soon as it has drained the accumulator
      const TmemRelease rel{smem_u32(&tempty[acc]), false};
      hook.epilogue(t_base, m_blk, n_blk, q, lane, M, N, err, epi_stage, hstate, rel);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    hook.finish(hstate, epi_stage, q, lane, M, N, err);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace mm
