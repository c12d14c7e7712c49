// All-gather fused into a tensor-parallel GEMM (column-parallel projections whose input
// activations are sharded by rows over the ranks, i.e. sequence-parallel activations):
//
//     C[M, N] = gather_r(A_r[M/g, K]) * B[N, K]^T        A_r lives on rank r
//
// The shards interleave in chunks of `chunk_rows` rows: chunk c of the gathered matrix is chunk
// c / g of rank c % g (one chunk per rank = plain concatenation; for a [B, S, .] activation
// sharded on S a chunk is the S / g rows of one sequence).
//
// One kernel does both. Two helper warps per CTA pull the row shards - the peers' over NVLink
// with plain 16-byte loads, the own one from local memory - into a local [M, K] buffer, 128-row
// block by block, and count their arrivals per block; the TMA producer of the tcgen05 main
// loop waits (bounded) for a block's count before it loads the block's tiles from that local
// buffer. Row blocks are visited starting with this rank's own shard and then the peers' in
// ring order, so the tensor cores start on local rows while the first remote rows are still
// in flight, and the transfer of block i+1 overlaps the math of block i. TMA only ever reads
// this GPU's memory; no multicast is used.
#include <cstdlib>

#include "gemm_core.cuh"
#include "gemm_pair_core.cuh"
#include "host_common.h"

namespace mm {

constexpr int AG_MAX_RANKS = 8;

struct AllGatherHook {
  void* C;
  int64_t ldc;
  bool vec_ok;
  const uint4* a_src[AG_MAX_RANKS];  // row shard of every rank (own: local; others: peer memory), [M/g, K]
  uint4* gathered;                   // local [M, K]
  int* ready;                        // local, one counter per 128-row block, never reset
  int target;                        // value a block's counter reaches when all its pieces of this call arrived
  int nranks, me;
  int blocks_per_shard;              // 128-row blocks per rank shard
  int chunk_blocks;                  // 128-row blocks per chunk
  int num_m;

  static constexpr int kStageBytes = 0;
  static constexpr int kAuxWarps = 2;
  struct State {};
  __device__ __forceinline__ void finish(State&, uint8_t*, int, int, int, int, int*) const {}

  // scheduler index -> row block of the gathered matrix: the blocks of this rank's own shard
  // first, then the peers' in ring order
  __device__ __forceinline__ int map_m(int m_blk) const {
    if (m_blk >= num_m) return m_blk;     // the empty half of the last CTA pair
    const int hop = m_blk / blocks_per_shard, in_shard = m_blk - hop * blocks_per_shard;
    int owner = me + hop;
    if (owner >= nranks) owner -= nranks;
    const int chunk = in_shard / chunk_blocks, within = in_shard - chunk * chunk_blocks;
    return (chunk * nranks + owner) * chunk_blocks + within;
  }
  __device__ __forceinline__ int a_row(int m_blk) const { return m_blk * GEMM_BM; }

  __device__ __forceinline__ bool before_tile_loads(int m_blk, int, int* err) const {
    if (m_blk >= num_m) return true;
    unsigned long long t0 = 0, limit = 0;
    for (uint32_t i = 0;; ++i) {
      int v;
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ready + m_blk) : "memory");
      if (v >= target) {
        fence_proxy_async_all();   // the rows were written with plain stores, TMA reads them next
        return true;
      }
      if (i > 32) __nanosleep(100);
      if ((i & 255) == 255) {
        if (*reinterpret_cast<volatile int*>(err) != 0) return false;
        if (t0 == 0) {
          t0 = global_timer_ns();
          limit = status_wait_limit_ns(err);
        } else if (global_timer_ns() - t0 > limit) {
          break;
        }
      }
    }
    atomicCAS(err, 0, MM_ERR_WAIT_PEER);
    return false;
  }

  // Helper warps: copy this CTA's slice of every row block, in the order the blocks are used.
  __device__ __forceinline__ void aux(int w, int lane, int M, int K, int* err) const {
    (void)err;
    const int64_t vec_per_block = static_cast<int64_t>(GEMM_BM) * K / 8;
    const int64_t vec_per_shard = vec_per_block * blocks_per_shard;
    const int workers = gridDim.x * kAuxWarps;
    const int wid = blockIdx.x * kAuxWarps + w;
    const int64_t per = (vec_per_block + workers - 1) / workers;
    (void)vec_per_shard;
    for (int i = 0; i < num_m; ++i) {
      const int blk = map_m(i);
      const int hop = i / blocks_per_shard;
      int owner = me + hop;
      if (owner >= nranks) owner -= nranks;
      const uint4* src = a_src[owner] + static_cast<int64_t>(i - hop * blocks_per_shard) * vec_per_block;
      uint4* dst = gathered + static_cast<int64_t>(blk) * vec_per_block;
      const int64_t lo = wid * per, hi = min(vec_per_block, lo + per);
      int64_t v = lo + lane;
      for (; v + 96 < hi; v += 128) {     // four loads in flight per lane
        const uint4 x0 = __ldcg(src + v), x1 = __ldcg(src + v + 32), x2 = __ldcg(src + v + 64), x3 = __ldcg(src + v + 96);
        dst[v] = x0; dst[v + 32] = x1; dst[v + 64] = x2; dst[v + 96] = x3;
      }
      for (; v < hi; v += 32) dst[v] = __ldcg(src + v);
      fence_proxy_async_all();
      __threadfence();
      __syncwarp();
      if (lane == 0) atomicAdd(ready + blk, 1);
    }
  }

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
      if (row < M) gemm_store_chunk<OUT_BF16>(C, ldc, row, col0, N, r, vec_ok);
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) rel.arrive();
  }
};

int make_gemm_tmaps(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, int a_mn, int64_t lda, const void* B,
                    int b_mn, int64_t ldb, int M, int N, int K);

}  // namespace mm

extern "C" {

// C[M, N] (bf16, row stride ldc) = concat_r(A_r) * B[N, K]^T. a_src: `nranks` addresses of the
// [M/nranks, K] row shards (contiguous; entry `me` is local); gathered: local [M, K] buffer;
// ready: local int counters, one per 128-row block, zero before the first call and never
// reset; *target (host memory, 0 before the first call) carries the value the counters reach
// after this call and is updated here. chunk_rows (0: M / nranks) must be a multiple of 128 and
// M a multiple of nranks * chunk_rows; K a multiple of 8.
int mm_allgather_gemm_bf16(const int64_t* a_src, int nranks, int me, void* gathered, int* ready, int* target,
                           const void* B, int b_mn, int64_t ldb, void* C, int64_t ldc, int M, int N, int K,
                           int chunk_rows, cudaStream_t stream) {
  using namespace mm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (nranks < 1 || nranks > AG_MAX_RANKS || (K % 8) || (ldb % 8) || (ldc % 8)) return -2;
  if (chunk_rows <= 0) chunk_rows = M / nranks;
  if ((chunk_rows % GEMM_BM) || (M % (nranks * chunk_rows))) return -2;
  DeviceState* ds = device_state();
  if (!ds) return -1;
  // CTA pairs (256x256 tile per two SMs) from 256 rows on; MM_AG_PAIR=0 keeps the single-CTA loop
  static const bool pair_ok = [] {
    const char* e = getenv("MM_AG_PAIR");
    return !(e && e[0] == '0');
  }();
  const bool pair = pair_ok && M >= 2 * GEMM_BM;
  CUtensorMap tmA, tmB;
  int rc = pair ? make_pair_tmaps(&tmA, &tmB, gathered, 0, K, B, b_mn, ldb, M, N, K)
                : make_gemm_tmaps(&tmA, &tmB, gathered, 0, K, B, b_mn, ldb, M, N, K);
  if (rc) return rc;
  const int num_m = M / GEMM_BM;
  int grid;
  if (pair) {
    // the same number of pairs the launch below will use: every launched CTA's helper warps
    // contribute to each block's arrival count
    const int pairs = b_mn ? pair_kernel_pairs<false, true, AllGatherHook>(M, N, ds->sm_count)
                           : pair_kernel_pairs<false, false, AllGatherHook>(M, N, ds->sm_count);
    if (pairs < 1) return -1;
    grid = 2 * pairs;
  } else {
    const int num_tiles = num_m * ((N + GEMM_BN - 1) / GEMM_BN);
    grid = num_tiles < ds->sm_count ? num_tiles : ds->sm_count;
  }
  AllGatherHook hook;
  hook.C = C;
  hook.ldc = ldc;
  hook.vec_ok = (reinterpret_cast<uintptr_t>(C) % 16 == 0) && (ldc % 8 == 0);
  for (int r = 0; r < nranks; ++r) hook.a_src[r] = reinterpret_cast<const uint4*>(a_src[r]);
  hook.gathered = static_cast<uint4*>(gathered);
  hook.ready = ready;
  hook.target = *target + grid * AllGatherHook::kAuxWarps;
  *target = hook.target;
  hook.nranks = nranks;
  hook.me = me;
  hook.blocks_per_shard = num_m / nranks;
  hook.chunk_blocks = chunk_rows / GEMM_BM;
  hook.num_m = num_m;
  if (pair) {
    if (b_mn) return launch_pair_kernel<false, true>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream);
    return launch_pair_kernel<false, false>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream);
  }
  GemmShape shape{M, N, K};
  constexpr int threads = GEMM_THREADS + 32 * AllGatherHook::kAuxWarps;
  static bool configured[2][kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (b_mn) {
    auto kern = gemm_bf16_kernel<false, true, AllGatherHook>;
    if (!configured[1][dev]) {
      MM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES));
      configured[1][dev] = true;
    }
    kern<<<grid, threads, GEMM_SMEM_BYTES, stream>>>(tmA, tmB, shape, hook, ds->status);
  } else {
    auto kern = gemm_bf16_kernel<false, false, AllGatherHook>;
    if (!configured[0][dev]) {
      MM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES));
      configured[0][dev] = true;
    }
    kern<<<grid, threads, GEMM_SMEM_BYTES, stream>>>(tmA, tmB, shape, hook, ds->status);
  }
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // extern "C"
