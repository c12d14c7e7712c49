// All-gather fused into a tensor-parallel GEMM (column-parallel projections whose input
// activations are sharded by rows over the ranks, i.e. sequence-parallel activations):
//
//     C[M, N] = gather_r(A_r[M/g, K]) * B[N, K]^T        A_r lives on rank r
//
// The shards interleave in chunks of `chunk_rows` rows: chunk c of the gathered matrix is chunk
// c / g of rank c % g (one chunk per rank = plain concatenation; for a [B, S, .] activation
// sharded on S a chunk is the S / g rows of one sequence).
//
// One kernel does both. Helper warps of every CTA pull the row shards - the peers' over NVLink
// with plain 16-byte loads, the own one from local memory - into a local [M, K] buffer, 128-row
// block by block, and count their arrivals per block; the TMA producer of the tcgen05 main
// loop waits (bounded) for a remote block's count before it loads the block's tiles from that
// local buffer. The tensor cores start with this rank's own rows, which the producer loads
// straight from the shard through a second tensor map (nothing to wait for, no copy on the
// critical path), while the helper warps - six per CTA, eight 16-byte loads in flight per lane -
// bring in the peers' rows in the order the main loop will ask for them; the own rows are
// copied into the gathered buffer last, for the caller. TMA only ever reads this GPU's memory;
// no multicast is used.
#include <cstdlib>

#include "gemm_core.cuh"
#include "gemm_pair_core.cuh"
#include "host_common.h"

namespace mm {

constexpr int AG_MAX_RANKS = 8;
constexpr int AG_ROUND = 4;   // row blocks the helper warps of the grid copy at the same time

struct AllGatherHook {
  void* C;
  int64_t ldc;
  bool vec_ok;
  CUtensorMap tm_own;                // this rank's own row shard [M/g, K]: its blocks are loaded from where they are
  const uint4* a_src[AG_MAX_RANKS];  // row shard of every rank (own: local; others: peer memory), [M/g, K]
  uint4* gathered;                   // local [M, K]: the gathered matrix (an output; the peers' rows are read from it)
  int* ready;                        // local, one counter per 128-row block, never reset
  int target;                        // value a remote block's counter reaches when all its pieces of this call arrived
  int nranks, me;
  int blocks_per_shard;              // 128-row blocks per rank shard
  int chunk_blocks;                  // 128-row blocks per chunk
  int num_m;
  int workers_per_block;             // helper warps that copy (and signal) each row block
  const int* shard_ready[AG_MAX_RANKS];  // local flag per rank: reaches `epoch` once that rank's shard may be
                                         // pulled (null: the caller has synchronised the group already)
  int epoch;

  static constexpr int kStageBytes = 0;
  static constexpr int kAuxWarps = 6;
  struct State {};
  __device__ __forceinline__ void finish(State&, uint8_t*, int, int, int, int, int*) const {}

  // gathered row block -> (hop along the ring from this rank, block inside that rank's shard)
  __device__ __forceinline__ void locate(int blk, int& hop, int& in_shard) const {
    const int chunk = blk / chunk_blocks, within = blk - chunk * chunk_blocks;
    const int owner = chunk % nranks;
    hop = owner - me;
    if (hop < 0) hop += nranks;
    in_shard = (chunk / nranks) * chunk_blocks + within;
  }
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
  __device__ __forceinline__ bool own_block(int m_blk) const {
    if (m_blk >= num_m) return false;
    return (m_blk / chunk_blocks) % nranks == me;
  }
  // own rows come straight from the shard (no copy on the critical path), the peers' from `gathered`
  __device__ __forceinline__ const CUtensorMap* a_map(int m_blk, const CUtensorMap* dflt) const {
    return own_block(m_blk) ? &tm_own : dflt;
  }
  __device__ __forceinline__ int a_row(int m_blk) const {
    if (!own_block(m_blk)) return m_blk * GEMM_BM;
    int hop, in_shard;
    locate(m_blk, hop, in_shard);
    return in_shard * GEMM_BM;
  }

  __device__ __forceinline__ bool before_tile_loads(int m_blk, int, int* err) const {
    if (m_blk >= num_m || own_block(m_blk)) return true;
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

  // Helper warps copy the row blocks into `gathered` - the peers' blocks first, in the order the
  // tensor cores will want them (they are what the main loop waits for), this rank's own blocks
  // last (only the caller needs them in `gathered`). Blocks are taken AG_ROUND at a time: in a
  // round every helper warp of the grid copies one contiguous piece of one of the round's blocks
  // with up to eight 16-byte loads in flight per lane, so a round costs about one NVLink round
  // trip whatever the block size, and `workers_per_block` warps signal each block.
  __device__ __forceinline__ void aux(int w, int lane, int M, int K, int* err) const {
    (void)M;
    const int wid = blockIdx.x * kAuxWarps + w;
    if (wid >= workers_per_block * AG_ROUND) return;
    const int slot = wid % AG_ROUND, sub = wid / AG_ROUND;
    const int64_t vec_per_block = static_cast<int64_t>(GEMM_BM) * K / 8;
    const int64_t per = (vec_per_block + workers_per_block - 1) / workers_per_block;
    const int64_t lo = sub * per, hi = min(vec_per_block, lo + per);
    unsigned waited = 0;   // owners whose shard this warp has already seen published
    for (int k = slot; k < num_m; k += AG_ROUND) {
      int i = k + blocks_per_shard;                    // scheduler index: remote blocks, then own ones
      if (i >= num_m) i -= num_m;
      const int blk = map_m(i);
      const int hop = i / blocks_per_shard;
      int owner = me + hop;
      if (owner >= nranks) owner -= nranks;
      MM_CHECK_OR(blk >= 0 && blk < num_m && owner >= 0 && owner < nranks && hop < nranks, err, continue);
      if (hop != 0 && shard_ready[owner] != nullptr && !((waited >> owner) & 1u)) {
        // the owner raises this flag behind the write of its shard; waiting here instead of in a
        // barrier ahead of the kernel lets the tensor cores start on this rank's own rows meanwhile
        int ok = 1;
        if (lane == 0) ok = wait_flag_ge(shard_ready[owner], epoch, err) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return;    // status word is set; the blocks' counters never arrive, the main loop gives up too
        waited |= 1u << owner;
      }
      const uint4* src = a_src[owner] + static_cast<int64_t>(i - hop * blocks_per_shard) * vec_per_block;
      uint4* dst = gathered + static_cast<int64_t>(blk) * vec_per_block;
      for (int64_t v = lo + lane; v < hi; v += 256) {
        uint4 x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v + 32 * u < hi) x[u] = __ldcg(src + v + 32 * u);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v + 32 * u < hi) dst[v + 32 * u] = x[u];
      }
      if (hop != 0) {
        fence_proxy_async_all();
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(ready + blk, 1);
      }
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
// M a multiple of nranks * chunk_rows; K a multiple of 8. shard_ready (may be null): `nranks`
// local flag addresses; the helper warps pull rank r's shard only once *shard_ready[r] >= epoch
// (entry `me` is ignored) - null when the caller has already synchronised the group. own_rows
// (may be null): where this rank's shard is read from instead of a_src[me].
int mm_allgather_gemm_bf16(const int64_t* a_src, int nranks, int me, void* gathered, int* ready, int* target,
                           const void* B, int b_mn, int64_t ldb, void* C, int64_t ldc, int M, int N, int K,
                           int chunk_rows, const int64_t* shard_ready, int epoch, const void* own_rows,
                           cudaStream_t stream) {
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
  // this rank's own rows are read where they are: same box as the map of the gathered matrix
  const void* own = own_rows ? own_rows : reinterpret_cast<const void*>(a_src[me]);
  if (reinterpret_cast<uintptr_t>(own) % 16) return -2;
  rc = encode_tmap_2d_bf16(&hook.tm_own, own, K, M / nranks,
                           static_cast<uint64_t>(K) * 2, GEMM_BK, GEMM_BM);
  if (rc) return rc;
  hook.C = C;
  hook.ldc = ldc;
  hook.vec_ok = (reinterpret_cast<uintptr_t>(C) % 16 == 0) && (ldc % 8 == 0);
  for (int r = 0; r < nranks; ++r) {
    hook.a_src[r] = reinterpret_cast<const uint4*>(r == me ? own : reinterpret_cast<const void*>(a_src[r]));
    hook.shard_ready[r] = (shard_ready && r != me) ? reinterpret_cast<const int*>(shard_ready[r]) : nullptr;
  }
  hook.epoch = epoch;
  hook.gathered = static_cast<uint4*>(gathered);
  hook.ready = ready;
  hook.workers_per_block = grid * AllGatherHook::kAuxWarps / AG_ROUND;
  if (hook.workers_per_block < 1) return -2;
  hook.target = *target + hook.workers_per_block;
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
