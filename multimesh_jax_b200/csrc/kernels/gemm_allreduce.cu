// Tensor-parallel GEMM fused with its all-reduce over NVLink (row-parallel projections
// and the input-gradient of column-parallel ones).
//
// Every rank computes a partial C = A_shard * B_shard^T with the tcgen05 main loop. The
// epilogue of each 128x256 tile
//   1. converts the accumulator to bf16 and *pushes* it into the receive buffer of every
//      peer with plain peer stores (posted writes over NVLink), then raises that tile's
//      flag in the peer's memory (release, system scope);
//   2. waits - bounded - for the same tile's flags from its peers, re-reads its own
//      accumulator from TMEM, adds the received partials from local memory and writes the
//      reduced tile.
// Ranks walk the tiles in the same order, so a peer's tile usually arrives while this
// rank's MMA warp is already working on the next tile (the second TMEM accumulator): the
// transfer overlaps the math tile by tile and no separate collective runs. Receive
// buffers are double-buffered by call parity; flags carry the call's epoch and are never
// reset. No TMA load touches peer memory and no multicast is used.
#include "gemm_core.cuh"
#include "host_common.h"

namespace mm {

constexpr int AR_MAX_PEERS = 7;

struct AllReduceHook {
  __nv_bfloat16* out;                      // reduced result (local), row stride ldo
  int64_t ldo;
  const __nv_bfloat16* recv_local[AR_MAX_PEERS];  // where peer p's partial lands in local memory [M][N]
  __nv_bfloat16* recv_peer[AR_MAX_PEERS];         // this rank's slot in peer p's memory [M][N]
  const int* flag_local[AR_MAX_PEERS];            // flags raised by peer p, one per tile
  int* flag_peer[AR_MAX_PEERS];                   // this rank's flags in peer p's memory
  int npeers;
  int epoch;
  int num_n;

  __device__ __forceinline__ bool before_tile_loads(int, int, int*) const { return true; }
  __device__ __forceinline__ int a_row(int m_blk) const { return m_blk * GEMM_BM; }

  __device__ __forceinline__ void epilogue(uint32_t t_base, int m_blk, int n_blk, int q, int lane, int M, int N,
                                           int* err) const {
    const int row = m_blk * GEMM_BM + q * 32 + lane;
    const int tile = m_blk * num_n + n_blk;
    // pass 1: push the bf16 partial to every peer
#pragma unroll 1
    for (int c = 0; c < GEMM_BN / 32; ++c) {
      const int col0 = n_blk * GEMM_BN + c * 32;
      if (col0 >= N) break;
      uint32_t r[32];
      tmem_ld_32x32(t_base + c * 32, r);
      tmem_ld_wait();
      if (row < M) {
        uint4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v[i].x = pack_bf16(__uint_as_float(r[i * 8 + 0]), __uint_as_float(r[i * 8 + 1]));
          v[i].y = pack_bf16(__uint_as_float(r[i * 8 + 2]), __uint_as_float(r[i * 8 + 3]));
          v[i].z = pack_bf16(__uint_as_float(r[i * 8 + 4]), __uint_as_float(r[i * 8 + 5]));
          v[i].w = pack_bf16(__uint_as_float(r[i * 8 + 6]), __uint_as_float(r[i * 8 + 7]));
        }
        for (int p = 0; p < npeers; ++p) {
          uint4* dst = reinterpret_cast<uint4*>(recv_peer[p] + static_cast<int64_t>(row) * N + col0);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = v[i];
        }
      }
    }
    __threadfence_system();
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
    if (q == 0 && lane == 0)
      for (int p = 0; p < npeers; ++p) st_release_sys(flag_peer[p] + tile, epoch);
    // pass 2: wait for the peers' partials of this tile, add, write the reduced tile
    int ok = 1;
    if (lane == 0)
      for (int p = 0; p < npeers && ok; ++p) ok = wait_flag_ge(flag_local[p] + tile, epoch, err) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
#pragma unroll 1
    for (int c = 0; c < GEMM_BN / 32; ++c) {
      const int col0 = n_blk * GEMM_BN + c * 32;
      if (col0 >= N) break;
      uint32_t r[32];
      tmem_ld_32x32(t_base + c * 32, r);
      tmem_ld_wait();
      if (row >= M || !ok) continue;
      float f[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
      for (int p = 0; p < npeers; ++p) {
        const uint4* src = reinterpret_cast<const uint4*>(recv_local[p] + static_cast<int64_t>(row) * N + col0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 u = __ldcg(src + i);  // bypass L1: the line was written by a peer
          float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
          f[i * 8 + 0] += a.x; f[i * 8 + 1] += a.y; f[i * 8 + 2] += b.x; f[i * 8 + 3] += b.y;
          f[i * 8 + 4] += cc.x; f[i * 8 + 5] += cc.y; f[i * 8 + 6] += d.x; f[i * 8 + 7] += d.y;
        }
      }
      uint4* o4 = reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * ldo + col0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 o;
        o.x = pack_bf16(f[i * 8 + 0], f[i * 8 + 1]);
        o.y = pack_bf16(f[i * 8 + 2], f[i * 8 + 3]);
        o.z = pack_bf16(f[i * 8 + 4], f[i * 8 + 5]);
        o.w = pack_bf16(f[i * 8 + 6], f[i * 8 + 7]);
        o4[i] = o;
      }
    }
  }
};

int make_gemm_tmaps(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, int a_mn, int64_t lda, const void* B,
                    int b_mn, int64_t ldb, int M, int N, int K);

template <bool A_MN, bool B_MN>
static int launch_ar(const CUtensorMap& tmA, const CUtensorMap& tmB, const AllReduceHook& hook, int M, int N, int K,
                     cudaStream_t stream) {
  DeviceState* ds = device_state();
  if (!ds) return -1;
  auto kern = gemm_bf16_kernel<A_MN, B_MN, AllReduceHook>;
  static bool configured[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev]) {
    MM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES));
    configured[dev] = true;
  }
  const int num_tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + GEMM_BN - 1) / GEMM_BN);
  const int grid = num_tiles < ds->sm_count ? num_tiles : ds->sm_count;
  GemmShape shape{M, N, K};
  kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, stream>>>(tmA, tmB, shape, hook, ds->status);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // namespace mm

extern "C" {

// out[M,N] = sum over ranks of (A[M,K] * B[N,K]^T) with this rank's K-shard; operand layout
// flags as in mm_gemm_bf16. recv_local / flag_local: npeers local addresses (one slot per
// peer); recv_peer / flag_peer: this rank's slot inside each peer's memory. N must be a
// multiple of 32 and out / receive rows 16-byte aligned.
int mm_gemm_allreduce_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* out,
                           int64_t ldo, int M, int N, int K, const int64_t* recv_local, const int64_t* recv_peer,
                           const int64_t* flag_local, const int64_t* flag_peer, int npeers, int epoch,
                           cudaStream_t stream) {
  using namespace mm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (npeers < 1 || npeers > AR_MAX_PEERS) return -2;
  if ((lda % 8) || (ldb % 8) || (N % 32) || (ldo % 8)) {
    fprintf(stderr, "[mm_kernels] gemm_allreduce: N must be a multiple of 32 and leading dimensions of 8\n");
    return -2;
  }
  CUtensorMap tmA, tmB;
  int rc = make_gemm_tmaps(&tmA, &tmB, A, a_mn, lda, B, b_mn, ldb, M, N, K);
  if (rc) return rc;
  AllReduceHook hook;
  hook.out = static_cast<__nv_bfloat16*>(out);
  hook.ldo = ldo;
  for (int p = 0; p < npeers; ++p) {
    hook.recv_local[p] = reinterpret_cast<const __nv_bfloat16*>(recv_local[p]);
    hook.recv_peer[p] = reinterpret_cast<__nv_bfloat16*>(recv_peer[p]);
    hook.flag_local[p] = reinterpret_cast<const int*>(flag_local[p]);
    hook.flag_peer[p] = reinterpret_cast<int*>(flag_peer[p]);
  }
  hook.npeers = npeers;
  hook.epoch = epoch;
  hook.num_n = (N + GEMM_BN - 1) / GEMM_BN;
  if (!a_mn && !b_mn) return launch_ar<false, false>(tmA, tmB, hook, M, N, K, stream);
  if (!a_mn && b_mn) return launch_ar<false, true>(tmA, tmB, hook, M, N, K, stream);
  if (a_mn && b_mn) return launch_ar<true, true>(tmA, tmB, hook, M, N, K, stream);
  return launch_ar<true, false>(tmA, tmB, hook, M, N, K, stream);
}

}  // extern "C"
