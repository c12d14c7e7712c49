// Tensor-parallel GEMM fused with its all-reduce over NVLink (row-parallel projections
// and the input-gradient of column-parallel ones).
//
// Every rank computes a partial C = A_shard * B_shard^T with the tcgen05 main loop. The
// epilogue of each 128x256 tile
//   1. drains the accumulator from TMEM, converts it to bf16 and transposes it through a
//      swizzled shared-memory staging area so that every store instruction of a warp covers
//      whole 256-byte row segments; the tile is written to the local output and *pushed*
//      into the receive buffer of every peer with plain peer stores (posted writes over
//      NVLink); the accumulator is released to the MMA warp right after the drain;
//   2. raises, per epilogue warp, the flag of its 32 rows of that tile in every peer's memory
//      (release, system scope);
//   3. reduces the tile this CTA pushed one iteration earlier: waits - bounded - for the
//      peers' flags of that tile and adds their partials (read from local memory) to the
//      local output. Deferring the reduction by one tile hides the NVLink latency and small
//      skew between ranks behind the next tile's math; the last tile is reduced after the
//      loop.
// Ranks walk the tiles in the same order. Receive buffers are double-buffered by call
// parity; flags carry the call's epoch and are never reset. No TMA load touches peer
// memory and no multicast is used.
#include <cstdlib>

#include "gemm_core.cuh"
#include "gemm_pair_core.cuh"
#include "host_common.h"

namespace mm {

constexpr int AR_MAX_PEERS = 7;
constexpr int AR_HALF_COLS = 128;                    // columns staged at a time
constexpr int AR_ROW_BYTES = AR_HALF_COLS * 2;       // 256 B of bf16 per staged row
constexpr int AR_WARP_STAGE = 32 * AR_ROW_BYTES;     // 8 KiB per epilogue warp

struct AllReduceHook {
  __nv_bfloat16* out;                      // reduced result (local), row stride ldo
  int64_t ldo;
  const __nv_bfloat16* recv_local[AR_MAX_PEERS];  // where peer p's partial lands in local memory [M][N]
  __nv_bfloat16* recv_peer[AR_MAX_PEERS];         // this rank's slot in peer p's memory [M][N]
  const int* flag_local[AR_MAX_PEERS];            // flags raised by peer p: four per tile (one per 32-row quarter)
  int* flag_peer[AR_MAX_PEERS];                   // this rank's flags in peer p's memory
  int npeers;
  int epoch;
  int num_n;

  static constexpr int kStageBytes = 4 * AR_WARP_STAGE;  // 32 KiB
  static constexpr int kAuxWarps = 0;
  __device__ __forceinline__ int map_m(int m_blk) const { return m_blk; }
  __device__ __forceinline__ void aux(int, int, int, int, int*) const {}
  struct State {
    int prev_m = -1, prev_n = -1;
  };

  __device__ __forceinline__ bool before_tile_loads(int, int, int*) const { return true; }
  __device__ __forceinline__ int a_row(int m_blk) const { return m_blk * GEMM_BM; }
  __device__ __forceinline__ const CUtensorMap* a_map(int, const CUtensorMap* dflt) const { return dflt; }

  // out[tile] += sum of the peers' partials of that tile (rows of warp q).
  __device__ __forceinline__ void reduce_tile(int m_blk, int n_blk, int q, int lane, int M, int N, int* err) const {
    const int tile = m_blk * num_n + n_blk;
    int ok = 1;
    if (lane == 0)
      for (int p = 0; p < npeers && ok; ++p) ok = wait_flag_ge(flag_local[p] + tile * 4 + q, epoch, err) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return;
    const int col = n_blk * GEMM_BN + lane * 8;   // one 512-byte tile row per warp instruction
    if (col >= N) return;
    const int row0 = m_blk * GEMM_BM + q * 32;
    // 8 rows at a time with all loads issued before the first use: the loop is bound by
    // memory latency, so the loads in flight per thread set its speed
    constexpr int R = 8;
#pragma unroll 1
    for (int rb = 0; rb < 32; rb += R) {
      if (row0 + rb >= M) break;
      float acc[R][8];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int row = min(row0 + rb + r, M - 1);
        const uint4 own = __ldcg(reinterpret_cast<const uint4*>(out + static_cast<int64_t>(row) * ldo + col));
        const float2 a = unpack_bf16(own.x), b = unpack_bf16(own.y), c = unpack_bf16(own.z), d = unpack_bf16(own.w);
        acc[r][0] = a.x; acc[r][1] = a.y; acc[r][2] = b.x; acc[r][3] = b.y;
        acc[r][4] = c.x; acc[r][5] = c.y; acc[r][6] = d.x; acc[r][7] = d.y;
      }
      for (int p = 0; p < npeers; ++p) {
        uint4 u[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int row = min(row0 + rb + r, M - 1);
          // bypass L1: the line was written by a peer
          u[r] = __ldcg(reinterpret_cast<const uint4*>(recv_local[p] + static_cast<int64_t>(row) * N + col));
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float2 ua = unpack_bf16(u[r].x), ub = unpack_bf16(u[r].y), uc = unpack_bf16(u[r].z),
                       ud = unpack_bf16(u[r].w);
          acc[r][0] += ua.x; acc[r][1] += ua.y; acc[r][2] += ub.x; acc[r][3] += ub.y;
          acc[r][4] += uc.x; acc[r][5] += uc.y; acc[r][6] += ud.x; acc[r][7] += ud.y;
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int row = row0 + rb + r;
        if (row < M) {
          uint4 o;
          o.x = pack_bf16(acc[r][0], acc[r][1]);
          o.y = pack_bf16(acc[r][2], acc[r][3]);
          o.z = pack_bf16(acc[r][4], acc[r][5]);
          o.w = pack_bf16(acc[r][6], acc[r][7]);
          *reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * ldo + col) = o;
        }
      }
    }
  }

  __device__ __forceinline__ void epilogue(uint32_t t_base, int m_blk, int n_blk, int q, int lane, int M, int N,
                                           int* err, uint8_t* stage, State& st, const TmemRelease& rel) const {
    if (m_blk * GEMM_BM >= M) {
      // A CTA pair covers 256 rows: with an odd number of 128-row blocks the second CTA of the last
      // pair has no rows. It owns no flags and no receive rows either, so it only hands the
      // accumulator back (the MMA lane counts its arrival) and reduces what it pushed before.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) rel.arrive();
      if (st.prev_m >= 0) reduce_tile(st.prev_m, st.prev_n, q, lane, M, N, err);
      st.prev_m = -1;
      return;
    }
    uint8_t* ws = stage + q * AR_WARP_STAGE;          // this warp's 32 rows x 256 B
    const int row0 = m_blk * GEMM_BM + q * 32;
    const int tile = m_blk * num_n + n_blk;
    MM_CHECK_OR(m_blk >= 0 && n_blk >= 0 && n_blk < num_n && npeers >= 1 && npeers <= AR_MAX_PEERS, err, {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) rel.arrive();
      return;
    });
#pragma unroll 1
    for (int h = 0; h < GEMM_BN / AR_HALF_COLS; ++h) {
      const int hcol0 = n_blk * GEMM_BN + h * AR_HALF_COLS;
      if (hcol0 < N) {
        // TMEM -> registers -> swizzled staging: lane = row, 16-byte unit j goes to j ^ (row & 7)
#pragma unroll 1
        for (int c = 0; c < AR_HALF_COLS / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_base + h * AR_HALF_COLS + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[i * 8 + 0]), __uint_as_float(r[i * 8 + 1]));
            v.y = pack_bf16(__uint_as_float(r[i * 8 + 2]), __uint_as_float(r[i * 8 + 3]));
            v.z = pack_bf16(__uint_as_float(r[i * 8 + 4]), __uint_as_float(r[i * 8 + 5]));
            v.w = pack_bf16(__uint_as_float(r[i * 8 + 6]), __uint_as_float(r[i * 8 + 7]));
            const int j = (c * 4 + i) ^ (lane & 7);
            *reinterpret_cast<uint4*>(ws + lane * AR_ROW_BYTES + j * 16) = v;
          }
        }
      }
      if (h == GEMM_BN / AR_HALF_COLS - 1) {
        // accumulator fully drained: hand it back to the MMA warp before touching NVLink
        tc_fence_before();
        __syncwarp();
        if (lane == 0) rel.arrive();
      } else {
        __syncwarp();
      }
      if (hcol0 < N) {
        // staging -> local output and peers: half a warp covers one 256-byte row segment
        const int unit = lane & 15;
        const int col = hcol0 + unit * 8;
        if (col < N) {
#pragma unroll 4
          for (int it = 0; it < 16; ++it) {
            const int rr = it * 2 + (lane >> 4);
            const int row = row0 + rr;
            if (row >= M) break;
            const uint4 v = *reinterpret_cast<const uint4*>(ws + rr * AR_ROW_BYTES + ((unit ^ (rr & 7)) * 16));
            *reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * ldo + col) = v;
            for (int p = 0; p < npeers; ++p)
              *reinterpret_cast<uint4*>(recv_peer[p] + static_cast<int64_t>(row) * N + col) = v;
          }
        }
      }
      __syncwarp();   // staging is reused by the next half
    }
    // each warp publishes its own 32 rows: no barrier between the epilogue warps
    __threadfence_system();
    __syncwarp();
    if (lane == 0)
      for (int p = 0; p < npeers; ++p) st_release_sys(flag_peer[p] + tile * 4 + q, epoch);
    // deferred reduction of the tile pushed one iteration ago
    if (st.prev_m >= 0) reduce_tile(st.prev_m, st.prev_n, q, lane, M, N, err);
    st.prev_m = m_blk;
    st.prev_n = n_blk;
  }

  __device__ __forceinline__ void finish(State& st, uint8_t*, int q, int lane, int M, int N, int* err) const {
    if (st.prev_m >= 0) reduce_tile(st.prev_m, st.prev_n, q, lane, M, N, err);
  }
};

// ---------------------------------------------------------------------------
// GEMM -> reduce-scatter (row-parallel projections and the input gradient of column-parallel
// ones when the activations between the tensor-parallel regions are sharded by rows).
//
// The M rows of the product are cut into chunks of `chunk_rows` rows that the g ranks own in
// turn (chunk c belongs to rank c % g: for a [B, S, .] activation sharded on S that is S / g
// rows per sequence). A rank keeps only the rows it owns: for a tile of its own rows it writes
// its partial sums to the output shard and later adds the g - 1 partials that the other ranks
// pushed; a tile of another rank's rows is pushed to that rank and never written locally. Per
// call a rank moves (g-1)/g of the product over NVLink once - half of what the all-reduce
// epilogue pushes at g = 2 - and reads / writes 1/g of it for the reduction.
struct ReduceScatterHook {
  __nv_bfloat16* out;                              // this rank's rows of the reduced product [M / g, N]
  int64_t ldo;
  const __nv_bfloat16* recv_local[AR_MAX_PEERS];   // partials of my rows from sender slot p [M / g, N]
  const int* flag_local[AR_MAX_PEERS];             // four flags per local tile from sender slot p
  __nv_bfloat16* recv_peer[AR_MAX_PEERS + 1];      // my slot in rank r's receive buffers (unused for r == me)
  int* flag_peer[AR_MAX_PEERS + 1];
  int g, me;
  int chunk_rows;                                  // a multiple of 128
  int epoch;
  int num_n;

  static constexpr int kStageBytes = 4 * AR_WARP_STAGE;
  static constexpr int kAuxWarps = 0;
  __device__ __forceinline__ int map_m(int m_blk) const { return m_blk; }
  __device__ __forceinline__ void aux(int, int, int, int, int*) const {}
  struct State {
    int prev_local_m = -1, prev_n = -1;   // last owned tile whose reduction is still due
  };
  __device__ __forceinline__ bool before_tile_loads(int, int, int*) const { return true; }
  __device__ __forceinline__ int a_row(int m_blk) const { return m_blk * GEMM_BM; }
  __device__ __forceinline__ const CUtensorMap* a_map(int, const CUtensorMap* dflt) const { return dflt; }

  // out[tile of my shard] += the other ranks' partials of that tile (rows of warp q)
  __device__ __forceinline__ void reduce_tile(int local_m, int n_blk, int q, int lane, int Ms, int N, int* err) const {
    const int tile = local_m * num_n + n_blk;
    int ok = 1;
    if (lane == 0)
      for (int p = 0; p < g - 1 && ok; ++p) ok = wait_flag_ge(flag_local[p] + tile * 4 + q, epoch, err) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return;
    const int col = n_blk * GEMM_BN + lane * 8;
    if (col >= N) return;
    const int row0 = local_m * GEMM_BM + q * 32;
    constexpr int R = 8;
#pragma unroll 1
    for (int rb = 0; rb < 32; rb += R) {
      if (row0 + rb >= Ms) break;
      float acc[R][8];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int row = min(row0 + rb + r, Ms - 1);
        const uint4 own = __ldcg(reinterpret_cast<const uint4*>(out + static_cast<int64_t>(row) * ldo + col));
        const float2 a = unpack_bf16(own.x), b = unpack_bf16(own.y), c = unpack_bf16(own.z), d = unpack_bf16(own.w);
        acc[r][0] = a.x; acc[r][1] = a.y; acc[r][2] = b.x; acc[r][3] = b.y;
        acc[r][4] = c.x; acc[r][5] = c.y; acc[r][6] = d.x; acc[r][7] = d.y;
      }
      for (int p = 0; p < g - 1; ++p) {
        uint4 u[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int row = min(row0 + rb + r, Ms - 1);
          u[r] = __ldcg(reinterpret_cast<const uint4*>(recv_local[p] + static_cast<int64_t>(row) * N + col));
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float2 ua = unpack_bf16(u[r].x), ub = unpack_bf16(u[r].y), uc = unpack_bf16(u[r].z),
                       ud = unpack_bf16(u[r].w);
          acc[r][0] += ua.x; acc[r][1] += ua.y; acc[r][2] += ub.x; acc[r][3] += ub.y;
          acc[r][4] += uc.x; acc[r][5] += uc.y; acc[r][6] += ud.x; acc[r][7] += ud.y;
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int row = row0 + rb + r;
        if (row < Ms) {
          uint4 o;
          o.x = pack_bf16(acc[r][0], acc[r][1]);
          o.y = pack_bf16(acc[r][2], acc[r][3]);
          o.z = pack_bf16(acc[r][4], acc[r][5]);
          o.w = pack_bf16(acc[r][6], acc[r][7]);
          *reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * ldo + col) = o;
        }
      }
    }
  }

  __device__ __forceinline__ void epilogue(uint32_t t_base, int m_blk, int n_blk, int q, int lane, int M, int N,
                                           int* err, uint8_t* stage, State& st, const TmemRelease& rel) const {
    const int Ms = M / g;
    if (m_blk * GEMM_BM >= M) {   // the empty half of the last CTA pair (odd number of 128-row blocks)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) rel.arrive();
      return;
    }
    // owner of these 128 rows and where they sit in the owner's shard
    const int grow0 = m_blk * GEMM_BM;
    const int chunk = grow0 / chunk_rows;
    const int owner = chunk % g;
    const int local_row0 = (chunk / g) * chunk_rows + (grow0 - chunk * chunk_rows);
    const int local_m = local_row0 / GEMM_BM;
    MM_CHECK_OR(owner >= 0 && owner < g && local_row0 >= 0 && local_row0 + GEMM_BM <= Ms && n_blk < num_n, err, {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) rel.arrive();
      return;
    });
    const bool mine = owner == me;
    __nv_bfloat16* dst = mine ? out : recv_peer[owner];
    const int64_t ld = mine ? ldo : static_cast<int64_t>(N);
    uint8_t* ws = stage + q * AR_WARP_STAGE;
    const int row0 = local_row0 + q * 32;
#pragma unroll 1
    for (int h = 0; h < GEMM_BN / AR_HALF_COLS; ++h) {
      const int hcol0 = n_blk * GEMM_BN + h * AR_HALF_COLS;
      if (hcol0 < N) {
#pragma unroll 1
        for (int c = 0; c < AR_HALF_COLS / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_base + h * AR_HALF_COLS + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[i * 8 + 0]), __uint_as_float(r[i * 8 + 1]));
            v.y = pack_bf16(__uint_as_float(r[i * 8 + 2]), __uint_as_float(r[i * 8 + 3]));
            v.z = pack_bf16(__uint_as_float(r[i * 8 + 4]), __uint_as_float(r[i * 8 + 5]));
            v.w = pack_bf16(__uint_as_float(r[i * 8 + 6]), __uint_as_float(r[i * 8 + 7]));
            const int j = (c * 4 + i) ^ (lane & 7);
            *reinterpret_cast<uint4*>(ws + lane * AR_ROW_BYTES + j * 16) = v;
          }
        }
      }
      if (h == GEMM_BN / AR_HALF_COLS - 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) rel.arrive();
      } else {
        __syncwarp();
      }
      if (hcol0 < N) {
        const int unit = lane & 15;
        const int col = hcol0 + unit * 8;
        if (col < N) {
#pragma unroll 4
          for (int it = 0; it < 16; ++it) {
            const int rr = it * 2 + (lane >> 4);
            const int row = row0 + rr;
            if (row >= Ms) break;
            const uint4 v = *reinterpret_cast<const uint4*>(ws + rr * AR_ROW_BYTES + ((unit ^ (rr & 7)) * 16));
            *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(row) * ld + col) = v;
          }
        }
      }
      __syncwarp();
    }
    if (!mine) {
      // publish my partial of these 32 rows to their owner
      __threadfence_system();
      __syncwarp();
      if (lane == 0) st_release_sys(flag_peer[owner] + (local_m * num_n + n_blk) * 4 + q, epoch);
    }
    // deferred reduction of the last tile of my own rows; a tile just written becomes the next one
    if (mine || st.prev_local_m >= 0) {
      if (st.prev_local_m >= 0) reduce_tile(st.prev_local_m, st.prev_n, q, lane, Ms, N, err);
      st.prev_local_m = mine ? local_m : -1;
      st.prev_n = n_blk;
    }
  }

  __device__ __forceinline__ void finish(State& st, uint8_t*, int q, int lane, int M, int N, int* err) const {
    if (st.prev_local_m >= 0) reduce_tile(st.prev_local_m, st.prev_n, q, lane, M / g, N, err);
  }
};

int make_gemm_tmaps(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, int a_mn, int64_t lda, const void* B,
                    int b_mn, int64_t ldb, int M, int N, int K);

constexpr int AR_SMEM_BYTES = GEMM_SMEM_BYTES + AllReduceHook::kStageBytes;
static_assert(AR_SMEM_BYTES <= 232448, "shared memory of the fused GEMM + all-reduce kernel exceeds the CTA limit");

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
    MM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AR_SMEM_BYTES));
    configured[dev] = true;
  }
  const int num_tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + GEMM_BN - 1) / GEMM_BN);
  const int grid = num_tiles < ds->sm_count ? num_tiles : ds->sm_count;
  GemmShape shape{M, N, K};
  kern<<<grid, GEMM_THREADS, AR_SMEM_BYTES, stream>>>(tmA, tmB, shape, hook, ds->status);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // namespace mm

extern "C" {

// out[M,N] = sum over ranks of (A[M,K] * B[N,K]^T) with this rank's K-shard; operand layout
// flags as in mm_gemm_bf16. recv_local / flag_local: npeers local addresses (one slot per
// peer); recv_peer / flag_peer: this rank's slot inside each peer's memory (a flag slot
// holds 4 ints per 128x256 tile). N must be a multiple of 32 and out / receive rows 16-byte
// aligned.
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
  // CTA pairs (256x256 tile per two SMs) from 256 rows on; MM_AR_PAIR=0 keeps the single-CTA loop
  static const bool pair_ok = [] {
    const char* e = getenv("MM_AR_PAIR");
    return !(e && e[0] == '0');
  }();
  if (pair_ok && M >= 2 * GEMM_BM) {
    DeviceState* ds = device_state();
    if (!ds) return -1;
    rc = make_pair_tmaps(&tmA, &tmB, A, a_mn, lda, B, b_mn, ldb, M, N, K);
    if (rc) return rc;
    if (!a_mn && !b_mn) return launch_pair_kernel<false, false>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream);
    if (!a_mn && b_mn) return launch_pair_kernel<false, true>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream);
    if (a_mn && b_mn) return launch_pair_kernel<true, true>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream);
    return launch_pair_kernel<true, false>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream);
  }
  if (!a_mn && !b_mn) return launch_ar<false, false>(tmA, tmB, hook, M, N, K, stream);
  if (!a_mn && b_mn) return launch_ar<false, true>(tmA, tmB, hook, M, N, K, stream);
  if (a_mn && b_mn) return launch_ar<true, true>(tmA, tmB, hook, M, N, K, stream);
  return launch_ar<true, false>(tmA, tmB, hook, M, N, K, stream);
}


// out[M / g, N] = this rank's rows of sum over ranks of (A[M,K] * B[N,K]^T) with this rank's K-shard.
// Rows are owned in chunks of `chunk_rows` (a multiple of 128; M a multiple of g * chunk_rows):
// chunk c belongs to rank c % g. recv_local / flag_local: g - 1 local addresses, one per sender
// slot ([M/g][N] bf16 and 4 ints per 128x256 tile of the shard). recv_peer / flag_peer: g
// addresses, entry r = this rank's sender slot inside rank r's buffers (entry `me` is ignored).
int mm_gemm_reducescatter_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* out,
                               int64_t ldo, int M, int N, int K, const int64_t* recv_local, const int64_t* recv_peer,
                               const int64_t* flag_local, const int64_t* flag_peer, int g, int me, int chunk_rows,
                               int epoch, cudaStream_t stream) {
  using namespace mm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (g < 2 || g > AR_MAX_PEERS + 1 || me < 0 || me >= g) return -2;
  if ((lda % 8) || (ldb % 8) || (N % 32) || (ldo % 8) || chunk_rows <= 0 || (chunk_rows % GEMM_BM) ||
      (M % (g * chunk_rows))) {
    fprintf(stderr, "[mm_kernels] gemm_reducescatter: N %% 32, chunk_rows %% 128 and M %% (g * chunk_rows) must be 0\n");
    return -2;
  }
  DeviceState* ds = device_state();
  if (!ds) return -1;
  ReduceScatterHook hook;
  hook.out = static_cast<__nv_bfloat16*>(out);
  hook.ldo = ldo;
  for (int p = 0; p < g - 1; ++p) {
    hook.recv_local[p] = reinterpret_cast<const __nv_bfloat16*>(recv_local[p]);
    hook.flag_local[p] = reinterpret_cast<const int*>(flag_local[p]);
  }
  for (int r = 0; r < g; ++r) {
    hook.recv_peer[r] = reinterpret_cast<__nv_bfloat16*>(recv_peer[r]);
    hook.flag_peer[r] = reinterpret_cast<int*>(flag_peer[r]);
  }
  hook.g = g;
  hook.me = me;
  hook.chunk_rows = chunk_rows;
  hook.epoch = epoch;
  hook.num_n = (N + GEMM_BN - 1) / GEMM_BN;
  CUtensorMap tmA, tmB;
  int rc = make_pair_tmaps(&tmA, &tmB, A, a_mn, lda, B, b_mn, ldb, M, N, K);
  if (rc) return rc;
  if (!a_mn && !b_mn) return launch_pair_kernel<false, false>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream);
  if (!a_mn && b_mn) return launch_pair_kernel<false, true>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream);
  if (a_mn && b_mn) return launch_pair_kernel<true, true>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream);
  return launch_pair_kernel<true, false>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream);
}

}  // extern "C"
