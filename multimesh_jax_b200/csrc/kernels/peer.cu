// Peer-memory plumbing and the cross-submesh reshard kernel.
//
// One process drives one GPU. Each process allocates a "symmetric arena" with
// cudaMalloc, exports it with a CUDA IPC handle and maps the arenas of the
// other processes of the node, so every kernel can address any peer's HBM
// directly over NVLink (plain ld/st, no TMA multicast anywhere).
//
// The reshard kernel is a *pull*: the destination GPU reads the rectangular
// pieces it needs straight out of the source GPUs' tiles and writes its own
// tile, so stores stay local, nothing is staged and no all-to-all runs. The
// host supplies the pieces (boxes from the reshard planner). Readiness of a
// source tile and permission to overwrite it again are exchanged through
// epoch counters in the arenas' flag areas, with bounded waits that record an
// error in the status word instead of spinning forever.
#include <cstdlib>

#include "host_common.h"
#include "ptx.cuh"

namespace mm {

constexpr int RS_MAX_DIMS = 4;
constexpr int RS_MAX_CHUNKS = 64;
constexpr int RS_MAX_WAITS = 16;

struct ReshardChunkDesc {
  const uint8_t* src;            // address of the chunk's first byte in the source tile (peer or local)
  uint8_t* dst;                  // address of the chunk's first byte in the destination tile (local)
  int64_t extent[RS_MAX_DIMS];   // extent[RS_MAX_DIMS-1] is in 16-byte vectors, the others in rows
  int64_t src_stride[RS_MAX_DIMS];  // byte strides (innermost unused: contiguous)
  int64_t dst_stride[RS_MAX_DIMS];
  int64_t vec_begin;             // first global vector index of this chunk
};

struct ReshardArgs {
  ReshardChunkDesc chunk[RS_MAX_CHUNKS];
  int num_chunks;
  int64_t total_vecs;
  // flags: wait until *wait_flag[i] >= wait_value before reading; afterwards the last CTA
  // stores done_value to every done_flag[i] (peer addresses)
  const int* wait_flag[RS_MAX_WAITS];
  int num_waits;
  int wait_value;
  int* done_flag[RS_MAX_WAITS];
  int num_done;
  int done_value;
  unsigned int* cta_counter;     // local scratch word, zero on entry, reset on exit
};

__global__ void __launch_bounds__(256)
    reshard_pull_kernel(const __grid_constant__ ReshardArgs args, int* __restrict__ err) {
  __shared__ int ok_shared;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int i = 0; i < args.num_waits && ok; ++i) ok = wait_flag_ge(args.wait_flag[i], args.wait_value, err) ? 1 : 0;
    ok_shared = ok;
  }
  __syncthreads();
  if (ok_shared) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    constexpr int UNROLL = 4;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; base < args.total_vecs;
         base += stride * UNROLL) {
      uint4 v[UNROLL];
      uint4* dptr[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int64_t idx = base + u * stride;
        dptr[u] = nullptr;
        if (idx >= args.total_vecs) continue;
        int c = 0;
        while (c + 1 < args.num_chunks && args.chunk[c + 1].vec_begin <= idx) ++c;
        const ReshardChunkDesc& ch = args.chunk[c];
        int64_t rem = idx - ch.vec_begin;
        const int64_t inner = rem % ch.extent[RS_MAX_DIMS - 1];
        rem /= ch.extent[RS_MAX_DIMS - 1];
        int64_t so = inner * 16, dof = inner * 16;
#pragma unroll
        for (int d = RS_MAX_DIMS - 2; d >= 0; --d) {
          const int64_t i = rem % ch.extent[d];
          rem /= ch.extent[d];
          so += i * ch.src_stride[d];
          dof += i * ch.dst_stride[d];
        }
        // the index must decode completely inside the chunk's box
        MM_CHECK_OR(rem == 0 && c < args.num_chunks, err, continue);
        v[u] = *reinterpret_cast<const uint4*>(ch.src + so);
        dptr[u] = reinterpret_cast<uint4*>(ch.dst + dof);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (dptr[u]) *dptr[u] = v[u];
    }
  }
  // the last CTA to finish tells the sources that their tiles have been consumed
  __syncthreads();
  if (threadIdx.x == 0 && args.cta_counter) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(args.cta_counter, 1u);
    if (prev == gridDim.x - 1) {
      if (ok_shared)
        for (int i = 0; i < args.num_done; ++i) st_release_sys(args.done_flag[i], args.done_value);
      *args.cta_counter = 0;
    }
  }
}

// Plain copy with 16-byte loads and stores, eight loads in flight per thread. With `src` a peer
// address this is the bandwidth probe that the reshard benchmark reports its fractions against:
// the rate at which this GPU can pull from one peer with nothing else in the way.
__global__ void __launch_bounds__(256) peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int64_t nvec) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  constexpr int UNROLL = 8;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; base < nvec; base += stride * UNROLL) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t i = base + u * stride;
      if (i < nvec) v[u] = src[i];
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t i = base + u * stride;
      if (i < nvec) dst[i] = v[u];
    }
  }
}

// Sets a flag in (peer or local) memory after all prior work of the stream.
__global__ void set_flag_kernel(int* flag, int value) {
  __threadfence_system();
  st_release_sys(flag, value);
}
// Waits (bounded) for a flag.
__global__ void wait_flag_kernel(const int* flag, int value, int* err) {
  wait_flag_ge(flag, value, err);
}

// Up to eight flags at once. The wait is bounded by wall-clock time (the global timer), not
// by a poll count: stage-boundary hand-offs may legitimately wait for a pipeline bubble.
struct FlagList {
  int* flag[8];
  int n;
};
__global__ void set_flags_kernel(FlagList f, int value) {
  __threadfence_system();
  if (threadIdx.x < f.n) st_release_sys(f.flag[threadIdx.x], value);
}
__global__ void wait_flags_timeout_kernel(FlagList f, int value, unsigned long long limit_ns, int* err) {
  if (threadIdx.x >= f.n) return;
  unsigned long long t0, t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    if (ld_acquire_sys(f.flag[threadIdx.x]) >= value) return;
    __nanosleep(200);
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > limit_ns || *reinterpret_cast<volatile int*>(err) != 0) {
      atomicCAS(err, 0, MM_ERR_WAIT_PEER);
      return;
    }
  }
}

// out[v] = scale * sum over sources of src[s][v], 16-byte vectors, fp32 accumulation. Sources are
// this GPU's own buffer and its peers' buffers (plain loads over NVLink): the reduce-scatter
// half of an all-reduce done as a pull, and - with one source - a plain pull copy.
struct ReducePullArgs {
  const uint4* src[8];
  uint4* out;
  int nsrc;
  int is_fp32;      // 1: fp32 elements, 0: bf16 elements
  int64_t nvec;     // vectors written (all chunks)
  int64_t chunk_vecs, src_stride_vecs;   // the sources are read in chunks of chunk_vecs, src_stride_vecs apart
  float scale;
};
__global__ void __launch_bounds__(256) reduce_pull_kernel(ReducePullArgs a) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < a.nvec; v += stride) {
    const int64_t chunk = v / a.chunk_vecs;
    const int64_t sv = chunk * a.src_stride_vecs + (v - chunk * a.chunk_vecs);
    if (a.is_fp32) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < a.nsrc; ++s) {
        const uint4 u = __ldcg(a.src[s] + sv);
        acc.x += __uint_as_float(u.x); acc.y += __uint_as_float(u.y);
        acc.z += __uint_as_float(u.z); acc.w += __uint_as_float(u.w);
      }
      uint4 o;
      o.x = __float_as_uint(acc.x * a.scale); o.y = __float_as_uint(acc.y * a.scale);
      o.z = __float_as_uint(acc.z * a.scale); o.w = __float_as_uint(acc.w * a.scale);
      a.out[v] = o;
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < a.nsrc; ++s) {
        const uint4 u = __ldcg(a.src[s] + sv);
        const float2 p0 = unpack_bf16(u.x), p1 = unpack_bf16(u.y), p2 = unpack_bf16(u.z), p3 = unpack_bf16(u.w);
        acc[0] += p0.x; acc[1] += p0.y; acc[2] += p1.x; acc[3] += p1.y;
        acc[4] += p2.x; acc[5] += p2.y; acc[6] += p3.x; acc[7] += p3.y;
      }
      uint4 o;
      o.x = pack_bf16(acc[0] * a.scale, acc[1] * a.scale);
      o.y = pack_bf16(acc[2] * a.scale, acc[3] * a.scale);
      o.z = pack_bf16(acc[4] * a.scale, acc[5] * a.scale);
      o.w = pack_bf16(acc[6] * a.scale, acc[7] * a.scale);
      a.out[v] = o;
    }
  }
}

}  // namespace mm

extern "C" {
using namespace mm;

int mm_peer_alloc(void** ptr, size_t bytes) {
  MM_CUDA_TRY(cudaMalloc(ptr, bytes));
  MM_CUDA_TRY(cudaMemset(*ptr, 0, bytes));
  return 0;
}
int mm_peer_free(void* ptr) {
  MM_CUDA_TRY(cudaFree(ptr));
  return 0;
}
// handle_out must hold 64 bytes
int mm_ipc_get_handle(void* ptr, void* handle_out) {
  cudaIpcMemHandle_t h;
  MM_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
int mm_ipc_open_handle(const void* handle_in, void** ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_in, sizeof(h));
  MM_CUDA_TRY(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
int mm_ipc_close(void* ptr) {
  MM_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return 0;
}
// Single-process multi-GPU: enable direct access from the current device to `peer`.
int mm_enable_peer_access(int peer) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return 0; }
  MM_CUDA_TRY(e);
  return 0;
}

// chunks: num_chunks records of (src ptr, dst ptr, extent[4], src_stride[4], dst_stride[4]) as int64,
// extents in elements of `elem_size` bytes with the innermost dimension contiguous on both sides.
int mm_reshard_pull(const int64_t* chunks, int num_chunks, int elem_size, const int64_t* wait_flags,
                    int num_waits, int wait_value, const int64_t* done_flags, int num_done, int done_value,
                    void* cta_counter, int max_ctas, cudaStream_t stream) {
  if (num_chunks <= 0) return 0;
  if (num_chunks > RS_MAX_CHUNKS || num_waits > RS_MAX_WAITS || num_done > RS_MAX_WAITS) return -2;
  DeviceState* ds = device_state();
  if (!ds) return -1;
  ReshardArgs args;
  memset(&args, 0, sizeof(args));
  int64_t total = 0;
  for (int c = 0; c < num_chunks; ++c) {
    const int64_t* r = chunks + c * 14;
    ReshardChunkDesc& d = args.chunk[c];
    d.src = reinterpret_cast<const uint8_t*>(r[0]);
    d.dst = reinterpret_cast<uint8_t*>(r[1]);
    const int64_t inner_bytes = r[2 + 3] * elem_size;
    if (inner_bytes % 16 || (r[0] & 15) || (r[1] & 15)) {
      fprintf(stderr, "[mm_kernels] reshard: chunk %d is not 16-byte aligned (inner %lld bytes)\n", c,
              (long long)inner_bytes);
      return -2;
    }
    int64_t vol = 1;
    for (int k = 0; k < RS_MAX_DIMS; ++k) {
      d.extent[k] = k == RS_MAX_DIMS - 1 ? inner_bytes / 16 : r[2 + k];
      d.src_stride[k] = r[6 + k] * elem_size;
      d.dst_stride[k] = r[10 + k] * elem_size;
      if (k < RS_MAX_DIMS - 1 && ((d.src_stride[k] & 15) || (d.dst_stride[k] & 15)) && d.extent[k] > 1) return -2;
      vol *= d.extent[k];
    }
    d.vec_begin = total;
    total += vol;
  }
  args.num_chunks = num_chunks;
  args.total_vecs = total;
  for (int i = 0; i < num_waits; ++i) args.wait_flag[i] = reinterpret_cast<const int*>(wait_flags[i]);
  args.num_waits = num_waits;
  args.wait_value = wait_value;
  for (int i = 0; i < num_done; ++i) args.done_flag[i] = reinterpret_cast<int*>(done_flags[i]);
  args.num_done = num_done;
  args.done_value = done_value;
  args.cta_counter = reinterpret_cast<unsigned int*>(cta_counter);
  int64_t want = (total + 256 * 4 - 1) / (256 * 4);
  int cap = max_ctas > 0 ? max_ctas : ds->sm_count * 8;
  int grid = static_cast<int>(want < cap ? want : cap);
  if (grid < 1) grid = 1;
  reshard_pull_kernel<<<grid, 256, 0, stream>>>(args, ds->status);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int mm_set_flag(void* flag, int value, cudaStream_t stream) {
  set_flag_kernel<<<1, 1, 0, stream>>>(reinterpret_cast<int*>(flag), value);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int mm_wait_flag(const void* flag, int value, cudaStream_t stream) {
  DeviceState* ds = device_state();
  if (!ds) return -1;
  wait_flag_kernel<<<1, 1, 0, stream>>>(reinterpret_cast<const int*>(flag), value, ds->status);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// out = scale * sum of `nsrc` buffers of `nbytes` bytes each (16-byte aligned, a multiple of 16
// bytes); sources may be peer addresses. elem_size 4 = fp32, 2 = bf16.
int mm_reduce_pull_chunked(const int64_t* srcs, int nsrc, void* out, int64_t chunk_bytes, int64_t nchunks,
                           int64_t src_stride_bytes, int elem_size, float scale, cudaStream_t stream);

// dst[0, bytes) = src[0, bytes): both 16-byte aligned, bytes a multiple of 16; src may be a peer address.
int mm_peer_copy(void* dst, const void* src, int64_t bytes, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  if ((bytes % 16) || (reinterpret_cast<uintptr_t>(dst) % 16) || (reinterpret_cast<uintptr_t>(src) % 16)) return -2;
  DeviceState* ds = device_state();
  if (!ds) return -1;
  const int64_t nvec = bytes / 16;
  int64_t want = (nvec + 256 * 8 - 1) / (256 * 8);
  const int cap = ds->sm_count * 8;
  const int grid = static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
  peer_copy_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), nvec);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int mm_reduce_pull(const int64_t* srcs, int nsrc, void* out, int64_t nbytes, int elem_size, float scale,
                   cudaStream_t stream) {
  return mm_reduce_pull_chunked(srcs, nsrc, out, nbytes, 1, nbytes, elem_size, scale, stream);
}

// Chunked form: `nchunks` pieces of `chunk_bytes` bytes, `src_stride_bytes` apart in every source,
// written back to back to `out` (the reduce-scatter of an inner dimension: every outer index
// contributes one piece of this rank's share).
int mm_reduce_pull_chunked(const int64_t* srcs, int nsrc, void* out, int64_t chunk_bytes, int64_t nchunks,
                           int64_t src_stride_bytes, int elem_size, float scale, cudaStream_t stream) {
  const int64_t nbytes = chunk_bytes * nchunks;
  if (nbytes <= 0) return 0;
  if (nsrc < 1 || nsrc > 8 || (chunk_bytes & 15) || (src_stride_bytes & 15) || (elem_size != 4 && elem_size != 2))
    return -2;
  DeviceState* ds = device_state();
  if (!ds) return -1;
  ReducePullArgs a;
  for (int i = 0; i < nsrc; ++i) {
    if (srcs[i] & 15) return -2;
    a.src[i] = reinterpret_cast<const uint4*>(srcs[i]);
  }
  if (reinterpret_cast<uintptr_t>(out) & 15) return -2;
  a.out = reinterpret_cast<uint4*>(out);
  a.nsrc = nsrc;
  a.is_fp32 = elem_size == 4;
  a.nvec = nbytes / 16;
  a.chunk_vecs = chunk_bytes / 16;
  a.src_stride_vecs = src_stride_bytes / 16;
  a.scale = scale;
  int64_t want = (a.nvec + 256 * 4 - 1) / (256 * 4);
  // The kernel is bound by NVLink latency x bandwidth, not by SM count: two CTAs per SM keep
  // about 4.8 MB of loads in flight (three times what 770 GB/s x 2 us needs) and leave the
  // other thread slots to the kernels it overlaps with (the optimizer pieces that run on the
  // compute stream while later gradients are still being reduced). MM_REDUCE_PULL_CTAS_PER_SM
  // changes the share (1..8).
  static const int per_sm = [] {
    const char* v = std::getenv("MM_REDUCE_PULL_CTAS_PER_SM");
    const int n = v && *v ? std::atoi(v) : 2;
    return n < 1 ? 1 : (n > 8 ? 8 : n);
  }();
  const int cap = ds->sm_count * per_sm;
  const int grid = static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
  reduce_pull_kernel<<<grid, 256, 0, stream>>>(a);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// Raises up to eight flags (local or peer addresses) to `value` after all earlier work of
// the stream.
int mm_set_flags(const int64_t* flags, int n, int value, cudaStream_t stream) {
  if (n < 1) return 0;
  if (n > 8) return -2;
  FlagList f;
  f.n = n;
  for (int i = 0; i < n; ++i) f.flag[i] = reinterpret_cast<int*>(flags[i]);
  set_flags_kernel<<<1, 32, 0, stream>>>(f, value);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
// Holds the stream until up to eight local flags are >= `value`, for at most `limit_ms`
// milliseconds; on expiry the status word gets MM_ERR_WAIT_PEER and the stream continues.
int mm_wait_flags(const int64_t* flags, int n, int value, int limit_ms, cudaStream_t stream) {
  if (n < 1) return 0;
  if (n > 8) return -2;
  DeviceState* ds = device_state();
  if (!ds) return -1;
  FlagList f;
  f.n = n;
  for (int i = 0; i < n; ++i) f.flag[i] = reinterpret_cast<int*>(flags[i]);
  wait_flags_timeout_kernel<<<1, 32, 0, stream>>>(f, value, static_cast<unsigned long long>(limit_ms) * 1000000ull,
                                                  ds->status);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // extern "C"
