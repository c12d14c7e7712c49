// Expert-parallel mixture-of-experts data movement for sm_100a, fused with the router.
//
//   moe_route_dispatch_kernel : one warp per token. Reads the token row once, computes the router
//       logits against all experts, picks the top-k, soft-maxes the chosen logits into gates and
//       - the "dispatch all-to-all" - writes the row straight into the receive buffer of the GPU
//       that owns each chosen expert (plain peer stores over NVLink, 16-byte vectors). The slot
//       inside the expert's region comes from a counter in the owner's memory (system-scope
//       atomic add over NVLink). Optionally a second row per token (the output gradient, scaled by
//       the gate) goes to a second buffer at the same slot (backward pass).
//   moe_combine_kernel : one warp per token. The "combine all-to-all" as a pull: reads the k
//       result rows from the owners' buffers (peer loads), weights them with the gates and writes
//       the sum; optionally also returns the k dot products <other[t], row> (gate gradients).
//
// The reference has no MoE path at all; these kernels exist for the Mixtral-shaped configuration.
// Nothing here waits: ordering between the phases is done by the callers with flag kernels.
#include "host_common.h"
#include "ptx.cuh"

namespace mm {

constexpr int MOE_MAX_RANKS = 8;
constexpr int MOE_MAX_E = 64;
constexpr int MOE_MAX_K = 4;
constexpr int MM_ERR_MOE_CAPACITY = 9;   // a receive region overflowed (more rows than its capacity)

struct RouteDispatchArgs {
  const __nv_bfloat16* x;      // [T, D]
  const __nv_bfloat16* wr;     // [E, D]
  const __nv_bfloat16* other;  // optional [T, D]: second row per token (scaled by the gate)
  int T, D, E, k, experts_per_rank, capacity, nranks;
  __nv_bfloat16* recv[MOE_MAX_RANKS];        // [experts_per_rank][capacity][D] in every owner's memory
  __nv_bfloat16* recv_other[MOE_MAX_RANKS];  // same shape, for `other`
  int* counter[MOE_MAX_RANKS];               // [experts_per_rank] in every owner's memory
  int* idx;        // out [T, k] chosen experts
  float* gates;    // out [T, k]
  int* slot;       // out [T, k] slot inside the chosen expert's region
};

__global__ void __launch_bounds__(256)
    moe_route_dispatch_kernel(RouteDispatchArgs a, int* __restrict__ err) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= a.T) return;
  const int t = warp;
  const int nvec = a.D / 8;  // 16-byte vectors per row
  const uint4* xrow = reinterpret_cast<const uint4*>(a.x + static_cast<int64_t>(t) * a.D);
  // ---- router logits: every lane owns the vectors lane, lane + 32, ...
  float logit[MOE_MAX_E];
#pragma unroll 1
  for (int e = 0; e < a.E; ++e) {
    const uint4* wrow = reinterpret_cast<const uint4*>(a.wr + static_cast<int64_t>(e) * a.D);
    float acc = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 xv = xrow[v], wv = __ldg(wrow + v);
      const float2 x0 = unpack_bf16(xv.x), x1 = unpack_bf16(xv.y), x2 = unpack_bf16(xv.z), x3 = unpack_bf16(xv.w);
      const float2 w0 = unpack_bf16(wv.x), w1 = unpack_bf16(wv.y), w2 = unpack_bf16(wv.z), w3 = unpack_bf16(wv.w);
      acc += x0.x * w0.x + x0.y * w0.y + x1.x * w1.x + x1.y * w1.y + x2.x * w2.x + x2.y * w2.y + x3.x * w3.x + x3.y * w3.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    logit[e] = acc;
  }
  // ---- top-k (ties: lowest index) and softmax over the chosen logits; identical in every lane
  int chosen[MOE_MAX_K];
  float val[MOE_MAX_K];
  float mx = -INFINITY;
  for (int j = 0; j < a.k; ++j) {
    int best = -1;
    float bv = -INFINITY;
    for (int e = 0; e < a.E; ++e) {
      bool taken = false;
      for (int i = 0; i < j; ++i) taken |= chosen[i] == e;
      if (!taken && logit[e] > bv) { bv = logit[e]; best = e; }
    }
    if (best < 0) {
      // no logit compares greater than -inf (all NaN or -inf, a diverging run): the choice must
      // still be an expert, so take the lowest index not chosen yet, with a neutral logit
      for (int e = 0; e < a.E && best < 0; ++e) {
        bool taken = false;
        for (int i = 0; i < j; ++i) taken |= chosen[i] == e;
        if (!taken) best = e;
      }
      bv = 0.f;
    }
    chosen[j] = best;
    val[j] = bv;
    mx = fmaxf(mx, bv);
  }
  float den = 0.f;
  for (int j = 0; j < a.k; ++j) { val[j] = __expf(val[j] - mx); den += val[j]; }
  // ---- dispatch
  const uint4* orow = a.other ? reinterpret_cast<const uint4*>(a.other + static_cast<int64_t>(t) * a.D) : nullptr;
  for (int j = 0; j < a.k; ++j) {
    const float gate = val[j] / den;
    const int e = chosen[j];
    if (e < 0 || e >= a.E || e / a.experts_per_rank >= a.nranks) {
      // cannot happen with a total selection; checked because the stores below go to a peer
      if (lane == 0) {
        atomicCAS(err, 0, MM_ERR_BOUNDS);
        a.idx[t * a.k + j] = 0;
        a.gates[t * a.k + j] = 0.f;
        a.slot[t * a.k + j] = a.capacity;    // marks "no row": combine skips it
      }
      continue;
    }
    const int owner = e / a.experts_per_rank, el = e - owner * a.experts_per_rank;
    int s = 0;
    if (lane == 0) s = atomicAdd_system(a.counter[owner] + el, 1);
    s = __shfl_sync(0xffffffffu, s, 0);
    if (lane == 0) {
      a.idx[t * a.k + j] = e;
      a.gates[t * a.k + j] = gate;
      a.slot[t * a.k + j] = s;
    }
    if (s < 0 || s >= a.capacity) {
      if (lane == 0) atomicCAS(err, 0, s < 0 ? static_cast<int>(MM_ERR_BOUNDS) : MM_ERR_MOE_CAPACITY);
      continue;
    }
    const int64_t off = (static_cast<int64_t>(el) * a.capacity + s) * a.D;
    uint4* dst = reinterpret_cast<uint4*>(a.recv[owner] + off);
    for (int v = lane; v < nvec; v += 32) dst[v] = xrow[v];
    if (orow) {
      uint4* dst2 = reinterpret_cast<uint4*>(a.recv_other[owner] + off);
      for (int v = lane; v < nvec; v += 32) {
        const uint4 u = orow[v];
        const float2 p0 = unpack_bf16(u.x), p1 = unpack_bf16(u.y), p2 = unpack_bf16(u.z), p3 = unpack_bf16(u.w);
        uint4 o;
        o.x = pack_bf16(p0.x * gate, p0.y * gate);
        o.y = pack_bf16(p1.x * gate, p1.y * gate);
        o.z = pack_bf16(p2.x * gate, p2.y * gate);
        o.w = pack_bf16(p3.x * gate, p3.y * gate);
        dst2[v] = o;
      }
    }
  }
}

struct CombineArgs {
  const __nv_bfloat16* buf[MOE_MAX_RANKS];   // [experts_per_rank][capacity][D] in every owner's memory
  const int* idx;       // [T, k]
  const int* slot;      // [T, k]
  const float* gates;   // [T, k] or null (weights of 1)
  const __nv_bfloat16* other;  // optional [T, D] for the dot products
  float* dots;          // optional out [T, k]: <other[t], row_k>
  __nv_bfloat16* y;     // optional out [T, D]: sum_k w_k * row_k
  int T, D, k, experts_per_rank, capacity, nranks;
};

__global__ void __launch_bounds__(256) moe_combine_kernel(CombineArgs a) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= a.T) return;
  const int t = warp;
  const int nvec = a.D / 8;
  const uint4* rows[MOE_MAX_K];
  float w[MOE_MAX_K], dot[MOE_MAX_K];
  for (int j = 0; j < a.k; ++j) {
    const int e = a.idx[t * a.k + j], s = a.slot[t * a.k + j];
    const int owner = e / a.experts_per_rank, el = e - owner * a.experts_per_rank;
    const bool valid = s >= 0 && s < a.capacity && e >= 0 && owner < a.nranks;
    rows[j] = valid ? reinterpret_cast<const uint4*>(a.buf[owner] + (static_cast<int64_t>(el) * a.capacity + s) * a.D)
                    : nullptr;
    w[j] = a.gates ? a.gates[t * a.k + j] : 1.f;
    dot[j] = 0.f;
  }
  const uint4* orow = a.other ? reinterpret_cast<const uint4*>(a.other + static_cast<int64_t>(t) * a.D) : nullptr;
  uint4* yrow = a.y ? reinterpret_cast<uint4*>(a.y + static_cast<int64_t>(t) * a.D) : nullptr;
  for (int v = lane; v < nvec; v += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float ov[8];
    if (orow) {
      const uint4 u = orow[v];
      const float2 p0 = unpack_bf16(u.x), p1 = unpack_bf16(u.y), p2 = unpack_bf16(u.z), p3 = unpack_bf16(u.w);
      ov[0] = p0.x; ov[1] = p0.y; ov[2] = p1.x; ov[3] = p1.y; ov[4] = p2.x; ov[5] = p2.y; ov[6] = p3.x; ov[7] = p3.y;
    }
    for (int j = 0; j < a.k; ++j) {
      if (!rows[j]) continue;
      const uint4 u = __ldcg(rows[j] + v);   // written by another GPU: not through L1
      const float2 p0 = unpack_bf16(u.x), p1 = unpack_bf16(u.y), p2 = unpack_bf16(u.z), p3 = unpack_bf16(u.w);
      const float r[8] = {p0.x, p0.y, p1.x, p1.y, p2.x, p2.y, p3.x, p3.y};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        acc[i] += w[j] * r[i];
        if (orow) dot[j] += ov[i] * r[i];
      }
    }
    if (yrow) {
      uint4 o;
      o.x = pack_bf16(acc[0], acc[1]);
      o.y = pack_bf16(acc[2], acc[3]);
      o.z = pack_bf16(acc[4], acc[5]);
      o.w = pack_bf16(acc[6], acc[7]);
      yrow[v] = o;
    }
  }
  if (a.dots) {
    for (int j = 0; j < a.k; ++j) {
      float d = dot[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (lane == 0) a.dots[t * a.k + j] = d;
    }
  }
}

}  // namespace mm

extern "C" {

// Router + dispatch for T local tokens. recv / recv_other / counter: `nranks` addresses (this
// rank's own buffers at its own position). D must be a multiple of 8, E <= 64, k <= 4.
int mm_moe_route_dispatch(const void* x, const void* wr, const void* other, int T, int D, int E, int k,
                          int experts_per_rank, int capacity, const int64_t* recv, const int64_t* recv_other,
                          const int64_t* counter, int nranks, int* idx, float* gates, int* slot, cudaStream_t stream) {
  using namespace mm;
  if (T <= 0) return 0;
  if (D % 8 || E > MOE_MAX_E || k > MOE_MAX_K || k > E || nranks > MOE_MAX_RANKS || E != experts_per_rank * nranks) return -2;
  DeviceState* ds = device_state();
  if (!ds) return -1;
  RouteDispatchArgs a;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.wr = static_cast<const __nv_bfloat16*>(wr);
  a.other = static_cast<const __nv_bfloat16*>(other);
  a.T = T; a.D = D; a.E = E; a.k = k; a.experts_per_rank = experts_per_rank; a.capacity = capacity;
  a.nranks = nranks;
  for (int r = 0; r < nranks; ++r) {
    a.recv[r] = reinterpret_cast<__nv_bfloat16*>(recv[r]);
    a.recv_other[r] = recv_other ? reinterpret_cast<__nv_bfloat16*>(recv_other[r]) : nullptr;
    a.counter[r] = reinterpret_cast<int*>(counter[r]);
  }
  a.idx = idx; a.gates = gates; a.slot = slot;
  const int threads = 256;
  const int blocks = (T * 32 + threads - 1) / threads;
  moe_route_dispatch_kernel<<<blocks, threads, 0, stream>>>(a, ds->status);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// Combine (pull) for T local tokens; y and / or dots may be null.
int mm_moe_combine(const int64_t* buf, int nranks, const int* idx, const int* slot, const float* gates,
                   const void* other, float* dots, void* y, int T, int D, int k, int experts_per_rank, int capacity,
                   cudaStream_t stream) {
  using namespace mm;
  if (T <= 0) return 0;
  if (D % 8 || k > MOE_MAX_K || nranks > MOE_MAX_RANKS) return -2;
  CombineArgs a;
  for (int r = 0; r < nranks; ++r) a.buf[r] = reinterpret_cast<const __nv_bfloat16*>(buf[r]);
  a.idx = idx; a.slot = slot; a.gates = gates;
  a.other = static_cast<const __nv_bfloat16*>(other);
  a.dots = dots;
  a.y = static_cast<__nv_bfloat16*>(y);
  a.T = T; a.D = D; a.k = k; a.experts_per_rank = experts_per_rank; a.capacity = capacity;
  a.nranks = nranks;
  const int threads = 256;
  const int blocks = (T * 32 + threads - 1) / threads;
  moe_combine_kernel<<<blocks, threads, 0, stream>>>(a);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // extern "C"
