// Memory-bound transformer kernels for sm_100a: RMSNorm, RoPE, SwiGLU, fused
// softmax cross-entropy, embedding gather / scatter-add, residual add,
// gradient accumulation, and the fused AdamW update over flat buffers.
// All use 16-byte vector accesses and keep each row resident in registers so
// every tensor is read once and written once.
#include "host_common.h"
#include "ptx.cuh"

namespace mm {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : -INFINITY;
  t = warp_max(t);
  return t;
}

// ------------------------------------------------------------------ RMSNorm
// One block per row; each thread keeps VPT 8-element vectors in registers.
// THREADS x VPT x 8 >= hidden size; instantiated for hidden sizes up to 16384.
template <int RN_THREADS, int RN_MAX_VEC>
__global__ void __launch_bounds__(RN_THREADS)
    rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int D, float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * D);
  const int nvec = D / 8;
  uint4 xv[RN_MAX_VEC];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < RN_MAX_VEC; ++i) {
    const int v = threadIdx.x + i * RN_THREADS;
    if (v < nvec) {
      xv[i] = xr[v];
      float2 a = unpack_bf16(xv[i].x), b = unpack_bf16(xv[i].y), c = unpack_bf16(xv[i].z),
             d = unpack_bf16(xv[i].w);
      ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x +
            d.y * d.y;
    }
  }
  ss = block_sum<RN_THREADS>(ss, red);
  const float r = rsqrtf(ss / D + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < RN_MAX_VEC; ++i) {
    const int v = threadIdx.x + i * RN_THREADS;
    if (v < nvec) {
      uint4 wv = wr[v];
      uint4 o;
      float2 a, g;
      a = unpack_bf16(xv[i].x); g = unpack_bf16(wv.x); o.x = pack_bf16(a.x * r * g.x, a.y * r * g.y);
      a = unpack_bf16(xv[i].y); g = unpack_bf16(wv.y); o.y = pack_bf16(a.x * r * g.x, a.y * r * g.y);
      a = unpack_bf16(xv[i].z); g = unpack_bf16(wv.z); o.z = pack_bf16(a.x * r * g.x, a.y * r * g.y);
      a = unpack_bf16(xv[i].w); g = unpack_bf16(wv.w); o.w = pack_bf16(a.x * r * g.x, a.y * r * g.y);
      yr[v] = o;
    }
  }
}

// Backward. dx = rstd * (dy*w) - x * rstd^3 * mean(dy*w*x).  Weight-gradient
// partial sums go to a scratch buffer `dw_partial` [gridDim.x, D] (fp32) that a
// second kernel reduces. Blocks stride over rows so the partial count is small.
template <int RN_THREADS, int RN_MAX_VEC>
__global__ void __launch_bounds__(RN_THREADS)
    rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd,
                       __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int rows,
                       int D, int add_to_dx) {
  // Two rows per iteration: the loads of both rows are in flight before the one block-wide sum
  // that serves both, and the rows stay packed (bf16) in registers between the two passes.
  __shared__ float red[64];
  const int nvec = D / 8;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float wreg[RN_MAX_VEC][8];
  float dwacc[RN_MAX_VEC][8];
#pragma unroll
  for (int i = 0; i < RN_MAX_VEC; ++i) {
    const int v = threadIdx.x + i * RN_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dwacc[i][j] = 0.f; wreg[i][j] = 0.f; }
    if (v < nvec) {
      uint4 wv = wr[v];
      float2 a = unpack_bf16(wv.x), b = unpack_bf16(wv.y), c = unpack_bf16(wv.z),
             d = unpack_bf16(wv.w);
      wreg[i][0] = a.x; wreg[i][1] = a.y; wreg[i][2] = b.x; wreg[i][3] = b.y;
      wreg[i][4] = c.x; wreg[i][5] = c.y; wreg[i][6] = d.x; wreg[i][7] = d.y;
    }
  }
  for (int64_t row = 2 * static_cast<int64_t>(blockIdx.x); row < rows; row += 2 * static_cast<int64_t>(gridDim.x)) {
    const int nr = (row + 1 < rows) ? 2 : 1;
    uint4 xv[2][RN_MAX_VEC], gv[2][RN_MAX_VEC];
    float rr[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int64_t rk = row + (k < nr ? k : 0);
      const uint4* xr = reinterpret_cast<const uint4*>(x + rk * D);
      const uint4* gr = reinterpret_cast<const uint4*>(dy + rk * D);
      rr[k] = k < nr ? rstd[rk] : 0.f;
#pragma unroll
      for (int i = 0; i < RN_MAX_VEC; ++i) {
        const int v = threadIdx.x + i * RN_THREADS;
        if (v < nvec) {
          xv[k][i] = xr[v];
          gv[k][i] = gr[v];
        } else {
          xv[k][i] = make_uint4(0, 0, 0, 0);
          gv[k][i] = make_uint4(0, 0, 0, 0);
        }
      }
    }
    float dot[2] = {0.f, 0.f};
#pragma unroll
    for (int k = 0; k < 2; ++k) {
#pragma unroll
      for (int i = 0; i < RN_MAX_VEC; ++i) {
        const uint32_t xw[4] = {xv[k][i].x, xv[k][i].y, xv[k][i].z, xv[k][i].w};
        const uint32_t gw[4] = {gv[k][i].x, gv[k][i].y, gv[k][i].z, gv[k][i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 xf = unpack_bf16(xw[j]), gf = unpack_bf16(gw[j]);
          const float p0 = gf.x * xf.x, p1 = gf.y * xf.y;
          dwacc[i][2 * j] += p0 * rr[k];          // rr is 0 for a missing second row
          dwacc[i][2 * j + 1] += p1 * rr[k];
          dot[k] += p0 * wreg[i][2 * j] + p1 * wreg[i][2 * j + 1];
        }
      }
    }
    // one pair of barriers for both rows
    dot[0] = warp_sum(dot[0]);
    dot[1] = warp_sum(dot[1]);
    {
      const int wi = threadIdx.x >> 5, l = threadIdx.x & 31;
      __syncthreads();
      if (l == 0) { red[wi] = dot[0]; red[32 + wi] = dot[1]; }
      __syncthreads();
      const float t0 = (l < RN_THREADS / 32) ? red[l] : 0.f;
      const float t1 = (l < RN_THREADS / 32) ? red[32 + l] : 0.f;
      dot[0] = warp_sum(t0);
      dot[1] = warp_sum(t1);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (k < nr) {
        const float r = rr[k];
        const float c = dot[k] * r * r * r / D;
        uint4* dxr = reinterpret_cast<uint4*>(dx + (row + k) * D);
#pragma unroll
        for (int i = 0; i < RN_MAX_VEC; ++i) {
          const int v = threadIdx.x + i * RN_THREADS;
          if (v < nvec) {
            const uint32_t xw[4] = {xv[k][i].x, xv[k][i].y, xv[k][i].z, xv[k][i].w};
            const uint32_t gw[4] = {gv[k][i].x, gv[k][i].y, gv[k][i].z, gv[k][i].w};
            uint32_t ow[4] = {0, 0, 0, 0};
            if (add_to_dx) {
              const uint4 old = dxr[v];
              ow[0] = old.x; ow[1] = old.y; ow[2] = old.z; ow[3] = old.w;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 xf = unpack_bf16(xw[j]), gf = unpack_bf16(gw[j]), of = unpack_bf16(ow[j]);
              const float o0 = gf.x * wreg[i][2 * j] * r - xf.x * c + of.x;
              const float o1 = gf.y * wreg[i][2 * j + 1] * r - xf.y * c + of.y;
              ow[j] = pack_bf16(o0, o1);
            }
            dxr[v] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
        }
      }
    }
  }
  float* out = dw_partial + static_cast<int64_t>(blockIdx.x) * D;
#pragma unroll
  for (int i = 0; i < RN_MAX_VEC; ++i) {
    const int v = threadIdx.x + i * RN_THREADS;
    if (v < nvec) {
      float4* o4 = reinterpret_cast<float4*>(out + v * 8);
      o4[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      o4[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// dw[j] (+)= sum_p partial[p, j]
__global__ void __launch_bounds__(256) colsum_partials_kernel(const float* __restrict__ partial, float* __restrict__ dw,
                                                               int parts, int D, int accumulate) {
  // 32 columns x 8 slices of the partials per block: the loads of a warp are one 128-byte line
  // and eight of them are in flight per column before the shared-memory reduction
  __shared__ float red[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (j < D) {
    int p = ty;
    for (; p + 24 < parts; p += 32) {
      const float a0 = partial[static_cast<int64_t>(p) * D + j];
      const float a1 = partial[static_cast<int64_t>(p + 8) * D + j];
      const float a2 = partial[static_cast<int64_t>(p + 16) * D + j];
      const float a3 = partial[static_cast<int64_t>(p + 24) * D + j];
      s += (a0 + a1) + (a2 + a3);
    }
    for (; p < parts; p += 8) s += partial[static_cast<int64_t>(p) * D + j];
  }
  red[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && j < D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][tx];
    dw[j] = accumulate ? dw[j] + t : t;
  }
}

// --------------------------------------------------------------------- RoPE
// In-place rotate-half rotary embedding on a [T, H, Dh] view with row stride
// `stride_t` elements (lets q and k be slices of one fused QKV buffer).
// cos/sin tables are fp32 [S, Dh/2]; position of token t is t % S.
// `sign` = +1 forward, -1 backward (inverse rotation).
// Heads may be packed in groups of `group_size` of which only the first `rot_per_group`
// are rotated (query heads and the key head of a grouped-query group; the value head is
// skipped): logical head h maps to (h / rot_per_group) * group_size + h % rot_per_group.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qk, const float* __restrict__ cs,
                            const float* __restrict__ sn, int64_t T, int S, int H, int Dh,
                            int64_t stride_t, float sign, int rot_per_group, int group_size) {
  // one thread rotates 8 adjacent pairs: two 16-byte loads and stores of the head, and the
  // matching 32 bytes of each table, are in flight per thread
  const int half = Dh / 2;
  const int per_head = half / 8;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_tok = H * per_head;
  const int64_t total = T * per_tok;
  if (idx >= total) return;
  const int64_t t = idx / per_tok;
  const int rem = static_cast<int>(idx - t * per_tok);
  int h = rem / per_head;
  const int i = (rem - h * per_head) * 8;
  h = (h / rot_per_group) * group_size + h % rot_per_group;
  const int pos = static_cast<int>(t % S);
  __nv_bfloat16* base = qk + t * stride_t + static_cast<int64_t>(h) * Dh;
  const uint4 lo = *reinterpret_cast<const uint4*>(base + i);
  const uint4 hi = *reinterpret_cast<const uint4*>(base + i + half);
  const float4* cp = reinterpret_cast<const float4*>(cs + static_cast<int64_t>(pos) * half + i);
  const float4* sp = reinterpret_cast<const float4*>(sn + static_cast<int64_t>(pos) * half + i);
  const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
  uint32_t ol[4], oh[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 a = unpack_bf16(lw[j]), b = unpack_bf16(hw[j]);
    const float sx = sv[2 * j] * sign, sy = sv[2 * j + 1] * sign;
    ol[j] = pack_bf16(a.x * c[2 * j] - b.x * sx, a.y * c[2 * j + 1] - b.y * sy);
    oh[j] = pack_bf16(b.x * c[2 * j] + a.x * sx, b.y * c[2 * j + 1] + a.y * sy);
  }
  *reinterpret_cast<uint4*>(base + i) = make_uint4(ol[0], ol[1], ol[2], ol[3]);
  *reinterpret_cast<uint4*>(base + i + half) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
}

// ------------------------------------------------------------------- SwiGLU
// gu is [T, 2F]: gate in columns [0,F), up in [F,2F).  h = silu(gate) * up.
// rows_dev (may be null): device-side count of the rows that hold data; rows behind it are skipped.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ h, int64_t T, int F, const int* __restrict__ rows_dev) {
  // two 8-element groups per thread (half the array apart), all four loads issued first
  if (rows_dev) {
    const int64_t live = *rows_dev;
    T = live < 0 ? 0 : (live < T ? live : T);
  }
  const int fv = F / 8;
  const int64_t total = T * fv;
  const int64_t half = (total + 1) / 2;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= half) return;
  const int64_t e[2] = {idx, idx + half};
  uint4 g[2], u[2];
  int64_t t[2];
  int v[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int64_t ek = e[k] < total ? e[k] : idx;
    t[k] = ek / fv;
    v[k] = static_cast<int>(ek - t[k] * fv);
    g[k] = reinterpret_cast<const uint4*>(gu + t[k] * 2 * F)[v[k]];
    u[k] = reinterpret_cast<const uint4*>(gu + t[k] * 2 * F + F)[v[k]];
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    if (e[k] >= total) break;
    const uint32_t gg[4] = {g[k].x, g[k].y, g[k].z, g[k].w}, uu[4] = {u[k].x, u[k].y, u[k].z, u[k].w};
    uint32_t oo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16(gg[j]), b = unpack_bf16(uu[j]);
      float s0 = a.x / (1.f + __expf(-a.x)), s1 = a.y / (1.f + __expf(-a.y));
      oo[j] = pack_bf16(s0 * b.x, s1 * b.y);
    }
    reinterpret_cast<uint4*>(h + t[k] * F)[v[k]] = make_uint4(oo[0], oo[1], oo[2], oo[3]);
  }
}

// dgu[:, :F] = dh * up * silu'(gate),  dgu[:, F:] = dh * silu(gate)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  const __nv_bfloat16* __restrict__ dh,
                                  __nv_bfloat16* __restrict__ dgu, int64_t T, int F, const int* __restrict__ rows_dev) {
  if (rows_dev) {
    const int64_t live = *rows_dev;
    T = live < 0 ? 0 : (live < T ? live : T);
  }
  const int fv = F / 8;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * fv) return;
  const int64_t t = idx / fv;
  const int v = static_cast<int>(idx - t * fv);
  const uint4 g = reinterpret_cast<const uint4*>(gu + t * 2 * F)[v];
  const uint4 u = reinterpret_cast<const uint4*>(gu + t * 2 * F + F)[v];
  const uint4 d = reinterpret_cast<const uint4*>(dh + t * F)[v];
  const uint32_t gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w},
                 dd[4] = {d.x, d.y, d.z, d.w};
  uint32_t og[4], ou[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 a = unpack_bf16(gg[j]), b = unpack_bf16(uu[j]), e = unpack_bf16(dd[j]);
    float sg0 = 1.f / (1.f + __expf(-a.x)), sg1 = 1.f / (1.f + __expf(-a.y));
    float si0 = a.x * sg0, si1 = a.y * sg1;
    float ds0 = sg0 * (1.f + a.x * (1.f - sg0)), ds1 = sg1 * (1.f + a.y * (1.f - sg1));
    og[j] = pack_bf16(e.x * b.x * ds0, e.y * b.y * ds1);
    ou[j] = pack_bf16(e.x * si0, e.y * si1);
  }
  reinterpret_cast<uint4*>(dgu + t * 2 * F)[v] = make_uint4(og[0], og[1], og[2], og[3]);
  reinterpret_cast<uint4*>(dgu + t * 2 * F + F)[v] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
}

struct CeCombineArgs {
  const float* stats[8];
  int nranks;
};
__global__ void __launch_bounds__(256)
    ce_combine_kernel(CeCombineArgs a, const int64_t* __restrict__ targets, float* __restrict__ stats2,
                      float* __restrict__ loss, int64_t rows) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float m[8], s[8], tl = 0.f, mx = -INFINITY;
  for (int r = 0; r < a.nranks; ++r) {
    // written by another GPU: read past L1
    m[r] = __ldcg(a.stats[r] + row * 3);
    s[r] = __ldcg(a.stats[r] + row * 3 + 1);
    tl += __ldcg(a.stats[r] + row * 3 + 2);
    mx = fmaxf(mx, m[r]);
  }
  float se = 0.f;
  for (int r = 0; r < a.nranks; ++r) se += (m[r] == -INFINITY) ? 0.f : s[r] * __expf(m[r] - mx);
  stats2[row * 2] = mx;
  stats2[row * 2 + 1] = se;
  loss[row] = targets[row] >= 0 ? logf(se) + mx - tl : 0.f;
}

// ----------------------------------------------------------- cross-entropy
// One block per row. Pass 1: online max / sum-exp. Pass 2 (optional): write
// dlogits = (softmax - onehot) * grad_scale in place of the logits.
// loss[row] = logsumexp - logit[target]; rows with target < 0 are ignored.
// For a vocabulary sharded over ranks, `vocab_start` is this shard's first id
// and stats_out receives (max, sumexp, target_logit) for a later combine.
constexpr int CE_THREADS = 256;
__global__ void __launch_bounds__(CE_THREADS)
    cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                         float* __restrict__ loss, float* __restrict__ stats_out,
                         const float* __restrict__ stats_in, int V, int64_t ld, int vocab_start,
                         float grad_scale, int write_grad) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int64_t tgt = targets[row];
  const int nvec = V / 8;
  float mx, se;
  if (stats_in) {
    mx = stats_in[row * 2];
    se = stats_in[row * 2 + 1];
  } else {
    float m = -INFINITY, s = 0.f;
    for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
      uint4 x = reinterpret_cast<const uint4*>(lr)[v];
      const uint32_t xx[4] = {x.x, x.y, x.z, x.w};
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 a = unpack_bf16(xx[j]); f[2 * j] = a.x; f[2 * j + 1] = a.y; }
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      const float nm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
    for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) {
      const float f = __bfloat162float(lr[j]);
      const float nm = fmaxf(m, f);
      s = s * __expf(m - nm) + __expf(f - nm);
      m = nm;
    }
    mx = block_max<CE_THREADS>(m, red);
    const float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - mx);
    se = block_sum<CE_THREADS>(contrib, red);
  }
  const int64_t local_t = tgt - vocab_start;
  const bool has_t = tgt >= 0 && local_t >= 0 && local_t < V;
  if (threadIdx.x == 0) {
    const float tl = has_t ? __bfloat162float(lr[local_t]) : 0.f;
    if (stats_out) {
      stats_out[row * 3] = mx;
      stats_out[row * 3 + 1] = se;
      stats_out[row * 3 + 2] = tl;
    }
    if (loss) loss[row] = (tgt >= 0) ? (logf(se) + mx - tl) : 0.f;
  }
  if (!write_grad) return;
  const float inv = (tgt >= 0) ? grad_scale / se : 0.f;
  const float gs = (tgt >= 0) ? grad_scale : 0.f;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    uint4 x = reinterpret_cast<const uint4*>(lr)[v];
    const uint32_t xx[4] = {x.x, x.y, x.z, x.w};
    uint32_t oo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16(xx[j]);
      float g0 = __expf(a.x - mx) * inv, g1 = __expf(a.y - mx) * inv;
      const int c = v * 8 + 2 * j;
      if (has_t && c == local_t) g0 -= gs;
      if (has_t && c + 1 == local_t) g1 -= gs;
      oo[j] = pack_bf16(g0, g1);
    }
    reinterpret_cast<uint4*>(lr)[v] = make_uint4(oo[0], oo[1], oo[2], oo[3]);
  }
  for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) {
    float g = __expf(__bfloat162float(lr[j]) - mx) * inv;
    if (has_t && j == local_t) g -= gs;
    lr[j] = __float2bfloat16(g);
  }
}

// ---------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const __nv_bfloat16* __restrict__ table,
                                     const int64_t* __restrict__ ids, __nv_bfloat16* __restrict__ out,
                                     int64_t T, int D, int vocab_start, int vocab_size, int* __restrict__ err) {
  const int dv = D / 8;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * dv) return;
  const int64_t t = idx / dv;
  const int v = static_cast<int>(idx - t * dv);
  (void)err;
  MM_CHECK_OR(ids[t] >= 0, err, (void)0);     // ids of other vocabulary shards are legal, negative ones never are
  const int64_t id = ids[t] - vocab_start;
  uint4 val = make_uint4(0, 0, 0, 0);
  if (id >= 0 && id < vocab_size) val = reinterpret_cast<const uint4*>(table + id * D)[v];
  reinterpret_cast<uint4*>(out + t * D)[v] = val;
}
// grad_table (fp32) [V, D] += scatter of dout rows.
__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                     const int64_t* __restrict__ ids, float* __restrict__ grad,
                                     int64_t T, int D, int vocab_start, int vocab_size, int* __restrict__ err) {
  const int dv = D / 2;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= T * dv) return;
  const int64_t t = idx / dv;
  const int v = static_cast<int>(idx - t * dv);
  (void)err;
  MM_CHECK_OR(ids[t] >= 0, err, return);
  const int64_t id = ids[t] - vocab_start;
  if (id < 0 || id >= vocab_size) return;
  const float2 g = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(dout + t * D)[v]);
  float* dst = grad + id * D + v * 2;
  atomicAdd(dst, g.x);
  atomicAdd(dst + 1, g.y);
}

// ------------------------------------------------------- adds / accumulation
// out = a + b (bf16); out may alias a.
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, int64_t n8) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 x = reinterpret_cast<const uint4*>(a)[i], y = reinterpret_cast<const uint4*>(b)[i];
  const uint32_t xx[4] = {x.x, x.y, x.z, x.w}, yy[4] = {y.x, y.y, y.z, y.w};
  uint32_t oo[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 p = unpack_bf16(xx[j]), q = unpack_bf16(yy[j]);
    oo[j] = pack_bf16(p.x + q.x, p.y + q.y);
  }
  reinterpret_cast<uint4*>(out)[i] = make_uint4(oo[0], oo[1], oo[2], oo[3]);
}
// acc(fp32) += src(bf16)
__global__ void accumulate_f32_bf16_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ src,
                                           int64_t n8) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 x = reinterpret_cast<const uint4*>(src)[i];
  float4* a4 = reinterpret_cast<float4*>(acc) + i * 2;
  float4 a0 = a4[0], a1 = a4[1];
  float2 p;
  p = unpack_bf16(x.x); a0.x += p.x; a0.y += p.y;
  p = unpack_bf16(x.y); a0.z += p.x; a0.w += p.y;
  p = unpack_bf16(x.z); a1.x += p.x; a1.y += p.y;
  p = unpack_bf16(x.w); a1.z += p.x; a1.w += p.y;
  a4[0] = a0;
  a4[1] = a1;
}

// --------------------------------------------------------------------- AdamW
// Flat-buffer update: fp32 master weights, moments and gradients; writes the
// bf16 working copy in the same pass. grad is multiplied by grad_scale first
// (1/num_microbatches, loss scaling or clip coefficient).
__global__ void adamw_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ param,
                             float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ grad, int64_t n4, float lr, float beta1,
                             float beta2, float eps, float wd, float bc1, float bc2,
                             float grad_scale, const int64_t* __restrict__ step_dev) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  if (step_dev) {  // step count lives on the device: no host synchronisation per update
    const float t = static_cast<float>(*step_dev);
    bc1 = 1.f - powf(beta1, t);
    bc2 = 1.f - powf(beta2, t);
  }
  float4 p = reinterpret_cast<float4*>(master)[i];
  float4 mm_ = reinterpret_cast<float4*>(m)[i];
  float4 vv = reinterpret_cast<float4*>(v)[i];
  const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
  float pa[4] = {p.x, p.y, p.z, p.w}, ma[4] = {mm_.x, mm_.y, mm_.z, mm_.w},
        va[4] = {vv.x, vv.y, vv.z, vv.w}, ga[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float g = ga[j] * grad_scale;
    ma[j] = beta1 * ma[j] + (1.f - beta1) * g;
    va[j] = beta2 * va[j] + (1.f - beta2) * g * g;
    const float mh = ma[j] / bc1, vh = va[j] / bc2;
    pa[j] = pa[j] * (1.f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
  }
  reinterpret_cast<float4*>(master)[i] = make_float4(pa[0], pa[1], pa[2], pa[3]);
  reinterpret_cast<float4*>(m)[i] = make_float4(ma[0], ma[1], ma[2], ma[3]);
  reinterpret_cast<float4*>(v)[i] = make_float4(va[0], va[1], va[2], va[3]);
  uint2 o;
  o.x = pack_bf16(pa[0], pa[1]);
  o.y = pack_bf16(pa[2], pa[3]);
  reinterpret_cast<uint2*>(param)[i] = o;
}

// sum of squares of an fp32 buffer into out[0] (atomic), for gradient clipping.
__global__ void sumsq_f32_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float f = x[i];
    s += f * f;
  }
  s = block_sum<256>(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

}  // namespace mm

// -------------------------------------------------------------------- C API
extern "C" {
using namespace mm;

static inline unsigned blocks_for(int64_t n, int threads) {
  return static_cast<unsigned>((n + threads - 1) / threads);
}

int mm_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int64_t rows, int D,
                   float eps, cudaStream_t stream) {
  if (D % 8 || D > 16384) return -2;
  if (rows == 0) return 0;
#define MM_RN_FWD(TH, VPT)                                                              \
  rmsnorm_fwd_kernel<TH, VPT><<<static_cast<unsigned>(rows), TH, 0, stream>>>(          \
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),       \
      static_cast<__nv_bfloat16*>(y), rstd, D, eps)
  if (D <= 1024) MM_RN_FWD(128, 1);
  else if (D <= 2048) MM_RN_FWD(128, 2);
  else if (D <= 4096) MM_RN_FWD(128, 4);
  else if (D <= 8192) MM_RN_FWD(256, 4);
  else MM_RN_FWD(512, 4);
#undef MM_RN_FWD
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// Number of row-partials the backward kernel produces for `rows` rows; the
// scratch buffer must hold mm_rmsnorm_bwd_parts(rows) * D floats.
int mm_rmsnorm_bwd_parts(int64_t rows) {
  DeviceState* ds = device_state();
  // enough blocks for 16-24 resident warps per SM: the kernel is bound by memory latency, and
  // the loads in flight per SM set its bandwidth
  const int cap = ds ? ds->sm_count * 4 : 592;
  return static_cast<int>(rows < cap ? rows : cap);
}

// dw_out is fp32 [D]; accumulate_dw != 0 adds into it. add_to_dx != 0 adds
// the result into dx (fuses the residual-branch gradient add).
int mm_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                   float* dw_out, float* scratch, int64_t rows, int D, int accumulate_dw,
                   int add_to_dx, cudaStream_t stream) {
  if (D % 8 || D > 16384) return -2;
  if (rows < 0 || rows > 2147483647LL) return -2;   // the kernel indexes rows with an int
  if (rows == 0) return 0;
  const int parts = mm_rmsnorm_bwd_parts(rows);
#define MM_RN_BWD(TH, VPT)                                                                   \
  rmsnorm_bwd_kernel<TH, VPT><<<parts, TH, 0, stream>>>(                                     \
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),            \
      static_cast<const __nv_bfloat16*>(dy), rstd, static_cast<__nv_bfloat16*>(dx), scratch, \
      static_cast<int>(rows), D, add_to_dx)
  if (D <= 1024) MM_RN_BWD(128, 1);
  else if (D <= 2048) MM_RN_BWD(128, 2);
  else if (D <= 4096) MM_RN_BWD(256, 2);
  else if (D <= 8192) MM_RN_BWD(512, 2);
  else MM_RN_BWD(512, 4);
#undef MM_RN_BWD
  MM_CUDA_TRY(cudaGetLastError());
  colsum_partials_kernel<<<(D + 31) / 32, 256, 0, stream>>>(scratch, dw_out, parts, D,
                                                               accumulate_dw);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int mm_rope(void* qk, const float* cos_t, const float* sin_t, int64_t T, int S, int H, int Dh,
            int64_t stride_t, int backward, int rot_per_group, int group_size, cudaStream_t stream) {
  if (Dh % 16 || (stride_t % 8) || (reinterpret_cast<uintptr_t>(qk) & 15)) return -2;
  if (rot_per_group <= 0 || group_size <= 0) { rot_per_group = 1; group_size = 1; }
  const int64_t total = T * H * (Dh / 16);
  if (total == 0) return 0;
  rope_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(qk), cos_t,
                                                         sin_t, T, S, H, Dh, stride_t,
                                                         backward ? -1.f : 1.f, rot_per_group,
                                                         group_size);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// rows_dev (may be null): one int in device memory, the number of leading rows that hold data
// (T is then the capacity the launch is sized for).
int mm_swiglu_fwd_rows(const void* gu, void* h, int64_t T, int F, const int* rows_dev, cudaStream_t stream) {
  if (F % 8) return -2;
  const int64_t total = T * (F / 8);
  if (total == 0) return 0;
  swiglu_fwd_kernel<<<blocks_for((total + 1) / 2, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(h), T, F, rows_dev);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int mm_swiglu_fwd(const void* gu, void* h, int64_t T, int F, cudaStream_t stream) {
  return mm_swiglu_fwd_rows(gu, h, T, F, nullptr, stream);
}
int mm_swiglu_bwd_rows(const void* gu, const void* dh, void* dgu, int64_t T, int F, const int* rows_dev,
                       cudaStream_t stream) {
  if (F % 8) return -2;
  const int64_t total = T * (F / 8);
  if (total == 0) return 0;
  swiglu_bwd_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dh),
      static_cast<__nv_bfloat16*>(dgu), T, F, rows_dev);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int mm_swiglu_bwd(const void* gu, const void* dh, void* dgu, int64_t T, int F, cudaStream_t stream) {
  return mm_swiglu_bwd_rows(gu, dh, dgu, T, F, nullptr, stream);
}

int mm_cross_entropy(void* logits, const int64_t* targets, float* loss, float* stats_out,
                     const float* stats_in, int64_t rows, int V, int64_t ld, int vocab_start,
                     float grad_scale, int write_grad, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (ld % 8) return -2;
  cross_entropy_kernel<<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(
      static_cast<__nv_bfloat16*>(logits), targets, loss, stats_out, stats_in, V, ld, vocab_start,
      grad_scale, write_grad);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// Combines the per-shard softmax statistics of a vocabulary-sharded cross-entropy: stats[r] is
// rank r's [rows, 3] array of (max, sum-exp relative to that max, target logit or 0) - local
// memory for this rank, peer memory for the others. Writes the global (max, sum-exp) per row
// to stats2 [rows, 2] and the loss per row (0 for ignored rows).
int mm_ce_combine(const int64_t* stats, int nranks, const int64_t* targets, float* stats2, float* loss,
                  int64_t rows, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (nranks < 1 || nranks > 8) return -2;
  CeCombineArgs a;
  for (int r = 0; r < nranks; ++r) a.stats[r] = reinterpret_cast<const float*>(stats[r]);
  a.nranks = nranks;
  ce_combine_kernel<<<blocks_for(rows, 256), 256, 0, stream>>>(a, targets, stats2, loss, rows);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int mm_embedding_fwd(const void* table, const int64_t* ids, void* out, int64_t T, int D,
                     int vocab_start, int vocab_size, cudaStream_t stream) {
  if (D % 8) return -2;
  const int64_t total = T * (D / 8);
  if (total == 0) return 0;
  embedding_fwd_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(table), ids, static_cast<__nv_bfloat16*>(out), T, D,
      vocab_start, vocab_size, device_state() ? device_state()->status : nullptr);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int mm_embedding_bwd(const void* dout, const int64_t* ids, float* grad, int64_t T, int D,
                     int vocab_start, int vocab_size, cudaStream_t stream) {
  if (D % 2) return -2;
  const int64_t total = T * (D / 2);
  if (total == 0) return 0;
  embedding_bwd_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dout), ids, grad, T, D, vocab_start, vocab_size,
      device_state() ? device_state()->status : nullptr);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int mm_add_bf16(const void* a, const void* b, void* out, int64_t n, cudaStream_t stream) {
  if (n % 8) return -2;
  if (n == 0) return 0;
  add_bf16_kernel<<<blocks_for(n / 8, 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b),
      static_cast<__nv_bfloat16*>(out), n / 8);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int mm_accumulate_f32_bf16(float* acc, const void* src, int64_t n, cudaStream_t stream) {
  if (n % 8) return -2;
  if (n == 0) return 0;
  accumulate_f32_bf16_kernel<<<blocks_for(n / 8, 256), 256, 0, stream>>>(
      acc, static_cast<const __nv_bfloat16*>(src), n / 8);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int mm_adamw(float* master, void* param, float* m, float* v, const float* grad, int64_t n, float lr,
             float beta1, float beta2, float eps, float wd, int step, float grad_scale,
             const int64_t* step_dev, cudaStream_t stream) {
  if (n % 4) return -2;
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
  adamw_kernel<<<blocks_for(n / 4, 256), 256, 0, stream>>>(master, static_cast<__nv_bfloat16*>(param),
                                                         m, v, grad, n / 4, lr, beta1, beta2, eps,
                                                         wd, bc1, bc2, grad_scale, step_dev);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int mm_sumsq_f32(const float* x, int64_t n, float* out, cudaStream_t stream) {
  if (n == 0) return 0;
  DeviceState* ds = device_state();
  const int grid = ds ? ds->sm_count * 4 : 592;
  sumsq_f32_kernel<<<grid, 256, 0, stream>>>(x, n, out);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------ allocation-free variant
// See no_alloc.h. The scratch for the weight-gradient partial sums lives in the library
// image; host code must not pass the symbol itself to a kernel (on the host it is only a
// stand-in), so the device address is looked up once per device and cached.
#include "no_alloc.h"

#include <mutex>

static __device__ __align__(256) float g_noalloc_scratch[MM_NOALLOC_MAX_PARTS * MM_NOALLOC_MAX_D];

namespace {
float* g_noalloc_ptr[mm::kMaxDevices] = {};
std::mutex g_noalloc_mu;

// Device address of the scratch array on the current device (looked up on first use).
float* noalloc_scratch_for_current_device(int* rc) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= mm::kMaxDevices) {
    fprintf(stderr, "[mm_kernels] rmsnorm_bwd_noalloc: cannot identify the current device\n");
    *rc = -1;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      fprintf(stderr, "[mm_kernels] rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s\n",
              cudaGetErrorString(e));
      *rc = static_cast<int>(e ? e : cudaErrorUnknown);
      return nullptr;
    }
    g_noalloc_ptr[dev] = p;
  }
  *rc = 0;
  return g_noalloc_ptr[dev];
}
}  // namespace

extern "C" int mm_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd,
                                      void* dx, float* dw_out, int64_t rows, int D, int accumulate_dw,
                                      int add_to_dx, cudaStream_t stream) {
  using namespace mm;
  if (D <= 0 || D % 8 != 0 || D > MM_NOALLOC_MAX_D) {
    fprintf(stderr,
            "[mm_kernels] rmsnorm_bwd_noalloc: hidden size %d is not supported (multiple of 8, at most %d); "
            "use mm_rmsnorm_bwd with a caller-provided scratch buffer\n",
            D, MM_NOALLOC_MAX_D);
    return -2;
  }
  if (rows < 0 || rows > 2147483647LL) {
    fprintf(stderr, "[mm_kernels] rmsnorm_bwd_noalloc: %lld rows are not supported (0 .. 2^31 - 1)\n",
            static_cast<long long>(rows));
    return -2;
  }
  if (rows == 0) return 0;
  int rc = 0;
  float* scratch = noalloc_scratch_for_current_device(&rc);
  if (!scratch) return rc;
  const int parts = static_cast<int>(rows < MM_NOALLOC_MAX_PARTS ? rows : MM_NOALLOC_MAX_PARTS);
#define MM_RN_BWD_NA(TH, VPT)                                                                 \
  rmsnorm_bwd_kernel<TH, VPT><<<parts, TH, 0, stream>>>(                                      \
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),             \
      static_cast<const __nv_bfloat16*>(dy), rstd, static_cast<__nv_bfloat16*>(dx), scratch,  \
      static_cast<int>(rows), D, add_to_dx)
  if (D <= 1024) MM_RN_BWD_NA(128, 1);
  else if (D <= 2048) MM_RN_BWD_NA(128, 2);
  else if (D <= 4096) MM_RN_BWD_NA(128, 4);
  else MM_RN_BWD_NA(256, 4);
#undef MM_RN_BWD_NA
  MM_CUDA_TRY(cudaGetLastError());
  // every block wrote its full row of partials above, so the reduction reads only fresh data
  colsum_partials_kernel<<<(D + 31) / 32, 256, 0, stream>>>(scratch, dw_out, parts, D, accumulate_dw);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
