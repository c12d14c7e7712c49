// Small data-movement and scalar kernels that a natively launched task needs between the big
// ones: copies and fills, conversions between fp32 and bf16 for any element count, fp32
// accumulation, a deterministic scaled sum, and scaling by a scalar that lives on the device.
// With them a task body is a flat list of calls into this library and never needs an operator
// of the tensor framework.
#include "host_common.h"
#include "ptx.cuh"

namespace mm {

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = __float2bfloat16(src[i]);
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, int64_t n,
                                   int accumulate) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = __bfloat162float(src[i]);
    dst[i] = accumulate ? dst[i] + v : v;
  }
}
__global__ void accumulate_f32_kernel(float* __restrict__ acc, const float* __restrict__ src, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) acc[i] += src[i];
}
__global__ void fill_f32_kernel(float* __restrict__ dst, float value, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = value;
}
// out[0] = scale * sum(src[0..n)): one block, fixed summation order (the loss of a microbatch)
__global__ void __launch_bounds__(1024) sum_scale_f32_kernel(const float* __restrict__ src, int64_t n, float scale,
                                                            float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += 1024) s += src[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = red[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) out[0] = s * scale;
  }
}
// out = x * s with s a bf16 scalar in device memory; 16-byte vectors plus a scalar tail
__global__ void scale_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ s,
                                  __nv_bfloat16* __restrict__ out, int64_t n) {
  const float f = __bfloat162float(*s);
  const int64_t nvec = n / 8;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    const uint4 u = reinterpret_cast<const uint4*>(x)[v];
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
    uint4 o;
    o.x = pack_bf16(a.x * f, a.y * f);
    o.y = pack_bf16(b.x * f, b.y * f);
    o.z = pack_bf16(c.x * f, c.y * f);
    o.w = pack_bf16(d.x * f, d.y * f);
    reinterpret_cast<uint4*>(out)[v] = o;
  }
  for (int64_t i = nvec * 8 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = __float2bfloat16(__bfloat162float(x[i]) * f);
}
// dst[0] = src[0] + delta (the optimizer's step counter)
__global__ void add_i64_kernel(const int64_t* __restrict__ src, int64_t delta, int64_t* __restrict__ dst, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[i] + delta;
}

static inline unsigned grid_for(int64_t n, int threads, int cap) {
  int64_t b = (n + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return static_cast<unsigned>(b);
}

}  // namespace mm

namespace mm {
// blockIdx.y = which of the (at most `multiple` - 1) tail rows; see mm_zero_row_tail
__global__ void zero_row_tail_kernel(uint4* __restrict__ base, int64_t vecs_per_row, const int* __restrict__ count,
                                     int multiple, int capacity) {
  int c = *count;
  if (c < 0) c = 0;
  const int64_t row = static_cast<int64_t>(c) + blockIdx.y;
  const int64_t end = (static_cast<int64_t>(c) + multiple - 1) / multiple * multiple;
  if (row >= end || row >= capacity) return;
  const int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (v < vecs_per_row) base[row * vecs_per_row + v] = make_uint4(0, 0, 0, 0);
}

}  // namespace mm

extern "C" {
using namespace mm;

// Zeroes rows [*count, round_up(*count, multiple)) of a row-major matrix with `row_bytes` bytes per
// row (a multiple of 16) and `capacity` rows: the rows a GEMM with a run-time contraction extent
// still reads in its last k-block.
int mm_zero_row_tail(void* base, int64_t row_bytes, const int* count, int multiple, int capacity, cudaStream_t stream) {
  if (row_bytes <= 0 || (row_bytes & 15) || multiple < 1 || multiple > 1024) return -2;
  const int64_t vecs = row_bytes / 16;
  const int threads = 256;
  const int blocks = static_cast<int>((vecs + threads - 1) / threads);
  zero_row_tail_kernel<<<dim3(blocks, multiple), threads, 0, stream>>>(static_cast<uint4*>(base), vecs, count, multiple,
                                                                       capacity);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int mm_memcpy_d2d(void* dst, const void* src, int64_t bytes, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  MM_CUDA_TRY(cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice, stream));
  return 0;
}
int mm_zero(void* dst, int64_t bytes, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  MM_CUDA_TRY(cudaMemsetAsync(dst, 0, static_cast<size_t>(bytes), stream));
  return 0;
}
int mm_f32_to_bf16(const float* src, void* dst, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  f32_to_bf16_kernel<<<grid_for(n, 256, 4096), 256, 0, stream>>>(src, static_cast<__nv_bfloat16*>(dst), n);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
// dst(fp32) = src(bf16), or dst += src with accumulate != 0; any element count
int mm_bf16_to_f32(const void* src, float* dst, int64_t n, int accumulate, cudaStream_t stream) {
  if (n <= 0) return 0;
  bf16_to_f32_kernel<<<grid_for(n, 256, 4096), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), dst, n,
                                                                 accumulate);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int mm_accumulate_f32(float* acc, const float* src, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  accumulate_f32_kernel<<<grid_for(n, 256, 4096), 256, 0, stream>>>(acc, src, n);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int mm_fill_f32(float* dst, float value, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  fill_f32_kernel<<<grid_for(n, 256, 4096), 256, 0, stream>>>(dst, value, n);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int mm_sum_scale_f32(const float* src, int64_t n, float scale, float* out, cudaStream_t stream) {
  sum_scale_f32_kernel<<<1, 1024, 0, stream>>>(src, n, scale, out);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int mm_scale_bf16(const void* x, const void* scalar, void* out, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -2;
  scale_bf16_kernel<<<grid_for(n / 8 + 1, 256, 8192), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(scalar), static_cast<__nv_bfloat16*>(out), n);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int mm_add_i64(const int64_t* src, int64_t delta, int64_t* dst, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  add_i64_kernel<<<grid_for(n, 256, 65535), 256, 0, stream>>>(src, delta, dst, n);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // extern "C"
