#include "host_common.h"

#include <cstdlib>
#include <mutex>

namespace mm {

static DeviceState g_states[kMaxDevices];
static std::mutex g_mu;

DeviceState* device_state() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  DeviceState* s = &g_states[dev];
  if (s->ready) return s;
  std::lock_guard<std::mutex> lock(g_mu);
  if (s->ready) return s;
  if (cudaDeviceGetAttribute(&s->sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return nullptr;
  if (cudaMalloc(&s->status, 64) != cudaSuccess) return nullptr;
  if (cudaMemset(s->status, 0, 64) != cudaSuccess) return nullptr;
  // bytes 8..15: time limit of peer waits in nanoseconds (MM_PEER_WAIT_MS, default 20 s)
  unsigned long long limit_ns = 20000ull * 1000000ull;
  if (const char* e = getenv("MM_PEER_WAIT_MS")) {
    const long long ms = atoll(e);
    if (ms > 0) limit_ns = static_cast<unsigned long long>(ms) * 1000000ull;
  }
  if (cudaMemcpy(reinterpret_cast<char*>(s->status) + 8, &limit_ns, sizeof(limit_ns), cudaMemcpyHostToDevice) !=
      cudaSuccess)
    return nullptr;
  s->ready = true;
  return s;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int encode_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, int swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    fprintf(stderr, "[mm_kernels] cuTensorMapEncodeTiled is not available\n");
    return -1;
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstrides[i - 1] = strides_bytes[i];
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdims,
                  gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[mm_kernels] tensor map encode failed (%d): base=%p rank=%d dims=[%llu,%llu] "
            "stride1=%llu box=[%u,%u]\n",
            static_cast<int>(r), base, rank, (unsigned long long)dims[0],
            (unsigned long long)(rank > 1 ? dims[1] : 0),
            (unsigned long long)(rank > 1 ? strides_bytes[1] : 0), box[0], rank > 1 ? box[1] : 0);
    return static_cast<int>(r) + 10000;
  }
  return 0;
}

int encode_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                        uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[2] = {0, row_stride_bytes};
  uint32_t box[2] = {box_inner, box_outer};
  return encode_tmap_bf16(out, base, 2, dims, strides, box, 1);
}

}  // namespace mm

// ---------------------------------------------------------------- C API
extern "C" {

// Reads and clears the current device's kernel status word (synchronises the device).
int mm_read_status(int clear) {
  mm::DeviceState* s = mm::device_state();
  if (!s) return -1;
  int v = 0;
  if (cudaMemcpy(&v, s->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (clear && v != 0) cudaMemset(s->status, 0, sizeof(int));
  return v;
}

// Sets the time limit of peer waits on the current device (milliseconds; takes effect for kernels
// launched afterwards).
int mm_set_peer_wait_ms(int ms) {
  mm::DeviceState* s = mm::device_state();
  if (!s || ms <= 0) return -1;
  const unsigned long long limit_ns = static_cast<unsigned long long>(ms) * 1000000ull;
  if (cudaMemcpy(reinterpret_cast<char*>(s->status) + 8, &limit_ns, sizeof(limit_ns), cudaMemcpyHostToDevice) !=
      cudaSuccess)
    return -2;
  return 0;
}

// Device address of the current device's 64-byte status block (word 0 = status).
void* mm_status_ptr() {
  mm::DeviceState* s = mm::device_state();
  return s ? s->status : nullptr;
}

int mm_sm_count() {
  mm::DeviceState* s = mm::device_state();
  return s ? s->sm_count : -1;
}

}  // extern "C"
