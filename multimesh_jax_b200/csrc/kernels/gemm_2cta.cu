// bf16 GEMM entry point on CTA pairs (tcgen05 cta_group::2, 256x256 tile per pair of SMs).
#include "gemm_pair_core.cuh"

namespace mm {

template <bool A_MN, bool B_MN, int OUT>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int64_t ldc, int M, int N, int K,
                       bool vec_ok, cudaStream_t stream, const int* m_dev, const int* k_dev) {
  DeviceState* ds = device_state();
  if (!ds) return -1;
  PlainHook<OUT> hook{C, ldc, vec_ok};
  return launch_pair_kernel<A_MN, B_MN>(tmA, tmB, hook, M, N, K, ds->sm_count, ds->status, stream, m_dev, k_dev);
}

template <bool A_MN, bool B_MN>
static int dispatch_pair(int out_mode, const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int64_t ldc, int M,
                         int N, int K, bool vec_ok, cudaStream_t stream, const int* m_dev, const int* k_dev) {
  switch (out_mode) {
    case OUT_BF16: return launch_pair<A_MN, B_MN, OUT_BF16>(tmA, tmB, C, ldc, M, N, K, vec_ok, stream, m_dev, k_dev);
    case OUT_F32: return launch_pair<A_MN, B_MN, OUT_F32>(tmA, tmB, C, ldc, M, N, K, vec_ok, stream, m_dev, k_dev);
    case OUT_F32_ACC: return launch_pair<A_MN, B_MN, OUT_F32_ACC>(tmA, tmB, C, ldc, M, N, K, vec_ok, stream, m_dev, k_dev);
    case OUT_BF16_ACC: return launch_pair<A_MN, B_MN, OUT_BF16_ACC>(tmA, tmB, C, ldc, M, N, K, vec_ok, stream, m_dev, k_dev);
  }
  return -3;
}

}  // namespace mm

extern "C" {

int mm_gemm_pair_dyn_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* C,
                          int out_mode, int64_t ldc, int M, int N, int K, const int* m_dev, const int* k_dev,
                          cudaStream_t stream);

// Same contract as mm_gemm_bf16, computed by CTA pairs (256x256 tile per pair).
int mm_gemm_pair_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* C,
                      int out_mode, int64_t ldc, int M, int N, int K, cudaStream_t stream) {
  return mm_gemm_pair_dyn_bf16(A, a_mn, lda, B, b_mn, ldb, C, out_mode, ldc, M, N, K, nullptr, nullptr, stream);
}

// The same GEMM with run-time extents: M and K are upper bounds (operands and output are
// allocated for them), the kernel works on min(M, *m_dev) rows and min(K, *k_dev) contraction
// elements read from device memory when it starts (either pointer may be null). With a k_dev
// the rows of both operands between *k_dev and the next multiple of 64 must be zero
// (mm_zero_row_tail); *k_dev == 0 leaves C untouched.
int mm_gemm_pair_dyn_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* C,
                          int out_mode, int64_t ldc, int M, int N, int K, const int* m_dev, const int* k_dev,
                          cudaStream_t stream) {
  using namespace mm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8)) {
    fprintf(stderr, "[mm_kernels] gemm_pair: leading dimensions must be multiples of 8 elements\n");
    return -2;
  }
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) {
    fprintf(stderr, "[mm_kernels] gemm_pair: operands must be 16-byte aligned\n");
    return -2;
  }
  CUtensorMap tmA, tmB;
  int rc = make_pair_tmaps(&tmA, &tmB, A, a_mn, lda, B, b_mn, ldb, M, N, K);
  if (rc) return rc;
  const int esz = (out_mode == OUT_BF16 || out_mode == OUT_BF16_ACC) ? 2 : 4;
  const bool vec_ok = ((ldc * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
  if (!a_mn && !b_mn) return dispatch_pair<false, false>(out_mode, tmA, tmB, C, ldc, M, N, K, vec_ok, stream, m_dev, k_dev);
  if (!a_mn && b_mn) return dispatch_pair<false, true>(out_mode, tmA, tmB, C, ldc, M, N, K, vec_ok, stream, m_dev, k_dev);
  if (a_mn && b_mn) return dispatch_pair<true, true>(out_mode, tmA, tmB, C, ldc, M, N, K, vec_ok, stream, m_dev, k_dev);
  return dispatch_pair<true, false>(out_mode, tmA, tmB, C, ldc, M, N, K, vec_ok, stream, m_dev, k_dev);
}

}  // extern "C"
