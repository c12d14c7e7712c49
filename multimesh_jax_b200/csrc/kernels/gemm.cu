// bf16 GEMM entry points (forward, dgrad and wgrad layouts) on the tcgen05 main loop.
#include "gemm_core.cuh"
#include "host_common.h"

namespace mm {

template <bool A_MN, bool B_MN, int OUT>
static int launch_plain(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int64_t ldc,
                        int M, int N, int K, bool vec_ok, cudaStream_t stream) {
  DeviceState* ds = device_state();
  if (!ds) return -1;
  using Hook = PlainHook<OUT>;
  auto kern = gemm_bf16_kernel<A_MN, B_MN, Hook>;
  static bool configured[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev]) {
    MM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     GEMM_SMEM_BYTES));
    configured[dev] = true;
  }
  const int num_tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + GEMM_BN - 1) / GEMM_BN);
  const int grid = num_tiles < ds->sm_count ? num_tiles : ds->sm_count;
  Hook hook{C, ldc, vec_ok};
  GemmShape shape{M, N, K};
  kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, stream>>>(tmA, tmB, shape, hook, ds->status);
  MM_CUDA_TRY(cudaGetLastError());
  return 0;
}

template <bool A_MN, bool B_MN>
static int dispatch_out(int out_mode, const CUtensorMap& tmA, const CUtensorMap& tmB, void* C,
                        int64_t ldc, int M, int N, int K, bool vec_ok, cudaStream_t stream) {
  switch (out_mode) {
    case OUT_BF16: return launch_plain<A_MN, B_MN, OUT_BF16>(tmA, tmB, C, ldc, M, N, K, vec_ok, stream);
    case OUT_F32: return launch_plain<A_MN, B_MN, OUT_F32>(tmA, tmB, C, ldc, M, N, K, vec_ok, stream);
    case OUT_F32_ACC: return launch_plain<A_MN, B_MN, OUT_F32_ACC>(tmA, tmB, C, ldc, M, N, K, vec_ok, stream);
    case OUT_BF16_ACC: return launch_plain<A_MN, B_MN, OUT_BF16_ACC>(tmA, tmB, C, ldc, M, N, K, vec_ok, stream);
  }
  return -3;
}

// Builds the tensor maps of both operands. Operand A is logically [M, K]:
// a_mn == 0 means memory is [M][K] (row stride lda), a_mn == 1 means [K][M].
// Operand B is logically [N, K] with the same convention.
int make_gemm_tmaps(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, int a_mn, int64_t lda,
                    const void* B, int b_mn, int64_t ldb, int M, int N, int K) {
  int rc;
  if (!a_mn)
    rc = encode_tmap_2d_bf16(tmA, A, K, M, lda * 2, GEMM_BK, GEMM_BM);
  else
    rc = encode_tmap_2d_bf16(tmA, A, M, K, lda * 2, 64, GEMM_BK);
  if (rc) return rc;
  if (!b_mn)
    rc = encode_tmap_2d_bf16(tmB, B, K, N, ldb * 2, GEMM_BK, GEMM_BN);
  else
    rc = encode_tmap_2d_bf16(tmB, B, N, K, ldb * 2, 64, GEMM_BK);
  return rc;
}

}  // namespace mm

extern "C" {

// C[M,N] (op)= A[M,K] * B[N,K]^T with bf16 operands and fp32 accumulation.
//   a_mn / b_mn : 0 = operand stored K-contiguous, 1 = stored M/N-contiguous
//   out_mode    : 0 bf16 store, 1 fp32 store, 2 fp32 accumulate, 3 bf16 accumulate
// Leading dimensions are in elements. Returns 0 on success.
int mm_gemm_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb,
                 void* C, int out_mode, int64_t ldc, int M, int N, int K, cudaStream_t stream) {
  using namespace mm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8)) {
    fprintf(stderr, "[mm_kernels] gemm: leading dimensions must be multiples of 8 elements\n");
    return -2;
  }
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) {
    fprintf(stderr, "[mm_kernels] gemm: operands must be 16-byte aligned\n");
    return -2;
  }
  CUtensorMap tmA, tmB;
  int rc = make_gemm_tmaps(&tmA, &tmB, A, a_mn, lda, B, b_mn, ldb, M, N, K);
  if (rc) return rc;
  const int esz = (out_mode == OUT_BF16 || out_mode == OUT_BF16_ACC) ? 2 : 4;
  const bool vec_ok = ((ldc * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
  if (!a_mn && !b_mn) return dispatch_out<false, false>(out_mode, tmA, tmB, C, ldc, M, N, K, vec_ok, stream);
  if (!a_mn && b_mn) return dispatch_out<false, true>(out_mode, tmA, tmB, C, ldc, M, N, K, vec_ok, stream);
  if (a_mn && b_mn) return dispatch_out<true, true>(out_mode, tmA, tmB, C, ldc, M, N, K, vec_ok, stream);
  return dispatch_out<true, false>(out_mode, tmA, tmB, C, ldc, M, N, K, vec_ok, stream);
}

}  // extern "C"
