// Library matrix products of the fp32-residual decoders: C (fp32) = beta * C + A x W^T with bf16 or fp32 operands
// and fp32 accumulation (cuBLAS, as the fp16 path's `mode 0` arm in dense_gemm.cu).  fp32 operands run with the
// pedantic compute type: no TF32 or other reduced-precision mode.
#include <cublas_v2.h>

#include <mutex>

#include "../../include/b200_vllm.h"
#include "seqmix.cuh"

namespace b200 {
static std::mutex g_mu;
static cublasHandle_t g_h[16] = {nullptr};
static void* g_ws[16] = {nullptr};
static cublasHandle_t handle() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_h[dev]) {
    if (cublasCreate(&g_h[dev]) != CUBLAS_STATUS_SUCCESS) {
      g_h[dev] = nullptr;
      return nullptr;
    }
    cublasSetMathMode(g_h[dev], CUBLAS_PEDANTIC_MATH);
    // a fixed workspace keeps the calls capturable and their algorithm choice independent of the allocator
    if (cudaMalloc(&g_ws[dev], 32u << 20) == cudaSuccess) cublasSetWorkspace(g_h[dev], g_ws[dev], 32u << 20);
  }
  return g_h[dev];
}

bool gemm_f32out(const void* a, int lda, long long stride_a, const void* w, int ldw, long long stride_w, float* c,
                 int ldc, long long stride_c, int M, int N, int K, int batch, float beta, int w_kn, int dt,
                 cudaStream_t st) {
  return gemm_f32out_scaled(a, lda, stride_a, w, ldw, stride_w, c, ldc, stride_c, M, N, K, batch, 1.f, beta, w_kn, dt, st);
}

bool gemm_f32out_scaled(const void* a, int lda, long long stride_a, const void* w, int ldw, long long stride_w, float* c,
                        int ldc, long long stride_c, int M, int N, int K, int batch, float alpha, float beta, int w_kn,
                        int dt, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return true;
  cublasHandle_t h = handle();
  if (!h) {
    set_error(2, "gemm: cublasCreate failed");
    return false;
  }
  cublasSetStream(h, st);
  {
    int dev = 0;
    cudaGetDevice(&dev);       // setting the stream drops the user workspace: give it back (keeps the call capturable)
    if (g_ws[dev]) cublasSetWorkspace(h, g_ws[dev], 32u << 20);
  }
  const cudaDataType_t in = dt ? CUDA_R_32F : CUDA_R_16BF;
  const cublasComputeType_t comp = dt ? CUBLAS_COMPUTE_32F_PEDANTIC : CUBLAS_COMPUTE_32F;
  const cublasOperation_t opw = w_kn ? CUBLAS_OP_N : CUBLAS_OP_T;
  cublasStatus_t s;
  if (batch == 1)
    s = cublasGemmEx(h, opw, CUBLAS_OP_N, N, M, K, &alpha, w, in, ldw, a, in, lda, &beta, c, CUDA_R_32F, ldc, comp,
                     CUBLAS_GEMM_DEFAULT);
  else
    s = cublasGemmStridedBatchedEx(h, opw, CUBLAS_OP_N, N, M, K, &alpha, w, in, ldw, stride_w, a, in, lda, stride_a,
                                   &beta, c, CUDA_R_32F, ldc, stride_c, batch, comp, CUBLAS_GEMM_DEFAULT);
  count_launch(1);
  if (s != CUBLAS_STATUS_SUCCESS) {
    set_error(2, "gemm: cublasGemmEx failed");
    return false;
  }
  return true;
}
}  // namespace b200
