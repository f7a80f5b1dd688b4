// Integer and boolean matrix multiplication: solid_gpu_gemm_<T>, solid_gpu_gemm_with_plan_<T>,
// solid_gpu_gemm_create_plan.  Replaces solid/src/core/gpu/template_blas.cu:26-259 (floating-point GEMM is
// cuBLAS's business in Ocean and not part of this library).
//
//   C = alpha * op(A) * op(B) + beta * C      column-major, leading dimensions in ELEMENTS, op = identity or transpose
//
// in the wrap-around arithmetic of the element type (bool: and / or), as the CPU file
// solid/src/core/cpu/template_blas.c:30-200 computes it.  Products and sums of 1-, 2- and 4-byte types are formed in
// 32-bit unsigned arithmetic, whose low bits are those of the narrow type; 8-byte types use 64-bit arithmetic.
// A block of 32 x 8 threads produces a 32 x 32 tile of C from 32-deep slices of A and B staged in shared memory;
// each operand is read with the lanes running along its contiguous dimension, whatever the transposition.
#include "solid_core_gpu.h"
#include "dtypes.cuh"
#include "layout.h"

namespace sd {

constexpr int GT = 32;                       // tile of C and depth of a slice

template <class T, bool IS_BOOL, bool TA, bool TB>
__global__ void __launch_bounds__(GT * 8) gemm_kernel(size_t M, size_t N, size_t K, T alpha, const T *palpha, T beta, const T *pbeta,
                                                      const T *__restrict__ A, ptrdiff_t ldA, const T *__restrict__ B, ptrdiff_t ldB,
                                                      T *__restrict__ C, ptrdiff_t ldC)
{
   using W = typename std::conditional<sizeof(T) == 8, uint64_t, uint32_t>::type;
   __shared__ W As[GT][GT + 1];              // As[k][m]
   __shared__ W Bs[GT][GT + 1];              // Bs[k][n]
   const int tx = threadIdx.x, ty = threadIdx.y;
   const size_t row0 = (size_t)blockIdx.x * GT, col0 = (size_t)blockIdx.y * GT;
   if (palpha) alpha = *palpha;              // scalars in device memory
   if (pbeta)  beta  = *pbeta;
   W acc[4] = {0, 0, 0, 0};                  // C(row0 + tx, col0 + ty + 8 r)

   if (alpha != 0) {
      for (size_t k0 = 0; k0 < K; k0 += GT) {
#pragma unroll
         for (int r = 0; r < 4; r++) {
            const int s = ty + 8 * r;
            if (!TA) {  // A is M x K: lanes along the rows
               const size_t m = row0 + tx, k = k0 + s;
               As[s][tx] = (m < M && k < K) ? (W)A[m + k * ldA] : (W)0;
            } else {    // A is K x M: lanes along the depth
               const size_t k = k0 + tx, m = row0 + s;
               As[tx][s] = (m < M && k < K) ? (W)A[k + m * ldA] : (W)0;
            }
            if (!TB) {  // B is K x N: lanes along the depth
               const size_t k = k0 + tx, n = col0 + s;
               Bs[tx][s] = (n < N && k < K) ? (W)B[k + n * ldB] : (W)0;
            } else {    // B is N x K: lanes along the columns of C
               const size_t n = col0 + tx, k = k0 + s;
               Bs[s][tx] = (n < N && k < K) ? (W)B[n + k * ldB] : (W)0;
            }
         }
         __syncthreads();
#pragma unroll 8
         for (int k = 0; k < GT; k++) {
            const W a = As[k][tx];
#pragma unroll
            for (int r = 0; r < 4; r++) {
               if (IS_BOOL) acc[r] |= a & Bs[k][ty + 8 * r];
               else         acc[r] += a * Bs[k][ty + 8 * r];
            }
         }
         __syncthreads();
      }
   }
   const size_t row = row0 + tx;
#pragma unroll
   for (int r = 0; r < 4; r++) {
      const size_t col = col0 + ty + 8 * r;
      if (row < M && col < N) {
         T *c = C + row + col * ldC;
         const W old = (W)*c;
         const W v = IS_BOOL ? (((W)alpha & acc[r]) | ((W)beta & old)) : ((W)alpha * acc[r] + (W)beta * old);
         *c = (T)v;
      }
   }
}

template <class T, bool IS_BOOL>
int gemm_launch(const solid_gpu_gemm_plan *plan, void *ptrAlpha, void *ptrA, ptrdiff_t ldA, void *ptrB, ptrdiff_t ldB,
                void *ptrBeta, void *ptrC, ptrdiff_t ldC, int scalarModeHost, cudaStream_t stream)
{
   if (plan == nullptr) SD_ERROR("gemm: missing plan");
   const size_t M = plan->M, N = plan->N, K = plan->K;
   if (M == 0 || N == 0) return 0;
   T alpha = 1, beta = 0; const T *pa = nullptr, *pb = nullptr;          // absent scalars: alpha = 1, beta = 0
   if (scalarModeHost) {
      if (ptrAlpha) alpha = *(const T *)ptrAlpha;
      if (ptrBeta)  beta  = *(const T *)ptrBeta;
   } else { pa = (const T *)ptrAlpha; pb = (const T *)ptrBeta; }
   if (!aligned_to(ptrA, sizeof(T)) || !aligned_to(ptrB, sizeof(T)) || !aligned_to(ptrC, sizeof(T)))
      SD_ERROR("Tensor data must be aligned to the element size");
   const dim3 grid((unsigned)((M + GT - 1) / GT), (unsigned)((N + GT - 1) / GT), 1), block(GT, 8, 1);
   if ((N + GT - 1) / GT > 65535) SD_ERROR("gemm: more than 65535 column tiles");
   const bool ta = plan->transA == 'T', tb = plan->transB == 'T';
   const T *A = (const T *)ptrA, *B = (const T *)ptrB; T *C = (T *)ptrC;
   if (!ta && !tb) gemm_kernel<T, IS_BOOL, false, false><<<grid, block, 0, stream>>>(M, N, K, alpha, pa, beta, pb, A, ldA, B, ldB, C, ldC);
   if (!ta &&  tb) gemm_kernel<T, IS_BOOL, false, true ><<<grid, block, 0, stream>>>(M, N, K, alpha, pa, beta, pb, A, ldA, B, ldB, C, ldC);
   if ( ta && !tb) gemm_kernel<T, IS_BOOL, true,  false><<<grid, block, 0, stream>>>(M, N, K, alpha, pa, beta, pb, A, ldA, B, ldB, C, ldC);
   if ( ta &&  tb) gemm_kernel<T, IS_BOOL, true,  true ><<<grid, block, 0, stream>>>(M, N, K, alpha, pa, beta, pb, A, ldA, B, ldB, C, ldC);
   SD_LAUNCH_CHECK();
   return 0;
}

static int gemm_mode(char c, const char *which, char *out)
{
   if (c == 'n' || c == 'N') { *out = 'N'; return 0; }
   if (c == 't' || c == 'T') { *out = 'T'; return 0; }
   SD_ERROR("Invalid mode for matrix %s in gemm", which);
}

} // namespace sd

extern "C" int solid_gpu_gemm_create_plan(char transA, char transB, size_t M, size_t N, size_t K, int elemsize, int device,
                                          solid_gpu_gemm_plan *plan)
{
   (void)elemsize; (void)device;                              // one tile shape serves every type and device here
   if (plan == nullptr) SD_ERROR("gemm: missing plan");
   if (sd::gemm_mode(transA, "A", &plan->transA) != 0 || sd::gemm_mode(transB, "B", &plan->transB) != 0) return -1;
   plan->M = M; plan->N = N; plan->K = K;
   plan->gridsize = dim3((unsigned)((M + sd::GT - 1) / sd::GT), (unsigned)((N + sd::GT - 1) / sd::GT), 1);
   plan->blocksize = dim3(sd::GT, 8, 1);
   plan->tilesize = sd::GT; plan->sharedmem = 0;
   return 0;
}

#define SD_DEFINE_GEMM(CT, TYPE, IS_BOOL)                                                                             \
   extern "C" int solid_gpu_gemm_with_plan_##TYPE(SOLID_GPU_ARGS_GEMM_WITH_PLAN)                                      \
   {  return sd::gemm_launch<CT, IS_BOOL>(plan, ptrAlpha, ptrA, ldA, ptrB, ldB, ptrBeta, ptrC, ldC, scalarModeHost, stream); } \
   extern "C" int solid_gpu_gemm_##TYPE(SOLID_GPU_ARGS_GEMM)                                                          \
   {  solid_gpu_gemm_plan plan;                                                                                       \
      if (solid_gpu_gemm_create_plan(transA, transB, M, N, K, (int)sizeof(CT), 0, &plan) != 0) return -1;             \
      return sd::gemm_launch<CT, IS_BOOL>(&plan, ptrAlpha, ptrA, ldA, ptrB, ldB, ptrBeta, ptrC, ldC, scalarModeHost, stream); }
SD_DEFINE_GEMM(uint8_t, bool, true)
SD_DEFINE_GEMM(uint8_t, uint8, false) SD_DEFINE_GEMM(uint16_t, uint16, false) SD_DEFINE_GEMM(uint32_t, uint32, false)
SD_DEFINE_GEMM(uint64_t, uint64, false)
SD_DEFINE_GEMM(int8_t, int8, false) SD_DEFINE_GEMM(int16_t, int16, false) SD_DEFINE_GEMM(int32_t, int32, false)
SD_DEFINE_GEMM(int64_t, int64, false)
