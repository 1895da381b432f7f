// Exact-order GEMM schedule on CUDA cores.
//
// Every output element is computed with the reference recurrence: accumulator
// starts at +0.0f, k increases from 0, each step is one IEEE f32 product
// followed by one IEEE f32 sum (no fused contraction), then the optional
// epilogue alpha*acc + beta*c as two products and one sum
// (examples/tiled_gemm_v1/src/oracle.rs:284-321,
//  examples/tiled_gemm_v1/src/numerical_contract.rs:310-326,
//  examples/scalar_gemm_v1/src/kernel.rs:8-27).  Results are therefore
// bit-identical to the CPU oracle for every finite or non-finite input, any
// strides and any tails.  64x64 output tile per 256-thread block, 4x4 outputs
// per thread, K staged through shared memory 16 deep.
#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename T>
__device__ __forceinline__ float widen(T v);
template <>
__device__ __forceinline__ float widen<float>(float v) { return v; }
template <>
__device__ __forceinline__ float widen<uint16_t>(uint16_t v) { return bf16_bits_to_f32(v); }

template <typename T, bool EPILOGUE>
__global__ void __launch_bounds__(256)
gemm_exact_kernel(const T *__restrict__ A, const T *__restrict__ B, float *C, uint32_t M, uint32_t N, uint32_t K,
                  uint32_t lda, uint32_t ldb, uint32_t ldc, float alpha, float beta) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const uint32_t row0 = blockIdx.y * TM, col0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (uint32_t k0 = 0; k0 < K; k0 += TK) {
        // A tile: 64 rows x 16 k; each thread loads 4 elements (k fastest for coalescing)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 256;
            const int r = e >> 4, kk = e & 15;
            const uint32_t gr = row0 + r, gk = k0 + kk;
            As[kk][r] = (gr < M && gk < K) ? widen<T>(A[(uint64_t)gr * lda + gk]) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 256;
            const int kk = e >> 6, c = e & 63;
            const uint32_t gk = k0 + kk, gc = col0 + c;
            Bs[kk][c] = (gk < K && gc < N) ? widen<T>(B[(uint64_t)gk * ldb + gc]) : 0.0f;
        }
        __syncthreads();
        const int kmax = (K - k0) < (uint32_t)TK ? (int)(K - k0) : TK;
        // Tail steps must not run: adding a zero product could turn -0 into +0
        // only when acc is -0, which the recurrence never produces from +0, but
        // stopping at kmax keeps the step count identical to the oracle anyway.
        for (int kk = 0; kk < kmax; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t r = row0 + ty * 4 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t c = col0 + tx * 4 + j;
            if (c >= N) continue;
            float *dst = C + (uint64_t)r * ldc + c;
            if (EPILOGUE)
                *dst = __fadd_rn(__fmul_rn(alpha, acc[i][j]), __fmul_rn(beta, *dst));
            else
                *dst = acc[i][j];
        }
    }
}

}  // namespace

// dtype: FE2O3_DTYPE_F32 or FE2O3_DTYPE_BF16 inputs.
int32_t launch_gemm_exact(cudaStream_t s, uint32_t dtype, bool epilogue, uint64_t a, uint64_t b, uint64_t c,
                          uint32_t M, uint32_t N, uint32_t K, uint32_t lda, uint32_t ldb, uint32_t ldc, float alpha,
                          float beta, fe2o3_geometry *geo, bool plan_only) {
    dim3 grid(ceil_div_u32(N, TN), ceil_div_u32(M, TM), 1);
    if (geo) *geo = fe2o3_geometry{{grid.x, grid.y, 1}, {256, 1, 1}, 0, 1};
    if (plan_only || M == 0 || N == 0) return FE2O3_OK;
    float *C = reinterpret_cast<float *>(c);
    if (dtype == FE2O3_DTYPE_F32) {
        const float *A = reinterpret_cast<const float *>(a), *B = reinterpret_cast<const float *>(b);
        if (epilogue) gemm_exact_kernel<float, true><<<grid, 256, 0, s>>>(A, B, C, M, N, K, lda, ldb, ldc, alpha, beta);
        else gemm_exact_kernel<float, false><<<grid, 256, 0, s>>>(A, B, C, M, N, K, lda, ldb, ldc, alpha, beta);
    } else {
        const uint16_t *A = reinterpret_cast<const uint16_t *>(a), *B = reinterpret_cast<const uint16_t *>(b);
        if (epilogue) gemm_exact_kernel<uint16_t, true><<<grid, 256, 0, s>>>(A, B, C, M, N, K, lda, ldb, ldc, alpha, beta);
        else gemm_exact_kernel<uint16_t, false><<<grid, 256, 0, s>>>(A, B, C, M, N, K, lda, ldb, ldc, alpha, beta);
    }
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "gemm_exact");
}

static Fe2o3KernelRegistration reg_scalar("scalar_gemm_v1", reinterpret_cast<const void *>(gemm_exact_kernel<float, false>));
