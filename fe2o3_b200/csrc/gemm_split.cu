// f32-input GEMM on the tensor cores by bf16 splitting.
//
// examples/scalar_gemm_v1/src/kernel.rs:8-27 multiplies f32 matrices.  tcgen05
// has no f32 x f32 product, so each f32 operand is split into two bf16 terms,
// hi = bf16(v) and mid = bf16(v - hi) (v - hi is exact in f32), and the product is
// taken as  A_hi*B_mid + A_mid*B_hi + A_hi*B_hi,  three bf16 GEMMs accumulated in
// f32.  They run as ONE launch of the bf16 tensor-core kernel on operands
// concatenated along K:
//     A' = [A_hi | A_mid | A_hi]   (M x 3K)        B' = [B_mid ; B_hi ; B_hi]   (3K x N)
// (small terms first, so they are not rounded away against the large partial sum).
// What is left out is A_mid*B_mid and the third terms of both operands, each below
// 2^-16 of |a||b|: per element |C - A*B| <= 2^-14 * (|A|*|B|) plus the f32
// accumulation error, 32 times tighter than TF32's 2^-10 * (|A|*|B|) at a cost
// of three bf16 passes (against two bf16-equivalents for one TF32 pass).  The
// exact-order CUDA-core schedule stays the bit-exact lane.
#include "common.cuh"

namespace {

// One thread per 8 source values along the contiguous dimension.
// layout 0 (operand A, [rows][cols] -> [rows][3*cols]): columns [0,cols) hi, [cols,2cols) mid, [2cols,3cols) hi
// layout 1 (operand B, [rows][cols] -> [3*rows][cols]): rows    [0,rows) mid, [rows,2rows) hi,  [2rows,3rows) hi
__global__ void __launch_bounds__(256)
split_bf16_kernel(const float *__restrict__ src, uint16_t *__restrict__ dst, uint32_t rows, uint32_t cols, uint32_t layout) {
    const uint64_t groups_per_row = cols / 8;
    const uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= (uint64_t)rows * groups_per_row) return;
    const uint32_t r = (uint32_t)(g / groups_per_row), c = (uint32_t)(g % groups_per_row) * 8;
    const float4 v0 = __ldg(reinterpret_cast<const float4 *>(src + (uint64_t)r * cols + c));
    const float4 v1 = __ldg(reinterpret_cast<const float4 *>(src + (uint64_t)r * cols + c) + 1);
    const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t hi[4], mid[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint16_t h[2], m[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float x = v[2 * i + j];
            h[j] = f32_to_bf16_bits(x);
            m[j] = f32_to_bf16_bits(__fsub_rn(x, bf16_bits_to_f32(h[j])));
        }
        hi[i] = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
        mid[i] = (uint32_t)m[0] | ((uint32_t)m[1] << 16);
    }
    const uint4 H = make_uint4(hi[0], hi[1], hi[2], hi[3]), M = make_uint4(mid[0], mid[1], mid[2], mid[3]);
    if (layout == 0) {
        uint16_t *row = dst + (uint64_t)r * 3 * cols;
        *reinterpret_cast<uint4 *>(row + c) = H;
        *reinterpret_cast<uint4 *>(row + cols + c) = M;
        *reinterpret_cast<uint4 *>(row + 2 * cols + c) = H;
    } else {
        *reinterpret_cast<uint4 *>(dst + (uint64_t)r * cols + c) = M;
        *reinterpret_cast<uint4 *>(dst + ((uint64_t)rows + r) * cols + c) = H;
        *reinterpret_cast<uint4 *>(dst + (2ull * rows + r) * cols + c) = H;
    }
}

}  // namespace

// f32 operands must be 16-byte aligned with K and N multiples of 8 (the split rows are copied 8 values at a time
// and the bf16 operands' leading dimensions must suit the copy engine).
bool gemm_split_supported(uint64_t a, uint64_t b, uint32_t N, uint32_t K) {
    return K > 0 && (a & 15u) == 0 && (b & 15u) == 0 && K % 8u == 0 && N % 8u == 0;
}

int32_t gemm_split_launch(cudaStream_t s, const float *a, const float *b, uint16_t *a3, uint16_t *b3, uint32_t M, uint32_t N,
                          uint32_t K) {
    const uint64_t ga = (uint64_t)M * (K / 8), gb = (uint64_t)K * (N / 8);
    if (ga) split_bf16_kernel<<<(uint32_t)((ga + 255) / 256), 256, 0, s>>>(a, a3, M, K, 0u);
    if (gb) split_bf16_kernel<<<(uint32_t)((gb + 255) / 256), 256, 0, s>>>(b, b3, K, N, 1u);
    fe2o3_count_launch(2);
    return fe2o3_cuda_status(cudaGetLastError(), "scalar_gemm_v1(split)");
}
