// Row softmax: examples/row_softmax_v1/src/kernel.rs:13-42 generalised from one
// 64-element row to rows x cols, with the oracle's optional activity mask
// (src/numerical_contract.rs:130-199): f32 maximum over active elements,
// weights exp(x - max), row sum, quotient; masked outputs are +0.0; a row with
// a non-finite physical input or no active element is left unwritten and a
// status word is recorded instead of trapping.
//
// HBM-bound: each element is read once and written once (8 bytes per element).
// The fast path keeps a whole row in the registers of one warp (cols <= 1024,
// cols % 4 == 0, 16-byte aligned rows): 128-bit coalesced loads, two shuffle
// trees, 128-bit stores.  Other shapes (cols <= 4096, the reference's bound)
// use one 256-thread block per row with scalar accesses.
#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
__device__ __forceinline__ bool finite4(float4 v) {
    return isfinite(v.x) && isfinite(v.y) && isfinite(v.z) && isfinite(v.w);
}

constexpr int kWarpsPerBlock = 8;

// NV = float4 loads per lane; the row has 128*NV columns at most.
template <int NV, bool MASKED>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
row_softmax_warp_kernel(const float *__restrict__ in, float *__restrict__ out, const uint8_t *__restrict__ mask,
                        uint32_t rows, uint32_t cols, uint32_t *status) {
    const uint32_t row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint32_t nvec = cols >> 2;
    const float4 *src = reinterpret_cast<const float4 *>(in + (uint64_t)row * cols);
    float4 v[NV];
    uint32_t act[NV];  // 4 activity bits per vector
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const uint32_t idx = i * 32 + lane;
        if (idx < nvec) {
            v[i] = __ldcs(src + idx);
            act[i] = 0xfu;
            if (MASKED) {
                uchar4 m = *reinterpret_cast<const uchar4 *>(mask + (uint64_t)row * cols + 4ull * idx);
                act[i] = (m.x ? 1u : 0u) | (m.y ? 2u : 0u) | (m.z ? 4u : 0u) | (m.w ? 8u : 0u);
            }
        } else {
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            act[i] = 0u;
        }
    }
    bool ok = true;
    float mx = -INFINITY;
    uint32_t any = 0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        ok = ok && finite4(v[i]);
        any |= act[i];
        if (act[i] & 1u) mx = fmaxf(mx, v[i].x);
        if (act[i] & 2u) mx = fmaxf(mx, v[i].y);
        if (act[i] & 4u) mx = fmaxf(mx, v[i].z);
        if (act[i] & 8u) mx = fmaxf(mx, v[i].w);
    }
    mx = warp_max(mx);
    ok = __all_sync(0xffffffffu, ok);
    any = __any_sync(0xffffffffu, any != 0u);
    if (!ok || !any) {
        if (lane == 0) kstatus_set(status, FE2O3_KSTATUS_NONFINITE);
        return;
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        v[i].x = (act[i] & 1u) ? expf(v[i].x - mx) : 0.f;
        v[i].y = (act[i] & 2u) ? expf(v[i].y - mx) : 0.f;
        v[i].z = (act[i] & 4u) ? expf(v[i].z - mx) : 0.f;
        v[i].w = (act[i] & 8u) ? expf(v[i].w - mx) : 0.f;
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;  // one IEEE division per row
    float4 *dst = reinterpret_cast<float4 *>(out + (uint64_t)row * cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const uint32_t idx = i * 32 + lane;
        if (idx < nvec) {
            float4 r;
            r.x = v[i].x * inv;
            r.y = v[i].y * inv;
            r.z = v[i].z * inv;
            r.w = v[i].w * inv;
            __stcs(dst + idx, r);
        }
    }
}

// One 256-thread block per row, up to 4096 columns, scalar accesses.
constexpr int kBlockRowThreads = 256;
constexpr int kBlockRowItems = 16;

__global__ void __launch_bounds__(kBlockRowThreads)
row_softmax_block_kernel(const float *__restrict__ in, float *__restrict__ out, const uint8_t *__restrict__ mask,
                         uint32_t rows, uint32_t cols, uint32_t *status) {
    __shared__ float red[kBlockRowThreads / 32];
    __shared__ int flags[2];
    const uint32_t row = blockIdx.x;
    if (row >= rows) return;
    const float *src = in + (uint64_t)row * cols;
    const uint8_t *msk = mask ? mask + (uint64_t)row * cols : nullptr;
    float v[kBlockRowItems];
    bool on[kBlockRowItems];
    if (threadIdx.x == 0) { flags[0] = 1; flags[1] = 0; }
    __syncthreads();
    bool ok = true, any = false;
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kBlockRowItems; ++i) {
        const uint32_t c = i * kBlockRowThreads + threadIdx.x;
        on[i] = false;
        v[i] = 0.f;
        if (c < cols) {
            v[i] = src[c];
            ok = ok && isfinite(v[i]);
            on[i] = msk ? (msk[c] != 0) : true;
            if (on[i]) { mx = fmaxf(mx, v[i]); any = true; }
        }
    }
    if (!ok) atomicExch(&flags[0], 0);
    if (any) atomicExch(&flags[1], 1);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (!flags[0] || !flags[1]) {
        if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_NONFINITE);
        return;
    }
    mx = red[0];
#pragma unroll
    for (int w = 1; w < kBlockRowThreads / 32; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kBlockRowItems; ++i) {
        v[i] = on[i] ? expf(v[i] - mx) : 0.f;
        sum += v[i];
    }
    sum = warp_sum(sum);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w = 0; w < kBlockRowThreads / 32; ++w) sum += red[w];
    float *dst = out + (uint64_t)row * cols;
#pragma unroll
    for (int i = 0; i < kBlockRowItems; ++i) {
        const uint32_t c = i * kBlockRowThreads + threadIdx.x;
        if (c < cols) dst[c] = on[i] ? v[i] / sum : 0.0f;
    }
}

template <int NV>
void launch_warp(const fe2o3_row_softmax_v1_args *a, cudaStream_t s, uint32_t grid, uint32_t *status) {
    const float *in = reinterpret_cast<const float *>(a->input.ptr);
    float *out = reinterpret_cast<float *>(a->output.ptr);
    const uint8_t *mask = reinterpret_cast<const uint8_t *>(a->mask.ptr);
    if (mask)
        row_softmax_warp_kernel<NV, true><<<grid, kWarpsPerBlock * 32, 0, s>>>(in, out, mask, a->rows, a->cols, status);
    else
        row_softmax_warp_kernel<NV, false><<<grid, kWarpsPerBlock * 32, 0, s>>>(in, out, mask, a->rows, a->cols, status);
}

}  // namespace

int32_t launch_row_softmax(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_row_softmax_v1_args *a = static_cast<const fe2o3_row_softmax_v1_args *>(args);
    const bool fast = a->cols <= 1024 && (a->cols & 3u) == 0 && ((a->input.ptr | a->output.ptr) & 15u) == 0 &&
                      (a->mask.ptr & 3u) == 0;
    uint32_t grid = fast ? ceil_div_u32(a->rows, kWarpsPerBlock) : a->rows;
    uint32_t block = fast ? kWarpsPerBlock * 32 : kBlockRowThreads;
    if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {block, 1, 1}, 0, 1};
    if (plan_only || a->rows == 0) return FE2O3_OK;
    if (fast) {
        const uint32_t nv = ceil_div_u32(a->cols, 128);
        switch (nv) {
            case 1: launch_warp<1>(a, s, grid, ctx->status_word); break;
            case 2: launch_warp<2>(a, s, grid, ctx->status_word); break;
            case 3: case 4: launch_warp<4>(a, s, grid, ctx->status_word); break;
            default: launch_warp<8>(a, s, grid, ctx->status_word); break;
        }
    } else {
        row_softmax_block_kernel<<<grid, kBlockRowThreads, 0, s>>>(
            reinterpret_cast<const float *>(a->input.ptr), reinterpret_cast<float *>(a->output.ptr),
            reinterpret_cast<const uint8_t *>(a->mask.ptr), a->rows, a->cols, ctx->status_word);
    }
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "row_softmax_v1");
}

static Fe2o3KernelRegistration reg_softmax("row_softmax_v1", reinterpret_cast<const void *>(row_softmax_warp_kernel<8, false>));
