// CUDA-core attention: the reference kernel's per-key online recurrence
// (examples/flash_attention_v1/src/kernel.rs:56-113: m' = max(m, s),
// p = exp(m - m'), c = exp(s - m'), l = l*p + c, acc = acc*p + v*c, out = acc/l,
// first key initialises m = s, l = 1, acc = v) for any [B][H][S][D] shape, f32
// or bf16 inputs, causal or not.  One warp owns one query row; lanes split the
// head dimension.  It serves the fixed f32 B1/H1/N8/D16 profile and every shape
// the tensor-core kernel does not admit.
#include "common.cuh"

namespace {

constexpr int kMaxPerLane = 8;  // head_dim <= 256

template <typename T>
__device__ __forceinline__ float ld(const T *p, uint64_t i);
template <>
__device__ __forceinline__ float ld<float>(const float *p, uint64_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ld<uint16_t>(const uint16_t *p, uint64_t i) { return bf16_bits_to_f32(p[i]); }

template <typename T>
__global__ void __launch_bounds__(128)
attention_simt_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                      float *__restrict__ out, uint32_t bh, uint32_t seq, uint32_t dim, float scale, uint32_t causal,
                      uint32_t *status) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t row = (uint64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= (uint64_t)bh * seq) return;
    const uint32_t head = (uint32_t)(row / seq), qr = (uint32_t)(row % seq);
    const uint64_t base = (uint64_t)head * seq * dim;
    float qv[kMaxPerLane], acc[kMaxPerLane];
    bool finite = true;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const uint32_t f = lane + 32 * i;
        qv[i] = f < dim ? ld<T>(q, base + (uint64_t)qr * dim + f) : 0.0f;
        acc[i] = 0.0f;
        finite = finite && isfinite(qv[i]);
    }
    float m = 0.0f, l = 0.0f;
    const uint32_t keys = causal ? qr + 1 : seq;
    for (uint32_t kr = 0; kr < keys; ++kr) {
        float part = 0.0f;
        float vv[kMaxPerLane];
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
            const uint32_t f = lane + 32 * i;
            float kv = 0.0f;
            vv[i] = 0.0f;
            if (f < dim) {
                kv = ld<T>(k, base + (uint64_t)kr * dim + f);
                vv[i] = ld<T>(v, base + (uint64_t)kr * dim + f);
            }
            finite = finite && isfinite(kv) && isfinite(vv[i]);
            part = fmaf(qv[i], kv, part);
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        const float s = part * scale;
        if (kr == 0) {
            m = s;
            l = 1.0f;
#pragma unroll
            for (int i = 0; i < kMaxPerLane; ++i) acc[i] = vv[i];
            continue;
        }
        const float nm = fmaxf(m, s);
        const float pw = expf(m - nm), cw = expf(s - nm);
        l = l * pw + cw;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) acc[i] = acc[i] * pw + vv[i] * cw;
        m = nm;
    }
    finite = __all_sync(0xffffffffu, finite && isfinite(l) && l > 0.0f);
    if (!finite) {  // finite-input policy: leave the row unwritten, record a status word
        if (lane == 0) kstatus_set(status, FE2O3_KSTATUS_NONFINITE);
        return;
    }
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const uint32_t f = lane + 32 * i;
        if (f < dim) out[base + (uint64_t)qr * dim + f] = acc[i] / l;
    }
}

}  // namespace

int32_t launch_attention_simt(fe2o3_ctx *ctx, cudaStream_t s, const fe2o3_flash_attention_v1_args *a,
                              fe2o3_geometry *geo, bool plan_only) {
    const uint64_t rows = (uint64_t)a->batch * a->heads * a->seq;
    const uint32_t grid = ceil_div_u32(rows, 4);
    if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {128, 1, 1}, 0, 1};
    if (plan_only || rows == 0) return FE2O3_OK;
    float *out = reinterpret_cast<float *>(a->output.ptr);
    if (a->input_dtype == FE2O3_DTYPE_F32)
        attention_simt_kernel<float><<<grid, 128, 0, s>>>(
            reinterpret_cast<const float *>(a->q.ptr), reinterpret_cast<const float *>(a->k.ptr),
            reinterpret_cast<const float *>(a->v.ptr), out, a->batch * a->heads, a->seq, a->dim, a->scale, a->causal,
            ctx->status_word);
    else
        attention_simt_kernel<uint16_t><<<grid, 128, 0, s>>>(
            reinterpret_cast<const uint16_t *>(a->q.ptr), reinterpret_cast<const uint16_t *>(a->k.ptr),
            reinterpret_cast<const uint16_t *>(a->v.ptr), out, a->batch * a->heads, a->seq, a->dim, a->scale,
            a->causal, ctx->status_word);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "flash_attention_v1(simt)");
}
