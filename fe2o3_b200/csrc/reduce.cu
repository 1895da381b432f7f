// Masked u32 reductions and the small wave64 / workgroup collectives.
//
// The reference expresses these as wave64 (64-lane) and 256-thread workgroup
// collectives on gfx942 (crates/fe2o3-device/src/collective.rs:187-229,391-501).
// On sm_100a a warp has 32 lanes, so a "wave64" is two warps and the trees are
// warp shuffles followed by a shared-memory stage.  u32 wrapping addition is
// associative and commutative, so any tree gives the reference's bits.
#include "common.cuh"

namespace {

constexpr int kReduceThreads = 512;

__device__ __forceinline__ uint32_t warp_sum_u32(uint32_t v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ uint32_t block_sum_u32(uint32_t v, uint32_t *smem /* >= 32 */) {
    v = warp_sum_u32(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    uint32_t total = 0;
    if (warp == 0) {
        total = lane < nwarps ? smem[lane] : 0u;
        total = warp_sum_u32(total);
    }
    return total;  // valid in warp 0
}

__device__ __forceinline__ uint4 ldg_stream_u4(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t masked4(uint4 v, uint4 a) {
    return (a.x ? v.x : 0u) + (a.y ? v.y : 0u) + (a.z ? v.z : 0u) + (a.w ? v.w : 0u);
}

// Final stage shared by both forms: publish the block partial; the last block
// to arrive adds the partials in index order, writes the single output and
// re-arms the counter for the next launch.
__device__ __forceinline__ void grid_finish(uint32_t block_total, uint32_t *partials, uint32_t *counter,
                                            uint32_t *out, uint32_t *smem) {
    __shared__ bool is_last;
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = block_total;
        __threadfence();
        uint32_t ticket = atomicAdd(counter, 1u);
        is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    uint32_t acc = 0;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += blockDim.x) acc += __ldcg(partials + i);
    __syncthreads();
    acc = block_sum_u32(acc, smem);
    if (threadIdx.x == 0) {
        *out = acc;
        *counter = 0u;
    }
}

// values/active as u32 flags: 8 algorithmic bytes per element.
__global__ void __launch_bounds__(kReduceThreads)
masked_reduce_u32_kernel(fe2o3_masked_reduce_u32_args args, uint32_t *partials, uint32_t *counter,
                         uint32_t *status) {
    __shared__ uint32_t smem[32];
    if (args.values.len != args.active.len || args.output.len != 1) {
        if (blockIdx.x == 0 && threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_LENGTH);
        return;
    }
    const uint64_t n = args.values.len;
    const uint32_t *values = reinterpret_cast<const uint32_t *>(args.values.ptr);
    const uint32_t *active = reinterpret_cast<const uint32_t *>(args.active.ptr);
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;
    uint32_t acc = 0;
    const bool vec_ok = ((args.values.ptr | args.active.ptr) & 15u) == 0;
    uint64_t done = 0;
    if (vec_ok) {
        const uint64_t n4 = n >> 2;
        const uint4 *v4 = reinterpret_cast<const uint4 *>(values);
        const uint4 *a4 = reinterpret_cast<const uint4 *>(active);
        uint64_t i = tid;
        // four independent 128-bit load pairs in flight per thread
        for (; i + 3 * nthreads < n4; i += 4 * nthreads) {
            uint4 v0 = ldg_stream_u4(v4 + i), a0 = ldg_stream_u4(a4 + i);
            uint4 v1 = ldg_stream_u4(v4 + i + nthreads), a1 = ldg_stream_u4(a4 + i + nthreads);
            uint4 v2 = ldg_stream_u4(v4 + i + 2 * nthreads), a2 = ldg_stream_u4(a4 + i + 2 * nthreads);
            uint4 v3 = ldg_stream_u4(v4 + i + 3 * nthreads), a3 = ldg_stream_u4(a4 + i + 3 * nthreads);
            acc += masked4(v0, a0) + masked4(v1, a1) + masked4(v2, a2) + masked4(v3, a3);
        }
        for (; i < n4; i += nthreads) acc += masked4(ldg_stream_u4(v4 + i), ldg_stream_u4(a4 + i));
        done = n4 << 2;
    }
    for (uint64_t i = done + tid; i < n; i += nthreads)
        if (active[i] != 0u) acc += values[i];
    uint32_t total = block_sum_u32(acc, smem);
    __syncthreads();
    grid_finish(total, partials, counter, reinterpret_cast<uint32_t *>(args.output.ptr), smem);
}

// Packed activity: bit (i % 64) of mask[i / 64]; 4 + 1/8 algorithmic bytes per
// element.  One thread handles 64-element words' quarter: a warp covers
// 32 x 4 = 128 consecutive values per load, i.e. two mask words.
__global__ void __launch_bounds__(kReduceThreads)
masked_reduce_u32_packed_kernel(fe2o3_masked_reduce_u32_packed_args args, uint32_t *partials,
                                uint32_t *counter, uint32_t *status) {
    __shared__ uint32_t smem[32];
    const uint64_t n = args.values.len;
    if (args.mask.len != (n + 63) / 64 || args.output.len != 1) {
        if (blockIdx.x == 0 && threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_LENGTH);
        return;
    }
    const uint32_t *values = reinterpret_cast<const uint32_t *>(args.values.ptr);
    const uint64_t *mask = reinterpret_cast<const uint64_t *>(args.mask.ptr);
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;
    uint32_t acc = 0;
    uint64_t done = 0;
    if ((args.values.ptr & 15u) == 0) {
        const uint64_t n4 = n >> 2;
        const uint4 *v4 = reinterpret_cast<const uint4 *>(values);
        uint64_t i = tid;
        for (; i + 3 * nthreads < n4; i += 4 * nthreads) {
            uint4 v[4];
            uint64_t m[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                uint64_t idx = i + u * nthreads;
                v[u] = ldg_stream_u4(v4 + idx);
                m[u] = __ldg(mask + (idx >> 4)) >> ((idx & 15u) << 2);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                acc += ((m[u] & 1u) ? v[u].x : 0u) + ((m[u] & 2u) ? v[u].y : 0u) + ((m[u] & 4u) ? v[u].z : 0u) +
                       ((m[u] & 8u) ? v[u].w : 0u);
        }
        for (; i < n4; i += nthreads) {
            uint4 v = ldg_stream_u4(v4 + i);
            uint64_t m = __ldg(mask + (i >> 4)) >> ((i & 15u) << 2);
            acc += ((m & 1u) ? v.x : 0u) + ((m & 2u) ? v.y : 0u) + ((m & 4u) ? v.z : 0u) + ((m & 8u) ? v.w : 0u);
        }
        done = n4 << 2;
    }
    for (uint64_t i = done + tid; i < n; i += nthreads)
        if ((mask[i >> 6] >> (i & 63u)) & 1ull) acc += values[i];
    uint32_t total = block_sum_u32(acc, smem);
    __syncthreads();
    grid_finish(total, partials, counter, reinterpret_cast<uint32_t *>(args.output.ptr), smem);
}

// The wave64 + workgroup256 profile: one 256-thread block per 256 elements;
// every lane receives its 64-lane segment's sum and its block's sum
// (crates/dialect-amdgcn/tests/fixtures/gfx942_wave_lds_v1_runner.cpp:76-94).
__global__ void __launch_bounds__(256)
wave_lds_v1_kernel(fe2o3_wave_lds_v1_args args, uint32_t *status) {
    __shared__ uint32_t warp_sums[8];
    const uint64_t n = args.values.len;
    if (args.active.len != n || args.wave_out.len != n || args.workgroup_out.len != n || (n % 256u) != 0) {
        if (blockIdx.x == 0 && threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_LENGTH);
        return;
    }
    const uint64_t i = (uint64_t)blockIdx.x * 256u + threadIdx.x;
    const uint32_t value = reinterpret_cast<const uint32_t *>(args.values.ptr)[i];
    const uint32_t flag = reinterpret_cast<const uint32_t *>(args.active.ptr)[i];
    uint32_t contribution = flag != 0u ? value : 0u;
    uint32_t w = warp_sum_u32(contribution);
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) warp_sums[warp] = w;
    __syncthreads();
    uint32_t wave = warp_sums[warp & ~1] + warp_sums[warp | 1];  // two warps form one 64-lane wave
    uint32_t group = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) group += warp_sums[k];
    reinterpret_cast<uint32_t *>(args.wave_out.ptr)[i] = wave;
    reinterpret_cast<uint32_t *>(args.workgroup_out.ptr)[i] = group;
}

// f32 masked wave64 reduce + inclusive/exclusive scans, one 64-thread block per
// segment, following the reference's round structure exactly: six XOR exchange
// rounds with distances 1,2,4,8,16,32 and six Hillis-Steele rounds
// (examples/wave64_collectives_v1/src/oracle.rs:150-172).
__global__ void __launch_bounds__(64)
wave64_collectives_kernel(const float *input, const uint64_t *masks, uint64_t single_mask, float *reduction,
                          float *inclusive, float *exclusive) {
    __shared__ float buf[2][64];
    const int lane = threadIdx.x;
    const uint64_t base = (uint64_t)blockIdx.x * 64u;
    const uint64_t mask = masks ? masks[blockIdx.x] : single_mask;
    const bool on = (mask >> lane) & 1ull;
    const float contribution = on ? input[base + lane] : 0.0f;

    int cur = 0;
    buf[cur][lane] = contribution;
    __syncthreads();
    for (int dist = 1; dist <= 32; dist <<= 1) {
        float v = __fadd_rn(buf[cur][lane], buf[cur][lane ^ dist]);
        buf[cur ^ 1][lane] = v;
        cur ^= 1;
        __syncthreads();
    }
    const float red = buf[cur][lane];
    __syncthreads();
    cur = 0;
    buf[cur][lane] = contribution;
    __syncthreads();
    for (int dist = 1; dist <= 32; dist <<= 1) {
        float v = buf[cur][lane];
        if (lane >= dist) v = __fadd_rn(v, buf[cur][lane - dist]);
        buf[cur ^ 1][lane] = v;
        cur ^= 1;
        __syncthreads();
    }
    const float inc = buf[cur][lane];
    const float exc = lane == 0 ? 0.0f : buf[cur][lane - 1];
    reduction[base + lane] = on ? red : 0.0f;
    inclusive[base + lane] = on ? inc : 0.0f;
    exclusive[base + lane] = on ? exc : 0.0f;
}

// i32 sum of 64 lanes through a shared-memory tree with offsets 32..1
// (crates/fe2o3-device/src/collective.rs:469-501).
__global__ void __launch_bounds__(64)
lds_publish_read_reduce_i32_kernel(fe2o3_lds_publish_read_reduce_i32_v1_args args, uint32_t *status) {
    extern __shared__ uint32_t slots[];  // exactly 64 * 4 bytes of dynamic shared memory
    if (args.values.len != 64 || args.output.len != 1 || blockDim.x != 64 || gridDim.x != 1) {
        if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_LENGTH);
        return;
    }
    const int lane = threadIdx.x;
    slots[lane] = (uint32_t) reinterpret_cast<const int32_t *>(args.values.ptr)[lane];
    __syncthreads();
    for (int off = 32; off >= 1; off >>= 1) {
        uint32_t v = 0;
        if (lane < off) v = slots[lane] + slots[lane + off];
        __syncthreads();
        if (lane < off) slots[lane] = v;
        __syncthreads();
    }
    if (lane == 0) reinterpret_cast<int32_t *>(args.output.ptr)[0] = (int32_t)slots[0];
}

// Eligible lanes add their value to one u32 with a relaxed system-scope atomic
// (examples/workgroup_sync_v1/src/scoped_atomic.rs:21-32).
__global__ void __launch_bounds__(64)
scoped_atomic_add_u32_kernel(fe2o3_scoped_atomic_add_u32_v1_args args, uint32_t *status) {
    if (args.values.len != 64 || args.eligible.len != 64 || blockDim.x != 64) {
        if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_LENGTH);
        return;
    }
    const int lane = threadIdx.x;
    if (reinterpret_cast<const uint32_t *>(args.eligible.ptr)[lane] != 0u)
        atomicAdd_system(reinterpret_cast<uint32_t *>(args.target), reinterpret_cast<const uint32_t *>(args.values.ptr)[lane]);
}

uint32_t reduce_grid(const fe2o3_ctx *ctx, uint64_t n) {
    // resident blocks: 4 x 512 threads per SM
    uint64_t want = (n / 4 + kReduceThreads - 1) / kReduceThreads;
    uint64_t cap = (uint64_t)ctx->sm_count * 4u;
    if (cap > FE2O3_REDUCE_MAX_BLOCKS) cap = FE2O3_REDUCE_MAX_BLOCKS;
    if (want < 1) want = 1;
    return (uint32_t)(want < cap ? want : cap);
}

}  // namespace

int32_t launch_masked_reduce_u32(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_masked_reduce_u32_args *a = static_cast<const fe2o3_masked_reduce_u32_args *>(args);
    uint32_t grid = reduce_grid(ctx, a->values.len);
    if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {kReduceThreads, 1, 1}, 0, 1};
    if (plan_only) return FE2O3_OK;
    masked_reduce_u32_kernel<<<grid, kReduceThreads, 0, s>>>(*a, ctx->reduce_scratch,
                                                              ctx->reduce_scratch + FE2O3_REDUCE_MAX_BLOCKS,
                                                              ctx->status_word);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "masked_reduce_u32");
}

int32_t launch_masked_reduce_u32_packed(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo,
                                        bool plan_only) {
    const fe2o3_masked_reduce_u32_packed_args *a = static_cast<const fe2o3_masked_reduce_u32_packed_args *>(args);
    uint32_t grid = reduce_grid(ctx, a->values.len);
    if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {kReduceThreads, 1, 1}, 0, 1};
    if (plan_only) return FE2O3_OK;
    masked_reduce_u32_packed_kernel<<<grid, kReduceThreads, 0, s>>>(*a, ctx->reduce_scratch,
                                                                     ctx->reduce_scratch + FE2O3_REDUCE_MAX_BLOCKS,
                                                                     ctx->status_word);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "masked_reduce_u32_packed");
}

int32_t launch_wave_lds_v1(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_wave_lds_v1_args *a = static_cast<const fe2o3_wave_lds_v1_args *>(args);
    uint32_t grid = (uint32_t)(a->values.len / 256u);
    if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {256, 1, 1}, 0, 1};
    if (plan_only || grid == 0) return FE2O3_OK;
    wave_lds_v1_kernel<<<grid, 256, 0, s>>>(*a, ctx->status_word);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "wave_lds_v1");
}

static int32_t launch_w64(cudaStream_t s, uint64_t input, uint64_t masks, uint64_t single_mask, uint64_t segments,
                          uint64_t red, uint64_t inc, uint64_t exc, fe2o3_geometry *geo, bool plan_only) {
    if (geo) *geo = fe2o3_geometry{{(uint32_t)segments, 1, 1}, {64, 1, 1}, 0, 1};
    if (plan_only || segments == 0) return FE2O3_OK;
    wave64_collectives_kernel<<<(uint32_t)segments, 64, 0, s>>>(
        reinterpret_cast<const float *>(input), reinterpret_cast<const uint64_t *>(masks), single_mask,
        reinterpret_cast<float *>(red), reinterpret_cast<float *>(inc), reinterpret_cast<float *>(exc));
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "wave64_collectives_v1");
}

int32_t launch_wave64_collectives_v1(fe2o3_ctx *, cudaStream_t s, const void *args, fe2o3_geometry *geo,
                                     bool plan_only) {
    const fe2o3_wave64_collectives_v1_args *a = static_cast<const fe2o3_wave64_collectives_v1_args *>(args);
    return launch_w64(s, a->input.ptr, 0, a->active_mask, 1, a->reduction_output.ptr, a->inclusive_output.ptr,
                      a->exclusive_output.ptr, geo, plan_only);
}

int32_t launch_wave64_collectives_segmented(fe2o3_ctx *, cudaStream_t s, const void *args, fe2o3_geometry *geo,
                                            bool plan_only) {
    const fe2o3_wave64_collectives_segmented_args *a = static_cast<const fe2o3_wave64_collectives_segmented_args *>(args);
    return launch_w64(s, a->input.ptr, a->masks.ptr, 0, a->masks.len, a->reduction_output.ptr,
                      a->inclusive_output.ptr, a->exclusive_output.ptr, geo, plan_only);
}

int32_t launch_lds_reduce_i32(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_lds_publish_read_reduce_i32_v1_args *a = static_cast<const fe2o3_lds_publish_read_reduce_i32_v1_args *>(args);
    if (geo) *geo = fe2o3_geometry{{1, 1, 1}, {64, 1, 1}, 256, 1};
    if (plan_only) return FE2O3_OK;
    lds_publish_read_reduce_i32_kernel<<<1, 64, 256, s>>>(*a, ctx->status_word);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "lds_publish_read_reduce_i32_v1");
}

int32_t launch_scoped_atomic_add(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_scoped_atomic_add_u32_v1_args *a = static_cast<const fe2o3_scoped_atomic_add_u32_v1_args *>(args);
    if (geo) *geo = fe2o3_geometry{{1, 1, 1}, {64, 1, 1}, 0, 1};
    if (plan_only) return FE2O3_OK;
    scoped_atomic_add_u32_kernel<<<1, 64, 0, s>>>(*a, ctx->status_word);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "scoped_atomic_add_u32_v1");
}

// ---- allocation-free entry point ---------------------------------------------------
// Some hosts must not call the device allocator once they are running: a process
// whose device memory is already handed out in full to another runtime's pool
// (cudaMalloc would fail), or a caller inside a section that cannot absorb the
// device-wide synchronisation an allocation or free may imply.  For them the
// masked sum is also offered with its scratch (per-block partial sums plus the
// arrival counter) in a fixed device array that every GPU loading this library
// carries until the process exits.
//
// The array's name in host code is only a host-side stand-in, not a device
// address, so the address is taken once per device with cudaGetSymbolAddress
// while that device is current and handed to the kernel as an ordinary pointer.
#define FE2O3_NOALLOC_MAX_BLOCKS 1024u
static __device__ __align__(256) uint32_t g_noalloc_scratch[FE2O3_NOALLOC_MAX_BLOCKS + 64];  // 4352 bytes

#include <mutex>

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
uint32_t *g_noalloc_ptr[kMaxDevices];
int g_noalloc_sms[kMaxDevices];
}  // namespace

extern "C" int32_t fe2o3_masked_reduce_u32_noalloc(const uint32_t *values, const uint32_t *active, uint64_t n,
                                                   uint32_t *output, void *cuda_stream) {
    if (!output || (n && (!values || !active))) {
        fe2o3_set_error("NullAddress: values, active and output must be device pointers");
        return FE2O3_ERR_NULL_ADDRESS;
    }
    if (((reinterpret_cast<uintptr_t>(values) | reinterpret_cast<uintptr_t>(active) | reinterpret_cast<uintptr_t>(output)) & 3u) != 0) {
        fe2o3_set_error("Alignment: u32 pointers must be 4-byte aligned");
        return FE2O3_ERR_ALIGNMENT;
    }
    if (n > FE2O3_NOALLOC_MAX_ELEMENTS) {
        fe2o3_set_error("UnsupportedShape: %llu elements exceed the allocation-free limit of %llu; use "
                        "fe2o3_masked_reduce_u32_prepare for larger inputs",
                        (unsigned long long)n, (unsigned long long)FE2O3_NOALLOC_MAX_ELEMENTS);
        return FE2O3_ERR_UNSUPPORTED_SHAPE;
    }
    int device = -1;
    FE2O3_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) {
        fe2o3_set_error("device index %d outside the supported range", device);
        return FE2O3_ERR_INVALID_ARGUMENT;
    }
    uint32_t *scratch;
    int sms;
    {
        // One-time set-up per device (the first call on that device does it).
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_ptr[device]) {
            void *p = nullptr;
            FE2O3_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
            int v = 0;
            FE2O3_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device));
            g_noalloc_sms[device] = v;
            g_noalloc_ptr[device] = static_cast<uint32_t *>(p);
        }
        scratch = g_noalloc_ptr[device];
        sms = g_noalloc_sms[device];
    }
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    uint64_t want = (n / 4 + kReduceThreads - 1) / kReduceThreads;
    uint64_t cap = (uint64_t)sms * 4u;
    if (cap > FE2O3_NOALLOC_MAX_BLOCKS) cap = FE2O3_NOALLOC_MAX_BLOCKS;
    if (want < 1) want = 1;
    const uint32_t grid = (uint32_t)(want < cap ? want : cap);
    uint32_t *counter = scratch + FE2O3_NOALLOC_MAX_BLOCKS;
    // The array keeps whatever the previous call left: the arrival counter must start at zero.
    FE2O3_CUDA(cudaMemsetAsync(counter, 0, sizeof(uint32_t), s));
    fe2o3_masked_reduce_u32_args a;
    a.values = fe2o3_slice{reinterpret_cast<uint64_t>(values), n};
    a.active = fe2o3_slice{reinterpret_cast<uint64_t>(active), n};
    a.output = fe2o3_slice{reinterpret_cast<uint64_t>(output), 1};
    masked_reduce_u32_kernel<<<grid, kReduceThreads, 0, s>>>(a, scratch, counter, nullptr);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "masked_reduce_u32_noalloc");
}

static Fe2o3KernelRegistration reg_reduce("masked_reduce_sum_u32", reinterpret_cast<const void *>(masked_reduce_u32_kernel));
static Fe2o3KernelRegistration reg_reduce_packed("masked_reduce_sum_u32_packed", reinterpret_cast<const void *>(masked_reduce_u32_packed_kernel));
static Fe2o3KernelRegistration reg_wave_lds("gfx942_wave_lds_v1_hw", reinterpret_cast<const void *>(wave_lds_v1_kernel));
static Fe2o3KernelRegistration reg_wave64("wave64_collectives_v1", reinterpret_cast<const void *>(wave64_collectives_kernel));
static Fe2o3KernelRegistration reg_wave64_seg("wave64_collectives_segmented", reinterpret_cast<const void *>(wave64_collectives_kernel));
static Fe2o3KernelRegistration reg_lds_i32("lds_publish_read_reduce_i32_v1", reinterpret_cast<const void *>(lds_publish_read_reduce_i32_kernel));
static Fe2o3KernelRegistration reg_atomic("scoped_atomic_add_u32_v1", reinterpret_cast<const void *>(scoped_atomic_add_u32_kernel));
