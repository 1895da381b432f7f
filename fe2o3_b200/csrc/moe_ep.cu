// Expert-parallel exchange for the MoE layer over peer memory (NVLink).
//
// The reference has no multi-device path; this is the B200 design for the
// expert-parallel layout.  Every rank owns tokens/world tokens and
// experts/world experts.  Instead of a host-driven all-to-all, the kernels
// below move rows with plain peer stores and loads and synchronise with
// monotonically increasing epoch flags in peer-visible memory:
//
//   DISPATCH  publish this rank's per-expert route counts to every rank, wait
//             for everybody's counts, derive where this rank's rows start in each
//             destination's receive buffer (source-rank major, local expert
//             minor), copy x rows straight from the token array into the
//             destinations' receive buffers (compaction and dispatch in one
//             pass), then raise the "rows complete" flag on every rank.
//   WAIT_ROWS one block: wait until every source has raised "rows complete".
//   FFN_DONE  one block: raise "expert outputs ready" on every rank.
//   COMBINE   wait for "expert outputs ready" from the ranks that own this
//             token's experts, load the two expert rows from their memory and
//             combine them in rank order (the arithmetic of
//             examples/moe_expert_v1/src/kernel.rs:104-157).
//
// Flags compare against an epoch that the host increases by one per layer pass,
// so nothing is ever reset.  Buffer reuse is safe without further flags: a rank
// starts the next pass's dispatch only after its combine, which has seen every
// rank's "expert outputs ready", and a rank's FFN starts only after every
// source's "rows complete", which each source raises after its own combine of
// the previous pass.  Every wait is bounded and records
// FE2O3_KSTATUS_WAIT_EXPIRED instead of hanging.  One rank per GPU.
#include "common.cuh"

namespace {

constexpr uint32_t kDrop = 0xffffffffu;
constexpr int kThreads = 256;
constexpr uint32_t kFlagSpin = 1u << 24;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// true when flags[i] >= epoch for every i < n (bounded)
__device__ __forceinline__ bool wait_flags(const uint32_t *flags, uint32_t n, uint32_t epoch) {
    for (uint32_t i = 0; i < n; ++i) {
        uint32_t spins = 0;
        while ((int32_t)(ld_acquire_sys(flags + i) - epoch) < 0) {
            if (++spins > kFlagSpin) return false;
            __nanosleep(64);
        }
    }
    return true;
}

// the pass number: from the device counter when one is given, else the scalar in the argument block
__device__ __forceinline__ uint32_t current_epoch(const fe2o3_moe_ep_exchange_v1_args &a) {
    return a.epoch_counter.len ? __ldcg(reinterpret_cast<const uint32_t *>(a.epoch_counter.ptr)) + 1u : a.epoch;
}

__global__ void __launch_bounds__(kThreads)
moe_ep_dispatch_kernel(fe2o3_moe_ep_exchange_v1_args a, uint32_t *status) {
    __shared__ uint32_t s_counts[32 * 32];   // [world][experts], world * experts <= 1024
    __shared__ uint32_t s_base[32];          // first row of this rank's segment for expert e on e's owner
    __shared__ uint32_t s_off[33];           // local expert_offsets
    __shared__ int s_ok;
    __shared__ bool s_last;
    const uint32_t E = a.experts, W = a.world, me = a.rank, per = E / W;
    a.epoch = current_epoch(a);
    const uint64_t *peer_counts = reinterpret_cast<const uint64_t *>(a.peer_counts.ptr);
    const uint64_t *peer_flags = reinterpret_cast<const uint64_t *>(a.peer_flags.ptr);
    const uint64_t *peer_recv = reinterpret_cast<const uint64_t *>(a.peer_recv_x.ptr);
    uint32_t *my_flags = reinterpret_cast<uint32_t *>(peer_flags[me]);   // [3][W] + counter at [3*W]
    const uint32_t *my_counts = reinterpret_cast<const uint32_t *>(peer_counts[me]);

    if (blockIdx.x == 0) {
        // publish this rank's requested counts into every rank's table, then the flag
        const uint32_t *requested = reinterpret_cast<const uint32_t *>(a.requested_counts.ptr);
        for (uint32_t i = threadIdx.x; i < W * E; i += kThreads) {
            const uint32_t p = i / E, e = i % E;
            reinterpret_cast<uint32_t *>(peer_counts[p])[me * E + e] = requested[e];
        }
        __threadfence_system();
        __syncthreads();
        for (uint32_t p = threadIdx.x; p < W; p += kThreads)
            st_release_sys(reinterpret_cast<uint32_t *>(peer_flags[p]) + 0 * W + me, a.epoch);
    }
    if (threadIdx.x == 0) s_ok = wait_flags(my_flags + 0 * W, W, a.epoch) ? 1 : 0;
    __syncthreads();
    if (!s_ok) {
        if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
        return;
    }
    for (uint32_t i = threadIdx.x; i < W * E; i += kThreads) s_counts[i] = __ldcg(my_counts + i);
    for (uint32_t i = threadIdx.x; i <= E; i += kThreads) s_off[i] = reinterpret_cast<const uint32_t *>(a.expert_offsets.ptr)[i];
    __syncthreads();
    if (threadIdx.x < E) {
        // rows on expert e's owner arrive source-major, local-expert minor
        const uint32_t e = threadIdx.x, d = e / per, le = e % per;
        uint32_t base = 0;
        for (uint32_t s = 0; s < me; ++s)
            for (uint32_t l2 = 0; l2 < per; ++l2) base += s_counts[s * E + d * per + l2];
        for (uint32_t l2 = 0; l2 < le; ++l2) base += s_counts[me * E + d * per + l2];
        s_base[e] = base;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        // row partition of what this rank receives: group g = source * per + local expert
        uint32_t *group_offsets = reinterpret_cast<uint32_t *>(a.group_offsets.ptr);
        uint32_t run = 0;
        group_offsets[0] = 0;
        for (uint32_t s = 0; s < W; ++s)
            for (uint32_t le = 0; le < per; ++le) {
                run += s_counts[s * E + me * per + le];
                group_offsets[s * per + le + 1] = run;
            }
        if (run > a.max_rows) kstatus_set(status, FE2O3_KSTATUS_SLOT_RANGE);
    }
    __syncthreads();

    // rows: one block copies one accepted local slot per iteration (16 bytes per thread per pass)
    const uint32_t accepted = s_off[E];
    const uint32_t *perm = reinterpret_cast<const uint32_t *>(a.permutation.ptr);
    uint32_t *remote_rows = reinterpret_cast<uint32_t *>(a.remote_rows.ptr);
    const uint32_t vec_per_row = a.d_model / 8;
    const uint4 *x = reinterpret_cast<const uint4 *>(a.x.ptr);
    // one warp per row; a lane keeps up to eight 16-byte loads in flight before the peer stores
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t gwarp = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5), nwarps = gridDim.x * (kThreads / 32);
    for (uint32_t slot = gwarp; slot < accepted; slot += nwarps) {
        uint32_t e = 0;
        while (e + 1 < E && slot >= s_off[e + 1]) ++e;
        const uint32_t route = perm[slot];
        const uint32_t dst_rank = e / per;
        const uint32_t dst_row = s_base[e] + (slot - s_off[e]);
        if (route == kDrop || (route >> 1) >= a.tokens || dst_row >= a.max_rows) {
            if (lane == 0) kstatus_set(status, FE2O3_KSTATUS_SLOT_RANGE);
            continue;
        }
        if (lane == 0) remote_rows[slot] = dst_row;
        const uint4 *src = x + (uint64_t)(route >> 1) * vec_per_row;
        uint4 *dst = reinterpret_cast<uint4 *>(peer_recv[dst_rank]) + (uint64_t)dst_row * vec_per_row;
        for (uint32_t i0 = lane; i0 < vec_per_row; i0 += 32 * 8) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (i0 + 32 * u < vec_per_row) v[u] = __ldg(src + i0 + 32 * u);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (i0 + 32 * u < vec_per_row) dst[i0 + 32 * u] = v[u];
        }
    }
    // all of this rank's rows are written: the last block raises "rows complete" everywhere
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(my_flags + 3 * W, 1u) == gridDim.x - 1;
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        for (uint32_t p = threadIdx.x; p < W; p += kThreads)
            st_release_sys(reinterpret_cast<uint32_t *>(peer_flags[p]) + 1 * W + me, a.epoch);
        if (threadIdx.x == 0) my_flags[3 * W] = 0u;
    }
}

__global__ void moe_ep_flag_kernel(fe2o3_moe_ep_exchange_v1_args a, uint32_t *status) {
    const uint32_t W = a.world, me = a.rank;
    if (a.phase == FE2O3_MOE_EP_ADVANCE) {
        if (threadIdx.x == 0 && a.epoch_counter.len) *reinterpret_cast<uint32_t *>(a.epoch_counter.ptr) += 1u;
        return;
    }
    a.epoch = current_epoch(a);
    const uint64_t *peer_flags = reinterpret_cast<const uint64_t *>(a.peer_flags.ptr);
    if (a.phase == FE2O3_MOE_EP_WAIT_ROWS) {
        if (threadIdx.x == 0 && !wait_flags(reinterpret_cast<uint32_t *>(peer_flags[me]) + 1 * W, W, a.epoch))
            kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
    } else {  // FE2O3_MOE_EP_FFN_DONE: this rank's expert outputs are in memory
        __threadfence_system();
        for (uint32_t p = threadIdx.x; p < W; p += blockDim.x)
            st_release_sys(reinterpret_cast<uint32_t *>(peer_flags[p]) + 2 * W + me, a.epoch);
    }
}

__global__ void __launch_bounds__(kThreads)
moe_ep_combine_kernel(fe2o3_moe_ep_exchange_v1_args a, uint32_t *status) {
    __shared__ int s_ok;
    const uint32_t W = a.world, me = a.rank, per = a.experts / W;
    a.epoch = current_epoch(a);
    const uint64_t *peer_flags = reinterpret_cast<const uint64_t *>(a.peer_flags.ptr);
    const uint64_t *peer_out = reinterpret_cast<const uint64_t *>(a.peer_ffn_out.ptr);
    const uint32_t t = blockIdx.x;
    if (t >= a.tokens) return;
    const uint32_t *top2 = reinterpret_cast<const uint32_t *>(a.top2_experts.ptr);
    const uint32_t *inverse = reinterpret_cast<const uint32_t *>(a.inverse.ptr);
    const uint32_t *remote_rows = reinterpret_cast<const uint32_t *>(a.remote_rows.ptr);
    const float *weights = reinterpret_cast<const float *>(a.route_weights.ptr);
    const uint32_t e0 = top2[2ull * t], e1 = top2[2ull * t + 1];
    const uint32_t s0 = inverse[2ull * t], s1 = inverse[2ull * t + 1];
    const uint32_t r0 = e0 / per, r1 = e1 / per;
    if (threadIdx.x == 0) {
        const uint32_t *flags = reinterpret_cast<const uint32_t *>(peer_flags[me]) + 2 * W;
        bool ok = true;
        if (s0 != kDrop) ok = ok && wait_flags(flags + r0, 1, a.epoch);
        if (s1 != kDrop) ok = ok && wait_flags(flags + r1, 1, a.epoch);
        s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!s_ok) {
        if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
        return;
    }
    const float w0 = weights[2ull * t], w1 = weights[2ull * t + 1];
    if (!isfinite(w0) || !isfinite(w1) || w0 < 0.f || w1 < 0.f || __fadd_rn(w0, w1) != 1.0f) {
        if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_WEIGHTS);
        return;
    }
    const uint32_t nv = a.d_model / 4;
    const float4 *p0 = s0 != kDrop ? reinterpret_cast<const float4 *>(peer_out[r0]) + (uint64_t)remote_rows[s0] * nv : nullptr;
    const float4 *p1 = s1 != kDrop ? reinterpret_cast<const float4 *>(peer_out[r1]) + (uint64_t)remote_rows[s1] * nv : nullptr;
    float4 *dst = reinterpret_cast<float4 *>(a.combined_output.ptr) + (uint64_t)t * nv;
    // all of a thread's peer loads are issued before any is used (remote latency is microseconds)
    constexpr int U = 4;
    for (uint32_t i0 = threadIdx.x; i0 < nv; i0 += kThreads * U) {
        float4 v0[U], v1[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t i = i0 + u * kThreads;
            v0[u] = (p0 && i < nv) ? p0[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            v1[u] = (p1 && i < nv) ? p1[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t i = i0 + u * kThreads;
            if (i >= nv) continue;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p0) {
                acc.x = __fadd_rn(acc.x, __fmul_rn(w0, v0[u].x)); acc.y = __fadd_rn(acc.y, __fmul_rn(w0, v0[u].y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(w0, v0[u].z)); acc.w = __fadd_rn(acc.w, __fmul_rn(w0, v0[u].w));
            }
            if (p1) {
                acc.x = __fadd_rn(acc.x, __fmul_rn(w1, v1[u].x)); acc.y = __fadd_rn(acc.y, __fmul_rn(w1, v1[u].y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(w1, v1[u].z)); acc.w = __fadd_rn(acc.w, __fmul_rn(w1, v1[u].w));
            }
            dst[i] = acc;
        }
    }
}

}  // namespace

int32_t launch_moe_ep_exchange(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_moe_ep_exchange_v1_args *a = static_cast<const fe2o3_moe_ep_exchange_v1_args *>(args);
    switch (a->phase) {
        case FE2O3_MOE_EP_DISPATCH: {
            const uint32_t grid = (uint32_t)ctx->sm_count * 4u;
            if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {kThreads, 1, 1}, 0, 1};
            if (plan_only) return FE2O3_OK;
            moe_ep_dispatch_kernel<<<grid, kThreads, 0, s>>>(*a, ctx->status_word);
            break;
        }
        case FE2O3_MOE_EP_WAIT_ROWS:
        case FE2O3_MOE_EP_FFN_DONE:
        case FE2O3_MOE_EP_ADVANCE:
            if (geo) *geo = fe2o3_geometry{{1, 1, 1}, {32, 1, 1}, 0, 1};
            if (plan_only) return FE2O3_OK;
            moe_ep_flag_kernel<<<1, 32, 0, s>>>(*a, ctx->status_word);
            break;
        case FE2O3_MOE_EP_COMBINE:
            if (geo) *geo = fe2o3_geometry{{a->tokens, 1, 1}, {kThreads, 1, 1}, 0, 1};
            if (plan_only || a->tokens == 0) return FE2O3_OK;
            moe_ep_combine_kernel<<<a->tokens, kThreads, 0, s>>>(*a, ctx->status_word);
            break;
        default:
            fe2o3_set_error("unknown exchange phase %u", a->phase);
            return FE2O3_ERR_INVALID_ARGUMENT;
    }
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "moe_ep_exchange_v1");
}
