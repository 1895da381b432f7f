// Expert-parallel exchange for the MoE layer over peer memory (NVLink).
//
// The reference has no multi-device path; this is the B200 design for the
// expert-parallel layout.  Every rank owns tokens/world tokens and
// experts/world experts.  Instead of a host-driven all-to-all, rows move by
// plain peer stores issued from the kernels that produce them, and ranks
// synchronise through monotonically increasing epoch flags in peer-visible
// memory (layout: FE2O3_EP_FLAG_* in common.cuh):
//
//   DISPATCH  publish this rank's admitted per-expert route counts to every
//             rank, wait for everybody's counts, derive where this rank's rows
//             start in each owner's receive buffer (local-expert major, source
//             rank minor: every expert's rows are one contiguous segment),
//             copy x rows straight from the token array into the owners'
//             receive buffers together with a (route id, home rank) record per
//             row (compaction and dispatch in one pass), then raise "rows
//             complete" on every rank.
//   expert FFN  (gemm_tc.cu) the first grouped GEMM waits for "rows complete"
//             per source inside the kernel; the second stores each output row
//             into the home rank's return buffer from its epilogue and raises
//             "outputs ready" everywhere when its last tile has been stored.
//   COMBINE   wait for "outputs ready" from every rank, then combine each
//             token's two rows from the local return buffer in rank order (the
//             arithmetic of examples/moe_expert_v1/src/kernel.rs:104-157) and
//             advance the pass counter.
//
// Flags compare against an epoch that grows by one per layer pass, so nothing is
// ever reset.  Buffer reuse needs no further flags: a rank starts the dispatch
// of pass p+1 only after its combine of pass p, which has seen "outputs ready"
// of pass p from EVERY rank, i.e. every rank has finished reading its receive
// buffers and counts of pass p; and a rank's return buffer is written in pass
// p+1 only with rows that this rank itself dispatched after that combine.
// Every wait is bounded and records FE2O3_KSTATUS_WAIT_EXPIRED instead of
// hanging; a block whose wait ran out still takes part in the arrival counting,
// so the counters are re-armed for the next pass.  One rank per GPU.
#include "common.cuh"

namespace {

constexpr uint32_t kDrop = 0xffffffffu;
constexpr int kThreads = 256;
constexpr uint32_t kFailedTicket = 0x10001u;   // arrival of a block whose wait expired (high half marks the failure)

// the pass number: from the device counter when one is given, else the scalar in the argument block
__device__ __forceinline__ uint32_t current_epoch(const fe2o3_moe_ep_exchange_v1_args &a) {
    return a.epoch_counter.len ? __ldcg(reinterpret_cast<const uint32_t *>(a.epoch_counter.ptr)) + 1u : a.epoch;
}

__global__ void __launch_bounds__(kThreads)
moe_ep_dispatch_kernel(fe2o3_moe_ep_exchange_v1_args a, uint32_t *status) {
    __shared__ uint32_t s_counts[32 * 32];   // [world][experts], world * experts <= 1024
    __shared__ uint32_t s_base[32];          // first row of this rank's segment for expert e on e's owner
    __shared__ uint32_t s_off[33];           // local expert_offsets
    __shared__ bool s_last, s_clean;
    const uint32_t E = a.experts, W = a.world, me = a.rank, per = E / W;
    const uint32_t epoch = current_epoch(a);
    const uint32_t limit = a.spin_limit ? a.spin_limit : FE2O3_EP_DEFAULT_SPIN;
    const uint64_t *peer_counts = reinterpret_cast<const uint64_t *>(a.peer_counts.ptr);
    const uint64_t *peer_flags = reinterpret_cast<const uint64_t *>(a.peer_flags.ptr);
    const uint64_t *peer_recv = reinterpret_cast<const uint64_t *>(a.peer_recv_x.ptr);
    const uint64_t *peer_meta = reinterpret_cast<const uint64_t *>(a.peer_recv_meta.ptr);
    uint32_t *my_flags = reinterpret_cast<uint32_t *>(peer_flags[me]);
    const uint32_t *my_counts = reinterpret_cast<const uint32_t *>(peer_counts[me]);

    // routing that reported a fault (non-finite logits) leaves no table to dispatch: the pass is void
    const bool dead = status && __ldcg(status) != 0u;
    if (blockIdx.x == 0 && threadIdx.x == 0) ep_trace(my_flags, FE2O3_EP_T_DISPATCH_BEGIN);
    if (blockIdx.x == 0 && !dead) {
        // publish this rank's admitted counts into every rank's table, then the flag
        const uint32_t *admitted = reinterpret_cast<const uint32_t *>(a.admitted_counts.ptr);
        for (uint32_t i = threadIdx.x; i < W * E; i += kThreads) {
            const uint32_t p = i / E, e = i % E;
            reinterpret_cast<uint32_t *>(peer_counts[p])[me * E + e] = admitted[e];
        }
        __threadfence_system();
        __syncthreads();
        for (uint32_t p = threadIdx.x; p < W; p += kThreads)
            st_release_sys(reinterpret_cast<uint32_t *>(peer_flags[p]) + FE2O3_EP_FLAG_COUNTS(W) + me, epoch);
    }
    if (a.logits.len && !dead) {
        // Route weights of this rank's tokens, one token per thread of the grid, computed while the counts
        // of the other ranks are still on their way (the combine phase reads them).
        const float *logits = reinterpret_cast<const float *>(a.logits.ptr);
        const uint32_t *top2 = reinterpret_cast<const uint32_t *>(a.top2_experts.ptr);
        float *weights = reinterpret_cast<float *>(a.route_weights.ptr);
        for (uint32_t t = blockIdx.x * kThreads + threadIdx.x; t < a.tokens; t += gridDim.x * kThreads) {
            const uint32_t e0 = top2[2ull * t], e1 = top2[2ull * t + 1];
            if (e0 >= E || e1 >= E) { kstatus_set(status, FE2O3_KSTATUS_SLOT_RANGE); continue; }
            float w0, w1;
            route_weight_pair(logits[(uint64_t)t * E + e0], logits[(uint64_t)t * E + e1], w0, w1);
            weights[2ull * t] = w0;
            weights[2ull * t + 1] = w1;
        }
    }
    // every block waits for the counts of every source (thread s polls source s: local memory)
    int ok = dead ? 0 : (threadIdx.x < W ? (flag_wait(my_flags + FE2O3_EP_FLAG_COUNTS(W) + threadIdx.x, epoch, limit) ? 1 : 0) : 1);
    ok = __syncthreads_and(ok);
    if (blockIdx.x == 0 && threadIdx.x == 0) ep_trace(my_flags, FE2O3_EP_T_COUNTS_HERE);
    if (ok) {
        for (uint32_t i = threadIdx.x; i < W * E; i += kThreads) s_counts[i] = __ldcg(my_counts + i);
        for (uint32_t i = threadIdx.x; i <= E; i += kThreads)
            s_off[i] = reinterpret_cast<const uint32_t *>(a.expert_offsets.ptr)[i];
        __syncthreads();
        if (threadIdx.x < E) {
            // on expert e's owner: whole segments of the owner's earlier experts, then the rows of earlier sources
            const uint32_t e = threadIdx.x, d = e / per, le = e % per;
            uint32_t base = 0;
            for (uint32_t l2 = 0; l2 < le; ++l2)
                for (uint32_t s = 0; s < W; ++s) base += s_counts[s * E + d * per + l2];
            for (uint32_t s = 0; s < me; ++s) base += s_counts[s * E + e];
            s_base[e] = base;
        }
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            // row partition of what this rank receives: pair (local expert, source)
            uint32_t *pair_offsets = reinterpret_cast<uint32_t *>(a.pair_offsets.ptr);
            uint32_t run = 0;
            pair_offsets[0] = 0;
            for (uint32_t le = 0; le < per; ++le)
                for (uint32_t s = 0; s < W; ++s) {
                    run += s_counts[s * E + me * per + le];
                    // a table that overruns the receive buffer is cut off: the FFN must never index past it
                    pair_offsets[le * W + s + 1] = run < a.max_rows ? run : a.max_rows;
                }
            if (run > a.max_rows) kstatus_set(status, FE2O3_KSTATUS_SLOT_RANGE);
        }
        __syncthreads();

        // rows: one warp per accepted local slot; a lane keeps up to eight 16-byte loads in flight before the peer stores
        const uint32_t accepted = s_off[E];
        const uint32_t *perm = reinterpret_cast<const uint32_t *>(a.permutation.ptr);
        const uint32_t vec_per_row = a.d_model / 8;
        const uint4 *x = reinterpret_cast<const uint4 *>(a.x.ptr);
        const uint32_t lane = threadIdx.x & 31;
        const uint32_t gwarp = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5), nwarps = gridDim.x * (kThreads / 32);
        for (uint32_t slot = gwarp; slot < accepted; slot += nwarps) {
            // the slot's expert = number of expert segments that end at or before it
            const uint32_t e = __popc(__ballot_sync(0xffffffffu, lane < E && slot >= s_off[lane + 1]));
            const uint32_t route = perm[slot];
            if (e >= E || route == kDrop || (route >> 1) >= a.tokens) {
                if (lane == 0) kstatus_set(status, FE2O3_KSTATUS_SLOT_RANGE);
                continue;
            }
            const uint32_t dst_rank = e / per;
            const uint32_t dst_row = s_base[e] + (slot - s_off[e]);
            if (dst_row >= a.max_rows) {
                if (lane == 0) kstatus_set(status, FE2O3_KSTATUS_SLOT_RANGE);
                continue;
            }
            if (lane == 0) reinterpret_cast<uint2 *>(peer_meta[dst_rank])[dst_row] = make_uint2(route, me);
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
    } else if (threadIdx.x == 0) {
        kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
    }
    // all of this block's rows are written; the last block to arrive raises "rows complete" everywhere,
    // unless some block's wait ran out (the pass is void then, and the peers' waits expire in turn)
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t old = atomicAdd(my_flags + FE2O3_EP_COUNTER_DISPATCH(W), ok ? 1u : kFailedTicket);
        s_last = (old & 0xffffu) == gridDim.x - 1;
        s_clean = ok && (old >> 16) == 0;
        if (s_last) atomicExch(my_flags + FE2O3_EP_COUNTER_DISPATCH(W), 0u);   // re-arm for the next pass
    }
    __syncthreads();
    if (s_last && s_clean) {
        __threadfence_system();
        for (uint32_t p = threadIdx.x; p < W; p += kThreads)
            st_release_sys(reinterpret_cast<uint32_t *>(peer_flags[p]) + FE2O3_EP_FLAG_ROWS(W) + me, epoch);
    }
    if (s_last && threadIdx.x == 0) ep_trace(my_flags, FE2O3_EP_T_ROWS_SENT);
}

// One block per token.  The two rows of a token were stored into this rank's return buffer, indexed by
// route id, by the ranks that own the token's experts (peer stores, visible after the acquire of the
// owners' flags; they are read past L1).
__global__ void __launch_bounds__(kThreads)
moe_ep_combine_kernel(fe2o3_moe_ep_exchange_v1_args a, uint32_t *status) {
    const uint32_t W = a.world, me = a.rank;
    const uint32_t epoch = current_epoch(a);
    const uint32_t limit = a.spin_limit ? a.spin_limit : FE2O3_EP_DEFAULT_SPIN;
    const uint64_t *peer_flags = reinterpret_cast<const uint64_t *>(a.peer_flags.ptr);
    const uint64_t *peer_ret = reinterpret_cast<const uint64_t *>(a.peer_ret.ptr);
    uint32_t *my_flags = reinterpret_cast<uint32_t *>(peer_flags[me]);
    const uint32_t t = blockIdx.x;
    if (blockIdx.x == 0 && threadIdx.x == 0) ep_trace(my_flags, FE2O3_EP_T_COMBINE_BEGIN);
    // a pass in which an earlier kernel reported a fault is void: write nothing
    const bool dead = status && __ldcg(status) != 0u;
    int ok = (!dead && threadIdx.x < W) ? (flag_wait(my_flags + FE2O3_EP_FLAG_OUTPUTS(W) + threadIdx.x, epoch, limit) ? 1 : 0) : 1;
    ok = __syncthreads_and(ok);
    if (blockIdx.x == 0 && threadIdx.x == 0) ep_trace(my_flags, FE2O3_EP_T_OUTPUTS_HERE);
    if (!ok) {
        if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
    } else if (!dead && t < a.tokens) {
        const uint32_t *inverse = reinterpret_cast<const uint32_t *>(a.inverse.ptr);
        const float *weights = reinterpret_cast<const float *>(a.route_weights.ptr);
        const uint32_t s0 = inverse[2ull * t], s1 = inverse[2ull * t + 1];
        const float w0 = weights[2ull * t], w1 = weights[2ull * t + 1];
        if (!isfinite(w0) || !isfinite(w1) || w0 < 0.f || w1 < 0.f || __fadd_rn(w0, w1) != 1.0f) {
            if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_WEIGHTS);
        } else {
            const uint32_t nv = a.d_model / 4;
            const float4 *ret = reinterpret_cast<const float4 *>(peer_ret[me]);
            const float4 *p0 = s0 != kDrop ? ret + (2ull * t) * nv : nullptr;        // a dropped route contributes nothing
            const float4 *p1 = s1 != kDrop ? ret + (2ull * t + 1) * nv : nullptr;
            float4 *dst = reinterpret_cast<float4 *>(a.combined_output.ptr) + (uint64_t)t * nv;
            constexpr int U = 2;
            for (uint32_t i0 = threadIdx.x; i0 < nv; i0 += kThreads * U) {
                float4 v0[U], v1[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const uint32_t i = i0 + u * kThreads;
                    v0[u] = (p0 && i < nv) ? __ldcg(p0 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    v1[u] = (p1 && i < nv) ? __ldcg(p1 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
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
                    __stcs(dst + i, acc);
                }
            }
        }
    }
    // the last block to finish advances the pass counter (all reads of this pass's flags are done)
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t old = atomicAdd(my_flags + FE2O3_EP_COUNTER_COMBINE(W), 1u);
        if (old == gridDim.x - 1) {
            ep_trace(my_flags, FE2O3_EP_T_COMBINE_END);
            atomicExch(my_flags + FE2O3_EP_COUNTER_COMBINE(W), 0u);
            if (a.epoch_counter.len) *reinterpret_cast<uint32_t *>(a.epoch_counter.ptr) += 1u;
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
        case FE2O3_MOE_EP_COMBINE: {
            const uint32_t grid = a->tokens ? a->tokens : 1u;   // a rank without tokens still advances its pass counter
            if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {kThreads, 1, 1}, 0, 1};
            if (plan_only) return FE2O3_OK;
            moe_ep_combine_kernel<<<grid, kThreads, 0, s>>>(*a, ctx->status_word);
            break;
        }
        default:
            fe2o3_set_error("unknown exchange phase %u", a->phase);
            return FE2O3_ERR_INVALID_ARGUMENT;
    }
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "moe_ep_exchange_v1");
}
