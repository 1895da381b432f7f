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
//             complete" on each rank as soon as the last row for it is stored.  The kernel
//             lets the FFN kernel start beside it (programmatic dependent launch).
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
// hanging; the arrival counters are re-armed even then (a block that gave up
// still arrives; the per-destination row counters alternate between two sets,
// each cleared a pass ahead).  One rank per GPU.
#include "common.cuh"

namespace {

constexpr uint32_t kDrop = 0xffffffffu;
constexpr int kThreads = 256;
// The dispatch kernel shares every SM with one block of the GEMM that follows it (320 threads x 168 registers,
// nearly all of the shared memory): 192 threads x 64 registers fit the register file beside it (registers go out to four warps at a time: 8 x 32 x 64 beside the 12 x 32 x 128 of the GEMM).
constexpr int kDispatchThreads = 192;
#ifndef FE2O3_DISPATCH_INFLIGHT
#define FE2O3_DISPATCH_INFLIGHT 4
#endif
constexpr int kInFlight = FE2O3_DISPATCH_INFLIGHT;   // 16-byte loads a lane issues before the matching stores

// the pass number: from the device counter when one is given, else the scalar in the argument block
__device__ __forceinline__ uint32_t current_epoch(const fe2o3_moe_ep_exchange_v1_args &a) {
    return a.epoch_counter.len ? __ldcg(reinterpret_cast<const uint32_t *>(a.epoch_counter.ptr)) + 1u : a.epoch;
}

// One block per SM, few registers and almost no shared memory: the first GEMM of the expert FFN is
// launched right behind this kernel with programmatic stream serialization and runs beside it on the same
// SMs (one GEMM block and one block of this kernel fit an SM together), computing on the rows that have
// arrived while the others still travel.  Rows go out destination by destination, this rank's own first,
// then ranks me-1, me-2, ... so that every rank receives from me+1 first, then me+2, ... which is the order
// in which its GEMM takes the tiles; "rows complete" is raised per destination as soon as the last row for
// it has been stored.
__global__ void __launch_bounds__(kDispatchThreads, 5)
moe_ep_dispatch_kernel(fe2o3_moe_ep_exchange_v1_args a, uint32_t *status) {
    launch_dependents();
    const uint32_t E = a.experts, W = a.world, me = a.rank, per = E / W;
    const uint32_t epoch = current_epoch(a);
    const uint32_t limit = a.spin_limit ? a.spin_limit : FE2O3_EP_DEFAULT_SPIN;
    const uint64_t *peer_counts = reinterpret_cast<const uint64_t *>(a.peer_counts.ptr);
    const uint64_t *peer_flags = reinterpret_cast<const uint64_t *>(a.peer_flags.ptr);
    const uint64_t *peer_recv = reinterpret_cast<const uint64_t *>(a.peer_recv_x.ptr);
    const uint64_t *peer_meta = reinterpret_cast<const uint64_t *>(a.peer_recv_meta.ptr);
    uint32_t *my_flags = reinterpret_cast<uint32_t *>(peer_flags[me]);
    const uint32_t *my_counts = reinterpret_cast<const uint32_t *>(peer_counts[me]);
    uint32_t *rows_done = my_flags + FE2O3_EP_ROWS_DONE(W, epoch & 1u);

    // routing that reported a fault (non-finite logits) leaves no table to dispatch: the pass is void
    const bool dead = status && __ldcg(status) != 0u;
    if (blockIdx.x == 0 && threadIdx.x == 0) ep_trace(my_flags, FE2O3_EP_T_DISPATCH_BEGIN);
    if (blockIdx.x == 0 && !dead) {
        // publish this rank's admitted counts into every rank's table, then the flag
        const uint32_t *admitted = reinterpret_cast<const uint32_t *>(a.admitted_counts.ptr);
        for (uint32_t i = threadIdx.x; i < W * E; i += kDispatchThreads) {
            const uint32_t p = i / E, e = i % E;
            reinterpret_cast<uint32_t *>(peer_counts[p])[me * E + e] = admitted[e];
        }
        __threadfence_system();
        __syncthreads();
        for (uint32_t p = threadIdx.x; p < W; p += kDispatchThreads)
            st_release_sys(reinterpret_cast<uint32_t *>(peer_flags[p]) + FE2O3_EP_FLAG_COUNTS(W) + me, epoch);
        // the per-destination row counters of the NEXT pass (nobody touches that set during this one)
        for (uint32_t p = threadIdx.x; p < W; p += kDispatchThreads) my_flags[FE2O3_EP_ROWS_DONE(W, (epoch & 1u) ^ 1u) + p] = 0u;
        if (threadIdx.x == 0) my_flags[FE2O3_EP_OWN_BLOCKS(W, (epoch & 1u) ^ 1u)] = 0u;
    }
    if (a.logits.len && !dead) {
        // Route weights of this rank's tokens, one token per thread of the grid, computed while the counts
        // of the other ranks are still on their way (the combine phase reads them).
        const float *logits = reinterpret_cast<const float *>(a.logits.ptr);
        const uint32_t *top2 = reinterpret_cast<const uint32_t *>(a.top2_experts.ptr);
        float *weights = reinterpret_cast<float *>(a.route_weights.ptr);
        for (uint32_t t = blockIdx.x * kDispatchThreads + threadIdx.x; t < a.tokens; t += gridDim.x * kDispatchThreads) {
            const uint32_t e0 = top2[2ull * t], e1 = top2[2ull * t + 1];
            if (e0 >= E || e1 >= E) { kstatus_set(status, FE2O3_KSTATUS_SLOT_RANGE); continue; }
            float w0, w1;
            route_weight_pair(logits[(uint64_t)t * E + e0], logits[(uint64_t)t * E + e1], w0, w1);
            weights[2ull * t] = w0;
            weights[2ull * t + 1] = w1;
        }
    }
    // Every warp keeps the small tables it needs in registers, one entry per lane (this kernel shares its
    // SMs with the GEMM that follows it, which leaves it no shared memory to speak of):
    //   lane e < E: off_lo/off_hi = local slots of expert e, base = first row of this rank's rows for e on e's owner
    //   lane j < W: the j-th destination in sending order, rank (me - j) mod W: v_lo/v_hi = its rows in that order
    // (the loops below are unrolled so that their loads, which are independent, are in flight together: a
    // chain of dependent round trips to L2 here delays the first row of the pass by microseconds)
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t *offsets = reinterpret_cast<const uint32_t *>(a.expert_offsets.ptr);
    const uint32_t off_lo = lane < E ? offsets[lane] : 0u, off_hi = lane < E ? offsets[lane + 1] : 0u;
    const uint32_t accepted = dead ? 0u : offsets[E];
    uint32_t v_lo = 0, v_hi = 0;
    if (lane < W) {
#pragma unroll 8
        for (uint32_t j = 0; j <= lane; ++j) {
            const uint32_t d = (me + W - j) % W;
            v_lo = v_hi;
            v_hi += offsets[(d + 1) * per] - offsets[d * per];
        }
    }
    uint32_t base = 0;   // all zero until the counts are here: correct for the one expert whose rows go before that

    // rows: one warp per accepted local slot, kInFlight 16-byte loads in flight per lane before the peer stores
    const uint32_t *perm = reinterpret_cast<const uint32_t *>(a.permutation.ptr);
    const uint32_t vec_per_row = a.d_model / 8;
    const uint4 *x = reinterpret_cast<const uint4 *>(a.x.ptr);
    const uint32_t own_rows = __shfl_sync(0xffffffffu, v_hi, 0);
    const uint32_t gwarp = blockIdx.x * (kDispatchThreads / 32) + (threadIdx.x >> 5), nwarps = gridDim.x * (kDispatchThreads / 32);
    // Rows this warp has stored and not yet accounted for, per destination: lane j counts the j-th destination
    // in sending order.  A warp accounts once per phase, after ALL its rows of the phase: the fence that must
    // precede the counter update waits for the stores to be acknowledged from the other GPU (microseconds),
    // which a warp that paid it per destination would pay seven times in a row at eight ranks.
    uint32_t pending = 0;
    auto account = [&]() {
        // every lane's stores are ordered before the counter updates; whoever completes a destination's
        // count raises "rows complete" there (lane j for destination j, all destinations at once)
        __threadfence_system();
        __syncwarp();
        if (lane < W && pending) {
            const uint32_t d = (me + W - lane) % W;
            const uint32_t done = atomicAdd(rows_done + d, pending) + pending;
            if (done == v_hi - v_lo) {
                __threadfence_system();
                st_release_sys(reinterpret_cast<uint32_t *>(peer_flags[d]) + FE2O3_EP_FLAG_ROWS(W) + me, epoch);
                if (d == me) ep_trace(my_flags, FE2O3_EP_T_OWN_ROWS_DONE);
            }
        }
        pending = 0;
        __syncwarp();
    };
    auto send_row = [&](uint32_t v) {
        // v-th row in sending order: which destination, which local slot, which expert
        const uint32_t j = __popc(__ballot_sync(0xffffffffu, lane < W && v >= v_hi));
        if (lane == j) ++pending;   // counted even when the row is refused below: the destination must not wait for it
        const uint32_t dst_rank = (me + W - j) % W;
        const uint32_t slot = offsets[dst_rank * per] + (v - __shfl_sync(0xffffffffu, v_lo, j));
        const uint32_t e = __popc(__ballot_sync(0xffffffffu, lane < E && slot >= off_hi));
        const uint32_t route = perm[slot];
        const uint32_t dst_row = __shfl_sync(0xffffffffu, base, e & 31) + (slot - __shfl_sync(0xffffffffu, off_lo, e & 31));
        if (e >= E || route == kDrop || (route >> 1) >= a.tokens || dst_row >= a.max_rows) {
            if (lane == 0) kstatus_set(status, FE2O3_KSTATUS_SLOT_RANGE);
            return;
        }
        if (lane == 0) reinterpret_cast<uint2 *>(peer_meta[dst_rank])[dst_row] = make_uint2(route, me);
        const uint4 *src = x + (uint64_t)(route >> 1) * vec_per_row;
        uint4 *dst = reinterpret_cast<uint4 *>(peer_recv[dst_rank]) + (uint64_t)dst_row * vec_per_row;
        for (uint32_t i0 = lane; i0 < vec_per_row; i0 += 32 * kInFlight) {
            uint4 q[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u)
                if (i0 + 32 * u < vec_per_row) q[u] = __ldg(src + i0 + 32 * u);
#pragma unroll
            for (int u = 0; u < kInFlight; ++u)
                if (i0 + 32 * u < vec_per_row) dst[i0 + 32 * u] = q[u];
        }
    };
    // Phase A, while the counts of the other ranks are still on their way: this rank's own rows for its first
    // local expert.  On its owner an expert's segment opens with the owner's own rows and the first local
    // expert's segment opens the buffer, so these rows start at row 0 whatever the other ranks send.  They are
    // what the GEMM beside this kernel starts on.
    const uint32_t first_own = (accepted && per) ? offsets[me * per + 1] - offsets[me * per] : 0u;
    for (uint32_t v = gwarp; v < first_own; v += nwarps) send_row(v);

    // every block waits for the counts of every source (thread s polls source s: local memory)
    int ok = dead ? 0 : (threadIdx.x < W ? (flag_wait(my_flags + FE2O3_EP_FLAG_COUNTS(W) + threadIdx.x, epoch, limit) ? 1 : 0) : 1);
    ok = __syncthreads_and(ok);
    if (blockIdx.x == 0 && threadIdx.x == 0) ep_trace(my_flags, FE2O3_EP_T_COUNTS_HERE);
    if (!ok) {
        // nothing more is sent and no flag is raised: the other ranks' waits run out in turn
        if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
        return;
    }
    if (lane < E) {
        // On expert e's owner d: whole segments of the owner's earlier experts, then the runs of the sources
        // that come before this rank in the owner's order d, d+1, ... (mod W).
        const uint32_t e = lane, d = e / per, le = e % per, k_me = (me + W - d) % W;
        for (uint32_t l2 = 0; l2 < le; ++l2) {
#pragma unroll 8
            for (uint32_t s = 0; s < W; ++s) base += __ldcg(my_counts + s * E + d * per + l2);
        }
#pragma unroll 8
        for (uint32_t k = 0; k < k_me; ++k) base += __ldcg(my_counts + ((d + k) % W) * E + e);
    }
    if (blockIdx.x == 0 && (threadIdx.x >> 5) == 1) {
        // Row partition of what this rank receives: pair (local expert, run k = source (me + k) mod W), a
        // running sum of the counts in that order, made by one warp (one count per lane, a shuffle scan, 32
        // pairs at a time); then tell the FFN kernel, which may already be running on this GPU, that the
        // table is there.
        uint32_t *pair_offsets = reinterpret_cast<uint32_t *>(a.pair_offsets.ptr);
        const uint32_t pairs = per * W;
        uint32_t run = 0;
        if (lane == 0) pair_offsets[0] = 0;
        for (uint32_t i0 = 0; i0 < pairs; i0 += 32) {
            const uint32_t i = i0 + lane, le = i / W, src = (me + i % W) % W;
            uint32_t c = i < pairs ? __ldcg(my_counts + src * E + me * per + le) : 0u;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t up = __shfl_up_sync(0xffffffffu, c, o);
                if (lane >= (uint32_t)o) c += up;
            }
            const uint32_t total = run + c;   // inclusive sum up to pair i
            // a table that overruns the receive buffer is cut off: the FFN must never index past it
            if (i < pairs) pair_offsets[i + 1] = total < a.max_rows ? total : a.max_rows;
            run = __shfl_sync(0xffffffffu, total, 31);
        }
        if (lane == 0 && run > a.max_rows) kstatus_set(status, FE2O3_KSTATUS_SLOT_RANGE);
        __threadfence();
        __syncwarp();
        if (lane == 0) st_release_sys(my_flags + FE2O3_EP_FLAG_TABLE(W), epoch);
    }
    if (blockIdx.x == 0 && threadIdx.x < W && v_hi == v_lo)   // nothing to send there: complete at once
        st_release_sys(reinterpret_cast<uint32_t *>(peer_flags[(me + W - threadIdx.x) % W]) + FE2O3_EP_FLAG_ROWS(W) + me, epoch);

    // Phase B1: the rest of this rank's own rows (its other local experts), by all blocks, accounted together
    // with phase A.  They copy at memory speed as long as nothing else is in the way: rows to other ranks
    // leave at NVLink speed and hold up everything behind them in the memory system (the flag polls of the
    // GEMM block on the same SM included), so no block starts on those before every block is through with
    // its own rows and block 0 has published the row table (all blocks of this grid are resident at once,
    // one per SM).
    for (uint32_t v = first_own + gwarp; v < own_rows; v += nwarps) send_row(v);
    if (__any_sync(0xffffffffu, pending != 0u)) account();
    if (W > 1) {
        uint32_t *own_blocks = my_flags + FE2O3_EP_OWN_BLOCKS(W, epoch & 1u);
        __syncthreads();
        if (threadIdx.x == 0) {
            atomicAdd(own_blocks, 1u);
            uint32_t spins = 0;
            while (*reinterpret_cast<volatile uint32_t *>(own_blocks) < gridDim.x && ++spins < limit) __nanosleep(64);
            // a wait that runs out only costs the ordering: the rows below are still sent
        }
        __syncthreads();
    }
    // Phase 2: the other ranks' rows, in sending order
    for (uint32_t v = own_rows + gwarp; v < accepted; v += nwarps) send_row(v);
    if (__any_sync(0xffffffffu, pending != 0u)) account();
    if (blockIdx.x == 0 && threadIdx.x == 0) ep_trace(my_flags, FE2O3_EP_T_ROWS_SENT);
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
            const uint32_t grid = (uint32_t)ctx->sm_count;
            if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {kDispatchThreads, 1, 1}, 0, 1};
            if (plan_only) return FE2O3_OK;
            // The GEMM that is to run beside this kernel needs nearly all of an SM's shared memory; an SM
            // changes its split between L1 and shared memory only when idle, so this kernel asks for the
            // largest shared-memory split although it uses none (per device, cheap: set at every launch).
            cudaFuncSetAttribute(moe_ep_dispatch_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 (int)cudaSharedmemCarveoutMaxShared);
            moe_ep_dispatch_kernel<<<grid, kDispatchThreads, 0, s>>>(*a, ctx->status_word);
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

static Fe2o3KernelRegistration reg_exchange("moe_ep_exchange_v1", reinterpret_cast<const void *>(moe_ep_dispatch_kernel));
