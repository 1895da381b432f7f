// MoE routing-side kernels: gate logits, top-2 selection with stable slot
// packing, route weights, activation compaction and the weighted combine.
// The expert FFN itself is the grouped tensor-core GEMM in gemm_tc.cu.
#include <stdlib.h>

#include "common.cuh"

namespace {

constexpr uint32_t kDrop = 0xffffffffu;

// ---- gate logits ------------------------------------------------------------
// logits[t,e] = sum_k x[t,k]*wg[k,e]; bf16 widened exactly, f32 accumulator from
// +0, increasing k, separate product and sum, so top-2 indices can be compared
// bit-for-bit with the CPU recurrence.  blockDim = (E, TPB): thread (e, t)
// owns one output; x and wg are staged through shared memory KC deep.
constexpr int kGateKC = 128;

__global__ void moe_gate_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ wg,
                                float *__restrict__ logits, uint32_t tokens, uint32_t d_model, uint32_t experts) {
    extern __shared__ float gate_smem[];
    const uint32_t tpb = blockDim.y;
    float *xs = gate_smem;                      // [tpb][kGateKC + 1]
    float *ws = gate_smem + tpb * (kGateKC + 1);  // [kGateKC][experts]
    const uint32_t e = threadIdx.x, tl = threadIdx.y;
    const uint32_t t0 = blockIdx.x * tpb;
    const uint32_t lin = tl * blockDim.x + e, nthr = blockDim.x * blockDim.y;
    float acc = 0.0f;
    for (uint32_t k0 = 0; k0 < d_model; k0 += kGateKC) {
        const uint32_t kc = min((uint32_t)kGateKC, d_model - k0);
        for (uint32_t i = lin; i < tpb * kGateKC; i += nthr) {
            const uint32_t r = i / kGateKC, kk = i % kGateKC;
            const uint32_t t = t0 + r;
            xs[r * (kGateKC + 1) + kk] = (t < tokens && kk < kc) ? bf16_bits_to_f32(x[(uint64_t)t * d_model + k0 + kk]) : 0.0f;
        }
        for (uint32_t i = lin; i < kc * experts; i += nthr) ws[i] = bf16_bits_to_f32(wg[(uint64_t)k0 * experts + i]);
        __syncthreads();
        for (uint32_t kk = 0; kk < kc; ++kk)
            acc = __fadd_rn(acc, __fmul_rn(xs[tl * (kGateKC + 1) + kk], ws[kk * experts + e]));
        __syncthreads();
    }
    if (t0 + tl < tokens) logits[(uint64_t)(t0 + tl) * experts + e] = acc;
}

// ---- top-2 routing ------------------------------------------------------------
// examples/moe_top2_v1/src/kernel.rs:25-59 (comparator and running top-2) and
// :132-202 (counts, clamp, exclusive scan, stable slots, permutation, inverse),
// widened from one lane to one 1024-thread block.  Thread i owns the contiguous
// token chunk [i*tpt, (i+1)*tpt), so route-id order is (thread, local order)
// and a per-expert exclusive scan over threads gives every route its stable
// rank without atomics: the packing is deterministic.
constexpr int kRouteThreads = 1024;

__device__ __forceinline__ bool precedes(float cs, uint32_t ce, float is, uint32_t ie) {
    return cs > is || (cs == is && ce < ie);
}

__global__ void __launch_bounds__(kRouteThreads)
moe_top2_kernel(fe2o3_moe_top2_v1_args a, uint32_t *status) {
    extern __shared__ uint32_t counts[];  // [experts][kRouteThreads]
    __shared__ uint32_t s_offsets[65];
    __shared__ uint32_t s_requested[64];
    __shared__ int s_bad;
    const uint32_t T = a.tokens, E = a.experts, cap = a.capacity;
    const uint64_t R = 2ull * T;
    const uint32_t tid = threadIdx.x;
    if (a.logits.len != (uint64_t)T * E || a.top2_experts.len != R || a.requested_counts.len != E ||
        a.admitted_counts.len != E || a.expert_offsets.len != E + 1 || a.route_slots.len != R ||
        a.permutation.len != R || a.inverse.len != R || E < 2 || E > 32) {
        if (tid == 0) kstatus_set(status, FE2O3_KSTATUS_LENGTH);
        return;
    }
    const float *logits = reinterpret_cast<const float *>(a.logits.ptr);
    uint32_t *top2 = reinterpret_cast<uint32_t *>(a.top2_experts.ptr);
    uint32_t *requested = reinterpret_cast<uint32_t *>(a.requested_counts.ptr);
    uint32_t *admitted = reinterpret_cast<uint32_t *>(a.admitted_counts.ptr);
    uint32_t *offsets = reinterpret_cast<uint32_t *>(a.expert_offsets.ptr);
    uint32_t *slots = reinterpret_cast<uint32_t *>(a.route_slots.ptr);
    uint32_t *perm = reinterpret_cast<uint32_t *>(a.permutation.ptr);
    uint32_t *inverse = reinterpret_cast<uint32_t *>(a.inverse.ptr);

    // finite-logit admission before any output is written
    if (tid == 0) s_bad = 0;
    __syncthreads();
    bool bad = false;
    for (uint64_t i = tid; i < (uint64_t)T * E; i += kRouteThreads) bad |= !isfinite(logits[i]);
    if (bad) atomicExch(&s_bad, 1);
    __syncthreads();
    if (s_bad) {
        if (tid == 0) kstatus_set(status, FE2O3_KSTATUS_NONFINITE);
        return;
    }

    const uint32_t tpt = (T + kRouteThreads - 1) / kRouteThreads;
    const uint32_t t_begin = min(T, tid * tpt), t_end = min(T, t_begin + tpt);
    for (uint32_t e = 0; e < E; ++e) counts[e * kRouteThreads + tid] = 0;
    for (uint32_t t = t_begin; t < t_end; ++t) {
        const float *row = logits + (uint64_t)t * E;
        uint32_t best = kDrop, second = kDrop;
        float bs = 0.f, ss = 0.f;
        for (uint32_t e = 0; e < E; ++e) {
            const float sc = row[e];
            if (best == kDrop || precedes(sc, e, bs, best)) {
                second = best; ss = bs;
                best = e; bs = sc;
            } else if (second == kDrop || precedes(sc, e, ss, second)) {
                second = e; ss = sc;
            }
        }
        top2[2ull * t] = best;
        top2[2ull * t + 1] = second;
        counts[best * kRouteThreads + tid] += 1;
        counts[second * kRouteThreads + tid] += 1;
    }
    __syncthreads();
    // exclusive scan over threads, one warp per expert (strided over experts)
    const uint32_t warp = tid >> 5, lane = tid & 31;
    for (uint32_t e = warp; e < E; e += kRouteThreads / 32) {
        uint32_t running = 0;
        for (uint32_t c = 0; c < kRouteThreads; c += 32) {
            const uint32_t v = counts[e * kRouteThreads + c + lane];
            uint32_t inc = v;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                uint32_t n = __shfl_up_sync(0xffffffffu, inc, off);
                if ((int)lane >= off) inc += n;
            }
            counts[e * kRouteThreads + c + lane] = running + inc - v;
            running += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) s_requested[e] = running;
    }
    __syncthreads();
    if (tid == 0) {
        s_offsets[0] = 0;
        for (uint32_t e = 0; e < E; ++e) {
            const uint32_t adm = s_requested[e] > cap ? cap : s_requested[e];
            requested[e] = s_requested[e];
            admitted[e] = adm;
            s_offsets[e + 1] = s_offsets[e] + adm;
        }
        for (uint32_t e = 0; e <= E; ++e) offsets[e] = s_offsets[e];
    }
    __syncthreads();
    for (uint64_t s = s_offsets[E] + tid; s < R; s += kRouteThreads) perm[s] = kDrop;
    for (uint32_t t = t_begin; t < t_end; ++t) {
#pragma unroll
        for (int rank = 0; rank < 2; ++rank) {
            const uint64_t r = 2ull * t + rank;
            const uint32_t e = top2[r];
            const uint32_t stable_rank = counts[e * kRouteThreads + tid]++;
            uint32_t slot = kDrop;
            if (stable_rank < cap) {
                slot = s_offsets[e] + stable_rank;
                perm[slot] = (uint32_t)r;
            }
            slots[r] = slot;
            inverse[r] = slot;
        }
    }
}

// ---- gate logits, staged and prefetched -----------------------------------------
// Same arithmetic as moe_gate_kernel: every output runs its own sequential f32
// chain (product, then sum, increasing k).  A warp covers 32 tokens and a group
// of EPT = 4 experts: lane = token, so the x operand is one conflict-free
// shared-memory read per k and the four Wg operands one broadcast 16-byte read;
// four independent add chains per thread hide the add latency.  (One output per
// thread needs two shared-memory reads per multiply-add and is bound by
// shared-memory bandwidth; all E outputs per thread leaves one warp per
// scheduler and is bound by that warp's issue rate.)  Per 64-wide k chunk the x
// rows and Wg rows are fetched one chunk ahead into registers, so global latency
// overlaps the arithmetic.
constexpr int kGate2Tokens = 32, kGate2KC = 64;

template <int E>
__global__ void __launch_bounds__(32 * (E / (E >= 4 ? 4 : E)))
moe_gate_staged_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ wg, float *__restrict__ logits,
                       uint32_t tokens, uint32_t d_model) {
    constexpr int EPT = E >= 4 ? 4 : E;                     // experts per thread
    constexpr int kThreads = 32 * (E / EPT);
    constexpr int kXVec = kGate2Tokens * kGate2KC * 2 / 16; // 256 16-byte vectors of x per chunk
    constexpr int kXPer = kXVec / kThreads;
    constexpr int kWVec = kGate2KC * E * 2 / 16;            // 16-byte vectors of Wg per chunk
    constexpr int kWPer = (kWVec + kThreads - 1) / kThreads;
    __shared__ float xs[kGate2KC][kGate2Tokens + 1];
    __shared__ __align__(16) float ws[kGate2KC][E];
    const uint32_t tid = threadIdx.x, lane = tid & 31, e0 = (tid >> 5) * EPT;
    const uint32_t t0 = blockIdx.x * kGate2Tokens;
    float acc[EPT];
#pragma unroll
    for (int q = 0; q < EPT; ++q) acc[q] = 0.0f;
    uint64_t acc2[2] = {0ull, 0ull};   // the four accumulators as two packed pairs (EPT == 4)
    const bool vec = (d_model % 8u) == 0 && ((reinterpret_cast<uint64_t>(x) | reinterpret_cast<uint64_t>(wg)) & 15u) == 0;
    uint4 xpre[kXPer], wpre[kWPer];
    auto prefetch = [&](uint32_t k0) {
        // 8 consecutive threads cover one token's 64 k values (128 bytes)
#pragma unroll
        for (int q = 0; q < kXPer; ++q) {
            const uint32_t v = tid + q * kThreads;
            xpre[q] = make_uint4(0, 0, 0, 0);
            if (t0 + (v >> 3) < tokens)
                xpre[q] = __ldg(reinterpret_cast<const uint4 *>(x + (uint64_t)(t0 + (v >> 3)) * d_model + k0) + (v & 7));
        }
#pragma unroll
        for (int q = 0; q < kWPer; ++q) {
            const uint32_t v = tid + q * kThreads;
            wpre[q] = make_uint4(0, 0, 0, 0);
            if (v < (uint32_t)kWVec) wpre[q] = __ldg(reinterpret_cast<const uint4 *>(wg + (uint64_t)k0 * E) + v);
        }
    };
    if (vec && d_model >= kGate2KC) prefetch(0);
    for (uint32_t k0 = 0; k0 < d_model; k0 += kGate2KC) {
        const uint32_t kc = min((uint32_t)kGate2KC, d_model - k0);
        if (vec && kc == kGate2KC) {
#pragma unroll
            for (int q = 0; q < kXPer; ++q) {
                const uint32_t v = tid + q * kThreads, tt = v >> 3, c = v & 7;
                const uint32_t w[4] = {xpre[q].x, xpre[q].y, xpre[q].z, xpre[q].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    xs[c * 8 + 2 * i][tt] = __uint_as_float(w[i] << 16);
                    xs[c * 8 + 2 * i + 1][tt] = __uint_as_float(w[i] & 0xffff0000u);
                }
            }
#pragma unroll
            for (int q = 0; q < kWPer; ++q) {
                const uint32_t v = tid + q * kThreads;
                if (v < (uint32_t)kWVec) {
                    const uint32_t w[4] = {wpre[q].x, wpre[q].y, wpre[q].z, wpre[q].w};
                    float *dst = &ws[0][0] + v * 8;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        dst[2 * i] = __uint_as_float(w[i] << 16);
                        dst[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
                    }
                }
            }
            if (k0 + 2 * kGate2KC <= d_model) prefetch(k0 + kGate2KC);
        } else {
            for (uint32_t i = tid; i < (uint32_t)kGate2Tokens * kGate2KC; i += kThreads) {
                const uint32_t tt = i / kGate2KC, kk = i % kGate2KC;
                xs[kk][tt] = (t0 + tt < tokens && kk < kc) ? bf16_bits_to_f32(x[(uint64_t)(t0 + tt) * d_model + k0 + kk]) : 0.0f;
            }
            for (uint32_t i = tid; i < kc * E; i += kThreads) (&ws[0][0])[i] = bf16_bits_to_f32(wg[(uint64_t)k0 * E + i]);
        }
        __syncthreads();
        if (kc == kGate2KC) {
#pragma unroll 1
            for (uint32_t kk = 0; kk < kGate2KC; kk += 8) {
                float xv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) xv[i] = xs[kk + i][lane];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if constexpr (EPT == 4) {
                        // two experts per instruction: the packed forms round each half exactly as the
                        // scalar multiply and add do, so the logits keep their bits
                        const float4 v = *reinterpret_cast<const float4 *>(&ws[kk + i][e0]);
                        const uint64_t xx = pack_f32x2(xv[i], xv[i]);
                        acc2[0] = add_f32x2(acc2[0], mul_f32x2(xx, pack_f32x2(v.x, v.y)));
                        acc2[1] = add_f32x2(acc2[1], mul_f32x2(xx, pack_f32x2(v.z, v.w)));
                    } else {
                        float w[EPT];
#pragma unroll
                        for (int q = 0; q < EPT; ++q) w[q] = ws[kk + i][e0 + q];
#pragma unroll
                        for (int q = 0; q < EPT; ++q) acc[q] = __fadd_rn(acc[q], __fmul_rn(xv[i], w[q]));
                    }
                }
            }
        } else {
            if constexpr (EPT == 4) {   // leave the packed accumulators for the ragged chunk
                unpack_f32x2(acc2[0], acc[0], acc[1]);
                unpack_f32x2(acc2[1], acc[2], acc[3]);
            }
            for (uint32_t kk = 0; kk < kc; ++kk) {
                const float xv = xs[kk][lane];
#pragma unroll
                for (int q = 0; q < EPT; ++q) acc[q] = __fadd_rn(acc[q], __fmul_rn(xv, ws[kk][e0 + q]));
            }
            if constexpr (EPT == 4) {
                acc2[0] = pack_f32x2(acc[0], acc[1]);
                acc2[1] = pack_f32x2(acc[2], acc[3]);
            }
        }
        __syncthreads();
    }
    if constexpr (EPT == 4) {
        unpack_f32x2(acc2[0], acc[0], acc[1]);
        unpack_f32x2(acc2[1], acc[2], acc[3]);
    }
    if (t0 + lane < tokens) {
#pragma unroll
        for (int q = 0; q < EPT; ++q) logits[(uint64_t)(t0 + lane) * E + e0 + q] = acc[q];
    }
}

// One warp per block, eight tokens per warp: lane = (token, group of E/4 experts).  Same arithmetic and
// order as the kernel above (each logit is one sequential chain of separately rounded multiplies and
// adds over k), but eight times as many independent blocks, so that a few thousand tokens already
// occupy every SM; used for small token counts only (the block kernel issues fewer instructions per
// multiply-add and wins once there are enough tokens).
// Needs d_model to be a multiple of 64 and 16-byte aligned x and Wg.
template <int E>
__global__ void __launch_bounds__(32)
moe_gate_warp_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ wg, float *__restrict__ logits,
                     uint32_t tokens, uint32_t d_model) {
    constexpr int TPW = 8, KC = 64;
    constexpr int EPT = E / 4;                       // experts per lane
    constexpr int kXPer = TPW * KC * 2 / 16 / 32;    // 16-byte vectors of x per lane and chunk (2)
    constexpr int kWVec = KC * E * 2 / 16;           // 16-byte vectors of Wg per chunk
    constexpr int kWPer = (kWVec + 31) / 32;
    __shared__ float xs[KC][TPW];
    __shared__ __align__(16) float ws[KC][E];
    const uint32_t lane = threadIdx.x, tt = lane & 7, e0 = (lane >> 3) * EPT;
    const uint32_t t0 = blockIdx.x * TPW;
    float acc[EPT];
#pragma unroll
    for (int q = 0; q < EPT; ++q) acc[q] = 0.0f;
    uint4 xpre[kXPer], wpre[kWPer];
    auto prefetch = [&](uint32_t k0) {
#pragma unroll
        for (int q = 0; q < kXPer; ++q) {
            const uint32_t v = lane + q * 32;   // token v >> 3, 16-byte piece v & 7 of its 128-byte chunk
            xpre[q] = make_uint4(0, 0, 0, 0);
            if (t0 + (v >> 3) < tokens)
                xpre[q] = __ldg(reinterpret_cast<const uint4 *>(x + (uint64_t)(t0 + (v >> 3)) * d_model + k0) + (v & 7));
        }
#pragma unroll
        for (int q = 0; q < kWPer; ++q) {
            const uint32_t v = lane + q * 32;
            wpre[q] = make_uint4(0, 0, 0, 0);
            if (v < (uint32_t)kWVec) wpre[q] = __ldg(reinterpret_cast<const uint4 *>(wg + (uint64_t)k0 * E) + v);
        }
    };
    prefetch(0);
    for (uint32_t k0 = 0; k0 < d_model; k0 += KC) {
#pragma unroll
        for (int q = 0; q < kXPer; ++q) {
            const uint32_t v = lane + q * 32, tk = v >> 3, c = v & 7;
            const uint32_t w[4] = {xpre[q].x, xpre[q].y, xpre[q].z, xpre[q].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                xs[c * 8 + 2 * i][tk] = __uint_as_float(w[i] << 16);
                xs[c * 8 + 2 * i + 1][tk] = __uint_as_float(w[i] & 0xffff0000u);
            }
        }
#pragma unroll
        for (int q = 0; q < kWPer; ++q) {
            const uint32_t v = lane + q * 32;
            if (v < (uint32_t)kWVec) {
                const uint32_t w[4] = {wpre[q].x, wpre[q].y, wpre[q].z, wpre[q].w};
                float *dst = &ws[0][0] + v * 8;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    dst[2 * i] = __uint_as_float(w[i] << 16);
                    dst[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
                }
            }
        }
        if (k0 + KC < d_model) prefetch(k0 + KC);
        __syncwarp();
#pragma unroll 1
        for (uint32_t kk = 0; kk < KC; kk += 8) {
            float xv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) xv[i] = xs[kk + i][tt];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float w[EPT];
                if constexpr (EPT == 4) {
                    const float4 v = *reinterpret_cast<const float4 *>(&ws[kk + i][e0]);
                    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
                } else if constexpr (EPT == 2) {
                    const float2 v = *reinterpret_cast<const float2 *>(&ws[kk + i][e0]);
                    w[0] = v.x; w[1] = v.y;
                } else {
                    w[0] = ws[kk + i][e0];
                }
#pragma unroll
                for (int q = 0; q < EPT; ++q) acc[q] = __fadd_rn(acc[q], __fmul_rn(xv[i], w[q]));
            }
        }
        __syncwarp();
    }
    if (t0 + tt < tokens) {
#pragma unroll
        for (int q = 0; q < EPT; ++q) logits[(uint64_t)(t0 + tt) * E + e0 + q] = acc[q];
    }
}

// ---- gate logits: Wg resident in shared memory, x through an asynchronous copy ring ---------
// Same arithmetic and order again (each logit one sequential chain of separately rounded products
// and sums over k), laid out for what bounds the gate: the latency of that chain (2048 dependent
// additions per output whatever the token count) when there are few tokens, instruction issue and
// the HBM stream of x when there are many.
//   Wg is widened to f32 once per block into shared memory ([k][E], E * d_model * 4 bytes) and stays
//     there: the k loop stages no weights.
//   lane = (token, group of EPL experts).  Each warp streams the rows of its own tokens, 64 k values
//     at a time, into a private ring of STAGES shared-memory stages with 16-byte asynchronous copies
//     (no registers and no scoreboard are held while they fly, so the ring really is STAGES - 1
//     chunks deep; a ring of prefetched registers is not: the hardware tracks outstanding loads of a
//     warp with a handful of counters, and waiting for the oldest load waits for the youngest that
//     shares its counter).  The warp synchronises with itself only; there is no block barrier in
//     the loop.  Rows are padded by 16 bytes so that the 16-byte reads of eight tokens do not
//     collide on banks.
//   The EPL logits of a lane advance as EPL / 2 packed f32x2 products and sums per k (each half
//     rounded exactly like the scalar instruction).  EPL = 2 spreads a token over E / 2 lanes, so a
//     rank's 2048 tokens of an expert-parallel layer still make 256 warps, each running at the pace
//     of the dependent additions; EPL = 4 halves the instructions per multiply-add for large batches.
// Needs E in {4, 8, 16}, d_model a multiple of 64 with E * d_model * 4 bytes of shared memory
// available, 16-byte aligned x and Wg.
constexpr int kGateKC2 = 64;                       // k values per stage
constexpr int kGateRowBytes = kGateKC2 * 2 + 16;   // one token's stage row, padded

__device__ __forceinline__ void cp_async_16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int E, int EPL, int WARPS, int STAGES>
__global__ void __launch_bounds__(32 * WARPS)
moe_gate_lanes_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ wg, float *__restrict__ logits,
                      uint32_t tokens, uint32_t d_model) {
    extern __shared__ __align__(16) uint8_t gate_lanes_smem[];
    constexpr int LPT = E / EPL;        // lanes per token
    constexpr int TPW = 32 / LPT;       // tokens per warp
    constexpr int NP = EPL / 2;         // packed accumulators per lane
    constexpr int kStageBytes = TPW * kGateRowBytes;
    constexpr int kGranules = TPW * 8;  // 16-byte pieces per stage
    float *gate_w = reinterpret_cast<float *>(gate_lanes_smem);                 // [d_model][E]
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint8_t *ring = gate_lanes_smem + (size_t)d_model * E * 4 + (size_t)warp * STAGES * kStageBytes;
    const uint32_t tok0 = (blockIdx.x * WARPS + warp) * TPW;
    const uint32_t nchunks = d_model / kGateKC2;
    auto copy_chunk = [&](uint32_t chunk) {
        if (chunk < nchunks) {
            uint8_t *stage = ring + (chunk % STAGES) * kStageBytes;
#pragma unroll
            for (int g0 = 0; g0 < kGranules; g0 += 32) {
                const uint32_t g = g0 + lane;
                if (kGranules >= 32 || g < (uint32_t)kGranules) {
                    const uint32_t tk = g >> 3, piece = g & 7;
                    const uint32_t token = min(tok0 + tk, tokens - 1);   // rows beyond the batch re-read the last row
                    cp_async_16(stage + tk * kGateRowBytes + piece * 16,
                                x + (uint64_t)token * d_model + chunk * kGateKC2 + piece * 8);
                }
            }
        }
        cp_async_commit();   // an empty group keeps the group count uniform at the tail
    };
    // the first chunks are on their way while the block widens Wg
#pragma unroll
    for (int c = 0; c < STAGES - 1; ++c) copy_chunk(c);
    for (uint32_t v = tid; v < d_model * E / 8; v += 32 * WARPS) {
        const uint4 w = __ldg(reinterpret_cast<const uint4 *>(wg) + v);
        float4 *dst = reinterpret_cast<float4 *>(gate_w + v * 8);
        dst[0] = make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u), __uint_as_float(w.y << 16),
                             __uint_as_float(w.y & 0xffff0000u));
        dst[1] = make_float4(__uint_as_float(w.z << 16), __uint_as_float(w.z & 0xffff0000u), __uint_as_float(w.w << 16),
                             __uint_as_float(w.w & 0xffff0000u));
    }
    __syncthreads();
    const uint32_t tt = lane / LPT, e0 = (lane % LPT) * EPL;
    uint64_t acc[NP];
#pragma unroll
    for (int q = 0; q < NP; ++q) acc[q] = 0ull;   // {+0.0f, +0.0f}
    for (uint32_t c = 0; c < nchunks; ++c) {
        cp_async_wait<STAGES - 2>();   // this lane's pieces of chunk c have landed
        __syncwarp();                  // every lane's have, and nobody still reads the stage refilled next
        copy_chunk(c + STAGES - 1);
        const uint4 *xrow = reinterpret_cast<const uint4 *>(ring + (c % STAGES) * kStageBytes + tt * kGateRowBytes);
        const float *wk = gate_w + (uint64_t)c * kGateKC2 * E + e0;
#pragma unroll
        for (int v = 0; v < kGateKC2 / 8; ++v) {
            const uint4 xv = xrow[v];
            const uint32_t words[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float xf = __uint_as_float(h ? (words[i] & 0xffff0000u) : (words[i] << 16));
                    const uint64_t xx = pack_f32x2(xf, xf);
                    const float *w = wk + (v * 8 + 2 * i + h) * E;
                    if constexpr (EPL == 2) {
                        const float2 a = *reinterpret_cast<const float2 *>(w);
                        acc[0] = add_f32x2(acc[0], mul_f32x2(xx, pack_f32x2(a.x, a.y)));
                    } else {
#pragma unroll
                        for (int q = 0; q < EPL / 4; ++q) {
                            const float4 a = *reinterpret_cast<const float4 *>(w + 4 * q);
                            acc[2 * q] = add_f32x2(acc[2 * q], mul_f32x2(xx, pack_f32x2(a.x, a.y)));
                            acc[2 * q + 1] = add_f32x2(acc[2 * q + 1], mul_f32x2(xx, pack_f32x2(a.z, a.w)));
                        }
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    if (tok0 + tt < tokens) {
#pragma unroll
        for (int q = 0; q < NP; ++q) {
            float lo, hi;
            unpack_f32x2(acc[q], lo, hi);
            *reinterpret_cast<float2 *>(logits + (uint64_t)(tok0 + tt) * E + e0 + 2 * q) = make_float2(lo, hi);
        }
    }
}

template <int E, int EPL, int WARPS, int STAGES>
static cudaError_t launch_gate_lanes(cudaStream_t s, const uint16_t *x, const uint16_t *wg, float *lg, uint32_t tokens,
                                     uint32_t d_model, fe2o3_geometry *geo) {
    constexpr uint32_t tokens_per_block = WARPS * (32 / (E / EPL));
    const uint32_t grid = ceil_div_u32(tokens, tokens_per_block);
    const uint32_t smem = d_model * E * 4 + WARPS * STAGES * (32 / (E / EPL)) * kGateRowBytes;
    if (geo) { *geo = fe2o3_geometry{{grid, 1, 1}, {32 * WARPS, 1, 1}, smem, 1}; return cudaSuccess; }
    // the attribute is per device and cheap to set: set it on every launch for the current device
    cudaError_t e = cudaFuncSetAttribute(moe_gate_lanes_kernel<E, EPL, WARPS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    moe_gate_lanes_kernel<E, EPL, WARPS, STAGES><<<grid, 32 * WARPS, smem, s>>>(x, wg, lg, tokens, d_model);
    return cudaSuccess;
}

// ---- top-2 routing over many blocks --------------------------------------------
// Same result as moe_top2_kernel.  Block b owns tokens [256 b, 256 b + 256).
// Pass 1 counts, per block and expert, the routes the block requests and checks
// its logits; the last block to arrive scans the per-block counts over blocks
// (exclusive, in block order) and publishes requested / admitted / offsets.
// Pass 2 recomputes the selections, ranks each route inside its block with warp
// ballots (route order = token order, rank 0 before rank 1) and adds the block's
// base: a deterministic stable rank without atomics.  Nothing is written when any
// logit is non-finite.
constexpr int kRouteBlock = 256;

__device__ __forceinline__ void top2_of_row(const float *row, uint32_t E, uint32_t &best, uint32_t &second, bool &finite) {
    best = kDrop;
    second = kDrop;
    float bs = 0.f, ss = 0.f;
    finite = true;
    for (uint32_t e = 0; e < E; ++e) {
        const float sc = row[e];
        finite = finite && isfinite(sc);
        if (best == kDrop || precedes(sc, e, bs, best)) {
            second = best; ss = bs;
            best = e; bs = sc;
        } else if (second == kDrop || precedes(sc, e, ss, second)) {
            second = e; ss = sc;
        }
    }
}

// Ranks of this thread's two routes among the block's routes to the same experts, and the block's
// per-expert totals in s_total[E].  All 256 threads must call it.
__device__ __forceinline__ void block_ranks(uint32_t best, uint32_t second, bool active, uint32_t E, uint32_t (*s_warp)[32],
                                            uint32_t *s_total, uint32_t &rank_best, uint32_t &rank_second) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t lt = (1u << lane) - 1u;
    uint32_t pa = 0, pb = 0;
    for (uint32_t e = 0; e < E; ++e) {
        const uint32_t mb = __ballot_sync(0xffffffffu, active && best == e);
        const uint32_t ms = __ballot_sync(0xffffffffu, active && second == e);
        const uint32_t before = __popc(mb & lt) + __popc(ms & lt);
        if (best == e) pa = before;
        if (second == e) pb = before;
        if (lane == 0) s_warp[warp][e] = __popc(mb) + __popc(ms);
    }
    __syncthreads();
    uint32_t base_a = 0, base_b = 0;
    for (uint32_t w = 0; w < warp; ++w) {
        if (active) { base_a += s_warp[w][best]; base_b += s_warp[w][second]; }
    }
    rank_best = pa + base_a;
    rank_second = pb + base_b;
    if (threadIdx.x < E) {
        uint32_t tot = 0;
        for (uint32_t w = 0; w < kRouteBlock / 32; ++w) tot += s_warp[w][threadIdx.x];
        s_total[threadIdx.x] = tot;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kRouteBlock)
moe_route_count_kernel(fe2o3_moe_top2_v1_args a, uint32_t *scratch, uint32_t *status) {
    __shared__ uint32_t s_warp[kRouteBlock / 32][32];
    __shared__ uint32_t s_total[32];
    __shared__ int s_bad;
    __shared__ bool s_last;
    const uint32_t T = a.tokens, E = a.experts;
    const uint64_t R = 2ull * T;
    uint32_t *counts = scratch;                                   // [blocks][32]
    uint32_t *flags = scratch + FE2O3_ROUTE_MAX_BLOCKS * 32u;      // [blocks]
    uint32_t *summary = flags + FE2O3_ROUTE_MAX_BLOCKS;            // [0] = any non-finite logit
    uint32_t *counter = summary + 1;
    if (a.logits.len != (uint64_t)T * E || a.top2_experts.len != R || a.requested_counts.len != E ||
        a.admitted_counts.len != E || a.expert_offsets.len != E + 1 || a.route_slots.len != R ||
        a.permutation.len != R || a.inverse.len != R || E < 2 || E > 32) {
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            kstatus_set(status, FE2O3_KSTATUS_LENGTH);
            summary[0] = 2u;
        }
        return;
    }
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
    const uint32_t t = blockIdx.x * kRouteBlock + threadIdx.x;
    const bool active = t < T;
    uint32_t best = 0, second = 0;
    bool finite = true;
    if (active) top2_of_row(reinterpret_cast<const float *>(a.logits.ptr) + (uint64_t)t * E, E, best, second, finite);
    if (!finite) atomicExch(&s_bad, 1);
    uint32_t ra, rb;
    block_ranks(best, second, active, E, s_warp, s_total, ra, rb);
    if (threadIdx.x < E) counts[blockIdx.x * 32u + threadIdx.x] = s_total[threadIdx.x];
    if (threadIdx.x == 0) {
        flags[blockIdx.x] = (uint32_t)s_bad;
        __threadfence();
        s_last = atomicAdd(counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // last block: exclusive scan of the per-block counts over blocks, one warp per expert
    uint32_t bad = 0;
    for (uint32_t b = threadIdx.x; b < gridDim.x; b += kRouteBlock) bad |= __ldcg(flags + b);
    if (bad) atomicExch(&s_bad, 2);
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t e = warp; e < E; e += kRouteBlock / 32) {
        uint32_t running = 0;
        for (uint32_t b0 = 0; b0 < gridDim.x; b0 += 32) {
            const uint32_t b = b0 + lane;
            const uint32_t v = b < gridDim.x ? __ldcg(counts + b * 32u + e) : 0u;
            uint32_t inc = v;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const uint32_t n = __shfl_up_sync(0xffffffffu, inc, off);
                if ((int)lane >= off) inc += n;
            }
            if (b < gridDim.x) counts[b * 32u + e] = running + inc - v;
            running += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) s_total[e] = running;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool any_bad = s_bad != 0;
        summary[0] = any_bad ? 1u : 0u;
        if (any_bad) {
            kstatus_set(status, FE2O3_KSTATUS_NONFINITE);
        } else {
            uint32_t *requested = reinterpret_cast<uint32_t *>(a.requested_counts.ptr);
            uint32_t *admitted = reinterpret_cast<uint32_t *>(a.admitted_counts.ptr);
            uint32_t *offsets = reinterpret_cast<uint32_t *>(a.expert_offsets.ptr);
            uint32_t off = 0;
            offsets[0] = 0;
            for (uint32_t e = 0; e < E; ++e) {
                const uint32_t adm = s_total[e] > a.capacity ? a.capacity : s_total[e];
                requested[e] = s_total[e];
                admitted[e] = adm;
                off += adm;
                offsets[e + 1] = off;
            }
        }
        *counter = 0u;  // re-arm for the next launch
    }
}

__global__ void __launch_bounds__(kRouteBlock)
moe_route_place_kernel(fe2o3_moe_top2_v1_args a, const uint32_t *scratch) {
    __shared__ uint32_t s_warp[kRouteBlock / 32][32];
    __shared__ uint32_t s_total[32];
    const uint32_t T = a.tokens, E = a.experts, cap = a.capacity;
    const uint64_t R = 2ull * T;
    const uint32_t *base = scratch + blockIdx.x * 32u;
    const uint32_t *summary = scratch + FE2O3_ROUTE_MAX_BLOCKS * 33u;
    if (__ldcg(summary) != 0u) return;  // failure preserves every output
    const uint32_t *offsets = reinterpret_cast<const uint32_t *>(a.expert_offsets.ptr);
    uint32_t *top2 = reinterpret_cast<uint32_t *>(a.top2_experts.ptr);
    uint32_t *slots = reinterpret_cast<uint32_t *>(a.route_slots.ptr);
    uint32_t *perm = reinterpret_cast<uint32_t *>(a.permutation.ptr);
    uint32_t *inverse = reinterpret_cast<uint32_t *>(a.inverse.ptr);
    const uint32_t t = blockIdx.x * kRouteBlock + threadIdx.x;
    const bool active = t < T;
    uint32_t best = 0, second = 0;
    bool finite = true;
    if (active) top2_of_row(reinterpret_cast<const float *>(a.logits.ptr) + (uint64_t)t * E, E, best, second, finite);
    uint32_t ra, rb;
    block_ranks(best, second, active, E, s_warp, s_total, ra, rb);
    // unused tail of the permutation
    const uint64_t accepted = offsets[E];
    for (uint64_t s = accepted + (uint64_t)blockIdx.x * kRouteBlock + threadIdx.x; s < R; s += (uint64_t)gridDim.x * kRouteBlock)
        perm[s] = kDrop;
    if (!active) return;
    const uint32_t ga = __ldcg(base + best) + ra, gb = __ldcg(base + second) + rb;
    const uint32_t sa = ga < cap ? offsets[best] + ga : kDrop;
    const uint32_t sb = gb < cap ? offsets[second] + gb : kDrop;
    top2[2ull * t] = best;
    top2[2ull * t + 1] = second;
    slots[2ull * t] = sa;
    slots[2ull * t + 1] = sb;
    inverse[2ull * t] = sa;
    inverse[2ull * t + 1] = sb;
    if (sa != kDrop) perm[sa] = 2u * t;
    if (sb != kDrop) perm[sb] = 2u * t + 1u;
}

// ---- route weights ------------------------------------------------------------
// One thread per token; the arithmetic is route_weight_pair (common.cuh).
__global__ void moe_route_weights_kernel(const float *__restrict__ logits, const uint32_t *__restrict__ top2,
                                         float *__restrict__ weights, uint32_t tokens, uint32_t experts) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens) return;
    const float l0 = logits[(uint64_t)t * experts + top2[2ull * t]];
    const float l1 = logits[(uint64_t)t * experts + top2[2ull * t + 1]];
    float w0, w1;
    route_weight_pair(l0, l1, w0, w1);
    weights[2ull * t] = w0;
    weights[2ull * t + 1] = w1;
}

// ---- compaction ---------------------------------------------------------------
// compact_x[slot,:] = x[permutation[slot] / 2, :] for accepted slots, zero rows
// elsewhere (examples/moe_expert_v1/src/pipeline.rs:181-215 builds zero-padded
// per-expert activation tiles the same way).  One block per slot, 16-byte copies.
__global__ void __launch_bounds__(256)
moe_compact_kernel(const uint4 *__restrict__ x, const uint32_t *__restrict__ perm, uint4 *__restrict__ compact_x,
                   uint32_t vec_per_row, uint32_t tokens) {
    const uint32_t slot = blockIdx.x;
    const uint32_t route = perm[slot];
    uint4 *dst = compact_x + (uint64_t)slot * vec_per_row;
    if (route == kDrop || (route >> 1) >= tokens) {
        for (uint32_t i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    const uint4 *src = x + (uint64_t)(route >> 1) * vec_per_row;
    for (uint32_t i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = __ldg(src + i);
}

// ---- combine --------------------------------------------------------------------
// examples/moe_expert_v1/src/kernel.rs:104-157: out[t,c] = sum over rank 0,1 in
// that order, from +0, of w[2t+rank] * compact[inverse[2t+rank], c]; dropped
// routes contribute nothing; a token whose weights are non-finite, negative or
// do not sum to exactly 1.0 is left unwritten and a status word is recorded.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float *__restrict__ compact, const uint32_t *__restrict__ inverse,
                   const float *__restrict__ weights, float *__restrict__ out, uint32_t tokens, uint32_t width,
                   uint64_t compact_rows, uint32_t *status) {
    const uint32_t t = blockIdx.x;
    if (t >= tokens) return;
    const float w0 = weights[2ull * t], w1 = weights[2ull * t + 1];
    if (!isfinite(w0) || !isfinite(w1) || w0 < 0.f || w1 < 0.f || __fadd_rn(w0, w1) != 1.0f) {
        if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_WEIGHTS);
        return;
    }
    const uint32_t s0 = inverse[2ull * t], s1 = inverse[2ull * t + 1];
    if ((s0 != kDrop && s0 >= compact_rows) || (s1 != kDrop && s1 >= compact_rows)) {
        if (threadIdx.x == 0) kstatus_set(status, FE2O3_KSTATUS_SLOT_RANGE);
        return;
    }
    const bool vec = (width & 3u) == 0 && ((reinterpret_cast<uint64_t>(compact) | reinterpret_cast<uint64_t>(out)) & 15u) == 0;
    if (vec) {
        const uint32_t nv = width >> 2;
        const float4 *r0 = s0 != kDrop ? reinterpret_cast<const float4 *>(compact + (uint64_t)s0 * width) : nullptr;
        const float4 *r1 = s1 != kDrop ? reinterpret_cast<const float4 *>(compact + (uint64_t)s1 * width) : nullptr;
        float4 *dst = reinterpret_cast<float4 *>(out + (uint64_t)t * width);
        for (uint32_t i = threadIdx.x; i < nv; i += blockDim.x) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r0) {
                float4 v = __ldcs(r0 + i);
                acc.x = __fadd_rn(acc.x, __fmul_rn(w0, v.x)); acc.y = __fadd_rn(acc.y, __fmul_rn(w0, v.y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(w0, v.z)); acc.w = __fadd_rn(acc.w, __fmul_rn(w0, v.w));
            }
            if (r1) {
                float4 v = __ldcs(r1 + i);
                acc.x = __fadd_rn(acc.x, __fmul_rn(w1, v.x)); acc.y = __fadd_rn(acc.y, __fmul_rn(w1, v.y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(w1, v.z)); acc.w = __fadd_rn(acc.w, __fmul_rn(w1, v.w));
            }
            __stcs(dst + i, acc);
        }
    } else {
        for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
            float acc = 0.f;
            if (s0 != kDrop) acc = __fadd_rn(acc, __fmul_rn(w0, compact[(uint64_t)s0 * width + c]));
            if (s1 != kDrop) acc = __fadd_rn(acc, __fmul_rn(w1, compact[(uint64_t)s1 * width + c]));
            out[(uint64_t)t * width + c] = acc;
        }
    }
}

}  // namespace

int32_t launch_moe_gate(fe2o3_ctx *, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_moe_gate_v1_args *a = static_cast<const fe2o3_moe_gate_v1_args *>(args);
    const uint32_t E = a->experts;
    const uint32_t tpb = E >= 256 ? 1 : 256 / E;
    const uint32_t grid = ceil_div_u32(a->tokens, tpb);
    const uint32_t smem = (tpb * (kGateKC + 1) + kGateKC * E) * sizeof(float);
    const bool per_token = E == 4 || E == 8 || E == 16;
    if (per_token) {
        // FE2O3_GATE_KERNEL=block | warp selects one of the two older kernels where the pairs kernel applies
        static const char *force = getenv("FE2O3_GATE_KERNEL");
        const bool aligned = ((a->x.ptr | a->wg.ptr) & 15u) == 0;
        const bool lanes_ok = !force && aligned && a->d_model % 64u == 0 && a->d_model >= 64u && (a->logits.ptr & 7u) == 0 &&
                              (uint64_t)a->d_model * E * 4u <= 96u * 1024u && a->tokens > 0;
        const uint16_t *x = reinterpret_cast<const uint16_t *>(a->x.ptr), *wg = reinterpret_cast<const uint16_t *>(a->wg.ptr);
        float *lg = reinterpret_cast<float *>(a->logits.ptr);
        if (lanes_ok) {
            // few tokens: two experts per lane (most warps, pace of the dependent sums); many: four per lane
            const bool wide = a->tokens > 4096u;
#define FE2O3_GATE_LANES(EE, g)                                                                                            \
    (wide ? launch_gate_lanes<EE, 4, 8, 6>(s, x, wg, lg, a->tokens, a->d_model, g)                                         \
          : launch_gate_lanes<EE, 2, 4, 8>(s, x, wg, lg, a->tokens, a->d_model, g))
            fe2o3_geometry g{};
            cudaError_t e = E == 4 ? FE2O3_GATE_LANES(4, &g) : E == 8 ? FE2O3_GATE_LANES(8, &g) : FE2O3_GATE_LANES(16, &g);
            if (geo) *geo = g;
            if (plan_only) return FE2O3_OK;
            e = E == 4 ? FE2O3_GATE_LANES(4, nullptr) : E == 8 ? FE2O3_GATE_LANES(8, nullptr) : FE2O3_GATE_LANES(16, nullptr);
#undef FE2O3_GATE_LANES
            if (e != cudaSuccess) return fe2o3_cuda_status(e, "moe_gate_v1");
            fe2o3_count_launch(1);
            return fe2o3_cuda_status(cudaGetLastError(), "moe_gate_v1");
        }
        const bool force_block = force && force[0] == 'b';
        // other shapes: up to 4096 tokens the warp-per-eight-tokens kernel (measured on B200 with d_model
        // 2048, 8 experts: 26 us against 34 us for the block kernel at 2048 tokens, 80 against 50 us at
        // 16384), beyond that the 32-token block kernel
        const bool warp_ok = !force_block && a->tokens <= 4096u && a->d_model % 64u == 0 && a->d_model >= 64u && aligned;
        const uint32_t g2 = ceil_div_u32(a->tokens, warp_ok ? 8u : (uint32_t)kGate2Tokens), thr = warp_ok ? 32u : 32 * (E / 4);
        if (geo) *geo = fe2o3_geometry{{g2, 1, 1}, {thr, 1, 1}, 0, 1};
        if (plan_only || a->tokens == 0) return FE2O3_OK;
        if (warp_ok) {
            if (E == 4) moe_gate_warp_kernel<4><<<g2, 32, 0, s>>>(x, wg, lg, a->tokens, a->d_model);
            else if (E == 8) moe_gate_warp_kernel<8><<<g2, 32, 0, s>>>(x, wg, lg, a->tokens, a->d_model);
            else moe_gate_warp_kernel<16><<<g2, 32, 0, s>>>(x, wg, lg, a->tokens, a->d_model);
            fe2o3_count_launch(1);
            return fe2o3_cuda_status(cudaGetLastError(), "moe_gate_v1");
        }
        if (E == 4) moe_gate_staged_kernel<4><<<g2, thr, 0, s>>>(x, wg, lg, a->tokens, a->d_model);
        else if (E == 8) moe_gate_staged_kernel<8><<<g2, thr, 0, s>>>(x, wg, lg, a->tokens, a->d_model);
        else moe_gate_staged_kernel<16><<<g2, thr, 0, s>>>(x, wg, lg, a->tokens, a->d_model);
        fe2o3_count_launch(1);
        return fe2o3_cuda_status(cudaGetLastError(), "moe_gate_v1");
    }
    if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {E, tpb, 1}, smem, 1};
    if (plan_only || a->tokens == 0) return FE2O3_OK;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(moe_gate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    moe_gate_kernel<<<grid, dim3(E, tpb, 1), smem, s>>>(reinterpret_cast<const uint16_t *>(a->x.ptr),
                                                        reinterpret_cast<const uint16_t *>(a->wg.ptr),
                                                        reinterpret_cast<float *>(a->logits.ptr), a->tokens,
                                                        a->d_model, E);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "moe_gate_v1");
}

int32_t launch_moe_top2(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_moe_top2_v1_args *a = static_cast<const fe2o3_moe_top2_v1_args *>(args);
    const uint32_t blocks = ceil_div_u32(a->tokens ? a->tokens : 1, kRouteBlock);
    // FE2O3_ROUTE_SINGLE_BLOCK=1 selects the one-block kernel (otherwise used beyond 4M tokens)
    static const bool force_single = getenv("FE2O3_ROUTE_SINGLE_BLOCK") != nullptr;
    if (blocks <= FE2O3_ROUTE_MAX_BLOCKS && !force_single) {
        if (geo) *geo = fe2o3_geometry{{blocks, 1, 1}, {kRouteBlock, 1, 1}, 0, 2};
        if (plan_only) return FE2O3_OK;
        moe_route_count_kernel<<<blocks, kRouteBlock, 0, s>>>(*a, ctx->route_scratch, ctx->status_word);
        moe_route_place_kernel<<<blocks, kRouteBlock, 0, s>>>(*a, ctx->route_scratch);
        fe2o3_count_launch(2);
        return fe2o3_cuda_status(cudaGetLastError(), "moe_top2_v1");
    }
    const uint32_t smem = a->experts * kRouteThreads * sizeof(uint32_t);
    if (geo) *geo = fe2o3_geometry{{1, 1, 1}, {kRouteThreads, 1, 1}, smem, 1};
    if (plan_only) return FE2O3_OK;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(moe_top2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    moe_top2_kernel<<<1, kRouteThreads, smem, s>>>(*a, ctx->status_word);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "moe_top2_v1");
}

int32_t launch_moe_route_weights(fe2o3_ctx *, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_moe_route_weights_v1_args *a = static_cast<const fe2o3_moe_route_weights_v1_args *>(args);
    const uint32_t grid = ceil_div_u32(a->tokens, 256);
    if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {256, 1, 1}, 0, 1};
    if (plan_only || a->tokens == 0) return FE2O3_OK;
    moe_route_weights_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const float *>(a->logits.ptr),
                                                  reinterpret_cast<const uint32_t *>(a->top2_experts.ptr),
                                                  reinterpret_cast<float *>(a->route_weights.ptr), a->tokens,
                                                  a->experts);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "moe_route_weights_v1");
}

int32_t launch_moe_compact(cudaStream_t s, uint64_t x, uint64_t perm, uint64_t compact_x, uint32_t rows,
                           uint32_t d_model, uint32_t tokens) {
    if (rows == 0) return FE2O3_OK;
    moe_compact_kernel<<<rows, 256, 0, s>>>(reinterpret_cast<const uint4 *>(x), reinterpret_cast<const uint32_t *>(perm),
                                            reinterpret_cast<uint4 *>(compact_x), d_model / 8, tokens);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "moe_compact");
}

int32_t launch_moe_combine(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_moe_expert_combine_v1_args *a = static_cast<const fe2o3_moe_expert_combine_v1_args *>(args);
    if (geo) *geo = fe2o3_geometry{{a->tokens, 1, 1}, {256, 1, 1}, 0, 1};
    if (plan_only || a->tokens == 0) return FE2O3_OK;
    moe_combine_kernel<<<a->tokens, 256, 0, s>>>(
        reinterpret_cast<const float *>(a->compact_output.ptr), reinterpret_cast<const uint32_t *>(a->inverse.ptr),
        reinterpret_cast<const float *>(a->route_weights.ptr), reinterpret_cast<float *>(a->combined_output.ptr),
        a->tokens, a->width, a->width ? a->compact_output.len / a->width : 0, ctx->status_word);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "moe_expert_combine_v1");
}

static Fe2o3KernelRegistration reg_top2("moe_top2_v1", reinterpret_cast<const void *>(moe_route_place_kernel));
static Fe2o3KernelRegistration reg_gate("moe_gate_v1", reinterpret_cast<const void *>(moe_gate_lanes_kernel<8, 4, 8, 6>));
static Fe2o3KernelRegistration reg_weights("moe_route_weights_v1", reinterpret_cast<const void *>(moe_route_weights_kernel));
static Fe2o3KernelRegistration reg_compact("moe_compact_v1", reinterpret_cast<const void *>(moe_compact_kernel));
static Fe2o3KernelRegistration reg_combine("moe_expert_combine_v1", reinterpret_cast<const void *>(moe_combine_kernel));
