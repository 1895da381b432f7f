// Tensor-core attention for sm_100a: bf16 Q/K/V, f32 output, head_dim 64.
//
// Same recurrence as the reference kernel
// (examples/flash_attention_v1/src/kernel.rs:56-113: running maximum, rescale by
// exp(m_old - m_new), running denominator, out = acc / l) applied per block of
// 128 keys instead of per key, with both contractions on tcgen05:
//   S = Q * K^T   (A = Q tile, B = K tile, both K-major, accumulator in TMEM)
//   O += P * V    (A = P written as packed bf16 into tensor memory, B = V tile,
//                  MN-major, accumulator O stays in TMEM for the whole key loop)
// One CTA owns one (batch, head) and 256 query rows as two 128-row tiles that
// share every K/V tile.  Ten warps: 0 = TMA producer, 1 = MMA issuer and TMEM
// owner, 2-5 = softmax for tile 0, 6-9 = softmax for tile 1.  A softmax thread
// owns one query row (one TMEM lane): it reads its 128 scores once into
// registers and releases S at once, so the next Q*K^T overlaps the exponentials.
// The exponent offset is a per-row reference maximum that is only moved (and O
// and l rescaled through TMEM) when the block maximum exceeds it by more than
// 2^8; the final quotient O / l is independent of the offset, so the result is
// the same function as the reference recurrence.  Scores are scaled inside
// exp2: p = 2^(s*c - m*c), c = scale * log2(e).  All waits are bounded.
#include "common.cuh"
#include "gemm_tc.h"

#include <mutex>
#include <new>

namespace {

constexpr int D = 64;            // head dimension handled by this kernel
constexpr int BQ = 128;          // query rows per tile
constexpr int BKV = 128;         // keys per block
constexpr int QT = 2;            // query tiles per CTA
constexpr int KV_STAGES = 4;
constexpr int kThreads = 32 * (2 + 4 * QT);
constexpr float kRescaleThreshold = 8.0f;  // log2 units

constexpr uint32_t kTileBytes = 128 * D * 2;     // 16 KiB: a 128 x 64 bf16 tile
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + QT * kTileBytes;
constexpr uint32_t kOffV = kOffK + KV_STAGES * kTileBytes;
constexpr uint32_t kOffBar = kOffV + KV_STAGES * kTileBytes;
constexpr uint32_t kSmemTotal = kOffBar + 512 + 1024;

// TMEM columns: S tile t at t*128 (128 f32 columns), O tile t at 256 + t*64 (64 f32 columns),
// P tile t at 384 + t*64 (128 bf16 per row = 64 columns).
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 256, kColP = 384;
constexpr uint32_t kIssuerIdleLimit = 1u << 22;

struct AttnParams {
    float *out;
    uint32_t bh, seq;
    float scale_log2;   // scale * log2(e)
    uint32_t causal;
    uint32_t *status;
};

// Two probabilities to packed bf16 on the integer pipe (round half up: add half an ulp, keep the
// upper 16 bits).  The conversion instruction shares the quarter-rate unit with ex2, which is the
// bottleneck of this kernel; inputs here are finite and non-negative, so no NaN handling is needed.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}

__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBar);
    uint64_t *q_full = bars;                       // 1
    uint64_t *k_full = q_full + 1;                 // KV_STAGES
    uint64_t *k_empty = k_full + KV_STAGES;
    uint64_t *v_full = k_empty + KV_STAGES;
    uint64_t *v_empty = v_full + KV_STAGES;
    uint64_t *s_full = v_empty + KV_STAGES;        // QT
    uint64_t *s_empty = s_full + QT;
    uint64_t *p_ready = s_empty + QT;
    uint64_t *pv_done = p_ready + QT;
    uint64_t *stagger = pv_done + QT;              // 1: tile 0 finished its first exponential phase
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(stagger + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_blocks = (p.seq + QT * BQ - 1) / (QT * BQ);
    const uint32_t head = blockIdx.x / q_blocks;
    const uint32_t q0 = (blockIdx.x % q_blocks) * (QT * BQ);
    // keys this CTA must visit
    const uint32_t kv_limit = p.causal ? min(p.seq, q0 + QT * BQ) : p.seq;
    const uint32_t nkv = (kv_limit + BKV - 1) / BKV;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < KV_STAGES; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int t = 0; t < QT; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&s_empty[t], 4);
            mbar_init(&p_ready[t], 4);
            mbar_init(&pv_done[t], 1);
        }
        mbar_init(stagger, 4);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------- TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmQ);
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmV);
            bool ok = true;
            mbar_arrive_expect_tx(q_full, QT * kTileBytes);
            for (int t = 0; t < QT; ++t)
                tma_load_3d(smem + kOffQ + t * kTileBytes, &tmQ, q_full, 0, (int32_t)(q0 + t * BQ), (int32_t)head);
            uint32_t last_k[KV_STAGES], last_v[KV_STAGES];
            bool k_armed[KV_STAGES], v_armed[KV_STAGES];
            for (int i = 0; i < KV_STAGES; ++i) { last_k[i] = last_v[i] = 0; k_armed[i] = v_armed[i] = false; }
            uint32_t stage = 0, phase = 0;
            for (uint32_t j = 0; j < nkv && ok; ++j) {
                if (!mbar_wait(&k_empty[stage], phase ^ 1)) { ok = false; break; }
                mbar_arrive_expect_tx(&k_full[stage], kTileBytes);
                tma_load_3d(smem + kOffK + stage * kTileBytes, &tmK, &k_full[stage], 0, (int32_t)(j * BKV), (int32_t)head);
                last_k[stage] = phase;
                k_armed[stage] = true;
                if (!mbar_wait(&v_empty[stage], phase ^ 1)) { ok = false; break; }
                mbar_arrive_expect_tx(&v_full[stage], kTileBytes);
                tma_load_3d(smem + kOffV + stage * kTileBytes, &tmV, &v_full[stage], 0, (int32_t)(j * BKV), (int32_t)head);
                last_v[stage] = phase;
                v_armed[stage] = true;
                if (++stage == KV_STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
            // drain this thread's copies before the CTA can exit
            mbar_wait(q_full, 0);
            for (int i = 0; i < KV_STAGES; ++i) {
                if (k_armed[i]) mbar_wait(&k_full[i], last_k[i]);
                if (v_armed[i]) mbar_wait(&v_full[i], last_v[i]);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc(1u, BQ, BKV, 0u, 0u);
            constexpr uint32_t idesc_pv = umma_idesc(1u, BQ, D, 0u, 1u);
            const uint32_t sQ = smem_u32(smem + kOffQ), sK = smem_u32(smem + kOffK), sV = smem_u32(smem + kOffV);
            bool ok = mbar_wait(q_full, 0);
            // Descriptors are built once; inside the loops only the 16-byte-unit start address field moves.
            const uint64_t dQ = umma_smem_desc(sQ, 16, 1024), dK = umma_smem_desc(sK, 16, 1024),
                           dV = umma_smem_desc(sV, 8192, 1024);
            // The issuer polls: whichever of the four next operations (Q*K^T or P*V, tile 0 or 1) has
            // its operands ready is issued, so one tile never waits behind the other tile's softmax.
            uint32_t qk_j[QT], pv_j[QT], k_used[KV_STAGES], v_used[KV_STAGES];
            for (int t = 0; t < QT; ++t) qk_j[t] = pv_j[t] = 0;
            for (int i = 0; i < KV_STAGES; ++i) k_used[i] = v_used[i] = 0;
            uint32_t idle = 0;
            while (ok && (pv_j[0] < nkv || pv_j[QT - 1] < nkv)) {
                bool progress = false;
#pragma unroll
                for (int t = 0; t < QT; ++t) {
                    uint32_t j = pv_j[t];
                    if (j < nkv) {
                        const uint32_t st = j % KV_STAGES, ph = (j / KV_STAGES) & 1;
                        if (mbar_try_wait(&p_ready[t], j & 1) && mbar_try_wait(&v_full[st], ph)) {
                            tc_fence_after();
                            const uint64_t dVs = dV + ((st * kTileBytes) >> 4);
                            const uint32_t dst = tmem_base + kColO + t * D, src = tmem_base + kColP + t * (BKV / 2);
                            umma_f16_ts(dst, src, dVs, idesc_pv, j != 0u);
#pragma unroll
                            for (int kk = 1; kk < BKV / 16; ++kk)
                                umma_f16_ts(dst, src + kk * 8, dVs + ((kk * 2048) >> 4), idesc_pv, 1u);
                            umma_commit(&pv_done[t]);
                            if (++v_used[st] == QT) { umma_commit(&v_empty[st]); v_used[st] = 0; }
                            pv_j[t] = j + 1;
                            progress = true;
                        }
                    }
                    j = qk_j[t];
                    if (j < nkv) {
                        const uint32_t st = j % KV_STAGES, ph = (j / KV_STAGES) & 1;
                        if (mbar_try_wait(&s_empty[t], (j & 1) ^ 1) && mbar_try_wait(&k_full[st], ph)) {
                            tc_fence_after();
                            const uint64_t dQt = dQ + ((t * kTileBytes) >> 4), dKs = dK + ((st * kTileBytes) >> 4);
#pragma unroll
                            for (int kk = 0; kk < D / 16; ++kk)
                                umma_f16(tmem_base + t * BKV, dQt + ((kk * 32) >> 4), dKs + ((kk * 32) >> 4), idesc_qk, kk != 0);
                            umma_commit(&s_full[t]);
                            if (++k_used[st] == QT) { umma_commit(&k_empty[st]); k_used[st] = 0; }
                            qk_j[t] = j + 1;
                            progress = true;
                        }
                    }
                }
                if (progress) idle = 0;
                else if (++idle > kIssuerIdleLimit) ok = false;
            }
            if (!ok) kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
        }
    } else {
        // ---------------------------------------------------------- softmax warps
        const uint32_t t = (warp - 2) / 4;          // query tile of this warp
        const uint32_t quad = warp & 3;             // TMEM lane quadrant
        const uint32_t r = quad * 32 + lane;        // row inside the tile
        const uint32_t qrow = q0 + t * BQ + r;      // query index inside the head
        const uint32_t lane_addr = (quad * 32u) << 16;
        const uint32_t tS = tmem_base + t * BKV + lane_addr;
        const uint32_t tO = tmem_base + kColO + t * D + lane_addr;
        const uint32_t tP = tmem_base + kColP + t * (BKV / 2) + lane_addr;
        const float c = p.scale_log2;
        float m_ref = -INFINITY;   // exponent offset, in raw score units
        float l = 0.0f;
        bool ok = true;

        for (uint32_t j = 0; j < nkv; ++j) {
            if (!mbar_wait(&s_full[t], j & 1)) { ok = false; break; }
            tc_fence_after();
            // the whole score row into registers, then S is free for the next Q*K^T
            uint32_t s0[32], s1[32], s2[32], s3[32];
            tmem_ld_32x32b_x32(tS, s0);
            tmem_ld_32x32b_x32(tS + 32, s1);
            tmem_ld_32x32b_x32(tS + 64, s2);
            tmem_ld_32x32b_x32(tS + 96, s3);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[t]);

            const uint32_t key0 = j * BKV;
            const bool need_mask = (key0 + BKV > p.seq) || (p.causal && key0 + BKV - 1 > q0 + t * BQ);
            if (need_mask) {
                auto mask32 = [&](uint32_t (&s)[32], uint32_t base) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const uint32_t key = base + i;
                        const bool valid = key < p.seq && (!p.causal || key <= qrow);
                        if (!valid) s[i] = 0xff800000u;  // -inf
                    }
                };
                mask32(s0, key0);
                mask32(s1, key0 + 32);
                mask32(s2, key0 + 64);
                mask32(s3, key0 + 96);
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                mx0 = fmaxf(mx0, __uint_as_float(s0[i]));
                mx1 = fmaxf(mx1, __uint_as_float(s1[i]));
                mx2 = fmaxf(mx2, __uint_as_float(s2[i]));
                mx3 = fmaxf(mx3, __uint_as_float(s3[i]));
            }
            const float rowmax = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            // move the reference only when the block maximum outgrows it by more than the threshold
            const bool move = (rowmax - m_ref) * c > kRescaleThreshold;  // true for the first admitted key (m_ref = -inf)
            const float factor = move ? ex2_approx((m_ref - rowmax) * c) : 1.0f;  // 0 when m_ref = -inf
            if (move) m_ref = rowmax;
            // p = 2^(s*c - m_ref*c); a row with no admitted key so far keeps m_ref = -inf: use offset 0, p = 0
            const float mc = (m_ref == -INFINITY ? 0.0f : m_ref) * c;
            // The two tiles share the exponential unit: tile 1 starts its first exponential phase when
            // tile 0 has finished its own, so that afterwards one tile's exponentials overlap the other
            // tile's loads, maxima and stores instead of competing with them.
            if (j == 0 && t == 1 && !mbar_wait(stagger, 0)) { ok = false; break; }
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
            // exponentials stay in registers as packed bf16 pairs until the P buffer is free
            auto exp32 = [&](const uint32_t (&s)[32], uint32_t (&pk)[16]) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float e[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) e[i] = ex2_approx(fmaf(__uint_as_float(s[q * 8 + i]), c, -mc));
                    sum0 += e[0] + e[4];
                    sum1 += e[1] + e[5];
                    sum2 += e[2] + e[6];
                    sum3 += e[3] + e[7];
#pragma unroll
                    for (int i = 0; i < 4; ++i) pk[q * 4 + i] = pack_bf16x2(e[2 * i], e[2 * i + 1]);
                }
            };
            uint32_t pk0[16], pk1[16], pk2[16], pk3[16];
            exp32(s0, pk0);
            exp32(s1, pk1);
            exp32(s2, pk2);
            exp32(s3, pk3);
            if (j == 0 && t == 0) {
                __syncwarp();
                if (lane == 0) mbar_arrive(stagger);
            }
            // P of the previous block must have been consumed and O must be quiescent
            if (j > 0) {
                if (!mbar_wait(&pv_done[t], (j - 1) & 1)) { ok = false; break; }
                tc_fence_after();
                if (__any_sync(0xffffffffu, move)) {
#pragma unroll 1
                    for (int h = 0; h < D / 8; ++h) {
                        uint32_t ov[8];
                        tmem_ld_32x32b_x8(tO + h * 8, ov);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 8; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * factor);
                        tmem_st_32x32b_x8(tO + h * 8, ov);
                    }
                    tmem_st_wait();
                }
            }
            l = fmaf(l, factor, (sum0 + sum1) + (sum2 + sum3));
            // P as packed bf16 pairs into tensor memory: 16 columns per 32 keys
            tmem_st_32x32b_x16(tP, pk0);
            tmem_st_32x32b_x16(tP + 16, pk1);
            tmem_st_32x32b_x16(tP + 32, pk2);
            tmem_st_32x32b_x16(tP + 48, pk3);
            tmem_st_wait();
            // publish P and any O rescale (both TMEM stores) to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[t]);
        }
        if (ok && nkv > 0 && !mbar_wait(&pv_done[t], (nkv - 1) & 1)) ok = false;
        if (!ok) {
            if (lane == 0) kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
        } else if (nkv > 0) {
            tc_fence_after();
            const float inv = 1.0f / l;
            bool finite = isfinite(l) && l > 0.0f;
            float *dst = p.out + ((uint64_t)head * p.seq + qrow) * D;
            uint32_t ov[D];
            {
                uint32_t (&o0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&ov[0]);
                uint32_t (&o1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&ov[32]);
                tmem_ld_32x32b_x32(tO, o0);  // every lane takes part in the collective loads
                tmem_ld_32x32b_x32(tO + 32, o1);
                tmem_ld_wait();
            }
            float o[D];
#pragma unroll
            for (int i = 0; i < D; ++i) {
                o[i] = __uint_as_float(ov[i]) * inv;
                finite = finite && isfinite(o[i]);
            }
            // finite-input policy: a row with a non-finite result is left unwritten and reported
            if (qrow < p.seq) {
                if (!finite) {
                    kstatus_set(p.status, FE2O3_KSTATUS_NONFINITE);
                } else {
#pragma unroll
                    for (int i = 0; i < D / 4; ++i)
                        reinterpret_cast<float4 *>(dst)[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

struct AttnTcPlan {
    CUtensorMap tmQ, tmK, tmV;
    AttnParams p;
    uint32_t grid;
};

bool attention_tc_supported(const fe2o3_flash_attention_v1_args *a) {
    return a->input_dtype == FE2O3_DTYPE_BF16 && a->dim == D && a->seq >= 1 && a->batch * a->heads >= 1 &&
           ((a->q.ptr | a->k.ptr | a->v.ptr | a->output.ptr) & 15u) == 0 && a->scale > 0.0f && a->scale < 1e30f;
}

int32_t attention_tc_plan(fe2o3_ctx *ctx, const fe2o3_flash_attention_v1_args *a, AttnTcPlan **out) {
    AttnTcPlan *plan = new (std::nothrow) AttnTcPlan();
    if (!plan) return FE2O3_ERR_SIZE_OVERFLOW;
    const uint32_t bh = a->batch * a->heads;
    uint64_t dims[3] = {D, a->seq, bh};
    uint64_t strides[2] = {D * 2, (uint64_t)a->seq * D * 2};
    uint32_t box[3] = {D, 128, 1};
    int32_t st = fe2o3_make_tmap_bf16(&plan->tmQ, a->q.ptr, 3, dims, strides, box);
    if (st == FE2O3_OK) st = fe2o3_make_tmap_bf16(&plan->tmK, a->k.ptr, 3, dims, strides, box);
    if (st == FE2O3_OK) st = fe2o3_make_tmap_bf16(&plan->tmV, a->v.ptr, 3, dims, strides, box);
    if (st != FE2O3_OK) { delete plan; return st; }
    plan->p = AttnParams{reinterpret_cast<float *>(a->output.ptr), bh, a->seq, a->scale * 1.4426950408889634f, a->causal,
                         ctx->status_word};
    plan->grid = bh * ((a->seq + QT * BQ - 1) / (QT * BQ));
    *out = plan;
    return FE2O3_OK;
}

int32_t attention_tc_launch(const AttnTcPlan *plan, cudaStream_t s) {
    static std::once_flag once;
    std::call_once(once, [] {
        cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal);
    });
    if (plan->grid == 0) return FE2O3_OK;
    attention_tc_kernel<<<plan->grid, kThreads, kSmemTotal, s>>>(plan->tmQ, plan->tmK, plan->tmV, plan->p);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "flash_attention_v1(tcgen05)");
}

void attention_tc_geometry(const AttnTcPlan *plan, fe2o3_geometry *geo) {
    *geo = fe2o3_geometry{{plan->grid, 1, 1}, {kThreads, 1, 1}, kSmemTotal, 1};
}

void attention_tc_free(AttnTcPlan *plan) { delete plan; }
