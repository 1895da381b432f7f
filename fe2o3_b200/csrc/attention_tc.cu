// Tensor-core attention for sm_100a: bf16 Q/K/V, f32 output, head_dim 64.
//
// Same recurrence as the reference kernel
// (examples/flash_attention_v1/src/kernel.rs:56-113: running maximum, rescale by
// exp(m_old - m_new), running denominator, out = acc / l) applied per block of
// 128 keys instead of per key, with both contractions on tcgen05:
//   S = Q * K^T   (A = Q tile, B = K tile, both K-major, accumulator in TMEM)
//   PV = P * V    (A = P written to shared memory as bf16, B = V tile, MN-major)
// One CTA owns one (batch, head) and 256 query rows as two 128-row tiles that
// share every K/V tile.  Ten warps: 0 = TMA producer, 1 = MMA issuer and TMEM
// owner, 2-5 = softmax for tile 0, 6-9 = softmax for tile 1.  A softmax thread
// owns one query row (TMEM lane), so row maxima and sums need no shuffles; the
// output accumulator lives in registers and each PV block is added with the
// block's rescale factor.  Scores are scaled inside exp2: p = 2^(s*c - m*c),
// c = scale * log2(e).  All waits are bounded.
#include "common.cuh"
#include "gemm_tc.h"

#include <mutex>
#include <new>

namespace {

constexpr int D = 64;            // head dimension handled by this kernel
constexpr int BQ = 128;          // query rows per tile
constexpr int BKV = 128;         // keys per block
constexpr int QT = 2;            // query tiles per CTA
constexpr int KV_STAGES = 2;
constexpr int kThreads = 32 * (2 + 4 * QT);

constexpr uint32_t kTileBytes = 128 * D * 2;     // 16 KiB: a 128 x 64 bf16 tile
constexpr uint32_t kPBytes = BQ * BKV * 2;       // 32 KiB: P tile as two 64-key sub-tiles
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + QT * kTileBytes;
constexpr uint32_t kOffV = kOffK + KV_STAGES * kTileBytes;
constexpr uint32_t kOffP = kOffV + KV_STAGES * kTileBytes;
constexpr uint32_t kOffBar = kOffP + QT * kPBytes;
constexpr uint32_t kSmemTotal = kOffBar + 512 + 1024;

// TMEM columns: S tile t at t*128 (128 f32 columns), PV tile t at 256 + t*64.
constexpr uint32_t kTmemCols = 512;

struct AttnParams {
    float *out;
    uint32_t bh, seq;
    float scale_log2;   // scale * log2(e)
    uint32_t causal;
    uint32_t *status;
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
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
    uint64_t *pv_full = p_ready + QT;
    uint64_t *pv_empty = pv_full + QT;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(pv_empty + QT);

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
            mbar_init(&pv_full[t], 1);
            mbar_init(&pv_empty[t], 4);
        }
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
            bool ever[KV_STAGES];
            for (int i = 0; i < KV_STAGES; ++i) { last_k[i] = last_v[i] = 0; ever[i] = false; }
            uint32_t stage = 0, phase = 0;
            for (uint32_t j = 0; j < nkv && ok; ++j) {
                if (!mbar_wait(&k_empty[stage], phase ^ 1)) { ok = false; break; }
                mbar_arrive_expect_tx(&k_full[stage], kTileBytes);
                tma_load_3d(smem + kOffK + stage * kTileBytes, &tmK, &k_full[stage], 0, (int32_t)(j * BKV), (int32_t)head);
                last_k[stage] = phase;
                if (!mbar_wait(&v_empty[stage], phase ^ 1)) { ever[stage] = true; last_v[stage] = 2; ok = false; break; }
                mbar_arrive_expect_tx(&v_full[stage], kTileBytes);
                tma_load_3d(smem + kOffV + stage * kTileBytes, &tmV, &v_full[stage], 0, (int32_t)(j * BKV), (int32_t)head);
                last_v[stage] = phase;
                ever[stage] = true;
                if (++stage == KV_STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
            // drain this thread's copies before the CTA can exit
            mbar_wait(q_full, 0);
            for (int i = 0; i < KV_STAGES; ++i) {
                if (!ever[i]) continue;
                mbar_wait(&k_full[i], last_k[i]);
                if (last_v[i] != 2) mbar_wait(&v_full[i], last_v[i]);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc(1u, BQ, BKV, 0u, 0u);
            constexpr uint32_t idesc_pv = umma_idesc(1u, BQ, D, 0u, 1u);
            const uint32_t sQ = smem_u32(smem + kOffQ), sK = smem_u32(smem + kOffK), sV = smem_u32(smem + kOffV),
                           sP = smem_u32(smem + kOffP);
            bool ok = mbar_wait(q_full, 0);
            uint32_t kst = 0, kph = 0, vst = 0, vph = 0;
            auto issue_pv = [&](uint32_t jj) -> bool {
                if (!mbar_wait(&v_full[vst], vph)) return false;
                for (int t = 0; t < QT; ++t) {
                    if (!mbar_wait(&p_ready[t], jj & 1)) return false;
                    if (!mbar_wait(&pv_empty[t], (jj & 1) ^ 1)) return false;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < BKV / 16; ++kk) {
                        const uint64_t adesc = umma_smem_desc(sP + t * kPBytes + (kk / 4) * kTileBytes + (kk % 4) * 32, 16, 1024);
                        const uint64_t bdesc = umma_smem_desc(sV + vst * kTileBytes + kk * 2048, 8192, 1024);
                        umma_f16(tmem_base + 256 + t * D, adesc, bdesc, idesc_pv, kk != 0);
                    }
                    umma_commit(&pv_full[t]);
                }
                umma_commit(&v_empty[vst]);
                if (++vst == KV_STAGES) { vst = 0; vph ^= 1; }
                return true;
            };
            for (uint32_t j = 0; j < nkv && ok; ++j) {
                if (!mbar_wait(&k_full[kst], kph)) { ok = false; break; }
                for (int t = 0; t < QT && ok; ++t) {
                    if (!mbar_wait(&s_empty[t], (j & 1) ^ 1)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint64_t adesc = umma_smem_desc(sQ + t * kTileBytes + kk * 32, 16, 1024);
                        const uint64_t bdesc = umma_smem_desc(sK + kst * kTileBytes + kk * 32, 16, 1024);
                        umma_f16(tmem_base + t * BKV, adesc, bdesc, idesc_qk, kk != 0);
                    }
                    umma_commit(&s_full[t]);
                }
                if (!ok) break;
                umma_commit(&k_empty[kst]);
                if (++kst == KV_STAGES) { kst = 0; kph ^= 1; }
                if (j > 0 && !issue_pv(j - 1)) { ok = false; break; }
            }
            if (ok && nkv > 0 && !issue_pv(nkv - 1)) ok = false;
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
        const uint32_t tPV = tmem_base + 256 + t * D + lane_addr;
        uint8_t *prow = smem + kOffP + t * kPBytes + (r >> 3) * 1024 + (r & 7) * 128;
        const float c = p.scale_log2;
        float m = -INFINITY, l = 0.0f, alpha_prev = 0.0f;
        float o[D];
#pragma unroll
        for (int i = 0; i < D; ++i) o[i] = 0.0f;
        bool ok = true;

        auto consume_pv = [&](uint32_t jj) -> bool {
            if (!mbar_wait(&pv_full[t], jj & 1)) return false;
            tc_fence_after();
#pragma unroll
            for (int h = 0; h < D / 32; ++h) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tPV + h * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[h * 32 + i] = fmaf(o[h * 32 + i], alpha_prev, __uint_as_float(v[i]));
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&pv_empty[t]);
            return true;
        };

        for (uint32_t j = 0; j < nkv; ++j) {
            if (!mbar_wait(&s_full[t], j & 1)) { ok = false; break; }
            tc_fence_after();
            const uint32_t key0 = j * BKV;
            const bool need_mask = (key0 + BKV > p.seq) || (p.causal && key0 + BKV - 1 > q0 + t * BQ);
            // pass 1: row maximum of the raw scores
            float rowmax = -INFINITY;
#pragma unroll 1
            for (int ch = 0; ch < BKV / 32; ++ch) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tS + ch * 32, v);
                tmem_ld_wait();
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const uint32_t key = key0 + ch * 32 + i;
                        const bool valid = key < p.seq && (!p.causal || key <= qrow);
                        rowmax = fmaxf(rowmax, valid ? __uint_as_float(v[i]) : -INFINITY);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) rowmax = fmaxf(rowmax, __uint_as_float(v[i]));
                }
            }
            const float m_new = fmaxf(m, rowmax);
            // a row with no admitted key yet keeps m = -inf; use 0 as the exponent offset then
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            const float alpha = exp2f((m - m_use) * c);
            // previous block's PV must be complete before P is overwritten; fold it in now
            if (j > 0 && !consume_pv(j - 1)) { ok = false; break; }
            // pass 2: p = 2^(s*c - m*c), row sum, P tile to shared memory (128-byte swizzled rows)
            const float mc = m_use * c;
            float rowsum = 0.0f;
#pragma unroll 1
            for (int ch = 0; ch < BKV / 32; ++ch) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tS + ch * 32, v);
                tmem_ld_wait();
                float pr[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float s = __uint_as_float(v[i]);
                    if (need_mask) {
                        const uint32_t key = key0 + ch * 32 + i;
                        const bool valid = key < p.seq && (!p.causal || key <= qrow);
                        s = valid ? s : -INFINITY;
                    }
                    pr[i] = exp2f(fmaf(s, c, -mc));
                    rowsum += pr[i];
                }
                // 32 keys = four 16-byte chunks; chunk index inside the 64-key sub-tile is XOR-swizzled by row
                uint8_t *sub = prow + (ch >> 1) * kTileBytes;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t chunk = ((ch & 1) * 4 + q) ^ (r & 7);
                    uint4 w = make_uint4(pack_bf16x2(pr[q * 8 + 0], pr[q * 8 + 1]), pack_bf16x2(pr[q * 8 + 2], pr[q * 8 + 3]),
                                         pack_bf16x2(pr[q * 8 + 4], pr[q * 8 + 5]), pack_bf16x2(pr[q * 8 + 6], pr[q * 8 + 7]));
                    *reinterpret_cast<uint4 *>(sub + chunk * 16) = w;
                }
            }
            l = fmaf(l, alpha, rowsum);
            m = m_new;
            alpha_prev = alpha;
            // S has been read twice: release it; publish P to the async proxy
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&s_empty[t]);
                mbar_arrive(&p_ready[t]);
            }
        }
        if (ok && nkv > 0 && !consume_pv(nkv - 1)) ok = false;
        if (!ok) {
            if (lane == 0) kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
        } else if (qrow < p.seq) {
            const float inv = 1.0f / l;
            bool finite = isfinite(l) && l > 0.0f;
#pragma unroll
            for (int i = 0; i < D; ++i) {
                o[i] *= inv;
                finite = finite && isfinite(o[i]);
            }
            if (!finite) {
                kstatus_set(p.status, FE2O3_KSTATUS_NONFINITE);  // finite-input policy: row left unwritten
            } else {
                float4 *dst = reinterpret_cast<float4 *>(p.out + ((uint64_t)head * p.seq + qrow) * D);
#pragma unroll
                for (int i = 0; i < D / 4; ++i) dst[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
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
