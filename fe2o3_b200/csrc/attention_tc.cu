// Tensor-core attention for sm_100a: bf16 Q/K/V, f32 output, head_dim 64.
//
// Same recurrence as the reference kernel
// (examples/flash_attention_v1/src/kernel.rs:56-113: running maximum, rescale by
// exp(m_old - m_new), running denominator, out = acc / l) applied per block of
// 128 keys instead of per key, with both contractions on tcgen05:
//   S = Q * K^T   (A = Q tile, B = K tile, both K-major, accumulator in TMEM)
//   O += P * V    (A = P written as packed bf16 into tensor memory, B = V tile,
//                  MN-major, accumulator O stays in TMEM for the whole key loop)
//
// Work units.  A unit is one (batch, head) and 256 query rows handled as two
// 128-row tiles that share every K/V tile.  The kernel is persistent: one CTA
// per SM walks units b, b + grid, b + 2*grid, ... with every mbarrier ring
// running on across units, so the loads and the first Q*K^T of the next unit
// overlap the last exponentials and the output of the current one.  When the
// last round would leave more than half of the SMs idle its units are split
// into single 128-row tiles, one per CTA.
//
// Twelve warps: 0 = TMA producer, 1 and 2 = MMA issuers of tile 0 and tile 1
// (warp 1 owns the TMEM allocation), 3 idle, 4-7 = softmax for tile 0, 8-11 =
// softmax for tile 1.  A softmax thread owns one query row (one TMEM lane): it
// reads its 128 scores once into registers and releases S at once, so the next
// Q*K^T overlaps the exponentials.  (Splitting every row between two threads, 64
// keys and 32 output columns each, with the row maximum exchanged through
// shared memory, was measured on B200 and is slower, 495 against 566 TFLOP/s at
// the benchmark shape: the extra exchange lengthens each warp's chain more than
// the second warp per scheduler shortens the exponentials.)  Registers are
// re-balanced at the start: the warpgroup of the producer and the issuers gives
// most of its registers up, the two softmax warpgroups take them, so that a
// softmax thread keeps its 128 scores and 64 packed probabilities in registers.
// The exponent offset is a per-row reference
// maximum that is only moved (and O and l rescaled through TMEM) when the block
// maximum exceeds it by more than 2^8; the final quotient O / l is independent
// of the offset, so the result is the same function as the reference
// recurrence.  Scores are scaled inside exp2: p = 2^(s*c - m*c),
// c = scale * log2(e).  The output leaves through shared memory and bulk tensor
// stores.  All waits are bounded.
#include "common.cuh"
#include "gemm_tc.h"

#include <mutex>
#include <new>

namespace {

constexpr int D = 64;            // head dimension handled by this kernel
constexpr int BQ = 128;          // query rows per tile
constexpr int BKV = 128;         // keys per block
constexpr int QT = 2;            // query tiles per unit
constexpr int Q_STAGES = 2;
constexpr int KV_STAGES = 4;
constexpr uint32_t kTileParties = 1 + 4;             // per tile: its issuer and its four softmax warps (output staging)
constexpr uint32_t kQEmptyParties = QT * kTileParties;
constexpr int kSoftmaxWarps = 4 * QT;
#ifndef FE2O3_ATTN_REGS_CONTROL
#define FE2O3_ATTN_REGS_CONTROL 48
#define FE2O3_ATTN_REGS_SOFTMAX 224
#endif
constexpr int kRegsControl = FE2O3_ATTN_REGS_CONTROL;   // registers per thread of warps 0-3 after the re-balance
constexpr int kRegsSoftmax = FE2O3_ATTN_REGS_SOFTMAX;   // and of the softmax warps: 128 * 48 + 256 * 224 = 63488 <= 65536
static_assert(128 * kRegsControl + 256 * kRegsSoftmax <= 65536, "register file");
constexpr int kThreads = 32 * (4 + kSoftmaxWarps);
constexpr float kRescaleThreshold = 8.0f;  // log2 units
constexpr float kTruncGain = 1.001953125f;           // 1 + 2^-9: half a bf16 ulp, relative
constexpr float kTruncBiasLog2 = 0.0028150157f;      // log2(kTruncGain)

constexpr uint32_t kTileBytes = 128 * D * 2;     // 16 KiB: a 128 x 64 bf16 tile
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + Q_STAGES * QT * kTileBytes;
constexpr uint32_t kOffV = kOffK + KV_STAGES * kTileBytes;
constexpr uint32_t kOffBar = kOffV + KV_STAGES * kTileBytes;
constexpr uint32_t kSmemTotal = kOffBar + 512 + 1024;   // + alignment slack

// TMEM columns: S tile t at t*128 (128 f32 columns), O tile t at 256 + t*64 (64 f32 columns),
// P tile t at 384 + t*64 (128 bf16 per row = 64 columns).
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 256, kColP = 384;

struct AttnParams {
    float *out;
    uint32_t bh, seq;
    float scale_log2;   // scale * log2(e)
    uint32_t causal;
    uint32_t q_blocks;  // 256-row blocks per head
    uint32_t n_full;    // units of two tiles: indices [0, n_full)
    uint32_t n_half;    // single-tile units: indices [n_full, n_full + n_half), two per 256-row block
    uint32_t *status;
};

struct Unit {
    uint32_t head, q0, nt, nkv;
};

// The i-th unit of this CTA; false when the CTA has no i-th unit.  Every role walks the same sequence.
__device__ __forceinline__ bool unit_at(const AttnParams &p, uint32_t i, Unit &u) {
    const uint32_t idx = blockIdx.x + i * gridDim.x;
    uint32_t block, sub;
    if (idx < p.n_full) {
        block = idx; sub = 0; u.nt = QT;
    } else if (idx - p.n_full < p.n_half) {
        block = p.n_full + ((idx - p.n_full) >> 1); sub = (idx - p.n_full) & 1; u.nt = 1;
    } else {
        return false;
    }
    u.head = block / p.q_blocks;
    uint32_t qb = block % p.q_blocks;
    if (p.causal) qb = p.q_blocks - 1 - qb;   // the longest key ranges first
    u.q0 = qb * (QT * BQ) + sub * BQ;
    const uint32_t kv_limit = p.causal ? min(p.seq, u.q0 + u.nt * BQ) : p.seq;
    u.nkv = u.q0 < p.seq ? (kv_limit + BKV - 1) / BKV : 0;
    return true;
}

#ifdef FE2O3_ATTN_TRACE
// Development aid, compiled in only with -DFE2O3_ATTN_TRACE (the library built by `build.py --trace`): SM
// clock stamps of CTA 0's softmax warps (slot layout below) and, for every CTA, clock and wall-clock time at
// its start and end.  Read back with fe2o3_debug_attn_trace (fe2o3_b200/trace.py prints them).
//   [(tile*8 + block)*8 + k]          first unit, blocks 0..7: k = 0 before the S wait, 1 S here, 2 scores
//                                     loaded, 3 maximum done, 4 exponentials done, 5 P stored, 6 arrival made
//   [512 + (tile*8 + unit)*8 + k]     units 0..5: k = 0 begin, 1 blocks done, 2 last P*V done, 3 output done
//   [1024 + cta*4 + k]                k = 0/1 clock64 / globaltimer at the CTA's start, 2/3 at its end
__device__ unsigned long long g_attn_trace[2048];
__device__ __forceinline__ void attn_stamp(uint32_t slot) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
    g_attn_trace[slot] = t;
}
__device__ __forceinline__ void attn_stamp_cta(uint32_t slot) {
    unsigned long long t, ns;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns)::"memory");
    g_attn_trace[slot] = t;
    g_attn_trace[slot + 1] = ns;
}
#define ATTN_STAMP(cond, slot) do { if (cond) attn_stamp(slot); } while (0)
#define ATTN_STAMP_CTA(cond, slot) do { if (cond) attn_stamp_cta(slot); } while (0)
#else
#define ATTN_STAMP(cond, slot) do { } while (0)
#define ATTN_STAMP_CTA(cond, slot) do { } while (0)
#endif

// Register re-balance between warpgroups (all four warps of a warpgroup execute it).
template <int N>
__device__ __forceinline__ void regs_release() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void regs_take() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBar);
    uint64_t *q_full = bars;                       // Q_STAGES
    uint64_t *q_empty = q_full + Q_STAGES;
    uint64_t *k_full = q_empty + Q_STAGES;         // KV_STAGES
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
    ATTN_STAMP_CTA(threadIdx.x == 0 && blockIdx.x < 256, 1024 + blockIdx.x * 4);

    if (threadIdx.x == 0) {
        for (int i = 0; i < Q_STAGES; ++i) {
            mbar_init(&q_full[i], 1);
            mbar_init(&q_empty[i], kQEmptyParties);
        }
        for (int i = 0; i < KV_STAGES; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], QT);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], QT);
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
    // Each branch below opens with its own register re-balance, so that the code of a role is compiled
    // against that role's register count (a re-balance ahead of the branches would hold every role to
    // the smaller count).
    if (warp < 4) {
    regs_release<kRegsControl>();
    if (warp == 0) {
        // ---------------------------------------------------------- TMA producer
        // The whole warp runs the loop converged; one elected lane issues the copies.
        if (elect_one()) {
            tma_prefetch_desc(&tmQ);
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmV);
            tma_prefetch_desc(&tmO);
        }
        __syncwarp();
        bool ok = true;
        uint32_t g = 0;          // K/V blocks loaded so far, over all units
        uint32_t n_units = 0;
        Unit u;
        for (uint32_t i = 0; ok && unit_at(p, i, u); ++i) {
            if (u.nkv == 0) continue;   // every role skips a unit without keys (rows beyond seq)
            const uint32_t qs = n_units % Q_STAGES, qph = (n_units / Q_STAGES) & 1;
            ++n_units;
            if (!mbar_wait_warp(&q_empty[qs], qph ^ 1)) { ok = false; break; }
            if (elect_one()) {
                mbar_arrive_expect_tx(&q_full[qs], u.nt * kTileBytes);
                for (uint32_t t = 0; t < u.nt; ++t)
                    tma_load_3d(smem + kOffQ + (qs * QT + t) * kTileBytes, &tmQ, &q_full[qs], 0, (int32_t)(u.q0 + t * BQ),
                                (int32_t)u.head);
            }
            __syncwarp();
            for (uint32_t j = 0; j < u.nkv; ++j, ++g) {
                const uint32_t st = g % KV_STAGES, ph = (g / KV_STAGES) & 1;
                if (!mbar_wait_warp(&k_empty[st], ph ^ 1)) { ok = false; break; }
                if (elect_one()) {
                    mbar_arrive_expect_tx(&k_full[st], kTileBytes);
                    tma_load_3d(smem + kOffK + st * kTileBytes, &tmK, &k_full[st], 0, (int32_t)(j * BKV), (int32_t)u.head);
                }
                __syncwarp();
                if (!mbar_wait_warp(&v_empty[st], ph ^ 1)) {
                    ok = false;
                    mbar_wait_warp(&k_full[st], ph);   // the K copy just issued must land before the CTA exits
                    break;
                }
                if (elect_one()) {
                    mbar_arrive_expect_tx(&v_full[st], kTileBytes);
                    tma_load_3d(smem + kOffV + st * kTileBytes, &tmV, &v_full[st], 0, (int32_t)(j * BKV), (int32_t)u.head);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
        // drain the copies before the CTA can exit: the newest phase of every ring slot in use
        for (uint32_t b = 0; b < KV_STAGES && b < g; ++b) {
            const uint32_t last = g - 1 - b, st = last % KV_STAGES, ph = (last / KV_STAGES) & 1;
            mbar_wait_warp(&k_full[st], ph);
            mbar_wait_warp(&v_full[st], ph);
        }
        for (uint32_t b = 0; b < Q_STAGES && b < n_units; ++b) {
            const uint32_t last = n_units - 1 - b;
            mbar_wait_warp(&q_full[last % Q_STAGES], (last / Q_STAGES) & 1);
        }
    } else if (warp == 1 || warp == 2) {
        // ---------------------------------------------------------- MMA issuers, one warp per query tile
        // A single thread cannot issue the 24 small MMAs of a step (eight of them only 32 tensor-core
        // cycles long) fast enough for two tiles, so each tile has its own issuer.  The warp runs
        // converged and one elected lane issues.  Per tile the order is fixed: Q*K^T of block b+1 (its
        // S buffer is free as soon as the softmax has read block b), then P*V of block b (ready at the
        // end of that softmax step); block b+1 may already belong to the next unit.
        const uint32_t t = warp - 1;
        constexpr uint32_t idesc_qk = umma_idesc(1u, BQ, BKV, 0u, 0u);
        constexpr uint32_t idesc_pv = umma_idesc(1u, BQ, D, 0u, 1u);
        const uint32_t sQ = smem_u32(smem + kOffQ), sK = smem_u32(smem + kOffK), sV = smem_u32(smem + kOffV);
        // Descriptors are built once; inside the loops only the 16-byte-unit start address field moves.
        const uint64_t dQ = umma_smem_desc(sQ, 16, 1024), dK = umma_smem_desc(sK, 16, 1024),
                       dV = umma_smem_desc(sV, 8192, 1024);
        const uint32_t tS = tmem_base + t * BKV, tO = tmem_base + kColO + t * D, tP = tmem_base + kColP + t * (BKV / 2);
        bool ok = true;
        uint32_t g = 0;    // key blocks over all units: ring position of K/V
        uint32_t gt = 0;   // key blocks this tile has processed: parity of s_* / p_ready / pv_done
        uint32_t n = 0;    // units with keys seen so far (selects the Q stage)
        bool pending = false;                       // a P*V whose Q*K^T successor has been issued (or has none)
        uint32_t pv_st = 0, pv_ph = 0, pv_gt = 0, pv_acc = 0;
        auto issue_pv = [&]() {
            if (!mbar_wait_warp(&p_ready[t], pv_gt & 1) || !mbar_wait_warp(&v_full[pv_st], pv_ph)) { ok = false; return; }
            tc_fence_after();
            if (elect_one()) {
                const uint64_t dVs = dV + ((pv_st * kTileBytes) >> 4);
                umma_f16_ts(tO, tP, dVs, idesc_pv, pv_acc);
#pragma unroll
                for (int kk = 1; kk < BKV / 16; ++kk) umma_f16_ts(tO, tP + kk * 8, dVs + ((kk * 2048) >> 4), idesc_pv, 1u);
                umma_commit(&pv_done[t]);
                umma_commit(&v_empty[pv_st]);
            }
            __syncwarp();
            pending = false;
        };
        Unit u;
        for (uint32_t i = 0; ok && unit_at(p, i, u); ++i) {
            if (u.nkv == 0) continue;
            const uint32_t qs = n % Q_STAGES, qph = (n / Q_STAGES) & 1;
            ++n;
            if (t >= u.nt) {
                // a unit of one tile: this tile only hands its K/V blocks and its Q stage on
                if (pending) issue_pv();
                for (uint32_t j = 0; ok && j < u.nkv; ++j, ++g) {
                    const uint32_t st = g % KV_STAGES, ph = (g / KV_STAGES) & 1;
                    if (!mbar_wait_warp(&k_full[st], ph)) { ok = false; break; }
                    if (lane == 0) mbar_arrive(&k_empty[st]);
                    if (!mbar_wait_warp(&v_full[st], ph)) { ok = false; break; }
                    if (lane == 0) mbar_arrive(&v_empty[st]);
                }
                if (ok && !mbar_wait_warp(&q_full[qs], qph)) ok = false;
                if (ok && lane == 0) mbar_arrive_n(&q_empty[qs], kTileParties);   // for the absent tile's issuer and softmax warps
                continue;
            }
            if (!mbar_wait_warp(&q_full[qs], qph)) { ok = false; break; }
            const uint64_t dQt = dQ + (((qs * QT + t) * kTileBytes) >> 4);
            for (uint32_t j = 0; ok && j < u.nkv; ++j, ++g, ++gt) {
                const uint32_t st = g % KV_STAGES, ph = (g / KV_STAGES) & 1;
                if (!mbar_wait_warp(&s_empty[t], (gt & 1) ^ 1) || !mbar_wait_warp(&k_full[st], ph)) { ok = false; break; }
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t dKs = dK + ((st * kTileBytes) >> 4);
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk)
                        umma_f16(tS, dQt + ((kk * 32) >> 4), dKs + ((kk * 32) >> 4), idesc_qk, kk != 0);
                    umma_commit(&s_full[t]);
                    umma_commit(&k_empty[st]);
                    if (j + 1 == u.nkv) umma_commit(&q_empty[qs]);
                }
                __syncwarp();
                if (pending) issue_pv();
                pv_st = st; pv_ph = ph; pv_gt = gt; pv_acc = j != 0u;
                pending = true;
            }
        }
        if (ok && pending) issue_pv();
        if (!ok && lane == 0) kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
    }
    // warp 3 idles: it keeps the softmax warps at four per scheduler and their TMEM quadrant equal to warp % 4
    } else {
        regs_take<kRegsSoftmax>();
        // ---------------------------------------------------------- softmax warps
        constexpr int NCH = BKV / 32;                       // 32-column chunks of the score row
        constexpr int OCOLS = D;                            // output columns per thread
        const uint32_t sw = warp - 4;                       // 0 .. kSoftmaxWarps-1
        const uint32_t t = sw / 4;                          // query tile of this warp
        const uint32_t quad = warp & 3;                     // TMEM lane quadrant this warp may access
        const uint32_t r = quad * 32 + lane;                // row inside the tile
        const uint32_t lane_addr = (quad * 32u) << 16;
        const uint32_t tS = tmem_base + t * BKV + lane_addr;
        const uint32_t tO = tmem_base + kColO + t * D + lane_addr;
        const uint32_t tP = tmem_base + kColP + t * (BKV / 2) + lane_addr;
        const float c = p.scale_log2;
        bool ok = true;
        uint32_t gt = 0;             // key blocks this tile has processed, over all units
        uint32_t n = 0;              // units with keys seen so far (selects the Q stage)
        uint32_t ui = 0;
        Unit u;
        for (; ok && unit_at(p, ui, u); ++ui) {
            if (u.nkv == 0) continue;
            const uint32_t qs = n % Q_STAGES;
            ++n;
            if (t >= u.nt) continue;
            const uint32_t qrow = u.q0 + t * BQ + r;   // query index inside the head
            const bool utr = blockIdx.x == 0 && quad == 0 && lane == 0 && n <= 6;
            const uint32_t uslot = 512 + (t * 8 + (n - 1)) * 8;
            ATTN_STAMP(utr, uslot + 0);
            float m_ref = -INFINITY;   // exponent offset, in raw score units (identical in both halves)
            float l = 0.0f;            // this thread's share of the denominator
            bool s_early = false;      // s_full of the coming block was seen complete by the early probe

            for (uint32_t j = 0; j < u.nkv; ++j, ++gt) {
                // A probe of a barrier takes about 200 cycles even when the phase is complete, so the two
                // waits of a step are probed ahead of the long phases (S of the next block before the P
                // store of this one, P*V of the previous block before the exponentials) and only fall
                // back to the bounded wait when the early answer was "not yet".
                const bool tr = blockIdx.x == 0 && ui == 0 && quad == 0 && lane == 0 && j < 8;
                const uint32_t tslot = (t * 8 + j) * 8;
                ATTN_STAMP(tr, tslot + 0);
                if (!__all_sync(0xffffffffu, s_early) && !mbar_wait_warp(&s_full[t], gt & 1)) { ok = false; break; }
                s_early = false;
                ATTN_STAMP(tr, tslot + 1);
                tc_fence_after();
                // this thread's part of the score row into registers, then S is free for the next Q*K^T
                uint32_t s[NCH][32];
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch) tmem_ld_32x32b_x32(tS + ch * 32, s[ch]);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_empty[t]);
                ATTN_STAMP(tr, tslot + 2);

                const uint32_t key0 = j * BKV;
                const bool need_mask = (j * BKV + BKV > p.seq) || (p.causal && j * BKV + BKV - 1 > u.q0 + t * BQ);
                if (need_mask) {
#pragma unroll
                    for (int ch = 0; ch < NCH; ++ch) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const uint32_t key = key0 + ch * 32 + i;
                            const bool valid = key < p.seq && (!p.causal || key <= qrow);
                            if (!valid) s[ch][i] = 0xff800000u;  // -inf
                        }
                    }
                }
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            mx[q] = max3(mx[q], __uint_as_float(s[ch][i + 2 * q]), __uint_as_float(s[ch][i + 2 * q + 1]));
                    }
                }
                const float rowmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                // move the reference only when the block maximum outgrows it by more than the threshold
                const bool move = (rowmax - m_ref) * c > kRescaleThreshold;  // true for the first admitted key (m_ref = -inf)
                const float factor = move ? ex2_approx((m_ref - rowmax) * c) : 1.0f;  // 0 when m_ref = -inf
                if (move) m_ref = rowmax;
                // p = 2^(s*c - m_ref*c); a row with no admitted key so far keeps m_ref = -inf: use offset 0, p = 0
                const float mc = (m_ref == -INFINITY ? 0.0f : m_ref) * c;
                // The two tiles share the exponential unit: tile 1 starts its first exponential phase when
                // tile 0 has finished its own, so that afterwards one tile's exponentials (two warps per
                // scheduler, enough to keep the unit busy) overlap the other tile's loads, maxima and stores.
                if (gt == 0 && t == 1 && u.nt == QT && !mbar_wait_warp(stagger, 0)) { ok = false; break; }
                // Exponentials stay in registers as packed bf16 pairs until the P buffer is free.  The scale
                // and the sums run as packed pairs of f32.  P is cut to bf16 by truncation, which one byte
                // permute does for two values; the exponent carries a bias of log2(1 + 2^-9) so that the
                // truncation error is centred on zero like a rounding error, and the bias (also present in
                // the sums) is divided out with the denominator at the end.
                const bool pv_early = j > 0 && mbar_test(&pv_done[t], (gt - 1) & 1);
                const float mcb = mc - kTruncBiasLog2;
                ATTN_STAMP(tr && mcb < 1e30f, tslot + 3);
                const uint64_t c2 = pack_f32x2(c, c), nmc2 = pack_f32x2(-mcb, -mcb);
                uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};   // four pairs of +0.0f
                uint32_t pk[NCH][16];
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float e[8];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint64_t x2 = fma_f32x2(
                                pack_f32x2(__uint_as_float(s[ch][q * 8 + 2 * i]), __uint_as_float(s[ch][q * 8 + 2 * i + 1])), c2, nmc2);
                            float x0, x1;
                            unpack_f32x2(x2, x0, x1);
                            e[2 * i] = ex2_approx(x0);
                            e[2 * i + 1] = ex2_approx(x1);
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) sum2[i] = add_f32x2(sum2[i], pack_f32x2(e[2 * i], e[2 * i + 1]));
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            pk[ch][q * 4 + i] = __byte_perm(__float_as_uint(e[2 * i]), __float_as_uint(e[2 * i + 1]), 0x7632);
                    }
                }
                float sum[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float lo, hi;
                    unpack_f32x2(sum2[i], lo, hi);
                    sum[i] = lo + hi;
                }
                if (gt == 0 && t == 0) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(stagger);
                }
                // P of the previous block must have been consumed and O must be quiescent
                if (j > 0) {
                    if (!__all_sync(0xffffffffu, pv_early) && !mbar_wait_warp(&pv_done[t], (gt - 1) & 1)) { ok = false; break; }
                    tc_fence_after();
                    if (__any_sync(0xffffffffu, move)) {   // each thread rescales its own output columns
#pragma unroll 1
                        for (int g = 0; g < OCOLS / 8; ++g) {
                            uint32_t ov[8];
                            tmem_ld_32x32b_x8(tO + g * 8, ov);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 8; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * factor);
                            tmem_st_32x32b_x8(tO + g * 8, ov);
                        }
                    }
                }
                l = fmaf(l, factor, (sum[0] + sum[1]) + (sum[2] + sum[3]));
                ATTN_STAMP(tr && l < 1e38f, tslot + 4);
                if (j + 1 < u.nkv) s_early = mbar_test(&s_full[t], (gt + 1) & 1);
                // P as packed bf16 pairs into tensor memory: 16 columns per 32 keys
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch) tmem_st_32x32b_x16(tP + ch * 16, pk[ch]);
                tmem_st_wait();
                ATTN_STAMP(tr, tslot + 5);
                // publish P and any O rescale (both TMEM stores) to the MMA issuer
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_ready[t]);
                ATTN_STAMP(tr, tslot + 6);
            }
            if (!ok) break;
            ATTN_STAMP(utr, uslot + 1);
            if (!mbar_wait_warp(&pv_done[t], (gt - 1) & 1)) { ok = false; break; }
            ATTN_STAMP(utr, uslot + 2);
            tc_fence_after();
            const float l_row = l;
            // Output.  The unit's Q tile is dead once its last Q*K^T has completed (the s_full wait above
            // proved that), so the warp stages its 32 rows, 32 columns at a time, in a 4 KiB slice
            // (128-byte swizzle, so the 16-byte writes of a warp spread over all banks) and hands them to
            // the copy engine: full-line writes that do not hold the warp.  The Q stage is given back to
            // the producer when the copies have read the slices.
            const float inv = kTruncGain / l_row;   // the sums carry the gain of the truncation bias
            bool finite = isfinite(l_row) && l_row > 0.0f;
            uint8_t *slice = smem + kOffQ + (qs * QT + t) * kTileBytes + quad * 4096;
            const uint32_t row0 = u.q0 + t * BQ + quad * 32;   // first query row of this warp
#pragma unroll
            for (int g = 0; g < OCOLS / 32; ++g) {
                uint32_t ov[32];
                tmem_ld_32x32b_x32(tO + g * 32, ov);  // every lane takes part in the collective load
                tmem_ld_wait();
                float o[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    o[i] = __uint_as_float(ov[i]) * inv;
                    finite = finite && isfinite(o[i]);
                }
                if (g > 0) {
                    if (lane == 0) tma_store_wait_read();   // the slice is still being read by the previous copy
                    __syncwarp();
                }
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    *reinterpret_cast<float4 *>(slice + lane * 128 + ((k ^ (lane & 7)) * 16)) =
                        make_float4(o[4 * k], o[4 * k + 1], o[4 * k + 2], o[4 * k + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && row0 < p.seq) {   // rows beyond seq are clipped by the copy engine
                    tma_store_3d(&tmO, slice, (int32_t)(g * 32), (int32_t)row0, (int32_t)u.head);
                    tma_store_commit();
                }
            }
            // finite-input policy: a non-finite result is reported through the status word
            if (!finite && qrow < p.seq) kstatus_set(p.status, FE2O3_KSTATUS_NONFINITE);
            if (lane == 0) {
                tma_store_wait_read();
                mbar_arrive(&q_empty[qs]);
            }
            // the next unit's first P*V overwrites O: order this thread's reads of O before its p_ready arrival
            tc_fence_before();
            __syncwarp();
            ATTN_STAMP(utr, uslot + 3);
        }
        if (!ok && lane == 0) kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
    }
    tc_fence_before();
    __syncthreads();
    ATTN_STAMP_CTA(threadIdx.x == 0 && blockIdx.x < 256, 1024 + blockIdx.x * 4 + 2);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

struct AttnTcPlan {
    CUtensorMap tmQ, tmK, tmV, tmO;
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
    if (st == FE2O3_OK) {
        // output: f32 [bh][seq][64], stored in boxes of 32 rows x 32 columns (128 bytes per row)
        uint64_t ostrides[2] = {D * 4, (uint64_t)a->seq * D * 4};
        uint32_t obox[3] = {32, 32, 1};
        st = fe2o3_make_tmap_f32(&plan->tmO, a->output.ptr, 3, dims, ostrides, obox);
    }
    if (st != FE2O3_OK) { delete plan; return st; }
    // Schedule: one CTA per SM; full rounds of two-tile units, and a last partial round that is split
    // into single tiles when that keeps every tile on its own CTA.
    const uint32_t q_blocks = (a->seq + QT * BQ - 1) / (QT * BQ);
    const uint32_t units = bh * q_blocks;
    const uint32_t sms = ctx->sm_count > 0 ? (uint32_t)ctx->sm_count : 1u;
    uint32_t grid, n_full = units, n_half = 0;
    if (2 * units <= sms) {
        grid = 2 * units;
        n_full = 0;
        n_half = 2 * units;
    } else {
        grid = units < sms ? units : sms;
        const uint32_t rem = units % grid;
        if (rem != 0 && 2 * rem <= grid) {
            n_full = units - rem;
            n_half = 2 * rem;
        }
    }
    plan->p = AttnParams{reinterpret_cast<float *>(a->output.ptr), bh, a->seq, a->scale * 1.4426950408889634f, a->causal,
                         q_blocks, n_full, n_half, ctx->status_word};
    plan->grid = grid;
    *out = plan;
    return FE2O3_OK;
}

// Function attributes are per device: called by fe2o3_ctx_create with the context's device current.
int32_t attention_tc_init_device() {
    FE2O3_CUDA(cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal));
    return FE2O3_OK;
}

int32_t attention_tc_launch(const AttnTcPlan *plan, cudaStream_t s) {
    if (plan->grid == 0) return FE2O3_OK;
    attention_tc_kernel<<<plan->grid, kThreads, kSmemTotal, s>>>(plan->tmQ, plan->tmK, plan->tmV, plan->tmO, plan->p);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "flash_attention_v1(tcgen05)");
}

void attention_tc_geometry(const AttnTcPlan *plan, fe2o3_geometry *geo) {
    *geo = fe2o3_geometry{{plan->grid, 1, 1}, {kThreads, 1, 1}, kSmemTotal, 1};
}

void attention_tc_free(AttnTcPlan *plan) { delete plan; }

#ifdef FE2O3_ATTN_TRACE
// copies the 2048 stamps of the last launches to `out` (trace builds only; not part of the ABI header)
extern "C" int32_t fe2o3_debug_attn_trace(unsigned long long *out) {
    return cudaMemcpyFromSymbol(out, g_attn_trace, sizeof(unsigned long long) * 2048) == cudaSuccess ? 0 : -1;
}
#endif

static Fe2o3KernelRegistration reg_attention("flash_attention_v1", reinterpret_cast<const void *>(attention_tc_kernel));
