// Tensor-core GEMM schedule for sm_100a: bf16 x bf16 -> f32 on tcgen05 with the
// accumulator in TMEM, operands staged by TMA into 128-byte-swizzled shared
// memory through an mbarrier ring.
//
// Replaces the MFMA + LDS schedule of examples/tiled_gemm_v1/src/kernel.rs:63-124
// and examples/tiled_gemm_general_v1/src/kernel.rs:67-120 (one wave per 16x16
// tile, single-buffered LDS, two barriers per K phase) and, in grouped mode,
// the per-expert GEMM launches of examples/moe_expert_v1/src/pipeline.rs:181-187.
//
// Layout.  A is row-major [M][K] (K contiguous, "K-major"); B is row-major
// [K][N] (N contiguous, "MN-major") exactly as the reference stores them, so no
// transpose pass is needed: the instruction descriptor marks B as MN-major.
// A CTA owns a 128 x BN output tile; one K block is 64 bf16 = 128 bytes.
//   A stage: one TMA box {64 k, 128 rows}  -> 128 rows x 128 B, 8-row groups 1 KiB apart
//   B stage: BN/64 TMA boxes {64 n, 64 k}   -> per box 64 k-rows x 128 B (8 KiB)
// Persistent CTAs (one per SM) walk a static tile list; ten warps:
//   warp 0  TMA producer (one lane)        warp 1  MMA issuer (one lane) + TMEM owner
//   warps 2-9  epilogue: TMEM -> registers -> shared memory -> bulk tensor store,
//              two warps per TMEM lane quadrant, half of the tile's columns each
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the main
// loop of tile i+1.  Every wait is bounded: on expiry the kernel records
// FE2O3_KSTATUS_WAIT_EXPIRED, drains its own copies and returns.
#include "gemm_tc.h"

#include <mutex>

namespace {

constexpr int BM = 128;
constexpr int BK = 64;          // bf16 elements per K block (128 bytes)
constexpr int UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 32 * (2 + kEpilogueWarps);
constexpr int kGatherThreads = 128;  // four more warps when A is gathered row by row: fourteen warps count as sixteen in
                                     // the register file (registers go out to four warps at a time), which the
                                     // 128-register build of the kernel fills exactly; with two loader warps on the
                                     // 168-register build the gathered GEMM was 6 % slower than the one fed by TMA
                                     // and gained 11-18 us per MoE pass against the compaction pass, with four 40 us
constexpr int kGroupM = 16;     // m-tiles per rasterisation band (keeps a wave's A and B panels in L2)

template <int BN>
struct SmemLayout {
    static constexpr uint32_t kABytes = BM * BK * 2;
    static constexpr uint32_t kBBytes = BN * BK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kStagingOffset = kStages * kStageBytes;          // 4 KiB output slice per epilogue warp
    static constexpr uint32_t kBarOffset = kStagingOffset + kEpilogueWarps * 4096;
    static constexpr uint32_t kTotal = kBarOffset + 256 + 1024;  // barriers + alignment slack
};

struct TileCoord {
    uint32_t m0, n0, m_end, expert;
    uint32_t mt_index;   // running index of the 128-row tile over all groups (expert-parallel hand-over counters)
    bool valid;
};

// Static tile order.  Plain: bands of kGroupM m-tiles, m fastest inside a band.
// Grouped: expert-major; inside an expert m fastest.  Grouped with per-source waiting (first GEMM of
// the expert-parallel FFN): by the source rank of the tile's first row, this rank's own rows first
// (they never cross NVLink), then ranks +1, +2, ... which is the order in which the other ranks send
// to this one; inside a source by local expert, then m, n fastest.
__device__ __forceinline__ TileCoord decode_tile(uint32_t id, const GemmParams &p, uint32_t n_tiles,
                                                 const uint32_t *s_off, const uint32_t *s_pair) {
    TileCoord t;
    t.valid = false;
    t.expert = 0;
    t.m0 = t.n0 = t.m_end = t.mt_index = 0;
    if (p.experts == 0) {
        const uint32_t m_tiles = (p.M + BM - 1) / BM;
        if (id >= m_tiles * n_tiles) return t;
        const uint32_t band = id / (kGroupM * n_tiles);
        const uint32_t first_m = band * kGroupM;
        const uint32_t band_m = min((uint32_t)kGroupM, m_tiles - first_m);
        const uint32_t local = id - band * kGroupM * n_tiles;
        t.m0 = (first_m + local % band_m) * BM;
        t.n0 = (local / band_m);
        t.m_end = p.M;
        t.valid = true;
        return t;
    }
    if (p.ep.rows_flags || p.ep.progress_mode) {
        // groups = (run j, local expert le): the tiles whose first row belongs to source (rank + j) mod W; inside
        // an expert's segment the runs lie in exactly that order (the owner's own rows first)
        const uint32_t W = p.ep.world;
        uint32_t base = 0;
        for (uint32_t g = 0; g < W * p.experts; ++g) {
            const uint32_t j = g / p.experts, le = g % p.experts;
            const uint32_t pi = le * W + j;
            const uint32_t seg = s_off[le], lo = s_pair[pi] - seg, hi = s_pair[pi + 1] - seg;
            const uint32_t i0 = (lo + BM - 1) / BM, i1 = (hi + BM - 1) / BM;   // tile starts seg + i * BM in [lo, hi)
            const uint32_t cnt = hi > lo ? (i1 - i0) * n_tiles : 0u;
            if (id < base + cnt) {
                const uint32_t local = id - base;
                const uint32_t mi = i0 + local / n_tiles;
                t.m0 = seg + mi * BM;
                t.n0 = local % n_tiles;
                t.m_end = s_off[le + 1];
                t.expert = le;
                t.mt_index = mi;
                for (uint32_t l2 = 0; l2 < le; ++l2) t.mt_index += (s_off[l2 + 1] - s_off[l2] + BM - 1) / BM;
                t.valid = true;
                break;
            }
            base += cnt;
        }
    } else {
        uint32_t base = 0;
        for (uint32_t e = 0; e < p.experts; ++e) {
            const uint32_t rows = s_off[e + 1] - s_off[e];
            const uint32_t mt = (rows + BM - 1) / BM;
            const uint32_t cnt = mt * n_tiles;
            if (id < base + cnt) {
                const uint32_t local = id - base;
                t.m0 = s_off[e] + (local % mt) * BM;
                t.n0 = local / mt;
                t.m_end = s_off[e + 1];
                t.expert = p.expert_mod ? e % p.expert_mod : e;   // index of the B matrix
                t.valid = true;
                break;
            }
            base += cnt;
        }
    }
    // The offsets come from shared memory, which the compiler must treat as lane-varying.  Every lane
    // of the (converged) calling warp holds the same values; taking them from lane 0 lets the TMA
    // coordinates live in uniform registers instead of being made uniform instruction by instruction
    // (that made the producer, not the tensor pipe, set the pace of the grouped GEMMs).
    t.m0 = __shfl_sync(0xffffffffu, t.m0, 0);
    t.n0 = __shfl_sync(0xffffffffu, t.n0, 0);
    t.m_end = __shfl_sync(0xffffffffu, t.m_end, 0);
    t.expert = __shfl_sync(0xffffffffu, t.expert, 0);
    t.mt_index = __shfl_sync(0xffffffffu, t.mt_index, 0);
    t.valid = __shfl_sync(0xffffffffu, (uint32_t)t.valid, 0) != 0;
    return t;
}

// erf by Abramowitz & Stegun 7.1.26 (absolute error below 1.5e-7, far under the bf16 step of the
// hidden activations this feeds): one reciprocal, one exp2 and a degree-5 polynomial, no branches.
__device__ __forceinline__ float gelu_erf(float x) {
    const float z = fabsf(x) * 0.70710678118654752440f;
    float t;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.0f)));
    float poly = fmaf(t, 1.061405429f, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    poly *= t;
    const float erf_abs = fmaf(-poly, ex2_approx(-1.4426950408889634f * z * z), 1.0f);
    const float half_x = 0.5f * x;
    return fmaf(half_x, copysignf(erf_abs, x), half_x);
}

// Two f32 to packed bf16, round to nearest even (hardware conversion; lo in the lower half).
__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// REGS = 168 is what the block's 320 threads can have; REGS = 128 (still no spills) is for the GEMM that runs
// beside the expert-parallel dispatch kernel: registers are handed out to four warps at a time, so the ten
// warps count as twelve, and 12 x 32 x 128 leaves room for one block of that kernel on the same SM.
template <int BN, int REGS>
__global__ void __maxnreg__(REGS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, GemmParams p) {
    using L = SmemLayout<BN>;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle atoms are 1 KiB: align the tile region.
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L::kBarOffset);
    uint64_t *empty = full + kStages;
    uint64_t *tmem_full = empty + kStages;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
    __shared__ uint32_t s_off[33];             // row segments of the groups
    __shared__ uint32_t s_pair[33];            // expert-parallel: rows of (local expert, source) pairs
    __shared__ unsigned long long s_peer[32];  // expert-parallel: return buffer of every rank
    __shared__ int s_abort;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n_tiles = (p.N + BN - 1) / BN;
    const uint32_t num_kb = (p.K + BK - 1) / BK;
    // the second GEMM of the expert FFN may take over each SM as this kernel's CTA leaves it
    if (p.ep.progress_mode == 1) launch_dependents();

    if (threadIdx.x == 0) {
        // Expert-parallel passes chain kernels through flags on other ranks: once a kernel of the pass has
        // reported a fault (a wait that ran out, a bad table), the later ones must not publish anything.
        // They find the status word set and do nothing but their arrival counting.
        s_abort = (p.ep.pair_offsets && p.status && __ldcg(p.status) != 0u) ? 1 : 0;
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&full[i], p.gather_perm ? 1 + kGatherThreads : 1);   // the producer's expect-tx arrival + every loader thread
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tmem_full[i], 1);
            mbar_init(&tmem_empty[i], kEpilogueWarps);
        }
        mbar_fence_init();
    }
    __shared__ int s_table_bad;
    const uint32_t ep_epoch = p.ep.epoch_counter ? __ldcg(p.ep.epoch_counter) + 1u : p.ep.epoch;
    // hand-over counters: two sets used by alternate passes; this pass's set was cleared during the previous one
    uint32_t *const progress = p.ep.progress ? p.ep.progress + (ep_epoch & 1u) * p.ep.progress_len : nullptr;
    if (p.experts && threadIdx.x == 64) {
        // The dispatch kernel that writes the table may still be running beside this kernel: wait for its
        // "table written" flag before reading (bounded like every wait).
        s_table_bad = 0;
        if (p.ep.table_flag && !flag_wait(p.ep.table_flag, ep_epoch, p.ep.spin_limit)) {
            s_table_bad = 1;
            kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
        }
#ifdef FE2O3_EP_TRACE
        if (p.ep.trace_flags && p.ep.table_flag && p.ep.progress_mode != 2 && blockIdx.x == 0) ep_trace(p.ep.trace_flags, FE2O3_EP_T_FFN1_TABLE_HERE);
#endif
        // The segment table is device data (in the expert-parallel layer it derives from other ranks'
        // counts): it is made monotone and cut off at M here, so that no row index derived from it can
        // leave A or C, and the fault is reported instead.
        const uint32_t stride = p.ep.pair_offsets ? p.ep.world : 1u;
        uint32_t prev = 0;
        bool bad = false;
        for (uint32_t i = 0; i <= p.experts; ++i) {
            uint32_t v = __ldcg(p.expert_offsets + i * stride);
            if (v < prev || v > p.M) { bad = true; v = v < prev ? prev : p.M; }
            s_off[i] = v;
            prev = v;
        }
        if (bad) kstatus_set(p.status, FE2O3_KSTATUS_SLOT_RANGE);
    }
    if (p.ep.pair_offsets && threadIdx.x == 64) {   // the thread that has waited for the table
        const uint32_t pairs = p.experts * p.ep.world;   // at most 32
        uint32_t prev = 0;
        for (uint32_t i = 0; i <= pairs; ++i) {   // monotone and inside A, like the segment table
            uint32_t v = __ldcg(p.ep.pair_offsets + i);
            v = v < prev ? prev : (v > p.M ? p.M : v);
            s_pair[i] = v;
            prev = v;
        }
    }
    if (p.ep.peer_ret)
        for (uint32_t i = threadIdx.x; i < p.ep.world; i += blockDim.x) s_peer[i] = p.ep.peer_ret[i];
#ifdef FE2O3_EP_TRACE
    if (p.ep.trace_flags && blockIdx.x == 0 && threadIdx.x == 0)
        ep_trace(p.ep.trace_flags, p.ep.rows_flags ? FE2O3_EP_T_FFN1_BEGIN : FE2O3_EP_T_FFN2_BEGIN);
#endif
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool dead = s_abort != 0 || (p.experts && s_table_bad);   // uniform over the CTA: read after the barrier, before any role can set it

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (warp converged, one elected lane issues)
        if (elect_one()) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmB);
        }
        __syncwarp();
        uint32_t stage = 0, phase = 0, loaded = 0;
        uint32_t seen = 0;   // sources whose "rows complete" flag this CTA has already acquired
        bool ok = !dead;
        for (uint32_t id = blockIdx.x; ok; id += gridDim.x) {
            TileCoord t = decode_tile(id, p, n_tiles, s_off, s_pair);
            if (!t.valid) break;
            if (p.ep.rows_flags) {
                // Sources with rows in this tile.  Their rows were written by the source ranks' SMs
                // (generic proxy, then a system-scope release of the flag); this warp acquires the flag
                // and orders that observation before its bulk tensor loads (asynchronous proxy) with a
                // proxy fence.
                const uint32_t hi = min(t.m0 + BM, t.m_end);
                uint32_t need = 0;
                if (lane < p.experts * p.ep.world && s_pair[lane] < hi && s_pair[lane + 1] > t.m0)
                    need = 1u << (lane % p.ep.world);
                need = __reduce_or_sync(0xffffffffu, need) & ~seen;
                seen |= need;
                while (need) {   // bit k = run k of a segment = source (rank + k) mod W
                    const uint32_t src = (p.ep.rank + __ffs(need) - 1) % p.ep.world;
                    need &= need - 1;
                    if (!__all_sync(0xffffffffu, flag_wait(p.ep.rows_flags + src, ep_epoch, p.ep.spin_limit))) { ok = false; break; }
                }
                if (!ok) break;
                fence_proxy_async_global();
#ifdef FE2O3_EP_TRACE
                if (blockIdx.x == 0 && lane == 0 && p.ep.trace_flags) {
                    if (id == blockIdx.x) ep_trace(p.ep.trace_flags, FE2O3_EP_T_FFN1_FIRST_WAIT_DONE);
                    if (seen == (1u << p.ep.world) - 1u) ep_trace(p.ep.trace_flags, FE2O3_EP_T_FFN1_LAST_WAIT_DONE);
                }
#endif
            }
            if (p.ep.progress_mode == 2) {
                // The rows of this tile are the first GEMM's output, stored by the copy engine (asynchronous
                // proxy) and announced through a counter: acquire the count, then order it before the bulk
                // tensor loads below.
                if (t.mt_index >= p.ep.progress_len ||
                    !__all_sync(0xffffffffu, flag_wait(progress + t.mt_index, p.ep.progress_target, p.ep.spin_limit))) {
                    ok = false;
                    break;
                }
                fence_proxy_async_global();
            }
            for (uint32_t kb = 0; kb < num_kb; ++kb, ++loaded) {
                if (!mbar_wait_warp(&empty[stage], phase ^ 1, &s_abort)) { ok = false; break; }
                if (elect_one()) {
                    uint8_t *sa = smem + stage * L::kStageBytes;
                    uint8_t *sb = sa + L::kABytes;
                    mbar_arrive_expect_tx(&full[stage], p.gather_perm ? L::kBBytes : L::kStageBytes);
                    if (!p.gather_perm) tma_load_2d(sa, &tmA, &full[stage], (int32_t)(kb * BK), (int32_t)t.m0);
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j) {
                        if (p.experts)
                            tma_load_3d(sb + j * 8192, &tmB, &full[stage], (int32_t)(t.n0 * BN + j * 64), (int32_t)(kb * BK),
                                        (int32_t)t.expert);
                        else
                            tma_load_2d(sb + j * 8192, &tmB, &full[stage], (int32_t)(t.n0 * BN + j * 64), (int32_t)(kb * BK));
                    }
                }
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok && lane == 0) {
            kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
            atomicExch(&s_abort, 1);
        }
        // Drain: every copy issued must have landed before the CTA exits (the newest phase of each ring slot).
        for (uint32_t b = 0; b < kStages && b < loaded; ++b) {
            const uint32_t last = loaded - 1 - b;
            mbar_wait_warp(&full[last % kStages], (last / kStages) & 1);
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (warp converged, one elected lane issues)
        constexpr uint32_t idesc = umma_idesc(1u, BM, BN, 0u, 1u);
        uint32_t stage = 0, phase = 0, it = 0;
        bool ok = !dead;
        const uint64_t desc_a0 = umma_smem_desc(smem_u32(smem), 16, 1024);
        const uint64_t desc_b0 = umma_smem_desc(smem_u32(smem) + L::kABytes, 8192, 1024);
        for (uint32_t id = blockIdx.x; ok; id += gridDim.x, ++it) {
            TileCoord t = decode_tile(id, p, n_tiles, s_off, s_pair);
            if (!t.valid) break;
            const uint32_t buf = it & 1, acc_phase = (it >> 1) & 1;
            if (!mbar_wait_warp(&tmem_empty[buf], acc_phase ^ 1, &s_abort)) { ok = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * BN;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_warp(&full[stage], phase, &s_abort)) { ok = false; break; }
                // gathered A rows were written by cp.async (generic proxy): order them before the tensor core's reads
                if (p.gather_perm) fence_proxy_async_smem();
                tc_fence_after();
                if (elect_one()) {
                    // only the 16-byte-unit start address field of the descriptors moves
                    const uint64_t adesc = desc_a0 + ((stage * L::kStageBytes) >> 4);
                    const uint64_t bdesc = desc_b0 + ((stage * L::kStageBytes) >> 4);
                    // A: K-major, advance 16 elements = 32 bytes inside the 128-byte row
                    // B: MN-major, advance 16 k-rows = 2 KiB; 64-column groups are 8 KiB apart
                    umma_f16(d_tmem, adesc, bdesc, idesc, kb != 0u);
#pragma unroll
                    for (int k = 1; k < BK / UMMA_K; ++k)
                        umma_f16(d_tmem, adesc + ((k * UMMA_K * 2) >> 4), bdesc + ((k * UMMA_K * 128) >> 4), idesc, 1u);
                    umma_commit(&empty[stage]);
                    if (kb + 1 == num_kb) umma_commit(&tmem_full[buf]);
                }
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok && lane == 0) {
            kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
            atomicExch(&s_abort, 1);
        }
    } else if (warp >= 2 + kEpilogueWarps) {
        // ------------------------------------------------ gather loaders (blocks launched with them only)
        // 128 threads fetch the tile's 128 rows of A for every K block: thread = (row mod 16, 16-byte chunk of
        // the row's 128 bytes), eight rows each, so that eight neighbouring lanes read one whole line.  The
        // rows go straight into the 128-byte-swizzled stage the tensor core reads; a row that is not a route
        // (past the group's end, or a dropped slot) is filled with zeros.  Completion is signalled to the
        // stage's barrier by the copies themselves.
        const uint32_t lt = threadIdx.x - 32 * (2 + kEpilogueWarps);
        const uint32_t chunk = lt & 7, r0 = lt >> 3;   // r0 in 0..15
        const uint8_t *src_base = reinterpret_cast<const uint8_t *>(p.gather_src);
        uint32_t stage = 0, phase = 0;
        bool ok = !dead;
        for (uint32_t id = blockIdx.x; ok; id += gridDim.x) {
            TileCoord t = decode_tile(id, p, n_tiles, s_off, s_pair);
            if (!t.valid) break;
            constexpr int kRowsPerThread = 128 * 8 / kGatherThreads;
            uint32_t tok[kRowsPerThread];
#pragma unroll
            for (int i = 0; i < kRowsPerThread; ++i) {
                const uint32_t row = t.m0 + r0 + (kGatherThreads / 8) * i;
                const uint32_t route = row < t.m_end ? __ldg(p.gather_perm + row) : 0xffffffffu;
                tok[i] = (route == 0xffffffffu || (route >> 1) >= p.gather_tokens) ? 0xffffffffu : (route >> 1);
            }
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_warp(&empty[stage], phase ^ 1, &s_abort)) { ok = false; break; }
                const uint32_t sa = smem_u32(smem + stage * L::kStageBytes) + r0 * 128 + ((chunk ^ (r0 & 7)) << 4);
                const uint64_t col = (uint64_t)kb * (BK * 2) + chunk * 16;
#pragma unroll
                for (int i = 0; i < kRowsPerThread; ++i) {
                    const bool live = tok[i] != 0xffffffffu;
                    const uint8_t *src = live ? src_base + (uint64_t)tok[i] * p.K * 2 + col : src_base;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sa + i * (kGatherThreads / 8) * 128), "l"(src), "r"(live ? 16 : 0) : "memory");
                }
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[stage])) : "memory");
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");   // no copy may be in flight when the block exits
        if (!ok && lane == 0) {
            kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
            atomicExch(&s_abort, 1);
        }
    } else {
        // ------------------------------------------------ epilogue warps
        // Eight warps: two per TMEM lane quadrant, each taking half of the tile's columns.  A warp
        // turns 128 bytes of each of its 32 rows at a time (32 f32 or 64 bf16 columns) into a
        // 128-byte-swizzled 4 KiB slice of shared memory and hands it to the copy engine, so the
        // global writes are full lines and do not hold the warp; ragged rows, the alpha/beta form and
        // outputs the copy engine cannot address are written by the threads directly.
        const uint32_t ew = warp - 2;
        const uint32_t quad = warp & 3;  // TMEM lane quadrant this warp may read
        const uint32_t col_half = ew >> 2;
        constexpr int kChunks = BN / 32 / 2;   // 32-column chunks per warp
        uint8_t *slice = smem + L::kStagingOffset + ew * 4096;
        const bool out_bf16 = p.epilogue == EPI_GELU_BF16;
        uint32_t it = 0;
        bool ok = !dead;
        bool store_pending = false;
        if (p.zero_ptr && !dead) {
            const uint64_t stride = (uint64_t)gridDim.x * (kEpilogueWarps * 32);
            for (uint64_t i = (uint64_t)blockIdx.x * (kEpilogueWarps * 32) + ew * 32 + lane; i < p.zero_vecs; i += stride)
                p.zero_ptr[i] = make_uint4(0u, 0u, 0u, 0u);
        }
        for (uint32_t id = blockIdx.x; ok; id += gridDim.x, ++it) {
            TileCoord t = decode_tile(id, p, n_tiles, s_off, s_pair);
            if (!t.valid) break;
            const uint32_t buf = it & 1, acc_phase = (it >> 1) & 1;
            if (!mbar_wait_warp(&tmem_full[buf], acc_phase, &s_abort)) { ok = false; break; }
            tc_fence_after();
            const uint32_t row0 = t.m0 + quad * 32;
            const uint32_t row = row0 + lane;
            const bool row_ok = row < t.m_end;
            const bool bulk = p.bulk_store && row0 + 32 <= t.m_end;   // warp-uniform
            const uint32_t col_base = t.n0 * BN + col_half * (BN / 2);
            const uint32_t taddr = tmem_base + buf * BN + col_half * (BN / 2) + ((quad * 32u) << 16);
            // scatter epilogue: where this lane's row goes (0 = nowhere)
            unsigned long long dst_row = 0;
            if (p.epilogue == EPI_SCATTER_PEER && row_ok) {
                const uint2 meta = __ldcg(p.ep.row_meta + row);   // (route id, home rank), written by the source rank
                if (meta.y < p.ep.world && meta.x < p.ep.ret_rows)
                    dst_row = s_peer[meta.y] + (unsigned long long)meta.x * p.N * sizeof(float);
                else
                    kstatus_set(p.status, FE2O3_KSTATUS_SLOT_RANGE);
            }
            float row_weight = 0.0f;
            if (p.epilogue == EPI_COMBINE_ADD && row_ok) {
                // where this lane's row is added and with which weight: route id of the slot, the token's two
                // weights checked like the separate combine does (finite, non-negative, summing to exactly 1)
                const uint32_t route = __ldg(p.combine_perm + row);
                if (route != 0xffffffffu && (route >> 1) < p.combine_tokens) {
                    const float w0 = __ldg(p.combine_weights + (route & ~1u)), w1 = __ldg(p.combine_weights + (route | 1u));
                    if (!isfinite(w0) || !isfinite(w1) || w0 < 0.f || w1 < 0.f || __fadd_rn(w0, w1) != 1.0f) {
                        kstatus_set(p.status, FE2O3_KSTATUS_WEIGHTS);
                    } else {
                        dst_row = reinterpret_cast<unsigned long long>(p.c) + (unsigned long long)(route >> 1) * p.N * sizeof(float);
                        row_weight = (route & 1u) ? w1 : w0;
                    }
                }
            }
            if (out_bf16) {
                // ---- GELU, bf16 output: two chunks (64 columns) per 128-byte group
#pragma unroll 1
                for (int g = 0; g < kChunks / 2; ++g) {
                    uint32_t w[32];
#pragma unroll
                    for (int c2 = 0; c2 < 2; ++c2) {
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(taddr + (g * 2 + c2) * 32, r);
                        tmem_ld_wait();
                        if (g == kChunks / 2 - 1 && c2 == 1) {   // the accumulator has been read completely
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            w[c2 * 16 + j] = cvt_bf16x2(gelu_erf(__uint_as_float(r[2 * j])), gelu_erf(__uint_as_float(r[2 * j + 1])));
                    }
                    const uint32_t col = col_base + g * 64;
                    if (col >= p.N) continue;
                    if (bulk) {
                        if (store_pending) {
                            if (lane == 0) tma_store_wait_read();
                            __syncwarp();
                        }
#pragma unroll
                        for (int k = 0; k < 8; ++k)
                            *reinterpret_cast<uint4 *>(slice + lane * 128 + ((k ^ (lane & 7)) * 16)) =
                                make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&tmC, slice, (int32_t)col, (int32_t)row0);
                            tma_store_commit();
                        }
                        store_pending = true;
                    } else if (row_ok) {
                        uint16_t *dst = reinterpret_cast<uint16_t *>(p.c) + (uint64_t)row * p.ldc + col;
                        if (col + 64 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
                            for (int k = 0; k < 8; ++k)
                                reinterpret_cast<uint4 *>(dst)[k] = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 64; ++j)
                                if (col + j < p.N) dst[j] = (uint16_t)(w[j >> 1] >> ((j & 1) * 16));
                        }
                    }
                }
            } else {
                // ---- f32 output: one chunk (32 columns) per 128-byte group
#pragma unroll 1
                for (int g = 0; g < kChunks; ++g) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(taddr + g * 32, r);
                    tmem_ld_wait();
                    if (g == kChunks - 1) {   // the accumulator has been read completely
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
                    }
                    const uint32_t col = col_base + g * 32;
                    if (col >= p.N) continue;
                    if (p.epilogue == EPI_SCATTER_PEER || p.epilogue == EPI_COMBINE_ADD) {
                        // Every row of the tile has its own destination (the return buffer of its home
                        // rank, at its route id).  The chunk is transposed through the warp's slice of
                        // shared memory so that each store instruction writes four whole 128-byte
                        // segments: eight lanes per row, one 16-byte piece each.
                        __syncwarp();   // the previous chunk has been read out of the slice
#pragma unroll
                        for (int k = 0; k < 8; ++k)
                            *reinterpret_cast<uint4 *>(slice + lane * 128 + ((k ^ (lane & 7)) * 16)) =
                                make_uint4(r[4 * k], r[4 * k + 1], r[4 * k + 2], r[4 * k + 3]);
                        __syncwarp();
                        const uint32_t piece = lane & 7;
#pragma unroll
                        for (int it = 0; it < 8; ++it) {
                            const uint32_t rr = it * 4 + (lane >> 3);
                            const uint4 v = *reinterpret_cast<const uint4 *>(slice + rr * 128 + ((piece ^ (rr & 7)) * 16));
                            const unsigned long long dst = __shfl_sync(0xffffffffu, dst_row, rr);
                            const float wgt = __shfl_sync(0xffffffffu, row_weight, rr);
                            if (dst != 0 && col + piece * 4 < p.N) {
                                const unsigned long long at = dst + (unsigned long long)(col + piece * 4) * sizeof(float);
                                if (p.epilogue == EPI_COMBINE_ADD)   // weight * row (one rounding), then one addition per element
                                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(at),
                                                 "f"(__fmul_rn(wgt, __uint_as_float(v.x))), "f"(__fmul_rn(wgt, __uint_as_float(v.y))),
                                                 "f"(__fmul_rn(wgt, __uint_as_float(v.z))), "f"(__fmul_rn(wgt, __uint_as_float(v.w)))
                                                 : "memory");
                                else
                                    *reinterpret_cast<uint4 *>(at) = v;
                            }
                        }
                    } else if (bulk && p.epilogue == EPI_STORE) {
                        if (store_pending) {
                            if (lane == 0) tma_store_wait_read();
                            __syncwarp();
                        }
#pragma unroll
                        for (int k = 0; k < 8; ++k)
                            *reinterpret_cast<uint4 *>(slice + lane * 128 + ((k ^ (lane & 7)) * 16)) =
                                make_uint4(r[4 * k], r[4 * k + 1], r[4 * k + 2], r[4 * k + 3]);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&tmC, slice, (int32_t)col, (int32_t)row0);
                            tma_store_commit();
                        }
                        store_pending = true;
                    } else if (row_ok) {
                        float *dst = reinterpret_cast<float *>(p.c) + (uint64_t)row * p.ldc + col;
                        const bool vec = col + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
                        if (p.epilogue == EPI_ALPHA_BETA) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < p.N)
                                    dst[j] = __fadd_rn(__fmul_rn(p.alpha, __uint_as_float(r[j])), __fmul_rn(p.beta, dst[j]));
                        } else if (vec) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                reinterpret_cast<uint4 *>(dst)[q] = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < p.N) dst[j] = __uint_as_float(r[j]);
                        }
                    }
                }
            }
            if (p.ep.progress_mode == 1) {
                // this warp's part of the hidden rows of the tile is in memory: bulk stores complete (not merely
                // read out of shared memory), direct stores fenced; then one count per warp
                if (store_pending) {
                    if (lane == 0) tma_store_wait_all();
                    store_pending = false;
                }
                __threadfence();
                __syncwarp();
                fence_proxy_async_global();
                if (lane == 0 && t.mt_index < p.ep.progress_len) atomicAdd(progress + t.mt_index, 1u);
            }
        }
        // the staging slice must stay intact until the last copy has read it
        if (store_pending && lane == 0) tma_store_wait_read();
        // rows stored into other ranks' memory must be visible there before "outputs ready" is raised
        if (p.epilogue == EPI_SCATTER_PEER) __threadfence_system();
        if (!ok && lane == 0) {
            kstatus_set(p.status, FE2O3_KSTATUS_WAIT_EXPIRED);
            atomicExch(&s_abort, 1);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * BN);
    }
#ifdef FE2O3_EP_TRACE
    if (p.ep.trace_flags && blockIdx.x == gridDim.x - 1 && threadIdx.x == 0)
        ep_trace(p.ep.trace_flags, p.ep.rows_flags ? FE2O3_EP_T_FFN1_END : FE2O3_EP_T_FFN2_END);
#endif
    if (p.ep.done_counter && threadIdx.x == 0) {
        // The last CTA of the grid to finish raises "outputs ready" on every rank, unless some CTA gave
        // up on a wait (the pass is void then).  A failed CTA still arrives, so the counter is re-armed.
        const bool failed = s_abort != 0;
        const uint32_t old = atomicAdd(p.ep.done_counter, failed ? 0x10001u : 1u);
        if ((old & 0xffffu) == gridDim.x - 1) {
            atomicExch(p.ep.done_counter, 0u);
            if (p.ep.progress_mode == 2)   // the other set of hand-over counters, for the next pass (nobody uses it during this one)
                for (uint32_t i = 0; i < p.ep.progress_len; ++i) p.ep.progress[((ep_epoch & 1u) ^ 1u) * p.ep.progress_len + i] = 0u;
            if (!failed && (old >> 16) == 0) {
                __threadfence_system();
                for (uint32_t w = 0; w < p.ep.world; ++w)
                    st_release_sys(reinterpret_cast<uint32_t *>(p.ep.peer_flags[w]) + FE2O3_EP_FLAG_OUTPUTS(p.ep.world) + p.ep.rank,
                                   ep_epoch);
            }
        }
    }
}

// ---- host side ------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

}  // namespace

// Encodes a tensor map with 128-byte swizzle.  dims/strides innermost first;
// strides in bytes for dimensions 1..rank-1.
static int32_t make_tmap(CUtensorMap *out, CUtensorMapDataType dtype, uint64_t base, uint32_t rank, const uint64_t *dims,
                         const uint64_t *strides_bytes, const uint32_t *box) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        fe2o3_set_error("cuTensorMapEncodeTiled is not available from the driver");
        return FE2O3_ERR_NO_DEVICE;
    }
    cuuint64_t d[5];
    cuuint64_t st[4];
    cuuint32_t b[5], es[5];
    for (uint32_t i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; es[i] = 1; }
    for (uint32_t i = 0; i + 1 < rank; ++i) st[i] = strides_bytes[i];
    CUresult r = fn(out, dtype, rank, reinterpret_cast<void *>(base), d, st, b, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fe2o3_set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return FE2O3_ERR_INVALID_ARGUMENT;
    }
    return FE2O3_OK;
}

int32_t fe2o3_make_tmap_bf16(CUtensorMap *out, uint64_t base, uint32_t rank, const uint64_t *dims,
                             const uint64_t *strides_bytes, const uint32_t *box) {
    return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box);
}
int32_t fe2o3_make_tmap_f32(CUtensorMap *out, uint64_t base, uint32_t rank, const uint64_t *dims,
                            const uint64_t *strides_bytes, const uint32_t *box) {
    return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box);
}

// The tensor-core schedule needs 16-byte aligned bases and leading dimensions
// that are multiples of 8 elements (TMA strides are multiples of 16 bytes).
bool gemm_tc_supported(uint64_t a, uint64_t b, uint32_t lda, uint32_t ldb, uint32_t K) {
    return K > 0 && (a & 15u) == 0 && (b & 15u) == 0 && (lda % 8u) == 0 && (ldb % 8u) == 0;
}

// experts == 0: plain C[M][N] = A[M][K] * B[K][N].  experts > 0: grouped, A rows
// partitioned by expert_offsets (device array), B = [experts][K][N], M = upper
// bound on rows (the capacity of A and C).
int32_t gemm_tc_plan(fe2o3_ctx *ctx, GemmTcPlan *plan, uint64_t a, uint64_t b, uint64_t c, uint32_t M, uint32_t N,
                     uint32_t K, uint32_t lda, uint32_t ldb, uint32_t ldc, float alpha, float beta, uint32_t epilogue,
                     const uint32_t *expert_offsets, uint32_t experts, uint32_t expert_mod, uint32_t b_matrices,
                     const GemmEp *ep, uint32_t expected_rows) {
    // 256-wide tiles whenever N allows.  Half-width tiles would fill the last round of SMs better when a rank
    // has few row tiles (512 tiles on 148 SMs are 4 rounds, 1024 half tiles 7 half rounds), but they re-read A
    // twice as often and were measured slower, not faster, on 4096 and 8192 rows (passes of 530 against 481 us
    // and 686 against 590 us).
    plan->bn = (N > 128) ? 256 : 128;
    (void)expected_rows;
    uint64_t dA[2] = {K, M}, sA[1] = {(uint64_t)lda * 2};
    uint32_t bA[2] = {BK, BM};
    int32_t st = fe2o3_make_tmap_bf16(&plan->tmA, a, 2, dA, sA, bA);
    if (st != FE2O3_OK) return st;
    if (experts) {
        uint64_t dB[3] = {N, K, b_matrices ? b_matrices : experts}, sB[2] = {(uint64_t)ldb * 2, (uint64_t)ldb * 2 * K};
        uint32_t bB[3] = {64, BK, 1};
        st = fe2o3_make_tmap_bf16(&plan->tmB, b, 3, dB, sB, bB);
    } else {
        uint64_t dB[2] = {N, K}, sB[1] = {(uint64_t)ldb * 2};
        uint32_t bB[2] = {64, BK};
        st = fe2o3_make_tmap_bf16(&plan->tmB, b, 2, dB, sB, bB);
    }
    if (st != FE2O3_OK) return st;
    // Output through the copy engine when it can address C: 16-byte aligned base and row pitch.
    const uint32_t esize = epilogue == EPI_GELU_BF16 ? 2u : 4u;
    uint32_t bulk = 0;
    plan->tmC = plan->tmA;   // a valid map when the bulk path is off (never used then)
    if (epilogue != EPI_ALPHA_BETA && epilogue != EPI_SCATTER_PEER && epilogue != EPI_COMBINE_ADD && (c & 15u) == 0 && ((uint64_t)ldc * esize) % 16u == 0 &&
        M > 0 && N > 0) {
        uint64_t dC[2] = {N, M}, sC[1] = {(uint64_t)ldc * esize};
        uint32_t bC[2] = {128u / esize, 32};
        st = esize == 2 ? fe2o3_make_tmap_bf16(&plan->tmC, c, 2, dC, sC, bC) : fe2o3_make_tmap_f32(&plan->tmC, c, 2, dC, sC, bC);
        if (st != FE2O3_OK) return st;
        bulk = 1;
    }
    plan->p = GemmParams{reinterpret_cast<void *>(c), M, N, K, ldc, alpha, beta, epilogue, expert_offsets, experts,
                         expert_mod, bulk, ctx->status_word, ep ? *ep : GemmEp{}, nullptr, nullptr, 0u, nullptr, nullptr, 0u, nullptr, 0ull};
    const uint32_t n_tiles = (N + plan->bn - 1) / plan->bn;
    const uint64_t m_tiles = (uint64_t)(M + BM - 1) / BM + experts;  // grouped: each expert may add a ragged tile
    uint64_t tiles = m_tiles * n_tiles;
    plan->grid = (uint32_t)(tiles < (uint64_t)ctx->sm_count ? (tiles ? tiles : 1) : (uint64_t)ctx->sm_count);
    plan->smem = plan->bn == 256 ? SmemLayout<256>::kTotal : SmemLayout<128>::kTotal;
    plan->overlap_previous = 0;
    return FE2O3_OK;
}

// Function attributes are per device: called by fe2o3_ctx_create with the context's device current.
int32_t gemm_tc_init_device() {
    FE2O3_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<256, 168>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)SmemLayout<256>::kTotal));
    FE2O3_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<128, 168>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)SmemLayout<128>::kTotal));
    FE2O3_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<256, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)SmemLayout<256>::kTotal));
    FE2O3_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<128, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)SmemLayout<128>::kTotal));
    return FE2O3_OK;
}

int32_t gemm_tc_launch(const GemmTcPlan *plan, cudaStream_t s) {
    if (plan->p.M == 0 || plan->p.N == 0) return FE2O3_OK;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(plan->grid, 1, 1);
    cfg.blockDim = dim3(kThreads + (plan->p.gather_perm ? kGatherThreads : 0), 1, 1);
    cfg.dynamicSmemBytes = plan->smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    if (plan->overlap_previous) {
        // programmatic dependent launch: the kernel may start while the kernel before it in the stream (the
        // expert-parallel dispatch, which says when) is still running; the two synchronise through flags
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e;
    // the 128-register build: for a block that shares its SM with the small blocks of the kernel before it, and for
    // one that carries the loader warps of a gathered A
    if (plan->overlap_previous == 1 || plan->p.gather_perm)
        e = plan->bn == 256 ? cudaLaunchKernelEx(&cfg, gemm_tc_kernel<256, 128>, plan->tmA, plan->tmB, plan->tmC, plan->p)
                            : cudaLaunchKernelEx(&cfg, gemm_tc_kernel<128, 128>, plan->tmA, plan->tmB, plan->tmC, plan->p);
    else
        e = plan->bn == 256 ? cudaLaunchKernelEx(&cfg, gemm_tc_kernel<256, 168>, plan->tmA, plan->tmB, plan->tmC, plan->p)
                            : cudaLaunchKernelEx(&cfg, gemm_tc_kernel<128, 168>, plan->tmA, plan->tmB, plan->tmC, plan->p);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(e, "gemm_tc");
}

// Makes the plan's A operand a gather: row r of A = row (perm[r] >> 1) of src.  Needs whole 64-column K blocks.
bool gemm_tc_set_gather(GemmTcPlan *plan, const uint32_t *perm, const void *src, uint32_t tokens) {
    if (plan->p.K % BK != 0 || (reinterpret_cast<uintptr_t>(src) & 15u) != 0) return false;
    plan->p.gather_perm = perm;
    plan->p.gather_src = src;
    plan->p.gather_tokens = tokens;
    return true;
}

// Makes the plan's output a weighted accumulation into token rows (see GemmParams); the plan must have been made
// with EPI_COMBINE_ADD and c = the [tokens][N] f32 output.
void gemm_tc_set_combine(GemmTcPlan *plan, const uint32_t *perm, const float *weights, uint32_t tokens) {
    plan->p.combine_perm = perm;
    plan->p.combine_weights = weights;
    plan->p.combine_tokens = tokens;
}

void gemm_tc_geometry(const GemmTcPlan *plan, fe2o3_geometry *geo) {
    *geo = fe2o3_geometry{{plan->grid, 1, 1}, {(uint32_t)(kThreads + (plan->p.gather_perm ? kGatherThreads : 0)), 1, 1}, plan->smem, 1};
}

// kernel symbols of the runtime adapter carried by this source (the schedule a large launch resolves to)
static Fe2o3KernelRegistration reg_tiled("tiled_gemm_lds_slice1", reinterpret_cast<const void *>(gemm_tc_kernel<256, 168>));
static Fe2o3KernelRegistration reg_general("tiled_gemm_general_v1", reinterpret_cast<const void *>(gemm_tc_kernel<256, 168>));
static Fe2o3KernelRegistration reg_ffn("moe_expert_ffn_v1", reinterpret_cast<const void *>(gemm_tc_kernel<256, 168>));
static Fe2o3KernelRegistration reg_gffn("moe_grouped_ffn_v1", reinterpret_cast<const void *>(gemm_tc_kernel<256, 168>));
static Fe2o3KernelRegistration reg_ffnc("moe_expert_ffn_combine_v1", reinterpret_cast<const void *>(gemm_tc_kernel<256, 128>));
static Fe2o3KernelRegistration reg_epffn("moe_ep_ffn_v1", reinterpret_cast<const void *>(gemm_tc_kernel<256, 168>));
