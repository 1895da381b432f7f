// Device-wide inclusive / exclusive prefix sum of u32 values (wrapping addition) and of f32 values
// (each addition rounded to nearest; one kernel template, values carried as 32-bit patterns).
//
// The reference defines prefix sums at two scopes: a 64-lane wave
// (crates/fe2o3-device/src/collective.rs:413-460, Hillis-Steele over lane
// shuffles; lane 0 of the exclusive form receives zero) and a workgroup through
// LDS scratch (collective.rs:503-571).  This kernel keeps their meaning (element
// i of the inclusive form is values[0] + ... + values[i], the exclusive form
// shifts by one and starts at zero, addition wraps) and extends the scope to a
// whole array in one pass over HBM: 4 bytes read and 4 bytes written per element.
//
// Single pass, staged through shared memory, with the carries between tiles taken
// from published tile sums.  One persistent block per SM; tiles of 8192 elements are
// handed out by an atomic ticket, so a tile only ever waits for tiles that started
// before it.  Four roles:
//   warp 0      producer: takes tickets and fills a six-stage ring of 32 KiB tiles
//               with bulk copies (an mbarrier per stage counts the bytes)
//   warps 1-4   aggregate: as soon as a tile has landed they sum it and publish its
//               aggregate, so the aggregates of all tiles in flight appear at the
//               speed of the memory system, whatever the rest of the block waits for
//   warp 5      prefix: keeps the sum of everything up to the block's previous tile and
//               adds the aggregates of the tiles between that one and the next (about
//               one per SM, fetched in one round trip).  No block waits for another
//               block's prefix, only for aggregates, so there is no chain across blocks
//   warps 6-13  finish: scan the tile from shared memory with that prefix and store it
//               with 16-byte writes; the warp scans of a tile run in lockstep
// The ring keeps 192 KiB per SM in flight, three times what a register-resident tile
// per thread allows.  Two earlier forms were measured and replaced: one pass over
// registers with a decoupled look-back in the same warps (0.53 of the HBM copy rate,
// bound by the wait for the predecessor's prefix), and this staging with a look-back
// warp that walked back to the nearest published inclusive prefix (0.68-0.76: with
// every tile of a wave in flight at once the nearest such prefix is a wave or more
// behind, and the walk became a serial chain of L2 round trips per SM).
// In the f32 form the order of additions must not depend on scheduling, so the prefix warp only
// ever accumulates whole chunks of 192 tiles from tile 0 and adds the part of the current chunk
// separately: whichever block computes a tile's prefix performs the same chain of additions, and
// repeated runs give identical bits.  The lane prefix inside a warp scan comes from a shuffle
// instead of a subtraction.
// A descriptor is one 64-bit word {state, value}; it carries everything its reader
// needs, so relaxed device-scope accesses are enough.  The launch clears the ticket
// and the descriptors first.  Every wait is bounded and records
// FE2O3_KSTATUS_WAIT_EXPIRED.
#include "common.cuh"

#include <mutex>

namespace {

constexpr int kStages = 6;
constexpr uint32_t kTileElems = 8192;
constexpr uint32_t kTileBytes = kTileElems * 4;
constexpr int kAggWarps = 4;                                        // aggregate warps: 2048 consecutive elements each
constexpr int kFinishWarps = 8;                                     // scan-and-store warps: 1024 consecutive elements each
constexpr uint32_t kPart = kTileElems / kFinishWarps;               // 1024
constexpr int kPartVecs = kPart / 128;                              // a part is 8 rows of 32 lanes x 16 bytes
constexpr int kLaneVecs = 2;                                        // consecutive 16-byte groups a finish lane owns per pass
constexpr int kPasses = kPartVecs / kLaneVecs;                      // warp scans per finish warp and tile
constexpr int kScanThreads = 32 * (1 + kAggWarps + 1 + kFinishWarps);   // 448
constexpr int kWindow = 6;                                          // descriptors per lane and step of the prefix warp: 192, a little over one tile per SM
constexpr uint32_t kStateAggregate = 1;   // state 0: not yet published (the launch clears the descriptors)
constexpr uint32_t kDescSpin = 1u << 22;
constexpr uint32_t kNoTile = 0xffffffffu;

struct __align__(16) ScanShared {
    uint64_t full[kStages], empty[kStages], agg_ready[kStages], prefix_ready[kStages];
    uint32_t tile[kStages];                // ticket of the tile in each stage (kNoTile: the array is exhausted)
    uint32_t part[kStages][kFinishWarps];  // sums of the eight parts of the tile
    uint32_t prefix[kStages];              // exclusive prefix of the tile (sum of everything before it)
    uint32_t arrivals[kStages];            // aggregate warps done with the stage
};
constexpr uint32_t kSmemBytes = kStages * kTileBytes + sizeof(ScanShared) + 1024;

__device__ __forceinline__ void desc_store(uint64_t *p, uint32_t state, uint32_t value) {
    const uint64_t v = ((uint64_t)state << 32) | value;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t desc_load(const uint64_t *p) {
    uint64_t v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Values travel as 32-bit patterns; kFloat selects IEEE binary32 addition (round to nearest) instead of
// wrapping integer addition.  Zero is the all-zero pattern in both.
template <bool kFloat>
__device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b) {
    if constexpr (kFloat) return __float_as_uint(__fadd_rn(__uint_as_float(a), __uint_as_float(b)));
    else return a + b;
}
template <bool kFloat>
__device__ __forceinline__ uint32_t sum4(const uint4 &x) {
    return add<kFloat>(add<kFloat>(x.x, x.y), add<kFloat>(x.z, x.w));
}
// sum over the warp in a fixed order (every lane receives it)
template <bool kFloat>
__device__ __forceinline__ uint32_t warp_sum(uint32_t v) {
    if constexpr (kFloat) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = add<true>(v, __shfl_xor_sync(0xffffffffu, v, o));
        return v;
    } else {
        return __reduce_add_sync(0xffffffffu, v);
    }
}

template <bool kFloat>
__global__ void __launch_bounds__(kScanThreads, 1)
device_scan_kernel(const uint32_t *in, uint32_t *out, uint64_t n, uint32_t exclusive, uint32_t *ticket,
                   uint64_t *desc, uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint32_t *ring = reinterpret_cast<uint32_t *>(smem);
    ScanShared &sh = *reinterpret_cast<ScanShared *>(smem + kStages * kTileBytes);
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&sh.full[i], 1);
            mbar_init(&sh.empty[i], kFinishWarps);
            mbar_init(&sh.agg_ready[i], 1);
            mbar_init(&sh.prefix_ready[i], 1);
            sh.arrivals[i] = 0;
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        bool ok = true;
        for (uint32_t k = 0; ok; ++k) {
            const uint32_t st = k % kStages, ph = (k / kStages) & 1;
            if (!mbar_wait_warp(&sh.empty[st], ph ^ 1)) { ok = false; break; }
            uint32_t t = 0;
            if (lane == 0) t = atomicAdd(ticket, 1u);
            t = __shfl_sync(0xffffffffu, t, 0);
            const uint64_t base = (uint64_t)t * kTileElems;
            if (base >= n) {
                // the array is exhausted: tell the consumers and stop
                if (lane == 0) {
                    sh.tile[st] = kNoTile;
                    mbar_arrive(&sh.full[st]);
                }
                __syncwarp();
                break;
            }
            uint32_t *dst = ring + st * kTileElems;
            if (aligned && base + kTileElems <= n) {
                if (lane == 0) {
                    sh.tile[st] = t;
                    mbar_arrive_expect_tx(&sh.full[st], kTileBytes);
                    bulk_load_1d(dst, in + base, kTileBytes, &sh.full[st]);
                }
            } else {   // the last tile, or input the copy engine cannot address: plain loads, zero beyond the end
                for (uint32_t i = lane; i < kTileElems; i += 32) dst[i] = base + i < n ? in[base + i] : 0u;
                __syncwarp();
                if (lane == 0) {
                    sh.tile[st] = t;
                    mbar_arrive(&sh.full[st]);
                }
            }
            __syncwarp();
        }
        if (!ok && lane == 0) kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
    } else if (warp <= kAggWarps) {
        // ------------------------------------------------------------ aggregate warps
        const uint32_t w = warp - 1;
        for (uint32_t k = 0;; ++k) {
            const uint32_t st = k % kStages, ph = (k / kStages) & 1;
            if (!mbar_wait_warp(&sh.full[st], ph)) {
                if (lane == 0) kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
                break;
            }
            const uint32_t tile = sh.tile[st];
            if (tile == kNoTile) break;
            // this warp sums parts 2w and 2w + 1 of the tile
            const uint4 *src = reinterpret_cast<const uint4 *>(ring + st * kTileElems + w * 2 * kPart) + lane;
            uint32_t sum0 = 0, sum1 = 0;
#pragma unroll
            for (int j = 0; j < kPartVecs; ++j) {
                const uint4 x = src[j * 32], y = src[(kPartVecs + j) * 32];
                sum0 = add<kFloat>(sum0, sum4<kFloat>(x));
                sum1 = add<kFloat>(sum1, sum4<kFloat>(y));
            }
            sum0 = warp_sum<kFloat>(sum0);
            sum1 = warp_sum<kFloat>(sum1);
            // the last of the four warps to finish publishes the tile's aggregate
            uint32_t last = 0;
            if (lane == 0) {
                sh.part[st][2 * w] = sum0;
                sh.part[st][2 * w + 1] = sum1;
                __threadfence_block();
                last = atomicAdd(&sh.arrivals[st], 1u) == kAggWarps - 1 ? 1u : 0u;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last && lane == 0) {
                __threadfence_block();
                uint32_t aggregate = 0;
                for (int q = 0; q < kFinishWarps; ++q) aggregate = add<kFloat>(aggregate, sh.part[st][q]);
                sh.arrivals[st] = 0;
                desc_store(desc + tile, kStateAggregate, aggregate);
                mbar_arrive(&sh.agg_ready[st]);
            }
        }
    } else if (warp == kAggWarps + 1) {
        // ------------------------------------------------------------ prefix warp: runs ahead of the finish warps
        // The block's tiles arrive in ticket order.  The warp keeps the sum of everything up to and
        // including the block's previous tile, so the prefix of the next one only needs the aggregates
        // of the tiles in between (about one per SM), which other blocks publish as their data lands.
        bool ok = true;
        uint32_t covered = 0;   // tiles [0, covered) are summed in `running`
        uint32_t running = 0;
        for (uint32_t k = 0; ok; ++k) {
            const uint32_t st = k % kStages, ph = (k / kStages) & 1;
            if (!mbar_wait_warp(&sh.full[st], ph)) { ok = false; break; }
            const uint32_t tile = sh.tile[st];
            if (tile == kNoTile) break;
            // sum of the published aggregates of tiles [lo, hi): lanes take them 32 apart, then a warp sum
            auto range_sum = [&](uint32_t lo, uint32_t hi) -> uint32_t {
                uint32_t acc = 0;
                for (uint32_t b = lo; ok && b < hi; b += 32 * kWindow) {
                    uint64_t d[kWindow];
#pragma unroll
                    for (int q = 0; q < kWindow; ++q) {   // all loads of the step in flight together
                        const uint32_t mine = b + 32 * q + lane;
                        d[q] = mine < hi ? desc_load(desc + mine) : ((uint64_t)kStateAggregate << 32);
                    }
#pragma unroll
                    for (int q = 0; q < kWindow; ++q) {
                        const uint32_t mine = b + 32 * q + lane;
                        uint32_t spins = 0;
                        while ((d[q] >> 32) == 0) {
                            if (++spins > kDescSpin) { ok = false; break; }
                            __nanosleep(100);
                            d[q] = desc_load(desc + mine);
                        }
                        acc = add<kFloat>(acc, (uint32_t)d[q]);
                    }
                    ok = __all_sync(0xffffffffu, ok);
                }
                return warp_sum<kFloat>(acc);
            };
            uint32_t prefix;
            if constexpr (kFloat) {
                // Rounding makes the order matter.  `running` only ever stops at multiples of kChunk tiles and
                // advances by whole chunks, so the prefix of a tile is the same chain of additions whichever
                // block computes it: results do not depend on how the tickets fell.
                constexpr uint32_t kChunk = 32 * kWindow;
                while (ok && covered + 2 * kChunk <= tile) {
                    running = add<true>(running, range_sum(covered, covered + kChunk));
                    covered += kChunk;
                }
                if (covered + kChunk <= tile) {
                    // the usual case, one whole chunk and a part of the next: both windows' loads go out
                    // together, so the step costs one round trip; the additions are the same as above
                    const uint32_t mid = covered + kChunk;
                    uint64_t d[2][kWindow];
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int q = 0; q < kWindow; ++q) {
                            const uint32_t mine = (h ? mid : covered) + 32 * q + lane;
                            d[h][q] = mine < (h ? tile : mid) ? desc_load(desc + mine) : ((uint64_t)kStateAggregate << 32);
                        }
                    uint32_t acc[2] = {0, 0};
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int q = 0; q < kWindow; ++q) {
                            const uint32_t mine = (h ? mid : covered) + 32 * q + lane;
                            uint32_t spins = 0;
                            while ((d[h][q] >> 32) == 0) {
                                if (++spins > kDescSpin) { ok = false; break; }
                                __nanosleep(100);
                                d[h][q] = desc_load(desc + mine);
                            }
                            acc[h] = add<true>(acc[h], (uint32_t)d[h][q]);
                        }
                    ok = __all_sync(0xffffffffu, ok);
                    running = add<true>(running, warp_sum<true>(acc[0]));
                    covered = mid;
                    prefix = add<true>(running, warp_sum<true>(acc[1]));
                } else {
                    prefix = add<true>(running, range_sum(covered, tile));
                }
            } else {
                prefix = running + range_sum(covered, tile);
            }
            if (!ok) break;
            if (!mbar_wait_warp(&sh.agg_ready[st], ph)) { ok = false; break; }
            // The stage's partial sums are read BEFORE the arrival below: that arrival lets the finish
            // warps release the stage, after which the aggregate warps may overwrite sh.part[st].
            uint32_t aggregate = 0;
            if constexpr (!kFloat) {
                for (int q = 0; q < kFinishWarps; ++q) aggregate += sh.part[st][q];
            }
            __syncwarp();
            if (lane == 0) {
                sh.prefix[st] = prefix;
                mbar_arrive(&sh.prefix_ready[st]);
            }
            if constexpr (!kFloat) {
                running = prefix + aggregate;
                covered = tile + 1;
            }
        }
        if (!ok && lane == 0) kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);   // the finish warps' waits expire in turn
    } else {
        // ------------------------------------------------------------ finish warps
        const uint32_t w = warp - 2 - kAggWarps;
        for (uint32_t k = 0;; ++k) {
            const uint32_t st = k % kStages, ph = (k / kStages) & 1;
            const bool ok = mbar_wait_warp(&sh.full[st], ph);
            const uint32_t tile = ok ? sh.tile[st] : kNoTile;
            if (!ok && lane == 0) kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
            if (tile == kNoTile) break;
            if (!mbar_wait_warp(&sh.prefix_ready[st], ph)) {
                if (lane == 0) kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
                break;
            }
            uint32_t carry = sh.prefix[st];   // everything before this warp's first element
            for (uint32_t q = 0; q < w; ++q) carry = add<kFloat>(carry, sh.part[st][q]);
            const uint64_t base = (uint64_t)tile * kTileElems + (uint64_t)w * kPart + lane * (4 * kLaneVecs);
            const bool vec = aligned && (uint64_t)tile * kTileElems + kTileElems <= n;
            const uint4 *src = reinterpret_cast<const uint4 *>(ring + st * kTileElems + w * kPart) + lane * kLaneVecs;
            // Each lane owns kLaneVecs consecutive 16-byte groups per pass, so one warp scan covers
            // 32 * 4 * kLaneVecs elements.  The passes' warp scans are independent and run in
            // lockstep: each shuffle step issues one shuffle per pass back to back, and the latency
            // of a chain is paid once per tile, not once per pass.
            uint4 x[kPasses][kLaneVecs];
            uint32_t own[kPasses], t[kPasses];   // each lane's total per pass; the same scanned over the warp
#pragma unroll
            for (int j = 0; j < kPasses; ++j) {
                own[j] = 0;
#pragma unroll
                for (int c = 0; c < kLaneVecs; ++c) {
                    x[j][c] = src[j * 32 * kLaneVecs + c];
                    own[j] = add<kFloat>(own[j], sum4<kFloat>(x[j][c]));
                }
                t[j] = own[j];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.empty[st]);   // the part is in registers: the stage may be refilled
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
                for (int j = 0; j < kPasses; ++j) {
                    const uint32_t up = __shfl_up_sync(0xffffffffu, t[j], o);
                    if (lane >= (uint32_t)o) t[j] = add<kFloat>(up, t[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < kPasses; ++j) {
                // everything before this lane's first element of the pass
                uint32_t run;
                if constexpr (kFloat) {   // no subtraction in floating point: take the lower lane's inclusive total
                    const uint32_t below = __shfl_up_sync(0xffffffffu, t[j], 1);
                    run = lane == 0 ? carry : add<true>(carry, below);
                } else {
                    run = carry + t[j] - own[j];
                }
                carry = add<kFloat>(carry, __shfl_sync(0xffffffffu, t[j], 31));
#pragma unroll
                for (int c = 0; c < kLaneVecs; ++c) {
                    // inclusive values of the four elements, each the previous one plus the element
                    uint32_t inc[4];
                    inc[0] = add<kFloat>(run, x[j][c].x);
                    inc[1] = add<kFloat>(inc[0], x[j][c].y);
                    inc[2] = add<kFloat>(inc[1], x[j][c].z);
                    inc[3] = add<kFloat>(inc[2], x[j][c].w);
                    uint32_t r[4];
                    if (exclusive) {   // element i of the exclusive form is the inclusive value of element i - 1
                        r[0] = run; r[1] = inc[0]; r[2] = inc[1]; r[3] = inc[2];
                    } else {
                        r[0] = inc[0]; r[1] = inc[1]; r[2] = inc[2]; r[3] = inc[3];
                    }
                    run = inc[3];
                    const uint64_t e = base + (uint64_t)j * (128 * kLaneVecs) + c * 4;
                    if (vec) {
                        __stcs(reinterpret_cast<uint4 *>(out + e), make_uint4(r[0], r[1], r[2], r[3]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (e + i < n) out[e + i] = r[i];
                    }
                }
            }
        }
    }
}

}  // namespace

template <bool kFloat>
int32_t launch_device_scan(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_device_scan_u32_args *a = static_cast<const fe2o3_device_scan_u32_args *>(args);
    const uint64_t n = a->values.len;
    const uint32_t tiles = (uint32_t)((n + kTileElems - 1) / kTileElems);
    const uint32_t sms = ctx->sm_count > 0 ? (uint32_t)ctx->sm_count : 1u;
    const uint32_t grid = tiles < sms ? (tiles ? tiles : 1u) : sms;
    if (geo) *geo = fe2o3_geometry{{grid, 1, 1}, {kScanThreads, 1, 1}, kSmemBytes, 1};
    if (plan_only || n == 0) return FE2O3_OK;
    // ticket at word 0, descriptors from byte 64
    uint32_t *ticket = ctx->scan_scratch;
    uint64_t *desc = reinterpret_cast<uint64_t *>(ctx->scan_scratch + 16);
    FE2O3_CUDA(cudaMemsetAsync(ctx->scan_scratch, 0, 64 + (size_t)tiles * 8, s));
    device_scan_kernel<kFloat><<<grid, kScanThreads, kSmemBytes, s>>>(reinterpret_cast<const uint32_t *>(a->values.ptr),
                                                                      reinterpret_cast<uint32_t *>(a->output.ptr), n,
                                                                      a->exclusive, ticket, desc, ctx->status_word);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), kFloat ? "device_scan_sum_f32" : "device_scan_sum_u32");
}

// Function attributes are per device: called by fe2o3_ctx_create with the context's device current.
int32_t device_scan_init_device() {
    FE2O3_CUDA(cudaFuncSetAttribute(device_scan_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    FE2O3_CUDA(cudaFuncSetAttribute(device_scan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    return FE2O3_OK;
}

int32_t launch_device_scan_u32(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    return launch_device_scan<false>(ctx, s, args, geo, plan_only);
}
int32_t launch_device_scan_f32(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    return launch_device_scan<true>(ctx, s, args, geo, plan_only);
}

static Fe2o3KernelRegistration reg_scan_u32("device_scan_sum_u32", reinterpret_cast<const void *>(device_scan_kernel<false>));
static Fe2o3KernelRegistration reg_scan_f32("device_scan_sum_f32", reinterpret_cast<const void *>(device_scan_kernel<true>));
