// Device-wide inclusive / exclusive prefix sum of u32 values (wrapping addition).
//
// The reference defines prefix sums at two scopes: a 64-lane wave
// (crates/fe2o3-device/src/collective.rs:413-460, Hillis-Steele over lane
// shuffles; lane 0 of the exclusive form receives zero) and a workgroup through
// LDS scratch (collective.rs:503-571).  This kernel keeps their meaning (element
// i of the inclusive form is values[0] + ... + values[i], the exclusive form
// shifts by one and starts at zero, addition wraps) and extends the scope to a
// whole array in one pass over HBM: 4 bytes read and 4 bytes written per element.
//
// Single pass with decoupled look-back.  A tile is 16384 elements: each of the eight
// warps owns 2048 consecutive elements and walks them in sixteen coalesced passes of
// 32 lanes x 16 bytes, carrying its running total from pass to pass in registers,
// so the block synchronises only once per tile (to combine the warp totals).  Tiles
// are handed out by an atomic ticket, so a tile only ever waits for tiles that
// started before it.  Each tile publishes its aggregate, then warp 0 walks back over
// its predecessors' descriptors, 128 at a time (four per lane, the four loads in
// flight together), up to the nearest one whose inclusive prefix is known, and
// publishes the tile's own inclusive prefix.  Measured at 2^28 elements on B200:
// 32-wide steps over 4096-element tiles 2.3 TB/s, this form 3.4 TB/s (8192- and
// 16384-element tiles alike); without the
// look-back the same loads and stores run at 6.6 TB/s, so what is left is the wait
// for the predecessors.  Two variants were slower and are not kept: a block-wide
// 1024-descriptor step (more polling traffic on the descriptor lines) and
// persistent blocks that prefetch their next tile (a prefetched tile cannot publish
// its aggregate until its block has finished the tile before it, which lengthens
// every successor's wait).
// A descriptor is one 64-bit word {state, value}; it carries everything its reader
// needs, so relaxed device-scope accesses are enough (acquire loads would also
// serialise the four loads of a step: each would have to complete before the
// next could issue).  The launch clears the ticket and the descriptors first.
// Waits are bounded and record FE2O3_KSTATUS_WAIT_EXPIRED.
#include "common.cuh"

namespace {

constexpr int kScanThreads = 256;
constexpr int kPasses = 16;                                         // 16-byte vectors per thread
constexpr uint32_t kWarpElems = kPasses * 32 * 4;                   // 2048 consecutive elements per warp
constexpr uint32_t kTileElems = (kScanThreads / 32) * kWarpElems;   // 16384
constexpr int kWindow = 4;                                          // descriptors per lane and look-back step
constexpr uint32_t kStateAggregate = 1, kStateInclusive = 2;
constexpr uint32_t kLookbackSpin = 1u << 22;

__device__ __forceinline__ void desc_store(uint64_t *p, uint32_t state, uint32_t value) {
    const uint64_t v = ((uint64_t)state << 32) | value;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t desc_load(const uint64_t *p) {
    uint64_t v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kScanThreads)
device_scan_u32_kernel(const uint32_t *in, uint32_t *out, uint64_t n, uint32_t exclusive,
                       uint32_t *ticket, uint64_t *desc, uint32_t *status) {
    __shared__ uint32_t s_tile, s_warp[kScanThreads / 32], s_prefix;
    __shared__ int s_ok;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_tile = atomicAdd(ticket, 1u);
    __syncthreads();
    const uint32_t tile = s_tile;
    const uint64_t base = (uint64_t)tile * kTileElems;
    if (base >= n) return;
    const bool vec = base + kTileElems <= n && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;

    // pass j of this warp is elements [2048 warp + 128 j, +128) of the tile; this lane owns elements 4 lane .. 4 lane + 3 of it
    const uint64_t wbase = base + (uint64_t)warp * kWarpElems + lane * 4;
    uint32_t incl[kPasses][4];
#pragma unroll
    for (int j = 0; j < kPasses; ++j) {
        const uint64_t e = wbase + (uint64_t)j * 128;
        if (vec) {
            const uint4 x = __ldcs(reinterpret_cast<const uint4 *>(in + e));
            incl[j][0] = x.x; incl[j][1] = x.y; incl[j][2] = x.z; incl[j][3] = x.w;
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) incl[j][c] = e + c < n ? in[e + c] : 0u;
        }
    }
    // inclusive scan inside the warp's 2048 elements, in place: thread-local, across the lanes, carried over the passes
    uint32_t before[kPasses];   // sum of everything in the warp's part before this lane's four elements of pass j
    uint32_t carry = 0;         // sum of this warp's passes before the current one
#pragma unroll
    for (int j = 0; j < kPasses; ++j) {
#pragma unroll
        for (int c = 1; c < 4; ++c) incl[j][c] += incl[j][c - 1];
        const uint32_t own = incl[j][3];
        uint32_t t = own;   // this lane's total, scanned over the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, t, o);
            if (lane >= (uint32_t)o) t += up;
        }
        before[j] = carry + t - own;
#pragma unroll
        for (int c = 0; c < 4; ++c) incl[j][c] += before[j];
        carry += __shfl_sync(0xffffffffu, t, 31);
    }
    if (lane == 0) s_warp[warp] = carry;
    __syncthreads();
    uint32_t warp_before = 0, aggregate = 0;
#pragma unroll
    for (int w = 0; w < kScanThreads / 32; ++w) {
        const uint32_t wt = s_warp[w];
        if ((uint32_t)w < warp) warp_before += wt;
        aggregate += wt;
    }

    // decoupled look-back by warp 0, 128 predecessors per step (four descriptors per lane, loads in flight together)
    if (warp == 0) {
        uint32_t prefix = 0;
        bool ok = true;
        if (tile == 0) {
            if (lane == 0) desc_store(desc, kStateInclusive, aggregate);
        } else {
            if (lane == 0) desc_store(desc + tile, kStateAggregate, aggregate);
            int64_t idx = (int64_t)tile - 1;   // nearest predecessor not yet accounted for
            bool done = false;
            while (ok && !done) {
                // descriptor q of this lane is predecessor idx - (32 q + lane): q = 0 holds the nearest 32
                uint64_t d[kWindow];
#pragma unroll
                for (int q = 0; q < kWindow; ++q) {
                    const int64_t mine = idx - (32 * q + (int64_t)lane);
                    d[q] = mine >= 0 ? desc_load(desc + mine) : ((uint64_t)kStateInclusive << 32);   // before the array: 0, final
                }
#pragma unroll
                for (int q = 0; q < kWindow; ++q) {
                    if (done || !ok) continue;
                    const int64_t mine = idx - (32 * q + (int64_t)lane);
                    uint32_t spins = 0;
                    while ((d[q] >> 32) == 0) {
                        if (++spins > kLookbackSpin) { ok = false; break; }
                        __nanosleep(100);   // few reloads: pollers and writers share the descriptor lines in L2
                        d[q] = desc_load(desc + mine);
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) continue;
                    // lanes 0 .. first lane holding an inclusive prefix contribute; the walk ends there
                    const uint32_t final_mask = __ballot_sync(0xffffffffu, (uint32_t)(d[q] >> 32) == kStateInclusive);
                    const uint32_t last = final_mask ? (uint32_t)__ffs(final_mask) - 1 : 31u;
                    uint32_t contrib = lane <= last ? (uint32_t)d[q] : 0u;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
                    prefix += contrib;
                    done = final_mask != 0;
                }
                idx -= 32 * kWindow;
            }
            if (ok && lane == 0) desc_store(desc + tile, kStateInclusive, prefix + aggregate);
        }
        if (lane == 0) {
            s_prefix = prefix;
            s_ok = ok ? 1 : 0;
            if (!ok) kstatus_set(status, FE2O3_KSTATUS_WAIT_EXPIRED);
        }
    }
    __syncthreads();
    if (!s_ok) return;
    const uint32_t prefix = s_prefix + warp_before;
#pragma unroll
    for (int j = 0; j < kPasses; ++j) {
        const uint64_t e = wbase + (uint64_t)j * 128;
        uint32_t r[4];
        if (exclusive) {   // element i of the exclusive form is the inclusive value of element i - 1
            r[0] = before[j] + prefix;
#pragma unroll
            for (int c = 1; c < 4; ++c) r[c] = incl[j][c - 1] + prefix;
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) r[c] = incl[j][c] + prefix;
        }
        if (vec) {
            __stcs(reinterpret_cast<uint4 *>(out + e), make_uint4(r[0], r[1], r[2], r[3]));
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (e + c < n) out[e + c] = r[c];
        }
    }
}

}  // namespace

int32_t launch_device_scan_u32(fe2o3_ctx *ctx, cudaStream_t s, const void *args, fe2o3_geometry *geo, bool plan_only) {
    const fe2o3_device_scan_u32_args *a = static_cast<const fe2o3_device_scan_u32_args *>(args);
    const uint64_t n = a->values.len;
    const uint32_t tiles = (uint32_t)((n + kTileElems - 1) / kTileElems);
    if (geo) *geo = fe2o3_geometry{{tiles ? tiles : 1, 1, 1}, {kScanThreads, 1, 1}, 0, 1};
    if (plan_only || n == 0) return FE2O3_OK;
    // ticket at word 0, descriptors from byte 64
    uint32_t *ticket = ctx->scan_scratch;
    uint64_t *desc = reinterpret_cast<uint64_t *>(ctx->scan_scratch + 16);
    FE2O3_CUDA(cudaMemsetAsync(ctx->scan_scratch, 0, 64 + (size_t)tiles * 8, s));
    device_scan_u32_kernel<<<tiles, kScanThreads, 0, s>>>(reinterpret_cast<const uint32_t *>(a->values.ptr),
                                                           reinterpret_cast<uint32_t *>(a->output.ptr), n, a->exclusive,
                                                           ticket, desc, ctx->status_word);
    fe2o3_count_launch(1);
    return fe2o3_cuda_status(cudaGetLastError(), "device_scan_sum_u32");
}
