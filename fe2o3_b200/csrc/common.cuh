// Shared declarations for the fe2o3_b200 CUDA sources: the context object,
// launch bookkeeping, and thin wrappers over the sm_100a PTX used by the
// tensor-core kernels (mbarrier, TMA, tcgen05 / TMEM).
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

#include "../../include/fe2o3_b200.h"

// ---------------------------------------------------------------- host side
struct fe2o3_ctx {
    int device;
    int sm_count;
    int cc_major, cc_minor;
    cudaStream_t default_stream;
    uint32_t *status_word;     // device: kernel status (0 = ok), written instead of trapping
    uint32_t *reduce_scratch;  // device: per-block partial sums + arrival counter
    uint32_t reduce_scratch_elems;
    uint32_t *host_status;     // pinned mirror for status read-back
    uint32_t *route_scratch;   // device: per-block expert counts, per-block flags, arrival counter (MoE routing)
    uint32_t *scan_scratch;    // device: ticket + one 64-bit descriptor per tile (device-wide scan)
};

// Routing scratch layout: [FE2O3_ROUTE_MAX_BLOCKS][32] counts, [FE2O3_ROUTE_MAX_BLOCKS] flags, 1 summary, 1 counter.
#define FE2O3_ROUTE_MAX_BLOCKS 16384u
#define FE2O3_ROUTE_SCRATCH_ELEMS (FE2O3_ROUTE_MAX_BLOCKS * 33u + 64u)
// Scan scratch: 64 bytes (ticket) + 8 bytes per tile at the largest admitted length (sized for 8192-element tiles;
// the kernel's tiles are at least that large).
#define FE2O3_SCAN_SCRATCH_BYTES (64u + (uint32_t)(FE2O3_SCAN_MAX_ELEMENTS / 8192u) * 8u)

struct fe2o3_stream {
    fe2o3_ctx *ctx;
    cudaStream_t s;
    bool owned;
};

void fe2o3_set_error(const char *fmt, ...);
// Names the device function that carries a kernel symbol of the runtime adapter, for
// fe2o3_observe_kernel_resources.  Each source registers its kernels with a file-scope object.
void fe2o3_register_kernel(const char *symbol, const void *entry);
struct Fe2o3KernelRegistration {
    Fe2o3KernelRegistration(const char *symbol, const void *entry) { fe2o3_register_kernel(symbol, entry); }
};
void fe2o3_count_launch(uint32_t n);
int32_t fe2o3_cuda_status(cudaError_t e, const char *what);

#define FE2O3_CUDA(call)                                       \
    do {                                                       \
        cudaError_t e__ = (call);                              \
        if (e__ != cudaSuccess) return fe2o3_cuda_status(e__, #call); \
    } while (0)

static inline uint32_t ceil_div_u32(uint64_t a, uint64_t b) { return (uint32_t)((a + b - 1) / b); }

// Flag block of one rank of the expert-parallel layer, in u32 words (world = W):
//   [0, W)    counts published by source rank s        [W, 2W)  rows complete from source rank s
//   [2W, 3W)  outputs ready from owner rank o          3W+1, 3W+2  arrival counters of the second FFN
//   GEMM and the combine kernel (each re-armed by its last block)   3W+3  "row table written" (local:
//   the dispatch kernel to the FFN kernel that may already be running beside it)
//   [3W+4, 5W+4)  rows stored so far per destination rank, two sets used by alternate passes (the set of
//   the next pass is cleared by the dispatch kernel of this one)
#define FE2O3_EP_FLAG_COUNTS(W) (0u)
#define FE2O3_EP_FLAG_ROWS(W) (W)
#define FE2O3_EP_FLAG_OUTPUTS(W) (2u * (W))
#define FE2O3_EP_COUNTER_FFN(W) (3u * (W) + 1u)
#define FE2O3_EP_COUNTER_COMBINE(W) (3u * (W) + 2u)
#define FE2O3_EP_FLAG_TABLE(W) (3u * (W) + 3u)
#define FE2O3_EP_ROWS_DONE(W, parity) (3u * (W) + 4u + (parity) * (W))
//   5W+4, 5W+5  blocks of the dispatch kernel that have stored their share of this rank's own rows (two
//   alternating counters like the row counters)
#define FE2O3_EP_OWN_BLOCKS(W, parity) (5u * (W) + 4u + (parity))
#define FE2O3_EP_FLAG_WORDS(W) (5u * (W) + 6u)
#define FE2O3_EP_DEFAULT_SPIN (1u << 24)
// Diagnostic build (-DFE2O3_EP_TRACE): the kernels of the expert-parallel layer stamp the global
// nanosecond timer into 64-bit slots at byte 2048 of the rank's flag block (which must then be at
// least 4096 bytes), one slot per event, overwritten every pass.
#define FE2O3_EP_TRACE_WORD 512u
enum {
    FE2O3_EP_T_DISPATCH_BEGIN = 0, FE2O3_EP_T_COUNTS_HERE = 1, FE2O3_EP_T_ROWS_SENT = 2, FE2O3_EP_T_FFN1_BEGIN = 3,
    FE2O3_EP_T_FFN1_FIRST_WAIT_DONE = 4, FE2O3_EP_T_FFN1_LAST_WAIT_DONE = 5, FE2O3_EP_T_FFN1_END = 6,
    FE2O3_EP_T_FFN2_BEGIN = 7, FE2O3_EP_T_FFN2_END = 8, FE2O3_EP_T_COMBINE_BEGIN = 9, FE2O3_EP_T_OUTPUTS_HERE = 10,
    FE2O3_EP_T_COMBINE_END = 11, FE2O3_EP_T_OWN_ROWS_DONE = 12, FE2O3_EP_T_FFN1_TABLE_HERE = 13
};

// Capacity of the context's reduction scratch: partials followed by one counter.
#define FE2O3_REDUCE_MAX_BLOCKS 4096u

// -------------------------------------------------------------- device side
#ifdef __CUDACC__

__device__ __forceinline__ void kstatus_set(uint32_t *status, uint32_t code) {
    if (status) atomicCAS(status, 0u, code);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// Round-to-nearest-even narrowing with quieted NaNs
// (crates/fe2o3-device/src/half.rs:182-190).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
    uint32_t bits = __float_as_uint(v);
    if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x007fffffu) != 0u)
        return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t lsb = (bits >> 16) & 1u;
    return (uint16_t)((bits + 0x7fffu + lsb) >> 16);
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// Route weights of one token (softmax over the experts renormalised over the two winners = softmax
// over the two winning logits): e1 = exp(l1 - l0) <= 1, w0 = 1 / (1 + e1) in [1/2, 1], w1 = 1 - w0,
// which is exact, so w0 + w1 == 1.0f as examples/moe_expert_v1/src/contract.rs:34 requires.
__device__ __forceinline__ void route_weight_pair(float l0, float l1, float &w0, float &w1) {
    const float e1 = expf(l1 - l0);
    w0 = __fdiv_rn(1.0f, __fadd_rn(1.0f, e1));
    w1 = __fsub_rn(1.0f, w0);
}

// ---- system-scope flags (expert-parallel exchange) -----------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until *flag has reached `epoch` (flags only grow; the comparison survives wrap-around).
// Returns false after `limit` polls.
__device__ __forceinline__ bool flag_wait(const uint32_t *flag, uint32_t epoch, uint32_t limit) {
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
        if (++spins > limit) return false;
        __nanosleep(64);
    }
    return true;
}
#ifdef FE2O3_EP_TRACE
__device__ __forceinline__ void ep_trace(uint32_t *flags, uint32_t slot) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    reinterpret_cast<unsigned long long *>(flags + FE2O3_EP_TRACE_WORD)[slot] = t;
}
#else
__device__ __forceinline__ void ep_trace(uint32_t *, uint32_t) {}
#endif
// Programmatic dependent launch: lets the next kernel of the stream, if it was launched with programmatic
// stream serialization, start once every block of this grid has executed this (or exited).  That kernel
// sees none of this grid's memory effects unless it synchronises by other means (flags, here).
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Orders this thread's earlier generic-proxy observations (a flag it acquired) before its later
// asynchronous-proxy reads of global memory (bulk tensor loads of the rows that flag covers).
__device__ __forceinline__ void fence_proxy_async_global() {
    asm volatile("fence.proxy.async.global;" ::: "memory");
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// One lane of a converged warp.  A role that runs its loop with the whole warp converged and issues
// its TMA / tcgen05 instructions under this predicate lets the compiler keep descriptors and
// addresses in uniform registers; the same loop under `if (lane == 0)` is a divergent region where
// every operand has to be moved into a uniform register per instruction.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
// Non-blocking probe: try_wait may suspend the thread for a hardware-chosen time before it
// answers, which stalls a thread that polls several barriers in turn; test_wait returns at once.
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls so a protocol error can never hang
// the device; the caller records FE2O3_KSTATUS_WAIT_EXPIRED and unwinds.
#define FE2O3_SPIN_LIMIT (1u << 22)
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    if (mbar_test(bar, parity)) return true;   // the common case in a running pipeline: already complete
    for (uint32_t i = 0; i < FE2O3_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(32);
    }
    return false;
}
// The same wait for a role that keeps its whole warp converged: every lane polls and the verdict is
// made warp-uniform, so no lane can leave the role's loop while the others go on to a warp-wide
// instruction (elect, __syncwarp, a collective TMEM load).
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity)) != 0;
}
// Waits of roles that depend on another role of the same CTA: when that role has given up (it sets
// *abort), the pipeline will never advance, so the wait ends at its next look at the flag instead of
// running out its own limit.  The flag is only read on the slow path.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, const volatile int *abort) {
    bool done = mbar_test(bar, parity);
    for (uint32_t i = 0; !done && i < FE2O3_SPIN_LIMIT; ++i) {
        done = mbar_try_wait(bar, parity);
        if (!done && i > 64) {
            __nanosleep(32);
            if ((i & 127u) == 127u && *abort) break;
        }
    }
    return __all_sync(0xffffffffu, done) != 0;
}
// Arrival with a count: stands in for `n` parties at once.
__device__ __forceinline__ void mbar_arrive_n(uint64_t *bar, uint32_t n) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA (tiled bulk tensor copies, no cluster broadcast) ------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// Untiled bulk copy global -> shared: both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load_1d(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Tiled bulk store shared -> global (rows outside the tensor are clipped), tracked by bulk groups.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *m, const void *src, int32_t x, int32_t y, int32_t z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *m, const void *src, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_u32(src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the committed bulk stores of this thread are complete (their writes performed).
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Waits until the committed bulk stores of this thread have finished READING shared memory.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *m, uint64_t *bar, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *m, uint64_t *bar, int32_t x, int32_t y,
                                            int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// ---- tcgen05 / TMEM ---------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate == 0 overwrites D.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Makes the mbarrier observe completion of all MMAs issued so far by this thread.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane
// (taddr.lane + t), columns taddr.col .. +31.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Store counterpart of tmem_ld_32x32b_x32: thread t writes lane (taddr.lane + t), 32 consecutive columns.
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
          "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
          "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]: the A operand is read from tensor memory (128 lanes = rows,
// two 16-bit K elements per 32-bit column, lower K index in the lower half).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// 8-column variants for rarely taken read-modify-write paths (few live registers).
__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Packed pairs of f32 in one 64-bit register: one instruction does two independent f32 operations
// (each lane rounded as the scalar instruction would), halving the issue slots of elementwise work.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// Three-input maximum (one instruction).
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading and
// stride byte offsets in 16-byte units, descriptor version 1 in bits 46-47,
// swizzle mode in bits 61-63 (2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16 / kind::tf32 with f32 accumulation.
// format: 0 = f16, 1 = bf16, 2 = tf32.  a_mn / b_mn: 1 when the operand's
// contiguous dimension is M (resp. N) instead of K.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t format, uint32_t m, uint32_t n, uint32_t a_mn,
                                                  uint32_t b_mn) {
    return (1u << 4) | (format << 7) | (format << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) |
           ((m >> 4) << 24);
}

#endif  // __CUDACC__
