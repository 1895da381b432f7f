/*
 * fe2o3_b200 — C ABI of the B200-native example kernels.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an
 * int32 status (0 = ok, negative = FE2O3_ERR_*, positive = raw cudaError_t) and
 * never throws or unwinds.  Handles are opaque and single-owner: a handle may
 * be used from one thread at a time; distinct handles may be used from distinct
 * threads.  Each declaration cites the interface of harsh-nod/fe2o3 that it
 * replaces (paths are relative to that project's root).
 *
 * Kernel argument blocks reproduce the reference's explicit kernarg layout:
 * every slice is (u64 device address, u64 element count), in declaration
 * order, scalars packed naturally after the slices, little-endian, 8-byte
 * aligned (crates/fe2o3-host/src/lib.rs:462-480;
 * crates/fe2o3-host/src/generated_flash_attention_v1.rs:319-324).  The 256
 * hidden bytes AMD appends are not reproduced.
 */
#ifndef FE2O3_B200_H
#define FE2O3_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
/* Error classes of crates/fe2o3-core/src/error.rs:48-90 and of the generated
 * host adapters (generated_flash_attention_v1.rs:329-360). */
#define FE2O3_OK 0
#define FE2O3_ERR_NO_DEVICE -1
#define FE2O3_ERR_INVALID_ARGUMENT -2
#define FE2O3_ERR_SIZE_OVERFLOW -3
#define FE2O3_ERR_DEVICE_MISMATCH -4      /* OperationDeviceMismatch / WrongContext */
#define FE2O3_ERR_LENGTH -5               /* Length{role,expected,actual} */
#define FE2O3_ERR_ALIGNMENT -6            /* Alignment{role} */
#define FE2O3_ERR_NULL_ADDRESS -7         /* NullAddress{role} */
#define FE2O3_ERR_INVALID_REGION -8       /* InvalidRegion / RegionOverflow */
#define FE2O3_ERR_OUTPUT_ALIASES_INPUT -9 /* OutputAliasesInput{input} */
#define FE2O3_ERR_UNSUPPORTED_SHAPE -10   /* planner rejection (contract.rs:387-427) */
#define FE2O3_ERR_AMBIGUOUS_COMPLETION -11 /* bounded wait expired: keep buffers alive */
#define FE2O3_ERR_KERNEL_STATUS -12       /* kernel-side validation wrote a status word */
#define FE2O3_ERR_UNKNOWN_SYMBOL -13
#define FE2O3_ERR_NOT_SM100 -14           /* target check: device is not sm_100 */
#define FE2O3_ERR_NONFINITE -15           /* finite-input policy violated */
#define FE2O3_ERR_EXECUTABLE_REJECTED -16 /* load_executable: digest or image mismatch */
#define FE2O3_ERR_NO_DISPATCH 1000        /* not an error: plan says "nothing to launch" */

/* Device-side status words written instead of trapping
 * (reference kernels call fe2o3_device::trap(), e.g.
 * examples/moe_top2_v1/src/kernel.rs:118-131). */
#define FE2O3_KSTATUS_OK 0u
#define FE2O3_KSTATUS_LENGTH 1u
#define FE2O3_KSTATUS_NONFINITE 2u
#define FE2O3_KSTATUS_WEIGHTS 3u
#define FE2O3_KSTATUS_WAIT_EXPIRED 4u
#define FE2O3_KSTATUS_SLOT_RANGE 5u

typedef struct fe2o3_ctx fe2o3_ctx;
typedef struct fe2o3_stream fe2o3_stream;
typedef struct fe2o3_buf fe2o3_buf;
typedef struct fe2o3_event fe2o3_event;
typedef struct fe2o3_prepared fe2o3_prepared;

/* (u64 device address, u64 element count): crates/fe2o3-host/src/lib.rs:472-479 */
typedef struct fe2o3_slice {
    uint64_t ptr;
    uint64_t len;
} fe2o3_slice;

/* ---- context / stream / buffer / event --------------------------------- */

/* crates/fe2o3-core/src/context.rs:11-28 GpuContext::new(device_id).  Fails with
 * FE2O3_ERR_NOT_SM100 unless the device reports compute capability 10.x
 * (replaces the gfx942 target-id check of crates/fe2o3-amd-target). */
int32_t fe2o3_ctx_create(int32_t device, fe2o3_ctx **out);
int32_t fe2o3_ctx_destroy(fe2o3_ctx *ctx);
/* context.rs:44-62 bind_to_thread */
int32_t fe2o3_ctx_bind_to_thread(fe2o3_ctx *ctx);
int32_t fe2o3_ctx_device(const fe2o3_ctx *ctx, int32_t *device);

/* Fixed-width property record: crates/fe2o3-hip-sys/native/device_properties.h
 * and the adapter's observe_environment
 * (crates/fe2o3-host/src/hsa_executable_lifecycle.rs:963-975). */
typedef struct fe2o3_device_properties {
    char name[64];
    uint64_t total_global_bytes;
    uint32_t compute_major, compute_minor;
    uint32_t multiprocessors;
    uint32_t max_shared_bytes_per_block_optin;
    uint32_t l2_bytes;
    uint32_t sm_clock_khz, mem_clock_khz;
    uint32_t warp_size;
} fe2o3_device_properties;
int32_t fe2o3_ctx_observe_environment(fe2o3_ctx *ctx, fe2o3_device_properties *out);

/* context.rs:30-42 default_stream / create_stream; stream.rs:56-59 synchronize */
int32_t fe2o3_stream_default(fe2o3_ctx *ctx, fe2o3_stream **out);
int32_t fe2o3_stream_create(fe2o3_ctx *ctx, fe2o3_stream **out);
int32_t fe2o3_stream_sync(fe2o3_stream *stream);
int32_t fe2o3_stream_destroy(fe2o3_stream *stream);
/* The raw cudaStream_t, for callers that also drive NCCL on the same stream. */
int32_t fe2o3_stream_native(fe2o3_stream *stream, void **cuda_stream);
/* Wrap an existing cudaStream_t (not owned; destroy only frees the wrapper). */
int32_t fe2o3_stream_wrap(fe2o3_ctx *ctx, void *cuda_stream, fe2o3_stream **out);

/* crates/fe2o3-core/src/memory.rs:435-492 DeviceBuffer<T>::{zeroed, from_host,
 * to_host_vec, len, as_device_ptr}; from_host/to_host are synchronous with
 * respect to the stream; free = Drop (memory.rs:129-162).  A buffer remembers
 * its context; using it with another context's stream is
 * FE2O3_ERR_DEVICE_MISMATCH. */
int32_t fe2o3_buf_alloc_zeroed(fe2o3_stream *stream, uint64_t elements, uint32_t element_bytes,
                               fe2o3_buf **out);
int32_t fe2o3_buf_from_host(fe2o3_stream *stream, const void *host, uint64_t elements,
                            uint32_t element_bytes, fe2o3_buf **out);
int32_t fe2o3_buf_to_host(fe2o3_stream *stream, const fe2o3_buf *buf, void *host, uint64_t elements);
/* Copies into / out of an existing buffer (async on the stream; the host side
 * should be pinned for real overlap): crates/fe2o3-core/src/operation.rs:272-420. */
int32_t fe2o3_buf_copy_from_host_async(fe2o3_stream *stream, fe2o3_buf *buf, const void *host,
                                       uint64_t elements);
int32_t fe2o3_buf_copy_to_host_async(fe2o3_stream *stream, const fe2o3_buf *buf, void *host,
                                     uint64_t elements);
int32_t fe2o3_buf_free(fe2o3_buf *buf);
/* Marks the buffer as possibly still in use by the device: free becomes a
 * deliberate leak (memory.rs:129-161 "leak rather than free"). */
int32_t fe2o3_buf_quarantine(fe2o3_buf *buf);
uint64_t fe2o3_buf_ptr(const fe2o3_buf *buf);
uint64_t fe2o3_buf_len(const fe2o3_buf *buf);
/* view / view_mut / split_at_mut (memory.rs:494-560) reduce to a checked
 * sub-slice: FE2O3_ERR_INVALID_REGION when [start, start+len) leaves the buffer. */
int32_t fe2o3_buf_slice(const fe2o3_buf *buf, uint64_t start, uint64_t len, fe2o3_slice *out);

/* ---- owned asynchronous operations -------------------------------------- */
/* crates/fe2o3-core/src/operation.rs:272-420 OwnedDeviceOperation: a submitted
 * operation owns every buffer it may touch until completion has been
 * established.  In Rust the buffers move into the operation; here submit marks
 * them as owned: fe2o3_buf_free on an owned buffer fails with FE2O3_ERR_BUSY and
 * frees nothing.  The work is a prepared launch (optional) preceded by
 * host-to-device copies and followed by device-to-host copies (both optional),
 * all asynchronous on `stream`.
 *   is_complete (operation.rs:318-324): non-blocking; errors leave it submitted.
 *   wait (:326-360): the completion event is polled up to timeout_ms; on completion
 *     the buffers are released, the kernel status word is read and the operation is
 *     destroyed.  If the event reports an error the whole stream is synchronised
 *     instead: when that succeeds the buffers are released and the event's error is
 *     returned; when both fail, completion is unknown: every buffer is quarantined
 *     (its free becomes a deliberate leak, crates/fe2o3-core/src/memory.rs:129-161),
 *     the operation is destroyed and FE2O3_ERR_AMBIGUOUS_COMPLETION is returned.
 *     When the deadline passes with the work still running the call returns
 *     FE2O3_ERR_STILL_RUNNING and the operation STAYS submitted and owning (wait
 *     again, or abandon); every other return value has consumed the operation.
 *   abandon: quarantines the buffers and destroys the operation without waiting
 *     (the Quiescent/Ambiguous policy of crates/fe2o3-completion/src/lib.rs:46-60). */
#define FE2O3_ERR_BUSY -17          /* the buffer is owned by a submitted operation */
#define FE2O3_ERR_STILL_RUNNING -18 /* operation wait: deadline passed, the operation stays submitted */
typedef struct fe2o3_operation fe2o3_operation;
typedef struct fe2o3_host_copy {
    fe2o3_buf *buffer;  /* owned by the operation until completion */
    void *host;         /* pinned for real overlap; must stay valid until completion */
    uint64_t elements;
} fe2o3_host_copy;
int32_t fe2o3_operation_submit(fe2o3_stream *stream, fe2o3_prepared *prepared, fe2o3_buf *const *buffers,
                               uint32_t n_buffers, const fe2o3_host_copy *copies_in, uint32_t n_in,
                               const fe2o3_host_copy *copies_out, uint32_t n_out, fe2o3_operation **out);
int32_t fe2o3_operation_is_complete(fe2o3_operation *op, int32_t *done);
int32_t fe2o3_operation_wait(fe2o3_operation *op, uint32_t timeout_ms, uint32_t *kernel_status);
int32_t fe2o3_operation_abandon(fe2o3_operation *op);

/* crates/fe2o3-core/src/pinned_memory.rs */
int32_t fe2o3_pinned_alloc(fe2o3_ctx *ctx, uint64_t bytes, void **out);
int32_t fe2o3_pinned_free(fe2o3_ctx *ctx, void *ptr);

/* crates/fe2o3-core/src/event.rs:82-148 */
int32_t fe2o3_event_create(fe2o3_ctx *ctx, fe2o3_event **out);
int32_t fe2o3_event_record(fe2o3_event *event, fe2o3_stream *stream);
int32_t fe2o3_event_sync(fe2o3_event *event);
/* *done = 1 when complete, 0 when still running */
int32_t fe2o3_event_query(fe2o3_event *event, int32_t *done);
int32_t fe2o3_event_elapsed_ms(fe2o3_event *start, fe2o3_event *end, float *ms);
/* Work enqueued on `stream` after this call starts only when `event` has completed (device-side
 * ordering between two streams of one context; the host does not block).  The reference runs one
 * stream per operation and names cross-stream ordering a caller obligation
 * (crates/fe2o3-core/src/operation.rs:296-305); this is the call that discharges it when copies
 * and kernels of consecutive steps overlap on separate streams. */
int32_t fe2o3_stream_wait_event(fe2o3_stream *stream, fe2o3_event *event);
int32_t fe2o3_event_destroy(fe2o3_event *event);

/* crates/fe2o3-core/src/peer_access.rs:24-60 */
int32_t fe2o3_peer_access_enable(fe2o3_ctx *ctx, int32_t peer_device);

/* Peer-visible device memory for one-process-per-GPU layouts (the capability of
 * crates/fe2o3-core/src/peer_access.rs:24-60 across process boundaries).  The
 * owner creates a zero-filled region and exports a 64-byte handle; it hands the
 * handle to the other processes of the node over any host channel; each of
 * them imports it and gets an address in its own address space through which
 * its kernels load and store the owner's memory over NVLink (peer access to the
 * owner's device is enabled on import).  Destroy closes an imported mapping or
 * frees an owned region; the owner must outlive the importers' use. */
typedef struct fe2o3_peer_region fe2o3_peer_region;
#define FE2O3_PEER_HANDLE_BYTES 64
int32_t fe2o3_peer_region_create(fe2o3_ctx *ctx, uint64_t bytes, fe2o3_peer_region **out);
int32_t fe2o3_peer_region_export(const fe2o3_peer_region *region, uint8_t handle[FE2O3_PEER_HANDLE_BYTES]);
int32_t fe2o3_peer_region_import(fe2o3_ctx *ctx, const uint8_t handle[FE2O3_PEER_HANDLE_BYTES],
                                 fe2o3_peer_region **out);
uint64_t fe2o3_peer_region_ptr(const fe2o3_peer_region *region);
uint64_t fe2o3_peer_region_bytes(const fe2o3_peer_region *region); /* 0 for an imported mapping */
int32_t fe2o3_peer_region_destroy(fe2o3_peer_region *region);

const char *fe2o3_status_string(int32_t status);
/* Human-readable detail of the calling thread's last failure (role, expected,
 * actual), mirroring the adapter error payloads. */
const char *fe2o3_last_error(void);

/* ---- kernel argument blocks -------------------------------------------- */

/* examples/scalar_gemm_v1/src/kernel.rs:8 scalar_gemm_v1(a,b,c,m,n,k): f32
 * row-major C = A*B, sequential k, separate product and sum. 64-byte block. */
typedef struct fe2o3_scalar_gemm_v1_args {
    fe2o3_slice a, b, c;
    uint32_t m, n, k, reserved;
} fe2o3_scalar_gemm_v1_args;

/* examples/tiled_gemm_v1/src/kernel.rs:63-67 tiled_gemm_lds_slice1(a:&[u16],
 * b:&[u16], c) generalised from one 16x16x16 tile to the planner's admitted
 * shapes (M,N,K multiples of 16, src/contract.rs:387-427): bf16 bits in, f32
 * out, zero accumulator, packed row-major. */
typedef struct fe2o3_tiled_gemm_v1_args {
    fe2o3_slice a, b, c;
    uint32_t m, n, k, reserved;
} fe2o3_tiled_gemm_v1_args;

/* examples/tiled_gemm_general_v1/src/kernel.rs:67-79 and the 80-byte explicit
 * block of hardware-harness/src/lib.rs:578-593 (scalars at offsets 48..76):
 * C = alpha*(A*B) + beta*C with leading dimensions, tails zero-filled. */
typedef struct fe2o3_tiled_gemm_general_v1_args {
    fe2o3_slice a, b, c;
    uint32_t m, n, k, lda, ldb, ldc;
    float alpha, beta;
} fe2o3_tiled_gemm_general_v1_args;

/* GEMM schedule selector (hardware-harness/src/lib.rs:135-136 names two
 * schedules for one kernel; here: the exact-order CUDA-core schedule that is
 * bit-identical to the CPU recurrence, and the tcgen05 tensor-core schedule). */
#define FE2O3_GEMM_SCHEDULE_EXACT_ORDER 0u
#define FE2O3_GEMM_SCHEDULE_TCGEN05 1u
#define FE2O3_GEMM_SCHEDULE_AUTO 2u

/* examples/flash_attention_v1/src/kernel.rs:130-136 (q,k,v,output), row-major
 * [seq][dim] per head, f32 output.  The fixed B1/H1/N8/D16 causal f32 profile
 * is batch=heads=1, seq=8, dim=16, scale=0.25, causal=1, input_dtype=F32. */
#define FE2O3_DTYPE_F32 0u
#define FE2O3_DTYPE_BF16 1u
typedef struct fe2o3_flash_attention_v1_args {
    fe2o3_slice q, k, v, output;
    uint32_t batch, heads, seq, dim;
    float scale;
    uint32_t causal;
    uint32_t input_dtype;
    uint32_t reserved;
} fe2o3_flash_attention_v1_args;

/* examples/row_softmax_v1/src/kernel.rs:13 row_softmax_v1(input, output)
 * generalised to rows x cols; mask.ptr == 0 means unmasked, else one u8 per
 * element (src/numerical_contract.rs:130-199: masked outputs are +0.0). */
typedef struct fe2o3_row_softmax_v1_args {
    fe2o3_slice input, output, mask;
    uint32_t rows, cols;
} fe2o3_row_softmax_v1_args;

/* examples/moe_top2_v1/src/kernel.rs:102-111: one input and seven u32 outputs
 * (128-byte slice block, crates/fe2o3-host/src/generated_moe_top2_v1.rs:19-28),
 * then tokens, experts, capacity.  The fixed profile is tokens=8, experts=4,
 * capacity=4.  `scratch` is experts*(blocks+1)+... u32 of device workspace; see
 * fe2o3_moe_top2_v1_scratch_elements. */
typedef struct fe2o3_moe_top2_v1_args {
    fe2o3_slice logits, top2_experts, requested_counts, admitted_counts, expert_offsets,
        route_slots, permutation, inverse;
    uint32_t tokens, experts, capacity, reserved;
} fe2o3_moe_top2_v1_args;

/* Gate logits (no reference kernel; arithmetic policy of
 * examples/tiled_gemm_v1/src/numerical_contract.rs:5-11): logits[t,e] =
 * sum_k x[t,k]*wg[k,e], bf16 widened exactly, f32, increasing k, separate
 * product and sum. */
typedef struct fe2o3_moe_gate_v1_args {
    fe2o3_slice x, wg, logits;
    uint32_t tokens, d_model, experts, reserved;
} fe2o3_moe_gate_v1_args;

/* Route weights over the two winners; each pair sums to exactly 1.0
 * (examples/moe_expert_v1/src/contract.rs:34). */
typedef struct fe2o3_moe_route_weights_v1_args {
    fe2o3_slice logits, top2_experts, route_weights;
    uint32_t tokens, experts;
} fe2o3_moe_route_weights_v1_args;

/* Expert schedule of examples/moe_expert_v1/src/pipeline.rs:166-270 (compact ->
 * GEMM per expert -> compact rows) with the expert widened to
 * GELU(x*W1)*W2 (GELU in its erf form; the kernel evaluates erf by Abramowitz &
 * Stegun 7.1.26, absolute error below 1.5e-7, before the hidden activation is
 * rounded to bf16, whose step is 4e-3 relative; the oracle uses the C library's
 * erf: outputs agree within the stated tolerance, not bit for bit).
 * x [tokens][d_model] bf16, w1 [E][d_model][d_ff] bf16,
 * w2 [E][d_ff][d_model] bf16, permutation/expert_offsets from routing;
 * compact_x [rows][d_model] bf16 and hidden [rows][d_ff] bf16 are
 * caller-provided workspace; compact_output [rows][d_model] f32.
 * rows = compact_output.len / d_model.  When d_model is a multiple of 64 the
 * first GEMM gathers the rows of x through `permutation` itself and compact_x
 * is left untouched (two launches instead of three; the prepared geometry says
 * which); the results are the same bits either way. */
typedef struct fe2o3_moe_expert_ffn_v1_args {
    fe2o3_slice x, w1, w2, permutation, expert_offsets, compact_x, hidden, compact_output;
    uint32_t tokens, d_model, d_ff, experts;
} fe2o3_moe_expert_ffn_v1_args;

/* The expert schedule and the combine of examples/moe_expert_v1/src/kernel.rs:104-157
 * in one operation, for callers that do not need the expert outputs by slot:
 * the first GEMM gathers the rows of x through `permutation`, and the second
 * one multiplies every output row by its route's weight and adds it to the
 * token's row of combined_output (cleared by the first GEMM).  A token has
 * at most two routes and the sum starts from +0, so the result is the same bits
 * as moe_expert_ffn_v1 followed by moe_expert_combine_v1, whichever route's row
 * is added first; dropped routes contribute nothing.  A token whose weights are
 * non-finite, negative or do not sum to exactly 1.0 records
 * FE2O3_KSTATUS_WEIGHTS and gets no contribution (its row stays zero, where
 * the separate combine leaves it unwritten).  rows = permutation.len;
 * hidden [rows][d_ff] bf16 is workspace.  Needs d_model a multiple of 64
 * (otherwise Unsupported: use the separate operations). */
typedef struct fe2o3_moe_expert_ffn_combine_v1_args {
    fe2o3_slice x, w1, w2, permutation, expert_offsets, route_weights, hidden, combined_output;
    uint32_t tokens, d_model, d_ff, experts;
} fe2o3_moe_expert_ffn_combine_v1_args;

/* The two halves of the expert schedule as separate launches, for the
 * expert-parallel layout where an all-to-all sits between them.
 * moe_compact_v1: compact_x[slot,:] = x[permutation[slot]/2,:], zero rows for
 * unused slots (pipeline.rs:181-215); rows = permutation.len.
 * moe_grouped_ffn_v1: GELU(x*W1)*W2 over `groups` consecutive row segments
 * given by group_offsets[0..groups]; segment g uses expert (g % experts_cycle)
 * of w1 [experts_cycle][d_model][d_ff] and w2 [experts_cycle][d_ff][d_model]
 * (rows that arrive source-rank-major, local-expert-minor). */
typedef struct fe2o3_moe_compact_v1_args {
    fe2o3_slice x, permutation, compact_x;
    uint32_t tokens, d_model;
} fe2o3_moe_compact_v1_args;

typedef struct fe2o3_moe_grouped_ffn_v1_args {
    fe2o3_slice compact_x, w1, w2, group_offsets, hidden, compact_output;
    uint32_t d_model, d_ff, groups, experts_cycle;
} fe2o3_moe_grouped_ffn_v1_args;

/* Expert-parallel layer over peer memory (no counterpart in the reference,
 * which is single-device).  One rank per GPU; rank r owns tokens/world tokens
 * and experts [r*per, (r+1)*per), per = experts/world.  The peer_* slices are
 * device arrays of `world` u64 addresses, entry p being rank p's buffer mapped
 * into this process (fe2o3_peer_region_* below, or any other peer mapping):
 *   recv_x    [max_rows][d_model] bf16   rows routed to the rank's experts
 *   recv_meta [max_rows] {u32 route id, u32 home rank}   where each row came from
 *   ret       [2*tokens][d_model] f32    expert outputs by route id, on the home rank
 *   counts    [world][experts] u32       admitted routes per (source rank, expert)
 *   flags     [5*world + 6] u32, zero before the first pass
 * Rows on the owner o of an expert are ordered local-expert-major, and inside an
 * expert's segment by source in the order o, o+1, ... (mod world): the owner's own
 * rows first.  Each expert's rows are one contiguous segment; pair_offsets[le*world + k]
 * is the first row of (local expert le, source (o + k) mod world),
 * pair_offsets[experts] the row count.
 *
 * The pass number ("epoch") must increase by one per layer pass on every rank:
 * either patch `epoch` in all three prepared blocks before each pass
 * (fe2o3_prepared_patch_kernarg) or give `epoch_counter`, one local u32 that
 * starts at 0: the kernels then use *epoch_counter + 1 and the COMBINE phase
 * increments it, so that a whole pass replays from one CUDA graph.
 *
 * One pass, in stream order:
 *   moe_ep_exchange_v1, phase DISPATCH  publish counts; when `logits`
 *       ([tokens][experts] f32, optional) is given, write route_weights from it as
 *       fe2o3_moe_route_weights_v1 does, while the counts travel; wait for every rank's
 *       counts, write pair_offsets, store this rank's accepted rows and their
 *       (route, home) records into the owners' receive buffers, raise
 *       "rows complete" on every rank.
 *   moe_ep_ffn_v1  GELU(x*W1)*W2 over the received rows as two grouped tcgen05
 *       GEMMs.  The first is launched so that it may start while the dispatch
 *       kernel before it in the stream is still sending (programmatic dependent
 *       launch); it waits per source rank, inside the kernel, for "rows complete"
 *       right before it first loads rows of that source, and takes the tiles in the
 *       order the rows arrive (this rank's own first, then ranks +1, +2, ...: every
 *       rank sends to rank-1 first, then rank-2, ...); the second stores every output row straight
 *       into the return buffer of the row's home rank from its epilogue and,
 *       when its last tile is stored, raises "outputs ready" on every rank.
 *   moe_ep_exchange_v1, phase COMBINE   wait for "outputs ready" of every rank,
 *       then out[t] = w0*ret[2t] + w1*ret[2t+1] in rank order from local memory
 *       (examples/moe_expert_v1/src/kernel.rs:104-157).
 * Every device-side wait gives up after `spin_limit` polls (0 = the default of
 * 2^24, about a second) and records FE2O3_KSTATUS_WAIT_EXPIRED; a pass that
 * reports it is void on every rank. */
#define FE2O3_MOE_EP_DISPATCH 0u
#define FE2O3_MOE_EP_COMBINE 1u
typedef struct fe2o3_moe_ep_exchange_v1_args {
    fe2o3_slice x, top2_experts, permutation, inverse, expert_offsets, admitted_counts, route_weights,
        pair_offsets, combined_output, peer_recv_x, peer_recv_meta, peer_ret, peer_counts, peer_flags,
        epoch_counter, logits;
    uint32_t tokens, d_model, experts, world, rank, epoch, max_rows, phase, spin_limit, reserved;
} fe2o3_moe_ep_exchange_v1_args;

/* The expert FFN of one rank of the expert-parallel layer (see above): recv_x,
 * recv_meta (two u32 per row) and flags are this rank's own buffers (the
 * entries `rank` of the peer tables), w1 [per][d_model][d_ff] and
 * w2 [per][d_ff][d_model] its experts, hidden [max_rows][d_ff] bf16 workspace.
 * `tokens` is the per-rank token count (a return buffer has 2*tokens rows).
 * `progress` (optional): 2 * (max_rows/128 + experts/world + 1) u32 of this rank,
 * zero before the first pass: one counter per 128-row tile of `hidden` (two sets,
 * used by alternate passes), through which
 * the first GEMM hands finished row tiles to the second, which is then launched
 * so that it takes over each SM as the first GEMM's block leaves it instead of
 * waiting for the whole first GEMM (it clears the other set for the next pass). */
typedef struct fe2o3_moe_ep_ffn_v1_args {
    fe2o3_slice recv_x, w1, w2, pair_offsets, hidden, recv_meta, flags, peer_ret, peer_flags, epoch_counter, progress;
    uint32_t tokens, d_model, d_ff, experts, world, rank, epoch, max_rows, spin_limit, reserved;
} fe2o3_moe_ep_ffn_v1_args;

/* examples/moe_expert_v1/src/kernel.rs:104-109
 * moe_expert_combine_f32_t8_k2_o16_v1(compact_output, inverse, route_weights,
 * combined_output) generalised to tokens x width. */
typedef struct fe2o3_moe_expert_combine_v1_args {
    fe2o3_slice compact_output, inverse, route_weights, combined_output;
    uint32_t tokens, width;
} fe2o3_moe_expert_combine_v1_args;

/* Device-wide masked u32 wrapping sum composed from
 * crates/fe2o3-device/src/collective.rs:202 wave64_reduce_sum_active_u32 and
 * :221 workgroup256_reduce_sum_active_u32: active flag 0 contributes zero, any
 * other flag contributes the value.  output.len == 1. */
typedef struct fe2o3_masked_reduce_u32_args {
    fe2o3_slice values, active, output;
} fe2o3_masked_reduce_u32_args;

/* Same sum with the activity packed one bit per lane in u64 words
 * (examples/wave64_collectives_v1/src/kernel.rs:25,44). */
typedef struct fe2o3_masked_reduce_u32_packed_args {
    fe2o3_slice values, mask, output;
} fe2o3_masked_reduce_u32_packed_args;

/* Device-wide prefix sum of u32 values with wrapping addition: the wave64 and
 * workgroup inclusive_scan_sum / exclusive_scan_sum of
 * crates/fe2o3-device/src/collective.rs:413-460 and :503-571 extended to a whole
 * array (output[i] = values[0] + ... + values[i]; the exclusive form is shifted
 * by one and starts at zero).  values.len == output.len <= 2^31; the output
 * may not overlap the input; one scan at a time per context. */
#define FE2O3_SCAN_MAX_ELEMENTS (1ull << 31)
typedef struct fe2o3_device_scan_u32_args {
    fe2o3_slice values, output;
    uint32_t exclusive; /* 0 inclusive, 1 exclusive */
    uint32_t reserved;
} fe2o3_device_scan_u32_args;

/* The same scan over IEEE binary32 values, each addition rounded to nearest.  No
 * reference order exists at array scope (the reference defines f32 scans inside one
 * wave only), so the result is specified by tolerance: output[i] is within
 * (128 + len / 8192 / 192) * 2^-24 * (|values[0]| + ... + |values[i]|) of the exact
 * prefix (the bracket bounds the roundings on any path).  The order of additions
 * depends only on element positions, not on scheduling: repeated runs give identical
 * bits. */
typedef fe2o3_device_scan_u32_args fe2o3_device_scan_f32_args;

/* crates/rustc-codegen-fe2o3/tests/fixtures/memory-v1-compiler/src/bin/gfx942_wave_lds_v1.rs:7-15
 * with the runner's (ptr,len)x4 arguments
 * (crates/dialect-amdgcn/tests/fixtures/gfx942_wave_lds_v1_runner.cpp:62-68):
 * every lane receives its 64-lane wave sum and its 256-lane workgroup sum. */
typedef struct fe2o3_wave_lds_v1_args {
    fe2o3_slice values, active, wave_out, workgroup_out;
} fe2o3_wave_lds_v1_args;

/* examples/wave64_collectives_v1/src/kernel.rs:23-29; 72-byte block with the
 * u64 mask between the slices
 * (crates/fe2o3-host/src/generated_wave64_collectives_v1.rs:19-24). */
typedef struct fe2o3_wave64_collectives_v1_args {
    fe2o3_slice input;
    uint64_t active_mask;
    fe2o3_slice reduction_output, inclusive_output, exclusive_output;
} fe2o3_wave64_collectives_v1_args;

/* Segmented extension: one u64 mask per 64-lane segment. */
typedef struct fe2o3_wave64_collectives_segmented_args {
    fe2o3_slice input, masks, reduction_output, inclusive_output, exclusive_output;
} fe2o3_wave64_collectives_segmented_args;

/* examples/workgroup_sync_v1/src/kernel.rs:28-31 */
typedef struct fe2o3_lds_publish_read_reduce_i32_v1_args {
    fe2o3_slice values, output;
} fe2o3_lds_publish_read_reduce_i32_v1_args;

/* examples/workgroup_sync_v1/src/scoped_atomic.rs:21 (40-byte block) */
typedef struct fe2o3_scoped_atomic_add_u32_v1_args {
    fe2o3_slice values, eligible;
    uint64_t target;
} fe2o3_scoped_atomic_add_u32_v1_args;

/* ---- checked prepare + launch ------------------------------------------ */
/* Each *_check is the pure host part of the generated adapters' prepare
 * (crates/fe2o3-host/src/generated_flash_attention_v1.rs:223-325): shape
 * admission, per-region length / null / alignment / overflow checks and
 * output-aliases-input rejection.  It makes no CUDA call.  *_prepare runs the
 * check, verifies that every region lives on the context's device, and packs
 * the argument block.  FE2O3_ERR_NO_DISPATCH from a GEMM prepare means the
 * plan is "empty output: nothing to launch" (contract.rs:401-407). */
int32_t fe2o3_scalar_gemm_v1_check(const fe2o3_scalar_gemm_v1_args *args);
int32_t fe2o3_tiled_gemm_v1_check(const fe2o3_tiled_gemm_v1_args *args);
int32_t fe2o3_tiled_gemm_general_v1_check(const fe2o3_tiled_gemm_general_v1_args *args);
int32_t fe2o3_flash_attention_v1_check(const fe2o3_flash_attention_v1_args *args);
int32_t fe2o3_row_softmax_v1_check(const fe2o3_row_softmax_v1_args *args);
int32_t fe2o3_moe_top2_v1_check(const fe2o3_moe_top2_v1_args *args);
int32_t fe2o3_moe_gate_v1_check(const fe2o3_moe_gate_v1_args *args);
int32_t fe2o3_moe_route_weights_v1_check(const fe2o3_moe_route_weights_v1_args *args);
int32_t fe2o3_moe_expert_ffn_v1_check(const fe2o3_moe_expert_ffn_v1_args *args);
int32_t fe2o3_moe_expert_combine_v1_check(const fe2o3_moe_expert_combine_v1_args *args);
int32_t fe2o3_moe_compact_v1_check(const fe2o3_moe_compact_v1_args *args);
int32_t fe2o3_moe_grouped_ffn_v1_check(const fe2o3_moe_grouped_ffn_v1_args *args);
int32_t fe2o3_moe_expert_ffn_combine_v1_check(const fe2o3_moe_expert_ffn_combine_v1_args *args);
int32_t fe2o3_moe_ep_exchange_v1_check(const fe2o3_moe_ep_exchange_v1_args *args);
int32_t fe2o3_moe_ep_ffn_v1_check(const fe2o3_moe_ep_ffn_v1_args *args);
int32_t fe2o3_masked_reduce_u32_check(const fe2o3_masked_reduce_u32_args *args);
int32_t fe2o3_masked_reduce_u32_packed_check(const fe2o3_masked_reduce_u32_packed_args *args);
int32_t fe2o3_device_scan_u32_check(const fe2o3_device_scan_u32_args *args);
int32_t fe2o3_device_scan_f32_check(const fe2o3_device_scan_f32_args *args);
int32_t fe2o3_wave_lds_v1_check(const fe2o3_wave_lds_v1_args *args);
int32_t fe2o3_wave64_collectives_v1_check(const fe2o3_wave64_collectives_v1_args *args);
int32_t fe2o3_wave64_collectives_segmented_check(const fe2o3_wave64_collectives_segmented_args *args);
int32_t fe2o3_lds_publish_read_reduce_i32_v1_check(const fe2o3_lds_publish_read_reduce_i32_v1_args *args);
int32_t fe2o3_scoped_atomic_add_u32_v1_check(const fe2o3_scoped_atomic_add_u32_v1_args *args);

int32_t fe2o3_scalar_gemm_v1_prepare(fe2o3_ctx *ctx, const fe2o3_scalar_gemm_v1_args *args,
                                     uint32_t schedule, fe2o3_prepared **out);
int32_t fe2o3_tiled_gemm_v1_prepare(fe2o3_ctx *ctx, const fe2o3_tiled_gemm_v1_args *args,
                                    uint32_t schedule, fe2o3_prepared **out);
int32_t fe2o3_tiled_gemm_general_v1_prepare(fe2o3_ctx *ctx, const fe2o3_tiled_gemm_general_v1_args *args,
                                            uint32_t schedule, fe2o3_prepared **out);
int32_t fe2o3_flash_attention_v1_prepare(fe2o3_ctx *ctx, const fe2o3_flash_attention_v1_args *args,
                                         fe2o3_prepared **out);
int32_t fe2o3_row_softmax_v1_prepare(fe2o3_ctx *ctx, const fe2o3_row_softmax_v1_args *args,
                                     fe2o3_prepared **out);
int32_t fe2o3_moe_top2_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_top2_v1_args *args,
                                  fe2o3_prepared **out);
int32_t fe2o3_moe_gate_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_gate_v1_args *args,
                                  fe2o3_prepared **out);
int32_t fe2o3_moe_route_weights_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_route_weights_v1_args *args,
                                           fe2o3_prepared **out);
int32_t fe2o3_moe_expert_ffn_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_expert_ffn_v1_args *args,
                                        fe2o3_prepared **out);
int32_t fe2o3_moe_expert_combine_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_expert_combine_v1_args *args,
                                            fe2o3_prepared **out);
int32_t fe2o3_moe_compact_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_compact_v1_args *args, fe2o3_prepared **out);
int32_t fe2o3_moe_grouped_ffn_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_grouped_ffn_v1_args *args,
                                         fe2o3_prepared **out);
int32_t fe2o3_moe_expert_ffn_combine_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_expert_ffn_combine_v1_args *args,
                                                fe2o3_prepared **out);
int32_t fe2o3_moe_ep_exchange_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_ep_exchange_v1_args *args,
                                         fe2o3_prepared **out);
int32_t fe2o3_moe_ep_ffn_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_ep_ffn_v1_args *args, fe2o3_prepared **out);
int32_t fe2o3_masked_reduce_u32_prepare(fe2o3_ctx *ctx, const fe2o3_masked_reduce_u32_args *args,
                                        fe2o3_prepared **out);
int32_t fe2o3_masked_reduce_u32_packed_prepare(fe2o3_ctx *ctx, const fe2o3_masked_reduce_u32_packed_args *args,
                                               fe2o3_prepared **out);
int32_t fe2o3_device_scan_u32_prepare(fe2o3_ctx *ctx, const fe2o3_device_scan_u32_args *args,
                                      fe2o3_prepared **out);
int32_t fe2o3_device_scan_f32_prepare(fe2o3_ctx *ctx, const fe2o3_device_scan_f32_args *args,
                                      fe2o3_prepared **out);
int32_t fe2o3_wave_lds_v1_prepare(fe2o3_ctx *ctx, const fe2o3_wave_lds_v1_args *args, fe2o3_prepared **out);
int32_t fe2o3_wave64_collectives_v1_prepare(fe2o3_ctx *ctx, const fe2o3_wave64_collectives_v1_args *args,
                                            fe2o3_prepared **out);
int32_t fe2o3_wave64_collectives_segmented_prepare(fe2o3_ctx *ctx,
                                                   const fe2o3_wave64_collectives_segmented_args *args,
                                                   fe2o3_prepared **out);
int32_t fe2o3_lds_publish_read_reduce_i32_v1_prepare(fe2o3_ctx *ctx,
                                                     const fe2o3_lds_publish_read_reduce_i32_v1_args *args,
                                                     fe2o3_prepared **out);
int32_t fe2o3_scoped_atomic_add_u32_v1_prepare(fe2o3_ctx *ctx, const fe2o3_scoped_atomic_add_u32_v1_args *args,
                                               fe2o3_prepared **out);

/* Launch geometry record of crates/fe2o3-host/src/hsa_executable_lifecycle.rs:823-853
 * (grid in blocks; AQL-style work-items = grid*workgroup). */
typedef struct fe2o3_geometry {
    uint32_t grid[3];
    uint32_t workgroup[3];
    uint32_t dynamic_shared_bytes;
    uint32_t launches; /* kernels one fe2o3_prepared_launch enqueues */
} fe2o3_geometry;

/* Asynchronous launch on a stream (crates/fe2o3-core/src/launch.rs:99-121). */
int32_t fe2o3_prepared_launch(fe2o3_prepared *prepared, fe2o3_stream *stream);
/* dispatch_and_wait of the one-shot lifecycles
 * (crates/fe2o3-host/src/flash_attention_v1_lifecycle.rs:348,577-618): launch,
 * then poll completion with a host deadline
 * (crates/fe2o3-hsa-runtime/src/dispatch.rs:40,788-827 uses 5 s and aborts;
 * here expiry returns FE2O3_ERR_AMBIGUOUS_COMPLETION and nothing is freed).
 * On completion the kernel status word is read back: nonzero gives
 * FE2O3_ERR_KERNEL_STATUS with the word in *kernel_status. */
int32_t fe2o3_prepared_launch_and_wait(fe2o3_prepared *prepared, fe2o3_stream *stream,
                                       uint32_t timeout_ms, uint32_t *kernel_status);
int32_t fe2o3_prepared_geometry(const fe2o3_prepared *prepared, fe2o3_geometry *out);
/* Copies the packed explicit argument block; *bytes in = capacity, out = size. */
int32_t fe2o3_prepared_kernarg(const fe2o3_prepared *prepared, void *out, uint64_t *bytes);
/* Overwrites `bytes` bytes of the packed block at `offset`; only the scalar area
 * after the slices may be patched (e.g. the epoch of fe2o3_moe_ep_exchange_v1). */
int32_t fe2o3_prepared_patch_kernarg(fe2o3_prepared *prepared, uint64_t offset, const void *data, uint64_t bytes);
const char *fe2o3_prepared_symbol(const fe2o3_prepared *prepared);
int32_t fe2o3_prepared_destroy(fe2o3_prepared *prepared);

/* Reads and clears the context's device status word (synchronises the stream). */
int32_t fe2o3_ctx_take_kernel_status(fe2o3_ctx *ctx, fe2o3_stream *stream, uint32_t *status);

/* ---- runtime adapter ---------------------------------------------------- */
/* The entry points of ReviewedHsaExecutableLifecycleAdapterV1
 * (crates/fe2o3-host/src/hsa_executable_lifecycle.rs:963-1071) over the
 * library's built-in sm_100a image; native shape:
 * crates/fe2o3-hsa-runtime/native/runtime.h:82-122.
 *
 * load_executable(bytes, digest) (hsa_executable_lifecycle.rs:977-990): the
 * artifact of this backend is the shared library file itself (the device code is
 * embedded in it).  The caller presents the bytes it holds a receipt for and
 * their SHA-256; the call fails with FE2O3_ERR_EXECUTABLE_REJECTED unless the
 * digest is the digest of those bytes AND of the library image loaded in this
 * process (fe2o3_image_digest), so a receipt for any other build cannot launch.
 * Nothing native stays live after a failed load.
 * resolve_kernel(exe, symbol) (:992-1003): the reference kernel function names.
 * observe_kernel_resources(exe, kernel) (:1005-1016): the compiled resources of
 * the device function that carries the symbol (the schedule large launches
 * resolve to, where an op has several).
 * launch_and_wait(exe, kernel, geometry, kernarg) (:1038-1060, geometry record
 * :823-853): `geometry` may be NULL; when given it must equal the geometry the
 * argument block plans to, else FE2O3_ERR_INVALID_ARGUMENT before submission.
 * initialize_implicit_kernarg has no counterpart: CUDA kernels take no hidden
 * arguments. */
typedef struct fe2o3_executable fe2o3_executable;
typedef struct fe2o3_kernel_resources {
    uint32_t registers_per_thread;
    uint32_t static_shared_bytes;
    uint32_t max_dynamic_shared_bytes;
    uint32_t max_threads_per_block;
    uint32_t local_bytes_per_thread; /* stack / spill space */
    uint32_t const_bytes;
} fe2o3_kernel_resources;
int32_t fe2o3_image_digest(uint8_t digest[32]);
int32_t fe2o3_load_executable(fe2o3_ctx *ctx, const void *bytes, uint64_t len, const uint8_t digest[32],
                              fe2o3_executable **out);
int32_t fe2o3_resolve_kernel(fe2o3_executable *exe, const char *symbol, uint32_t *kernel_id,
                             uint64_t *kernarg_bytes);
int32_t fe2o3_observe_kernel_resources(fe2o3_executable *exe, uint32_t kernel_id, fe2o3_kernel_resources *out);
struct fe2o3_geometry;
int32_t fe2o3_launch_and_wait(fe2o3_executable *exe, uint32_t kernel_id, const struct fe2o3_geometry *geometry,
                              const void *kernarg, uint64_t kernarg_bytes, fe2o3_stream *stream,
                              uint32_t timeout_ms, uint32_t *kernel_status);
int32_t fe2o3_unload_executable(fe2o3_executable *exe);

/* ---- deterministic synthetic inputs (host side) ------------------------- */
/* SplitMix64-keyed generators in the style of
 * examples/tiled_gemm_v1/src/inputs.rs:54-79: element i of stream
 * (seed, domain) is a pure function of (seed, domain, i). */
int32_t fe2o3_synth_uniform_f32(uint64_t seed, uint64_t domain, uint64_t n, float *out);      /* [-1,1) */
int32_t fe2o3_synth_normal_f32(uint64_t seed, uint64_t domain, uint64_t n, float sigma, float *out);
int32_t fe2o3_synth_normal_bf16(uint64_t seed, uint64_t domain, uint64_t n, float sigma, uint16_t *out);
int32_t fe2o3_synth_uniform_bf16(uint64_t seed, uint64_t domain, uint64_t n, uint16_t *out);  /* RNE of [-1,1) */
int32_t fe2o3_synth_u32_below(uint64_t seed, uint64_t domain, uint64_t n, uint32_t bound, uint32_t *out);
/* Bernoulli(p) activity as u32 flags {0, flag_value} and as packed u64 words
 * (bit i%64 of word i/64); either output may be NULL. */
int32_t fe2o3_synth_bernoulli(uint64_t seed, uint64_t domain, uint64_t n, double p, uint32_t flag_value,
                              uint32_t *flags, uint64_t *packed);
/* The reference's own alphabet generator (inputs.rs:61-88). */
int32_t fe2o3_synth_gemm_inputs_v1(uint32_t m, uint32_t n, uint32_t k, uint64_t seed, uint16_t *a_bits,
                                   uint16_t *b_bits);
/* crates/fe2o3-device/src/half.rs:182-190 */
uint16_t fe2o3_bf16_from_f32(float value);

/* ---- allocation-free masked sum ------------------------------------------ */
/* No counterpart in the reference.  The same masked u32 wrapping sum as
 * fe2o3_masked_reduce_u32_prepare + launch, for hosts that must not touch the
 * device allocator while they run: processes whose device memory is already
 * owned in full by another runtime's pool, or callers in a section that cannot
 * take the device-wide synchronisation an allocation may imply.  It needs no
 * fe2o3_ctx and calls no cudaMalloc, cudaFree or allocating library routine:
 * its scratch (per-block partial sums and an arrival counter) is a fixed
 * 4352-byte device array that every GPU loading the library holds until the
 * process exits.
 *   values, active : device pointers to n u32 each (flag 0 = inactive)
 *   output         : device pointer to one u32
 *   cuda_stream    : a cudaStream_t (NULL = default stream); the launch is
 *                    asynchronous on it, on the calling thread's current device
 * Limits and rules:
 *   - n <= FE2O3_NOALLOC_MAX_ELEMENTS, larger inputs are rejected with
 *     FE2O3_ERR_UNSUPPORTED_SHAPE (use the prepared entry point instead);
 *   - the first call on each device looks up the scratch array's device address
 *     (one-time set-up); make that first call before any stream capture begins;
 *   - all calls on a device share the one scratch array: two calls whose kernels
 *     can overlap on the GPU (different streams, or different threads) race and
 *     give wrong sums; issue them on one stream or order them with events. */
#define FE2O3_NOALLOC_MAX_ELEMENTS (1ull << 31)
int32_t fe2o3_masked_reduce_u32_noalloc(const uint32_t *values, const uint32_t *active, uint64_t n,
                                        uint32_t *output, void *cuda_stream);

/* Number of kernels this library has launched in the calling process. */
uint64_t fe2o3_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* FE2O3_B200_H */
