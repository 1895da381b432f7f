// Plan object shared by the tensor-core GEMM source and the ABI layer.
#pragma once
#include "common.cuh"

enum GemmEpilogue : uint32_t { EPI_STORE = 0, EPI_ALPHA_BETA = 1, EPI_GELU_BF16 = 2, EPI_SCATTER_PEER = 3, EPI_COMBINE_ADD = 4 };

// Expert-parallel extensions of the grouped GEMM (all zero otherwise).  The rows of A are this rank's
// receive buffer: `experts` contiguous segments (one per local expert), each made of `world` runs, one
// per source rank; pair_offsets[le * world + s] is the first row of (local expert le, source s).
struct GemmEp {
    const uint32_t *pair_offsets;   // [experts * world + 1]; null = not expert-parallel
    uint32_t world, rank;
    const uint32_t *epoch_counter;  // pass number - 1 on the device, or null to use `epoch`
    uint32_t epoch;
    uint32_t spin_limit;            // polls before a flag wait gives up
    // input side (first FFN GEMM): the producer waits for "rows complete" of a source right before the
    // first tile that holds rows of that source; tiles are taken m-tile major starting at this rank's own rows
    const uint32_t *rows_flags;     // this rank's flags, one per source; null = rows are already complete
    const uint32_t *table_flag;     // "pair_offsets written" flag of the dispatch kernel this GEMM may run beside
    // output side (EPI_SCATTER_PEER, second FFN GEMM): row r goes to ret[row_meta[r].y] + row_meta[r].x * N
    const uint2 *row_meta;          // (route id, home rank) per row of A / C
    const uint64_t *peer_ret;       // [world] base address of every rank's return buffer
    uint32_t ret_rows;              // rows of a return buffer
    const uint64_t *peer_flags;     // [world] base address of every rank's flag block
    uint32_t *done_counter;         // this rank's arrival counter of the kernel's CTAs
    uint32_t *trace_flags;          // this rank's flag block (diagnostic time stamps, FE2O3_EP_TRACE builds only)
    // Row-tile hand-over between the two GEMMs of the expert FFN, so that the second can start on the SMs the
    // first one leaves idle in its last round: one counter per 128-row tile of the hidden activations.
    //   mode 1 (producer, first GEMM): every epilogue warp adds one when its part of a tile is in memory;
    //   mode 2 (consumer, second GEMM): the TMA producer waits until a row tile's counter has reached
    //   progress_target (tiles across d_ff x epilogue warps) before its first load of those rows, takes the
    //   tiles in the first GEMM's order, and the last CTA of the grid clears the counters for the next pass.
    uint32_t *progress;
    uint32_t progress_mode, progress_target, progress_len;
};

struct GemmParams {
    void *c;                 // f32 (EPI_STORE / EPI_ALPHA_BETA) or bf16 bits (EPI_GELU_BF16)
    uint32_t M, N, K;
    uint32_t ldc;
    float alpha, beta;
    uint32_t epilogue;
    // grouped mode: rows of A/C are partitioned by expert_offsets[0..experts];
    // B has one [K][N] matrix per expert (third TMA coordinate).
    const uint32_t *expert_offsets;
    uint32_t experts;        // 0 = plain GEMM; otherwise the number of row groups
    uint32_t expert_mod;     // group g reads B matrix (g % expert_mod); 0 = identity
    uint32_t bulk_store;     // C is addressable by the copy engine (tensor map tmC is valid)
    uint32_t *status;
    GemmEp ep;
    // Gathered A (first GEMM of the single-GPU expert FFN): row r of A is row (gather_perm[r] >> 1) of
    // gather_src ([gather_tokens][K] bf16), or zero when gather_perm[r] names no route; the block is then
    // launched with four loader warps more, which fetch the rows straight into the swizzled A stage.
    const uint32_t *gather_perm;
    const void *gather_src;
    uint32_t gather_tokens;
    // EPI_COMBINE_ADD (second GEMM of the single-GPU expert FFN with the combine folded in): row r is the expert
    // output of route combine_perm[r]; it is multiplied by that route's weight and added to row (route >> 1) of
    // c ([combine_tokens][N] f32, zero before the launch).  A token has at most two routes and the sum starts
    // from +0, so the result does not depend on which of the two arrives first.
    const uint32_t *combine_perm;
    const float *combine_weights;
    uint32_t combine_tokens;
    // A buffer this launch clears before anything else (zero_vecs 16-byte pieces): the epilogue warps, which
    // have nothing to do while the first tile is being multiplied, write the zeros.  The first GEMM of the fused
    // expert FFN clears the output that the second one accumulates into.
    uint4 *zero_ptr;
    uint64_t zero_vecs;
};

struct GemmTcPlan {
    CUtensorMap tmA, tmB, tmC;
    GemmParams p;
    uint32_t bn;
    uint32_t grid;
    uint32_t smem;
    uint32_t overlap_previous;   // launch with programmatic stream serialization: 1 = may run beside the (small) blocks of the
                                 // kernel before it on the same SMs, 2 = takes over SMs as blocks of the kernel before it exit
};

int32_t fe2o3_make_tmap_bf16(CUtensorMap *out, uint64_t base, uint32_t rank, const uint64_t *dims,
                             const uint64_t *strides_bytes, const uint32_t *box);
int32_t fe2o3_make_tmap_f32(CUtensorMap *out, uint64_t base, uint32_t rank, const uint64_t *dims,
                            const uint64_t *strides_bytes, const uint32_t *box);
bool gemm_tc_supported(uint64_t a, uint64_t b, uint32_t lda, uint32_t ldb, uint32_t K);
int32_t gemm_tc_plan(fe2o3_ctx *ctx, GemmTcPlan *plan, uint64_t a, uint64_t b, uint64_t c, uint32_t M, uint32_t N,
                     uint32_t K, uint32_t lda, uint32_t ldb, uint32_t ldc, float alpha, float beta, uint32_t epilogue,
                     const uint32_t *expert_offsets, uint32_t experts, uint32_t expert_mod = 0, uint32_t b_matrices = 0,
                     const GemmEp *ep = nullptr, uint32_t expected_rows = 0);
int32_t gemm_tc_launch(const GemmTcPlan *plan, cudaStream_t s);
int32_t gemm_tc_init_device();
bool gemm_tc_set_gather(GemmTcPlan *plan, const uint32_t *perm, const void *src, uint32_t tokens);
void gemm_tc_set_combine(GemmTcPlan *plan, const uint32_t *perm, const float *weights, uint32_t tokens);
void gemm_tc_geometry(const GemmTcPlan *plan, fe2o3_geometry *geo);
