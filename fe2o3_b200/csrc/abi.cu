// The C ABI: context / stream / buffer / event objects, the checked prepare +
// launch surface, the runtime adapter and the bounded wait.  Mirrors
// fe2o3-core (crates/fe2o3-core/src/{context,stream,memory,event}.rs), the
// generated host adapters (crates/fe2o3-host/src/generated_*.rs) and the
// executable lifecycle adapter (crates/fe2o3-host/src/hsa_executable_lifecycle.rs).
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <dlfcn.h>

#include <atomic>
#include <chrono>
#include <mutex>
#include <new>
#include <thread>

#include "gemm_tc.h"

// ---- launchers implemented by the kernel sources -----------------------------
typedef int32_t (*LaunchFn)(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_masked_reduce_u32(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_masked_reduce_u32_packed(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_device_scan_u32(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_device_scan_f32(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_wave_lds_v1(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_wave64_collectives_v1(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_wave64_collectives_segmented(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_lds_reduce_i32(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_scoped_atomic_add(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_row_softmax(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_moe_gate(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_moe_top2(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_moe_route_weights(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_moe_combine(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_moe_ep_exchange(fe2o3_ctx *, cudaStream_t, const void *, fe2o3_geometry *, bool);
int32_t launch_moe_compact(cudaStream_t, uint64_t x, uint64_t perm, uint64_t compact_x, uint32_t rows,
                           uint32_t d_model, uint32_t tokens);
int32_t launch_gemm_exact(cudaStream_t, uint32_t dtype, bool epilogue, uint64_t a, uint64_t b, uint64_t c, uint32_t M,
                          uint32_t N, uint32_t K, uint32_t lda, uint32_t ldb, uint32_t ldc, float alpha, float beta,
                          fe2o3_geometry *, bool);
int32_t launch_attention_simt(fe2o3_ctx *, cudaStream_t, const fe2o3_flash_attention_v1_args *, fe2o3_geometry *, bool);

bool gemm_split_supported(uint64_t a, uint64_t b, uint32_t N, uint32_t K);
int32_t gemm_split_launch(cudaStream_t s, const float *a, const float *b, uint16_t *a3, uint16_t *b3, uint32_t M, uint32_t N,
                          uint32_t K);

struct AttnTcPlan;
bool attention_tc_supported(const fe2o3_flash_attention_v1_args *);
int32_t attention_tc_plan(fe2o3_ctx *, const fe2o3_flash_attention_v1_args *, AttnTcPlan **);
int32_t attention_tc_launch(const AttnTcPlan *, cudaStream_t);
void attention_tc_geometry(const AttnTcPlan *, fe2o3_geometry *);
void attention_tc_free(AttnTcPlan *);
int32_t attention_tc_init_device();
int32_t device_scan_init_device();

// ---- error bookkeeping ---------------------------------------------------------
static thread_local char g_error[512] = "";
static std::atomic<uint64_t> g_launches{0};

void fe2o3_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}
void fe2o3_count_launch(uint32_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int32_t fe2o3_cuda_status(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return FE2O3_OK;
    fe2o3_set_error("%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) return FE2O3_ERR_NO_DEVICE;
    return (int32_t)e;
}

struct fe2o3_buf {
    fe2o3_ctx *ctx;
    void *ptr;
    uint64_t elements;
    uint32_t element_bytes;
    bool quarantined;
    uint32_t owners;   // submitted operations that own the buffer
};
struct fe2o3_event {
    fe2o3_ctx *ctx;
    cudaEvent_t e;
};

enum OpId : uint32_t {
    OP_SCALAR_GEMM, OP_TILED_GEMM, OP_TILED_GEMM_GENERAL, OP_FLASH_ATTENTION, OP_ROW_SOFTMAX, OP_MOE_TOP2,
    OP_MOE_GATE, OP_MOE_ROUTE_WEIGHTS, OP_MOE_EXPERT_FFN, OP_MOE_COMBINE, OP_MASKED_REDUCE, OP_MASKED_REDUCE_PACKED,
    OP_WAVE_LDS, OP_WAVE64_COLLECTIVES, OP_WAVE64_SEGMENTED, OP_LDS_REDUCE_I32, OP_SCOPED_ATOMIC_ADD,
    OP_MOE_COMPACT, OP_MOE_GROUPED_FFN, OP_MOE_EP_EXCHANGE, OP_DEVICE_SCAN_U32, OP_DEVICE_SCAN_F32, OP_MOE_EP_FFN,
    OP_MOE_FFN_COMBINE, OP_COUNT
};

struct OpInfo {
    const char *symbol;  // the reference kernel function name this entry replaces
    uint64_t kernarg_bytes;
    LaunchFn simple;     // non-null for ops with a single uniform launcher
};

static const OpInfo kOps[OP_COUNT] = {
    {"scalar_gemm_v1", sizeof(fe2o3_scalar_gemm_v1_args), nullptr},
    {"tiled_gemm_lds_slice1", sizeof(fe2o3_tiled_gemm_v1_args), nullptr},
    {"tiled_gemm_general_v1", sizeof(fe2o3_tiled_gemm_general_v1_args), nullptr},
    {"flash_attention_v1", sizeof(fe2o3_flash_attention_v1_args), nullptr},
    {"row_softmax_v1", sizeof(fe2o3_row_softmax_v1_args), launch_row_softmax},
    {"moe_top2_v1", sizeof(fe2o3_moe_top2_v1_args), launch_moe_top2},
    {"moe_gate_v1", sizeof(fe2o3_moe_gate_v1_args), launch_moe_gate},
    {"moe_route_weights_v1", sizeof(fe2o3_moe_route_weights_v1_args), launch_moe_route_weights},
    {"moe_expert_ffn_v1", sizeof(fe2o3_moe_expert_ffn_v1_args), nullptr},
    {"moe_expert_combine_v1", sizeof(fe2o3_moe_expert_combine_v1_args), launch_moe_combine},
    {"masked_reduce_sum_u32", sizeof(fe2o3_masked_reduce_u32_args), launch_masked_reduce_u32},
    {"masked_reduce_sum_u32_packed", sizeof(fe2o3_masked_reduce_u32_packed_args), launch_masked_reduce_u32_packed},
    {"gfx942_wave_lds_v1_hw", sizeof(fe2o3_wave_lds_v1_args), launch_wave_lds_v1},
    {"wave64_collectives_v1", sizeof(fe2o3_wave64_collectives_v1_args), launch_wave64_collectives_v1},
    {"wave64_collectives_segmented", sizeof(fe2o3_wave64_collectives_segmented_args), launch_wave64_collectives_segmented},
    {"lds_publish_read_reduce_i32_v1", sizeof(fe2o3_lds_publish_read_reduce_i32_v1_args), launch_lds_reduce_i32},
    {"scoped_atomic_add_u32_v1", sizeof(fe2o3_scoped_atomic_add_u32_v1_args), launch_scoped_atomic_add},
    {"moe_compact_v1", sizeof(fe2o3_moe_compact_v1_args), nullptr},
    {"moe_grouped_ffn_v1", sizeof(fe2o3_moe_grouped_ffn_v1_args), nullptr},
    {"moe_ep_exchange_v1", sizeof(fe2o3_moe_ep_exchange_v1_args), launch_moe_ep_exchange},
    {"device_scan_sum_u32", sizeof(fe2o3_device_scan_u32_args), launch_device_scan_u32},
    {"device_scan_sum_f32", sizeof(fe2o3_device_scan_f32_args), launch_device_scan_f32},
    {"moe_ep_ffn_v1", sizeof(fe2o3_moe_ep_ffn_v1_args), nullptr},
    {"moe_expert_ffn_combine_v1", sizeof(fe2o3_moe_expert_ffn_combine_v1_args), nullptr},
};

struct fe2o3_prepared {
    fe2o3_ctx *ctx;
    uint32_t op;
    alignas(8) uint8_t kernarg[320];
    uint32_t schedule;   // GEMM: resolved schedule
    GemmTcPlan gemm[2];  // tcgen05 plans (FFN uses both)
    AttnTcPlan *attn;
    void *scratch[2];    // device workspace owned by the prepared object (split bf16 operands of the f32 GEMM)
    fe2o3_geometry geo;
};

struct fe2o3_executable {
    fe2o3_ctx *ctx;
    uint8_t digest[32];   // of the image the caller presented (and this library is)
};

// ---- kernel registry (symbol -> device function), filled by file-scope objects of the kernel sources ----
namespace {
struct KernelEntry {
    const char *symbol;
    const void *entry;
};
constexpr int kMaxKernelEntries = 64;
KernelEntry *kernel_table(int **count) {
    static KernelEntry table[kMaxKernelEntries];   // function-local: usable from other sources' static initialisers
    static int n = 0;
    *count = &n;
    return table;
}
}  // namespace
void fe2o3_register_kernel(const char *symbol, const void *entry) {
    int *n;
    KernelEntry *t = kernel_table(&n);
    if (*n < kMaxKernelEntries) t[(*n)++] = KernelEntry{symbol, entry};
}

// ---- SHA-256 (FIPS 180-4), for the image digest of load_executable ----------------------------
namespace {
struct Sha256 {
    uint32_t h[8];
    uint8_t block[64];
    uint64_t total;
    uint32_t fill;
    Sha256() : total(0), fill(0) {
        static const uint32_t init[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au,
                                         0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
        memcpy(h, init, sizeof h);
    }
    static uint32_t rotr(uint32_t v, int r) { return (v >> r) | (v << (32 - r)); }
    void compress(const uint8_t *p) {
        static const uint32_t K[64] = {
            0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u,
            0xd807aa98u, 0x12835b01u, 0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u,
            0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu, 0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau,
            0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u,
            0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u,
            0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u,
            0x19a4c116u, 0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u,
            0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};
        uint32_t w[64];
        for (int i = 0; i < 16; ++i)
            w[i] = ((uint32_t)p[4 * i] << 24) | ((uint32_t)p[4 * i + 1] << 16) | ((uint32_t)p[4 * i + 2] << 8) | p[4 * i + 3];
        for (int i = 16; i < 64; ++i) {
            const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; ++i) {
            const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + K[i] + w[i];
            const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    void update(const uint8_t *p, uint64_t n) {
        total += n;
        while (n) {
            const uint32_t take = (uint32_t)((64 - fill) < n ? (64 - fill) : n);
            memcpy(block + fill, p, take);
            fill += take; p += take; n -= take;
            if (fill == 64) { compress(block); fill = 0; }
        }
    }
    void finish(uint8_t out[32]) {
        const uint64_t bits = total * 8;
        const uint8_t one = 0x80, zero = 0;
        update(&one, 1);
        while (fill != 56) update(&zero, 1);
        uint8_t len[8];
        for (int i = 0; i < 8; ++i) len[i] = (uint8_t)(bits >> (56 - 8 * i));
        update(len, 8);
        for (int i = 0; i < 8; ++i)
            for (int j = 0; j < 4; ++j) out[4 * i + j] = (uint8_t)(h[i] >> (24 - 8 * j));
    }
};

// SHA-256 of this shared library's file, as found on disk at first use.  false when it cannot be read.
bool own_image_digest(uint8_t out[32]) {
    static std::once_flag once;
    static bool ok = false;
    static uint8_t digest[32];
    std::call_once(once, [] {
        Dl_info info;
        if (!dladdr(reinterpret_cast<const void *>(&fe2o3_register_kernel), &info) || !info.dli_fname) return;
        FILE *f = fopen(info.dli_fname, "rb");
        if (!f) return;
        Sha256 sha;
        static uint8_t buf[1 << 16];
        size_t n;
        while ((n = fread(buf, 1, sizeof buf, f)) > 0) sha.update(buf, n);
        fclose(f);
        sha.finish(digest);
        ok = true;
    });
    if (ok) memcpy(out, digest, 32);
    return ok;
}
}  // namespace

// ---- region checks ---------------------------------------------------------------
namespace {

struct Region {
    const char *role;
    fe2o3_slice s;
    uint64_t expected;
    uint32_t elem_bytes;
    bool output;
};

bool mul_overflow(uint64_t a, uint64_t b, uint64_t *r) { return __builtin_mul_overflow(a, b, r); }

int32_t check_regions(const Region *r, int n) {
    uint64_t lo[20], hi[20];
    for (int i = 0; i < n; ++i) {
        if (r[i].s.len != r[i].expected) {
            fe2o3_set_error("Length{role=%s, expected=%llu, actual=%llu}", r[i].role,
                            (unsigned long long)r[i].expected, (unsigned long long)r[i].s.len);
            return FE2O3_ERR_LENGTH;
        }
        uint64_t bytes;
        if (mul_overflow(r[i].s.len, r[i].elem_bytes, &bytes) || r[i].s.ptr + bytes < r[i].s.ptr) {
            fe2o3_set_error("RegionOverflow{role=%s}", r[i].role);
            return FE2O3_ERR_INVALID_REGION;
        }
        if (r[i].s.len != 0 && r[i].s.ptr == 0) {
            fe2o3_set_error("NullAddress{role=%s}", r[i].role);
            return FE2O3_ERR_NULL_ADDRESS;
        }
        if (r[i].s.ptr % r[i].elem_bytes != 0) {
            fe2o3_set_error("Alignment{role=%s}", r[i].role);
            return FE2O3_ERR_ALIGNMENT;
        }
        lo[i] = r[i].s.ptr;
        hi[i] = r[i].s.ptr + bytes;
    }
    for (int o = 0; o < n; ++o) {
        if (!r[o].output || lo[o] == hi[o]) continue;
        for (int i = 0; i < n; ++i) {
            if (i == o || lo[i] == hi[i]) continue;
            if (r[i].output && i < o) continue;  // output pairs are checked once
            if (lo[i] < hi[o] && lo[o] < hi[i]) {
                fe2o3_set_error("OutputAliasesInput{output=%s, input=%s}", r[o].role, r[i].role);
                return FE2O3_ERR_OUTPUT_ALIASES_INPUT;
            }
        }
    }
    return FE2O3_OK;
}

// storage extent of a strided matrix: (rows-1)*ld + cols, or 0 when empty
bool extent(uint64_t rows, uint64_t cols, uint64_t ld, uint64_t *out) {
    if (rows == 0 || cols == 0) { *out = 0; return true; }
    uint64_t t;
    if (mul_overflow(rows - 1, ld, &t) || t + cols < t) return false;
    *out = t + cols;
    return true;
}

int32_t unsupported(const char *why) {
    fe2o3_set_error("UnsupportedShape: %s", why);
    return FE2O3_ERR_UNSUPPORTED_SHAPE;
}

int32_t check_ctx_device(fe2o3_ctx *ctx, const Region *r, int n) {
    for (int i = 0; i < n; ++i) {
        if (r[i].s.len == 0) continue;
        cudaPointerAttributes attr;
        cudaError_t e = cudaPointerGetAttributes(&attr, reinterpret_cast<const void *>(r[i].s.ptr));
        if (e != cudaSuccess) { cudaGetLastError(); continue; }
        if ((attr.type == cudaMemoryTypeDevice) && attr.device != ctx->device) {
            fe2o3_set_error("WrongContext{role=%s, device=%d, context_device=%d}", r[i].role, attr.device, ctx->device);
            return FE2O3_ERR_DEVICE_MISMATCH;
        }
        if (attr.type == cudaMemoryTypeUnregistered || attr.type == cudaMemoryTypeHost) {
            fe2o3_set_error("WrongContext{role=%s}: not device memory", r[i].role);
            return FE2O3_ERR_DEVICE_MISMATCH;
        }
    }
    return FE2O3_OK;
}

#define RGN(role_, slice_, expected_, bytes_, out_) Region{role_, slice_, (uint64_t)(expected_), bytes_, out_}

// Per-op region tables.  Returns the number of regions, fills `r`.
int regions_for(uint32_t op, const void *args, Region *r, int32_t *status) {
    *status = FE2O3_OK;
    switch (op) {
        case OP_SCALAR_GEMM:
        case OP_TILED_GEMM: {
            const fe2o3_scalar_gemm_v1_args *a = static_cast<const fe2o3_scalar_gemm_v1_args *>(args);
            const uint32_t eb = op == OP_SCALAR_GEMM ? 4 : 2;
            if (op == OP_TILED_GEMM && ((a->m % 16) || (a->n % 16) || (a->k % 16))) {
                *status = unsupported("tiled_gemm_v1 admits M, N, K multiples of 16 (tails rejected)");
                return 0;
            }
            // empty output: no dispatch, operand storage is not inspected (oracle.rs:296-298)
            if ((uint64_t)a->m * a->n == 0) return 0;
            r[0] = RGN("A", a->a, (uint64_t)a->m * a->k, eb, false);
            r[1] = RGN("B", a->b, (uint64_t)a->k * a->n, eb, false);
            r[2] = RGN("C", a->c, (uint64_t)a->m * a->n, 4, true);
            return 3;
        }
        case OP_TILED_GEMM_GENERAL: {
            const fe2o3_tiled_gemm_general_v1_args *a = static_cast<const fe2o3_tiled_gemm_general_v1_args *>(args);
            // an operand without rows or columns has no stride rule (general_plan.rs:406-425 checked_extent)
            const bool a_bad = a->m && a->k && a->lda < a->k, b_bad = a->k && a->n && a->ldb < a->n,
                       c_bad = a->m && a->n && a->ldc < a->n;
            if (a_bad || b_bad || c_bad) {
                *status = unsupported("StrideTooSmall: lda >= k, ldb >= n, ldc >= n required for nonempty operands");
                return 0;
            }
            if ((uint64_t)a->m * a->n == 0) return 0;
            uint64_t ea, ebx, ec;
            if (!extent(a->m, a->k, a->lda, &ea) || !extent(a->k, a->n, a->ldb, &ebx) ||
                !extent(a->m, a->n, a->ldc, &ec)) {
                fe2o3_set_error("ExtentOverflow");
                *status = FE2O3_ERR_SIZE_OVERFLOW;
                return 0;
            }
            r[0] = RGN("A", a->a, ea, 2, false);
            r[1] = RGN("B", a->b, ebx, 2, false);
            r[2] = RGN("C", a->c, ec, 4, true);
            return 3;
        }
        case OP_FLASH_ATTENTION: {
            const fe2o3_flash_attention_v1_args *a = static_cast<const fe2o3_flash_attention_v1_args *>(args);
            if (a->input_dtype > FE2O3_DTYPE_BF16 || a->dim == 0 || a->dim > 256 || a->seq == 0 ||
                !(a->scale == a->scale)) {
                *status = unsupported("flash_attention_v1 needs f32/bf16 inputs, 1 <= dim <= 256, seq >= 1");
                return 0;
            }
            const uint64_t n = (uint64_t)a->batch * a->heads * a->seq * a->dim;
            const uint32_t eb = a->input_dtype == FE2O3_DTYPE_F32 ? 4 : 2;
            r[0] = RGN("Query", a->q, n, eb, false);
            r[1] = RGN("Key", a->k, n, eb, false);
            r[2] = RGN("Value", a->v, n, eb, false);
            r[3] = RGN("Output", a->output, n, 4, true);
            return 4;
        }
        case OP_ROW_SOFTMAX: {
            const fe2o3_row_softmax_v1_args *a = static_cast<const fe2o3_row_softmax_v1_args *>(args);
            if (a->cols == 0) { *status = unsupported("EmptyRow"); return 0; }
            if (a->cols > 4096) { *status = unsupported("RowTooLarge: at most 4096 columns"); return 0; }
            const uint64_t n = (uint64_t)a->rows * a->cols;
            r[0] = RGN("Input", a->input, n, 4, false);
            r[1] = RGN("Output", a->output, n, 4, true);
            if (a->mask.ptr == 0 && a->mask.len == 0) return 2;
            r[2] = RGN("Mask", a->mask, n, 1, false);
            return 3;
        }
        case OP_MOE_TOP2: {
            const fe2o3_moe_top2_v1_args *a = static_cast<const fe2o3_moe_top2_v1_args *>(args);
            if (a->experts < 2 || a->experts > 32) { *status = unsupported("2 <= experts <= 32"); return 0; }
            if (a->tokens > 0x7fffffffu) { *status = unsupported("route ids must fit u32"); return 0; }
            const uint64_t R = 2ull * a->tokens;
            r[0] = RGN("Logits", a->logits, (uint64_t)a->tokens * a->experts, 4, false);
            r[1] = RGN("Top2Experts", a->top2_experts, R, 4, true);
            r[2] = RGN("RequestedCounts", a->requested_counts, a->experts, 4, true);
            r[3] = RGN("AdmittedCounts", a->admitted_counts, a->experts, 4, true);
            r[4] = RGN("ExpertOffsets", a->expert_offsets, a->experts + 1, 4, true);
            r[5] = RGN("RouteSlots", a->route_slots, R, 4, true);
            r[6] = RGN("Permutation", a->permutation, R, 4, true);
            r[7] = RGN("Inverse", a->inverse, R, 4, true);
            return 8;
        }
        case OP_MOE_GATE: {
            const fe2o3_moe_gate_v1_args *a = static_cast<const fe2o3_moe_gate_v1_args *>(args);
            if (a->experts < 1 || a->experts > 256) { *status = unsupported("1 <= experts <= 256"); return 0; }
            r[0] = RGN("X", a->x, (uint64_t)a->tokens * a->d_model, 2, false);
            r[1] = RGN("Wg", a->wg, (uint64_t)a->d_model * a->experts, 2, false);
            r[2] = RGN("Logits", a->logits, (uint64_t)a->tokens * a->experts, 4, true);
            return 3;
        }
        case OP_MOE_ROUTE_WEIGHTS: {
            const fe2o3_moe_route_weights_v1_args *a = static_cast<const fe2o3_moe_route_weights_v1_args *>(args);
            r[0] = RGN("Logits", a->logits, (uint64_t)a->tokens * a->experts, 4, false);
            r[1] = RGN("Top2Experts", a->top2_experts, 2ull * a->tokens, 4, false);
            r[2] = RGN("RouteWeights", a->route_weights, 2ull * a->tokens, 4, true);
            return 3;
        }
        case OP_MOE_EXPERT_FFN: {
            const fe2o3_moe_expert_ffn_v1_args *a = static_cast<const fe2o3_moe_expert_ffn_v1_args *>(args);
            if (a->d_model == 0 || a->d_ff == 0 || (a->d_model % 8) || (a->d_ff % 8) || a->experts < 1 ||
                a->experts > 32) {
                *status = unsupported("d_model and d_ff must be positive multiples of 8; 1 <= experts <= 32");
                return 0;
            }
            if (a->compact_output.len % a->d_model) { *status = unsupported("compact_output is not whole rows"); return 0; }
            const uint64_t rows = a->compact_output.len / a->d_model;
            r[0] = RGN("X", a->x, (uint64_t)a->tokens * a->d_model, 2, false);
            r[1] = RGN("W1", a->w1, (uint64_t)a->experts * a->d_model * a->d_ff, 2, false);
            r[2] = RGN("W2", a->w2, (uint64_t)a->experts * a->d_ff * a->d_model, 2, false);
            r[3] = RGN("Permutation", a->permutation, rows, 4, false);
            r[4] = RGN("ExpertOffsets", a->expert_offsets, a->experts + 1, 4, false);
            r[5] = RGN("CompactX", a->compact_x, rows * a->d_model, 2, true);
            r[6] = RGN("Hidden", a->hidden, rows * a->d_ff, 2, true);
            r[7] = RGN("CompactOutput", a->compact_output, rows * a->d_model, 4, true);
            return 8;
        }
        case OP_MOE_FFN_COMBINE: {
            const fe2o3_moe_expert_ffn_combine_v1_args *a = static_cast<const fe2o3_moe_expert_ffn_combine_v1_args *>(args);
            if (a->d_model == 0 || a->d_ff == 0 || (a->d_model % 64) || (a->d_ff % 8) || a->experts < 1 || a->experts > 32) {
                *status = unsupported("d_model a positive multiple of 64, d_ff of 8; 1 <= experts <= 32");
                return 0;
            }
            const uint64_t rows = a->permutation.len;
            r[0] = RGN("X", a->x, (uint64_t)a->tokens * a->d_model, 2, false);
            r[1] = RGN("W1", a->w1, (uint64_t)a->experts * a->d_model * a->d_ff, 2, false);
            r[2] = RGN("W2", a->w2, (uint64_t)a->experts * a->d_ff * a->d_model, 2, false);
            r[3] = RGN("Permutation", a->permutation, rows, 4, false);
            r[4] = RGN("ExpertOffsets", a->expert_offsets, a->experts + 1, 4, false);
            r[5] = RGN("RouteWeights", a->route_weights, 2ull * a->tokens, 4, false);
            r[6] = RGN("Hidden", a->hidden, rows * a->d_ff, 2, true);
            r[7] = RGN("CombinedOutput", a->combined_output, (uint64_t)a->tokens * a->d_model, 4, true);
            return 8;
        }
        case OP_MOE_COMPACT: {
            const fe2o3_moe_compact_v1_args *a = static_cast<const fe2o3_moe_compact_v1_args *>(args);
            if (a->d_model == 0 || (a->d_model % 8)) { *status = unsupported("d_model must be a positive multiple of 8"); return 0; }
            r[0] = RGN("X", a->x, (uint64_t)a->tokens * a->d_model, 2, false);
            r[1] = RGN("Permutation", a->permutation, a->permutation.len, 4, false);
            r[2] = RGN("CompactX", a->compact_x, a->permutation.len * a->d_model, 2, true);
            return 3;
        }
        case OP_MOE_GROUPED_FFN: {
            const fe2o3_moe_grouped_ffn_v1_args *a = static_cast<const fe2o3_moe_grouped_ffn_v1_args *>(args);
            if (a->d_model == 0 || a->d_ff == 0 || (a->d_model % 8) || (a->d_ff % 8) || a->groups < 1 || a->groups > 32 ||
                a->experts_cycle < 1 || a->experts_cycle > a->groups) {
                *status = unsupported("d_model, d_ff positive multiples of 8; 1 <= experts_cycle <= groups <= 32");
                return 0;
            }
            if (a->compact_output.len % a->d_model) { *status = unsupported("compact_output is not whole rows"); return 0; }
            const uint64_t rows = a->compact_output.len / a->d_model;
            r[0] = RGN("CompactX", a->compact_x, rows * a->d_model, 2, false);
            r[1] = RGN("W1", a->w1, (uint64_t)a->experts_cycle * a->d_model * a->d_ff, 2, false);
            r[2] = RGN("W2", a->w2, (uint64_t)a->experts_cycle * a->d_ff * a->d_model, 2, false);
            r[3] = RGN("GroupOffsets", a->group_offsets, a->groups + 1, 4, false);
            r[4] = RGN("Hidden", a->hidden, rows * a->d_ff, 2, true);
            r[5] = RGN("CompactOutput", a->compact_output, rows * a->d_model, 4, true);
            return 6;
        }
        case OP_MOE_EP_EXCHANGE: {
            const fe2o3_moe_ep_exchange_v1_args *a = static_cast<const fe2o3_moe_ep_exchange_v1_args *>(args);
            if (a->world < 1 || a->world > 32 || a->experts < 2 || a->experts > 32 || a->experts % a->world ||
                a->d_model == 0 || (a->d_model % 8) || a->rank >= a->world || a->phase > FE2O3_MOE_EP_COMBINE ||
                a->tokens > 0x3fffffffu) {
                *status = unsupported("1 <= world <= 32 dividing experts (2..32), d_model a positive multiple of 8, rank < world");
                return 0;
            }
            const uint64_t R = 2ull * a->tokens;
            r[0] = RGN("X", a->x, (uint64_t)a->tokens * a->d_model, 2, false);
            r[1] = RGN("Top2Experts", a->top2_experts, R, 4, false);
            r[2] = RGN("Permutation", a->permutation, R, 4, false);
            r[3] = RGN("Inverse", a->inverse, R, 4, false);
            r[4] = RGN("ExpertOffsets", a->expert_offsets, a->experts + 1, 4, false);
            r[5] = RGN("AdmittedCounts", a->admitted_counts, a->experts, 4, false);
            r[6] = RGN("RouteWeights", a->route_weights, R, 4, false);
            r[7] = RGN("PeerRecvX", a->peer_recv_x, a->world, 8, false);
            r[8] = RGN("PeerRecvMeta", a->peer_recv_meta, a->world, 8, false);
            r[9] = RGN("PeerRet", a->peer_ret, a->world, 8, false);
            r[10] = RGN("PeerCounts", a->peer_counts, a->world, 8, false);
            r[11] = RGN("PeerFlags", a->peer_flags, a->world, 8, false);
            r[12] = RGN("PairOffsets", a->pair_offsets, a->experts + 1, 4, true);
            r[13] = RGN("CombinedOutput", a->combined_output, (uint64_t)a->tokens * a->d_model, 4, true);
            int n = 14;
            if (a->epoch_counter.ptr != 0 || a->epoch_counter.len != 0) r[n++] = RGN("EpochCounter", a->epoch_counter, 1, 4, true);
            if (a->logits.ptr != 0 || a->logits.len != 0) {
                r[n++] = RGN("Logits", a->logits, (uint64_t)a->tokens * a->experts, 4, false);
                r[6].output = a->phase == FE2O3_MOE_EP_DISPATCH;   // the dispatch phase writes the route weights then
            }
            return n;
        }
        case OP_MOE_EP_FFN: {
            const fe2o3_moe_ep_ffn_v1_args *a = static_cast<const fe2o3_moe_ep_ffn_v1_args *>(args);
            if (a->world < 1 || a->world > 32 || a->experts < 2 || a->experts > 32 || a->experts % a->world ||
                a->d_model == 0 || (a->d_model % 8) || a->d_ff == 0 || (a->d_ff % 8) || a->rank >= a->world ||
                a->max_rows == 0 || a->tokens > 0x3fffffffu) {
                *status = unsupported("1 <= world <= 32 dividing experts (2..32), d_model and d_ff positive multiples of 8, rank < world, max_rows > 0");
                return 0;
            }
            const uint64_t per = a->experts / a->world;
            r[0] = RGN("RecvX", a->recv_x, (uint64_t)a->max_rows * a->d_model, 2, false);
            r[1] = RGN("W1", a->w1, per * a->d_model * a->d_ff, 2, false);
            r[2] = RGN("W2", a->w2, per * a->d_ff * a->d_model, 2, false);
            r[3] = RGN("PairOffsets", a->pair_offsets, a->experts + 1, 4, false);
            r[4] = RGN("RecvMeta", a->recv_meta, 2ull * a->max_rows, 4, false);
            r[5] = RGN("PeerRet", a->peer_ret, a->world, 8, false);
            r[6] = RGN("PeerFlags", a->peer_flags, a->world, 8, false);
            r[7] = RGN("Hidden", a->hidden, (uint64_t)a->max_rows * a->d_ff, 2, true);
            r[8] = RGN("Flags", a->flags, FE2O3_EP_FLAG_WORDS((uint64_t)a->world), 4, true);
            int n = 9;
            if (a->epoch_counter.ptr != 0 || a->epoch_counter.len != 0) r[n++] = RGN("EpochCounter", a->epoch_counter, 1, 4, false);
            if (a->progress.ptr != 0 || a->progress.len != 0)
                r[n++] = RGN("Progress", a->progress, 2 * ((uint64_t)a->max_rows / 128 + per + 1), 4, true);
            return n;
        }
        case OP_MOE_COMBINE: {
            const fe2o3_moe_expert_combine_v1_args *a = static_cast<const fe2o3_moe_expert_combine_v1_args *>(args);
            if (a->width == 0 || a->compact_output.len % a->width) {
                *status = unsupported("compact_output is not whole rows");
                return 0;
            }
            r[0] = RGN("CompactOutput", a->compact_output, a->compact_output.len, 4, false);
            r[1] = RGN("Inverse", a->inverse, 2ull * a->tokens, 4, false);
            r[2] = RGN("RouteWeights", a->route_weights, 2ull * a->tokens, 4, false);
            r[3] = RGN("CombinedOutput", a->combined_output, (uint64_t)a->tokens * a->width, 4, true);
            return 4;
        }
        case OP_MASKED_REDUCE: {
            const fe2o3_masked_reduce_u32_args *a = static_cast<const fe2o3_masked_reduce_u32_args *>(args);
            r[0] = RGN("Values", a->values, a->values.len, 4, false);
            r[1] = RGN("Active", a->active, a->values.len, 4, false);
            r[2] = RGN("Output", a->output, 1, 4, true);
            return 3;
        }
        case OP_MASKED_REDUCE_PACKED: {
            const fe2o3_masked_reduce_u32_packed_args *a = static_cast<const fe2o3_masked_reduce_u32_packed_args *>(args);
            r[0] = RGN("Values", a->values, a->values.len, 4, false);
            r[1] = RGN("Mask", a->mask, (a->values.len + 63) / 64, 8, false);
            r[2] = RGN("Output", a->output, 1, 4, true);
            return 3;
        }
        case OP_DEVICE_SCAN_U32:
        case OP_DEVICE_SCAN_F32: {   // same block; elements are 4 bytes in both
            const fe2o3_device_scan_u32_args *a = static_cast<const fe2o3_device_scan_u32_args *>(args);
            if (a->values.len > FE2O3_SCAN_MAX_ELEMENTS || a->exclusive > 1u) {
                *status = unsupported("at most 2^31 elements; exclusive is 0 or 1");
                return 0;
            }
            r[0] = RGN("Values", a->values, a->values.len, 4, false);
            r[1] = RGN("Output", a->output, a->values.len, 4, true);
            return 2;
        }
        case OP_WAVE_LDS: {
            const fe2o3_wave_lds_v1_args *a = static_cast<const fe2o3_wave_lds_v1_args *>(args);
            if (a->values.len % 256) { *status = unsupported("length must be a multiple of the 256-lane workgroup"); return 0; }
            r[0] = RGN("Values", a->values, a->values.len, 4, false);
            r[1] = RGN("Active", a->active, a->values.len, 4, false);
            r[2] = RGN("WaveOut", a->wave_out, a->values.len, 4, true);
            r[3] = RGN("WorkgroupOut", a->workgroup_out, a->values.len, 4, true);
            return 4;
        }
        case OP_WAVE64_COLLECTIVES: {
            const fe2o3_wave64_collectives_v1_args *a = static_cast<const fe2o3_wave64_collectives_v1_args *>(args);
            r[0] = RGN("Input", a->input, 64, 4, false);
            r[1] = RGN("Reduction", a->reduction_output, 64, 4, true);
            r[2] = RGN("Inclusive", a->inclusive_output, 64, 4, true);
            r[3] = RGN("Exclusive", a->exclusive_output, 64, 4, true);
            return 4;
        }
        case OP_WAVE64_SEGMENTED: {
            const fe2o3_wave64_collectives_segmented_args *a = static_cast<const fe2o3_wave64_collectives_segmented_args *>(args);
            const uint64_t n = a->masks.len * 64;
            r[0] = RGN("Input", a->input, n, 4, false);
            r[1] = RGN("Masks", a->masks, a->masks.len, 8, false);
            r[2] = RGN("Reduction", a->reduction_output, n, 4, true);
            r[3] = RGN("Inclusive", a->inclusive_output, n, 4, true);
            r[4] = RGN("Exclusive", a->exclusive_output, n, 4, true);
            return 5;
        }
        case OP_LDS_REDUCE_I32: {
            const fe2o3_lds_publish_read_reduce_i32_v1_args *a = static_cast<const fe2o3_lds_publish_read_reduce_i32_v1_args *>(args);
            r[0] = RGN("Values", a->values, 64, 4, false);
            r[1] = RGN("Output", a->output, 1, 4, true);
            return 2;
        }
        case OP_SCOPED_ATOMIC_ADD: {
            const fe2o3_scoped_atomic_add_u32_v1_args *a = static_cast<const fe2o3_scoped_atomic_add_u32_v1_args *>(args);
            r[0] = RGN("Values", a->values, 64, 4, false);
            r[1] = RGN("Eligible", a->eligible, 64, 4, false);
            r[2] = RGN("Target", (fe2o3_slice{a->target, 1}), 1, 4, true);
            return 3;
        }
    }
    *status = FE2O3_ERR_INVALID_ARGUMENT;
    return 0;
}

int32_t check_op(uint32_t op, const void *args) {
    if (!args) { fe2o3_set_error("null argument block"); return FE2O3_ERR_INVALID_ARGUMENT; }
    Region r[20];
    int32_t st;
    int n = regions_for(op, args, r, &st);
    if (st != FE2O3_OK) return st;
    return check_regions(r, n);
}

int32_t resolve_gemm(fe2o3_prepared *p, uint32_t schedule, uint32_t dtype, uint64_t a, uint64_t b, uint64_t c,
                     uint32_t M, uint32_t N, uint32_t K, uint32_t lda, uint32_t ldb, uint32_t ldc, float alpha,
                     float beta, bool epilogue) {
    if (schedule > FE2O3_GEMM_SCHEDULE_AUTO) { fe2o3_set_error("unknown schedule"); return FE2O3_ERR_INVALID_ARGUMENT; }
    if (dtype == FE2O3_DTYPE_F32) {
        // f32 operands: the exact-order schedule unless the tensor-core one is asked for by name; that one splits
        // each operand into bf16 terms (gemm_split.cu) and is specified by a bound, not bit-exact
        if (schedule != FE2O3_GEMM_SCHEDULE_TCGEN05) {
            p->schedule = FE2O3_GEMM_SCHEDULE_EXACT_ORDER;
            return launch_gemm_exact(nullptr, dtype, epilogue, a, b, c, M, N, K, lda, ldb, ldc, alpha, beta, &p->geo, true);
        }
        if (epilogue || lda != K || ldb != N || !gemm_split_supported(a, b, N, K))
            return unsupported("tcgen05 schedule for f32 operands needs packed A and B, 16-byte aligned, K and N multiples of 8");
        p->schedule = FE2O3_GEMM_SCHEDULE_TCGEN05;
        FE2O3_CUDA(cudaSetDevice(p->ctx->device));
        FE2O3_CUDA(cudaMalloc(&p->scratch[0], (size_t)M * 3 * K * 2));
        FE2O3_CUDA(cudaMalloc(&p->scratch[1], (size_t)3 * K * N * 2));
        int32_t st = gemm_tc_plan(p->ctx, &p->gemm[0], reinterpret_cast<uint64_t>(p->scratch[0]), reinterpret_cast<uint64_t>(p->scratch[1]),
                                  c, M, N, 3 * K, 3 * K, N, ldc, 1.f, 0.f, 0u, nullptr, 0);
        if (st != FE2O3_OK) return st;
        gemm_tc_geometry(&p->gemm[0], &p->geo);
        p->geo.launches = 3;
        return FE2O3_OK;
    }
    const bool tc_ok = dtype == FE2O3_DTYPE_BF16 && gemm_tc_supported(a, b, lda, ldb, K);
    if (schedule == FE2O3_GEMM_SCHEDULE_TCGEN05 && !tc_ok)
        return unsupported("tcgen05 schedule needs bf16 operands, K > 0, 16-byte aligned bases, lda and ldb multiples of 8");
    if (schedule == FE2O3_GEMM_SCHEDULE_AUTO)
        schedule = (tc_ok && (uint64_t)M * N * K >= (1ull << 21)) ? FE2O3_GEMM_SCHEDULE_TCGEN05 : FE2O3_GEMM_SCHEDULE_EXACT_ORDER;
    p->schedule = schedule;
    if (schedule == FE2O3_GEMM_SCHEDULE_TCGEN05) {
        int32_t st = gemm_tc_plan(p->ctx, &p->gemm[0], a, b, c, M, N, K, lda, ldb, ldc, alpha, beta, epilogue ? 1u : 0u,
                                  nullptr, 0);
        if (st != FE2O3_OK) return st;
        gemm_tc_geometry(&p->gemm[0], &p->geo);
        return FE2O3_OK;
    }
    return launch_gemm_exact(nullptr, dtype, epilogue, a, b, c, M, N, K, lda, ldb, ldc, alpha, beta, &p->geo, true);
}

int32_t prepare_common(fe2o3_ctx *ctx, uint32_t op, const void *args, fe2o3_prepared **out) {
    if (!ctx || !out) { fe2o3_set_error("null context or output"); return FE2O3_ERR_INVALID_ARGUMENT; }
    *out = nullptr;
    int32_t st = check_op(op, args);
    if (st != FE2O3_OK) return st;
    Region r[20];
    int n = regions_for(op, args, r, &st);
    st = check_ctx_device(ctx, r, n);
    if (st != FE2O3_OK) return st;
    fe2o3_prepared *p = new (std::nothrow) fe2o3_prepared();
    if (!p) return FE2O3_ERR_SIZE_OVERFLOW;
    p->ctx = ctx;
    p->op = op;
    p->attn = nullptr;
    p->scratch[0] = p->scratch[1] = nullptr;
    p->schedule = 0;
    memset(p->kernarg, 0, sizeof p->kernarg);
    memcpy(p->kernarg, args, kOps[op].kernarg_bytes);
    memset(&p->geo, 0, sizeof p->geo);
    *out = p;
    return FE2O3_OK;
}

int32_t finish_simple(fe2o3_prepared *p) {
    return kOps[p->op].simple(p->ctx, nullptr, p->kernarg, &p->geo, true);
}

int32_t launch_prepared(fe2o3_prepared *p, cudaStream_t s) {
    fe2o3_ctx *ctx = p->ctx;
    switch (p->op) {
        case OP_SCALAR_GEMM:
        case OP_TILED_GEMM: {
            const fe2o3_scalar_gemm_v1_args *a = reinterpret_cast<const fe2o3_scalar_gemm_v1_args *>(p->kernarg);
            if (p->schedule == FE2O3_GEMM_SCHEDULE_TCGEN05 && p->op == OP_SCALAR_GEMM) {
                int32_t st = gemm_split_launch(s, reinterpret_cast<const float *>(a->a.ptr), reinterpret_cast<const float *>(a->b.ptr),
                                               static_cast<uint16_t *>(p->scratch[0]), static_cast<uint16_t *>(p->scratch[1]), a->m,
                                               a->n, a->k);
                if (st != FE2O3_OK) return st;
                return gemm_tc_launch(&p->gemm[0], s);
            }
            if (p->schedule == FE2O3_GEMM_SCHEDULE_TCGEN05) return gemm_tc_launch(&p->gemm[0], s);
            return launch_gemm_exact(s, p->op == OP_SCALAR_GEMM ? FE2O3_DTYPE_F32 : FE2O3_DTYPE_BF16, false, a->a.ptr,
                                     a->b.ptr, a->c.ptr, a->m, a->n, a->k, a->k, a->n, a->n, 1.f, 0.f, nullptr, false);
        }
        case OP_TILED_GEMM_GENERAL: {
            const fe2o3_tiled_gemm_general_v1_args *a = reinterpret_cast<const fe2o3_tiled_gemm_general_v1_args *>(p->kernarg);
            if (p->schedule == FE2O3_GEMM_SCHEDULE_TCGEN05) return gemm_tc_launch(&p->gemm[0], s);
            return launch_gemm_exact(s, FE2O3_DTYPE_BF16, true, a->a.ptr, a->b.ptr, a->c.ptr, a->m, a->n, a->k, a->lda,
                                     a->ldb, a->ldc, a->alpha, a->beta, nullptr, false);
        }
        case OP_FLASH_ATTENTION: {
            if (p->attn) return attention_tc_launch(p->attn, s);
            return launch_attention_simt(ctx, s, reinterpret_cast<const fe2o3_flash_attention_v1_args *>(p->kernarg),
                                         nullptr, false);
        }
        case OP_MOE_EXPERT_FFN: {
            const fe2o3_moe_expert_ffn_v1_args *a = reinterpret_cast<const fe2o3_moe_expert_ffn_v1_args *>(p->kernarg);
            const uint32_t rows = (uint32_t)(a->compact_output.len / a->d_model);
            int32_t st = FE2O3_OK;
            if (!p->gemm[0].p.gather_perm)   // the first GEMM reads compact_x: fill it (otherwise it gathers the rows of x itself)
                st = launch_moe_compact(s, a->x.ptr, a->permutation.ptr, a->compact_x.ptr, rows, a->d_model, a->tokens);
            if (st != FE2O3_OK) return st;
            st = gemm_tc_launch(&p->gemm[0], s);
            if (st != FE2O3_OK) return st;
            return gemm_tc_launch(&p->gemm[1], s);
        }
        case OP_MOE_FFN_COMBINE: {
            const fe2o3_moe_expert_ffn_combine_v1_args *a = reinterpret_cast<const fe2o3_moe_expert_ffn_combine_v1_args *>(p->kernarg);
            (void)a;   // (the first GEMM clears the output the second one adds into)
            int32_t st = gemm_tc_launch(&p->gemm[0], s);
            if (st != FE2O3_OK) return st;
            return gemm_tc_launch(&p->gemm[1], s);
        }
        case OP_MOE_COMPACT: {
            const fe2o3_moe_compact_v1_args *a = reinterpret_cast<const fe2o3_moe_compact_v1_args *>(p->kernarg);
            return launch_moe_compact(s, a->x.ptr, a->permutation.ptr, a->compact_x.ptr, (uint32_t)a->permutation.len,
                                      a->d_model, a->tokens);
        }
        case OP_MOE_EP_FFN: {
            // the scalars a caller may patch between passes are taken from the packed block at launch
            const fe2o3_moe_ep_ffn_v1_args *a = reinterpret_cast<const fe2o3_moe_ep_ffn_v1_args *>(p->kernarg);
            for (int g = 0; g < 2; ++g) {
                p->gemm[g].p.ep.epoch = a->epoch;
                p->gemm[g].p.ep.spin_limit = a->spin_limit ? a->spin_limit : FE2O3_EP_DEFAULT_SPIN;
            }
            int32_t st = gemm_tc_launch(&p->gemm[0], s);
            if (st != FE2O3_OK) return st;
            return gemm_tc_launch(&p->gemm[1], s);
        }
        case OP_MOE_GROUPED_FFN: {
            int32_t st = gemm_tc_launch(&p->gemm[0], s);
            if (st != FE2O3_OK) return st;
            return gemm_tc_launch(&p->gemm[1], s);
        }
        default:
            return kOps[p->op].simple(ctx, s, p->kernarg, nullptr, false);
    }
}

// Host deadline poll; never blocks past timeout_ms.
int32_t bounded_wait(cudaStream_t s, uint32_t timeout_ms) {
    cudaEvent_t ev;
    FE2O3_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(ev, s);
    if (e != cudaSuccess) { cudaEventDestroy(ev); return fe2o3_cuda_status(e, "cudaEventRecord"); }
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    int32_t result = FE2O3_OK;
    for (;;) {
        e = cudaEventQuery(ev);
        if (e == cudaSuccess) break;
        if (e != cudaErrorNotReady) { result = fe2o3_cuda_status(e, "cudaEventQuery"); break; }
        if (std::chrono::steady_clock::now() >= deadline) {
            fe2o3_set_error("AmbiguousCompletion: no completion within %u ms; buffers must stay alive", timeout_ms);
            result = FE2O3_ERR_AMBIGUOUS_COMPLETION;
            break;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (result != FE2O3_ERR_AMBIGUOUS_COMPLETION) cudaEventDestroy(ev);  // an unfinished event is leaked, not destroyed
    return result;
}

int32_t take_status(fe2o3_ctx *ctx, cudaStream_t s, uint32_t *status) {
    FE2O3_CUDA(cudaMemcpyAsync(ctx->host_status, ctx->status_word, 4, cudaMemcpyDeviceToHost, s));
    FE2O3_CUDA(cudaStreamSynchronize(s));
    const uint32_t v = *ctx->host_status;
    if (status) *status = v;
    if (v != 0) FE2O3_CUDA(cudaMemsetAsync(ctx->status_word, 0, 4, s));
    return FE2O3_OK;
}

}  // namespace

extern "C" {

// ---- context ---------------------------------------------------------------------
int32_t fe2o3_ctx_create(int32_t device, fe2o3_ctx **out) {
    if (!out) return FE2O3_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        fe2o3_set_error("NoDevice: %s", e == cudaSuccess ? "no CUDA device" : cudaGetErrorString(e));
        return FE2O3_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= count) {
        fe2o3_set_error("device %d out of range (count %d)", device, count);
        return FE2O3_ERR_INVALID_ARGUMENT;
    }
    FE2O3_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    FE2O3_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        fe2o3_set_error("target check: device %d is sm_%d%d, this library is built for sm_100a only", device, prop.major,
                        prop.minor);
        return FE2O3_ERR_NOT_SM100;
    }
    // opt-in shared memory sizes are a per-device function attribute: set them for this device
    int32_t init = gemm_tc_init_device();
    if (init == FE2O3_OK) init = attention_tc_init_device();
    if (init == FE2O3_OK) init = device_scan_init_device();
    if (init != FE2O3_OK) return init;
    fe2o3_ctx *ctx = new (std::nothrow) fe2o3_ctx();
    if (!ctx) return FE2O3_ERR_SIZE_OVERFLOW;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    ctx->default_stream = nullptr;
    ctx->reduce_scratch_elems = FE2O3_REDUCE_MAX_BLOCKS + 1;
    uint32_t *dev = nullptr;
    e = cudaMalloc(&dev, (ctx->reduce_scratch_elems + 1) * sizeof(uint32_t));
    if (e != cudaSuccess) { delete ctx; return fe2o3_cuda_status(e, "cudaMalloc(context scratch)"); }
    cudaMemset(dev, 0, (ctx->reduce_scratch_elems + 1) * sizeof(uint32_t));
    ctx->reduce_scratch = dev;
    ctx->status_word = dev + ctx->reduce_scratch_elems;
    e = cudaMallocHost(&ctx->host_status, 64);
    if (e != cudaSuccess) { cudaFree(dev); delete ctx; return fe2o3_cuda_status(e, "cudaMallocHost"); }
    e = cudaMalloc(&ctx->route_scratch, FE2O3_ROUTE_SCRATCH_ELEMS * sizeof(uint32_t));
    if (e != cudaSuccess) {
        cudaFree(dev);
        cudaFreeHost(ctx->host_status);
        delete ctx;
        return fe2o3_cuda_status(e, "cudaMalloc(routing scratch)");
    }
    cudaMemset(ctx->route_scratch, 0, FE2O3_ROUTE_SCRATCH_ELEMS * sizeof(uint32_t));
    e = cudaMalloc(&ctx->scan_scratch, FE2O3_SCAN_SCRATCH_BYTES);
    if (e != cudaSuccess) {
        cudaFree(dev);
        cudaFree(ctx->route_scratch);
        cudaFree(ctx->scan_scratch);
        cudaFreeHost(ctx->host_status);
        delete ctx;
        return fe2o3_cuda_status(e, "cudaMalloc(scan scratch)");
    }
    *out = ctx;
    return FE2O3_OK;
}

int32_t fe2o3_ctx_destroy(fe2o3_ctx *ctx) {
    if (!ctx) return FE2O3_OK;
    cudaSetDevice(ctx->device);
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) {  // quiescent: safe to free; otherwise leak (completion is ambiguous)
        cudaFree(ctx->reduce_scratch);
        cudaFree(ctx->route_scratch);
        cudaFree(ctx->scan_scratch);
        cudaFreeHost(ctx->host_status);
    }
    delete ctx;
    return fe2o3_cuda_status(e, "cudaDeviceSynchronize");
}

int32_t fe2o3_ctx_bind_to_thread(fe2o3_ctx *ctx) {
    if (!ctx) return FE2O3_ERR_INVALID_ARGUMENT;
    FE2O3_CUDA(cudaSetDevice(ctx->device));
    return FE2O3_OK;
}

int32_t fe2o3_ctx_device(const fe2o3_ctx *ctx, int32_t *device) {
    if (!ctx || !device) return FE2O3_ERR_INVALID_ARGUMENT;
    *device = ctx->device;
    return FE2O3_OK;
}

int32_t fe2o3_ctx_observe_environment(fe2o3_ctx *ctx, fe2o3_device_properties *out) {
    if (!ctx || !out) return FE2O3_ERR_INVALID_ARGUMENT;
    cudaDeviceProp prop;
    FE2O3_CUDA(cudaGetDeviceProperties(&prop, ctx->device));
    memset(out, 0, sizeof *out);
    strncpy(out->name, prop.name, sizeof out->name - 1);
    out->total_global_bytes = prop.totalGlobalMem;
    out->compute_major = prop.major;
    out->compute_minor = prop.minor;
    out->multiprocessors = prop.multiProcessorCount;
    out->max_shared_bytes_per_block_optin = (uint32_t)prop.sharedMemPerBlockOptin;
    out->l2_bytes = prop.l2CacheSize;
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, ctx->device);
    out->sm_clock_khz = v;
    cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, ctx->device);
    out->mem_clock_khz = v;
    out->warp_size = prop.warpSize;
    return FE2O3_OK;
}

// ---- streams -----------------------------------------------------------------------
static int32_t make_stream(fe2o3_ctx *ctx, cudaStream_t s, bool owned, fe2o3_stream **out) {
    fe2o3_stream *st = new (std::nothrow) fe2o3_stream();
    if (!st) return FE2O3_ERR_SIZE_OVERFLOW;
    st->ctx = ctx;
    st->s = s;
    st->owned = owned;
    *out = st;
    return FE2O3_OK;
}
int32_t fe2o3_stream_default(fe2o3_ctx *ctx, fe2o3_stream **out) {
    if (!ctx || !out) return FE2O3_ERR_INVALID_ARGUMENT;
    return make_stream(ctx, ctx->default_stream, false, out);
}
int32_t fe2o3_stream_create(fe2o3_ctx *ctx, fe2o3_stream **out) {
    if (!ctx || !out) return FE2O3_ERR_INVALID_ARGUMENT;
    FE2O3_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t s;
    FE2O3_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    return make_stream(ctx, s, true, out);
}
int32_t fe2o3_stream_wrap(fe2o3_ctx *ctx, void *cuda_stream, fe2o3_stream **out) {
    if (!ctx || !out) return FE2O3_ERR_INVALID_ARGUMENT;
    return make_stream(ctx, static_cast<cudaStream_t>(cuda_stream), false, out);
}
int32_t fe2o3_stream_sync(fe2o3_stream *stream) {
    if (!stream) return FE2O3_ERR_INVALID_ARGUMENT;
    FE2O3_CUDA(cudaStreamSynchronize(stream->s));
    return FE2O3_OK;
}
int32_t fe2o3_stream_native(fe2o3_stream *stream, void **cuda_stream) {
    if (!stream || !cuda_stream) return FE2O3_ERR_INVALID_ARGUMENT;
    *cuda_stream = stream->s;
    return FE2O3_OK;
}
int32_t fe2o3_stream_destroy(fe2o3_stream *stream) {
    if (!stream) return FE2O3_OK;
    int32_t st = FE2O3_OK;
    if (stream->owned) st = fe2o3_cuda_status(cudaStreamDestroy(stream->s), "cudaStreamDestroy");
    delete stream;
    return st;
}

// ---- buffers -------------------------------------------------------------------------
int32_t fe2o3_buf_alloc_zeroed(fe2o3_stream *stream, uint64_t elements, uint32_t element_bytes, fe2o3_buf **out) {
    if (!stream || !out || element_bytes == 0) return FE2O3_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    uint64_t bytes;
    if (mul_overflow(elements, element_bytes, &bytes)) {
        fe2o3_set_error("SizeOverflow: %llu elements of %u bytes", (unsigned long long)elements, element_bytes);
        return FE2O3_ERR_SIZE_OVERFLOW;
    }
    FE2O3_CUDA(cudaSetDevice(stream->ctx->device));
    void *ptr = nullptr;
    if (bytes) {
        FE2O3_CUDA(cudaMalloc(&ptr, bytes));
        cudaError_t e = cudaMemsetAsync(ptr, 0, bytes, stream->s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream->s);
        if (e != cudaSuccess) { cudaFree(ptr); return fe2o3_cuda_status(e, "zero-fill"); }
    }
    fe2o3_buf *b = new (std::nothrow) fe2o3_buf{stream->ctx, ptr, elements, element_bytes, false, 0};
    if (!b) { cudaFree(ptr); return FE2O3_ERR_SIZE_OVERFLOW; }
    *out = b;
    return FE2O3_OK;
}

int32_t fe2o3_buf_copy_from_host_async(fe2o3_stream *stream, fe2o3_buf *buf, const void *host, uint64_t elements) {
    if (!stream || !buf || (!host && elements)) return FE2O3_ERR_INVALID_ARGUMENT;
    if (stream->ctx != buf->ctx) { fe2o3_set_error("OperationDeviceMismatch"); return FE2O3_ERR_DEVICE_MISMATCH; }
    if (elements > buf->elements) { fe2o3_set_error("copy exceeds buffer"); return FE2O3_ERR_INVALID_REGION; }
    if (elements) FE2O3_CUDA(cudaMemcpyAsync(buf->ptr, host, elements * buf->element_bytes, cudaMemcpyHostToDevice, stream->s));
    return FE2O3_OK;
}
int32_t fe2o3_buf_copy_to_host_async(fe2o3_stream *stream, const fe2o3_buf *buf, void *host, uint64_t elements) {
    if (!stream || !buf || (!host && elements)) return FE2O3_ERR_INVALID_ARGUMENT;
    if (stream->ctx != buf->ctx) { fe2o3_set_error("OperationDeviceMismatch"); return FE2O3_ERR_DEVICE_MISMATCH; }
    if (elements > buf->elements) { fe2o3_set_error("copy exceeds buffer"); return FE2O3_ERR_INVALID_REGION; }
    if (elements) FE2O3_CUDA(cudaMemcpyAsync(host, buf->ptr, elements * buf->element_bytes, cudaMemcpyDeviceToHost, stream->s));
    return FE2O3_OK;
}
int32_t fe2o3_buf_from_host(fe2o3_stream *stream, const void *host, uint64_t elements, uint32_t element_bytes,
                            fe2o3_buf **out) {
    int32_t st = fe2o3_buf_alloc_zeroed(stream, elements, element_bytes, out);
    if (st != FE2O3_OK) return st;
    st = fe2o3_buf_copy_from_host_async(stream, *out, host, elements);
    if (st == FE2O3_OK) st = fe2o3_cuda_status(cudaStreamSynchronize(stream->s), "cudaStreamSynchronize");
    if (st != FE2O3_OK) { fe2o3_buf_free(*out); *out = nullptr; }
    return st;
}
int32_t fe2o3_buf_to_host(fe2o3_stream *stream, const fe2o3_buf *buf, void *host, uint64_t elements) {
    int32_t st = fe2o3_buf_copy_to_host_async(stream, buf, host, elements);
    if (st != FE2O3_OK) return st;
    return fe2o3_cuda_status(cudaStreamSynchronize(stream->s), "cudaStreamSynchronize");
}
int32_t fe2o3_buf_quarantine(fe2o3_buf *buf) {
    if (!buf) return FE2O3_ERR_INVALID_ARGUMENT;
    buf->quarantined = true;
    return FE2O3_OK;
}
int32_t fe2o3_buf_free(fe2o3_buf *buf) {
    if (!buf) return FE2O3_OK;
    if (buf->owners) {
        fe2o3_set_error("Busy: the buffer is owned by %u submitted operation(s)", buf->owners);
        return FE2O3_ERR_BUSY;
    }
    int32_t st = FE2O3_OK;
    if (buf->ptr && !buf->quarantined) st = fe2o3_cuda_status(cudaFree(buf->ptr), "cudaFree");
    delete buf;
    return st;
}
uint64_t fe2o3_buf_ptr(const fe2o3_buf *buf) { return buf ? reinterpret_cast<uint64_t>(buf->ptr) : 0; }
uint64_t fe2o3_buf_len(const fe2o3_buf *buf) { return buf ? buf->elements : 0; }
int32_t fe2o3_buf_slice(const fe2o3_buf *buf, uint64_t start, uint64_t len, fe2o3_slice *out) {
    if (!buf || !out) return FE2O3_ERR_INVALID_ARGUMENT;
    if (start > buf->elements || len > buf->elements - start) {
        fe2o3_set_error("InvalidRegion: [%llu, +%llu) of %llu", (unsigned long long)start, (unsigned long long)len,
                        (unsigned long long)buf->elements);
        return FE2O3_ERR_INVALID_REGION;
    }
    out->ptr = reinterpret_cast<uint64_t>(buf->ptr) + start * buf->element_bytes;
    out->len = len;
    return FE2O3_OK;
}

// ---- owned asynchronous operations ----------------------------------------------------------
struct fe2o3_operation {
    fe2o3_ctx *ctx;
    cudaStream_t stream;
    cudaEvent_t done;
    fe2o3_buf **buffers;
    uint32_t n_buffers;
    bool launched_kernel;
};
static void operation_release(fe2o3_operation *op, bool quarantine) {
    for (uint32_t i = 0; i < op->n_buffers; ++i) {
        if (op->buffers[i]->owners) op->buffers[i]->owners -= 1;
        if (quarantine) op->buffers[i]->quarantined = true;
    }
    if (!quarantine) cudaEventDestroy(op->done);   // an event whose completion is unknown is leaked with its buffers
    delete[] op->buffers;
    delete op;
}
int32_t fe2o3_operation_submit(fe2o3_stream *stream, fe2o3_prepared *prepared, fe2o3_buf *const *buffers, uint32_t n_buffers,
                               const fe2o3_host_copy *copies_in, uint32_t n_in, const fe2o3_host_copy *copies_out,
                               uint32_t n_out, fe2o3_operation **out) {
    if (!stream || !out || (n_buffers && !buffers) || (n_in && !copies_in) || (n_out && !copies_out))
        return FE2O3_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (prepared && prepared->ctx != stream->ctx) { fe2o3_set_error("WrongContext{role=stream}"); return FE2O3_ERR_DEVICE_MISMATCH; }
    const uint32_t total = n_buffers + n_in + n_out;
    fe2o3_operation *op = new (std::nothrow) fe2o3_operation{stream->ctx, stream->s, nullptr, nullptr, 0, prepared != nullptr};
    if (!op) return FE2O3_ERR_SIZE_OVERFLOW;
    op->buffers = new (std::nothrow) fe2o3_buf *[total ? total : 1];
    if (!op->buffers) { delete op; return FE2O3_ERR_SIZE_OVERFLOW; }
    auto own = [&](fe2o3_buf *b) -> bool {
        if (!b || b->ctx != stream->ctx) return false;
        b->owners += 1;
        op->buffers[op->n_buffers++] = b;
        return true;
    };
    bool ok = true;
    for (uint32_t i = 0; ok && i < n_buffers; ++i) ok = own(buffers[i]);
    for (uint32_t i = 0; ok && i < n_in; ++i) ok = own(copies_in[i].buffer) && copies_in[i].elements <= copies_in[i].buffer->elements;
    for (uint32_t i = 0; ok && i < n_out; ++i) ok = own(copies_out[i].buffer) && copies_out[i].elements <= copies_out[i].buffer->elements;
    cudaError_t e = cudaSuccess;
    if (ok) e = cudaSetDevice(stream->ctx->device);
    if (ok && e == cudaSuccess) e = cudaEventCreateWithFlags(&op->done, cudaEventDisableTiming);
    if (!ok || e != cudaSuccess) {
        // nothing has been submitted: hand everything back (Err before submission)
        for (uint32_t i = 0; i < op->n_buffers; ++i) op->buffers[i]->owners -= 1;
        delete[] op->buffers;
        delete op;
        if (!ok) { fe2o3_set_error("OperationDeviceMismatch or copy exceeds buffer"); return FE2O3_ERR_DEVICE_MISMATCH; }
        return fe2o3_cuda_status(e, "operation submit");
    }
    // From here on work may be pending: on any error the operation is still returned so that the caller
    // can establish quiescence through it (operation.rs:296-305), together with the error.
    int32_t st = FE2O3_OK;
    for (uint32_t i = 0; st == FE2O3_OK && i < n_in; ++i)
        st = fe2o3_cuda_status(cudaMemcpyAsync(copies_in[i].buffer->ptr, copies_in[i].host,
                                               copies_in[i].elements * copies_in[i].buffer->element_bytes, cudaMemcpyHostToDevice,
                                               stream->s), "operation copy in");
    if (st == FE2O3_OK && prepared) st = launch_prepared(prepared, stream->s);
    for (uint32_t i = 0; st == FE2O3_OK && i < n_out; ++i)
        st = fe2o3_cuda_status(cudaMemcpyAsync(copies_out[i].host, copies_out[i].buffer->ptr,
                                               copies_out[i].elements * copies_out[i].buffer->element_bytes, cudaMemcpyDeviceToHost,
                                               stream->s), "operation copy out");
    cudaEventRecord(op->done, stream->s);
    *out = op;
    return st;
}
int32_t fe2o3_operation_is_complete(fe2o3_operation *op, int32_t *done) {
    if (!op || !done) return FE2O3_ERR_INVALID_ARGUMENT;
    cudaError_t e = cudaEventQuery(op->done);
    if (e == cudaErrorNotReady) { *done = 0; return FE2O3_OK; }
    *done = e == cudaSuccess ? 1 : 0;
    return fe2o3_cuda_status(e, "cudaEventQuery");
}
int32_t fe2o3_operation_wait(fe2o3_operation *op, uint32_t timeout_ms, uint32_t *kernel_status) {
    if (!op) return FE2O3_ERR_INVALID_ARGUMENT;
    if (kernel_status) *kernel_status = 0;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    cudaError_t e;
    for (;;) {
        e = cudaEventQuery(op->done);
        if (e != cudaErrorNotReady) break;
        if (std::chrono::steady_clock::now() >= deadline) {
            fe2o3_set_error("StillRunning: not complete after %u ms; the operation keeps its buffers", timeout_ms);
            return FE2O3_ERR_STILL_RUNNING;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (e == cudaSuccess) {
        int32_t st = FE2O3_OK;
        uint32_t ks = 0;
        if (op->launched_kernel) st = take_status(op->ctx, op->stream, &ks);
        if (kernel_status) *kernel_status = ks;
        operation_release(op, false);
        if (st == FE2O3_OK && ks != 0) { fe2o3_set_error("kernel reported status word %u", ks); return FE2O3_ERR_KERNEL_STATUS; }
        return st;
    }
    // the event reported an execution error: quiescence of the whole stream decides
    const int32_t event_error = fe2o3_cuda_status(e, "operation event");
    if (cudaStreamSynchronize(op->stream) == cudaSuccess) {
        operation_release(op, false);
        return event_error;
    }
    operation_release(op, true);
    fe2o3_set_error("AmbiguousCompletion: neither the event nor the stream could establish completion; buffers are quarantined");
    return FE2O3_ERR_AMBIGUOUS_COMPLETION;
}
int32_t fe2o3_operation_abandon(fe2o3_operation *op) {
    if (!op) return FE2O3_OK;
    operation_release(op, true);
    return FE2O3_OK;
}

int32_t fe2o3_pinned_alloc(fe2o3_ctx *ctx, uint64_t bytes, void **out) {
    if (!ctx || !out) return FE2O3_ERR_INVALID_ARGUMENT;
    FE2O3_CUDA(cudaSetDevice(ctx->device));
    FE2O3_CUDA(cudaMallocHost(out, bytes ? bytes : 1));
    return FE2O3_OK;
}
int32_t fe2o3_pinned_free(fe2o3_ctx *ctx, void *ptr) {
    (void)ctx;
    if (ptr) FE2O3_CUDA(cudaFreeHost(ptr));
    return FE2O3_OK;
}

// ---- events ----------------------------------------------------------------------------
int32_t fe2o3_event_create(fe2o3_ctx *ctx, fe2o3_event **out) {
    if (!ctx || !out) return FE2O3_ERR_INVALID_ARGUMENT;
    FE2O3_CUDA(cudaSetDevice(ctx->device));
    cudaEvent_t e;
    FE2O3_CUDA(cudaEventCreate(&e));
    *out = new (std::nothrow) fe2o3_event{ctx, e};
    return *out ? FE2O3_OK : FE2O3_ERR_SIZE_OVERFLOW;
}
int32_t fe2o3_event_record(fe2o3_event *event, fe2o3_stream *stream) {
    if (!event || !stream) return FE2O3_ERR_INVALID_ARGUMENT;
    if (event->ctx != stream->ctx) { fe2o3_set_error("OperationDeviceMismatch"); return FE2O3_ERR_DEVICE_MISMATCH; }
    FE2O3_CUDA(cudaEventRecord(event->e, stream->s));
    return FE2O3_OK;
}
int32_t fe2o3_event_sync(fe2o3_event *event) {
    if (!event) return FE2O3_ERR_INVALID_ARGUMENT;
    FE2O3_CUDA(cudaEventSynchronize(event->e));
    return FE2O3_OK;
}
int32_t fe2o3_event_query(fe2o3_event *event, int32_t *done) {
    if (!event || !done) return FE2O3_ERR_INVALID_ARGUMENT;
    cudaError_t e = cudaEventQuery(event->e);
    if (e == cudaErrorNotReady) { *done = 0; return FE2O3_OK; }
    *done = 1;
    return fe2o3_cuda_status(e, "cudaEventQuery");
}
int32_t fe2o3_event_elapsed_ms(fe2o3_event *start, fe2o3_event *end, float *ms) {
    if (!start || !end || !ms) return FE2O3_ERR_INVALID_ARGUMENT;
    FE2O3_CUDA(cudaEventElapsedTime(ms, start->e, end->e));
    return FE2O3_OK;
}
int32_t fe2o3_stream_wait_event(fe2o3_stream *stream, fe2o3_event *event) {
    if (!stream || !event) return FE2O3_ERR_INVALID_ARGUMENT;
    if (event->ctx != stream->ctx) { fe2o3_set_error("OperationDeviceMismatch"); return FE2O3_ERR_DEVICE_MISMATCH; }
    FE2O3_CUDA(cudaStreamWaitEvent(stream->s, event->e, 0));
    return FE2O3_OK;
}
int32_t fe2o3_event_destroy(fe2o3_event *event) {
    if (!event) return FE2O3_OK;
    cudaError_t e = cudaEventDestroy(event->e);
    delete event;
    return fe2o3_cuda_status(e, "cudaEventDestroy");
}

int32_t fe2o3_peer_access_enable(fe2o3_ctx *ctx, int32_t peer_device) {
    if (!ctx) return FE2O3_ERR_INVALID_ARGUMENT;
    FE2O3_CUDA(cudaSetDevice(ctx->device));
    int can = 0;
    FE2O3_CUDA(cudaDeviceCanAccessPeer(&can, ctx->device, peer_device));
    if (!can) { fe2o3_set_error("peer access %d -> %d unavailable", ctx->device, peer_device); return FE2O3_ERR_INVALID_ARGUMENT; }
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return FE2O3_OK; }
    return fe2o3_cuda_status(e, "cudaDeviceEnablePeerAccess");
}

// ---- peer-visible regions (CUDA IPC) ---------------------------------------------------
struct fe2o3_peer_region {
    fe2o3_ctx *ctx;
    void *ptr;
    uint64_t bytes;   // 0 for an imported mapping
    bool imported;
};
static_assert(sizeof(cudaIpcMemHandle_t) == FE2O3_PEER_HANDLE_BYTES, "handle size");

int32_t fe2o3_peer_region_create(fe2o3_ctx *ctx, uint64_t bytes, fe2o3_peer_region **out) {
    if (!ctx || !out || bytes == 0) return FE2O3_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    FE2O3_CUDA(cudaSetDevice(ctx->device));
    void *ptr = nullptr;
    FE2O3_CUDA(cudaMalloc(&ptr, bytes));
    cudaError_t e = cudaMemset(ptr, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { cudaFree(ptr); return fe2o3_cuda_status(e, "zero-fill(peer region)"); }
    *out = new (std::nothrow) fe2o3_peer_region{ctx, ptr, bytes, false};
    if (!*out) { cudaFree(ptr); return FE2O3_ERR_SIZE_OVERFLOW; }
    return FE2O3_OK;
}
int32_t fe2o3_peer_region_export(const fe2o3_peer_region *region, uint8_t handle[FE2O3_PEER_HANDLE_BYTES]) {
    if (!region || !handle || region->imported) return FE2O3_ERR_INVALID_ARGUMENT;
    cudaIpcMemHandle_t h;
    FE2O3_CUDA(cudaIpcGetMemHandle(&h, region->ptr));
    memcpy(handle, &h, sizeof h);
    return FE2O3_OK;
}
int32_t fe2o3_peer_region_import(fe2o3_ctx *ctx, const uint8_t handle[FE2O3_PEER_HANDLE_BYTES], fe2o3_peer_region **out) {
    if (!ctx || !handle || !out) return FE2O3_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    FE2O3_CUDA(cudaSetDevice(ctx->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void *ptr = nullptr;
    FE2O3_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    *out = new (std::nothrow) fe2o3_peer_region{ctx, ptr, 0, true};
    if (!*out) { cudaIpcCloseMemHandle(ptr); return FE2O3_ERR_SIZE_OVERFLOW; }
    return FE2O3_OK;
}
uint64_t fe2o3_peer_region_ptr(const fe2o3_peer_region *region) { return region ? reinterpret_cast<uint64_t>(region->ptr) : 0; }
uint64_t fe2o3_peer_region_bytes(const fe2o3_peer_region *region) { return region ? region->bytes : 0; }
int32_t fe2o3_peer_region_destroy(fe2o3_peer_region *region) {
    if (!region) return FE2O3_OK;
    cudaSetDevice(region->ctx->device);
    cudaError_t e = region->imported ? cudaIpcCloseMemHandle(region->ptr) : cudaFree(region->ptr);
    delete region;
    return fe2o3_cuda_status(e, "peer region release");
}

const char *fe2o3_status_string(int32_t s) {
    switch (s) {
        case FE2O3_OK: return "Ok";
        case FE2O3_ERR_NO_DEVICE: return "NoDevice";
        case FE2O3_ERR_INVALID_ARGUMENT: return "InvalidArgument";
        case FE2O3_ERR_SIZE_OVERFLOW: return "SizeOverflow";
        case FE2O3_ERR_DEVICE_MISMATCH: return "OperationDeviceMismatch";
        case FE2O3_ERR_LENGTH: return "Length";
        case FE2O3_ERR_ALIGNMENT: return "Alignment";
        case FE2O3_ERR_NULL_ADDRESS: return "NullAddress";
        case FE2O3_ERR_INVALID_REGION: return "InvalidRegion";
        case FE2O3_ERR_OUTPUT_ALIASES_INPUT: return "OutputAliasesInput";
        case FE2O3_ERR_UNSUPPORTED_SHAPE: return "UnsupportedShape";
        case FE2O3_ERR_AMBIGUOUS_COMPLETION: return "AmbiguousCompletion";
        case FE2O3_ERR_KERNEL_STATUS: return "KernelStatus";
        case FE2O3_ERR_UNKNOWN_SYMBOL: return "UnknownSymbol";
        case FE2O3_ERR_NOT_SM100: return "NotSm100";
        case FE2O3_ERR_NONFINITE: return "NonFinite";
        case FE2O3_ERR_EXECUTABLE_REJECTED: return "ExecutableRejected";
        case FE2O3_ERR_BUSY: return "Busy";
        case FE2O3_ERR_STILL_RUNNING: return "StillRunning";
        case FE2O3_ERR_NO_DISPATCH: return "NoDispatch";
        default: return s > 0 ? "CudaError" : "Unknown";
    }
}
const char *fe2o3_last_error(void) { return g_error; }
uint64_t fe2o3_launch_count(void) { return g_launches.load(); }

// ---- checks --------------------------------------------------------------------------------
#define DEFINE_CHECK(name, op) \
    int32_t fe2o3_##name##_check(const fe2o3_##name##_args *args) { return check_op(op, args); }
DEFINE_CHECK(scalar_gemm_v1, OP_SCALAR_GEMM)
DEFINE_CHECK(tiled_gemm_v1, OP_TILED_GEMM)
DEFINE_CHECK(tiled_gemm_general_v1, OP_TILED_GEMM_GENERAL)
DEFINE_CHECK(flash_attention_v1, OP_FLASH_ATTENTION)
DEFINE_CHECK(row_softmax_v1, OP_ROW_SOFTMAX)
DEFINE_CHECK(moe_top2_v1, OP_MOE_TOP2)
DEFINE_CHECK(moe_gate_v1, OP_MOE_GATE)
DEFINE_CHECK(moe_route_weights_v1, OP_MOE_ROUTE_WEIGHTS)
DEFINE_CHECK(moe_expert_ffn_v1, OP_MOE_EXPERT_FFN)
DEFINE_CHECK(moe_expert_combine_v1, OP_MOE_COMBINE)
DEFINE_CHECK(masked_reduce_u32, OP_MASKED_REDUCE)
DEFINE_CHECK(masked_reduce_u32_packed, OP_MASKED_REDUCE_PACKED)
DEFINE_CHECK(device_scan_u32, OP_DEVICE_SCAN_U32)
DEFINE_CHECK(device_scan_f32, OP_DEVICE_SCAN_F32)
DEFINE_CHECK(wave_lds_v1, OP_WAVE_LDS)
DEFINE_CHECK(wave64_collectives_v1, OP_WAVE64_COLLECTIVES)
DEFINE_CHECK(wave64_collectives_segmented, OP_WAVE64_SEGMENTED)
DEFINE_CHECK(lds_publish_read_reduce_i32_v1, OP_LDS_REDUCE_I32)
DEFINE_CHECK(scoped_atomic_add_u32_v1, OP_SCOPED_ATOMIC_ADD)
DEFINE_CHECK(moe_ep_exchange_v1, OP_MOE_EP_EXCHANGE)

// ---- prepare ---------------------------------------------------------------------------------
#define DEFINE_SIMPLE_PREPARE(name, op)                                                                 \
    int32_t fe2o3_##name##_prepare(fe2o3_ctx *ctx, const fe2o3_##name##_args *args, fe2o3_prepared **out) { \
        int32_t st = prepare_common(ctx, op, args, out);                                                \
        if (st != FE2O3_OK) return st;                                                                  \
        return finish_simple(*out);                                                                     \
    }
DEFINE_SIMPLE_PREPARE(row_softmax_v1, OP_ROW_SOFTMAX)
DEFINE_SIMPLE_PREPARE(moe_top2_v1, OP_MOE_TOP2)
DEFINE_SIMPLE_PREPARE(moe_gate_v1, OP_MOE_GATE)
DEFINE_SIMPLE_PREPARE(moe_route_weights_v1, OP_MOE_ROUTE_WEIGHTS)
DEFINE_SIMPLE_PREPARE(moe_expert_combine_v1, OP_MOE_COMBINE)
DEFINE_SIMPLE_PREPARE(masked_reduce_u32, OP_MASKED_REDUCE)
DEFINE_SIMPLE_PREPARE(masked_reduce_u32_packed, OP_MASKED_REDUCE_PACKED)
DEFINE_SIMPLE_PREPARE(device_scan_u32, OP_DEVICE_SCAN_U32)
DEFINE_SIMPLE_PREPARE(device_scan_f32, OP_DEVICE_SCAN_F32)
DEFINE_SIMPLE_PREPARE(wave_lds_v1, OP_WAVE_LDS)
DEFINE_SIMPLE_PREPARE(wave64_collectives_v1, OP_WAVE64_COLLECTIVES)
DEFINE_SIMPLE_PREPARE(wave64_collectives_segmented, OP_WAVE64_SEGMENTED)
DEFINE_SIMPLE_PREPARE(lds_publish_read_reduce_i32_v1, OP_LDS_REDUCE_I32)
DEFINE_SIMPLE_PREPARE(scoped_atomic_add_u32_v1, OP_SCOPED_ATOMIC_ADD)
DEFINE_SIMPLE_PREPARE(moe_ep_exchange_v1, OP_MOE_EP_EXCHANGE)

static int32_t fail_prepare(fe2o3_prepared **out, int32_t st) {
    fe2o3_prepared_destroy(*out);
    *out = nullptr;
    return st;
}

int32_t fe2o3_scalar_gemm_v1_prepare(fe2o3_ctx *ctx, const fe2o3_scalar_gemm_v1_args *a, uint32_t schedule,
                                     fe2o3_prepared **out) {
    int32_t st = prepare_common(ctx, OP_SCALAR_GEMM, a, out);
    if (st != FE2O3_OK) return st;
    if ((uint64_t)a->m * a->n == 0) return fail_prepare(out, FE2O3_ERR_NO_DISPATCH);
    st = resolve_gemm(*out, schedule, FE2O3_DTYPE_F32, a->a.ptr, a->b.ptr, a->c.ptr, a->m, a->n, a->k, a->k, a->n, a->n,
                      1.f, 0.f, false);
    return st == FE2O3_OK ? st : fail_prepare(out, st);
}
int32_t fe2o3_tiled_gemm_v1_prepare(fe2o3_ctx *ctx, const fe2o3_tiled_gemm_v1_args *a, uint32_t schedule,
                                    fe2o3_prepared **out) {
    int32_t st = prepare_common(ctx, OP_TILED_GEMM, a, out);
    if (st != FE2O3_OK) return st;
    if ((uint64_t)a->m * a->n == 0) return fail_prepare(out, FE2O3_ERR_NO_DISPATCH);
    st = resolve_gemm(*out, schedule, FE2O3_DTYPE_BF16, a->a.ptr, a->b.ptr, a->c.ptr, a->m, a->n, a->k, a->k, a->n,
                      a->n, 1.f, 0.f, false);
    return st == FE2O3_OK ? st : fail_prepare(out, st);
}
int32_t fe2o3_tiled_gemm_general_v1_prepare(fe2o3_ctx *ctx, const fe2o3_tiled_gemm_general_v1_args *a,
                                            uint32_t schedule, fe2o3_prepared **out) {
    int32_t st = prepare_common(ctx, OP_TILED_GEMM_GENERAL, a, out);
    if (st != FE2O3_OK) return st;
    if ((uint64_t)a->m * a->n == 0) return fail_prepare(out, FE2O3_ERR_NO_DISPATCH);
    st = resolve_gemm(*out, schedule, FE2O3_DTYPE_BF16, a->a.ptr, a->b.ptr, a->c.ptr, a->m, a->n, a->k, a->lda, a->ldb,
                      a->ldc, a->alpha, a->beta, true);
    return st == FE2O3_OK ? st : fail_prepare(out, st);
}
int32_t fe2o3_flash_attention_v1_prepare(fe2o3_ctx *ctx, const fe2o3_flash_attention_v1_args *a, fe2o3_prepared **out) {
    int32_t st = prepare_common(ctx, OP_FLASH_ATTENTION, a, out);
    if (st != FE2O3_OK) return st;
    if (attention_tc_supported(a)) {
        st = attention_tc_plan(ctx, a, &(*out)->attn);
        if (st != FE2O3_OK) return fail_prepare(out, st);
        attention_tc_geometry((*out)->attn, &(*out)->geo);
        return FE2O3_OK;
    }
    return launch_attention_simt(ctx, nullptr, a, &(*out)->geo, true);
}
int32_t fe2o3_moe_expert_ffn_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_expert_ffn_v1_args *a, fe2o3_prepared **out) {
    int32_t st = prepare_common(ctx, OP_MOE_EXPERT_FFN, a, out);
    if (st != FE2O3_OK) return st;
    fe2o3_prepared *p = *out;
    const uint32_t rows = (uint32_t)(a->compact_output.len / a->d_model);
    const uint32_t *off = reinterpret_cast<const uint32_t *>(a->expert_offsets.ptr);
    st = gemm_tc_plan(ctx, &p->gemm[0], a->compact_x.ptr, a->w1.ptr, a->hidden.ptr, rows, a->d_ff, a->d_model,
                      a->d_model, a->d_ff, a->d_ff, 1.f, 0.f, 2u, off, a->experts);
    if (st == FE2O3_OK)
        st = gemm_tc_plan(ctx, &p->gemm[1], a->hidden.ptr, a->w2.ptr, a->compact_output.ptr, rows, a->d_model, a->d_ff,
                          a->d_ff, a->d_model, a->d_model, 1.f, 0.f, 0u, off, a->experts);
    if (st != FE2O3_OK) return fail_prepare(out, st);
    // The first GEMM fetches its rows of x through `permutation` itself when the row length allows it, which
    // saves the compaction pass (compact_x is then left untouched); FE2O3_FFN_GATHER=0 keeps the compaction.
    const char *gather_env = getenv("FE2O3_FFN_GATHER");
    bool gathered = false;
    if (!(gather_env && gather_env[0] == '0'))
        gathered = gemm_tc_set_gather(&p->gemm[0], reinterpret_cast<const uint32_t *>(a->permutation.ptr),
                                      reinterpret_cast<const void *>(a->x.ptr), a->tokens);
    gemm_tc_geometry(&p->gemm[0], &p->geo);
    p->geo.launches = gathered ? 2 : 3;
    return FE2O3_OK;
}

int32_t fe2o3_moe_expert_ffn_combine_v1_check(const fe2o3_moe_expert_ffn_combine_v1_args *args) {
    return check_op(OP_MOE_FFN_COMBINE, args);
}
int32_t fe2o3_moe_expert_ffn_combine_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_expert_ffn_combine_v1_args *a,
                                                fe2o3_prepared **out) {
    int32_t st = prepare_common(ctx, OP_MOE_FFN_COMBINE, a, out);
    if (st != FE2O3_OK) return st;
    fe2o3_prepared *p = *out;
    const uint32_t rows = (uint32_t)a->permutation.len;
    const uint32_t *off = reinterpret_cast<const uint32_t *>(a->expert_offsets.ptr);
    const uint32_t *perm = reinterpret_cast<const uint32_t *>(a->permutation.ptr);
    // A of the first GEMM is gathered (the address given for A only makes a valid tensor map: x itself)
    st = gemm_tc_plan(ctx, &p->gemm[0], a->x.ptr, a->w1.ptr, a->hidden.ptr, rows, a->d_ff, a->d_model,
                      a->d_model, a->d_ff, a->d_ff, 1.f, 0.f, EPI_GELU_BF16, off, a->experts);
    if (st == FE2O3_OK)
        st = gemm_tc_plan(ctx, &p->gemm[1], a->hidden.ptr, a->w2.ptr, a->combined_output.ptr, rows, a->d_model, a->d_ff,
                          a->d_ff, a->d_model, a->d_model, 1.f, 0.f, EPI_COMBINE_ADD, off, a->experts);
    if (st != FE2O3_OK) return fail_prepare(out, st);
    if (!gemm_tc_set_gather(&p->gemm[0], perm, reinterpret_cast<const void *>(a->x.ptr), a->tokens)) {
        fe2o3_set_error("Unsupported{x must be 16-byte aligned with whole 64-column blocks}");
        return fail_prepare(out, FE2O3_ERR_UNSUPPORTED_SHAPE);
    }
    gemm_tc_set_combine(&p->gemm[1], perm, reinterpret_cast<const float *>(a->route_weights.ptr), a->tokens);
    // the second GEMM adds into the output, which starts from +0: cleared by the first GEMM's idle epilogue warps
    p->gemm[0].p.zero_ptr = reinterpret_cast<uint4 *>(a->combined_output.ptr);
    p->gemm[0].p.zero_vecs = (uint64_t)a->tokens * a->d_model / 4;
    gemm_tc_geometry(&p->gemm[0], &p->geo);
    p->geo.launches = 2;
    return FE2O3_OK;
}

int32_t fe2o3_moe_compact_v1_check(const fe2o3_moe_compact_v1_args *args) { return check_op(OP_MOE_COMPACT, args); }
int32_t fe2o3_moe_grouped_ffn_v1_check(const fe2o3_moe_grouped_ffn_v1_args *args) {
    return check_op(OP_MOE_GROUPED_FFN, args);
}
int32_t fe2o3_moe_compact_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_compact_v1_args *a, fe2o3_prepared **out) {
    int32_t st = prepare_common(ctx, OP_MOE_COMPACT, a, out);
    if (st != FE2O3_OK) return st;
    (*out)->geo = fe2o3_geometry{{(uint32_t)a->permutation.len, 1, 1}, {256, 1, 1}, 0, 1};
    return FE2O3_OK;
}
int32_t fe2o3_moe_grouped_ffn_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_grouped_ffn_v1_args *a,
                                         fe2o3_prepared **out) {
    int32_t st = prepare_common(ctx, OP_MOE_GROUPED_FFN, a, out);
    if (st != FE2O3_OK) return st;
    fe2o3_prepared *p = *out;
    const uint32_t rows = (uint32_t)(a->compact_output.len / a->d_model);
    const uint32_t *off = reinterpret_cast<const uint32_t *>(a->group_offsets.ptr);
    st = gemm_tc_plan(ctx, &p->gemm[0], a->compact_x.ptr, a->w1.ptr, a->hidden.ptr, rows, a->d_ff, a->d_model,
                      a->d_model, a->d_ff, a->d_ff, 1.f, 0.f, 2u, off, a->groups, a->experts_cycle, a->experts_cycle);
    if (st == FE2O3_OK)
        st = gemm_tc_plan(ctx, &p->gemm[1], a->hidden.ptr, a->w2.ptr, a->compact_output.ptr, rows, a->d_model, a->d_ff,
                          a->d_ff, a->d_model, a->d_model, 1.f, 0.f, 0u, off, a->groups, a->experts_cycle,
                          a->experts_cycle);
    if (st != FE2O3_OK) return fail_prepare(out, st);
    gemm_tc_geometry(&p->gemm[0], &p->geo);
    p->geo.launches = 2;
    return FE2O3_OK;
}

int32_t fe2o3_moe_ep_ffn_v1_check(const fe2o3_moe_ep_ffn_v1_args *args) { return check_op(OP_MOE_EP_FFN, args); }
int32_t fe2o3_moe_ep_ffn_v1_prepare(fe2o3_ctx *ctx, const fe2o3_moe_ep_ffn_v1_args *a, fe2o3_prepared **out) {
    int32_t st = prepare_common(ctx, OP_MOE_EP_FFN, a, out);
    if (st != FE2O3_OK) return st;
    fe2o3_prepared *p = *out;
    const uint32_t W = a->world, per = a->experts / W;
    uint32_t *flags = reinterpret_cast<uint32_t *>(a->flags.ptr);
    GemmEp ep{};
    ep.pair_offsets = reinterpret_cast<const uint32_t *>(a->pair_offsets.ptr);
    ep.world = W;
    ep.rank = a->rank;
    ep.epoch_counter = a->epoch_counter.len ? reinterpret_cast<const uint32_t *>(a->epoch_counter.ptr) : nullptr;
    ep.epoch = a->epoch;
    ep.spin_limit = a->spin_limit ? a->spin_limit : FE2O3_EP_DEFAULT_SPIN;
    ep.trace_flags = flags;
    const bool handover = a->progress.len != 0;
    uint32_t *progress = reinterpret_cast<uint32_t *>(a->progress.ptr);
    // first GEMM: waits per source for "rows complete"; GELU + bf16 hidden rows
    GemmEp in = ep;
    if (handover) {
        in.progress = progress;
        in.progress_mode = 1;
        in.progress_len = (uint32_t)(a->progress.len / 2);
    }
    in.rows_flags = flags + FE2O3_EP_FLAG_ROWS(W);
    in.table_flag = flags + FE2O3_EP_FLAG_TABLE(W);
    st = gemm_tc_plan(ctx, &p->gemm[0], a->recv_x.ptr, a->w1.ptr, a->hidden.ptr, a->max_rows, a->d_ff, a->d_model,
                      a->d_model, a->d_ff, a->d_ff, 1.f, 0.f, EPI_GELU_BF16, in.pair_offsets, per, 0, per, &in, 2u * a->tokens);
    // second GEMM: every output row goes to its home rank's return buffer; the last CTA raises "outputs ready"
    GemmEp outp = ep;
    outp.row_meta = reinterpret_cast<const uint2 *>(a->recv_meta.ptr);
    outp.peer_ret = reinterpret_cast<const uint64_t *>(a->peer_ret.ptr);
    outp.ret_rows = 2u * a->tokens;
    outp.peer_flags = reinterpret_cast<const uint64_t *>(a->peer_flags.ptr);
    outp.done_counter = flags + FE2O3_EP_COUNTER_FFN(W);
    if (handover) {
        outp.progress = progress;
        outp.progress_mode = 2;
        outp.table_flag = flags + FE2O3_EP_FLAG_TABLE(W);   // started early, it may run ahead of the dispatch kernel too
        outp.progress_len = (uint32_t)(a->progress.len / 2);
        outp.progress_target = ((a->d_ff + 255u) / 256u) * 8u;   // tiles across d_ff x epilogue warps of the first GEMM
    }
    if (st == FE2O3_OK)
        st = gemm_tc_plan(ctx, &p->gemm[1], a->hidden.ptr, a->w2.ptr, 0, a->max_rows, a->d_model, a->d_ff, a->d_ff,
                          a->d_model, a->d_model, 1.f, 0.f, EPI_SCATTER_PEER, outp.pair_offsets, per, 0, per, &outp, 2u * a->tokens);
    if (st != FE2O3_OK) return fail_prepare(out, st);
    p->gemm[0].overlap_previous = 1;   // may start beside the dispatch kernel launched just before it
    p->gemm[1].overlap_previous = handover ? 2 : 0;   // takes over SMs as the first GEMM leaves them
    gemm_tc_geometry(&p->gemm[0], &p->geo);
    p->geo.launches = 2;
    return FE2O3_OK;
}

// ---- launch ------------------------------------------------------------------------------------
int32_t fe2o3_prepared_launch(fe2o3_prepared *p, fe2o3_stream *stream) {
    if (!p || !stream) return FE2O3_ERR_INVALID_ARGUMENT;
    if (stream->ctx != p->ctx) { fe2o3_set_error("WrongContext{role=stream}"); return FE2O3_ERR_DEVICE_MISMATCH; }
    // the launch goes to the context's device whatever device the calling thread had current
    int current = -1;
    FE2O3_CUDA(cudaGetDevice(&current));
    if (current != p->ctx->device) FE2O3_CUDA(cudaSetDevice(p->ctx->device));
    return launch_prepared(p, stream->s);
}
int32_t fe2o3_prepared_launch_and_wait(fe2o3_prepared *p, fe2o3_stream *stream, uint32_t timeout_ms,
                                       uint32_t *kernel_status) {
    if (kernel_status) *kernel_status = 0;
    int32_t st = fe2o3_prepared_launch(p, stream);
    if (st != FE2O3_OK) return st;
    st = bounded_wait(stream->s, timeout_ms);
    if (st != FE2O3_OK) return st;
    uint32_t ks = 0;
    st = take_status(p->ctx, stream->s, &ks);
    if (st != FE2O3_OK) return st;
    if (kernel_status) *kernel_status = ks;
    if (ks != 0) {
        fe2o3_set_error("kernel %s reported status word %u", kOps[p->op].symbol, ks);
        return FE2O3_ERR_KERNEL_STATUS;
    }
    return FE2O3_OK;
}
int32_t fe2o3_prepared_geometry(const fe2o3_prepared *p, fe2o3_geometry *out) {
    if (!p || !out) return FE2O3_ERR_INVALID_ARGUMENT;
    *out = p->geo;
    return FE2O3_OK;
}
int32_t fe2o3_prepared_kernarg(const fe2o3_prepared *p, void *out, uint64_t *bytes) {
    if (!p || !bytes) return FE2O3_ERR_INVALID_ARGUMENT;
    const uint64_t n = kOps[p->op].kernarg_bytes;
    if (out && *bytes >= n) memcpy(out, p->kernarg, n);
    const bool ok = *bytes >= n;
    *bytes = n;
    return ok || !out ? FE2O3_OK : FE2O3_ERR_LENGTH;
}
int32_t fe2o3_prepared_patch_kernarg(fe2o3_prepared *p, uint64_t offset, const void *data, uint64_t bytes) {
    if (!p || !data) return FE2O3_ERR_INVALID_ARGUMENT;
    const uint64_t n = kOps[p->op].kernarg_bytes;
    if (offset > n || bytes > n - offset) {
        fe2o3_set_error("InvalidRegion: patch [%llu, +%llu) outside the %llu-byte block", (unsigned long long)offset,
                        (unsigned long long)bytes, (unsigned long long)n);
        return FE2O3_ERR_INVALID_REGION;
    }
    memcpy(p->kernarg + offset, data, bytes);
    return FE2O3_OK;
}
const char *fe2o3_prepared_symbol(const fe2o3_prepared *p) { return p ? kOps[p->op].symbol : ""; }
int32_t fe2o3_prepared_destroy(fe2o3_prepared *p) {
    if (!p) return FE2O3_OK;
    if (p->attn) attention_tc_free(p->attn);
    // the workspace may still be read by a launch in flight: freeing synchronises with the device (cudaFree does)
    for (void *w : p->scratch)
        if (w) cudaFree(w);
    delete p;
    return FE2O3_OK;
}
int32_t fe2o3_ctx_take_kernel_status(fe2o3_ctx *ctx, fe2o3_stream *stream, uint32_t *status) {
    if (!ctx || !stream) return FE2O3_ERR_INVALID_ARGUMENT;
    return take_status(ctx, stream->s, status);
}

// ---- runtime adapter ---------------------------------------------------------------------------
int32_t fe2o3_image_digest(uint8_t digest[32]) {
    if (!digest) return FE2O3_ERR_INVALID_ARGUMENT;
    if (!own_image_digest(digest)) {
        fe2o3_set_error("the library image could not be read back from disk");
        return FE2O3_ERR_EXECUTABLE_REJECTED;
    }
    return FE2O3_OK;
}
int32_t fe2o3_load_executable(fe2o3_ctx *ctx, const void *bytes, uint64_t len, const uint8_t digest[32],
                              fe2o3_executable **out) {
    if (!ctx || !out || !digest || (!bytes && len)) return FE2O3_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    // the digest must be the digest of the bytes presented ...
    Sha256 sha;
    sha.update(static_cast<const uint8_t *>(bytes), len);
    uint8_t got[32];
    sha.finish(got);
    if (memcmp(got, digest, 32) != 0) {
        fe2o3_set_error("ExecutableRejected: the digest is not the SHA-256 of the %llu bytes presented", (unsigned long long)len);
        return FE2O3_ERR_EXECUTABLE_REJECTED;
    }
    // ... and those bytes must be the image that will run: this library's own file
    uint8_t mine[32];
    if (!own_image_digest(mine) || memcmp(mine, digest, 32) != 0) {
        fe2o3_set_error("ExecutableRejected: the artifact is not the sm_100a image loaded in this process");
        return FE2O3_ERR_EXECUTABLE_REJECTED;
    }
    fe2o3_executable *exe = new (std::nothrow) fe2o3_executable();
    if (!exe) return FE2O3_ERR_SIZE_OVERFLOW;
    exe->ctx = ctx;
    memcpy(exe->digest, digest, 32);
    *out = exe;
    return FE2O3_OK;
}
int32_t fe2o3_observe_kernel_resources(fe2o3_executable *exe, uint32_t kernel_id, fe2o3_kernel_resources *out) {
    if (!exe || !out || kernel_id >= OP_COUNT) return FE2O3_ERR_INVALID_ARGUMENT;
    int *n;
    KernelEntry *t = kernel_table(&n);
    for (int i = 0; i < *n; ++i) {
        if (strcmp(t[i].symbol, kOps[kernel_id].symbol) != 0) continue;
        FE2O3_CUDA(cudaSetDevice(exe->ctx->device));
        cudaFuncAttributes a;
        FE2O3_CUDA(cudaFuncGetAttributes(&a, t[i].entry));
        out->registers_per_thread = (uint32_t)a.numRegs;
        out->static_shared_bytes = (uint32_t)a.sharedSizeBytes;
        out->max_dynamic_shared_bytes = (uint32_t)a.maxDynamicSharedSizeBytes;
        out->max_threads_per_block = (uint32_t)a.maxThreadsPerBlock;
        out->local_bytes_per_thread = (uint32_t)a.localSizeBytes;
        out->const_bytes = (uint32_t)a.constSizeBytes;
        return FE2O3_OK;
    }
    fe2o3_set_error("UnknownSymbol: no device function registered for %s", kOps[kernel_id].symbol);
    return FE2O3_ERR_UNKNOWN_SYMBOL;
}
int32_t fe2o3_resolve_kernel(fe2o3_executable *exe, const char *symbol, uint32_t *kernel_id, uint64_t *kernarg_bytes) {
    if (!exe || !symbol || !kernel_id) return FE2O3_ERR_INVALID_ARGUMENT;
    for (uint32_t i = 0; i < OP_COUNT; ++i) {
        if (strcmp(kOps[i].symbol, symbol) == 0) {
            *kernel_id = i;
            if (kernarg_bytes) *kernarg_bytes = kOps[i].kernarg_bytes;
            return FE2O3_OK;
        }
    }
    fe2o3_set_error("UnknownSymbol: %s", symbol);
    return FE2O3_ERR_UNKNOWN_SYMBOL;
}
int32_t fe2o3_launch_and_wait(fe2o3_executable *exe, uint32_t kernel_id, const fe2o3_geometry *geometry, const void *kernarg,
                              uint64_t kernarg_bytes, fe2o3_stream *stream, uint32_t timeout_ms, uint32_t *kernel_status) {
    if (!exe || !kernarg || !stream || kernel_id >= OP_COUNT) return FE2O3_ERR_INVALID_ARGUMENT;
    if (kernarg_bytes != kOps[kernel_id].kernarg_bytes) {
        fe2o3_set_error("Length{role=kernarg, expected=%llu, actual=%llu}",
                        (unsigned long long)kOps[kernel_id].kernarg_bytes, (unsigned long long)kernarg_bytes);
        return FE2O3_ERR_LENGTH;
    }
    fe2o3_prepared *p = nullptr;
    int32_t st;
    switch (kernel_id) {
        case OP_SCALAR_GEMM: st = fe2o3_scalar_gemm_v1_prepare(exe->ctx, (const fe2o3_scalar_gemm_v1_args *)kernarg, FE2O3_GEMM_SCHEDULE_AUTO, &p); break;
        case OP_TILED_GEMM: st = fe2o3_tiled_gemm_v1_prepare(exe->ctx, (const fe2o3_tiled_gemm_v1_args *)kernarg, FE2O3_GEMM_SCHEDULE_AUTO, &p); break;
        case OP_TILED_GEMM_GENERAL: st = fe2o3_tiled_gemm_general_v1_prepare(exe->ctx, (const fe2o3_tiled_gemm_general_v1_args *)kernarg, FE2O3_GEMM_SCHEDULE_AUTO, &p); break;
        case OP_FLASH_ATTENTION: st = fe2o3_flash_attention_v1_prepare(exe->ctx, (const fe2o3_flash_attention_v1_args *)kernarg, &p); break;
        case OP_MOE_EXPERT_FFN: st = fe2o3_moe_expert_ffn_v1_prepare(exe->ctx, (const fe2o3_moe_expert_ffn_v1_args *)kernarg, &p); break;
        case OP_MOE_COMPACT: st = fe2o3_moe_compact_v1_prepare(exe->ctx, (const fe2o3_moe_compact_v1_args *)kernarg, &p); break;
        case OP_MOE_GROUPED_FFN: st = fe2o3_moe_grouped_ffn_v1_prepare(exe->ctx, (const fe2o3_moe_grouped_ffn_v1_args *)kernarg, &p); break;
        case OP_MOE_EP_FFN: st = fe2o3_moe_ep_ffn_v1_prepare(exe->ctx, (const fe2o3_moe_ep_ffn_v1_args *)kernarg, &p); break;
        case OP_MOE_FFN_COMBINE: st = fe2o3_moe_expert_ffn_combine_v1_prepare(exe->ctx, (const fe2o3_moe_expert_ffn_combine_v1_args *)kernarg, &p); break;
        default:
            st = prepare_common(exe->ctx, kernel_id, kernarg, &p);
            if (st == FE2O3_OK) st = finish_simple(p);
    }
    if (st == FE2O3_ERR_NO_DISPATCH) return FE2O3_OK;
    if (st != FE2O3_OK) return st;
    if (geometry) {
        // the caller's launch geometry must be the one this argument block plans to (the launch is rejected
        // before anything is submitted, like every other adapter failure)
        const fe2o3_geometry &g = p->geo;
        if (memcmp(geometry->grid, g.grid, sizeof g.grid) != 0 || memcmp(geometry->workgroup, g.workgroup, sizeof g.workgroup) != 0 ||
            geometry->dynamic_shared_bytes != g.dynamic_shared_bytes) {
            fe2o3_set_error("GeometryMismatch: caller grid %ux%ux%u block %ux%ux%u shared %u, plan grid %ux%ux%u block %ux%ux%u shared %u",
                            geometry->grid[0], geometry->grid[1], geometry->grid[2], geometry->workgroup[0], geometry->workgroup[1],
                            geometry->workgroup[2], geometry->dynamic_shared_bytes, g.grid[0], g.grid[1], g.grid[2],
                            g.workgroup[0], g.workgroup[1], g.workgroup[2], g.dynamic_shared_bytes);
            fe2o3_prepared_destroy(p);
            return FE2O3_ERR_INVALID_ARGUMENT;
        }
    }
    st = fe2o3_prepared_launch_and_wait(p, stream, timeout_ms, kernel_status);
    fe2o3_prepared_destroy(p);
    return st;
}
int32_t fe2o3_unload_executable(fe2o3_executable *exe) {
    delete exe;
    return FE2O3_OK;
}

}  // extern "C"
