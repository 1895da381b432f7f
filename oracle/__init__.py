"""ctypes binding of the CPU oracle (TEST INFRASTRUCTURE, not product).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module.  Every function is a thin numpy wrapper over `fe2o3_oracle.c`, whose
header lists the reference files each routine restates.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libfe2o3_oracle.so")
DROP_ROUTE = 0xFFFFFFFF


def build(force=False):
    src = os.path.join(_HERE, "fe2o3_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libfe2o3_oracle.so"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.orc_mix64.restype = C.c_uint64
        _lib.orc_mix64.argtypes = [C.c_uint64]
        _lib.orc_fnv1a_append.restype = C.c_uint64
        _lib.orc_fnv1a_append.argtypes = [C.c_uint64, C.c_void_p, C.c_uint64]
        _lib.orc_masked_sum_u32.restype = C.c_uint32
        _lib.orc_masked_sum_u32_parallel.restype = C.c_uint32
        _lib.orc_masked_sum_u32_packed.restype = C.c_uint32
        _lib.orc_row_softmax_compare.restype = C.c_int64
        _lib.orc_bf16_from_f32.restype = C.c_uint16
        _lib.orc_bf16_from_f32.argtypes = [C.c_float]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


u64, f32c, f64c, i32c = C.c_uint64, C.c_float, C.c_double, C.c_int


def set_threads(n):
    lib().orc_set_threads(C.c_int(int(n)))
    return int(lib().orc_get_max_threads())


def synth_normal_bf16(seed, domain, n, sigma):
    """The benchmark's N(0, sigma^2) bf16 stream (same bytes as fe2o3_b200.synth.normal_bf16)."""
    out = np.empty(n, np.uint16)
    lib().orc_synth_normal_bf16(u64(seed), u64(domain), u64(n), f32c(sigma), _p(out))
    return out


def synth_u32_below(seed, domain, n, bound):
    out = np.empty(n, np.uint32)
    lib().orc_synth_u32_below(u64(seed), u64(domain), u64(n), C.c_uint32(bound), _p(out))
    return out


def synth_bernoulli_flags(seed, domain, n, p, flag_value=7):
    out = np.empty(n, np.uint32)
    lib().orc_synth_bernoulli_flags(u64(seed), u64(domain), u64(n), f64c(p), C.c_uint32(flag_value), _p(out))
    return out


def mix64(v):
    return lib().orc_mix64(v & 0xFFFFFFFFFFFFFFFF)


def bf16_from_f32(x):
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_bf16_from_f32_array(_p(x), _p(out), u64(x.size))
    return out


def bf16_to_f32(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def gemm_inputs_v1(m, n, k, seed):
    a = np.empty(m * k, np.uint16)
    b = np.empty(k * n, np.uint16)
    lib().orc_gemm_inputs_v1(C.c_uint32(m), C.c_uint32(n), C.c_uint32(k), u64(seed), _p(a), _p(b))
    return a, b


def gemm_bf16(m, n, k, a_bits, b_bits, lda=None, ldb=None, ldc=None, alpha=1.0, beta=0.0,
              c=None, epilogue=None):
    lda = k if lda is None else lda
    ldb = n if ldb is None else ldb
    ldc = n if ldc is None else ldc
    a_bits = _c(a_bits, np.uint16)
    b_bits = _c(b_bits, np.uint16)
    if epilogue is None:
        epilogue = c is not None
    cin = _c(c, np.float32) if c is not None else np.zeros(max(1, (m - 1) * ldc + n if m else 0), np.float32)
    out = np.empty(m * n, np.float32)
    lib().orc_gemm_bf16(u64(m), u64(n), u64(k), u64(lda), u64(ldb), u64(ldc), f32c(alpha), f32c(beta),
                        _p(a_bits), _p(b_bits), _p(cin), _p(out), i32c(1 if epilogue else 0))
    return out


def gemm_f32(m, n, k, a, b, fast=False):
    a = _c(a, np.float32)
    b = _c(b, np.float32)
    out = np.empty(m * n, np.float32)
    fn = lib().orc_gemm_f32_rows if fast else lib().orc_gemm_f32
    fn(u64(m), u64(n), u64(k), _p(a), _p(b), _p(out))
    return out


def gemm_bf16_rows(m, n, k, a_bits, b_bits):
    a_bits = _c(a_bits, np.uint16)
    b_bits = _c(b_bits, np.uint16)
    out = np.empty(m * n, np.float32)
    st = lib().orc_gemm_bf16_rows(u64(m), u64(n), u64(k), _p(a_bits), _p(b_bits), _p(out))
    assert st == 0
    return out


def fnv1a(h, data: bytes):
    buf = (C.c_uint8 * len(data)).from_buffer_copy(data) if data else None
    return lib().orc_fnv1a_append(u64(h), buf, u64(len(data)))


def row_softmax(x, mask=None):
    """Batched oracle over the last axis; returns (status, out)."""
    x = _c(x, np.float32)
    x2 = x.reshape(-1, x.shape[-1]) if x.ndim > 1 else x.reshape(1, -1)
    m = None if mask is None else _c(np.asarray(mask).reshape(x2.shape), np.uint8)
    out = np.full(x2.shape, np.nan, np.float32)
    st = lib().orc_row_softmax_batch(_p(x2), _p(m), u64(x2.shape[0]), u64(x2.shape[1]), _p(out))
    return st, out.reshape(x.shape)


def row_softmax_kernel_f32(x):
    x = _c(x, np.float32)
    out = np.empty_like(x)
    lib().orc_row_softmax_kernel_f32(_p(x), u64(x.size), _p(out))
    return out


def row_softmax_compare(expected, actual, mask=None, abs_tol=3.0e-6, rel_tol=3.0e-5, sum_tol=6.0e-5,
                        max_ulps=64):
    e = _c(expected, np.float32)
    a = _c(actual, np.float32)
    m = None if mask is None else _c(mask, np.uint8)
    return lib().orc_row_softmax_compare(_p(e), _p(a), _p(m), u64(e.size), f32c(abs_tol), f32c(rel_tol),
                                         f32c(sum_tol), C.c_uint32(max_ulps))


def flash_attention(q, k, v, scale, causal, online_f32=False):
    """q,k,v: float32 arrays [B,H,S,D] (widen bf16 first)."""
    q = _c(q, np.float32)
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    B, H, S, D = q.shape
    out = np.empty_like(q)
    if online_f32:
        st = lib().orc_flash_attention_online_f32(_p(q), _p(k), _p(v), _p(out), u64(B), u64(H), u64(S), u64(D),
                                                  f32c(scale), i32c(int(causal)))
    else:
        st = lib().orc_flash_attention_f64(_p(q), _p(k), _p(v), _p(out), u64(B), u64(H), u64(S), u64(D),
                                           f64c(scale), i32c(int(causal)))
    return st, out


def moe_top2_route(logits, tokens, experts, capacity, independent=False):
    lg = _c(logits, np.float32)
    R = tokens * 2
    o = dict(top2_experts=np.zeros(R, np.uint32), requested_counts=np.zeros(experts, np.uint32),
             admitted_counts=np.zeros(experts, np.uint32), expert_offsets=np.zeros(experts + 1, np.uint32),
             route_slots=np.zeros(R, np.uint32), permutation=np.zeros(R, np.uint32),
             inverse=np.zeros(R, np.uint32))
    st = lib().orc_moe_top2_route(_p(lg), u64(tokens), u64(experts), C.c_uint32(capacity),
                                  i32c(int(independent)), *[_p(o[k]) for k in
                                                            ("top2_experts", "requested_counts",
                                                             "admitted_counts", "expert_offsets",
                                                             "route_slots", "permutation", "inverse")])
    return st, o


def moe_validate_routing(logits, tokens, experts, capacity, o):
    lg = _c(logits, np.float32)
    arrs = [_c(o[k], np.uint32) for k in ("top2_experts", "requested_counts", "admitted_counts",
                                           "expert_offsets", "route_slots", "permutation", "inverse")]
    return lib().orc_moe_validate_routing(_p(lg), u64(tokens), u64(experts), C.c_uint32(capacity),
                                          *[_p(a) for a in arrs])


def moe_gate_logits(x_bits, wg_bits, tokens, d_model, experts):
    x = _c(x_bits, np.uint16)
    w = _c(wg_bits, np.uint16)
    out = np.empty(tokens * experts, np.float32)
    lib().orc_moe_gate_logits(_p(x), _p(w), u64(tokens), u64(d_model), u64(experts), _p(out))
    return out


def moe_route_weights(logits, top2, tokens, experts):
    lg = _c(logits, np.float32)
    t2 = _c(top2, np.uint32)
    out = np.empty(tokens * 2, np.float32)
    lib().orc_moe_route_weights(_p(lg), _p(t2), u64(tokens), u64(experts), _p(out))
    return out


def moe_expert_ffn(x_bits, w1_bits, w2_bits, top2, inverse, tokens, d_model, d_ff, experts, compact_rows=None):
    x = _c(x_bits, np.uint16)
    w1 = _c(w1_bits, np.uint16)
    w2 = _c(w2_bits, np.uint16)
    t2 = _c(top2, np.uint32)
    inv = _c(inverse, np.uint32)
    rows = tokens * 2 if compact_rows is None else compact_rows
    out = np.zeros(rows * d_model, np.float32)
    lib().orc_moe_expert_ffn(_p(x), _p(w1), _p(w2), _p(t2), _p(inv), u64(tokens), u64(d_model), u64(d_ff),
                             u64(experts), _p(out))
    return out


def moe_combine(compact, inverse, weights, tokens, width):
    cp = _c(compact, np.float32)
    inv = _c(inverse, np.uint32)
    w = _c(weights, np.float32)
    out = np.empty(tokens * width, np.float32)
    st = lib().orc_moe_combine(_p(cp), _p(inv), _p(w), u64(tokens), u64(width), u64(cp.size // width), _p(out))
    return st, out


def masked_sum_u32(values, active, parallel=True):
    v = _c(values, np.uint32)
    a = _c(active, np.uint32)
    fn = lib().orc_masked_sum_u32_parallel if parallel else lib().orc_masked_sum_u32
    return int(fn(_p(v), _p(a), u64(v.size)))


def scan_sum_u32(values, exclusive=False):
    v = _c(values, np.uint32)
    out = np.empty_like(v)
    lib().orc_scan_sum_u32(_p(v), u64(v.size), C.c_uint32(1 if exclusive else 0), _p(out))
    return out


def scan_sum_f32(values, exclusive=False):
    """Prefix sums of binary32 values accumulated in binary64 (the exact sum to about 2^-53 per step), and the
    prefix sums of their magnitudes, which scale the tolerance of a binary32 scan.  The wave-scope definition it
    extends is crates/fe2o3-device/src/collective.rs:413-460; at array scope the reference fixes no order, so
    parity is by tolerance against this."""
    v = _c(values, np.float32).astype(np.float64)
    inc, mag = np.cumsum(v), np.cumsum(np.abs(v))
    if exclusive:
        inc = np.concatenate(([0.0], inc[:-1])) if v.size else inc
        mag = np.concatenate(([0.0], mag[:-1])) if v.size else mag
    return inc, mag


def masked_sum_u32_packed(values, mask):
    v = _c(values, np.uint32)
    m = _c(mask, np.uint64)
    return int(lib().orc_masked_sum_u32_packed(_p(v), _p(m), u64(v.size)))


def wave_workgroup_sums_u32(values, active):
    v = _c(values, np.uint32)
    a = _c(active, np.uint32)
    w = np.empty_like(v)
    g = np.empty_like(v)
    st = lib().orc_wave_workgroup_sums_u32(_p(v), _p(a), u64(v.size), _p(w), _p(g))
    return st, w, g


def wave64_collectives_f32(x, masks):
    x = _c(x, np.float32)
    m = _c(np.atleast_1d(masks), np.uint64)
    r, i, e = (np.full(x.shape, np.nan, np.float32) for _ in range(3))
    st = lib().orc_wave64_collectives_f32(_p(x), _p(m), u64(m.size), _p(r), _p(i), _p(e))
    return st, r, i, e


def workgroup_reduce_i32(values):
    v = _c(values, np.int32)
    out = C.c_int32(0)
    st = lib().orc_workgroup_reduce_i32(_p(v), u64(v.size), C.byref(out))
    return st, out.value


def scoped_atomic_add_u32(values, eligible, initial):
    v = _c(values, np.uint32)
    e = _c(eligible, np.uint32)
    out = C.c_uint32(0)
    st = lib().orc_scoped_atomic_add_u32(_p(v), _p(e), u64(v.size), C.c_uint32(initial), C.byref(out))
    return st, out.value
