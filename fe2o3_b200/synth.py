"""Deterministic synthetic inputs (host side), via the library's SplitMix64-keyed
generators: element i of stream (seed, domain) depends only on (seed, domain, i).
"""
import ctypes as C

import numpy as np

from ._lib import check, lib

u64 = C.c_uint64


def _out(n, dtype, out):
    if out is None:
        out = np.empty(n, dtype)
    assert out.dtype == np.dtype(dtype) and out.size == n and out.flags.c_contiguous
    return out


def uniform_f32(seed, domain, n, out=None):
    out = _out(n, np.float32, out)
    check(lib.fe2o3_synth_uniform_f32(u64(seed), u64(domain), u64(n), out.ctypes.data_as(C.c_void_p)))
    return out


def uniform_bf16(seed, domain, n, out=None):
    out = _out(n, np.uint16, out)
    check(lib.fe2o3_synth_uniform_bf16(u64(seed), u64(domain), u64(n), out.ctypes.data_as(C.c_void_p)))
    return out


def normal_f32(seed, domain, n, sigma, out=None):
    out = _out(n, np.float32, out)
    check(lib.fe2o3_synth_normal_f32(u64(seed), u64(domain), u64(n), C.c_float(sigma), out.ctypes.data_as(C.c_void_p)))
    return out


def normal_bf16(seed, domain, n, sigma, out=None):
    out = _out(n, np.uint16, out)
    check(lib.fe2o3_synth_normal_bf16(u64(seed), u64(domain), u64(n), C.c_float(sigma), out.ctypes.data_as(C.c_void_p)))
    return out


def u32_below(seed, domain, n, bound, out=None):
    out = _out(n, np.uint32, out)
    check(lib.fe2o3_synth_u32_below(u64(seed), u64(domain), u64(n), C.c_uint32(bound), out.ctypes.data_as(C.c_void_p)))
    return out


def bernoulli(seed, domain, n, p, flag_value=7, flags=True, packed=True, flags_out=None, packed_out=None):
    f = _out(n, np.uint32, flags_out) if flags else None
    m = _out((n + 63) // 64, np.uint64, packed_out) if packed else None
    check(lib.fe2o3_synth_bernoulli(u64(seed), u64(domain), u64(n), C.c_double(p), C.c_uint32(flag_value),
                                    f.ctypes.data_as(C.c_void_p) if f is not None else None,
                                    m.ctypes.data_as(C.c_void_p) if m is not None else None))
    return f, m


def gemm_inputs_v1(m, n, k, seed):
    a = np.empty(m * k, np.uint16)
    b = np.empty(k * n, np.uint16)
    check(lib.fe2o3_synth_gemm_inputs_v1(C.c_uint32(m), C.c_uint32(n), C.c_uint32(k), u64(seed),
                                         a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p)))
    return a, b


def bf16_to_f32(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)
