"""Host-side logic that needs no GPU: the library loads, exports every symbol
the header declares, argument blocks have the reference's explicit kernarg
sizes, and the pure-host admission checks return the reference's error classes
(crates/fe2o3-host/src/generated_flash_attention_v1.rs:223-325).
"""
import ctypes as C
import os
import re

import numpy as np
import pytest

import fe2o3_b200 as fe
from fe2o3_b200 import _lib, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "fe2o3_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fe2o3_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = header_functions()
    assert len(names) > 80
    for n in names:
        assert hasattr(_lib.lib, n), n
    assert set(names) == set(_lib.EXPORTS)


def test_kernarg_block_sizes_match_the_reference_layout():
    # 16 bytes per slice, scalars after (generated_flash_attention_v1.rs:319-324);
    # general GEMM 80 bytes (hardware-harness/src/lib.rs:578-593); wave64 72
    # (generated_wave64_collectives_v1.rs:20); scoped atomic 40; MoE routing 128 + scalars.
    for op, (cls, nbytes, _) in _lib.OPS.items():
        assert C.sizeof(cls) == nbytes, op
    g = _lib.TiledGemmGeneralArgs
    assert [getattr(g, f).offset for f in ("m", "n", "k", "lda", "ldb", "ldc", "alpha", "beta")] == list(range(48, 80, 4))
    assert _lib.Wave64CollectivesArgs.active_mask.offset == 16
    assert _lib.MoeTop2Args.tokens.offset == 128


def err(op, **kw):
    with pytest.raises(fe.Fe2o3Error) as e:
        fe.check_args(op, fe.make_args(op, **kw))
    return e.value.name


BASE = 0x7F0000000000


def sl(off, n):
    return (BASE + off, n)


def test_gemm_admission_matches_the_planner():
    ok = fe.make_args("tiled_gemm_v1", a=sl(0, 256), b=sl(4096, 256), c=sl(8192, 256), m=16, n=16, k=16)
    fe.check_args("tiled_gemm_v1", ok)
    # tails are rejected by the fixed-tile planner (contract.rs:387-427) ...
    assert err("tiled_gemm_v1", a=sl(0, 17 * 16), b=sl(4096, 256), c=sl(8192, 17 * 16), m=17, n=16, k=16) == "UnsupportedShape"
    # ... and admitted by the general kernel with storage extent (rows-1)*ld + cols
    fe.check_args("tiled_gemm_general_v1", fe.make_args("tiled_gemm_general_v1", a=sl(0, 18), b=sl(4096, 17),
                                                        c=sl(8192, 10), m=3, n=2, k=4, lda=7, ldb=5, ldc=4,
                                                        alpha=1.0, beta=0.0))
    assert err("tiled_gemm_general_v1", a=sl(0, 18), b=sl(4096, 17), c=sl(8192, 10), m=3, n=2, k=4, lda=3, ldb=5,
               ldc=4) == "UnsupportedShape"  # StrideTooSmall
    assert err("tiled_gemm_general_v1", a=sl(0, 17), b=sl(4096, 17), c=sl(8192, 10), m=3, n=2, k=4, lda=7, ldb=5,
               ldc=4) == "Length"
    # zero-K: A and B are empty, C still has its extent (tests/numerical_contract.rs:31-48)
    fe.check_args("tiled_gemm_general_v1", fe.make_args("tiled_gemm_general_v1", a=(0, 0), b=(0, 0), c=sl(0, 8), m=2,
                                                        n=3, k=0, lda=0, ldb=3, ldc=5))
    # empty output: nothing is dispatched and operand storage is not inspected (tests/inputs_oracle.rs:253-272)
    fe.check_args("tiled_gemm_v1", fe.make_args("tiled_gemm_v1", a=sl(0, 1), b=sl(4096, 1), c=(0, 0), m=0, n=16, k=16))
    assert err("scalar_gemm_v1", a=sl(0, 6), b=sl(4096, 6), c=sl(8, 4), m=2, n=2, k=3) == "OutputAliasesInput"
    assert err("scalar_gemm_v1", a=(0, 6), b=sl(4096, 6), c=sl(8192, 4), m=2, n=2, k=3) == "NullAddress"
    assert err("scalar_gemm_v1", a=(BASE + 2, 6), b=sl(4096, 6), c=sl(8192, 4), m=2, n=2, k=3) == "Alignment"


def test_attention_softmax_moe_reduction_admission():
    n = 128
    fe.check_args("flash_attention_v1", fe.make_args("flash_attention_v1", q=sl(0, n), k=sl(4096, n), v=sl(8192, n),
                                                     output=sl(12288, n), batch=1, heads=1, seq=8, dim=16,
                                                     scale=0.25, causal=1, input_dtype=fe.DTYPE_F32))
    assert err("flash_attention_v1", q=sl(0, n), k=sl(4096, n), v=sl(8192, n - 1), output=sl(12288, n), batch=1,
               heads=1, seq=8, dim=16, scale=0.25, causal=1) == "Length"
    assert err("flash_attention_v1", q=sl(0, n), k=sl(4096, n), v=sl(8192, n), output=sl(8192 + 256, n), batch=1,
               heads=1, seq=8, dim=16, scale=0.25, causal=1) == "OutputAliasesInput"
    fe.check_args("row_softmax_v1", fe.make_args("row_softmax_v1", input=sl(0, 64), output=sl(4096, 64), rows=1, cols=64))
    assert err("row_softmax_v1", input=sl(0, 4097), output=sl(1 << 20, 4097), rows=1, cols=4097) == "UnsupportedShape"
    assert err("row_softmax_v1", input=sl(0, 0), output=sl(4096, 0), rows=1, cols=0) == "UnsupportedShape"
    assert err("row_softmax_v1", input=sl(0, 64), output=sl(4096, 64), mask=sl(8192, 63), rows=1, cols=64) == "Length"
    R = 16
    kw = dict(logits=sl(0, 32), top2_experts=sl(4096, R), requested_counts=sl(8192, 4), admitted_counts=sl(8448, 4),
              expert_offsets=sl(8704, 5), route_slots=sl(12288, R), permutation=sl(16384, R), inverse=sl(20480, R),
              tokens=8, experts=4, capacity=4)
    fe.check_args("moe_top2_v1", fe.make_args("moe_top2_v1", **kw))
    assert err("moe_top2_v1", **{**kw, "expert_offsets": sl(8704, 4)}) == "Length"
    assert err("moe_top2_v1", **{**kw, "inverse": sl(16384 + 4, R)}) == "OutputAliasesInput"
    assert err("moe_top2_v1", **{**kw, "experts": 1, "logits": sl(0, 8)}) == "UnsupportedShape"
    fe.check_args("masked_reduce_u32", fe.make_args("masked_reduce_u32", values=sl(0, 1000), active=sl(1 << 20, 1000),
                                                    output=sl(1 << 21, 1)))
    assert err("masked_reduce_u32", values=sl(0, 1000), active=sl(1 << 20, 999), output=sl(1 << 21, 1)) == "Length"
    assert err("masked_reduce_u32", values=sl(0, 1000), active=sl(1 << 20, 1000), output=sl(1 << 21, 2)) == "Length"
    assert err("masked_reduce_u32_packed", values=sl(0, 130), mask=sl(1 << 20, 2), output=sl(1 << 21, 1)) == "Length"
    assert err("wave_lds_v1", values=sl(0, 100), active=sl(4096, 100), wave_out=sl(8192, 100),
               workgroup_out=sl(12288, 100)) == "UnsupportedShape"
    assert err("wave64_collectives_v1", input=sl(0, 63), active_mask=1, reduction_output=sl(4096, 64),
               inclusive_output=sl(8192, 64), exclusive_output=sl(12288, 64)) == "Length"
    assert err("moe_expert_combine_v1", compact_output=sl(0, 16 * 16), inverse=sl(1 << 20, 16),
               route_weights=sl(1 << 21, 16), combined_output=sl(512, 8 * 16), tokens=8, width=16) == "OutputAliasesInput"
    # expert FFN with the combine folded in: rows = permutation.len, d_model in whole 64-column blocks
    T, d, f, E = 8, 64, 16, 2
    fk = dict(x=sl(0, T * d), w1=sl(1 << 20, E * d * f), w2=sl(2 << 20, E * f * d), permutation=sl(3 << 20, 2 * T),
              expert_offsets=sl(4 << 20, E + 1), route_weights=sl(5 << 20, 2 * T), hidden=sl(6 << 20, 2 * T * f),
              combined_output=sl(7 << 20, T * d), tokens=T, d_model=d, d_ff=f, experts=E)
    fe.check_args("moe_expert_ffn_combine_v1", fe.make_args("moe_expert_ffn_combine_v1", **fk))
    assert err("moe_expert_ffn_combine_v1", **{**fk, "d_model": 72, "x": sl(0, T * 72), "w1": sl(1 << 20, E * 72 * f),
                                                "w2": sl(2 << 20, E * f * 72), "combined_output": sl(7 << 20, T * 72)}) == "UnsupportedShape"
    assert err("moe_expert_ffn_combine_v1", **{**fk, "route_weights": sl(5 << 20, 2 * T - 1)}) == "Length"
    assert err("moe_expert_ffn_combine_v1", **{**fk, "hidden": sl(6 << 20, 2 * T * f + 1)}) == "Length"
    assert err("moe_expert_ffn_combine_v1", **{**fk, "combined_output": sl(64, T * d)}) == "OutputAliasesInput"
    # u64 overflow of a region is a RegionOverflow, not a wrap-around
    assert err("masked_reduce_u32", values=(BASE, 1 << 63), active=(BASE, 1 << 63), output=sl(0, 1)) == "InvalidRegion"


def test_no_device_is_reported_not_faked():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(fe.Fe2o3Error) as e:
        fe.GpuContext(0)
    assert e.value.name == "NoDevice"


def test_synthetic_generators_are_deterministic_and_match_the_reference_recipe(orc):
    a, b = synth.gemm_inputs_v1(2, 3, 2, 0x1234)  # examples/tiled_gemm_v1/tests/inputs_oracle.rs:29-40
    assert list(a) == [0x0000, 0x4080, 0xBD80, 0x4040] and list(b) == [0xBE80, 0x4040, 0x4040, 0x3E80, 0x4080, 0x3E00]
    oa, ob = orc.gemm_inputs_v1(16, 32, 48, 99)
    sa, sb = synth.gemm_inputs_v1(16, 32, 48, 99)
    assert (oa == sa).all() and (ob == sb).all()
    u = synth.uniform_f32(0, 1, 1 << 16)
    assert u.min() >= -1 and u.max() < 1 and abs(float(u.mean())) < 0.02
    assert (u == synth.uniform_f32(0, 1, 1 << 16)).all() and not (u == synth.uniform_f32(0, 2, 1 << 16)).all()
    assert (u[:100] == synth.uniform_f32(0, 1, 100)).all()  # element i does not depend on n
    g = synth.normal_f32(2, 1, 1 << 16, 2.0)
    assert abs(float(g.mean())) < 0.05 and abs(float(g.std()) - 2.0) < 0.05
    v = synth.u32_below(1, 1, 1 << 16, 1 << 16)
    assert v.max() < (1 << 16) and v.min() >= 0
    f, m = synth.bernoulli(1, 2, 1000, 0.75)
    assert set(np.unique(f)) <= {0, 7} and abs((f != 0).mean() - 0.75) < 0.05
    bits = np.unpackbits(m.view(np.uint8), bitorder="little")[:1000]
    assert (bits == (f != 0)).all()
    x = synth.normal_bf16(4, 3, 4096, 1.0)
    assert (x == orc.bf16_from_f32(synth.normal_f32(4, 3, 4096, 1.0))).all()
    assert _lib.lib.fe2o3_bf16_from_f32(1.0) == 0x3F80


def test_image_digest_is_sha256_of_the_library_file():
    """load_executable(bytes, digest) compares the presented digest with the SHA-256 of the library's own
    file, computed by the library (no CUDA call): it must agree with an independent SHA-256."""
    import ctypes as C
    import hashlib
    from fe2o3_b200._lib import LIB_PATH, lib
    out = (C.c_uint8 * 32)()
    assert lib.fe2o3_image_digest(out) == 0
    assert bytes(out) == hashlib.sha256(open(LIB_PATH, "rb").read()).digest()
