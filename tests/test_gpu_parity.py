"""GPU parity: every kernel, called through the C ABI, against the CPU oracle on
the same seeded inputs.  Integer and index results are compared bit-for-bit;
floating point within the tolerance written at each comparison.  Guard
canaries surround every device allocation and inputs are checked unchanged,
as the reference's hardware tests do
(examples/tiled_gemm_general_v1/hardware-harness/src/lib.rs:48,1629-1638).
"""
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GUARD = 32


@pytest.fixture(scope="module")
def gpu():
    import fe2o3_b200 as fe
    ctx = fe.GpuContext(0)
    return fe, ctx, ctx.default_stream()


class Guarded:
    """Device array with 32 canary elements on both sides."""

    def __init__(self, fe, stream, array, canary=0xA5):
        a = np.ascontiguousarray(array)
        self.n, self.dtype = a.size, a.dtype
        pad = np.full(GUARD * a.dtype.itemsize, canary, np.uint8).view(a.dtype)
        self.host = np.concatenate([pad, a.ravel(), pad])
        self.buf = fe.DeviceBuffer.from_host(stream, self.host)
        self.stream = stream
        self.pad = pad

    @property
    def slice(self):
        return self.buf.view(GUARD, self.n)

    def read(self):
        full = self.buf.to_host_vec(self.stream)
        assert full[:GUARD].tobytes() == self.pad.tobytes(), "front canary overwritten"
        assert full[GUARD + self.n:].tobytes() == self.pad.tobytes(), "back canary overwritten"
        return full[GUARD:GUARD + self.n]

    def unchanged(self):
        assert self.read().tobytes() == self.host[GUARD:GUARD + self.n].tobytes(), "input was modified"


def bits(x):
    return np.asarray(x, np.float32).view(np.uint32)


def assert_close(got, want, rel, abs_frac, what=""):
    """The reference's bounded policy, |a - e| <= abs + rel * |e|
    (examples/tiled_gemm_v1/src/numerical_contract.rs:958-966), with the absolute
    term stated as a fraction of the largest expected magnitude."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.isfinite(got).all(), what
    limit = abs_frac * np.abs(want).max() + rel * np.abs(want)
    excess = np.abs(got - want) - limit
    assert excess.max() <= 0, (what, float(np.abs(got - want).max()), float(np.abs(want).max()))


def run(fe, ctx, stream, op, schedule=None, **kw):
    p = fe.prepare(ctx, op, **({"schedule": schedule} if schedule is not None else {}), **kw)
    if p is None:
        return None
    p.launch_and_wait(stream, 20000)
    return p


# ---------------------------------------------------------------- reductions

@pytest.mark.parametrize("n", [0, 1, 3, 255, 256, 1000, 4099, (1 << 20) + 5, 1 << 24])
def test_masked_reduce_u32_bit_exact(gpu, orc, n):
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    values = synth.u32_below(1, 1, n, 1 << 16) if n else np.zeros(0, np.uint32)
    if n >= 1000:
        values[::7] = 0xFFFFFFF1  # force wrap-around
    flags, packed = synth.bernoulli(1, 2, n, 0.75) if n else (np.zeros(0, np.uint32), np.zeros(0, np.uint64))
    v, a, m = Guarded(fe, stream, values), Guarded(fe, stream, flags), Guarded(fe, stream, packed)
    out = Guarded(fe, stream, np.full(1, 0xDEADBEEF, np.uint32))
    for _ in range(2):  # second launch checks that the arrival counter re-arms
        run(fe, ctx, stream, "masked_reduce_u32", values=v.slice, active=a.slice, output=out.slice)
        assert int(out.read()[0]) == orc.masked_sum_u32(values, flags)
    out2 = Guarded(fe, stream, np.full(1, 0xDEADBEEF, np.uint32))
    run(fe, ctx, stream, "masked_reduce_u32_packed", values=v.slice, mask=m.slice, output=out2.slice)
    assert int(out2.read()[0]) == orc.masked_sum_u32_packed(values, packed) == orc.masked_sum_u32(values, flags)
    v.unchanged(); a.unchanged(); m.unchanged()


def test_masked_reduce_unaligned_views(gpu, orc):
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    n = 70001
    values, (flags, _) = synth.u32_below(1, 3, n + 3, 1 << 16), synth.bernoulli(1, 4, n + 3, 0.75, packed=False)
    v, a = fe.DeviceBuffer.from_host(stream, values), fe.DeviceBuffer.from_host(stream, flags)
    out = fe.DeviceBuffer.zeroed(stream, 1, np.uint32)
    for off_v, off_a in [(1, 1), (1, 2), (0, 3)]:
        run(fe, ctx, stream, "masked_reduce_u32", values=v.view(off_v, n), active=a.view(off_a, n), output=out)
        assert int(out.to_host_vec(stream)[0]) == orc.masked_sum_u32(values[off_v:off_v + n], flags[off_a:off_a + n])


def test_wave_lds_runner_vector(gpu, orc):
    # crates/dialect-amdgcn/tests/fixtures/gfx942_wave_lds_v1_runner.cpp:26-29,76-94
    fe, ctx, stream = gpu
    for blocks in (1, 5):
        lane = np.arange(256 * blocks)
        values = (lane + 1).astype(np.uint32) * (1 if blocks == 1 else 0x01000193)
        active = np.where(lane % 3 == 1, 0, 7).astype(np.uint32)
        v, a = Guarded(fe, stream, values), Guarded(fe, stream, active)
        w = Guarded(fe, stream, np.full(values.size, 0xDEADBEEF, np.uint32))
        g = Guarded(fe, stream, np.full(values.size, 0xDEADBEEF, np.uint32))
        run(fe, ctx, stream, "wave_lds_v1", values=v.slice, active=a.slice, wave_out=w.slice, workgroup_out=g.slice)
        st, ew, eg = orc.wave_workgroup_sums_u32(values, active)
        assert st == 0 and (w.read() == ew).all() and (g.read() == eg).all()


def test_wave64_collectives_masks(gpu, orc):
    # examples/wave64_collectives_v1/tests/oracle.rs:6-98
    fe, ctx, stream = gpu
    x = ((np.arange(64) * 5 + 3) % 17).astype(np.float32) - 8
    masks = [0, (1 << 19) - 1, (1 << 0) | (1 << 3) | (1 << 8) | (1 << 34) | (1 << 63), 0xAAAAAAAAAAAAAAAA,
             0xFFFFFFFFFFFFFFFF]
    xin = Guarded(fe, stream, x)
    for mask in masks:
        outs = [Guarded(fe, stream, np.full(64, np.nan, np.float32)) for _ in range(3)]
        p = run(fe, ctx, stream, "wave64_collectives_v1", input=xin.slice, active_mask=mask,
                reduction_output=outs[0].slice, inclusive_output=outs[1].slice, exclusive_output=outs[2].slice)
        assert len(p.kernarg) == 72 and struct.unpack_from("<Q", p.kernarg, 16)[0] == mask
        _, r, i, e = orc.wave64_collectives_f32(x, mask)
        for got, want in zip(outs, (r, i, e)):
            assert (bits(got.read()) == bits(want)).all()
    rng = np.random.default_rng(7)
    segs = 37
    xs = rng.integers(-1024, 1025, segs * 64).astype(np.float32)
    ms = rng.integers(0, 1 << 63, segs, dtype=np.uint64) * 2 + rng.integers(0, 2, segs, dtype=np.uint64)
    bx, bm = Guarded(fe, stream, xs), Guarded(fe, stream, ms)
    outs = [Guarded(fe, stream, np.full(segs * 64, np.nan, np.float32)) for _ in range(3)]
    run(fe, ctx, stream, "wave64_collectives_segmented", input=bx.slice, masks=bm.slice,
        reduction_output=outs[0].slice, inclusive_output=outs[1].slice, exclusive_output=outs[2].slice)
    _, r, i, e = orc.wave64_collectives_f32(xs, ms)
    for got, want in zip(outs, (r, i, e)):
        assert (bits(got.read()) == bits(want)).all()


def test_workgroup_sync_vectors(gpu, orc):
    # examples/workgroup_sync_v1/src/vectors.rs:32-109
    fe, ctx, stream = gpu
    lane = np.arange(64)
    for values, want in [(np.zeros(64), 0), (np.where(lane % 2 == 0, 1000, -999), 32), (lane - 32, -32),
                         (np.where(lane % 11 == 0, lane * 7, 0), 1155)]:
        v = Guarded(fe, stream, values.astype(np.int32))
        o = Guarded(fe, stream, np.full(1, -7, np.int32))
        run(fe, ctx, stream, "lds_publish_read_reduce_i32_v1", values=v.slice, output=o.slice)
        assert int(o.read()[0]) == want == orc.workgroup_reduce_i32(values)[1]
    for initial, elig, want in [(17, np.zeros(64), 17), (0, np.ones(64), 2016), (11, lane % 2 == 0, 1003),
                                (1000, lane % 13 == 0, 1130)]:
        v, e = Guarded(fe, stream, lane.astype(np.uint32)), Guarded(fe, stream, elig.astype(np.uint32))
        t = Guarded(fe, stream, np.full(1, initial, np.uint32))
        p = run(fe, ctx, stream, "scoped_atomic_add_u32_v1", values=v.slice, eligible=e.slice, target=t.slice.ptr)
        assert len(p.kernarg) == 40 and int(t.read()[0]) == want


# ------------------------------------------------------------------- softmax

def softmax_case(gpu, orc, x, mask=None):
    fe, ctx, stream = gpu
    rows, cols = x.shape
    i = Guarded(fe, stream, x)
    o = Guarded(fe, stream, np.full(x.size, np.nan, np.float32))
    m = Guarded(fe, stream, mask.astype(np.uint8)) if mask is not None else None
    run(fe, ctx, stream, "row_softmax_v1", input=i.slice, output=o.slice, mask=m.slice if m else None, rows=rows,
        cols=cols)
    st, want = orc.row_softmax(x, mask)
    assert st == 0
    got = o.read().reshape(rows, cols)
    i.unchanged()
    # BASELINE tolerance: relative 1e-5 (denominator floored at 1e-30 so exact zeros compare equal)
    rel = np.abs(got - want) / np.maximum(np.abs(want), 1e-30)
    assert rel.max() <= 1e-5, rel.max()
    # and the reference's own comparator (abs 3e-6 + rel 3e-5 or 64 ulps, row sum within 6e-5)
    for r in range(0, rows, max(1, rows // 64)):
        assert orc.row_softmax_compare(want[r], got[r], None if mask is None else mask[r].astype(np.uint8)) == 0
    return got


@pytest.mark.parametrize("rows,cols", [(1, 64), (3, 1024), (257, 1024), (5, 128), (7, 260), (2, 4096), (9, 33), (4, 1)])
def test_row_softmax_shapes(gpu, orc, rows, cols):
    from fe2o3_b200 import synth
    x = synth.normal_f32(2, rows * 131 + cols, rows * cols, 2.0).reshape(rows, cols)
    softmax_case(gpu, orc, x)


def test_row_softmax_reference_pins(gpu, orc):
    # uniform row == exact 1/64 (examples/row_softmax_v1/tests/numerical_contract.rs:105-111)
    got = softmax_case(gpu, orc, np.full((1, 64), 3.25, np.float32))
    assert (bits(got) == bits(np.float32(1 / 64))).all()
    # mask policy (:46-64): masked outputs are +0.0
    from fe2o3_b200 import synth
    x = synth.normal_f32(2, 77, 6 * 1024, 2.0).reshape(6, 1024)
    mask = (synth.u32_below(2, 78, 6 * 1024, 4) != 0).reshape(6, 1024)
    got = softmax_case(gpu, orc, x, mask)
    assert (bits(got[~mask]) == 0).all()
    x = synth.normal_f32(2, 79, 3 * 100, 2.0).reshape(3, 100)
    mask = (synth.u32_below(2, 80, 300, 3) != 0).reshape(3, 100)
    softmax_case(gpu, orc, x, mask)


def test_row_softmax_nonfinite_is_reported_not_written(gpu):
    fe, ctx, stream = gpu
    x = np.ones((2, 64), np.float32)
    x[1, 5] = np.inf
    i, o = Guarded(fe, stream, x), Guarded(fe, stream, np.full(128, -1, np.float32))
    p = fe.prepare(ctx, "row_softmax_v1", input=i.slice, output=o.slice, rows=2, cols=64)
    with pytest.raises(fe.Fe2o3Error) as e:
        p.launch_and_wait(stream)
    assert e.value.name == "KernelStatus" and p.kernel_status == 2
    got = o.read()
    assert (got[64:] == -1).all() and abs(got[:64].sum() - 1) < 1e-6
    assert ctx.take_kernel_status(stream) == 0  # status word was cleared


# ---------------------------------------------------------------------- GEMM

def corpus(orc):
    from test_oracle_pins import corpus as c
    return c(orc)


def test_gemm_exact_order_matches_reference_corpus_bitwise(gpu, orc):
    # the 9-vector corpus of examples/tiled_gemm_v1/src/numerical_vectors.rs through the general kernel
    fe, ctx, stream = gpu
    for name, (m, n, k, lda, ldb, ldc), a, b, c, alpha, beta in corpus(orc):
        cin = np.array(c, np.float32)
        A, B, Cb = Guarded(fe, stream, np.array(a, np.uint16)), Guarded(fe, stream, np.array(b, np.uint16)), Guarded(fe, stream, cin)
        p = run(fe, ctx, stream, "tiled_gemm_general_v1", schedule=fe.SCHEDULE_EXACT_ORDER, a=A.slice, b=B.slice,
                c=Cb.slice, m=m, n=n, k=k, lda=lda, ldb=ldb, ldc=ldc, alpha=alpha, beta=beta)
        assert len(p.kernarg) == 80 and p.symbol == "tiled_gemm_general_v1"
        want = orc.gemm_bf16(m, n, k, a, b, lda=lda, ldb=ldb, ldc=ldc, alpha=alpha, beta=beta, c=cin)
        got = Cb.read()
        for r in range(m):
            assert (bits(got[r * ldc:r * ldc + n]) == bits(want[r * n:(r + 1) * n])).all(), name
            if ldc > n and r + 1 < m:  # padding untouched (bit compare: padding holds NaNs)
                assert (bits(got[r * ldc + n:(r + 1) * ldc]) == bits(cin[r * ldc + n:(r + 1) * ldc])).all(), name
        A.unchanged(); B.unchanged()


@pytest.mark.parametrize("m,n,k", [(16, 16, 16), (64, 48, 16), (512, 512, 512), (48, 80, 96)])
def test_tiled_gemm_v1_exact_bits_on_reference_alphabet(gpu, orc, m, n, k):
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    a, b = synth.gemm_inputs_v1(m, n, k, 0x1234)
    A, B = Guarded(fe, stream, a), Guarded(fe, stream, b)
    want = orc.gemm_bf16_rows(m, n, k, a, b)
    if m * n * k <= 1 << 18:
        assert (bits(want) == bits(orc.gemm_bf16(m, n, k, a, b))).all()
    for schedule in (fe.SCHEDULE_EXACT_ORDER, fe.SCHEDULE_TCGEN05):
        Cb = Guarded(fe, stream, np.full(m * n, np.nan, np.float32))
        run(fe, ctx, stream, "tiled_gemm_v1", schedule=schedule, a=A.slice, b=B.slice, c=Cb.slice, m=m, n=n, k=k)
        got = Cb.read()
        # dyadic alphabet (|v| <= 4, granularity 2^-4): every partial sum is exact in f32 for K <= 512, so the
        # tensor-core summation order must give the same bits as the sequential recurrence.
        assert (bits(got) == bits(want)).all(), (schedule, np.abs(got - want).max())


def test_scalar_gemm_f32_config0_bit_exact(gpu, orc):
    # BASELINE config: f32 C = A*B, M=N=K=512, uniform[-1,1) from seed 0
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    m = n = k = 512
    a, b = synth.uniform_f32(0, 1, m * k), synth.uniform_f32(0, 2, k * n)
    A, B = Guarded(fe, stream, a), Guarded(fe, stream, b)
    Cb = Guarded(fe, stream, np.full(m * n, np.nan, np.float32))
    p = run(fe, ctx, stream, "scalar_gemm_v1", a=A.slice, b=B.slice, c=Cb.slice, m=m, n=n, k=k)
    assert len(p.kernarg) == 64
    assert (bits(Cb.read()) == bits(orc.gemm_f32(m, n, k, a, b, fast=True))).all()
    # reference vectors: rectangular product and the FMA-distinguishing case (harness.rs:258-288)
    eps = np.float32(np.finfo(np.float32).eps)
    for (mm, nn, kk, aa, bb) in [(2, 3, 2, [1, 2, 3, 4], [5, 6, 7, 8, 9, 10]), (1, 1, 2, [1 + eps, 1], [1 - eps, -1])]:
        A2, B2 = Guarded(fe, stream, np.array(aa, np.float32)), Guarded(fe, stream, np.array(bb, np.float32))
        C2 = Guarded(fe, stream, np.full(mm * nn, np.nan, np.float32))
        run(fe, ctx, stream, "scalar_gemm_v1", a=A2.slice, b=B2.slice, c=C2.slice, m=mm, n=nn, k=kk)
        assert (bits(C2.read()) == bits(orc.gemm_f32(mm, nn, kk, aa, bb))).all()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 512), (384, 640, 1024), (1024, 1024, 2048), (130, 264, 72)])
def test_gemm_tcgen05_random_bf16(gpu, orc, m, n, k):
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    a, b = synth.uniform_bf16(0, 1, m * k), synth.uniform_bf16(0, 2, k * n)
    A, B = Guarded(fe, stream, a), Guarded(fe, stream, b)
    Cb = Guarded(fe, stream, np.zeros(m * n, np.float32))  # beta * C is evaluated even for beta = 0
    run(fe, ctx, stream, "tiled_gemm_general_v1", schedule=fe.SCHEDULE_TCGEN05, a=A.slice, b=B.slice, c=Cb.slice, m=m,
        n=n, k=k, lda=k, ldb=n, ldc=n, alpha=1.0, beta=0.0)
    want = orc.gemm_bf16_rows(m, n, k, a, b)
    got = Cb.read()
    # f32 accumulation in a different order: |err| <= 1e-3 * sqrt(K)-scale; stated tolerance rel 1e-3 of the row scale
    scale = np.sqrt(k) / 3
    assert np.abs(got - want).max() <= 1e-3 * scale, np.abs(got - want).max()
    A.unchanged(); B.unchanged()


def test_gemm_general_tcgen05_alpha_beta_strides(gpu, orc):
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    m, n, k, lda, ldb, ldc = 200, 136, 96, 104, 144, 140
    a = synth.gemm_inputs_v1((m - 1) * lda + k, 1, 1, 5)[0]
    b = synth.gemm_inputs_v1(1, (k - 1) * ldb + n, 1, 6)[1]
    c = synth.uniform_f32(0, 9, (m - 1) * ldc + n)
    for schedule in (fe.SCHEDULE_EXACT_ORDER, fe.SCHEDULE_TCGEN05):
        A, B, Cb = Guarded(fe, stream, a), Guarded(fe, stream, b), Guarded(fe, stream, c)
        run(fe, ctx, stream, "tiled_gemm_general_v1", schedule=schedule, a=A.slice, b=B.slice, c=Cb.slice, m=m, n=n, k=k,
            lda=lda, ldb=ldb, ldc=ldc, alpha=2.0, beta=-1.0)
        want = orc.gemm_bf16(m, n, k, a, b, lda=lda, ldb=ldb, ldc=ldc, alpha=2.0, beta=-1.0, c=c)
        got = Cb.read()
        for r in range(m):
            assert (bits(got[r * ldc:r * ldc + n]) == bits(want[r * n:(r + 1) * n])).all(), (schedule, r)


# The reference's hardware matrix: seven shape / stride / coefficient profiles, each run by both of its schedules
# (examples/tiled_gemm_general_v1/hardware-harness/src/lib.rs:139-253), on its integer-pattern inputs (:372-386,
# 1640-1648) with NaN-poisoned padding between rows (:69-75).  Here each profile runs on the exact-order schedule
# and, where the copy engine can address the operands (16-byte rows), on the tcgen05 schedule as well.
HARDWARE_CASES = [("packed", (16, 16, 16), (16, 16, 16), 1.0, 0.0),
                  ("strided-all-tails", (17, 19, 18), (23, 29, 31), 0.5, -1.0),
                  ("multi-wg-multi-phase", (33, 35, 33), (37, 41, 43), 2.0, 0.25),
                  ("m-tail", (17, 16, 16), (16, 16, 16), -1.0, 1.0),
                  ("n-tail", (16, 17, 16), (16, 19, 23), 1.5, -0.5),
                  ("k-tail", (16, 16, 17), (21, 19, 16), -0.5, 2.0),
                  ("zero-k", (17, 19, 0), (0, 0, 23), 7.0, 0.5)]


def _pattern(rows, cols, rf, cf, modulus):
    r, c = np.meshgrid(np.arange(rows), np.arange(cols), indexing="ij")
    return ((r * rf + c * cf) % modulus).astype(np.float32) - np.float32(modulus // 2)


@pytest.mark.parametrize("name,shape,strides,alpha,beta", HARDWARE_CASES, ids=[c[0] for c in HARDWARE_CASES])
def test_gemm_general_reference_hardware_matrix(gpu, orc, name, shape, strides, alpha, beta):
    fe, ctx, stream = gpu
    (m, n, k), (lda, ldb, ldc) = shape, strides
    ext = lambda rows, cols, ld: (rows - 1) * ld + cols if rows and cols else 0
    a = np.full(ext(m, k, lda), 0x7fc1, np.uint16)                            # poisoned padding: a NaN pattern
    b = np.full(ext(k, n, ldb), 0x7fd1, np.uint16)
    c = np.full(ext(m, n, ldc), 0x7fc0c001, np.uint32).view(np.float32)
    pa, pb, pc = _pattern(m, k, 3, 5, 7), _pattern(k, n, 2, 3, 5), _pattern(m, n, 7, 11, 13)
    for r in range(m):
        a[r * lda:r * lda + k] = (pa[r].view(np.uint32) >> 16).astype(np.uint16)   # small integers: exact in bf16
        c[r * ldc:r * ldc + n] = pc[r]
    for r in range(k):
        b[r * ldb:r * ldb + n] = (pb[r].view(np.uint32) >> 16).astype(np.uint16)
    want = orc.gemm_bf16(m, n, k, a, b, lda=lda, ldb=ldb, ldc=ldc, alpha=alpha, beta=beta, c=c)
    ran = []
    for schedule in (fe.SCHEDULE_EXACT_ORDER, fe.SCHEDULE_TCGEN05):
        A, B, Cb = Guarded(fe, stream, a), Guarded(fe, stream, b), Guarded(fe, stream, c)
        try:
            p = fe.prepare(ctx, "tiled_gemm_general_v1", schedule=schedule, a=A.slice, b=B.slice, c=Cb.slice, m=m, n=n, k=k,
                           lda=lda, ldb=ldb, ldc=ldc, alpha=alpha, beta=beta)
        except fe.Fe2o3Error as err:
            # the tensor-core schedule admits 16-byte aligned operands with 16-byte row pitches and K > 0 only
            assert schedule == fe.SCHEDULE_TCGEN05 and err.status == -10, err
            continue
        assert len(p.kernarg) == 80   # the reference's explicit argument block (lib.rs:578-593)
        p.launch_and_wait(stream, 20000)
        got = Cb.read()
        for r in range(m):
            assert (bits(got[r * ldc:r * ldc + n]) == bits(want[r * n:(r + 1) * n])).all(), (name, schedule, r)
            pad = got[r * ldc + n:(r + 1) * ldc] if r + 1 < m else got[:0]
            assert (pad.view(np.uint32) == 0x7fc0c001).all(), (name, schedule, "padding of C was written")
        A.unchanged(); B.unchanged()
        ran.append(schedule)
    assert fe.SCHEDULE_EXACT_ORDER in ran
    if name == "packed":
        assert fe.SCHEDULE_TCGEN05 in ran   # every operand row is 16-byte aligned there


@pytest.mark.parametrize("m,n,k,rows", [(512, 512, 512, 512), (4096, 4096, 4096, 96), (136, 264, 72, 136)])
def test_scalar_gemm_f32_tcgen05_split_within_bound(gpu, orc, m, n, k, rows):
    """f32 operands on the tensor cores (split into two bf16 terms each, three products): the stated bound is
    |C - A*B| <= 2^-14 * (|A|*|B|) elementwise, plus the f32 accumulation term K * 2^-24 * (|A|*|B|)."""
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    a, b = synth.uniform_f32(0, 1, m * k), synth.uniform_f32(0, 2, k * n)
    A, B = Guarded(fe, stream, a), Guarded(fe, stream, b)
    Cb = Guarded(fe, stream, np.full(m * n, np.nan, np.float32))
    p = run(fe, ctx, stream, "scalar_gemm_v1", schedule=fe.SCHEDULE_TCGEN05, a=A.slice, b=B.slice, c=Cb.slice, m=m, n=n, k=k)
    assert p.geometry.launches == 3
    got = Cb.read().reshape(m, n)[:rows].astype(np.float64)
    a64, b64 = a.reshape(m, k)[:rows].astype(np.float64), b.reshape(k, n).astype(np.float64)
    exact, mag = a64 @ b64, np.abs(a64) @ np.abs(b64)
    bound = (2.0 ** -14 + k * 2.0 ** -24) * mag
    assert (np.abs(got - exact) <= bound).all(), float((np.abs(got - exact) / mag).max())
    A.unchanged(); B.unchanged()


def test_gemm_empty_and_zero_k(gpu, orc):
    fe, ctx, stream = gpu
    assert fe.prepare(ctx, "tiled_gemm_v1", a=(0, 0), b=(0, 0), c=(0, 0), m=0, n=16, k=16) is None  # NoDispatch
    Cb = Guarded(fe, stream, np.full(16 * 16, np.nan, np.float32))
    run(fe, ctx, stream, "tiled_gemm_v1", a=(0, 0), b=(0, 0), c=Cb.slice, m=16, n=16, k=0)
    assert (bits(Cb.read()) == 0).all()  # K = 0 gives +0.0 (contract.rs:409-415)


# ------------------------------------------------------------------ attention

def attn_run(gpu, q, k, v, scale, causal, dtype):
    fe, ctx, stream = gpu
    B, H, S, D = q.shape
    Q, K, V = Guarded(fe, stream, q), Guarded(fe, stream, k), Guarded(fe, stream, v)
    O = Guarded(fe, stream, np.full(q.size, np.nan, np.float32))
    p = run(fe, ctx, stream, "flash_attention_v1", q=Q.slice, k=K.slice, v=V.slice, output=O.slice, batch=B, heads=H,
            seq=S, dim=D, scale=scale, causal=int(causal), input_dtype=dtype)
    Q.unchanged(); K.unchanged(); V.unchanged()
    return O.read().reshape(q.shape), p


def test_attention_reference_profile_vectors(gpu, orc):
    # the four vectors of examples/flash_attention_v1/src/vectors.rs at B1/H1/N8/D16, causal, scale 0.25
    fe = gpu[0]
    from test_oracle_pins import attn_vectors
    for name, (q, k, v) in attn_vectors().items():
        got, p = attn_run(gpu, q, k, v, 0.25, True, fe.DTYPE_F32)
        _, want = orc.flash_attention(q, k, v, 0.25, True)
        assert np.abs(got - want).max() <= 1e-5, name  # the reference tests' absolute bound
        # the first 64 bytes are the reference's explicit block: four (address, 128) pairs
        assert len(p.kernarg) == 96 and [struct.unpack_from("<Q", p.kernarg, 16 * i + 8)[0] for i in range(4)] == [128] * 4


@pytest.mark.parametrize("B,H,S,D,causal", [(1, 2, 128, 64, False), (2, 2, 256, 64, False), (1, 1, 384, 64, True),
                                            (1, 1, 96, 32, False), (1, 2, 512, 128, False),
                                            # 208 two-tile units on 148 CTAs: one full round of the persistent
                                            # schedule, then a last round split into 120 single tiles
                                            (2, 13, 2048, 64, False), (2, 13, 2048, 64, True),
                                            # rows and keys that end inside a tile, several rounds
                                            (1, 5, 1000, 64, True), (3, 7, 1900, 64, False)])
def test_attention_bf16_vs_f64_oracle(gpu, orc, B, H, S, D, causal):
    fe = gpu[0]
    from fe2o3_b200 import synth
    n = B * H * S * D
    q, k, v = (synth.normal_bf16(3, d, n, 1.0).reshape(B, H, S, D) for d in (1, 2, 3))
    got, _ = attn_run(gpu, q, k, v, 1.0 / np.sqrt(D), causal, fe.DTYPE_BF16)
    _, want = orc.flash_attention(synth.bf16_to_f32(q), synth.bf16_to_f32(k), synth.bf16_to_f32(v), 1.0 / np.sqrt(D), causal)
    # BASELINE tolerance: rel 2e-2, plus an absolute term of 2e-3 of the largest output
    assert_close(got, want, 2e-2, 2e-3, "attention")


# ------------------------------------------------------------------------ MoE

def test_moe_routing_reference_vectors_bit_exact(gpu, orc):
    fe, ctx, stream = gpu
    from test_oracle_pins import MOE_VECTORS
    for name, logits in MOE_VECTORS.items():
        lg = np.array(logits, np.float32)
        L = Guarded(fe, stream, lg)
        outs = {k: Guarded(fe, stream, np.full(n, 0x12345678, np.uint32)) for k, n in
                [("top2_experts", 16), ("requested_counts", 4), ("admitted_counts", 4), ("expert_offsets", 5),
                 ("route_slots", 16), ("permutation", 16), ("inverse", 16)]}
        p = run(fe, ctx, stream, "moe_top2_v1", logits=L.slice, tokens=8, experts=4, capacity=4,
                **{k: g.slice for k, g in outs.items()})
        assert len(p.kernarg) == 144 and p.symbol == "moe_top2_v1"
        _, want = orc.moe_top2_route(lg, 8, 4, 4, independent=True)
        for k in outs:
            assert (outs[k].read() == want[k]).all(), (name, k)
        L.unchanged()


ROUTE_ARRAYS = ("top2_experts", "requested_counts", "admitted_counts", "expert_offsets", "route_slots", "permutation",
                "inverse")


@pytest.mark.parametrize("T,E,cap", [(1, 2, 1), (255, 4, 100), (256, 8, 512), (257, 8, 40), (5000, 8, 10000),
                                     (16384, 8, 32768), (3001, 16, 300), (1000, 32, 7), (70000, 8, 20000)])
def test_moe_routing_many_blocks_bit_exact(gpu, orc, T, E, cap):
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    # logits quantised to multiples of 1/4 so that equal scores (the tie-break) are common
    lg = np.round(synth.normal_f32(4, 50 + E, T * E, 1.5) * 4) / 4
    L = Guarded(fe, stream, lg.astype(np.float32))
    sizes = dict(top2_experts=2 * T, requested_counts=E, admitted_counts=E, expert_offsets=E + 1, route_slots=2 * T,
                 permutation=2 * T, inverse=2 * T)
    outs = {k: Guarded(fe, stream, np.full(n, 0x12345678, np.uint32)) for k, n in sizes.items()}
    for _ in range(2):  # the second launch checks that the arrival counter re-arms
        run(fe, ctx, stream, "moe_top2_v1", logits=L.slice, tokens=T, experts=E, capacity=cap,
            **{k: g.slice for k, g in outs.items()})
        st, want = orc.moe_top2_route(lg, T, E, cap, independent=True)
        assert st == 0
        got = {k: outs[k].read() for k in ROUTE_ARRAYS}
        for k in ROUTE_ARRAYS:
            assert (got[k] == want[k]).all(), k
        assert orc.moe_validate_routing(lg, T, E, cap, got) == 0
    L.unchanged()


def test_moe_routing_single_block_kernel_in_subprocess():
    """The one-block routing kernel (used beyond 4M tokens) is selected with an environment switch."""
    import os
    import subprocess
    import sys
    code = """
import numpy as np, sys
sys.path.insert(0, %r)
import fe2o3_b200 as fe, oracle
from fe2o3_b200 import synth
ctx = fe.GpuContext(0); s = ctx.default_stream()
T, E, cap = 3000, 8, 500
lg = (np.round(synth.normal_f32(4, 9, T * E, 1.5) * 4) / 4).astype(np.float32)
L = fe.DeviceBuffer.from_host(s, lg)
names = dict(top2_experts=2*T, requested_counts=E, admitted_counts=E, expert_offsets=E+1, route_slots=2*T, permutation=2*T, inverse=2*T)
outs = {k: fe.DeviceBuffer.zeroed(s, n, np.uint32) for k, n in names.items()}
p = fe.prepare(ctx, "moe_top2_v1", logits=L, tokens=T, experts=E, capacity=cap, **outs)
assert p.geometry.grid[0] == 1 and p.geometry.workgroup[0] == 1024
p.launch_and_wait(s)
st, want = oracle.moe_top2_route(lg, T, E, cap, independent=True)
for k in names:
    assert (outs[k].to_host_vec(s) == want[k]).all(), k
print("ok")
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, FE2O3_ROUTE_SINGLE_BLOCK="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


# d_model % 256 == 0 with 4, 8 or 16 experts takes the one-warp-per-block pairs kernel; otherwise up to 4096 tokens with
# d_model % 64 == 0 the warp-per-eight-tokens kernel, more tokens the 32-token block kernel, other expert counts the
# generic kernel
@pytest.mark.parametrize("T,d,E", [(100, 64, 8), (300, 200, 4), (257, 2048, 8), (64, 136, 16), (50, 96, 5), (33, 70, 8),
                                   (4500, 128, 8), (4200, 192, 16), (1000, 256, 4), (2048, 2048, 8), (101, 512, 16),
                                   (70, 768, 4), (5000, 256, 8)])
def test_moe_gate_logits_bit_exact(gpu, orc, T, d, E):
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    x, wg = synth.normal_bf16(4, 1, T * d, 1.0), synth.normal_bf16(4, 2, d * E, 0.02)
    X, W = Guarded(fe, stream, x), Guarded(fe, stream, wg)
    LG = Guarded(fe, stream, np.full(T * E, np.nan, np.float32))
    run(fe, ctx, stream, "moe_gate_v1", x=X.slice, wg=W.slice, logits=LG.slice, tokens=T, d_model=d, experts=E)
    assert (bits(LG.read()) == bits(orc.moe_gate_logits(x, wg, T, d, E))).all()
    X.unchanged(); W.unchanged()


def test_moe_routing_failure_preserves_outputs(gpu):
    # examples/moe_top2_v1/tests/oracle.rs:110-141
    fe, ctx, stream = gpu
    lg = np.ones(32, np.float32)
    lg[9] = np.nan
    L = Guarded(fe, stream, lg)
    outs = {k: Guarded(fe, stream, np.full(n, 0x12345678, np.uint32)) for k, n in
            [("top2_experts", 16), ("requested_counts", 4), ("admitted_counts", 4), ("expert_offsets", 5),
             ("route_slots", 16), ("permutation", 16), ("inverse", 16)]}
    p = fe.prepare(ctx, "moe_top2_v1", logits=L.slice, tokens=8, experts=4, capacity=4, **{k: g.slice for k, g in outs.items()})
    with pytest.raises(fe.Fe2o3Error):
        p.launch_and_wait(stream)
    assert p.kernel_status == 2
    for g in outs.values():
        assert (g.read() == 0x12345678).all()


def moe_pipeline(gpu, orc, T, d, f, E, capacity, seed=4):
    """gate -> top2 -> weights -> FFN -> combine on the GPU; returns device and oracle results."""
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    x = synth.normal_bf16(seed, 1, T * d, 1.0)
    wg = synth.normal_bf16(seed, 2, d * E, 0.02)
    w1 = synth.normal_bf16(seed, 3, E * d * f, 0.02)
    w2 = synth.normal_bf16(seed, 4, E * f * d, 0.02)
    R = 2 * T
    X, WG, W1, W2 = (Guarded(fe, stream, t) for t in (x, wg, w1, w2))
    LG = Guarded(fe, stream, np.zeros(T * E, np.float32))
    run(fe, ctx, stream, "moe_gate_v1", x=X.slice, wg=WG.slice, logits=LG.slice, tokens=T, d_model=d, experts=E)
    logits = LG.read()
    want_logits = orc.moe_gate_logits(x, wg, T, d, E)
    assert (bits(logits) == bits(want_logits)).all()  # exact-order gate: bit-identical logits
    outs = {k: Guarded(fe, stream, np.full(n, 0x12345678, np.uint32)) for k, n in
            [("top2_experts", R), ("requested_counts", E), ("admitted_counts", E), ("expert_offsets", E + 1),
             ("route_slots", R), ("permutation", R), ("inverse", R)]}
    run(fe, ctx, stream, "moe_top2_v1", logits=LG.slice, tokens=T, experts=E, capacity=capacity,
        **{k: g.slice for k, g in outs.items()})
    _, want = orc.moe_top2_route(want_logits, T, E, capacity, independent=True)
    got = {k: g.read() for k, g in outs.items()}
    for k in want:
        assert (got[k] == want[k]).all(), k  # routing indices, counts, offsets, slots: bit-exact
    assert orc.moe_validate_routing(want_logits, T, E, capacity, got) == 0
    WT = Guarded(fe, stream, np.zeros(R, np.float32))
    run(fe, ctx, stream, "moe_route_weights_v1", logits=LG.slice, top2_experts=outs["top2_experts"].slice,
        route_weights=WT.slice, tokens=T, experts=E)
    w = WT.read()
    want_w = orc.moe_route_weights(want_logits, want["top2_experts"], T, E)
    assert ((w[0::2] + w[1::2]) == 1.0).all() and np.abs(w - want_w).max() <= 1e-6
    CX = Guarded(fe, stream, np.zeros(R * d, np.uint16))
    HID = Guarded(fe, stream, np.zeros(R * f, np.uint16))
    CO = Guarded(fe, stream, np.zeros(R * d, np.float32))
    run(fe, ctx, stream, "moe_expert_ffn_v1", x=X.slice, w1=W1.slice, w2=W2.slice, permutation=outs["permutation"].slice,
        expert_offsets=outs["expert_offsets"].slice, compact_x=CX.slice, hidden=HID.slice, compact_output=CO.slice,
        tokens=T, d_model=d, d_ff=f, experts=E)
    compact = CO.read()
    want_compact = orc.moe_expert_ffn(x, w1, w2, want["top2_experts"], want["inverse"], T, d, f, E)
    OUT = Guarded(fe, stream, np.full(T * d, np.nan, np.float32))
    run(fe, ctx, stream, "moe_expert_combine_v1", compact_output=CO.slice, inverse=outs["inverse"].slice,
        route_weights=WT.slice, combined_output=OUT.slice, tokens=T, width=d)
    out = OUT.read()
    st, want_out = orc.moe_combine(want_compact, want["inverse"], want_w, T, d)
    assert st == 0
    # the combine kernel itself is exact-order: same bits as the oracle combine on the device's own inputs
    st, replay = orc.moe_combine(compact, got["inverse"], w, T, d)
    assert st == 0 and (bits(out) == bits(replay)).all()
    for t in (X, WG, W1, W2):
        t.unchanged()
    return compact, want_compact, out, want_out, int(want["expert_offsets"][E])


@pytest.mark.parametrize("T,d,f,E,cap", [(64, 128, 256, 4, 128), (300, 256, 512, 8, 600), (256, 128, 256, 8, 40),
                                         # a row length that is not whole 64-column blocks: the expert FFN
                                         # compacts the rows first instead of gathering them in its first GEMM
                                         (100, 136, 256, 4, 200),
                                         # ragged groups over several row tiles, some routes dropped
                                         (1500, 192, 320, 8, 300)])
def test_moe_end_to_end_small(gpu, orc, T, d, f, E, cap):
    compact, want_compact, out, want_out, accepted = moe_pipeline(gpu, orc, T, d, f, E, cap)
    # BASELINE tolerance: outputs rel 2e-2, plus an absolute term of 2e-3 of the largest output
    assert_close(out, want_out, 2e-2, 2e-3, "combined output")
    assert_close(compact[: accepted * d], want_compact[: accepted * d], 2e-2, 2e-3, "compact expert output")


def test_expert_ffn_gathered_rows_equal_compacted_rows(gpu, orc, monkeypatch):
    """The expert FFN's first GEMM either reads rows that a compaction pass has laid out, or gathers the
    rows of x through the permutation itself (loader warps, cp.async into the swizzled stage).  Both feed the
    tensor core the same operands in the same order, so the two outputs are the same bits, on several
    thousand row tiles, launch after launch."""
    fe, ctx, stream = gpu
    from fe2o3_b200 import synth
    T, d, f, E = 6000, 512, 768, 8
    R = 2 * T
    x = synth.normal_bf16(6, 1, T * d, 1.0)
    w1, w2 = synth.normal_bf16(6, 2, E * d * f, 0.05), synth.normal_bf16(6, 3, E * f * d, 0.05)
    logits = synth.normal_bf16(6, 4, T * E, 1.0).astype(np.float32) / 256.0
    _, routing = orc.moe_top2_route(logits, T, E, 1400)   # capacity below demand: dropped slots in every group
    B = lambda a: fe.DeviceBuffer.from_host(stream, a)
    X, W1, W2 = B(x), B(w1), B(w2)
    PERM, OFF = B(routing["permutation"]), B(routing["expert_offsets"])
    outs = {}
    for mode in ("0", "1"):
        monkeypatch.setenv("FE2O3_FFN_GATHER", mode)
        CX, HID, CO = (fe.DeviceBuffer.zeroed(stream, n, t) for n, t in ((R * d, np.uint16), (R * f, np.uint16), (R * d, np.float32)))
        p = fe.prepare(ctx, "moe_expert_ffn_v1", x=X, w1=W1, w2=W2, permutation=PERM, expert_offsets=OFF, compact_x=CX,
                       hidden=HID, compact_output=CO, tokens=T, d_model=d, d_ff=f, experts=E)
        assert p.geometry.launches == (2 if mode == "1" else 3)
        res = []
        for _ in range(3):
            p.launch_and_wait(stream, 20000)
            res.append(CO.to_host_vec(stream).copy())
        assert all((bits(r) == bits(res[0])).all() for r in res)
        outs[mode] = res[0]
    accepted = int(routing["expert_offsets"][E]) * d
    assert accepted > 0 and (bits(outs["0"][:accepted]) == bits(outs["1"][:accepted])).all()
    # ... and with the combine folded into the second GEMM (weighted rows added into the token rows): the same
    # bits as the separate combine kernel on those expert outputs, whichever of a token's two rows lands first
    weights = orc.moe_route_weights(logits, routing["top2_experts"], T, E)
    WT, INV = B(weights), B(routing["inverse"])
    SEP = fe.DeviceBuffer.from_host(stream, np.full(T * d, np.nan, np.float32))
    fe.prepare(ctx, "moe_expert_combine_v1", compact_output=CO, inverse=INV, route_weights=WT, combined_output=SEP,
               tokens=T, width=d).launch_and_wait(stream, 20000)
    want = SEP.to_host_vec(stream)
    FUSED = fe.DeviceBuffer.from_host(stream, np.full(T * d, np.nan, np.float32))   # the operation clears it itself
    HID2 = fe.DeviceBuffer.zeroed(stream, R * f, np.uint16)
    p = fe.prepare(ctx, "moe_expert_ffn_combine_v1", x=X, w1=W1, w2=W2, permutation=PERM, expert_offsets=OFF,
                   route_weights=WT, hidden=HID2, combined_output=FUSED, tokens=T, d_model=d, d_ff=f, experts=E)
    assert p.geometry.launches == 2 and p.symbol == "moe_expert_ffn_combine_v1"
    for _ in range(3):
        p.launch_and_wait(stream, 20000)
        assert p.kernel_status == 0
        assert (bits(FUSED.to_host_vec(stream)) == bits(want)).all()
    # a row length that is not whole 64-column blocks has no fused form
    with pytest.raises(fe.Fe2o3Error):
        fe.prepare(ctx, "moe_expert_ffn_combine_v1", x=X, w1=W1, w2=W2, permutation=PERM, expert_offsets=OFF,
                   route_weights=WT, hidden=HID2, combined_output=FUSED, tokens=T * d // 72, d_model=72, d_ff=f, experts=E)


# ------------------------------------------------------------ adapter surface

def test_runtime_adapter_resolves_reference_symbols(gpu, orc):
    import ctypes as C
    import hashlib
    fe, ctx, stream = gpu
    from fe2o3_b200._lib import lib, LIB_PATH, Geometry, KernelResources
    image = open(LIB_PATH, "rb").read()
    digest = hashlib.sha256(image).digest()
    dig = lambda b: (C.c_uint8 * 32).from_buffer_copy(b)
    mine = (C.c_uint8 * 32)()
    fe.check(lib.fe2o3_image_digest(mine))
    assert bytes(mine) == digest                                   # the library's own SHA-256 agrees with hashlib
    exe = C.c_void_p()
    # load_executable(bytes, digest): a digest that is not the digest of the bytes, and bytes that are not the
    # loaded image, are both refused and leave nothing loaded (hsa_executable_lifecycle.rs:977-990)
    assert lib.fe2o3_load_executable(ctx._h, image, C.c_uint64(len(image)), dig(bytes(32)), C.byref(exe)) == -16
    other = b"not the image"
    assert lib.fe2o3_load_executable(ctx._h, other, C.c_uint64(len(other)), dig(hashlib.sha256(other).digest()), C.byref(exe)) == -16
    assert not exe.value
    fe.check(lib.fe2o3_load_executable(ctx._h, image, C.c_uint64(len(image)), dig(digest), C.byref(exe)))
    kid, nbytes = C.c_uint32(), C.c_uint64()
    res = KernelResources()
    for sym in ("tiled_gemm_lds_slice1", "tiled_gemm_general_v1", "scalar_gemm_v1", "flash_attention_v1", "row_softmax_v1",
                "moe_top2_v1", "moe_expert_combine_v1", "wave64_collectives_v1", "gfx942_wave_lds_v1_hw",
                "lds_publish_read_reduce_i32_v1", "scoped_atomic_add_u32_v1"):
        fe.check(lib.fe2o3_resolve_kernel(exe, sym.encode(), C.byref(kid), C.byref(nbytes)), sym)
        fe.check(lib.fe2o3_observe_kernel_resources(exe, kid, C.byref(res)), sym)
        assert 0 < res.registers_per_thread <= 255 and 32 <= res.max_threads_per_block <= 1024, sym
    fe.check(lib.fe2o3_resolve_kernel(exe, b"flash_attention_v1", C.byref(kid), C.byref(nbytes)))
    fe.check(lib.fe2o3_observe_kernel_resources(exe, kid, C.byref(res)))
    assert res.max_dynamic_shared_bytes > 100 * 1024              # the tensor-core kernel's opted-in shared memory
    assert lib.fe2o3_resolve_kernel(exe, b"no_such_kernel", C.byref(kid), C.byref(nbytes)) == -13
    fe.check(lib.fe2o3_resolve_kernel(exe, b"row_softmax_v1", C.byref(kid), C.byref(nbytes)))
    x = np.linspace(-3, 3, 64, dtype=np.float32)
    i, o = Guarded(fe, stream, x), Guarded(fe, stream, np.zeros(64, np.float32))
    args = fe.make_args("row_softmax_v1", input=i.slice, output=o.slice, rows=1, cols=64)
    ks = C.c_uint32()
    # a geometry that is not the one the argument block plans to is refused before anything is submitted
    plan = fe.prepare(ctx, "row_softmax_v1", input=i.slice, output=o.slice, rows=1, cols=64).geometry
    wrong = Geometry()
    wrong.grid[:], wrong.workgroup[:] = (plan.grid[0] + 1, 1, 1), tuple(plan.workgroup)
    assert lib.fe2o3_launch_and_wait(exe, kid, C.byref(wrong), C.byref(args), nbytes, stream._h, C.c_uint32(5000), C.byref(ks)) == -2
    assert (o.read() == 0).all()
    fe.check(lib.fe2o3_launch_and_wait(exe, kid, C.byref(plan), C.byref(args), nbytes, stream._h, C.c_uint32(5000), C.byref(ks)))
    assert np.abs(o.read() - orc.row_softmax(x)[1]).max() < 1e-7
    o2 = Guarded(fe, stream, np.zeros(64, np.float32))
    args2 = fe.make_args("row_softmax_v1", input=i.slice, output=o2.slice, rows=1, cols=64)
    fe.check(lib.fe2o3_launch_and_wait(exe, kid, None, C.byref(args2), nbytes, stream._h, C.c_uint32(5000), C.byref(ks)))  # no geometry given
    assert np.abs(o2.read() - orc.row_softmax(x)[1]).max() < 1e-7
    fe.check(lib.fe2o3_unload_executable(exe))
    props = ctx.observe_environment()
    assert props.compute_major == 10 and props.multiprocessors > 100
    ev0, ev1 = fe.Event(ctx), fe.Event(ctx)
    ev0.record(stream); ev1.record(stream); ev1.synchronize()
    assert ev1.query() and ev1.elapsed_time_ms_since(ev0) >= 0
    assert fe.launch_count() > 0


def test_one_shot_lifecycle_over_the_cuda_adapter(gpu, orc):
    # join -> load -> dispatch_and_wait -> unload (crates/fe2o3-host/src/flash_attention_v1_lifecycle.rs:227-487)
    fe, ctx, stream = gpu
    from fe2o3_b200 import lifecycle as lc, _lib
    x = np.linspace(-4, 4, 4 * 256, dtype=np.float32)
    i, o = Guarded(fe, stream, x), Guarded(fe, stream, np.zeros(4 * 256, np.float32))
    prep = fe.prepare(ctx, "row_softmax_v1", input=i.slice, output=o.slice, rows=4, cols=256)
    receipt = lc.ArtifactReceipt.for_library(_lib.LIB_PATH, prep.symbol)
    adapter = lc.CudaRuntimeAdapter(ctx, stream)
    loaded = lc.join(receipt, lc.bind_prepared(ctx, prep, leases=[i, o])).load(adapter)
    assert loaded.resolution_observation.symbol == "row_softmax_v1"
    done = loaded.dispatch_and_wait().unload()
    assert np.abs(o.read() - orc.row_softmax(x.reshape(4, 256))[1].reshape(-1)).max() < 1e-7
    assert done.receipt_identity == receipt.identity and len(done.unload_identity) == 32
    # a receipt of other bytes is refused by the adapter before anything is loaded
    forged = lc.ArtifactReceipt(receipt.identity, receipt.artifact_identity, lc.ContentIdentity.calculate(b"x" * 64),
                                lc.TARGET, prep.symbol, b"x" * 64)
    with pytest.raises(lc.LoadError) as err:
        lc.join(forged, lc.bind_prepared(ctx, prep)).load(lc.CudaRuntimeAdapter(ctx, stream))
    assert err.value.kind == "LoadAdapter"
    # a kernel that reports a status word fails the dispatch, and the lifecycle still unloads
    bad = x.copy()
    bad[5] = np.nan
    ib = Guarded(fe, stream, bad)
    prep2 = fe.prepare(ctx, "row_softmax_v1", input=ib.slice, output=o.slice, rows=4, cols=256)
    loaded2 = lc.join(lc.ArtifactReceipt.for_library(_lib.LIB_PATH, prep2.symbol), lc.bind_prepared(ctx, prep2)).load(adapter)
    with pytest.raises(lc.DispatchError):
        loaded2.dispatch_and_wait()


@pytest.mark.parametrize("n", [1, 5, 63, 64, 4095, 4096, 4097, 12289, 100003, (1 << 22) + 3])
@pytest.mark.parametrize("exclusive", [0, 1])
def test_device_scan_sum_u32_bit_exact(gpu, orc, n, exclusive):
    # crates/fe2o3-device/src/collective.rs:413-460 at array scope
    fe, ctx, stream = gpu
    rng = np.random.default_rng(n * 2 + exclusive)
    v = rng.integers(0, 2**32, n, dtype=np.uint64).astype(np.uint32)      # sums wrap many times
    V, O = Guarded(fe, stream, v), Guarded(fe, stream, np.full(n, 0xdeadbeef, np.uint32))
    run(fe, ctx, stream, "device_scan_u32", values=V.slice, output=O.slice, exclusive=exclusive)
    assert (O.read() == orc.scan_sum_u32(v, bool(exclusive))).all()
    V.unchanged()


def test_device_scan_sum_u32_unaligned_repeated_and_rejections(gpu, orc):
    fe, ctx, stream = gpu
    v = (np.arange(1, 20001, dtype=np.uint64) * 2654435761 % (2**32)).astype(np.uint32)
    buf = fe.DeviceBuffer.from_host(stream, v)
    res = fe.DeviceBuffer.zeroed(stream, v.size, np.uint32)
    # slices that start one element in: 4-byte aligned only, so the scalar path runs
    src, dst = buf.view(1, v.size - 1), res.view(1, v.size - 1)
    p = fe.prepare(ctx, "device_scan_u32", values=src, output=dst, exclusive=0)
    p.launch_and_wait(stream)
    got = res.to_host_vec(stream)
    assert got[0] == 0 and (got[1:] == orc.scan_sum_u32(v[1:])).all()
    # the same prepared launch again gives the same answer (scratch is cleared by every launch)
    p.launch_and_wait(stream)
    assert (res.to_host_vec(stream)[1:] == orc.scan_sum_u32(v[1:])).all()
    # empty input: accepted, nothing launched
    fe.prepare(ctx, "device_scan_u32", values=buf.view(0, 0), output=res.view(0, 0), exclusive=1).launch_and_wait(stream)
    # output overlapping the input, and a short output, are refused by the host check
    for bad in (dict(values=src, output=src), dict(values=buf.view(0, 8), output=res.view(0, 7))):
        with pytest.raises(fe.Fe2o3Error):
            fe.check_args("device_scan_u32", fe.make_args("device_scan_u32", exclusive=0, **bad))


def scan_f32_tolerance(n, magnitudes):
    # the bound the header states: (128 + tiles / 192) roundings of 2^-24 each, scaled by the prefix of |values|
    return (128 + n / 8192 / 192) * 2.0 ** -24 * magnitudes + 1e-30


@pytest.mark.parametrize("n", [1, 63, 4097, 100003, (1 << 22) + 3, 1 << 24])
@pytest.mark.parametrize("exclusive", [0, 1])
def test_device_scan_sum_f32_within_stated_tolerance_and_reproducible(gpu, orc, n, exclusive):
    fe, ctx, stream = gpu
    rng = np.random.default_rng(n * 2 + exclusive)
    v = rng.standard_normal(n).astype(np.float32)             # mixed signs: the prefix keeps cancelling
    V, O = Guarded(fe, stream, v), Guarded(fe, stream, np.full(n, np.nan, np.float32))
    p = fe.prepare(ctx, "device_scan_f32", values=V.slice, output=O.slice, exclusive=exclusive)
    p.launch_and_wait(stream)
    first = O.read().copy()
    want, mag = orc.scan_sum_f32(v, bool(exclusive))
    err = np.abs(first.astype(np.float64) - want)
    assert (err <= scan_f32_tolerance(n, mag)).all(), float((err / scan_f32_tolerance(n, mag)).max())
    if exclusive:
        assert first[0] == 0.0
    # the order of additions is fixed by position: a second run gives the same bits
    p.launch_and_wait(stream)
    assert (O.read().view(np.uint32) == first.view(np.uint32)).all()
    V.unchanged()


def test_device_scan_sum_f32_exact_on_small_integers_and_propagates_specials(gpu, orc):
    fe, ctx, stream = gpu
    n = 300001
    v = (np.arange(n) % 7).astype(np.float32)                 # every partial sum is an integer below 2^24: exact
    V, O = Guarded(fe, stream, v), Guarded(fe, stream, np.zeros(n, np.float32))
    run(fe, ctx, stream, "device_scan_f32", values=V.slice, output=O.slice, exclusive=0)
    assert (O.read() == np.cumsum(v.astype(np.float64)).astype(np.float32)).all()
    v[200000] = np.inf                                        # an infinity reaches everything after it, nothing before
    V2 = Guarded(fe, stream, v)
    run(fe, ctx, stream, "device_scan_f32", values=V2.slice, output=O.slice, exclusive=0)
    got = O.read()
    assert np.isfinite(got[:200000]).all() and np.isposinf(got[200000:]).all()


def test_dispatch_record_of_a_prepared_launch(gpu):
    # crates/fe2o3-host-api/src/dispatch.rs:96-268: the record that describes one launch of this library
    import hashlib
    fe, ctx, stream = gpu
    from fe2o3_b200 import host_api as ha
    x = np.zeros(4 * 256, np.float32)
    i, o = Guarded(fe, stream, x), Guarded(fe, stream, x)
    args = fe.make_args("row_softmax_v1", input=i.slice, output=o.slice, rows=4, cols=256)
    prep = fe.prepare(ctx, "row_softmax_v1", input=i.slice, output=o.slice, rows=4, cols=256)
    context = ha.OperationContext(ha.commit("FlowScopeId", b"test"), ha.commit("OperationId", b"softmax"), 1)
    loaded = ha.LoadedResult(ha.commit("LoadResultId", b"lib"), ha.commit("LoadedObjectId", b"lib"), 1)
    req = ha.dispatch_request_for(prep, args, context, loaded, written=("output",))
    assert [b.ordinal for b in req.bindings] == [0, 1] and [b.access for b in req.bindings] == [ha.ACCESS_READ, ha.ACCESS_WRITE]
    assert all(b.byte_len == 4 * 256 * 4 for b in req.bindings)
    assert req.identity == hashlib.sha256(req.encode_identity_preimage()).digest()
    assert req.entry_point_identity == ha.commit("EntryPointId", b"row_softmax_v1")
