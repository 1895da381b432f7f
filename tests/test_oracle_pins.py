"""The CPU oracle against the reference's own known-answer vectors.

Every expected constant below is a golden value held by the reference's tests
(cited per test); the inputs are rebuilt from the recipes in the reference's
vector files.  These run without a GPU.
"""
import struct

import numpy as np

F32_NAN_BITS = 0x7FC00000


def bits(x):
    return [int(v) for v in np.asarray(x, np.float32).view(np.uint32).ravel()]


# --- GEMM: examples/tiled_gemm_v1/tests/inputs_oracle.rs --------------------

def test_generator_bytes_and_outputs_are_pinned(orc):
    # inputs_oracle.rs:29-59
    a, b = orc.gemm_inputs_v1(2, 3, 2, 0x1234)
    assert list(a) == [0x0000, 0x4080, 0xBD80, 0x4040]
    assert list(b) == [0xBE80, 0x4040, 0x4040, 0x3E80, 0x4080, 0x3E00]
    out = orc.gemm_bf16(2, 3, 2, a, b)
    assert bits(out) == [0x3F800000, 0x41800000, 0x3F000000, 0x3F440000, 0x413D0000, 0x3E400000]


def test_small_row_major_product(orc):
    # inputs_oracle.rs:227-239 and scalar_gemm_v1/src/harness.rs:258-268
    a = orc.bf16_from_f32([1, 2, 3, 4])
    b = orc.bf16_from_f32([5, 6, 7, 8, 9, 10])
    assert list(orc.gemm_bf16(2, 3, 2, a, b)) == [21, 24, 27, 47, 54, 61]
    assert list(orc.gemm_f32(2, 3, 2, [1, 2, 3, 4], [5, 6, 7, 8, 9, 10])) == [21, 24, 27, 47, 54, 61]
    assert list(orc.gemm_f32(2, 3, 2, [1, 2, 3, 4], [5, 6, 7, 8, 9, 10], fast=True)) == [21, 24, 27, 47, 54, 61]


def test_zero_k_gives_positive_zero(orc):
    # inputs_oracle.rs:241-251
    for m, n in [(1, 1), (16, 16), (17, 31), (0, 9), (9, 0)]:
        out = orc.gemm_bf16(m, n, 0, np.zeros(0, np.uint16), np.zeros(0, np.uint16))
        assert out.size == m * n and all(v == 0 for v in bits(out))


def test_rounding_order_and_signed_zero(orc):
    # inputs_oracle.rs:274-320
    one, p24, n24 = 0x3F80, 0x4B80, 0xCB80
    assert bits(orc.gemm_bf16(1, 1, 3, [one] * 3, [p24, one, n24])) == [0]
    assert bits(orc.gemm_bf16(1, 1, 3, [one] * 3, [p24, n24, one])) == [0x3F800000]
    assert bits(orc.gemm_bf16(1, 1, 1, [0x0000], [0xBF80])) == [0]
    assert bits(orc.gemm_bf16(1, 1, 1, [0x8000], [0x3F80])) == [0]


def test_fma_distinguishing_case(orc):
    # scalar_gemm_v1/src/harness.rs:271-288: separate roundings give +0.
    eps = np.float32(np.finfo(np.float32).eps)
    a = np.array([1 + eps, 1.0], np.float32)
    b = np.array([1 - eps, -1.0], np.float32)
    assert bits(orc.gemm_f32(1, 1, 2, a, b)) == [0]
    assert bits(orc.gemm_f32(1, 1, 2, a, b, fast=True)) == [0]


def test_alpha_beta_vector(orc):
    # tests/numerical_contract.rs:124-146
    a = [0x3F80, 0x4000, 0x4040, 0x4080, 0x40A0, 0x40C0]
    b = [0x40A0, 0x40C0, 0x40E0, 0x4100, 0x4110, 0x4120]
    c = np.array([4.0, -8.0, np.nan, 12.0, -16.0], np.float32)
    out = orc.gemm_bf16(2, 2, 3, a, b, lda=3, ldb=2, ldc=3, alpha=0.5, beta=0.25, c=c)
    assert bits(out) == [0x41C00000, 0x41C00000, 0x42660000, 0x42680000]


def test_zero_k_epilogue(orc):
    # tests/numerical_contract.rs:31-48
    c = np.array([2.0, 4.0, 6.0, np.nan, np.nan, 8.0, 10.0, 12.0], np.float32)
    out = orc.gemm_bf16(2, 3, 0, [], [], lda=0, ldb=3, ldc=5, alpha=7.0, beta=0.5, c=c)
    assert list(out) == [1, 2, 3, 4, 5, 6]


def corpus(orc):
    """examples/tiled_gemm_v1/src/numerical_vectors.rs:134-328, rebuilt."""
    import ctypes as C
    nan = np.float32(np.nan)
    V = []

    def packed(m, n, k):
        return (m, n, k, k, n, n)

    V.append(("zero-signed", packed(2, 3, 4),
              [0x0000, 0x8000, 0x0000, 0x8000, 0x8000, 0x0000, 0x8000, 0x0000],
              [0x0000, 0x8000] * 6, [0.0, -0.0, 0.0, -0.0, 0.0, -0.0], 1.0, 1.0))
    V.append(("identity-3x3", packed(3, 3, 3),
              [0x3F80, 0, 0, 0, 0x3F80, 0, 0, 0, 0x3F80],
              [0x3F00, 0xBF80, 0x4000, 0x4040, 0xC000, 0x3E80, 0x4080, 0x3F80, 0xC040], [0.0] * 9, 1.0, 0.0))
    V.append(("dyadic-2x2x3", packed(2, 2, 3),
              [0x3F00, 0xBF80, 0x4000, 0x3E80, 0x4040, 0xC000],
              [0x3F80, 0x3E00, 0xBF00, 0x4000, 0x4080, 0x3F00], [0.0] * 4, 1.0, 0.0))
    V.append(("cancellation-pairs", packed(1, 2, 4),
              [0x3F80, 0x3F80, 0x4000, 0x4000],
              [0x4080, 0x4040, 0xC080, 0xC040, 0x3F00, 0xBF00, 0xBF00, 0x3F00], [0.0] * 2, 1.0, 0.0))
    alpha12 = [0xBD80, 0xBE00, 0xBE80, 0xBF00, 0xBF80, 0x0000, 0x3D80, 0x3E00, 0x3E80, 0x3F00, 0x3F80, 0x4000]
    state = C.c_uint64(0x10905EEDD15CA11E)
    nxt = orc.lib().orc_splitmix64_next
    nxt.restype = C.c_uint64
    gen = lambda n: [alpha12[nxt(C.byref(state)) % 12] for _ in range(n)]
    ra = gen(5 * 17)
    rb = gen(17 * 4)
    V.append(("randomized-seed-109", packed(5, 4, 17), ra, rb, [0.0] * 20, 1.0, 0.0))
    a = [0x7FC1] * 18
    b = [0x7F80] * 17
    c = [nan] * 10
    for r in range(3):
        for d in range(4):
            a[r * 7 + d] = [0x3F80, 0x4000, 0xBF80, 0x3F00][(r + d) % 4]
    for d in range(4):
        for col in range(2):
            b[d * 5 + col] = [0x3F00, 0xBF00, 0x4000, 0xC000][d]
    for r in range(3):
        for col in range(2):
            c[r * 4 + col] = 0.0
    V.append(("padded-independent-strides", (3, 2, 4, 7, 5, 4), a, b, c, 1.0, 0.0))
    al8 = [0xBE80, 0xBE00, 0x0000, 0x3E00, 0x3E80, 0x3F00, 0xBF00, 0x3F80]
    V.append(("tails-m17-n19-k23", packed(17, 19, 23),
              [al8[(i * 5 + i // 7 + 3) % 8] for i in range(17 * 23)],
              [al8[(i * 3 + i // 11 + 1) % 8] for i in range(23 * 19)], [0.0] * (17 * 19), 1.0, 0.0))
    V.append(("alpha-beta-nonzero-c", packed(2, 3, 3),
              [0x3F80, 0x4000, 0xBF80, 0x3F00, 0xC000, 0x4040],
              [0x3F80, 0x3F00, 0xBF00, 0x4000, 0xC000, 0x3E80, 0x4080, 0x3F80, 0xC080],
              [4.0, -8.0, 12.0, -16.0, 20.0, -24.0], 0.5, 0.25))
    V.append(("finite-extremes-and-signed-zero", packed(6, 1, 1),
              [0x7F7F, 0xFF7F, 0x0080, 0x8080, 0x0000, 0x8000], [0x3F80],
              [0.0, -0.0, 0.0, -0.0, 0.0, -0.0], 1.0, 0.0))
    return V


def test_corpus_digest_is_pinned(orc):
    # tests/numerical_contract.rs:488-519: FNV-1a over names, dims and strides
    # (usize, 8 LE bytes), operand bits, C bits, alpha/beta bits, expected bits.
    h = 0xCBF29CE484222325
    for name, (m, n, k, lda, ldb, ldc), a, b, c, alpha, beta in corpus(orc):
        cin = np.array(c, np.float32)
        out = orc.gemm_bf16(m, n, k, a, b, lda=lda, ldb=ldb, ldc=ldc, alpha=alpha, beta=beta, c=cin)
        h = orc.fnv1a(h, name.encode())
        h = orc.fnv1a(h, b"".join(struct.pack("<Q", v) for v in (m, n, k, lda, ldb, ldc)))
        h = orc.fnv1a(h, np.array(list(a) + list(b), np.uint16).tobytes())
        cb = cin.view(np.uint32).copy()
        cb[np.isnan(cin)] = F32_NAN_BITS  # Rust's f32::NAN bit pattern
        h = orc.fnv1a(h, cb.tobytes())
        h = orc.fnv1a(h, np.array([alpha, beta], np.float32).tobytes())
        h = orc.fnv1a(h, out.tobytes())
    assert h == 0x6131FB795A3C1C51


def test_bf16_narrowing(orc):
    # crates/fe2o3-device/src/half.rs:182-190
    assert orc.lib().orc_bf16_from_f32(1.0) == 0x3F80
    x = np.array([0x3F808000, 0x3F818000, 0x7F800001, 0xFFC00001, 0x3F807FFF, 0x3F808001], np.uint32).view(np.float32)
    assert list(orc.bf16_from_f32(x)) == [0x3F80, 0x3F82, 0x7FC0, 0xFFC0, 0x3F80, 0x3F81]


# --- softmax: examples/row_softmax_v1/tests/numerical_contract.rs -----------

def test_softmax_uniform_row_is_exact_reciprocal(orc):
    # :105-111
    st, out = orc.row_softmax(np.full(64, 3.25, np.float32))
    assert st == 0 and set(bits(out)) == {int(np.float32(1.0 / 64).view(np.uint32))}


def test_softmax_mask_policy(orc):
    # :46-64: masked outputs are +0.0; non-finite input rejected even if masked.
    x = np.array([1.0, -0.0, 1e-45, 5.0], np.float32)
    st, out = orc.row_softmax(x, mask=[1, 1, 1, 0])
    assert st == 0 and bits(out[3:]) == [0] and abs(out[:3].sum() - 1) < 1e-6
    st, _ = orc.row_softmax(np.array([1.0, np.inf], np.float32), mask=[1, 0])
    assert st != 0
    st, _ = orc.row_softmax(np.array([1.0, 2.0], np.float32), mask=[0, 0])
    assert st != 0
    st, _ = orc.row_softmax(np.zeros(4097, np.float32))
    assert st != 0


def test_softmax_comparator(orc):
    # :115-193 and src/numerical_contract.rs:7-13
    rng = np.random.default_rng(5)
    x = rng.normal(0, 2, 64).astype(np.float32)
    _, e = orc.row_softmax(x)
    assert orc.row_softmax_compare(e, e) == 0
    assert orc.row_softmax_compare(e, orc.row_softmax_kernel_f32(x)) == 0
    bad = e.copy()
    bad[3] *= np.float32(1.01)
    assert orc.row_softmax_compare(e, bad) == 4
    bad = e.copy()
    bad[0] = -bad[0]
    assert orc.row_softmax_compare(e, bad) == 1


# --- attention: examples/flash_attention_v1/tests/oracle.rs -----------------

def attn_vectors():
    n = 128
    i = np.arange(n)
    V = {}
    V["nominal"] = (((i * 17 + 3) % 29).astype(np.float32) / 16 - 0.75,
                    ((i * 11 + 5) % 31).astype(np.float32) / 20 - np.float32(0.70),
                    ((i * 7 + 2) % 37).astype(np.float32) / 12 - 1.25)
    V["equal"] = (np.zeros(n, np.float32), (i % 19).astype(np.float32) - 9,
                  (i // 16).astype(np.float32) * 0.5 + (i % 16).astype(np.float32) * 0.03125)
    q = np.zeros(n, np.float32); k = np.zeros(n, np.float32); v = np.zeros(n, np.float32)
    for r in range(8):
        q[r * 16] = 1; k[r * 16] = r * 64
        v[r * 16:(r + 1) * 16] = r * 10 + np.arange(16)
    V["dominant"] = (q, k, v)
    q = np.zeros(n, np.float32); k = np.zeros(n, np.float32); v = np.zeros(n, np.float32)
    for r in range(8):
        q[r * 16 + r] = 0.5; k[r * 16 + r] = 0.75; v[r * 16 + r] = 1
    V["probe"] = (q, k, v)
    return {k_: tuple(np.asarray(t, np.float32).reshape(1, 1, 8, 16) for t in v_) for k_, v_ in V.items()}


def test_attention_reference_profile(orc):
    V = attn_vectors()
    # oracle.rs:44-58 exact causal prefix means
    q, k, v = V["equal"]
    st, o = orc.flash_attention(q, k, v, 0.25, True)
    assert st == 0
    for r in range(8):
        want = (v[0, 0, :r + 1].astype(np.float64).sum(0) / (r + 1)).astype(np.float32)
        assert bits(o[0, 0, r]) == bits(want)
    # :60-72 dominant key
    q, k, v = V["dominant"]
    _, o = orc.flash_attention(q, k, v, 0.25, True)
    assert np.abs(o - v).max() <= 1e-5
    # :74-96 causal mask invariance
    q, k, v = V["nominal"]
    _, base = orc.flash_attention(q, k, v, 0.25, True)
    for first in range(1, 8):
        k2, v2 = k.copy(), v.copy()
        k2[0, 0, first:] += 1000
        v2[0, 0, first:] += 1000
        _, o = orc.flash_attention(q, k2, v2, 0.25, True)
        assert bits(o[0, 0, :first]) == bits(base[0, 0, :first])
    # :98-110 probability probe
    q, k, v = V["probe"]
    _, o = orc.flash_attention(q, k, v, 0.25, True)
    for r in range(8):
        row = o[0, 0, r]
        assert abs(np.float32(row[:8].sum()) - 1) <= 2e-7
        assert (row[r + 1:8] == 0).all() and (row[8:] == 0).all()
    # the strict-f32 online recurrence agrees with the f64 reference
    for name, (q, k, v) in V.items():
        _, a = orc.flash_attention(q, k, v, 0.25, True)
        _, b = orc.flash_attention(q, k, v, 0.25, True, online_f32=True)
        assert np.abs(a - b).max() <= 1e-5, name
    st, _ = orc.flash_attention(np.full((1, 1, 8, 16), np.inf, np.float32), k, v, 0.25, True)
    assert st != 0


# --- MoE routing: examples/moe_top2_v1/tests/oracle.rs ----------------------

FMAX, FMINP = np.finfo(np.float32).max, np.finfo(np.float32).tiny
MOE_VECTORS = {
    "nominal": [4, 3, 2, 1, 1, 4, 3, 2, 2, 1, 4, 3, 3, 2, 1, 4] * 2,
    "all_equal": [1.0] * 32,
    "repeated": [5, 5, 5, 4, 1, 3, 3, 3, -2, -2, -2, -2, 7, 6, 7, 6, 0, -1, -1, 0, 2, 2, 1, 2, 8, 9, 9, 8, -3, -2, -3, -2],
    "overflow": [10, 9, 2, 1, 10, 1, 9, 2, 10, 2, 1, 9, 10, 9, 2, 1, 10, 1, 9, 2, 10, 2, 1, 9, 10, 9, 2, 1, 10, 1, 9, 2],
    "empty": [2, 1, -4, -5, 2, 1, -3, -6, 2, 1, -2, -7, 2, 1, -1, -8, 2, 1, -8, -1, 2, 1, -7, -2, 2, 1, -6, -3, 2, 1, -5, -4],
    "adversarial": [FMAX, -FMAX, FMINP, -0.0, -FMINP, 0.0, -FMAX, FMAX, FMAX, FMAX, -FMAX, -FMAX, -FMAX, -0.0, 0.0,
                    FMINP, 1e30, -1e30, 1e-30, -1e-30, -42, -42, -42, -43, 17, 18, 17, 18, 3.5, 3.25, 3.75, 3.0],
}
DROP = 0xFFFFFFFF


def test_moe_routing_vectors(orc):
    def route(name, independent=False):
        st, o = orc.moe_top2_route(np.array(MOE_VECTORS[name], np.float32), 8, 4, 4, independent)
        assert st == 0
        return o
    o = route("nominal")  # oracle.rs:34-47
    assert list(o["requested_counts"]) == [4] * 4 and list(o["admitted_counts"]) == [4] * 4
    assert list(o["expert_offsets"]) == [0, 4, 8, 12, 16]
    assert (o["route_slots"] != DROP).all() and (o["permutation"] != DROP).all()
    o = route("all_equal")  # :49-64
    assert list(o["top2_experts"]) == [0, 1] * 8
    assert list(o["requested_counts"]) == [8, 8, 0, 0] and list(o["admitted_counts"]) == [4, 4, 0, 0]
    assert list(o["expert_offsets"]) == [0, 4, 8, 8, 8] and (o["permutation"][8:] == DROP).all()
    o = route("overflow")  # :66-80
    assert o["requested_counts"][0] == 8 and list(o["permutation"][0:4]) == [0, 2, 4, 6]
    for r in (8, 10, 12, 14):
        assert o["route_slots"][r] == DROP and o["inverse"][r] == DROP
    o = route("empty")  # :82-89
    assert list(o["requested_counts"]) == [8, 8, 0, 0]
    assert o["expert_offsets"][2] == o["expert_offsets"][3] == o["expert_offsets"][4]
    # the vectors file annotates the expected winners per token (src/vectors.rs:14-48)
    assert list(route("repeated")["top2_experts"]) == [0, 1, 1, 2, 0, 1, 0, 2, 0, 3, 0, 1, 1, 2, 1, 3]
    for name in MOE_VECTORS:  # :91-108 round trip, plus kernel-vs-independent agreement
        a, b = route(name), route(name, independent=True)
        for key in a:
            assert (a[key] == b[key]).all(), (name, key)
        acc = int(a["expert_offsets"][4])
        for slot in range(acc):
            r = int(a["permutation"][slot])
            assert r < 16 and a["route_slots"][r] == slot and a["inverse"][r] == slot
        assert (a["permutation"][acc:] == DROP).all()
        assert orc.moe_validate_routing(np.array(MOE_VECTORS[name], np.float32), 8, 4, 4, a) == 0
    st, _ = orc.moe_top2_route(np.array([np.nan] * 32, np.float32), 8, 4, 4)
    assert st != 0


def test_moe_combine_and_weights(orc):
    # examples/moe_expert_v1/src/kernel.rs:104-157
    rng = np.random.default_rng(1)
    logits = rng.normal(size=(8, 4)).astype(np.float32)
    _, o = orc.moe_top2_route(logits, 8, 4, 4)
    w = orc.moe_route_weights(logits, o["top2_experts"], 8, 4)
    assert ((w[0::2] + w[1::2]) == 1.0).all() and (w[0::2] >= 0.5).all()
    compact = rng.integers(-4, 5, size=(16, 16)).astype(np.float32)
    st, out = orc.moe_combine(compact, o["inverse"], w, 8, 16)
    assert st == 0
    for t in range(8):
        acc = np.zeros(16, np.float32)
        for rank in range(2):
            s = o["inverse"][2 * t + rank]
            if s != DROP:
                acc = acc + w[2 * t + rank] * compact[s]
        assert bits(out[t * 16:(t + 1) * 16]) == bits(acc)
    st, _ = orc.moe_combine(compact, o["inverse"], np.full(16, 0.75, np.float32), 8, 16)
    assert st != 0


# --- reductions --------------------------------------------------------------

def test_masked_u32_runner_vector(orc):
    # crates/dialect-amdgcn/tests/fixtures/gfx942_wave_lds_v1_runner.cpp:26-29,76-94
    lane = np.arange(256)
    values = (lane + 1).astype(np.uint32)
    active = np.where(lane % 3 == 1, 0, 7).astype(np.uint32)
    total = int(values[active != 0].sum())
    assert orc.masked_sum_u32(values, active) == total == orc.masked_sum_u32(values, active, parallel=False)
    st, w, g = orc.wave_workgroup_sums_u32(values, active)
    assert st == 0 and (g == total).all()
    for s in range(4):
        seg = slice(s * 64, s * 64 + 64)
        assert (w[seg] == int(values[seg][active[seg] != 0].sum())).all()
    big = np.full(1 << 17, 0xFFFFFFF0, np.uint32)  # wrapping
    assert orc.masked_sum_u32(big, np.ones_like(big)) == (0xFFFFFFF0 * (1 << 17)) % (1 << 32)
    packed = np.packbits((active != 0).astype(np.uint8), bitorder="little").view(np.uint64)
    assert orc.masked_sum_u32_packed(values, packed) == total


def test_wave64_collectives_masks(orc):
    # examples/wave64_collectives_v1/tests/oracle.rs:6-98
    x = ((np.arange(64) * 5 + 3) % 17).astype(np.float32) - 8
    for mask in (0, (1 << 19) - 1, (1 << 0) | (1 << 3) | (1 << 8) | (1 << 34) | (1 << 63),
                 0xAAAAAAAAAAAAAAAA, 0xFFFFFFFFFFFFFFFF):
        st, r, i, e = orc.wave64_collectives_f32(x, mask)
        assert st == 0
        on = np.array([(mask >> l) & 1 for l in range(64)], bool)
        total = np.float32(x[on].sum())
        prefix = np.float32(0)
        for l in range(64):
            if not on[l]:
                assert bits([r[l], i[l], e[l]]) == [0, 0, 0]
            else:
                assert r[l] == total and e[l] == prefix
                prefix += x[l]
                assert i[l] == prefix
    x = np.zeros(64, np.float32)
    x[0], x[1], x[63] = -0.0, -1024, 1024
    st, r, i, e = orc.wave64_collectives_f32(x, (1 << 0) | (1 << 1) | (1 << 63))
    assert st == 0 and bits([e[0]]) == [0] and i[1] == -1024 and e[63] == -1024 and i[63] == 0
    assert orc.wave64_collectives_f32(np.full(64, 0.5, np.float32), 1)[0] != 0
    assert orc.wave64_collectives_f32(np.full(64, 2048, np.float32), 1)[0] != 0


def test_workgroup_sync_vectors(orc):
    # examples/workgroup_sync_v1/src/vectors.rs:32-109
    lane = np.arange(64)
    cases = [(np.zeros(64, np.int32), 0), (np.where(lane % 2 == 0, 1000, -999), 32), (lane - 32, -32),
             (np.where(lane % 11 == 0, lane * 7, 0), 1155)]
    for values, want in cases:
        assert orc.workgroup_reduce_i32(values) == (0, want)
    assert orc.workgroup_reduce_i32(np.full(64, 2 ** 30, np.int32))[0] != 0
    for initial, elig, want in [(17, np.zeros(64), 17), (0, np.ones(64), 2016), (11, lane % 2 == 0, 1003),
                                (1000, lane % 13 == 0, 1130)]:
        assert orc.scoped_atomic_add_u32(lane, elig.astype(np.uint32), initial) == (0, want)


def test_scan_sum_u32_matches_the_reference_wave_and_workgroup_definitions(orc):
    # crates/fe2o3-device/src/collective.rs:413-460: inclusive prefix in increasing lane order; the exclusive
    # form gives lane 0 zero and lane r the inclusive value of lane r - 1; addition wraps
    rng = np.random.default_rng(7)
    v = rng.integers(0, 2**32, 64, dtype=np.uint64).astype(np.uint32)
    inc, exc = orc.scan_sum_u32(v), orc.scan_sum_u32(v, exclusive=True)
    hs = v.copy()                      # the reference's Hillis-Steele wave scan, step by step
    off = 1
    while off < 64:
        prev = hs.copy()
        hs[off:] = prev[off:] + prev[:-off]
        off <<= 1
    assert (inc == hs).all()
    assert exc[0] == 0 and (exc[1:] == inc[:-1]).all()
    assert (inc == np.cumsum(v.astype(np.uint64)).astype(np.uint32)).all()      # wrapping
    big = rng.integers(0, 2**32, 100003, dtype=np.uint64).astype(np.uint32)
    assert (orc.scan_sum_u32(big) == np.cumsum(big.astype(np.uint64)).astype(np.uint32)).all()
    assert orc.scan_sum_u32(np.zeros(0, np.uint32)).size == 0


def test_scan_sum_f32_reference_is_the_exact_prefix_and_magnitude(orc):
    v = np.array([1.5, -2.25, 1e-3, 4.0], np.float32)
    inc, mag = orc.scan_sum_f32(v)
    assert inc.tolist() == [1.5, -0.75, -0.75 + float(np.float32(1e-3)), 3.25 + float(np.float32(1e-3))]
    assert mag.tolist() == [1.5, 3.75, 3.75 + float(np.float32(1e-3)), 7.75 + float(np.float32(1e-3))]
    exc, emag = orc.scan_sum_f32(v, exclusive=True)
    assert exc.tolist() == [0.0] + inc[:-1].tolist() and emag.tolist() == [0.0] + mag[:-1].tolist()
    assert orc.scan_sum_f32(np.zeros(0, np.float32))[0].size == 0


def test_benchmark_generators_agree_with_the_library(orc):
    """The CPU reference arm builds its inputs with the oracle's restatement of the benchmark's keyed
    SplitMix64 streams; the GPU arm uses the library's host generators.  Same (seed, domain, n) must give
    the same bytes, or the two arms would not measure the same workload."""
    from fe2o3_b200 import synth
    n = 70001
    assert (orc.synth_normal_bf16(4, 1, n, 1.0) == synth.normal_bf16(4, 1, n, 1.0)).all()
    assert (orc.synth_normal_bf16(4, 107, n, 0.02) == synth.normal_bf16(4, 107, n, 0.02)).all()
    assert (orc.synth_u32_below(1, 1, n, 1 << 16) == synth.u32_below(1, 1, n, 1 << 16)).all()
    flags, _ = synth.bernoulli(1, 2, n, 0.75, flag_value=7, packed=False)
    assert (orc.synth_bernoulli_flags(1, 2, n, 0.75, 7) == flags).all()
