"""Pins the CPU oracle to the reference's own golden vectors and known-answer tests.

Each case names the reference test it restates (paths relative to the reference root).
"""
import json
import math
import os

import numpy as np
import pytest

import oracle


def _gen_values(n, seed):
    # crates/inference/tests/quantize_q4_reader_refactor.rs:35-38
    return np.array([float(((i * 37 + seed * 13) % 200) - 100) / 4.0 for i in range(n)], np.float32)


def _truncate_bf16(v):
    return ((v.view(np.uint32) >> 16) << 16).view(np.float32)


@pytest.mark.parametrize("name", ["gate_proj", "k_proj"])
def test_golden_q4_files_byte_identical(golden_dir, name):
    fx = json.load(open(os.path.join(golden_dir, "reference_q4_fixtures.json")))[name]
    want = bytes.fromhex(fx["hex"])
    n = int(np.prod(fx["shape"]))
    vals = _truncate_bf16(_gen_values(n, fx["seed"]))
    payload = oracle.quantize_f32_to_q4(vals)
    got = oracle.q4_file_bytes(fx["shape"], n, payload)
    assert got == want
    # same answer through the bf16-bits entry point (the values are bf16-exact)
    bits = (vals.view(np.uint32) >> 16).astype(np.uint16)
    assert oracle.quantize_bf16_to_q4(bits).tobytes() == payload.tobytes()
    shape, olen, off = oracle.q4_parse(want)
    assert shape == fx["shape"] and olen == n and off == 36


def test_q4_container_rejects_bad_images(golden_dir):
    fx = json.load(open(os.path.join(golden_dir, "reference_q4_fixtures.json")))["k_proj"]
    img = bytes.fromhex(fx["hex"])
    for bad in (img[:-1], img + b"\0", b"KHQ5" + img[4:], img[:4] + (1).to_bytes(4, "little") + img[8:]):
        with pytest.raises(oracle.OracleError):
            oracle.q4_parse(bad)


def test_partial_tail_uses_real_min_max():
    # q4_weights.rs:2184-2208
    p = oracle.quantize_f32_to_q4(np.array([5, 6, 7], np.float32))
    assert len(p) == 20
    assert int.from_bytes(p[0:2].tobytes(), "little") == oracle.f32_to_f16_bits(np.float32(2.0) / np.float32(15.0))
    assert int.from_bytes(p[2:4].tobytes(), "little") == oracle.f32_to_f16_bits(5.0)


def test_max_min_map_to_15_and_0():
    # q4_weights.rs:1754-1777
    src = np.zeros(32, np.float32)
    src[0], src[1] = 7.0, -7.0
    p = oracle.quantize_tensor_q4_0(src, 1, 32)
    assert p[4] & 0x0F == 15 and p[4] >> 4 == 0


def test_symmetric_layout_centre_is_8():
    v = np.zeros(32, np.float32)
    v[0], v[1], v[2] = 7.0, -7.0, 0.0
    blk = oracle.quantize_block(v, 32, symmetric=True)
    assert blk[4] & 0xF == 15 and blk[4] >> 4 == 1 and blk[5] & 0xF == 8
    scale = oracle.f16_bits_to_f32(int.from_bytes(blk[0:2], "little"))
    bias = oracle.f16_bits_to_f32(int.from_bytes(blk[2:4], "little"))
    assert scale == 1.0 and bias == -8.0


def test_degenerate_scale_and_overflow():
    # q4_weights.rs:2239-2314 (tiny range -> scale 1.0), :2344-2358 (too large -> rejected)
    tiny = np.float32(3.363e-37)
    v = np.zeros(32, np.float32)
    v[0], v[7] = tiny, -tiny / np.float32(3.0)
    assert oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(float(tiny / np.float32(7.0)))) == 0.0
    for sym in (True, False):
        blk = oracle.quantize_block(v, 32, symmetric=sym)
        assert oracle.f16_bits_to_f32(int.from_bytes(blk[0:2], "little")) == 1.0
    zero = oracle.quantize_block(np.zeros(32, np.float32), 32)
    assert oracle.f16_bits_to_f32(int.from_bytes(zero[0:2], "little")) == 1.0
    big = np.zeros(32, np.float32)
    big[0] = 1.0e7
    with pytest.raises(oracle.OracleError) as e:
        oracle.quantize_block(big, 32, symmetric=True)
    assert e.value.code == oracle.ERR_SCALE
    for bad in (np.nan, np.inf):
        w = np.zeros(32, np.float32)
        w[3] = bad
        with pytest.raises(oracle.OracleError) as e:
            oracle.quantize_block(w, 32)
        assert e.value.code == oracle.ERR_NONFINITE
    with pytest.raises(oracle.OracleError):
        oracle.quantize_block(np.zeros(32, np.float32), 0)


def test_f16_known_answers():
    # weights/half_bits.rs:309-420
    f, h = oracle.f32_to_f16_bits, oracle.f16_bits_to_f32
    assert h(0x3C00) == 1.0 and h(0xBC00) == -1.0 and h(0x7C00) == math.inf and h(0xFC00) == -math.inf
    assert math.isnan(h(0x7E00)) and h(0x0000) == 0.0 and math.copysign(1, h(0x8000)) == -1
    assert f(65504.0) == 0x7BFF and f(65519.0) == 0x7BFF and f(65520.0) == 0x7C00 and f(65521.0) == 0x7C00
    assert f(2.0 ** -14) == 0x0400 and f(2.0 ** -14 * (1023.0 / 1024.0)) == 0x03FF
    assert f(0.0) == 0 and f(-0.0) == 0x8000 and f(1.0e6) == 0x7C00 and f(-1.0e6) == 0xFC00
    nan = f(math.nan)
    assert nan & 0x7C00 == 0x7C00 and nan & 0x0200
    a, b, c = h(0x3C00), h(0x3C01), h(0x3C02)
    assert f((a + b) * 0.5) == 0x3C00 and f((b + c) * 0.5) == 0x3C02
    for bits in (0x0001, 0x0200, 0x03FF):
        assert f(h(bits)) == bits


def test_f16_exhaustive_against_numpy():
    # weights/half_bits.rs:174-255: every 16-bit pattern widens exactly and narrows back
    bits = np.arange(65536, dtype=np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_bits_to_f32(int(b)) for b in bits], np.float32)
    fin = np.isfinite(ref)
    assert np.array_equal(got[fin].view(np.uint32), ref[fin].view(np.uint32))
    assert np.all(np.isnan(got[np.isnan(ref)]))
    back = np.array([oracle.f32_to_f16_bits(float(v)) for v in got[fin]], np.uint16)
    assert np.array_equal(back, bits[fin])
    rng = np.random.default_rng(5)
    r = (rng.standard_normal(20000) * np.exp(rng.uniform(-20, 12, 20000))).astype(np.float32)
    with np.errstate(over="ignore"):
        want = r.astype(np.float16).view(np.uint16)
    have = np.array([oracle.f32_to_f16_bits(float(v)) for v in r], np.uint16)
    assert np.array_equal(want, have)


def test_walsh_hadamard_known_answers():
    # quant/quarot/hadamard.rs:684-707
    assert np.allclose(oracle.walsh_hadamard(np.array([1, 2], np.float32)), [3, -1], atol=1e-6)
    assert np.allclose(oracle.walsh_hadamard(np.array([1, 0, 0, 0], np.float32)), [1, 1, 1, 1], atol=1e-6)
    x = np.arange(16, dtype=np.float32) - 8
    assert np.allclose(oracle.walsh_hadamard(oracle.walsh_hadamard(x)), 16 * x, atol=1e-4)
    with pytest.raises(oracle.OracleError):
        oracle.walsh_hadamard(np.zeros(3, np.float32))
    y = oracle.walsh_hadamard(x, orthonormal=True)
    assert abs(np.linalg.norm(y) - np.linalg.norm(x)) < 1e-4
    assert np.allclose(oracle.walsh_hadamard(y, orthonormal=True), x, atol=1e-4)


def test_randomized_hadamard_is_orthogonal_and_seeded():
    s1, s2 = oracle.signs_from_seed(42, 64), oracle.signs_from_seed(42, 64)
    assert np.array_equal(s1, s2) and set(np.unique(s1)) <= {-1.0, 1.0}
    assert not np.array_equal(s1, oracle.signs_from_seed(43, 64))
    # independent restatement of the splitmix64 stream in Python integers
    M = (1 << 64) - 1
    g = 0x9E3779B97F4A7C15
    state = (42 + g) & M
    want = []
    for _ in range(64):
        state = (state + g) & M
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        z ^= z >> 31
        want.append(1.0 if z & 1 == 0 else -1.0)
    assert np.array_equal(s1, np.array(want, np.float32))
    x = np.random.default_rng(0).standard_normal(64).astype(np.float32)
    y = oracle.rh_apply(s1, x)
    assert np.allclose(oracle.rh_apply(s1, y, inverse=True), x, atol=1e-5)
    assert not np.allclose(oracle.rh_apply(s1, y), x, atol=1e-3)
    # adjacent block seeds are not shifted copies (hadamard.rs:147-160)
    a = oracle.signs_from_seed(oracle.derive_block_seed(7, 0), 128)
    b = oracle.signs_from_seed(oracle.derive_block_seed(7, 1), 128)
    assert not np.array_equal(a[1:], b[:-1])


def test_absorption_preserves_forward():
    # quant/quarot/rotation.rs:242-262, 390-410
    rng = np.random.default_rng(1)
    rows, cols = 8, 32
    w = rng.standard_normal((rows, cols))
    x = rng.standard_normal(cols)
    s = oracle.signs_from_seed(11, cols)
    w_rot = oracle.absorb_rotation(w, rows, cols, s, "input")
    assert np.max(np.abs(w_rot @ oracle.rh_apply(s, x) - w @ x)) < 1e-12
    w32 = oracle.absorb_rotation(w.astype(np.float32), rows, cols, s, "input")
    assert np.max(np.abs(w32 @ oracle.rh_apply(s, x.astype(np.float32)) - (w @ x))) < 1e-4
    so = oracle.signs_from_seed(12, rows)
    w_out = oracle.absorb_rotation(w, rows, cols, so, "output")
    assert np.max(np.abs(w_out @ x - oracle.rh_apply(so, w @ x))) < 1e-12


def test_lora_known_answers():
    # crates/tune/src/lora/apply.rs:99-147, crates/tune/src/lora/mod.rs:652-669
    out = np.array([100, 200], np.float32)
    assert oracle.apply_lora([1, 0, 0], [1, 0], 1, 3, 2, 2.0, [5, 3, 1], out)
    assert np.allclose(out, [110, 200], atol=1e-6)
    out = np.zeros(2, np.float32)
    oracle.apply_lora([1, 0, 0, 1], [1, 2, 3, 4], 2, 2, 2, 0.5, [1, 1], out)
    assert np.allclose(out, [1.5, 3.5], atol=1e-6)
    out = np.zeros(4, np.float32)
    oracle.apply_lora([1, 0, 0, 0, 0, 1, 0, 0], [1, 0, 0, 1, 0, 0, 0, 0], 2, 4, 4, 2.0, [1, 2, 3, 4], out)
    assert np.allclose(out, [2, 4, 0, 0], atol=1e-6)
    out = np.array([1, 2], np.float32)
    oracle.apply_lora([1, 0, 0], [1, 0], 1, 3, 2, 0.0, [5, 3, 1], out)
    assert np.array_equal(out, [1, 2])
    # malformed shapes are a silent no-op (exact output width required)
    out = np.array([1, 2, 3], np.float32)
    assert not oracle.apply_lora([1, 0, 0], [1, 0], 1, 3, 2, 2.0, [5, 3, 1], out)
    assert np.array_equal(out, [1, 2, 3])
    assert oracle.effective_scale(16, 32.0) == 2.0 and oracle.effective_scale(0, 32.0) == 0.0
    assert oracle.effective_scale(4, math.inf) == 0.0 and oracle.effective_scale(4, math.nan) == 0.0


def _lcg_f64(n, seed):
    out, state = [], seed
    for _ in range(n):
        state = (state * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        out.append((state >> 32) / 4294967295.0 * 2.0 - 1.0)
    return np.array(out, np.float64)


def test_composed_quarot_q4_gate():
    """q4_weights.rs:2487-2672: rotate -> symmetric Q4 -> dequant -> matvec against an
    independent re-implementation, bound 1e-5, same seeds and shapes."""
    H, QR, OR = 32, 2, 32
    q = _lcg_f64(QR * H, 0x1111111111111111)
    o = _lcg_f64(OR * H, 0x2222222222222222)
    xq = _lcg_f64(H, 0x3333333333333333)
    xo = _lcg_f64(H, 0x4444444444444444)
    signs = oracle.signs_from_seed(0x32000001, H)

    q_rot = oracle.absorb_rotation(q.reshape(QR, H), QR, H, signs, "input")
    o_rot = oracle.absorb_rotation(o.reshape(OR, H), OR, H, signs, "output")
    q_deq = oracle.dequantize_q4_to_f32(oracle.quantize_f64_to_q4(q_rot)).astype(np.float64).reshape(QR, H)
    o_deq = oracle.dequantize_q4_to_f32(oracle.quantize_f64_to_q4(o_rot)).astype(np.float64).reshape(OR, H)

    def ref_dequant(data):      # numpy restatement, independent of the C code
        out = []
        for chunk in data.reshape(-1, 32):
            f = chunk.astype(np.float32)
            amax = np.float32(np.max(np.abs(f)))
            scale = np.float32(1.0) if amax == 0 else amax / np.float32(7.0)
            bias = np.float32(-8.0) * scale
            sdq = np.float32(np.float16(scale))
            bdq = np.float32(np.float16(bias))
            inv = np.float32(1.0) / scale
            t = f * inv
            r = np.sign(t) * np.floor(np.abs(t) + np.float32(0.5))     # round half away from zero
            nib = np.clip(r + np.float32(8.0), 0, 15).astype(np.uint8).astype(np.float32)
            out.append((nib * sdq + bdq).astype(np.float64))
        return np.concatenate(out)

    # the manual rotation of the reference test: per row (input side), per column (output side)
    q_ref = np.stack([oracle.rh_apply(signs, r) for r in q.reshape(QR, H)])
    o_ref = np.stack([oracle.rh_apply(signs, c) for c in o.reshape(OR, H).T]).T
    yq, yo = q_deq @ xq, o_deq @ xo
    rq, ro = ref_dequant(q_ref).reshape(QR, H) @ xq, ref_dequant(o_ref).reshape(OR, H) @ xo
    assert np.max(np.abs(yq - rq)) <= 1e-5 and np.max(np.abs(yo - ro)) <= 1e-5


def test_dequant_roundtrip_error_bound_and_validity():
    rng = np.random.default_rng(3)
    w = (rng.standard_normal(32 * 50) * 0.02).astype(np.float32)
    p = oracle.quantize_f32_to_q4(w)
    d = oracle.dequantize_q4_to_f32(p)
    for blk in range(50):
        seg = w[blk * 32:(blk + 1) * 32]
        step = (seg.max() - seg.min()) / 15
        assert np.max(np.abs(d[blk * 32:(blk + 1) * 32] - seg)) <= 0.5 * step * 1.01 + 1e-3 * np.abs(seg).max()
    assert oracle.first_invalid_block(p) == -1
    bad = p.copy()
    bad[3 * 20:3 * 20 + 2] = np.frombuffer((0).to_bytes(2, "little"), np.uint8)       # scale == 0
    assert oracle.first_invalid_block(bad) == 3
    bad = p.copy()
    bad[7 * 20 + 2:7 * 20 + 4] = np.frombuffer((0x7C00).to_bytes(2, "little"), np.uint8)  # bias == inf
    assert oracle.first_invalid_block(bad) == 7
    assert np.array_equal(oracle.dequantize_q4_to_f32(p, 35), d[:35])


def test_matmul_variants_agree():
    rng = np.random.default_rng(4)
    for (m, k, n) in [(1, 64, 16), (1, 1024, 40), (3, 100, 7), (5, 256, 33), (8, 1024, 136), (4, 136, 8)]:
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((n, k)).astype(np.float32)
        ref = oracle.matmul_bt_f64acc(a, b, m, k, n)
        tol = 2e-5 * np.sqrt(k)
        for variant in ("dispatch", "scalar", "tiled_scalar", "tiled_avx2", "avx2"):
            got = oracle.matmul_bt(a, b, m, k, n, variant)
            assert np.max(np.abs(got - ref)) < tol, (variant, m, k, n)
    # dispatch rule: forward/cpu/matmul.rs:83-87
    oracle.set_force_scalar(True)
    try:
        assert oracle.matmul_bt_kernel(1, 1024, 3584) == "tiled-scalar"
        assert oracle.matmul_bt_kernel(1, 64, 64) == "scalar"
        assert oracle.matmul_bt_kernel(64, 64, 64) == "scalar"       # k < 128 never tiles
    finally:
        oracle.set_force_scalar(False)


def test_composed_linear_matches_plain_numpy():
    rng = np.random.default_rng(6)
    m, k, n, r = 3, 128, 24, 4
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    a = (rng.standard_normal((r, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal((n, r)) * 0.02).astype(np.float32)
    p = oracle.quantize_f32_to_q4(w)
    wd = oracle.dequantize_q4_to_f32(p).reshape(n, k).astype(np.float64)
    y = oracle.q4_linear(x, p, m, n, k, lora=(a, b, 2.0))
    ref = x.astype(np.float64) @ wd.T + 2.0 * (x.astype(np.float64) @ a.T.astype(np.float64)) @ b.T.astype(np.float64)
    assert np.max(np.abs(y - ref)) < 1e-5
    s = oracle.signs_from_seed(9, k)
    yr = oracle.q4_linear(x, p, m, n, k, rot_signs=s)
    xr = np.stack([oracle.rh_apply(s, row) for row in x]).astype(np.float64)
    assert np.max(np.abs(yr - xr @ wd.T)) < 1e-5
    y1 = oracle.gemv_q4_decode_form(x[0], p, n, k)
    assert np.max(np.abs(y1 - (x[0].astype(np.float64) @ wd.T))) < 1e-5
    with pytest.raises(oracle.OracleError):
        oracle.q4_linear(x[:, :100], p, m, n, 100)


def _reference_cpu_topk_ids(logits, k):
    """cpu_topk_token_ids of the reference's own tests (crates/inference/src/forward/metal_qwen35.rs:24943-24952):
    a stable sort of the ids by descending logit, truncated to k."""
    order = np.argsort(-logits.astype(np.float64), kind="stable")
    return order[:k].astype(np.uint32)


def test_topk_order_matches_the_reference_cpu_selection():
    rng = np.random.default_rng(171)
    # coarse values: many exact ties, so that the tie rule (lower id first) decides most of the order
    logits = rng.integers(-40, 40, 5000).astype(np.float32) * np.float32(0.25)
    for k in (1, 8, 16, 40, 50, 64, 256):
        vals, ids = oracle.topk(logits, k)
        assert np.array_equal(ids, _reference_cpu_topk_ids(logits, k))
        assert np.array_equal(vals, logits[ids])
    # continuous values
    logits = rng.standard_normal(3000).astype(np.float32)
    vals, ids = oracle.topk(logits, 50)
    assert np.array_equal(ids, _reference_cpu_topk_ids(logits, 50))


def test_topk_nan_and_short_rows_keep_the_sentinel():
    logits = np.array([1.0, np.nan, 5.0, -np.inf, 5.0, np.nan, 0.0, -0.0], np.float32)
    vals, ids = oracle.topk(logits, 4)
    assert ids.tolist() == [2, 4, 0, 6] and vals.tolist() == [5.0, 5.0, 1.0, 0.0]
    vals, ids = oracle.topk(logits, 10)
    # a real -inf logit ranks before the sentinel; the two NaN rows never appear
    assert ids.tolist() == [2, 4, 0, 6, 7, 3] + [0xFFFFFFFF] * 4
    assert np.all(np.isneginf(vals[5:]))
    vals, ids = oracle.topk(np.full(7, np.nan, np.float32), 3)
    assert ids.tolist() == [0xFFFFFFFF] * 3 and np.all(np.isneginf(vals))


# ---- BlockHadamard: the reference's own properties (quant/quarot/hadamard.rs tests, :502-1040) ----
def test_block_hadamard_signs_match_per_block_randomized_hadamard():
    seed, n, b = 0xC0FFEE, 3584, 128
    s = oracle.block_hadamard_signs(seed, n, b)
    for i in (0, 1, 13, 27):
        assert np.array_equal(s[i * b:(i + 1) * b], oracle.signs_from_seed(oracle.derive_block_seed(seed, i), b))
    # adjacent blocks' sign streams are not one-position-shifted copies (the defect derive_block_seed removes)
    assert not np.array_equal(s[1:b], s[b:2 * b - 1])
    assert set(np.unique(s).tolist()) == {-1.0, 1.0}


def test_block_hadamard_round_trip_norm_and_partition():
    rng = np.random.default_rng(4)
    for n, b in ((3584, 128), (17408, 256), (64, 64), (96, 32)):
        s = oracle.block_hadamard_signs(7, n, b)
        x = rng.standard_normal(n).astype(np.float32)
        y = oracle.block_hadamard_apply(s, x, b)
        assert abs(np.linalg.norm(y) / np.linalg.norm(x) - 1.0) < 1e-5
        assert np.max(np.abs(oracle.block_hadamard_apply(s, y, b, inverse=True) - x)) < 1e-5
        # every block is RandomizedHadamard::apply of its own slice, nothing crosses a block boundary
        i = (n // b) // 2
        assert np.array_equal(y[i * b:(i + 1) * b], oracle.rh_apply(s[i * b:(i + 1) * b], x[i * b:(i + 1) * b]))
        x2 = x.copy()
        x2[:b] += 1.0
        assert np.array_equal(oracle.block_hadamard_apply(s, x2, b)[b:], y[b:])


def test_block_hadamard_refuses_what_the_constructor_refuses():
    for n, b in ((0, 64), ((1 << 24) + 64, 64), (100, 64), (96, 48), (64, 0), (1 << 24, 1), (4097 * 2, 2)):
        with pytest.raises(oracle.OracleError):
            oracle.block_hadamard_signs(1, n, b)
    oracle.block_hadamard_signs(1, 4096 * 2, 2)          # exactly 4096 blocks is accepted


def test_cross_head_rotation_is_the_kronecker_factor_and_cancels_through_o_proj():
    # r3_reference.rs:521-640: the rotation equals (H_nh D) (x) I_head_dim, and an o_proj whose rows were
    # rotated the same way (input-side absorption) reproduces the dense product
    nh, dh, hidden = 8, 16, 12
    rng = np.random.default_rng(3)
    signs = oracle.signs_from_seed(0x703, nh)
    x = rng.standard_normal(nh * dh).astype(np.float32)
    y = oracle.cross_head_rotation(signs, x, dh)
    hmat = np.array([[1.0]])
    while hmat.shape[0] < nh:
        hmat = np.block([[hmat, hmat], [hmat, -hmat]])
    r = (hmat / np.sqrt(nh)) @ np.diag(signs.astype(np.float64))
    full = np.kron(r, np.eye(dh))
    assert np.max(np.abs(full @ x.astype(np.float64) - y)) < 1e-5
    # a block rotation over contiguous head_dim blocks is a different transform
    assert np.max(np.abs(oracle.block_hadamard_apply(oracle.block_hadamard_signs(0x703, nh * dh, dh), x, dh) - y)) > 1e-2
    w = rng.standard_normal((hidden, nh * dh)).astype(np.float32)
    w_rot = np.stack([oracle.cross_head_rotation(signs, w[i], dh) for i in range(hidden)])
    assert np.max(np.abs(w_rot.astype(np.float64) @ y - w.astype(np.float64) @ x)) < 1e-4
    with pytest.raises(oracle.OracleError):
        oracle.cross_head_rotation(np.ones(6, np.float32), np.zeros(6 * 4, np.float32), 4)


def test_silu_mul_matches_the_shader_formula():
    g = np.array([[-20.0, -1.0, 0.0, 0.5, 3.0, 30.0, 2.0, -0.5, 1.5, 0.25, -3.0, 7.0]], np.float32)
    out = oracle.silu_mul(g, 6)
    gate, up = g[0, :6].astype(np.float64), g[0, 6:].astype(np.float64)
    assert np.max(np.abs(out[0] - gate / (1.0 + np.exp(-gate)) * up)) < 1e-6
    assert out[0, 2] == 0.0
