"""CPU tests of the oracle: known-answer vectors derived from the bit-layout rules, the golden vectors produced
by the reference's own CUDA kernels on a B200 (tests/golden/ref_kernels.npz, made by make_golden_gpu.py), and the
fp16 arithmetic helpers against numpy."""
import math
import os

import numpy as np
import pytest

from helpers import exponent_field, k_planes_np, make_kvq, softmax_probs, v_planes_np
from oracle import akv_oracle as orc

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kernels.npz")


def u8(a):
    return np.ascontiguousarray(a).view(np.uint8)


def halves(*bits):
    return np.array(bits, dtype=np.uint16).view(np.float16)


# ------------------------------------------------------------------ fp16 arithmetic
def test_f16_roundtrip_exhaustive():
    for h in range(0, 65536, 1):
        ref = np.array([h], np.uint16).view(np.float16)[0]
        d = orc.f16_bits_to_f64(h)
        if np.isnan(ref):
            assert math.isnan(d)
            continue
        assert d == float(ref)
        assert orc.f64_to_f16_bits(d) == h


def test_f64_to_f16_rounding_cases():
    assert orc.f64_to_f16_bits(1.0 + 2.0 ** -11) == 0x3C00            # tie -> even
    assert orc.f64_to_f16_bits(1.0 + 2.0 ** -11 + 2.0 ** -24) == 0x3C01  # just above the tie (torch's cast via
    assert orc.f64_to_f16_bits(1.0 + 3 * 2.0 ** -11) == 0x3C02          # float would double-round this one)
    assert orc.f64_to_f16_bits(65519.9) == 0x7BFF and orc.f64_to_f16_bits(65520.0) == 0x7C00
    assert orc.f64_to_f16_bits(2.0 ** -25) == 0x0000 and orc.f64_to_f16_bits(2.0 ** -25 * 1.0001) == 0x0001
    assert orc.f64_to_f16_bits(-2.0 ** -24) == 0x8001
    assert orc.f64_to_f16_bits(float("nan")) == 0x7FFF


def test_hfma_against_numpy():
    rng = np.random.default_rng(0)
    a, b, c = (rng.integers(0, 65536, 30000, dtype=np.uint16) for _ in range(3))
    with np.errstate(all="ignore"):
        want = (a.view(np.float16).astype(np.float64) * b.view(np.float16).astype(np.float64)
                + c.view(np.float16).astype(np.float64)).astype(np.float16).view(np.uint16)
    for i in range(len(a)):
        got = orc.hfma(int(a[i]), int(b[i]), int(c[i]))
        if np.isnan(want[i:i + 1].view(np.float16)[0]):
            assert got == 0x7FFF
        else:
            assert got == int(want[i]), (hex(a[i]), hex(b[i]), hex(c[i]))


# ------------------------------------------------------------------ bit layout known answers
def test_k_layout_known_answers():
    # one head, one channel... D=2 channels, tokens 0 (0xBEEF), 1 (0x1234), 2 (0x3C00) in channel 0
    B, H, D = 1, 1, 2
    f8, m4, l4 = k_planes_np(B, H, 1, D)
    k = np.zeros((B, 64, H, D), np.float16)
    kb = k.view(np.uint16)
    kb[0, 0, 0, 0], kb[0, 1, 0, 0], kb[0, 2, 0, 0] = 0xBEEF, 0x1234, 0x3C00
    orc.k_cache_save(f8, m4, l4, u8(k), B, H, 1, 1, D, 64, 0, 64)
    assert f8[0, 0, 0, 0, 0] == 0xBE and f8[0, 0, 0, 0, 1] == 0x12 and f8[0, 0, 0, 0, 2] == 0x3C
    assert m4[0, 0, 0, 0, 0] == 0xE3 and l4[0, 0, 0, 0, 0] == 0xF4      # even token in the high nibble
    assert m4[0, 0, 0, 0, 1] == 0x00 and l4[0, 0, 0, 0, 1] == 0x00
    assert not f8[0, 0, 0, 1].any()
    # nibbles are ADDED: writing the same block again doubles them mod 256, the high byte is overwritten
    orc.k_cache_save(f8, m4, l4, u8(k), B, H, 1, 1, D, 64, 0, 64)
    assert m4[0, 0, 0, 0, 0] == (0xE3 * 2) & 0xFF and l4[0, 0, 0, 0, 0] == (0xF4 * 2) & 0xFF
    assert f8[0, 0, 0, 0, 0] == 0xBE


def test_v_layout_known_answers():
    B, H, D = 1, 1, 4
    f8, m4, l4 = v_planes_np(B, H, 2, D)
    v = np.zeros((B, 1, H, D), np.float16)
    vb = v.view(np.uint16)
    vb[0, 0, 0, 0], vb[0, 0, 0, 1] = 0xBEEF, 0x1234     # adjacent CHANNELS share a byte
    orc.v_cache_save(f8, m4, l4, u8(v), B, H, 2, D, 1, 1)
    assert list(f8[0, 0, 1]) == [0xBE, 0x12, 0, 0]
    assert list(m4[0, 0, 1]) == [0xE3, 0] and list(l4[0, 0, 1]) == [0xF4, 0]
    assert not f8[0, 0, 0].any()


def test_skip_constants_and_k_decision_thresholds():
    """skip-last reassembly of 0xBEEF is 0xBEE8, skip-both 0xBE80; mid is read iff (u8)(kqmax-kq) < 8, low iff < 4."""
    B, H, D = 1, 4, 16
    f8, m4, l4 = k_planes_np(B, H, 1, D)
    k = np.zeros((B, 64, H, D), np.float16)
    k.view(np.uint16)[...] = 0xBEEF
    orc.k_cache_save(f8, m4, l4, u8(k), B, H, 1, 1, D, 64, 0, 64)
    q = np.zeros((B, 1, H, D), np.float16)
    one = 0x3C00
    for diff, expect in ((0, 0xBEEF), (3, 0xBEEF), (4, 0xBEE8), (7, 0xBEE8), (8, 0xBE80), (200, 0xBE80)):
        kq = np.full((B, 1, H, D), 20, np.uint8)
        kqmax = np.full((B, 1, H, 1), (20 + diff) & 0xFF, np.uint8)
        q.view(np.uint16)[...] = 0
        q.view(np.uint16)[..., 5] = one                      # only channel 5 contributes: s = k~[5] * 1 * scale
        s, codes = orc.k_cache_compute(f8, m4, l4, kq, kqmax, u8(q), B, H, 1, 1, D, 64, 64, 1.0, False)
        got = s.view(np.uint16)[0, 0, 0, 0]
        assert got == expect, (diff, hex(got))
        assert (codes == (2 if diff >= 8 else 1 if diff >= 4 else 0)).all()
    # wrap-around: kqmax < kq gives a large unsigned difference -> both planes skipped
    kq = np.full((B, 1, H, D), 30, np.uint8)
    kqmax = np.full((B, 1, H, 1), 29, np.uint8)
    _, codes = orc.k_cache_compute(f8, m4, l4, kq, kqmax, u8(q), B, H, 1, 1, D, 64, 64, 1.0, False)
    assert (codes == 2).all()


def test_v_decision_thresholds_and_wraparound():
    """A = (int16)(amin << 10); diff = (int16)(A - bits(s)); mid iff diff < 0x0800, low iff diff < 0x0400."""
    B, H, D, n = 1, 1, 4, 6
    f8, m4, l4 = v_planes_np(B, H, n, D)
    v = np.zeros((B, n, H, D), np.float16)
    v.view(np.uint16)[...] = 0x3C00
    orc.v_cache_save(f8, m4, l4, u8(v), B, H, n, D, 0, n)
    amin = np.array([[[[12]]]], np.uint8)                    # A = 0x3000
    s = halves(0x3000, 0x2C01, 0x2C00, 0x2801, 0x2800, 0x3400).reshape(1, 1, 1, n)
    _, codes = orc.v_cache_compute(f8, m4, l4, u8(s), amin, B, H, n, D, n, n, False)
    assert list(codes[0, 0]) == [0, 0, 1, 1, 2, 0]            # negative differences read everything
    amin = np.array([[[[70]]]], np.uint8)                    # 70 << 10 wraps to 0x1800 in 16 bits
    s = halves(0x1800, 0x1000, 0x0C00).reshape(1, 1, 1, 3)
    _, codes = orc.v_cache_compute(f8, m4, l4, u8(np.ascontiguousarray(s)), amin, B, H, n, D, 3, 3, False)
    assert list(codes[0, 0]) == [0, 2, 2]


def test_reference_mode_equals_dense_fp16_chain():
    """reference=True reads all planes: scores equal the serial fp16 FMA chain over the ORIGINAL fp16 keys."""
    B, H, D, L = 1, 4, 32, 64
    k, v, q = make_kvq(3, B, L, H, D)
    planes = k_planes_np(B, H, 1, D)
    orc.k_cache_save(*planes, u8(k), B, H, 1, 1, D, 64, 0, L)
    z = np.zeros((B, 1, H, D), np.uint8)
    s, _ = orc.k_cache_compute(*planes, z, z[..., :1], u8(q), B, H, 1, 1, D, 64, L, 1 / math.sqrt(D), True)
    s = s.view(np.uint16)
    scale = orc.f64_to_f16_bits(float(np.float32(1 / math.sqrt(D))))
    for h in range(H):
        for t in (0, 1, 17, 63):
            acc = 0
            for d in range(D):
                acc = orc.hfma(int(k.view(np.uint16)[0, t, h, d]), int(q.view(np.uint16)[0, 0, h, d]), acc)
            assert s[0, h, 0, t] == orc.hmul(acc, scale)
    # V side: outputs equal the serial chain over tokens
    vp = v_planes_np(B, H, L, D)
    orc.v_cache_save(*vp, u8(v), B, H, L, D, 0, L)
    p = softmax_probs(4, B, H, L)
    o, _ = orc.v_cache_compute(*vp, u8(p), np.zeros((B, H, H, 1), np.uint8), B, H, L, D, L, L, True)
    o = o.view(np.uint16)
    for h in range(H):
        for d in (0, 1, 30):
            acc = 0
            for t in range(L):
                acc = orc.hfma(int(v.view(np.uint16)[0, t, h, d]), int(p.view(np.uint16)[0, h, 0, t]), acc)
            assert o[0, h, 0, d] == acc


def test_save_dispatch_matches_reference_branches():
    B, H, D = 1, 1, 4
    k, _, _ = make_kvq(9, B, 70, H, D)
    # start_pos != 0 and seqlen neither 1 nor a block multiple: silent no-op
    planes = k_planes_np(B, H, 2, D)
    orc.k_cache_save(*planes, u8(k[:, :3]), B, H, 0, 2, D, 64, 10, 3)
    assert not any(p.any() for p in planes)
    # n_blocks == 0 at start_pos 0: nothing written
    orc.k_cache_save(*planes, u8(k[:, :63]), B, H, 0, 2, D, 64, 0, 63)
    assert not any(p.any() for p in planes)
    # a prompt of 70 tokens writes exactly one block; the tail stays out
    orc.k_cache_save(*planes, u8(k), B, H, 1, 2, D, 64, 0, 70)
    assert planes[0][0, 0, 0].any() and not planes[0][0, 0, 1].any()
    # V: seq_len 0 is a no-op
    vp = v_planes_np(B, H, 8, D)
    orc.v_cache_save(*vp, u8(k[:, :4]), B, H, 8, D, 0, 0)
    assert not any(p.any() for p in vp)


# ------------------------------------------------------------------ golden vectors from the reference kernels
@pytest.fixture(scope="module")
def gold():
    assert os.path.exists(GOLD), "tests/golden/ref_kernels.npz is missing"
    return np.load(GOLD)


def test_oracle_reproduces_reference_kernel_outputs(gold):
    B, H, D, L, MAXLEN = 1, 4, 128, 128, 192
    nmb = 3
    k, v, q = make_kvq(101, B, L + 64 + 1, H, D)
    kp = k_planes_np(B, H, nmb, D)
    orc.k_cache_save(*kp, u8(k[:, :L]), B, H, L // 64, nmb, D, 64, 0, L)
    orc.k_cache_save(*kp, u8(k[:, L:L + 64]), B, H, 1, nmb, D, 64, L, 64)
    assert np.array_equal(np.concatenate([p.reshape(-1) for p in kp]), gold["k_planes_after_flush"])
    kp2 = [p.copy() for p in kp]
    orc.k_cache_save(*kp2, u8(k[:, L + 64:L + 65]), B, H, 0, nmb, D, 64, 70, 1)
    assert np.array_equal(np.concatenate([p.reshape(-1) for p in kp2]), gold["k_planes_after_token"])
    kexp = exponent_field(k[:, :L + 64].max(axis=1, keepdims=True))
    kq = (exponent_field(q) + kexp).astype(np.uint8)
    kqmax = kq.max(axis=3, keepdims=True)
    for reference in (False, True):
        s, _ = orc.k_cache_compute(*kp, kq, kqmax, u8(q), B, H, 3, nmb, D, 64, L + 64, 1.0 / math.sqrt(D), reference)
        assert np.array_equal(s.view(np.uint16)[..., :192], gold[f"k_scores_ref{int(reference)}"])
    vp = v_planes_np(B, H, MAXLEN, D)
    orc.v_cache_save(*vp, u8(v[:, :L]), B, H, MAXLEN, D, 0, L)
    orc.v_cache_save(*vp, u8(v[:, L:L + 64]), B, H, MAXLEN, D, L, 64)
    assert np.array_equal(np.concatenate([p.reshape(-1) for p in vp]), gold["v_planes"])
    n = L + 64
    p = softmax_probs(102, B, H, n, pad=64)
    grp = p[..., :n].reshape(B, H, n // 32, 32)
    val = np.ascontiguousarray(grp.max(axis=2, keepdims=True))
    idx = grp.argmax(axis=2).astype(np.int32)[:, :, None, :]
    o = orc.v_cache_test_compute(*vp, u8(val), u8(idx), B, H, MAXLEN, D, 32)
    assert np.array_equal(o.view(np.uint16), gold["v_probe"])
    pe = int(exponent_field(p[..., :n]).max())
    seen = set()
    for shift in (0, 2, 5):
        amin = np.full((B, H, H, 1), max(pe - shift, 0), np.uint8)
        for reference in (False, True):
            o, codes = orc.v_cache_compute(*vp, u8(p), amin, B, H, MAXLEN, D, p.shape[-1], n, reference)
            assert np.array_equal(o.view(np.uint16), gold[f"v_out_shift{shift}_ref{int(reference)}"])
            seen |= set(np.unique(codes))
    assert seen == {0, 1, 2}
