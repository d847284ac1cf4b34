"""CPU tests of the oracle: soft fp16, closed forms, the reference tests' own CPU formulas."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import h16, pattern_value, wkv_inputs


def test_soft_fp16_conversion_matches_ieee():
    rng = np.random.default_rng(1)
    xs = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in (1e-7, 1e-5, 1e-3, 1, 100, 30000)])
    xs = np.concatenate([xs, np.float32([0, -0.0, 65504, 65519.9, 65520, 2 ** -24, 2 ** -25, 3 * 2 ** -26])])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([orc.f2h(float(x)) for x in xs], np.uint16)
    assert (got == want).all()


def test_soft_fp16_fma_single_rounding():
    # product at an exact tie of the half grid, addend far below double's ulp of the product:
    # a double-rounded fma returns the even neighbour, a true fma must follow the addend
    a = np.float16(1 + 2 ** -10).view(np.uint16)      # 1.0009765625
    b = np.float16(1 + 2 ** -1).view(np.uint16)       # 1.5 -> product 1.50146484375 = tie of 11-bit grid
    tiny = np.float16(2 ** -24).view(np.uint16)
    up = orc.hfma(int(a), int(b), int(tiny))
    down = orc.hfma(int(a), int(b), int(tiny) | 0x8000)
    assert up == down + 1
    # numpy reference on random operands: exact in float64 when exponents are close
    rng = np.random.default_rng(2)
    v = h16(rng.standard_normal((2000, 3)))
    for x, y, z in v:
        exact = np.float64(x) * np.float64(y) + np.float64(z)
        assert orc.hfma(int(x.view(np.uint16)), int(y.view(np.uint16)), int(z.view(np.uint16))) == np.float16(exact).view(np.uint16)


def test_layer_norm_family_matches_reference_test_formulas():
    # the inline fp32 CPU references of test/cuda_non4096_kernels_test.cpp:84-213 at C=2560, rows 3,
    # same pattern_value inputs, same 2.5e-2 acceptance level
    C, rows = 2560, 3
    idx = np.arange(rows * C)
    x = h16(pattern_value(idx, 0.75, 0.05)).reshape(rows, C)
    res = h16(pattern_value(idx + 17, 0.5, -0.03)).reshape(rows, C)
    w = h16(pattern_value(np.arange(C) + 3, 0.25, 1.0))
    b = h16(pattern_value(np.arange(C) + 5, 0.1, 0.0))
    xk = h16(pattern_value(np.arange(C) + 7, 0.2, 0.5))
    shift = h16(pattern_value(idx + 29, 0.6, 0.01)).reshape(rows, C)

    v = x.astype(np.float32) + res.astype(np.float32)
    mean = v.mean(axis=1, keepdims=True)
    var = ((v - mean) ** 2).mean(axis=1, keepdims=True)
    yv = (v - mean) / np.sqrt(var + 1e-5) * w.astype(np.float32) + b.astype(np.float32)
    want_mixed = yv + (shift.astype(np.float32) - yv) * xk.astype(np.float32)

    xo, n = orc.add_layer_norm(x, res, w, b)
    np.testing.assert_allclose(xo.astype(np.float32), v, atol=2.5e-2)
    np.testing.assert_allclose(n.astype(np.float32), yv, atol=2.5e-2)
    sh = shift.copy()
    mixed = orc.cmix_mix(rows, 1, n, sh, xk)       # T=1: every row is its own sequence
    np.testing.assert_allclose(mixed.astype(np.float32), want_mixed, atol=2.5e-2)
    assert (sh == n).all()                          # shift state replaced by the LayerNorm output
    last = orc.add_last_layer_norm(1, rows, x, res, w, b)
    np.testing.assert_allclose(last.astype(np.float32), yv[-1:], atol=2.5e-2)


def test_wkv_fp32_matches_float64_recurrence():
    B, T, H = 2, 5, 2
    r, w, k, v, a, b = wkv_inputs(B, T, H, seed=3)
    state = np.zeros((B, H, 64, 64), np.float32)
    y = orc.wkv_fp32(B, T, H, state, r, w, k, v, a, b)
    S = np.zeros((B, H, 64, 64))
    want = np.zeros((B * T, H * 64))
    f = lambda z: z.astype(np.float64).reshape(B, T, H, 64)
    rr, ww, kk, vv, aa, bb = map(f, (r, w, k, v, a, b))
    dec = np.exp(-np.exp(-0.5) / (1 + np.exp(-ww)))
    for t in range(T):
        for bi in range(B):
            for h in range(H):
                s = S[bi, h]
                sa = s @ aa[bi, t, h]
                s = s * dec[bi, t, h][None, :] + np.outer(sa, bb[bi, t, h]) + np.outer(vv[bi, t, h], kk[bi, t, h])
                S[bi, h] = s
                want[bi * T + t, h * 64:(h + 1) * 64] = s @ rr[bi, t, h]
    np.testing.assert_allclose(state, S, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(y.astype(np.float64), want, rtol=2e-3, atol=2e-3)


def test_wkv_fp16_tracks_fp32_and_uses_elapsed_dither():
    B, T, H = 1, 16, 2
    r, w, k, v, a, b = wkv_inputs(B, T, H, seed=4)
    s32 = np.zeros((B, H, 64, 64), np.float32)
    y32 = orc.wkv_fp32(B, T, H, s32, r, w, k, v, a, b)
    s16 = np.zeros((B, H, 64, 64), np.float16)
    y16 = orc.wkv_fp16(B, T, H, s16, r, w, None, k, v, a, b, np.zeros(B, np.int32))
    assert np.abs(y16.astype(np.float32) - y32.astype(np.float32)).max() < 0.25
    s16b = np.zeros((B, H, 64, 64), np.float16)
    orc.wkv_fp16(B, T, H, s16b, r, w, None, k, v, a, b, np.full(B, 1000, np.int32))
    assert (s16b != s16).any()                      # the dither phase depends on elapsed
    # w0 folded in fp32 inside the kernel == adding it beforehand when the sum is exact in fp16
    w0 = np.zeros(H * 64, np.float16)
    s16c = np.zeros((B, H, 64, 64), np.float16)
    y16c = orc.wkv_fp16(B, T, H, s16c, r, w, w0, k, v, a, b, np.zeros(B, np.int32))
    assert (y16c == y16).all() and (s16c == s16).all()


def test_quant_formats_known_answers():
    # W8: scale = max|w|/127 ; values on the grid survive a round trip exactly
    W = h16([[0.0, 1.0, -1.0, 0.5, 0.25, -0.75, 0.125, 1.0] * 4])
    q, s = orc.quant_pack_w8(W)
    assert s[0] == np.float16(1.0 / 127.0)
    assert q[0, 1] == 127 and q[0, 2] == -127 and q[0, 0] == 0
    W2 = orc.quant_unpack_w8(q, s)
    q2, s2 = orc.quant_pack_w8(W2)
    assert (q2 == q).all() and (s2 == s).all()      # pack . unpack is idempotent on the grid
    # W4: a ramp 0..15 times 0.5 -> scale 0.5, zero 0, nibbles 0..15, low nibble = even element
    ramp = np.tile(np.arange(16, dtype=np.float32) * 0.5, 8)[None, :]
    q4, s4, z4 = orc.quant_pack_w4(h16(ramp))
    assert s4[0, 0] == np.float16(0.5) and z4[0, 0] == 0
    assert q4[0, 0] == (0 | (1 << 4)) and q4[0, 7] == (14 | (15 << 4))
    assert (orc.quant_unpack_w4(q4, s4, z4).astype(np.float32) == ramp).all()
    # negative range: zero point moves, all-zero group stays zero
    neg = np.tile(np.linspace(-1.5, 0.0, 16, dtype=np.float32), 8)[None, :]
    q4n, s4n, z4n = orc.quant_pack_w4(h16(neg))
    assert z4n[0, 0] == 15 and (q4n[0] & 15).min() == 0
    qz, sz, zz = orc.quant_pack_w4(np.zeros((1, 128), np.float16))
    assert (orc.quant_unpack_w4(qz, sz, zz) == 0).all()
    rng = np.random.default_rng(5)
    Wr = h16(rng.standard_normal((8, 256)) * 0.02)
    qa, sa, za = orc.quant_pack_w4(Wr)
    Wd = orc.quant_unpack_w4(qa, sa, za)
    assert np.abs(Wd.astype(np.float32) - Wr.astype(np.float32)).max() <= sa.astype(np.float32).max() * 0.51


def test_quant_linear_equals_linear_on_dequantised_weights():
    rng = np.random.default_rng(6)
    x = h16(rng.standard_normal((2, 256)))
    W = h16(rng.standard_normal((16, 256)) * 0.02)
    q4, s4, z4 = orc.quant_pack_w4(W)
    assert (orc.linear_w4a16(x, q4, s4, z4) == orc.linear_orig(x, orc.quant_unpack_w4(q4, s4, z4))).all()
    q8, s8 = orc.quant_pack_w8(W)
    y8 = orc.linear_w8a16(x, q8, s8).astype(np.float32)
    want = (x.astype(np.float64) @ q8.astype(np.float64).T) * s8.astype(np.float64)[None, :]
    np.testing.assert_allclose(y8, want, rtol=2e-3, atol=1e-4)
