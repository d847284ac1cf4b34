"""GPU parity tests of the op-level C-ABI entry points against the CPU oracle, and (when the
reference build under oracle/_ref is present) against the reference's own kernels on the same GPU.

Tolerances: integer/byte work (quant pack/unpack) bit-exact; fp16 outputs within 2 fp16 ulp of
the oracle with at least 97 % of the elements identical (the oracle sums in double, the kernels
in fp32, so results on a rounding boundary may differ by one ulp); the fp16-state WKV must equal
the reference's kernel bit for bit."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import h16, pattern_value, ref_lib, ulp_diff16, wkv_inputs

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def assert_close16(got, want, max_ulp=2, min_exact=0.97, what="", atol=1e-5):
    """ulp distance, except that differences below `atol` never count: next to zero an fp16 ulp
    (6e-8 for subnormals) is smaller than the rounding error of an fp32 dot product."""
    d = ulp_diff16(got, want)
    d = np.where(np.abs(got.astype(np.float32) - want.astype(np.float32)) <= atol, np.minimum(d, 1), d)
    exact = float((d == 0).mean())
    print(f"[parity] {what}: max ulp {int(d.max())}, exact {exact:.4f}")
    assert d.max() <= max_ulp, f"{what}: max ulp diff {d.max()}"
    assert exact >= min_exact, f"{what}: only {exact:.3f} of the elements identical"


@pytest.fixture(scope="module")
def ops():
    from rwkv_lightning_cuda_b200 import ops as o
    return o


def _p(t):
    return C.c_void_p(t.data_ptr())


@pytest.mark.parametrize("rows,Cc", [(1, 768), (3, 2560), (2, 4096), (5, 64)])
def test_layer_norm_family(ops, rows, Cc):
    idx = np.arange(rows * Cc)
    x = h16(pattern_value(idx, 0.75, 0.05)).reshape(rows, Cc)
    res = h16(pattern_value(idx + 17, 0.5, -0.03)).reshape(rows, Cc)
    w = h16(pattern_value(np.arange(Cc) + 3, 0.25, 1.0))
    b = h16(pattern_value(np.arange(Cc) + 5, 0.1, 0.0))
    assert_close16(host(ops.layer_norm_f16(dev(x), dev(w), dev(b))), orc.layer_norm(x, w, b), what="layer_norm")
    xo, y = ops.add_layer_norm_f16(dev(x), dev(res), dev(w), dev(b))
    oxo, oy = orc.add_layer_norm(x, res, w, b)
    assert (host(xo) == oxo).all()
    assert_close16(host(y), oy, what="add_layer_norm")
    # the reference test's own acceptance level (test/cuda_non4096_kernels_test.cpp:283-339)
    np.testing.assert_allclose(host(y).astype(np.float32), oy.astype(np.float32), atol=2.5e-2)
    last = ops.add_last_layer_norm_f16(1, rows, dev(x), dev(res), dev(w), dev(b))
    assert_close16(host(last), orc.add_last_layer_norm(1, rows, x, res, w, b), what="add_last_layer_norm")


@pytest.mark.parametrize("B,T,Cc", [(1, 1, 768), (2, 1, 2560), (1, 5, 768), (3, 4, 128), (2, 17, 256)])
def test_token_shift_fusions(ops, B, T, Cc):
    rng = np.random.default_rng(B * 100 + T)
    rows = B * T
    x = h16(rng.standard_normal((rows, Cc)))
    res = h16(rng.standard_normal((rows, Cc)) * 0.5)
    w = h16(1 + 0.1 * rng.standard_normal(Cc)); b = h16(0.1 * rng.standard_normal(Cc))
    mixes = [h16(rng.uniform(0, 1, Cc)) for _ in range(6)]
    shift0 = h16(rng.standard_normal((B, Cc)))

    # plain token shifts
    sh = dev(shift0.copy()); osh = shift0.copy()
    outs = ops.tmix_mix6(B, T, dev(x), sh, [dev(m) for m in mixes])
    oouts = orc.tmix_mix6(B, T, x, osh, mixes)
    for g, o in zip(outs, oouts):
        assert_close16(host(g), o, max_ulp=1, what="tmix_mix6")
    assert (host(sh) == osh).all()
    sh = dev(shift0.copy()); osh = shift0.copy()
    assert_close16(host(ops.cmix_mix(B, T, dev(x), sh, dev(mixes[0]))), orc.cmix_mix(B, T, x, osh, mixes[0]), max_ulp=1, what="cmix_mix")
    assert (host(sh) == osh).all()

    # residual + LayerNorm + shift, for every T (the reference fuses these for T == 1 only)
    oxo, on = orc.add_layer_norm(x, res, w, b)
    osh = shift0.copy()
    omixed = orc.cmix_mix(B, T, on, osh, mixes[2])
    sh = dev(shift0.copy())
    xo, mixed = ops.add_layer_norm_cmix_mix_f16(B, T, dev(x), dev(res), sh, dev(w), dev(b), dev(mixes[2]))
    assert (host(xo) == oxo).all()
    assert_close16(host(mixed), omixed, max_ulp=3, min_exact=0.9, what="add_ln_cmix_mix")
    assert_close16(host(sh), osh, what="shift after add_ln_cmix_mix")
    osh = shift0.copy()
    oouts = orc.tmix_mix6(B, T, on, osh, mixes)
    sh = dev(shift0.copy())
    xo, outs = ops.add_layer_norm_tmix_mix6_f16(B, T, dev(x), dev(res), sh, dev(w), dev(b), [dev(m) for m in mixes])
    assert (host(xo) == oxo).all()
    for g, o in zip(outs, oouts):
        assert_close16(host(g), o, max_ulp=3, min_exact=0.9, what="add_ln_tmix_mix6")
    assert_close16(host(sh), osh, what="shift after add_ln_tmix_mix6")


@pytest.mark.parametrize("rows,H", [(1, 12), (7, 2), (3, 40)])
def test_head_gates(ops, rows, H):
    rng = np.random.default_rng(rows + H)
    Cc = H * 64
    k = h16(rng.standard_normal((rows, Cc))); a12 = h16(rng.standard_normal((rows, Cc)))
    k_k = h16(rng.uniform(0.5, 1.5, Cc)); a0 = h16(rng.standard_normal(Cc)); k_a = h16(rng.uniform(0, 1, Cc))
    got = ops.tmix_kk_a_gate(rows, 1, H, dev(k), dev(k_k), dev(a0), dev(a12), dev(k_a))
    want = orc.kk_a_gate(k, k_k, a0, a12, k_a)
    for g, o, n in zip(got, want, ("new_k", "neg_kk", "kka")):
        assert_close16(host(g), o, what="kk_a_gate " + n)
    y = h16(rng.standard_normal((rows, Cc)) * 3); r = h16(rng.standard_normal((rows, Cc)))
    v = h16(rng.standard_normal((rows, Cc))); g = h16(rng.standard_normal((rows, Cc)))
    r_k = h16(rng.standard_normal(Cc) * 0.1); lw = h16(1 + 0.1 * rng.standard_normal(Cc)); lb = h16(0.1 * rng.standard_normal(Cc))
    got = ops.tmix_lnx_rkvres_xg(rows, 1, H, dev(y), dev(r), dev(k), dev(v), dev(r_k), dev(lw), dev(lb), dev(g))
    assert_close16(host(got), orc.lnx_rkvres_xg(y, r, k, v, r_k, lw, lb, g), what="lnx_rkvres_xg")
    vf = h16(rng.standard_normal((rows, Cc))); v0 = h16(rng.standard_normal(Cc)); v12 = h16(rng.standard_normal((rows, Cc)))
    assert_close16(host(ops.tmix_vres_gate(rows, 1, dev(v), dev(vf), dev(v0), dev(v12))), orc.vres_gate(v, vf, v0, v12), what="vres_gate")
    assert (host(ops.relu_square(dev(y))) == h16(np.maximum(y.astype(np.float32), 0) ** 2)).all()


@pytest.mark.parametrize("M,K,N", [(1, 768, 768), (2, 2560, 96), (4, 64, 768), (3, 4096, 130), (1, 3072, 768), (6, 256, 64),
                                   (128, 768, 768), (300, 1024, 640), (17, 96, 96), (256, 4096, 256),
                                   # 65 .. 128 rows, ragged N, K long enough for split-K
                                   (65, 256, 260), (100, 4096, 520), (128, 2048, 132), (96, 64, 1024)])
def test_linear_fp16(ops, M, K, N):
    from rwkv_lightning_cuda_b200 import lib as L
    rng = np.random.default_rng(M * 7 + N)
    x = h16(rng.standard_normal((M, K))); W = h16(rng.standard_normal((N, K)) * 0.02)
    assert_close16(host(ops.linear_f16_orig(dev(x), dev(W))), orc.linear_orig(x, W), max_ulp=1 if M <= 4 else 2, what="linear")
    # rows > 4 run on the tensor cores, whose fp32 accumulation is not round-to-nearest at every step
    assert_close16(host(ops.linear_f16_orig(dev(x), dev(W), epilogue=L.EPI_RELU2)), orc.linear_orig(x, W, epi=orc.EPI_RELU2),
                   max_ulp=2 if M <= 4 else 4, min_exact=0.97 if M <= 4 else 0.95, what="linear relu2")
    for act in (L.ACT_TANH, L.ACT_SIGMOID):
        # the kernels (like the reference, built with fast-math) use the hardware tanh/exp approximations
        got, want = host(ops.linear_f16_orig(dev(x), dev(W), in_act=act)), orc.linear_orig(x, W, in_act=act)
        np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), atol=2e-3, rtol=2e-3)
        if K <= 1024:
            assert_close16(got, want, max_ulp=2, min_exact=0.9, what="linear act")
    lg = host(ops.linear_f16_orig(dev(x), dev(W), epilogue=L.EPI_F32))
    assert lg.dtype == np.float32
    assert_close16(lg.astype(np.float16), orc.linear_orig(x, W), max_ulp=1 if M <= 4 else 2, what="linear f32 out")
    assert (lg == lg.astype(np.float16).astype(np.float32)).all()   # logits are fp16 values widened


@pytest.mark.parametrize("N,K", [(64, 256), (5, 1024), (130, 128)])
def test_quant_pack_bit_exact_and_linear(ops, N, K):
    rng = np.random.default_rng(N + K)
    W = h16(rng.standard_normal((N, K)) * 0.02)
    W[0, :128] = 0                                     # all-zero group / edge case
    W[1 % N, :] = np.float16(0.01)                     # constant row
    q8, s8 = ops.quant_pack_w8(dev(W)); oq8, os8 = orc.quant_pack_w8(W)
    assert (host(q8) == oq8).all() and (host(s8).view(np.uint16) == os8.view(np.uint16)).all()
    assert (host(ops.quant_unpack_w8(q8, s8)).view(np.uint16) == orc.quant_unpack_w8(oq8, os8).view(np.uint16)).all()
    q4, s4, z4 = ops.quant_pack_w4(dev(W)); oq4, os4, oz4 = orc.quant_pack_w4(W)
    assert (host(q4) == oq4).all() and (host(s4).view(np.uint16) == os4.view(np.uint16)).all() and (host(z4) == oz4).all()
    Wd = host(ops.quant_unpack_w4(q4, s4, z4))
    assert (Wd.view(np.uint16) == orc.quant_unpack_w4(oq4, os4, oz4).view(np.uint16)).all()
    # re-quantising dequantised W8 weights reproduces codes and scales (symmetric grid)
    W8d = ops.quant_unpack_w8(q8, s8)
    q8b, s8b = ops.quant_pack_w8(W8d)
    assert torch.equal(q8b, q8) and torch.equal(s8b, s8)
    for M in (1, 3):
        x = h16(rng.standard_normal((M, K)))
        assert_close16(host(ops.linear_w8a16(dev(x), q8, s8)), orc.linear_w8a16(x, oq8, os8), max_ulp=1, what="linear_w8a16")
        assert_close16(host(ops.linear_w4a16(dev(x), q4, s4, z4)), orc.linear_w4a16(x, oq4, os4, oz4), max_ulp=1, what="linear_w4a16")


@pytest.mark.parametrize("M,K,N", [(5, 256, 64), (64, 2048, 260), (256, 2560, 1024), (200, 1024, 132), (33, 8192, 128), (8, 128, 512)])
def test_linear_quantised_on_the_tensor_cores(ops, M, K, N):
    """More than four rows of W8A16 / W4A16 weights: the GEMM that expands the packed tiles in shared memory
    (ragged N, K long enough for split-K, K blocks that end in the middle of a 128-wide quantisation group)."""
    from rwkv_lightning_cuda_b200 import lib as L
    rng = np.random.default_rng(M + K + N)
    W = h16(rng.standard_normal((N, K)) * 0.02)
    W[0, :128] = 0
    W[N - 1, :] = np.float16(-0.015)
    x = h16(rng.standard_normal((M, K)))
    q8, s8 = orc.quant_pack_w8(W); q4, s4, z4 = orc.quant_pack_w4(W)
    got8 = host(ops.linear_w8a16(dev(x), dev(q8), dev(s8)))
    atol = 1e-5 * 4 * (K / 1024) ** 0.5     # near zero an fp16 ulp is smaller than the rounding of an fp32 sum of K products
    assert_close16(got8, orc.linear_w8a16(x, q8, s8), max_ulp=2, min_exact=0.95, what="linear_w8a16, tensor cores", atol=atol)
    got4 = host(ops.linear_w4a16(dev(x), dev(q4), dev(s4), dev(z4)))
    assert_close16(got4, orc.linear_w4a16(x, q4, s4, z4), max_ulp=2, min_exact=0.95, what="linear_w4a16, tensor cores", atol=atol)
    r4 = host(ops.linear_w4a16(dev(x), dev(q4), dev(s4), dev(z4), epilogue=L.EPI_RELU2))
    assert_close16(r4, orc.linear_w4a16(x, q4, s4, z4, epi=orc.EPI_RELU2), max_ulp=4, min_exact=0.95, what="linear_w4a16 relu2", atol=atol)
    assert L.timeout_flags(clear=True) == 0


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4100), (4, 4096, 1000), (2, 16384, 256), (3, 2560, 132), (1, 768, 64), (4, 10240, 48),
                                   (2, 256, 16), (1, 2048, 20)])
def test_linear_one_to_four_rows_on_the_warp_level_tensor_core_instruction(ops, M, K, N):
    """1..4 rows: 16-channel weight tiles (2-D tensor copies, 128-byte swizzle) against the activations with
    mma.sync -- W8A16 and W4A16 always, fp16 by option.  Channel counts that leave ragged tiles of 4, 8 and 12
    channels per CTA, K from one 128-byte box per row to many per warp, all epilogues the decode path uses."""
    from rwkv_lightning_cuda_b200 import lib as L
    rng = np.random.default_rng(M + K + N)
    W = h16(rng.standard_normal((N, K)) * 0.02)
    W[0, :128] = 0
    W[N - 1, :] = np.float16(-0.015)
    x = h16(rng.standard_normal((M, K)))
    q8, s8 = orc.quant_pack_w8(W); q4, s4, z4 = orc.quant_pack_w4(W)
    atol = 1e-5 * 4 * (K / 1024) ** 0.5
    got8 = host(ops.linear_w8a16(dev(x), dev(q8), dev(s8)))
    assert_close16(got8, orc.linear_w8a16(x, q8, s8), max_ulp=2, min_exact=0.97, what="linear_w8a16, mma", atol=atol)
    got4 = host(ops.linear_w4a16(dev(x), dev(q4), dev(s4), dev(z4)))
    assert_close16(got4, orc.linear_w4a16(x, q4, s4, z4), max_ulp=2, min_exact=0.97, what="linear_w4a16, mma", atol=atol)
    r4 = host(ops.linear_w4a16(dev(x), dev(q4), dev(s4), dev(z4), epilogue=L.EPI_RELU2))
    assert_close16(r4, orc.linear_w4a16(x, q4, s4, z4, epi=orc.EPI_RELU2), max_ulp=4, min_exact=0.95, what="linear_w4a16 relu2, mma", atol=atol)
    L.set_option("gemv_mma", 4)          # every launch the kernel accepts, whatever its size (fp16 and one row included)
    try:
        got = host(ops.linear_f16_orig(dev(x), dev(W)))
        lg = host(ops.linear_f16_orig(dev(x), dev(W), epilogue=L.EPI_F32))
        got8b = host(ops.linear_w8a16(dev(x), dev(q8), dev(s8)))
        L.set_option("gemv_mma_tall", 0)  # tiles of 16 channels
        got16 = host(ops.linear_f16_orig(dev(x), dev(W)))
        got4_16 = host(ops.linear_w4a16(dev(x), dev(q4), dev(s4), dev(z4)))
        L.set_option("gemv_mma_tall", 3)
        got4_32 = host(ops.linear_w4a16(dev(x), dev(q4), dev(s4), dev(z4)))
        got32 = host(ops.linear_f16_orig(dev(x), dev(W)))
    finally:
        L.set_option("gemv_mma", 3)
        L.set_option("gemv_mma_tall", 2)
    assert_close16(got, orc.linear_orig(x, W), max_ulp=2, min_exact=0.97, what="linear fp16, mma", atol=atol)
    assert (lg.astype(np.float16).view(np.uint16) == got.view(np.uint16)).all()
    assert_close16(got8b, orc.linear_w8a16(x, q8, s8), max_ulp=2, min_exact=0.97, what="linear_w8a16, mma, any size", atol=atol)
    # (the same sums in the same order when a row has a multiple of 16 boxes; otherwise the boxes fall to other warps)
    exact = (K * 2) % 2048 == 0
    assert_close16(got32, got16, max_ulp=0 if exact else 2, min_exact=1.0 if exact else 0.95, what="fp16, tiles of 32 vs 16", atol=0 if exact else atol)
    exact4 = (K // 2) % 2048 == 0
    assert_close16(got4_32, got4_16, max_ulp=0 if exact4 else 2, min_exact=1.0 if exact4 else 0.95, what="W4A16, tiles of 32 vs 16", atol=0 if exact4 else atol)
    assert_close16(got4_32, orc.linear_w4a16(x, q4, s4, z4), max_ulp=2, min_exact=0.97, what="linear_w4a16, mma, tiles of 32", atol=atol)
    # the scalar kernels give the same values up to the order of the fp32 sums
    L.set_option("gemv_mma", 0)
    try:
        old8 = host(ops.linear_w8a16(dev(x), dev(q8), dev(s8)))
    finally:
        L.set_option("gemv_mma", 3)
    assert_close16(got8b, old8, max_ulp=2, min_exact=0.95, what="mma vs scalar kernel", atol=atol)
    assert L.timeout_flags(clear=True) == 0


@pytest.mark.parametrize("B,T,H", [(1, 128, 12), (3, 1, 2), (2, 7, 3), (1, 1, 64),
                                   # 64 tokens and more: the matrix form on the tensor cores (ragged ends, several blocks)
                                   (1, 128, 64), (2, 100, 3), (1, 65, 2), (1, 256, 4), (3, 64, 2)])
def test_wkv_fp32(ops, B, T, H):
    r, w, k, v, a, b = wkv_inputs(B, T, H, seed=B * 10 + T)
    rng = np.random.default_rng(9)
    s0 = (rng.standard_normal((B, H, 64, 64)) * (0.0 if T == 128 else 0.5)).astype(np.float32)
    os_ = s0.copy()
    oy = orc.wkv_fp32(B, T, H, os_, r, w, k, v, a, b)
    st = dev(s0.copy())
    y = ops.wkv_fp32io16(B, T, H, st, *(dev(t) for t in (r, w, k, v, a, b)))
    gs = host(st)
    rel = np.abs(gs - os_).max() / max(np.abs(os_).max(), 1e-6)
    print(f"[parity] wkv_fp32 B={B} T={T} H={H}: state rel err {rel:.2e}")
    assert rel < 1e-4          # the stated tolerance for the fp32 state
    # The matrix form (T >= 64) sums the same products in another order and in split-TF32 arithmetic: its absolute error
    # is a few 1e-6 of the LARGEST output, which is many fp16 ulps of an output that happens to lie next to zero.
    atol = max(1e-5, 4e-6 * float(np.abs(oy.astype(np.float32)).max())) if T >= 64 else 1e-5
    assert_close16(host(y), oy, max_ulp=2, min_exact=0.9, what="wkv_fp32 y", atol=atol)
    if T >= 64:                # the matrix form against the per-token scan of the same library
        from rwkv_lightning_cuda_b200 import lib as L
        L.set_option("wkv_chunked", 0)
        try:
            st2 = dev(s0.copy())
            y2 = ops.wkv_fp32io16(B, T, H, st2, *(dev(t) for t in (r, w, k, v, a, b)))
        finally:
            L.set_option("wkv_chunked", 1)
        rel2 = np.abs(gs - host(st2)).max() / max(np.abs(host(st2)).max(), 1e-6)
        print(f"[parity] wkv_fp32 matrix form vs scan B={B} T={T} H={H}: state rel err {rel2:.2e}")
        assert rel2 < 1e-4
        assert_close16(host(y), host(y2), max_ulp=2, min_exact=0.9, what="wkv_fp32 y, matrix form vs scan", atol=atol)


@pytest.mark.parametrize("B,T,H,use_w0", [(1, 128, 12, False), (2, 1, 3, True), (3, 9, 2, True), (1, 16, 4, False)])
def test_wkv_fp16(ops, B, T, H, use_w0):
    r, w, k, v, a, b = wkv_inputs(B, T, H, seed=B * 10 + T)
    rng = np.random.default_rng(11)
    s0 = h16(rng.standard_normal((B, H, 64, 64)) * (0.0 if T == 128 else 0.5))
    elapsed = np.arange(B, dtype=np.int32) * 977 + 5
    w0 = h16(rng.uniform(-1, 1, H * 64)) if use_w0 else None
    os_ = s0.copy()
    oy = orc.wkv_fp16(B, T, H, os_, r, w, w0, k, v, a, b, elapsed)
    st = dev(s0.copy())
    y = ops.wkv_fp16_seq(B, T, H, st, *(dev(t) for t in (r, w, k, v, a, b)), dev(elapsed), w0=None if w0 is None else dev(w0))
    gy, gs = host(y), host(st)
    # vs the CPU oracle: identical half arithmetic; only the decay (exp2 / reciprocal approximations on
    # the GPU) can differ by one fp16 ulp on a rounding boundary, which then spreads through the row
    dy = np.abs(gy.astype(np.float32) - oy.astype(np.float32))
    print(f"[parity] wkv_fp16 B={B} T={T}: y exact {(gy.view(np.uint16) == oy.view(np.uint16)).mean():.4f} max abs {dy.max():.3e}; "
          f"state exact {(gs.view(np.uint16) == os_.view(np.uint16)).mean():.4f}")
    assert dy.max() <= 2e-2 * max(1.0, float(np.abs(oy.astype(np.float32)).max()))
    ref = ref_lib()
    if ref is not None:
        st2 = dev(s0.copy()); y2 = torch.empty_like(y)
        args = [_p(dev(t)) for t in (r, w)]
        tens = {n: dev(t) for n, t in zip("rwkvab", (r, w, k, v, a, b))}
        el = dev(elapsed)
        if w0 is None:
            rc = ref.ref_wkv_fp16_seq(B, T, H * 64, H, _p(st2), _p(tens["r"]), _p(tens["w"]), _p(tens["k"]), _p(tens["v"]),
                                      _p(tens["a"]), _p(tens["b"]), _p(y2), _p(el))
        else:
            w0d = dev(w0)
            rc = ref.ref_wkv_fp16_seq_w0(B, T, H * 64, H, _p(st2), _p(tens["r"]), _p(tens["w"]), _p(w0d), _p(tens["k"]), _p(tens["v"]),
                                         _p(tens["a"]), _p(tens["b"]), _p(y2), _p(el))
        assert rc == 0, ref.ref_last_error()
        assert (host(y2).view(np.uint16) == gy.view(np.uint16)).all(), "fp16 WKV output differs from the reference kernel"
        assert (host(st2).view(np.uint16) == gs.view(np.uint16)).all(), "fp16 WKV state differs from the reference kernel"


def test_emb_ln0_and_advance(ops):
    rng = np.random.default_rng(12)
    V, Cc = 50, 768
    emb = torch.from_numpy(rng.standard_normal((V, Cc)).astype(np.float32) * 0.02).to(torch.bfloat16)
    w = torch.from_numpy(1 + 0.02 * rng.standard_normal(Cc).astype(np.float32)).to(torch.bfloat16)
    b = torch.from_numpy(0.02 * rng.standard_normal(Cc).astype(np.float32)).to(torch.bfloat16)
    got = host(ops.emb_ln0(emb.cuda(), w.cuda(), b.cuda()))
    want = orc.emb_ln0(emb.float().numpy(), w.float().numpy(), b.float().numpy())
    assert_close16(got, want, what="emb_ln0")
    np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), atol=3e-2)  # reference test level
    e = torch.arange(5, dtype=torch.int32).cuda()
    ops.advance_i32(e, 7)
    assert host(e).tolist() == [7, 8, 9, 10, 11]


def test_bad_arguments_return_status_not_abort(ops):
    from rwkv_lightning_cuda_b200 import lib as L
    x = torch.zeros((1, 100), dtype=torch.float16).cuda()
    W = torch.zeros((4, 100), dtype=torch.float16).cuda()
    with pytest.raises(L.Rwkv7B200Error) as e:
        ops.linear_f16_orig(x, W)          # K not a multiple of 8
    assert e.value.status == 2
    with pytest.raises(L.Rwkv7B200Error):
        ops.wkv_fp32io16(1, 1, 0, torch.zeros(1).cuda(), *([x] * 6))


def test_linear_fp16_cta_pair_kernel():
    """The opt-in CTA-pair (cta_group::2) variant of the tensor-core GEMM gives the same results.  The switch is
    process-wide, so the check runs in a child process."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import numpy as np, torch\n"
        "from oracle import oracle as orc\n"
        "from rwkv_lightning_cuda_b200 import ops, lib\n"
        "from tests.helpers import h16\n"
        "from tests.test_ops_gpu import assert_close16\n"
        "lib.set_option('gemm_cta_pair', 1)\n"
        "rng = np.random.default_rng(5)\n"
        "for M, K, N in ((256, 1024, 640), (40, 96, 130 * 2), (300, 512, 128)):\n"
        "    x = h16(rng.standard_normal((M, K))); W = h16(rng.standard_normal((N, K)) * 0.02)\n"
        "    got = ops.linear_f16_orig(torch.from_numpy(x).cuda(), torch.from_numpy(W).cuda()).cpu().numpy()\n"
        "    assert_close16(got, orc.linear_orig(x, W), max_ulp=2, what='linear (CTA pair)')\n"
        "    got = ops.linear_f16_orig_static(torch.from_numpy(x).cuda(), torch.from_numpy(W).cuda()).cpu().numpy()\n"
        "    assert_close16(got, orc.linear_orig(x, W), max_ulp=2, what='linear split-K (CTA pair)')\n"
        "print('pair ok')\n")
    env = dict(os.environ, PYTHONPATH=root)
    res = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "pair ok" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


def test_ops_match_the_reference_kernels_golden(ops):
    """The library's kernels against outputs of the reference's own kernels recorded on a B200 (tests/golden/ref_ops.npz)."""
    import os
    from tests.helpers import GOLDEN
    g = np.load(os.path.join(GOLDEN, "ref_ops.npz"))
    B, T, H = int(g["wkv_B"]), int(g["wkv_T"]), int(g["wkv_H"])
    ins = [dev(g["wkv_" + n]) for n in "rwkvab"]
    for tag, w0 in (("wkv16", None), ("wkv16w0", g["wkv_w0"])):
        st = dev(g["wkv_s0"].copy())
        y = ops.wkv_fp16_seq(B, T, H, st, *ins, dev(g["wkv_elapsed"]), w0=None if w0 is None else dev(w0))
        assert (host(y).view(np.uint16) == g[tag + "_y"].reshape(host(y).shape).view(np.uint16)).all(), tag      # same instruction sequence
        assert (host(st).view(np.uint16) == g[tag + "_state"].view(np.uint16)).all(), tag
    st = dev(g["wkv32_s0"].copy())
    y = ops.wkv_fp32io16(B, T, H, st, *ins)
    assert np.abs(host(st) - g["wkv32_state"]).max() / np.abs(g["wkv32_state"]).max() < 1e-4
    assert_close16(host(y).reshape(g["wkv32_y"].shape), g["wkv32_y"], max_ulp=2, min_exact=0.9, what="wkv_fp32 vs reference")
    rows = g["gate_k"].shape[0]; Hg = g["gate_k"].shape[1] // 64
    got = ops.tmix_kk_a_gate(rows, 1, Hg, dev(g["gate_k"]), dev(g["gate_k_k"]), dev(g["gate_a0"]), dev(g["gate_a12"]), dev(g["gate_k_a"]))
    for i, n in enumerate(("new_k", "neg_kk", "kka")):
        assert_close16(host(got[i]), g["gate_out"][i], what="kk_a_gate vs reference " + n)
    got = ops.tmix_lnx_rkvres_xg(rows, 1, Hg, dev(g["lnx_y"]), dev(g["lnx_r"]), dev(g["gate_k"]), dev(g["lnx_v"]), dev(g["lnx_r_k"]),
                                 dev(g["lnx_w"]), dev(g["lnx_b"]), dev(g["lnx_g"]))
    assert_close16(host(got), g["lnx_out"], what="lnx_rkvres_xg vs reference")
    assert_close16(host(ops.tmix_vres_gate(rows, 1, dev(g["lnx_v"]), dev(g["vres_vf"]), dev(g["vres_v0"]), dev(g["vres_v12"]))),
                   g["vres_out"], what="vres_gate vs reference")
    x, res, w, b = g["ln_x"], g["ln_res"], g["ln_w"], g["ln_b"]
    sh = dev(g["mix_shift0"].copy())
    xo, outs = ops.add_layer_norm_tmix_mix6_f16(x.shape[0], 1, dev(x), dev(res), sh, dev(w), dev(b), [dev(m) for m in g["mix_coef"]])
    assert (host(xo).view(np.uint16) == g["lnmix6_xo"].view(np.uint16)).all()
    for i in range(6):
        assert_close16(host(outs[i]), g["lnmix6_out"][i], max_ulp=3, min_exact=0.9, what=f"add_ln_tmix_mix6[{i}] vs reference")
    assert_close16(host(sh), g["lnmix6_shift"], what="shift vs reference")
    assert_close16(host(ops.linear_f16_orig(dev(g["lin_x"]), dev(g["lin_W"]))), g["lin_y"], max_ulp=1, what="linear vs reference GEMV")


@pytest.mark.parametrize("V", [65536, 1030, 8])     # 1030: rows not 16-byte aligned (scalar loads)
def test_greedy_pick_matches_the_oracle(V):
    """Bit-exact ids and penalties against the numpy restatement of the reference sampler's greedy case, with NaN and
    infinite logits, masked tokens, repeated maxima and two consecutive picks (penalty == 0 versus != 0 branches)."""
    from rwkv_lightning_cuda_b200 import ops
    rng = np.random.default_rng(V)
    B = 5
    logits = rng.standard_normal((B, V)).astype(np.float32) * 4
    logits[0, V // 2] = np.nan; logits[1, 1] = np.inf; logits[1, V - 1] = np.inf; logits[2, 0] = -np.inf
    logits[3, [2, V - 2]] = logits[3].max() + 1          # a tie: the lower id wins
    pen = (rng.random((B, V)) < 0.3).astype(np.float32) * rng.random((B, V)).astype(np.float32)
    pen[4, int(logits[4].argmax())] = np.inf             # the best token of row 4 is masked
    pen_g = torch.from_numpy(pen.copy()).cuda()
    lg = torch.from_numpy(logits).cuda()
    nxt = torch.zeros(B, dtype=torch.int64, device="cuda")
    for _ in range(2):
        want = orc.greedy_pick(logits, pen, 0.7, 0.45, 0.996)
        got = ops.greedy_pick(lg, pen_g, 0.7, 0.45, 0.996, next_tokens=nxt)
        assert got.cpu().tolist() == want.tolist() and nxt.cpu().tolist() == want.tolist()
        assert np.array_equal(pen_g.cpu().numpy(), pen, equal_nan=True)
    assert ops.greedy_pick(lg).cpu().tolist() == orc.greedy_pick(logits).tolist()


def test_sampler_temperature_topk_topp_against_the_oracle(ops):
    """The sampler's general case: what is kept (top-k / top-p with ties sharing what is left of the budgets), the draw
    as a function of (seed, offset, row), the penalty update, the greedy limit, and the frequencies of many draws."""
    rng = np.random.default_rng(3)
    B, V = 3, 512
    lg = (rng.standard_normal((B, V)) * 2.5).astype(np.float32)
    lg[1, 100:110] = lg[1, 100]                       # a run of exactly tied logits
    lg[2, 7] = np.inf; lg[2, 9] = np.nan              # clamped / zeroed like the reference does
    dl = dev(lg)
    # (1) top_p == 0 and top_k == 1 are the greedy choice (no tie at the top here)
    for kw in (dict(top_p=0.0), dict(top_k=1)):
        got = host(ops.sample(dl, temperature=0.7, seed=1, offset=0, **kw))
        assert got.tolist() == orc.greedy_pick(lg).tolist()
    # (2) the draw equals the oracle's for the same (seed, offset); penalties are updated the same way
    agree = total = 0
    for temperature, top_k, top_p in ((1.0, 0, 1.0), (0.8, 20, 1.0), (1.3, 0, 0.6), (0.5, 8, 0.9), (2.0, 200, 0.95)):
        pen_g = torch.zeros((B, V), dtype=torch.float32, device="cuda"); pen_o = np.zeros((B, V), dtype=np.float32)
        pen_o[0, 5] = 1.5; pen_g[0, 5] = 1.5
        for off in range(40):
            got = host(ops.sample(dl, pen_g, 0.4, 0.3, 0.9, temperature, top_k, top_p, seed=99, offset=off))
            want = orc.sample(lg, pen_o, 0.4, 0.3, 0.9, temperature, top_k, top_p, seed=99, offset=off)
            same = got == want
            agree += int(same.sum()); total += B
            if not same.all():                        # a draw on the boundary between two tokens (fp32 vs float64 sums): re-align
                pen_g.copy_(torch.from_numpy(pen_o))
            else:
                assert np.allclose(host(pen_g), pen_o, rtol=1e-6, atol=1e-7)
            kept = orc.sample_weights(lg, None, temperature, top_k, top_p)        # (penalties move little here)
    print(f"[parity] sampler draws equal to the oracle's: {agree}/{total}")
    assert agree >= 0.98 * total
    # (3) every drawn token lies in the kept set, and frequencies follow the kept weights
    small = (rng.standard_normal((1, 64)) * 1.5).astype(np.float32)
    w = orc.sample_weights(small, None, 0.9, 10, 0.85)[0]
    counts = np.zeros(64)
    n_draws = 6000
    ds = dev(np.repeat(small, 8, axis=0))             # eight rows per launch, each with its own counter
    for off in range(n_draws // 8):
        for tok in host(ops.sample(ds, temperature=0.9, top_k=10, top_p=0.85, seed=5, offset=off)):
            counts[tok] += 1
    assert (counts[w == 0] == 0).all()
    expect = w / w.sum() * n_draws
    chi2 = (((counts - expect) ** 2) / np.maximum(expect, 1e-9))[w > 0].sum()
    print(f"[parity] sampler frequencies over {n_draws} draws: chi2 {chi2:.1f} with {int((w > 0).sum()) - 1} degrees of freedom")
    assert chi2 < 5 * max(1, int((w > 0).sum()))
    # (4) same (seed, offset) -> same token; argument errors
    a = host(ops.sample(dl, temperature=1.0, seed=11, offset=4)); b = host(ops.sample(dl, temperature=1.0, seed=11, offset=4))
    assert (a == b).all()
    from rwkv_lightning_cuda_b200 import lib as L
    with pytest.raises(L.Rwkv7B200Error, match="temperature"):
        ops.sample(dl, temperature=0.0)
