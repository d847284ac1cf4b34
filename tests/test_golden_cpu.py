"""The CPU oracle against the golden fixtures: outputs of the REFERENCE's own CUDA kernels, and of its whole
ModelBackend on a small random-init checkpoint, recorded on a B200 by tests/golden/make_golden.py.  These pin the
oracle to the reference itself; the GPU tests then compare the library with the oracle and with the same files."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import GOLDEN, ulp_diff16


def close16(got, want, max_ulp, min_exact, what, atol=1e-5):
    d = ulp_diff16(got, want)
    d = np.where(np.abs(got.astype(np.float32) - want.astype(np.float32)) <= atol, np.minimum(d, 1), d)
    exact = float((d == 0).mean())
    print(f"[golden] {what}: max ulp {int(d.max())}, exact {exact:.4f}")
    assert d.max() <= max_ulp, f"{what}: max ulp diff {d.max()}"
    assert exact >= min_exact, f"{what}: only {exact:.3f} identical"


@pytest.fixture(scope="module")
def g():
    return np.load(os.path.join(GOLDEN, "ref_ops.npz"))


def test_wkv_fp16_state_matches_the_reference_kernels(g):
    B, T, H = int(g["wkv_B"]), int(g["wkv_T"]), int(g["wkv_H"])
    ins = [g["wkv_" + n] for n in "rwkvab"]
    for tag, w0 in (("wkv16", None), ("wkv16w0", g["wkv_w0"])):
        st = g["wkv_s0"].copy()
        y = orc.wkv_fp16(B, T, H, st, ins[0], ins[1], w0, ins[2], ins[3], ins[4], ins[5], g["wkv_elapsed"]).reshape(B, T, H * 64)
        # identical half arithmetic; the decay's exp2/reciprocal approximations on the GPU can move it by one ulp
        dy = np.abs(y.astype(np.float32) - g[tag + "_y"].astype(np.float32))
        assert dy.max() <= 2e-2 * max(1.0, float(np.abs(g[tag + "_y"].astype(np.float32)).max()))
        exact = (y.view(np.uint16) == g[tag + "_y"].view(np.uint16)).mean()
        print(f"[golden] {tag}: y exact {exact:.4f}, max abs {dy.max():.3e}")
        assert exact > 0.5
        ds = np.abs(st.astype(np.float32) - g[tag + "_state"].astype(np.float32))
        assert ds.max() <= 2e-2 * max(1.0, float(np.abs(g[tag + "_state"].astype(np.float32)).max()))


def test_wkv_fp32_state_matches_the_reference_kernel(g):
    B, T, H = int(g["wkv_B"]), int(g["wkv_T"]), int(g["wkv_H"])
    ins = [g["wkv_" + n] for n in "rwkvab"]
    st = g["wkv32_s0"].copy()
    y = orc.wkv_fp32(B, T, H, st, *ins).reshape(B, T, H * 64)
    rel = np.abs(st - g["wkv32_state"]).max() / max(np.abs(g["wkv32_state"]).max(), 1e-6)
    print(f"[golden] wkv_fp32: state rel err {rel:.2e}")
    assert rel < 1e-4
    close16(y, g["wkv32_y"], 2, 0.9, "wkv_fp32 y")


def test_row_kernels_match_the_reference_kernels(g):
    x, res, w, b = g["ln_x"], g["ln_res"], g["ln_w"], g["ln_b"]
    close16(orc.layer_norm(x, w, b), g["ln_y"], 1, 0.97, "layer_norm")
    xo, y = orc.add_layer_norm(x, res, w, b)
    assert (xo.view(np.uint16) == g["addln_xo"].view(np.uint16)).all()
    close16(y, g["addln_y"], 1, 0.97, "add_layer_norm")
    close16(orc.add_last_layer_norm(2, 3, x, res, w, b), g["addlast_y"], 1, 0.97, "add_last_layer_norm")
    mixes = [m for m in g["mix_coef"]]
    # chunked token shift on raw rows
    sh = g["mix_shift0"][:2].copy()
    outs = orc.tmix_mix6(2, 3, x, sh, mixes)
    for i in range(6):
        close16(outs[i], g["mix6_out"][i], 1, 0.97, f"tmix_mix6[{i}]")
    assert (sh.view(np.uint16) == g["mix6_shift"].view(np.uint16)).all()
    sh = g["mix_shift0"][:2].copy()
    close16(orc.cmix_mix(2, 3, x, sh, mixes[0]), g["cmix_out"], 1, 0.97, "cmix_mix")
    assert (sh.view(np.uint16) == g["cmix_shift"].view(np.uint16)).all()
    # decode rows: add + LayerNorm + token shift = the composition of the oracle's pieces
    xo, n = orc.add_layer_norm(x, res, w, b)
    sh = g["mix_shift0"].copy()
    outs = orc.tmix_mix6(x.shape[0], 1, n, sh, mixes)
    for i in range(6):
        close16(outs[i], g["lnmix6_out"][i], 3, 0.9, f"add_ln_tmix_mix6[{i}]")
    close16(sh, g["lnmix6_shift"], 1, 0.97, "shift after add_ln_tmix_mix6")
    sh = g["mix_shift0"].copy()
    close16(orc.cmix_mix(x.shape[0], 1, n, sh, mixes[0]), g["lncmix_out"], 3, 0.9, "add_ln_cmix_mix")


def test_head_gates_and_linear_match_the_reference_kernels(g):
    got = orc.kk_a_gate(g["gate_k"], g["gate_k_k"], g["gate_a0"], g["gate_a12"], g["gate_k_a"])
    for i, n in enumerate(("new_k", "neg_kk", "kka")):
        close16(got[i], g["gate_out"][i], 2, 0.95, "kk_a_gate " + n)
    close16(orc.lnx_rkvres_xg(g["lnx_y"], g["lnx_r"], g["gate_k"], g["lnx_v"], g["lnx_r_k"], g["lnx_w"], g["lnx_b"], g["lnx_g"]),
            g["lnx_out"], 2, 0.95, "lnx_rkvres_xg")
    close16(orc.vres_gate(g["lnx_v"], g["vres_vf"], g["vres_v0"], g["vres_v12"]), g["vres_out"], 2, 0.95, "vres_gate")
    close16(orc.linear_orig(g["lin_x"], g["lin_W"]), g["lin_y"], 1, 0.97, "linear_orig (reference GEMV)")


def golden_model_calls(tag, name="ref_model_tiny.npz"):
    m = np.load(os.path.join(GOLDEN, name))
    calls = [(m[f"{tag}_tok{i}"], m[f"{tag}_logits{i}"]) for i in range(int(m[tag + "_n"]))]
    return m, calls


def oracle_model(dims):
    import torch
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic
    d = bk.ModelDims(**dims)
    ck = synthetic.make_checkpoint(d, seed=0, device="cpu", dtype=torch.float16)
    table = orc.emb_ln0(ck["emb.weight"].float().numpy(), ck["blocks.0.ln0.weight"].float().numpy(), ck["blocks.0.ln0.bias"].float().numpy())
    om = orc.Model(d.layers, d.channels, d.ffn, d.vocab, d.rank_w, d.rank_a, d.rank_v, d.rank_g)
    om.set("emb_ln0", table)
    for name, t in ck.items():
        if name not in ("emb.weight", "blocks.0.ln0.weight", "blocks.0.ln0.bias"):
            om.set(name, t.numpy())
    return d, om, ck, table


GOLDEN_DIMS = dict(layers=2, channels=768, ffn=3072, vocab=1024, rank_w=64, rank_a=64, rank_v=32, rank_g=128)
GOLDEN_WIDE_DIMS = dict(layers=2, channels=4096, ffn=16384, vocab=1024, rank_w=128, rank_a=128, rank_v=96, rank_g=480)
# fixture file -> the dimensions its checkpoint was drawn with (seed 0)
GOLDEN_MODELS = {"ref_model_tiny.npz": GOLDEN_DIMS, "ref_model_c4096.npz": GOLDEN_WIDE_DIMS}
from oracle.parity import FP32_STATE_REL, fp32_state_bound_vs_reference  # noqa: E402,F401


def available_golden_models():
    return [n for n in GOLDEN_MODELS if os.path.exists(os.path.join(GOLDEN, n))]


@pytest.mark.parametrize("name", list(GOLDEN_MODELS))
@pytest.mark.parametrize("wkv32", [False, True])
def test_whole_model_matches_the_reference_backend(wkv32, name):
    """Two prefill chunks, then four greedy decode steps: the logits the reference's ModelBackend produced
    (tolerance: 2e-2 abs for the fp16 state, FP32_STATE_REL of the largest logit for the fp32 state, greedy ids
    identical)."""
    if name not in available_golden_models():
        pytest.skip(name + " has not been recorded")
    tag = "s32" if wkv32 else "s16"
    m, calls = golden_model_calls(tag, name)
    d, om, _, _ = oracle_model(GOLDEN_MODELS[name])
    B = int(m["B"])
    shift, wkv, elapsed = om.new_state(B, wkv32)
    worst = 0.0
    for toks, want in calls:
        got = om.forward(toks, shift, wkv, elapsed, lora_round_act=int(toks.size > 4))
        err = float(np.abs(got - want).max() / (np.abs(want).max() if wkv32 else 1.0))
        worst = max(worst, err)
        assert err < (fp32_state_bound_vs_reference(toks.size, d.ffn) if wkv32 else 2e-2), (toks.shape, err)
        assert (got.argmax(-1) == want.argmax(-1)).all()
    print(f"[golden] oracle vs reference backend ({name}, {tag}): worst logit err {worst:.3e}")
    assert (elapsed == m[tag + "_elapsed"]).all()
    assert np.abs(shift.astype(np.float32) - m[tag + "_shift"].astype(np.float32)).max() < 2e-2
    ref_wkv = m[tag + "_wkv"].astype(np.float32)
    mine = wkv.astype(np.float32)[:, :, :ref_wkv.shape[2]]      # wide fixtures keep the first heads only
    assert np.abs(mine - ref_wkv).max() <= 2e-2 * max(1.0, float(np.abs(ref_wkv).max()))


def test_greedy_pick_reproduces_the_reference_sampler_tests_known_answers():
    """The known answers of the reference's own sampler test for its greedy case (test/sampler_test.cpp:30-75):
    top_p = 0 picks the largest logit, and with presence 2 / frequency 5 / decay 0.5 the chosen token's penalty
    goes 0 -> 2 -> 6 while the others stay 0."""
    logits = np.array([[0.25, 3.0, 1.0, -1.0]], dtype=np.float32)
    assert orc.greedy_pick(logits).tolist() == [1]
    pen = np.zeros((1, 4), dtype=np.float32)
    assert orc.greedy_pick(logits, pen, 0.0, 0.0, 0.996).tolist() == [1]
    assert np.all(pen == 0)
    logits = np.array([[100.0, 0.0, 0.0, 0.0]], dtype=np.float32)
    pen = np.zeros((1, 4), dtype=np.float32)
    assert orc.greedy_pick(logits, pen, 2.0, 5.0, 0.5).tolist() == [0]
    np.testing.assert_allclose(pen[0], [2.0, 0.0, 0.0, 0.0], atol=1e-6)
    assert orc.greedy_pick(logits, pen, 2.0, 5.0, 0.5).tolist() == [0]
    np.testing.assert_allclose(pen[0], [6.0, 0.0, 0.0, 0.0], atol=1e-6)


def test_greedy_pick_edge_values():
    """NaN logits count as 0, infinities are clamped, +inf penalties mask a token, the lowest id wins a tie."""
    inf, nan = np.inf, np.nan
    logits = np.array([[nan, -1.0, -inf, -0.5], [1.0, inf, inf, 0.0], [2.0, 5.0, 5.0, 1.0], [3.0, 9.0, 1.0, 0.0]], dtype=np.float32)
    assert orc.greedy_pick(logits).tolist() == [0, 1, 1, 1]
    pen = np.zeros((4, 4), dtype=np.float32)
    pen[3, 1] = inf
    pen[2, 1] = 0.5
    assert orc.greedy_pick(logits, pen, 1.0, 2.0, 0.5).tolist() == [0, 1, 2, 0]
    assert pen[2].tolist() == [0.0, 0.25, 1.0, 0.0] and pen[3, 0] == 1.0 and pen[3, 1] == inf


def test_sampler_oracle_known_answers():
    """The counter-based generator against the published known answer of Philox-4x32-10 (counter 0, key 0 -> first word
    0x6627e8d5), and the filtering rule on a case small enough to check by hand."""
    assert orc.philox4x32_first(0, 0, 0, 0, 0, 0) == 0x6627E8D5
    assert orc.philox4x32_first(0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF) == 0x408F276D
    lg = np.log(np.array([[0.4, 0.3, 0.2, 0.1]], dtype=np.float64)).astype(np.float32)
    np.testing.assert_allclose(orc.sample_weights(lg)[0], [0.4, 0.3, 0.2, 0.1], rtol=1e-6)
    np.testing.assert_allclose(orc.sample_weights(lg, top_k=2)[0], [0.4, 0.3, 0.0, 0.0], rtol=1e-6, atol=1e-9)
    # top_p = 0.6: 0.4 stays, the token on the threshold (0.3) is scaled so that the kept mass is exactly 0.6
    np.testing.assert_allclose(orc.sample_weights(lg, top_p=0.6)[0], [0.4, 0.2, 0.0, 0.0], rtol=1e-5, atol=1e-9)
    # ties on the threshold share what is left: two tokens of 0.25 under top_k = 3 after 0.5 keep one token's worth together
    lt = np.log(np.array([[0.5, 0.25, 0.25]], dtype=np.float64)).astype(np.float32)
    np.testing.assert_allclose(orc.sample_weights(lt, top_k=2)[0], [0.5, 0.125, 0.125], rtol=1e-5)
    assert orc.sample_weights(lg, top_p=0.0)[0].tolist() == orc.sample_weights(lg, top_k=1)[0].tolist()      # both greedy
    toks = [int(orc.sample(lg, seed=1, offset=i)[0]) for i in range(2000)]
    freq = np.bincount(toks, minlength=4) / 2000.0
    assert np.abs(freq - [0.4, 0.3, 0.2, 0.1]).max() < 0.04
