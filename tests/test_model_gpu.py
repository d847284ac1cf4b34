"""Whole-model parity: the C-ABI forward (prefill chunks + decode steps) against the CPU oracle
on a small seeded random-init model, for fp16 / fp32 WKV state and the three weight formats.
Tolerances are the benchmark definition's: logits within 2e-2 abs (fp16 state) and 1e-4 relative
(fp32 state, relative to the largest logit), greedy token ids identical."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import h16

pytestmark = pytest.mark.gpu

TINY = dict(layers=3, channels=128, ffn=512, vocab=320, rank_w=32, rank_a=32, rank_v=16, rank_g=64)


def build_pair(fmt, wkv32, seed=0, dims=TINY, **backend_kw):
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic
    d = bk.ModelDims(**dims)
    ck = synthetic.make_checkpoint(d, seed=seed, device="cpu", dtype=torch.float16)
    ck16 = {k: v for k, v in ck.items()}
    table = orc.emb_ln0(ck["emb.weight"].float().numpy(), ck["blocks.0.ln0.weight"].float().numpy(),
                        ck["blocks.0.ln0.bias"].float().numpy())
    om = orc.Model(d.layers, d.channels, d.ffn, d.vocab, d.rank_w, d.rank_a, d.rank_v, d.rank_g, fmt)
    om.set("emb_ln0", table)
    dev_tensors = {"emb_ln0": torch.from_numpy(table)}
    for name, t in ck16.items():
        if name in ("emb.weight", "blocks.0.ln0.weight", "blocks.0.ln0.bias"):
            continue
        om.set(name, t.numpy())
        dev_tensors[name] = t
    gm = bk.ModelBackend(d, dev_tensors, use_wkv32=wkv32, weight_format=fmt, **backend_kw)
    return d, om, gm


def run_both(d, om, gm, wkv32, B, chunks, n_decode, seed=1):
    from rwkv_lightning_cuda_b200 import backend as bk
    rng = np.random.default_rng(seed)
    shift, wkv, elapsed = om.new_state(B, wkv32)
    st = gm.create_state(B)
    lg = bk.DeviceLogits()
    worst = 0.0
    for T in chunks:
        toks = rng.integers(0, d.vocab, (B, T))
        want = om.forward(toks, shift, wkv, elapsed, lora_round_act=int(B * T > 4))
        gm.forward_prefill(toks.tolist(), st, lg)
        got = lg.values.cpu().numpy()
        worst = max(worst, np.abs(got - want).max() / (np.abs(want).max() if wkv32 else 1.0))
    ids_o = want.argmax(-1); ids_g = got.argmax(-1)
    agree = []
    for _ in range(n_decode):
        agree.append((ids_o == ids_g).all())
        want = om.forward(ids_o[:, None], shift, wkv, elapsed, lora_round_act=int(B > 4))
        gm.forward_decode(ids_o.tolist(), st, lg)
        got = lg.values.cpu().numpy()
        worst = max(worst, np.abs(got - want).max() / (np.abs(want).max() if wkv32 else 1.0))
        ids_o = want.argmax(-1); ids_g = got.argmax(-1)
    agree.append((ids_o == ids_g).all())
    return worst, all(agree), (shift, wkv, elapsed), st


@pytest.mark.parametrize("wkv32", [False, True])
@pytest.mark.parametrize("B,chunks,n_decode", [(1, (5, 3), 6), (2, (4,), 4), (1, (20,), 2), (6, (2,), 3)])   # last: 5..16 one-token rows
def test_forward_matches_oracle_fp16_weights(wkv32, B, chunks, n_decode):
    d, om, gm = build_pair(orc.FMT_F16, wkv32)
    worst, ids_ok, (shift, wkv, elapsed), st = run_both(d, om, gm, wkv32, B, chunks, n_decode)
    print(f"[parity] model fp16 weights wkv32={wkv32} B={B} chunks={chunks}: worst logit err {worst:.3e}")
    assert worst < (1e-4 * 50 if wkv32 else 2e-2)   # see module docstring; fp16 activations bound the fp32-state case
    assert ids_ok
    assert (st.elapsed.cpu().numpy() == elapsed).all()
    g_shift = st.shift.cpu().numpy().astype(np.float32)
    assert np.abs(g_shift - shift.astype(np.float32)).max() < 2e-2
    g_wkv = st.wkv_state.cpu().numpy().astype(np.float32)
    assert np.abs(g_wkv - wkv.astype(np.float32)).max() <= 2e-2 * max(1.0, np.abs(wkv.astype(np.float32)).max())


@pytest.mark.parametrize("B,chunks", [(2, (3,)), (3, (6, 2))])     # second case: more than four rows -> tensor-core path
@pytest.mark.parametrize("fmt", [orc.FMT_W8A16, orc.FMT_W4A16])
def test_forward_matches_oracle_quantised(fmt, B, chunks):
    d, om, gm = build_pair(fmt, False)
    worst, ids_ok, _, _ = run_both(d, om, gm, False, B, chunks, 4)
    print(f"[parity] model fmt={fmt}: worst logit err {worst:.3e}")
    assert worst < 2e-2
    assert ids_ok


def test_state_slices_and_capacity_and_errors():
    from rwkv_lightning_cuda_b200 import backend as bk, lib as L
    d, om, gm = build_pair(orc.FMT_F16, False)
    src = gm.create_state(3); dst = gm.create_state(2)
    lg = bk.DeviceLogits()
    gm.forward_prefill([[1, 2, 3], [4, 5, 6], [7, 8, 9]], src, lg)
    gm.copy_state_slice(src, 1, dst, 0, 2)
    assert torch.equal(dst.shift, src.shift[:, :, 1:3]) and torch.equal(dst.wkv_state, src.wkv_state[:, 1:3])
    assert dst.elapsed.tolist() == [3, 3]
    # a sequence continued alone from its slice gives the same logits as inside the batch
    one = gm.create_state(1); gm.copy_state_slice(src, 2, one, 0, 1)
    lg1 = bk.DeviceLogits()
    gm.forward_decode([11, 12, 13], src, lg); gm.forward_decode([13], one, lg1)
    assert torch.equal(lg.values[2], lg1.values[0])
    dst2 = bk.DeviceLogits(); dst2.rows, dst2.vocab_size = 1, d.vocab
    dst2.values = torch.zeros((1, d.vocab), device="cuda")
    gm.copy_logits_slice(lg, 2, dst2, 0, 1)
    assert torch.equal(dst2.values[0], lg.values[2])
    cap = gm.query_prefill_capacity(128)
    assert cap.max_batch_size > 0 and cap.bytes_per_batch > 0 and cap.free_vram_bytes <= cap.total_vram_bytes
    # error behaviour mirrors the reference: argument errors raise, nothing aborts, state untouched
    before = src.elapsed.clone()
    for bad, msg in (([[1, 2], [3]], "same length"), ([], "must not be empty"), ([[d.vocab, 1, 1]] * 3, "out of range")):
        with pytest.raises(L.Rwkv7B200Error, match=msg):
            gm.forward_prefill(bad, src, lg)
    with pytest.raises(L.Rwkv7B200Error, match="batch size mismatch"):
        gm.forward_decode([1], src, lg)
    with pytest.raises(L.Rwkv7B200Error, match="exceeds batch size"):
        gm.copy_state_slice(src, 2, dst, 0, 2)
    with pytest.raises(L.Rwkv7B200Error, match="positive"):
        gm.create_state(0)
    assert torch.equal(before, src.elapsed)


def test_decode_graph_replay_is_deterministic_and_matches_eager():
    from rwkv_lightning_cuda_b200 import backend as bk
    d, om, gm = build_pair(orc.FMT_F16, False)
    outs = []
    for use_stream in (False, True):
        st = gm.create_state(2); lg = bk.DeviceLogits()
        s = torch.cuda.Stream() if use_stream else torch.cuda.default_stream()
        seq = []
        with torch.cuda.stream(s):
            gm.forward_prefill([[5, 6, 7], [8, 9, 10]], st, lg)
            for step in range(5):          # default stream: eager launches; side stream: graph replay
                gm.forward_decode([step + 1, step + 2], st, lg)
                seq.append(lg.values.clone())
        torch.cuda.synchronize()
        outs.append(torch.stack(seq))
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("dims,B", [
    (dict(TINY, layers=2, ffn=16384), 4),      # four rows of ffn inputs do not fit the fused decode kernels' shared memory
    (dict(TINY, layers=2, ffn=16384), 2),      # two rows do
    (dict(TINY, layers=2, rank_w=64, rank_a=64, rank_v=32, rank_g=128), 1),   # 0.1B ranks: exactly 48 KiB of dynamic shared memory
])
def test_decode_shapes_at_the_edges_of_the_fused_path(dims, B):
    d, om, gm = build_pair(orc.FMT_F16, False, dims=dims)
    worst, ids_ok, _, _ = run_both(d, om, gm, False, B, (2,), 3)
    print(f"[parity] edge shapes {dims} B={B}: worst logit err {worst:.3e}")
    assert worst < 2e-2
    assert ids_ok


def test_full_size_0p1B_prefill_and_greedy_decode_match_the_oracle():
    """The smallest benchmark configuration at its real size (12 layers, d=768, FFN 3072, vocabulary 65536, LoRA ranks
    64/64/32/128): a 32-token prefill chunk on the tensor cores, then greedy decode steps on the GEMV path."""
    dims = dict(layers=12, channels=768, ffn=3072, vocab=65536, rank_w=64, rank_a=64, rank_v=32, rank_g=128)
    d, om, gm = build_pair(orc.FMT_F16, False, dims=dims)
    worst, ids_ok, (shift, wkv, elapsed), st = run_both(d, om, gm, False, 1, (32,), 4)
    print(f"[parity] 0.1B full size: worst logit err {worst:.3e}")
    assert worst < 2e-2
    assert ids_ok
    assert (st.elapsed.cpu().numpy() == elapsed).all()


@pytest.mark.parametrize("wkv32", [False, True])
def test_library_matches_the_reference_backend_golden(wkv32):
    """The library against what the reference's own ModelBackend produced on a B200 for the same checkpoint and tokens
    (tests/golden/ref_model_tiny.npz): prefill chunks of 5 and 3 tokens, four greedy decode steps, final state."""
    from rwkv_lightning_cuda_b200 import backend as bk
    from tests.test_golden_cpu import GOLDEN_DIMS, golden_model_calls
    tag = "s32" if wkv32 else "s16"
    m, calls = golden_model_calls(tag)
    d, om, gm = build_pair(orc.FMT_F16, wkv32, dims=GOLDEN_DIMS)
    B = int(m["B"])
    st = gm.create_state(B); lg = bk.DeviceLogits()
    worst = 0.0
    for toks, want in calls:
        if toks.shape[1] == 1:
            gm.forward_decode(toks[:, 0].tolist(), st, lg)
        else:
            gm.forward_prefill(toks.tolist(), st, lg)
        got = lg.values.cpu().numpy()
        worst = max(worst, float(np.abs(got - want).max() / (np.abs(want).max() if wkv32 else 1.0)))
        assert (got.argmax(-1) == want.argmax(-1)).all()
    print(f"[parity] library vs reference backend ({tag}): worst logit err {worst:.3e}")
    assert worst < (1e-4 * 50 if wkv32 else 2e-2)
    assert (st.elapsed.cpu().numpy() == m[tag + "_elapsed"]).all()
    assert np.abs(st.shift.cpu().numpy().astype(np.float32) - m[tag + "_shift"].astype(np.float32)).max() < 2e-2
    ref_wkv = m[tag + "_wkv"].astype(np.float32)
    assert np.abs(st.wkv_state.cpu().numpy().astype(np.float32) - ref_wkv).max() <= 2e-2 * max(1.0, float(np.abs(ref_wkv).max()))


@pytest.mark.parametrize("use_stream", [False, True])     # default stream: eager launches; side stream: graph replay
def test_decode_greedy_equals_the_step_by_step_loop_and_the_oracle(use_stream):
    """The on-device greedy loop against (1) the same library driven step by step from the host with the oracle's
    greedy pick on the copied-back logits: identical ids, penalties, logits and state; (2) the CPU oracle's own
    model + pick chain: identical ids."""
    from rwkv_lightning_cuda_b200 import backend as bk
    d, om, gm = build_pair(orc.FMT_F16, False)
    B, steps = 3, 6
    first = [7, 11, 200]
    prompt = [[5, 6, 7], [8, 9, 10], [3, 2, 1]]
    pres, rep, decay = 0.4, 0.3, 0.9
    s = torch.cuda.Stream() if use_stream else torch.cuda.default_stream()
    with torch.cuda.stream(s):
        # (a) on the device
        st_a = gm.create_state(B); lg_a = bk.DeviceLogits()
        gm.forward_prefill(prompt, st_a, lg_a)
        pen_a = torch.zeros((B, d.vocab), dtype=torch.float32, device="cuda")
        host = torch.empty((steps, B), dtype=torch.int32).pin_memory()
        ids_a = gm.decode_greedy(first, steps, st_a, lg_a, pen_a, pres, rep, decay, out_host=host)
        assert torch.equal(ids_a.cpu(), host)
        # (b) step by step from the host
        st_b = gm.create_state(B); lg_b = bk.DeviceLogits()
        gm.forward_prefill(prompt, st_b, lg_b)
        pen_b = np.zeros((B, d.vocab), dtype=np.float32)
        cur, ids_b = list(first), []
        for _ in range(steps):
            gm.forward_decode(cur, st_b, lg_b)
            cur = orc.greedy_pick(lg_b.values.cpu().numpy(), pen_b, pres, rep, decay).tolist()
            ids_b.append(cur)
    torch.cuda.synchronize()
    assert host.tolist() == ids_b
    assert np.array_equal(pen_a.cpu().numpy(), pen_b)
    assert torch.equal(lg_a.values, lg_b.values)
    assert torch.equal(st_a.wkv_state, st_b.wkv_state) and torch.equal(st_a.shift, st_b.shift)
    assert torch.equal(st_a.elapsed, st_b.elapsed)
    # (c) the oracle's own chain
    shift, wkv, elapsed = om.new_state(B, False)
    om.forward(np.array(prompt), shift, wkv, elapsed, lora_round_act=1)
    pen_c = np.zeros((B, d.vocab), dtype=np.float32)
    cur, ids_c = np.array(first), []
    for _ in range(steps):
        cur = orc.greedy_pick(om.forward(cur[:, None], shift, wkv, elapsed, lora_round_act=0), pen_c, pres, rep, decay)
        ids_c.append(cur.tolist())
    assert ids_c == ids_b


def test_decode_greedy_argument_errors():
    from rwkv_lightning_cuda_b200 import backend as bk, lib as L
    d, om, gm = build_pair(orc.FMT_F16, False)
    st = gm.create_state(2); lg = bk.DeviceLogits()
    with pytest.raises(L.Rwkv7B200Error, match="steps must be positive"):
        gm.decode_greedy([1, 2], 0, st, lg)
    with pytest.raises(L.Rwkv7B200Error, match="token id out of range"):
        gm.decode_greedy([1, d.vocab], 2, st, lg)
    with pytest.raises(L.Rwkv7B200Error, match="state batch size mismatch"):
        gm.decode_greedy([1, 2, 3], 2, st, lg)
    assert int(st.elapsed.sum()) == 0          # nothing ran


def test_from_pth_loads_a_bf16_checkpoint_like_the_reference_constructor(tmp_path):
    """A torch .pth file with the reference's tensor names in bf16 (the format its loader accepts): dimensions are
    inferred from the shapes, layer 0's unused value-residual tensors are skipped, and the logits equal those of a
    model given the same tensors directly."""
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic
    d = bk.ModelDims(**TINY)
    ck = {k: v.to(torch.bfloat16) for k, v in synthetic.make_checkpoint(d, seed=3, device="cpu", dtype=torch.float16).items()}
    ck["blocks.0.att.v0"] = torch.zeros(d.channels, dtype=torch.bfloat16)          # present in real files, never used
    ck["blocks.0.att.v1"] = torch.zeros((d.channels, d.rank_v), dtype=torch.bfloat16)
    ck["blocks.0.att.v2"] = torch.zeros((d.rank_v, d.channels), dtype=torch.bfloat16)
    path = str(tmp_path / "tiny.pth")
    torch.save(ck, path)
    a = bk.ModelBackend.from_pth(path)
    assert a.dims == d and a.model_path() == path
    b = bk.ModelBackend(d, {k: v for k, v in ck.items() if k not in ("blocks.0.att.v0", "blocks.0.att.v1", "blocks.0.att.v2")})
    toks = [[1, 2, 3, 4, 5], [9, 8, 7, 6, 5]]
    outs = []
    for m in (a, b):
        st = m.create_state(2); lg = bk.DeviceLogits()
        m.forward_prefill(toks, st, lg)
        m.forward_decode([11, 12], st, lg)
        outs.append(lg.values.clone())
    assert torch.isfinite(outs[0]).all() and torch.equal(outs[0], outs[1])
