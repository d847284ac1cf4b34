"""Whole-model parity: the C-ABI forward (prefill chunks + decode steps) against the CPU oracle
on a small seeded random-init model, for fp16 / fp32 WKV state and the three weight formats.
Tolerances: logits within 2e-2 abs (fp16 state, the benchmark definition's), within FP32_STATE_REL of the largest
logit for the fp32 state (the benchmark's 1e-4 holds for the state recurrence, checked at op level; whole logits carry
the fp16 rounding of every activation, see tests/test_golden_cpu.py), greedy token ids identical."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from oracle.parity import FP32_STATE_REL, TINY, build_pair, run_both  # noqa: F401

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("wkv32", [False, True])
@pytest.mark.parametrize("B,chunks,n_decode", [(1, (5, 3), 6), (2, (4,), 4), (1, (20,), 2), (6, (2,), 3),   # 5..16 one-token rows
                                               (2, (70, 64), 2)])   # chunks of 64 tokens and more: the matrix-form WKV for the fp32 state
def test_forward_matches_oracle_fp16_weights(wkv32, B, chunks, n_decode):
    d, om, gm = build_pair(orc.FMT_F16, wkv32)
    worst, ids_ok, (shift, wkv, elapsed), st = run_both(d, om, gm, wkv32, B, chunks, n_decode)
    print(f"[parity] model fp16 weights wkv32={wkv32} B={B} chunks={chunks}: worst logit err {worst:.3e}")
    assert worst < (FP32_STATE_REL if wkv32 else 2e-2)   # fp16 activations bound the fp32-state case: see FP32_STATE_REL
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


@pytest.mark.parametrize("name", ["ref_model_tiny.npz", "ref_model_c4096.npz"])
@pytest.mark.parametrize("wkv32", [False, True])
def test_library_matches_the_reference_backend_golden(wkv32, name):
    """The library against what the reference's own ModelBackend produced on a B200 for the same checkpoint and tokens
    (tests/golden/ref_model_*.npz): two prefill chunks, four greedy decode steps, final state; at the 0.1B layer shape
    and at the 7.2B layer shape (4096 channels, for which the reference has kernels of their own)."""
    from rwkv_lightning_cuda_b200 import backend as bk
    from oracle.parity import fp32_state_bound_vs_reference
    from tests.test_golden_cpu import GOLDEN_MODELS, available_golden_models, golden_model_calls
    if name not in available_golden_models():
        pytest.skip(name + " has not been recorded")
    tag = "s32" if wkv32 else "s16"
    m, calls = golden_model_calls(tag, name)
    d, om, gm = build_pair(orc.FMT_F16, wkv32, dims=GOLDEN_MODELS[name], oracle_model=False)
    B = int(m["B"])
    st = gm.create_state(B); lg = bk.DeviceLogits()
    worst = 0.0
    for toks, want in calls:
        if toks.shape[1] == 1:
            gm.forward_decode(toks[:, 0].tolist(), st, lg)
        else:
            gm.forward_prefill(toks.tolist(), st, lg)
        got = lg.values.cpu().numpy()
        err = float(np.abs(got - want).max() / (np.abs(want).max() if wkv32 else 1.0))
        worst = max(worst, err)
        assert err < (fp32_state_bound_vs_reference(toks.size, d.ffn) if wkv32 else 2e-2), (toks.shape, err)
        assert (got.argmax(-1) == want.argmax(-1)).all()
    print(f"[parity] library vs reference backend ({name}, {tag}): worst logit err {worst:.3e}")
    assert (st.elapsed.cpu().numpy() == m[tag + "_elapsed"]).all()
    assert np.abs(st.shift.cpu().numpy().astype(np.float32) - m[tag + "_shift"].astype(np.float32)).max() < 2e-2
    ref_wkv = m[tag + "_wkv"].astype(np.float32)
    mine = st.wkv_state.cpu().numpy().astype(np.float32)[:, :, :ref_wkv.shape[2]]
    assert np.abs(mine - ref_wkv).max() <= 2e-2 * max(1.0, float(np.abs(ref_wkv).max()))


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


def test_decode_sample_equals_the_step_by_step_loop():
    """The on-device sampling loop against the same library driven step by step (forward_decode, then the sampler entry
    point with offset + step): identical ids, penalties and state; and the ids are a function of the seed."""
    from rwkv_lightning_cuda_b200 import backend as bk, ops
    d, om, gm = build_pair(orc.FMT_F16, False)
    B, steps = 3, 6
    first, prompt = [7, 11, 200], [[5, 6, 7], [8, 9, 10], [3, 2, 1]]
    kw = dict(temperature=0.9, top_k=50, top_p=0.9)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        st_a = gm.create_state(B); lg_a = bk.DeviceLogits()
        gm.forward_prefill(prompt, st_a, lg_a)
        pen_a = torch.zeros((B, d.vocab), dtype=torch.float32, device="cuda")
        host_ids = torch.empty((steps, B), dtype=torch.int32).pin_memory()
        ids_a = gm.decode_sample(first, steps, st_a, lg_a, seed=42, offset=10, penalties=pen_a, presence_penalty=0.4,
                                 repetition_penalty=0.3, penalty_decay=0.9, out_host=host_ids, **kw)
        st_b = gm.create_state(B); lg_b = bk.DeviceLogits()
        gm.forward_prefill(prompt, st_b, lg_b)
        pen_b = torch.zeros((B, d.vocab), dtype=torch.float32, device="cuda")
        cur, ids_b = list(first), []
        for i in range(steps):
            gm.forward_decode(cur, st_b, lg_b)
            cur = ops.sample(lg_b.values, pen_b, 0.4, 0.3, 0.9, seed=42, offset=10 + i, **kw).cpu().tolist()
            ids_b.append(cur)
        st_c = gm.create_state(B); lg_c = bk.DeviceLogits()
        gm.forward_prefill(prompt, st_c, lg_c)
        ids_c = gm.decode_sample(first, steps, st_c, lg_c, seed=43, offset=10, **kw)
    torch.cuda.synchronize()
    assert host_ids.tolist() == ids_b and ids_a.cpu().tolist() == ids_b
    assert torch.equal(pen_a, pen_b) and torch.equal(st_a.wkv_state, st_b.wkv_state) and torch.equal(st_a.elapsed, st_b.elapsed)
    assert ids_c.cpu().tolist() != ids_b          # another seed, another sequence


@pytest.mark.parametrize("wkv32", [False, True])
def test_session_records_round_trip_and_match_the_reference_blob_layout(wkv32):
    """A sequence exported from one batch and imported into another place of another batch continues with identical
    logits; the blobs are the reference's session record (the sequence's slices of the three state buffers, contiguous);
    the WKV state converts between its two precisions as torch does."""
    from rwkv_lightning_cuda_b200 import backend as bk, lib as L
    import ctypes as C
    d, om, gm = build_pair(orc.FMT_F16, wkv32)
    lib = L.load_library()
    src = gm.create_state(3); lg = bk.DeviceLogits()
    gm.forward_prefill([[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 11, 12]], src, lg)
    blobs = gm.export_sequence(src, 1)
    assert torch.equal(blobs[0], src.shift[:, :, 1].cpu()) and torch.equal(blobs[1], src.wkv_state[:, 1].cpu())
    assert blobs[2].tolist() == [4]
    sizes = [C.c_size_t() for _ in range(3)]
    L.check(lib.rwkv7_b200_state_blob_sizes(gm._h, *[C.byref(s) for s in sizes]))
    assert [s.value for s in sizes] == [b.numel() * b.element_size() for b in blobs]
    dst = gm.create_state(2)
    gm.forward_prefill([[20, 21], [22, 23]], dst, bk.DeviceLogits())
    gm.import_sequence(blobs, dst, 0)
    la, lb = bk.DeviceLogits(), bk.DeviceLogits()
    gm.forward_decode([30, 31, 32], src, la)
    gm.forward_decode([31, 40], dst, lb)
    assert torch.equal(la.values[1], lb.values[0])
    with pytest.raises(L.Rwkv7B200Error, match="exceeds batch size"):
        gm.export_sequence(src, 3)
    # precision conversion of a WKV state
    w = src.wkv_state
    other = torch.empty_like(w, dtype=torch.float16 if wkv32 else torch.float32)
    s = torch.cuda.current_stream().cuda_stream
    L.check(lib.rwkv7_b200_state_convert_wkv(C.c_void_p(s), C.c_void_p(w.data_ptr()), C.c_void_p(other.data_ptr()), w.numel(), int(wkv32)))
    torch.cuda.synchronize()
    assert torch.equal(other, w.to(other.dtype))
