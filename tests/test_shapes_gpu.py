"""Whole-model parity at the layer shapes of the benchmark configurations (two layers each, so that both the
first layer and a layer with a value residual run): 7.2B fp16 (C=4096, FFN 16384, ranks 128/128/96/480, once with
the full 65536-entry vocabulary), 1.5B W8A16 (C=2048) at B = 1, 8, 32, 64 and 2.9B W4A16 (C=2560) at B=256 rows,
against the CPU oracle.  These are the shapes bench.py times; the small-model tests elsewhere do not reach their
code paths (register-resident C=4096 rows in the GEMV prologue, rank 480 in the fused time-mix kernel, uneven row
splits over 148 SMs, the 65536 x 4096 head).
Tolerances: logits within 2e-2 abs for the fp16 state; for the fp32 state the error relative to the largest logit is
printed and bounded by FP32_STATE_REL (oracle/parity.py)."""
import numpy as np
import pytest

from oracle import oracle as orc
from oracle.parity import build_pair, run_both

pytestmark = pytest.mark.gpu

from oracle.parity import FP32_STATE_REL  # noqa: E402  (why whole logits cannot meet 1e-4 is explained there)

D72 = dict(layers=2, channels=4096, ffn=16384, vocab=4096, rank_w=128, rank_a=128, rank_v=96, rank_g=480)
D15 = dict(layers=2, channels=2048, ffn=8192, vocab=4096, rank_w=96, rank_a=96, rank_v=64, rank_g=256)
D29 = dict(layers=2, channels=2560, ffn=10240, vocab=4096, rank_w=96, rank_a=96, rank_v=64, rank_g=320)


def check(tag, dims, fmt, wkv32, B, chunks, n_decode, pair=None):
    d, om, gm = pair or build_pair(fmt, wkv32, dims=dims)
    worst, ids_ok, (shift, wkv, elapsed), st = run_both(d, om, gm, wkv32, B, chunks, n_decode)
    print(f"[parity] {tag} wkv32={wkv32} B={B} chunks={chunks} decode={n_decode}: worst logit err {worst:.3e}")
    assert worst < (FP32_STATE_REL if wkv32 else 2e-2)
    assert ids_ok
    assert (st.elapsed.cpu().numpy() == elapsed).all()
    g_wkv = st.wkv_state.cpu().numpy().astype(np.float32)
    assert np.abs(g_wkv - wkv.astype(np.float32)).max() <= 2e-2 * max(1.0, np.abs(wkv.astype(np.float32)).max())
    gm.close()


@pytest.mark.parametrize("wkv32", [False, True])
@pytest.mark.parametrize("B,chunks,n_decode", [(1, (4,), 3), (1, (48,), 1), (4, (1,), 2), (16, (1,), 1), (1, (128,), 1)])
def test_7p2B_layer_shape(wkv32, B, chunks, n_decode):
    """B=1: the five-launch decode path the headline number times (after a 4-row prompt on the same path);
    a 48-token chunk and 16 one-token rows: the tensor-core path; B=4: four GEMV rows; a 128-token chunk: the prefill
    configuration's chunk (with the fp32 state: the matrix-form WKV)."""
    check("7.2B shape", D72, orc.FMT_F16, wkv32, B, chunks, n_decode)


def test_7p2B_layer_shape_with_the_full_vocabulary():
    """The 65536 x 4096 head and embedding table of the timed configuration."""
    check("7.2B shape, vocab 65536", dict(D72, vocab=65536), orc.FMT_F16, False, 1, (3,), 2)


@pytest.mark.parametrize("B", [1, 8, 32, 64])
def test_1p5B_w8a16_decode_sweep(B):
    check("1.5B shape W8A16", D15, orc.FMT_W8A16, False, B, (2,), 2)


def test_1p5B_w8a16_fp32_state():
    check("1.5B shape W8A16", D15, orc.FMT_W8A16, True, 8, (2,), 2)


@pytest.mark.parametrize("B,wkv32", [(256, False), (1, False), (8, True)])
def test_2p9B_w4a16(B, wkv32):
    check("2.9B shape W4A16", D29, orc.FMT_W4A16, wkv32, B, (1,), 1 if B == 256 else 2)


def test_2p9B_w4a16_many_rows_repeated_calls_never_expire_a_wait():
    """The grouped launch that mixes packed (r, k, v) and fp16 (LoRA) products at 256 rows, 40 times over with fresh
    state and logits buffers and other allocations moved in between (tile arrival order varies with where things
    live): the device's failure word stays clear and all runs give the same logits.  (A dequantisation thread that
    waited on only every other fill of a stage could take a tile for landed that had not.)"""
    import torch
    from rwkv_lightning_cuda_b200 import backend as bk, lib as L
    d, _, gm = build_pair(orc.FMT_W4A16, False, dims=D29, oracle_model=False)
    rng = np.random.default_rng(0)
    toks = torch.from_numpy(rng.integers(0, d.vocab, (3, 256, 1)))
    keep, first = [], None
    L.timeout_flags(clear=True)
    stream = torch.cuda.Stream()          # a stream of its own: the second and third step replay a CUDA graph
    for call in range(40):
        keep.append(torch.empty(int(rng.integers(1, 64)) * 1024 * 513, dtype=torch.uint8, device="cuda"))
        st, lg = gm.create_state(256), bk.DeviceLogits()
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            for i in range(3):
                gm.forward_decode(toks[i], st, lg, sync=False)
        torch.cuda.synchronize()
        assert L.timeout_flags(clear=True) == 0, (call, L.timeout_detail())
        out = lg.values.cpu().numpy()
        if first is None:
            first = out
        assert np.array_equal(out, first), call
        del st, lg
    gm.close()


@pytest.mark.parametrize("fmt,B", [(orc.FMT_W4A16, 1), (orc.FMT_W4A16, 4), (orc.FMT_W8A16, 2), (orc.FMT_F16, 2), (orc.FMT_F16, 1)])
def test_7p2B_shape_small_batches_repeated_calls_are_identical(fmt, B):
    """The five-launch decode path (weight boxes through per-warp rings, partial sums handed over between warps through
    mbarriers) 30 times over with fresh buffers at shifting addresses: identical logits every time, no expired wait."""
    import torch
    from rwkv_lightning_cuda_b200 import backend as bk, lib as L
    d, _, gm = build_pair(fmt, False, dims=D72, oracle_model=False)
    rng = np.random.default_rng(1)
    toks = torch.from_numpy(rng.integers(0, d.vocab, (4, B, 1)))
    keep, first = [], None
    L.timeout_flags(clear=True)
    stream = torch.cuda.Stream()
    for call in range(30):
        keep.append(torch.empty(int(rng.integers(1, 64)) * 1024 * 513, dtype=torch.uint8, device="cuda"))
        st, lg = gm.create_state(B), bk.DeviceLogits()
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            for i in range(4):
                gm.forward_decode(toks[i], st, lg, sync=False)
        torch.cuda.synchronize()
        assert L.timeout_flags(clear=True) == 0, call
        out = lg.values.cpu().numpy()
        if first is None:
            first = out
        assert np.array_equal(out, first), call
        del st, lg
    gm.close()
