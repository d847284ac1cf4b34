"""The 0.1B benchmark configuration as it is written -- 12 layers, d=768, vocabulary 65536, a 512-token prompt
prefilled in four chunks of 128, then 256 greedy decode steps at B=1, fp16 state -- against the reference's own
ModelBackend running beside the library on the same GPU (oracle/_ref, built from the reference's unmodified sources;
the test is skipped where that build is absent).

Both backends load the same bf16 checkpoint and are fed the SAME token at every step (the reference's greedy choice),
so one early near-tie cannot make the two runs drift apart and hide everything after it.  The reference is run twice:
its FFN down-projection for up to four rows adds fp16 partial sums with atomics in arbitrary order
(cuda/rwkv7_fast_ops_fp16.cu:618-679), so its own run-to-run difference is the noise floor a comparison has to be
read against."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle.oracle import ref_lib

pytestmark = pytest.mark.gpu

DIMS = dict(layers=12, channels=768, ffn=3072, vocab=65536, rank_w=64, rank_a=64, rank_v=32, rank_g=128)
PROMPT, CHUNK, STEPS = 512, 128, 256


def run_reference(ref, path, prompt, steps, forced=None):
    be = ref.ref_backend_create(path.encode(), 0)
    assert be, ref.ref_last_error().decode()
    st = ref.ref_state_create(be, 1)
    V = DIMS["vocab"]
    logits = np.empty((1, V), dtype=np.float32)
    out = []
    for c in range(0, len(prompt), CHUNK):
        t = np.ascontiguousarray(prompt[None, c:c + CHUNK].astype(np.int64))
        assert ref.ref_forward(be, st, t.ctypes.data_as(C.c_void_p), 1, t.shape[1], logits.ctypes.data_as(C.c_void_p)) == 0
    out.append(logits[0].copy())
    for i in range(steps):
        nxt = int(forced[i]) if forced is not None else int(out[-1].argmax())
        t = np.array([[nxt]], dtype=np.int64)
        assert ref.ref_forward(be, st, t.ctypes.data_as(C.c_void_p), 1, 1, logits.ctypes.data_as(C.c_void_p)) == 0
        out.append(logits[0].copy())
    ref.ref_state_destroy(st)
    ref.ref_backend_destroy(be)
    return np.stack(out)


def test_0p1B_prefill_512_then_256_greedy_steps_against_the_live_reference(tmp_path):
    ref = ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref/libref_rwkv7.so is not built here")
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic
    d = bk.ModelDims(**DIMS)
    ck = synthetic.make_checkpoint(d, seed=0, device="cpu", dtype=torch.bfloat16)
    path = str(tmp_path / "m.pth")
    torch.save({k: v.clone() for k, v in ck.items()}, path)
    prompt = np.random.default_rng(2).integers(0, d.vocab, PROMPT)
    ref_a = run_reference(ref, path, prompt, STEPS)
    ids = ref_a.argmax(-1)                                       # ids[i] feeds step i
    ref_b = run_reference(ref, path, prompt, STEPS, forced=ids)  # same inputs again: the reference's own noise
    os.unlink(path)
    noise = float(np.abs(ref_a - ref_b).max())
    flips = int((ref_a.argmax(-1) != ref_b.argmax(-1)).sum())

    gm = bk.ModelBackend(d, ck, use_wkv32=False)
    st = gm.create_state(1); lg = bk.DeviceLogits()
    mine = []
    for c in range(0, PROMPT, CHUNK):
        gm.forward_prefill([prompt[c:c + CHUNK].tolist()], st, lg)
    mine.append(lg.values[0].cpu().numpy())
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):                                   # a side stream: the captured-graph decode path
        for i in range(STEPS):
            gm.forward_decode([int(ids[i])], st, lg)
            mine.append(lg.values[0].cpu().numpy())
    mine = np.stack(mine)
    err = np.abs(mine - ref_a).max(-1)
    top2 = np.sort(ref_a, -1)[:, -2:]
    margin = top2[:, 1] - top2[:, 0]
    same = mine.argmax(-1) == ids
    print(f"[parity] 0.1B config, 512-token prefill + 256 greedy steps vs the live reference: worst |logit diff| {err.max():.3e} "
          f"(prefill {err[0]:.3e}), ids equal {int(same.sum())}/{len(same)}; reference run-to-run: |diff| {noise:.3e}, "
          f"{flips} id flips; smallest top-2 margin {margin.min():.3e}")
    assert err.max() < 2e-2
    # token-exact wherever the reference itself is decided by more than the two runs' combined error
    decided = margin > 2 * max(err.max(), noise)
    assert same[decided].all()
    # elsewhere (fp16 logits tie exactly now and then: the smallest margin is 0) no more disagreements than the
    # reference has with itself, give or take a few
    assert int((~same).sum()) <= 2 * flips + 3
