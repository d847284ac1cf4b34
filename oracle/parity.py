"""Checker helpers shared by the parity tests and by the parity leg of ``bench.py --gpus N``: build the library's
model and the CPU oracle's model from one seeded checkpoint, drive both through the same calls, report the worst
logit error.  Test infrastructure like the rest of this directory: the product package never imports it."""
import numpy as np
import torch

from . import oracle as orc

TINY = dict(layers=3, channels=128, ffn=512, vocab=320, rank_w=32, rank_a=32, rank_v=16, rank_g=64)

# fp32 WKV state: worst |logit error| / max |logit| allowed between two implementations of the model.  The benchmark's
# 1e-4 holds for the state recurrence itself (checked at op level) but not for whole logits: every activation between
# two kernels is rounded to fp16 (relative half-ulp 4.9e-4) by the reference, the oracle and the library alike, each
# with its own summation order.
FP32_STATE_REL = 5e-3


def build_pair(fmt, wkv32, seed=0, dims=TINY, oracle_model=True, **backend_kw):
    """(dims, oracle model or None, library model) from the checkpoint of `seed`."""
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic
    d = bk.ModelDims(**dims)
    ck = synthetic.make_checkpoint(d, seed=seed, device="cpu", dtype=torch.float16)
    ck16 = {k: v for k, v in ck.items()}
    table = orc.emb_ln0(ck["emb.weight"].float().numpy(), ck["blocks.0.ln0.weight"].float().numpy(),
                        ck["blocks.0.ln0.bias"].float().numpy())
    om = orc.Model(d.layers, d.channels, d.ffn, d.vocab, d.rank_w, d.rank_a, d.rank_v, d.rank_g, fmt) if oracle_model else None
    if om:
        om.set("emb_ln0", table)
    dev_tensors = {"emb_ln0": torch.from_numpy(table)}
    for name, t in ck16.items():
        if name in ("emb.weight", "blocks.0.ln0.weight", "blocks.0.ln0.bias"):
            continue
        if om:
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
