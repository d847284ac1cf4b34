"""Generates the golden fixtures of this directory from the REFERENCE's own CUDA code.

Needs a GPU and ``oracle/_ref/libref_rwkv7.so`` (the reference's unmodified sources compiled by ``make -C oracle ref``).
Inputs are small seeded tensors; outputs are what the reference's kernels, and its whole ``ModelBackend`` on a tiny
random-init checkpoint, produce for them.  The CPU tests check the oracle against these files, the GPU tests check
the library against them, so both are pinned to the reference without the reference being present.

    python tests/golden/make_golden.py [output directory]      (default: this directory)
"""
import ctypes as C
import os
import sys
import tempfile

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests.helpers import h16, ref_lib, wkv_inputs  # noqa: E402

# the smallest benchmark model's layer shape (the reference's kernels do not launch for much narrower layers), two layers
# deep and with a short vocabulary so that the fixture stays small
TINY = dict(layers=2, channels=768, ffn=3072, vocab=1024, rank_w=64, rank_a=64, rank_v=32, rank_g=128)
# the widest benchmark model's layer shape: the reference has kernels of their own for exactly 4096 channels
# (cuda/rwkv7_v3a_ops.cu:1353-1513,1637-1885), which no narrower fixture reaches
WIDE = dict(layers=2, channels=4096, ffn=16384, vocab=1024, rank_w=128, rank_a=128, rank_v=96, rank_g=480)


_KEEP = []   # device tensors stay alive until the script ends: a freed temporary's memory would be handed to the next one


def dev(a):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    _KEEP.append(t)
    return t


def p(t):
    return C.c_void_p(t.data_ptr())


def table(ts):
    arr = (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    return arr


def check(ref, rc):
    torch.cuda.synchronize()
    if rc != 0:
        raise RuntimeError(ref.ref_last_error().decode())


def ops(ref, out):
    rng = np.random.default_rng(2024)
    g = {}
    # ---- WKV, fp16 state with and without the decay bias, and fp32 state
    B, T, H = 2, 9, 2
    Cc = H * 64
    r, w, k, v, a, b = wkv_inputs(B, T, H, seed=5)
    s0 = h16(rng.standard_normal((B, H, 64, 64)) * 0.5)
    elapsed = (np.arange(B, dtype=np.int32) * 977 + 5).astype(np.int32)
    w0 = h16(rng.uniform(-1, 1, Cc))
    for name, use_w0 in (("wkv16", False), ("wkv16w0", True)):
        st = dev(s0.copy()); y = torch.empty((B, T, Cc), dtype=torch.float16, device="cuda")
        tens = [dev(t) for t in (r, w, k, v, a, b)]
        el = dev(elapsed)
        if use_w0:
            rc = ref.ref_wkv_fp16_seq_w0(B, T, Cc, H, p(st), p(tens[0]), p(tens[1]), p(dev(w0)), p(tens[2]), p(tens[3]), p(tens[4]),
                                         p(tens[5]), p(y), p(el))
        else:
            rc = ref.ref_wkv_fp16_seq(B, T, Cc, H, p(st), p(tens[0]), p(tens[1]), p(tens[2]), p(tens[3]), p(tens[4]), p(tens[5]),
                                      p(y), p(el))
        check(ref, rc)
        g[name + "_y"] = y.cpu().numpy(); g[name + "_state"] = st.cpu().numpy()
    g.update(wkv_B=B, wkv_T=T, wkv_H=H, wkv_r=r, wkv_w=w, wkv_k=k, wkv_v=v, wkv_a=a, wkv_b=b, wkv_s0=s0, wkv_elapsed=elapsed, wkv_w0=w0)
    s32 = (rng.standard_normal((B, H, 64, 64)) * 0.5).astype(np.float32)
    st = dev(s32.copy()); y = torch.empty((B, T, Cc), dtype=torch.float16, device="cuda")
    tens = [dev(t) for t in (r, w, k, v, a, b)]
    check(ref, ref.ref_wkv_fp32io16(B, T, Cc, H, p(st), *[p(t) for t in tens], p(y)))
    g.update(wkv32_s0=s32, wkv32_y=y.cpu().numpy(), wkv32_state=st.cpu().numpy())

    # ---- row kernels
    rows, Cn = 6, 768       # (the reference's row kernels are written for the model widths it ships: 768 and up)
    x = h16(rng.standard_normal((rows, Cn))); res = h16(rng.standard_normal((rows, Cn)) * 0.5)
    lw = h16(1 + 0.1 * rng.standard_normal(Cn)); lb = h16(0.1 * rng.standard_normal(Cn))
    y = torch.empty((rows, Cn), dtype=torch.float16, device="cuda")
    check(ref, ref.ref_layer_norm(rows, Cn, p(dev(x)), p(dev(lw)), p(dev(lb)), p(y), C.c_float(1e-5)))
    g.update(ln_x=x, ln_res=res, ln_w=lw, ln_b=lb, ln_y=y.cpu().numpy())
    xo = torch.empty_like(y)
    check(ref, ref.ref_add_layer_norm(rows, Cn, p(dev(x)), p(dev(res)), p(dev(lw)), p(dev(lb)), p(xo), p(y), C.c_float(1e-5)))
    g.update(addln_xo=xo.cpu().numpy(), addln_y=y.cpu().numpy())
    Bl, Tl = 2, 3
    yl = torch.empty((Bl, Cn), dtype=torch.float16, device="cuda")
    check(ref, ref.ref_add_last_layer_norm(Bl, Tl, Cn, p(dev(x)), p(dev(res)), p(dev(lw)), p(dev(lb)), p(yl), C.c_float(1e-5)))
    g.update(addlast_y=yl.cpu().numpy())
    # token shift fusions, decode rows (T = 1)
    shift0 = h16(rng.standard_normal((rows, Cn)))
    mixes = [h16(rng.uniform(0, 1, Cn)) for _ in range(6)]
    sh = dev(shift0.copy()); outs = [torch.empty_like(y) for _ in range(6)]
    check(ref, ref.ref_add_layer_norm_tmix_mix6(rows, Cn, p(dev(x)), p(dev(res)), p(sh), p(dev(lw)), p(dev(lb)),
                                                table([dev(m) for m in mixes]), p(xo), table(outs), C.c_float(1e-5)))
    g.update(mix_shift0=shift0, mix_coef=np.stack(mixes), lnmix6_xo=xo.cpu().numpy(), lnmix6_out=np.stack([o.cpu().numpy() for o in outs]),
             lnmix6_shift=sh.cpu().numpy())
    sh = dev(shift0.copy()); mixed = torch.empty_like(y)
    check(ref, ref.ref_add_layer_norm_cmix_mix(rows, Cn, p(dev(x)), p(dev(res)), p(sh), p(dev(lw)), p(dev(lb)), p(dev(mixes[0])), p(xo),
                                               p(mixed), C.c_float(1e-5)))
    g.update(lncmix_xo=xo.cpu().numpy(), lncmix_out=mixed.cpu().numpy(), lncmix_shift=sh.cpu().numpy())
    # plain token shift over a chunk
    sh = dev(shift0[:Bl].copy()); outs = [torch.empty_like(y) for _ in range(6)]
    check(ref, ref.ref_tmix_mix6(Bl, Tl, Cn, p(dev(x)), p(sh), table([dev(m) for m in mixes]), table(outs)))
    g.update(mix6_out=np.stack([o.cpu().numpy() for o in outs]), mix6_shift=sh.cpu().numpy())
    sh = dev(shift0[:Bl].copy())
    check(ref, ref.ref_cmix_mix(Bl, Tl, Cn, p(dev(x)), p(sh), p(dev(mixes[0])), p(mixed)))
    g.update(cmix_out=mixed.cpu().numpy(), cmix_shift=sh.cpu().numpy())

    # ---- per-head gates
    Hg = 3; Cg = Hg * 64; rg = 5
    kk = h16(rng.standard_normal((rg, Cg))); a12 = h16(rng.standard_normal((rg, Cg)))
    k_k = h16(rng.uniform(0.5, 1.5, Cg)); a0 = h16(rng.standard_normal(Cg)); k_a = h16(rng.uniform(0, 1, Cg))
    o3 = [torch.empty((rg, Cg), dtype=torch.float16, device="cuda") for _ in range(3)]
    check(ref, ref.ref_tmix_kk_a_gate(rg, 1, Cg, Hg, p(dev(kk)), p(dev(k_k)), p(dev(a0)), p(dev(a12)), p(dev(k_a)), p(o3[0]), p(o3[1]), p(o3[2])))
    g.update(gate_k=kk, gate_a12=a12, gate_k_k=k_k, gate_a0=a0, gate_k_a=k_a, gate_out=np.stack([o.cpu().numpy() for o in o3]))
    yy = h16(rng.standard_normal((rg, Cg)) * 3); rr = h16(rng.standard_normal((rg, Cg))); vv = h16(rng.standard_normal((rg, Cg)))
    gg = h16(rng.standard_normal((rg, Cg))); r_k = h16(rng.standard_normal(Cg) * 0.1)
    lxw = h16(1 + 0.1 * rng.standard_normal(Cg)); lxb = h16(0.1 * rng.standard_normal(Cg))
    o = torch.empty((rg, Cg), dtype=torch.float16, device="cuda")
    check(ref, ref.ref_tmix_lnx_rkvres_xg(rg, 1, Cg, Hg, p(dev(yy)), p(dev(rr)), p(dev(kk)), p(dev(vv)), p(dev(r_k)), p(dev(lxw)), p(dev(lxb)),
                                          p(dev(gg)), p(o)))
    g.update(lnx_y=yy, lnx_r=rr, lnx_v=vv, lnx_g=gg, lnx_r_k=r_k, lnx_w=lxw, lnx_b=lxb, lnx_out=o.cpu().numpy())
    vf = h16(rng.standard_normal((rg, Cg))); v0 = h16(rng.standard_normal(Cg)); v12 = h16(rng.standard_normal((rg, Cg)))
    check(ref, ref.ref_tmix_vres_gate(rg, 1, Cg, p(dev(vv)), p(dev(vf)), p(dev(v0)), p(dev(v12)), p(o)))
    g.update(vres_vf=vf, vres_v0=v0, vres_v12=v12, vres_out=o.cpu().numpy())

    # ---- linear (the reference's own GEMV for up to two rows) and relu^2
    M, K, N = 2, 768, 96
    lx = h16(rng.standard_normal((M, K))); lW = h16(rng.standard_normal((N, K)) * 0.02)
    ly = torch.empty((M, N), dtype=torch.float16, device="cuda")
    check(ref, ref.ref_linear_orig(M, K, N, p(dev(lx)), p(dev(lW)), p(ly), 1))
    g.update(lin_x=lx, lin_W=lW, lin_y=ly.cpu().numpy())
    np.savez_compressed(os.path.join(out, "ref_ops.npz"), **g)
    print("ref_ops.npz:", len(g), "arrays")


def model(ref, out, dims=TINY, name="ref_model_tiny.npz", lengths=(5, 3), wkv_heads=None):
    """Logits of every call and the final state of the reference's ModelBackend on the seeded checkpoint of `dims`.
    wkv_heads: keep only the first so many heads of the WKV state (keeps a wide fixture small)."""
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic
    d = bk.ModelDims(**dims)
    ck = synthetic.make_checkpoint(d, seed=0, device="cpu", dtype=torch.bfloat16)
    rng = np.random.default_rng(77)
    B = 1
    chunks = [rng.integers(0, d.vocab, (B, n)) for n in lengths]
    g = {"B": B}
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "tiny.pth")
        torch.save({k: v.clone() for k, v in ck.items()}, path)
        for wkv32 in (0, 1):
            be = ref.ref_backend_create(path.encode(), wkv32)
            if not be:
                raise RuntimeError("reference backend: " + ref.ref_last_error().decode())
            st = ref.ref_state_create(be, B)
            logits = np.empty((B, d.vocab), dtype=np.float32)
            calls = []
            toks = [c for c in chunks]
            for t in toks:
                t = np.ascontiguousarray(t.astype(np.int64))
                rc = ref.ref_forward(be, st, t.ctypes.data_as(C.c_void_p), B, t.shape[1], logits.ctypes.data_as(C.c_void_p))
                if rc:
                    raise RuntimeError(ref.ref_last_error().decode())
                calls.append((t, logits.copy()))
            ids = logits.argmax(-1)
            for _ in range(4):     # greedy decode steps
                t = np.ascontiguousarray(ids[:, None].astype(np.int64))
                rc = ref.ref_forward(be, st, t.ctypes.data_as(C.c_void_p), B, 1, logits.ctypes.data_as(C.c_void_p))
                if rc:
                    raise RuntimeError(ref.ref_last_error().decode())
                calls.append((t, logits.copy()))
                ids = logits.argmax(-1)
            shift = np.empty((d.layers, 2, B, d.channels), dtype=np.float16)
            wkv = np.empty((d.layers, B, d.heads, 64, 64), dtype=np.float32 if wkv32 else np.float16)
            el = np.empty((B,), dtype=np.int32)
            ref.ref_state_read(st, shift.ctypes.data_as(C.c_void_p), wkv.ctypes.data_as(C.c_void_p), el.ctypes.data_as(C.c_void_p))
            tag = "s32" if wkv32 else "s16"
            g[tag + "_n"] = len(calls)
            for i, (t, lg) in enumerate(calls):
                g[f"{tag}_tok{i}"] = t
                g[f"{tag}_logits{i}"] = lg
            if wkv_heads:
                wkv = np.ascontiguousarray(wkv[:, :, :wkv_heads])
            g[tag + "_shift"] = shift; g[tag + "_wkv"] = wkv; g[tag + "_elapsed"] = el
            ref.ref_state_destroy(st)
            ref.ref_backend_destroy(be)
    np.savez_compressed(os.path.join(out, name), **g)
    print(name + ":", len(g), "arrays")


def main():
    out = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--") else os.path.dirname(os.path.abspath(__file__))
    os.makedirs(out, exist_ok=True)
    ref = ref_lib()
    if ref is None:
        raise SystemExit("oracle/_ref/libref_rwkv7.so is missing: run `make -C oracle ref` where the reference sources are")
    if "--wide-only" in sys.argv:
        model(ref, out, WIDE, "ref_model_c4096.npz", lengths=(5, 20), wkv_heads=4)
        return
    if "--model-only" not in sys.argv:
        ops(ref, out)
    model(ref, out)
    model(ref, out, WIDE, "ref_model_c4096.npz", lengths=(5, 20), wkv_heads=4)


if __name__ == "__main__":
    main()
