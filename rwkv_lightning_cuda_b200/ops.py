"""Op-level bindings: one function per ``rwkv7_b200_*`` launcher export, on torch CUDA tensors.

Names follow the reference's launcher surface (cuda/rwkv7_fast_v4_kernels.cuh).  Everything is
enqueued on the current torch stream; nothing here computes on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import lib as L


def _s():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device-resident contiguous tensors only"
    return C.c_void_p(t.data_ptr())


def _ptr_table(ts: Sequence[torch.Tensor]):
    arr = (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
    return arr


def wkv_fp16_seq(B, T, H, state, r, w, k, v, a, b, elapsed, w0=None):
    y = torch.empty_like(r)
    lib = L.load_library()
    Cc = H * 64
    if w0 is None:
        L.check(lib.rwkv7_b200_wkv_fp16_seq(_s(), B, T, Cc, H, _p(state), _p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(y), _p(elapsed)))
    else:
        L.check(lib.rwkv7_b200_wkv_fp16_seq_w0(_s(), B, T, Cc, H, _p(state), _p(r), _p(w), _p(w0), _p(k), _p(v), _p(a), _p(b), _p(y), _p(elapsed)))
    return y


def wkv_fp32io16(B, T, H, state, r, w, k, v, a, b):
    y = torch.empty_like(r)
    L.check(L.load_library().rwkv7_b200_wkv_fp32io16(_s(), B, T, H * 64, H, _p(state), _p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(y)))
    return y


def tmix_mix6(B, T, x, shift, mixes: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    outs = [torch.empty_like(x) for _ in range(6)]
    L.check(L.load_library().rwkv7_b200_tmix_mix6(_s(), B, T, x.shape[-1], _p(x), _p(shift), _ptr_table(mixes), _ptr_table(outs)))
    return outs


def cmix_mix(B, T, x, shift, x_k):
    out = torch.empty_like(x)
    L.check(L.load_library().rwkv7_b200_cmix_mix(_s(), B, T, x.shape[-1], _p(x), _p(shift), _p(x_k), _p(out)))
    return out


def tmix_kk_a_gate(B, T, H, k, k_k, a0, a12, k_a):
    nk, nkk, kka = torch.empty_like(k), torch.empty_like(k), torch.empty_like(k)
    L.check(L.load_library().rwkv7_b200_tmix_kk_a_gate(_s(), B, T, H * 64, H, _p(k), _p(k_k), _p(a0), _p(a12), _p(k_a), _p(nk), _p(nkk), _p(kka)))
    return nk, nkk, kka


def tmix_lnx_rkvres_xg(B, T, H, x, r, k, v, r_k, weight, bias, g):
    out = torch.empty_like(x)
    L.check(L.load_library().rwkv7_b200_tmix_lnx_rkvres_xg(_s(), B, T, H * 64, H, _p(x), _p(r), _p(k), _p(v), _p(r_k), _p(weight), _p(bias), _p(g), _p(out)))
    return out


def tmix_vres_gate(B, T, v, v_first, v0, v12):
    out = torch.empty_like(v)
    L.check(L.load_library().rwkv7_b200_tmix_vres_gate(_s(), B, T, v.shape[-1], _p(v), _p(v_first), _p(v0), _p(v12), _p(out)))
    return out


def layer_norm_f16(x, weight, bias, eps=1e-5):
    y = torch.empty_like(x)
    L.check(L.load_library().rwkv7_b200_layer_norm_f16(_s(), x.shape[0], x.shape[1], _p(x), _p(weight), _p(bias), _p(y), eps))
    return y


def add_layer_norm_f16(x, residual, weight, bias, eps=1e-5):
    xo, y = torch.empty_like(x), torch.empty_like(x)
    L.check(L.load_library().rwkv7_b200_add_layer_norm_f16(_s(), x.shape[0], x.shape[1], _p(x), _p(residual), _p(weight), _p(bias), _p(xo), _p(y), eps))
    return xo, y


def add_last_layer_norm_f16(B, T, x, residual, weight, bias, eps=1e-5):
    y = torch.empty((B, x.shape[-1]), dtype=torch.float16, device=x.device)
    L.check(L.load_library().rwkv7_b200_add_last_layer_norm_f16(_s(), B, T, x.shape[-1], _p(x), _p(residual), _p(weight), _p(bias), _p(y), eps))
    return y


def add_layer_norm_cmix_mix_f16(B, T, x, residual, shift, weight, bias, x_k, eps=1e-5):
    xo, mixed = torch.empty_like(x), torch.empty_like(x)
    L.check(L.load_library().rwkv7_b200_add_layer_norm_cmix_mix_f16(_s(), B, T, x.shape[-1], _p(x), _p(residual), _p(shift), _p(weight), _p(bias), _p(x_k), _p(xo), _p(mixed), eps))
    return xo, mixed


def add_layer_norm_tmix_mix6_f16(B, T, x, residual, shift, weight, bias, mixes, eps=1e-5):
    xo = torch.empty_like(x)
    outs = [torch.empty_like(x) for _ in range(6)]
    L.check(L.load_library().rwkv7_b200_add_layer_norm_tmix_mix6_f16(_s(), B, T, x.shape[-1], _p(x), _p(residual), _p(shift), _p(weight), _p(bias), _ptr_table(mixes), _p(xo), _ptr_table(outs), eps))
    return xo, outs


def emb_ln0(emb, weight, bias, eps=1e-5):
    dt = L.DT_BF16 if emb.dtype == torch.bfloat16 else L.DT_F16
    out = torch.empty(emb.shape, dtype=torch.float16, device=emb.device)
    L.check(L.load_library().rwkv7_b200_emb_ln0(_s(), emb.shape[0], emb.shape[1], _p(emb), _p(weight), _p(bias), dt, _p(out), eps))
    return out


def relu_square(x):
    out = torch.empty_like(x)
    L.check(L.load_library().rwkv7_b200_relu_square(_s(), _p(x), _p(out), x.numel()))
    return out


def advance_i32(x, amount):
    L.check(L.load_library().rwkv7_b200_advance_i32(_s(), _p(x), amount, x.numel()))


def greedy_pick(logits, penalties=None, presence_penalty=0.0, repetition_penalty=0.0, penalty_decay=1.0, next_tokens=None):
    """Token ids int32 [B] = argmax(logits - penalties) per row; ``penalties`` is updated in place."""
    B, V = logits.shape
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    L.check(L.load_library().rwkv7_b200_greedy_pick(_s(), B, V, _p(logits), _p(penalties), presence_penalty, repetition_penalty,
                                                    penalty_decay, _p(out), _p(next_tokens)))
    return out


def _out(x, N, epi):
    return torch.empty((x.shape[0], N), dtype=torch.float32 if epi == L.EPI_F32 else torch.float16, device=x.device)


def linear_f16_orig(x, weight, in_act=L.ACT_NONE, epilogue=L.EPI_NONE):
    y = _out(x, weight.shape[0], epilogue)
    L.check(L.load_library().rwkv7_b200_linear_f16_orig(_s(), x.shape[0], x.shape[1], weight.shape[0], _p(x), _p(weight), in_act, epilogue, _p(y)))
    return y


def linear_f16_orig_static(x, weight, epilogue=L.EPI_NONE, out=None):
    """linear_f16_orig for more than four rows through the entry point that allocates nothing itself
    (its split-K scratch is a fixed device array inside the library).  Pass `out` to avoid the
    allocation of the result tensor as well."""
    y = _out(x, weight.shape[0], epilogue) if out is None else out
    L.check(L.load_library().rwkv7_b200_linear_f16_orig_static(_s(), x.shape[0], x.shape[1], weight.shape[0], _p(x), _p(weight), epilogue, _p(y)))
    return y


def linear_w8a16(x, q, scale, epilogue=L.EPI_NONE):
    y = _out(x, q.shape[0], epilogue)
    L.check(L.load_library().rwkv7_b200_linear_w8a16(_s(), x.shape[0], x.shape[1], q.shape[0], _p(x), _p(q), _p(scale), epilogue, _p(y)))
    return y


def linear_w4a16(x, q, scale, zero, epilogue=L.EPI_NONE):
    y = _out(x, q.shape[0], epilogue)
    L.check(L.load_library().rwkv7_b200_linear_w4a16(_s(), x.shape[0], x.shape[1], q.shape[0], _p(x), _p(q), _p(scale), _p(zero), epilogue, _p(y)))
    return y


def quant_pack_w8(W):
    N, K = W.shape
    q = torch.empty((N, K), dtype=torch.int8, device=W.device)
    s = torch.empty((N,), dtype=torch.float16, device=W.device)
    L.check(L.load_library().rwkv7_b200_quant_pack_w8(_s(), N, K, _p(W), _p(q), _p(s)))
    return q, s


def quant_unpack_w8(q, s):
    W = torch.empty(q.shape, dtype=torch.float16, device=q.device)
    L.check(L.load_library().rwkv7_b200_quant_unpack_w8(_s(), q.shape[0], q.shape[1], _p(q), _p(s), _p(W)))
    return W


def quant_pack_w4(W):
    N, K = W.shape
    q = torch.empty((N, K // 2), dtype=torch.uint8, device=W.device)
    s = torch.empty((N, K // 128), dtype=torch.float16, device=W.device)
    z = torch.empty((N, K // 128), dtype=torch.float16, device=W.device)
    L.check(L.load_library().rwkv7_b200_quant_pack_w4(_s(), N, K, _p(W), _p(q), _p(s), _p(z)))
    return q, s, z


def quant_unpack_w4(q, s, z):
    N, K = q.shape[0], q.shape[1] * 2
    W = torch.empty((N, K), dtype=torch.float16, device=q.device)
    L.check(L.load_library().rwkv7_b200_quant_unpack_w4(_s(), N, K, _p(q), _p(s), _p(z), _p(W)))
    return W


def sample(logits, penalties=None, presence=0.0, repetition=0.0, decay=1.0, temperature=1.0, top_k=0, top_p=1.0, seed=0, offset=0,
           next_tokens=None):
    """One token per row of fp32 logits [B, V] with the sampler's rule (temperature, top-k, top-p, penalties updated in
    place); the draw is a function of (seed, offset, row).  Returns int32 [B] on the device."""
    B, V = logits.shape
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    probs = torch.empty((B, V), dtype=torch.float32, device=logits.device)
    sp = L.Sampling(temperature, top_k, top_p, seed, offset)
    import ctypes as C
    L.check(L.load_library().rwkv7_b200_sample(_s(), B, V, _p(logits), _p(penalties), _p(probs), presence, repetition, decay,
                                                C.byref(sp), _p(out), _p(next_tokens)))
    return out
