"""ctypes front-end of the CPU oracle (``liboracle.so``).

Test infrastructure only: imported by the tests, by ``__graft_entry__.smoke()`` and by the
CPU-baseline legs of ``bench.py``; the product package never imports it.

All half tensors are numpy ``float16`` arrays (passed as raw bits), layouts as in the
reference: activations ``[B*T, C]`` row-major, WKV state ``[B, H, 64, 64]``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

ACT_NONE, ACT_TANH, ACT_SIGMOID = 0, 1, 2
EPI_NONE, EPI_RELU2 = 0, 1
FMT_F16, FMT_W8A16, FMT_W4A16 = 0, 1, 2


def build() -> str:
    """Compile the oracle with gcc if the shared object is missing or stale."""
    so = os.path.join(_HERE, "liboracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("rwkv7_oracle.c", "softfp16.h")]
    if not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.check_call(["make", "-s", "-C", _HERE, "all"])
    return so


def reference_dir() -> str:
    """Where the reference project's checkout is looked for when the oracle is built against it:
    $RWKV7_REFERENCE_DIR, else a directory named ``reference`` beside this repository."""
    return os.environ.get("RWKV7_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def ref_lib():
    """The reference's own kernels and backend, built unmodified under oracle/_ref/ by ``make -C oracle ref``
    (None when that build is absent).  A checker and a timed baseline, never part of the product path."""
    path = os.path.join(_HERE, "_ref", "libref_rwkv7.so")
    if not os.path.exists(path):
        return None
    r = C.CDLL(path)
    r.ref_last_error.restype = C.c_char_p
    r.ref_backend_create.restype = C.c_void_p
    r.ref_state_create.restype = C.c_void_p
    r.ref_backend_create.argtypes = [C.c_char_p, C.c_int]
    r.ref_backend_destroy.argtypes = [C.c_void_p]
    r.ref_state_create.argtypes = [C.c_void_p, C.c_int]
    r.ref_state_destroy.argtypes = [C.c_void_p]
    r.ref_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    r.ref_state_read.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    return r


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.orc_h2f.restype = C.c_float
        _LIB.orc_f2h.restype = C.c_uint16
        _LIB.orc_f2h.argtypes = [C.c_float]
        _LIB.orc_hfma.restype = C.c_uint16
        _LIB.orc_hadd.restype = C.c_uint16
        _LIB.orc_model_create.restype = C.c_void_p
        _LIB.orc_model_set.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_longlong]
        _LIB.orc_model_destroy.argtypes = [C.c_void_p]
    return _LIB


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle inputs must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _h(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def f2h(x: float) -> int:
    return lib().orc_f2h(float(x))


def hfma(a: int, b: int, c: int) -> int:
    return lib().orc_hfma(C.c_uint16(a), C.c_uint16(b), C.c_uint16(c))


def hadd(a: int, b: int) -> int:
    return lib().orc_hadd(C.c_uint16(a), C.c_uint16(b))


def layer_norm(x, w, b, eps=1e-5):
    x = _h(x); y = np.empty_like(x)
    lib().orc_layer_norm(x.shape[0], x.shape[1], _p(x), _p(_h(w)), _p(_h(b)), _p(y), C.c_float(eps))
    return y


def add_layer_norm(x, res, w, b, eps=1e-5):
    x = _h(x); res = _h(res); xo = np.empty_like(x); y = np.empty_like(x)
    lib().orc_add_layer_norm(x.shape[0], x.shape[1], _p(x), _p(res), _p(_h(w)), _p(_h(b)), _p(xo), _p(y), C.c_float(eps))
    return xo, y


def add_last_layer_norm(B, T, x, res, w, b, eps=1e-5):
    x = _h(x); res = _h(res); Cc = x.shape[-1]
    y = np.empty((B, Cc), np.float16)
    lib().orc_add_last_layer_norm(B, T, Cc, _p(x), _p(res), _p(_h(w)), _p(_h(b)), _p(y), C.c_float(eps))
    return y


def emb_ln0(emb, w, b, eps=1e-5):
    emb = np.ascontiguousarray(emb, np.float32); w = np.ascontiguousarray(w, np.float32); b = np.ascontiguousarray(b, np.float32)
    out = np.empty(emb.shape, np.float16)
    lib().orc_emb_ln0(emb.shape[0], emb.shape[1], _p(emb), _p(w), _p(b), _p(out), C.c_float(eps))
    return out


def tmix_mix6(B, T, x, shift, mixes):
    """Returns the six mixed tensors; ``shift`` ([B,C]) is updated in place."""
    x = _h(x); Cc = x.shape[-1]
    mixes = [_h(m) for m in mixes]
    outs = [np.empty_like(x) for _ in range(6)]
    MixArr = C.c_void_p * 6
    lib().orc_tmix_mix6(B, T, Cc, _p(x), _p(shift), MixArr(*[m.ctypes.data for m in mixes]),
                        MixArr(*[o.ctypes.data for o in outs]))
    return outs


def cmix_mix(B, T, x, shift, x_k):
    x = _h(x); out = np.empty_like(x)
    lib().orc_cmix_mix(B, T, x.shape[-1], _p(x), _p(shift), _p(_h(x_k)), _p(out))
    return out


def kk_a_gate(k, k_k, a0, a12, k_a):
    k = _h(k); rows, Cc = k.shape
    nk, nkk, kka = np.empty_like(k), np.empty_like(k), np.empty_like(k)
    lib().orc_kk_a_gate(rows, Cc, _p(k), _p(_h(k_k)), _p(_h(a0)), _p(_h(a12)), _p(_h(k_a)), _p(nk), _p(nkk), _p(kka))
    return nk, nkk, kka


def vres_gate(v, v_first, v0, v12):
    v = _h(v); out = np.empty_like(v)
    lib().orc_vres_gate(v.shape[0], v.shape[1], _p(v), _p(_h(v_first)), _p(_h(v0)), _p(_h(v12)), _p(out))
    return out


def lnx_rkvres_xg(y, r, k, v, r_k, w, b, g):
    y = _h(y); out = np.empty_like(y)
    lib().orc_lnx_rkvres_xg(y.shape[0], y.shape[1], _p(y), _p(_h(r)), _p(_h(k)), _p(_h(v)), _p(_h(r_k)),
                            _p(_h(w)), _p(_h(b)), _p(_h(g)), _p(out))
    return out


def linear_orig(x, W, in_act=ACT_NONE, epi=EPI_NONE):
    """y = act(x) @ W.T, W is [N,K]."""
    x = _h(x); W = _h(W); M, K = x.shape; N = W.shape[0]
    y = np.empty((M, N), np.float16)
    lib().orc_linear_orig(M, K, N, _p(x), _p(W), _p(y), in_act, epi)
    return y


def linear_kn(x, W, in_act=ACT_NONE):
    """y = act(x) @ W, W is [K,N]."""
    x = _h(x); W = _h(W); M, K = x.shape; N = W.shape[1]
    y = np.empty((M, N), np.float16)
    lib().orc_linear_kn(M, K, N, _p(x), _p(W), _p(y), in_act)
    return y


def quant_pack_w8(W):
    W = _h(W); N, K = W.shape
    q = np.empty((N, K), np.int8); s = np.empty((N,), np.float16)
    lib().orc_quant_pack_w8(N, K, _p(W), _p(q), _p(s))
    return q, s


def quant_unpack_w8(q, s):
    N, K = q.shape; W = np.empty((N, K), np.float16)
    lib().orc_quant_unpack_w8(N, K, _p(np.ascontiguousarray(q)), _p(_h(s)), _p(W))
    return W


def quant_pack_w4(W):
    W = _h(W); N, K = W.shape
    assert K % 128 == 0
    q = np.empty((N, K // 2), np.uint8); s = np.empty((N, K // 128), np.float16); z = np.empty((N, K // 128), np.float16)
    lib().orc_quant_pack_w4(N, K, _p(W), _p(q), _p(s), _p(z))
    return q, s, z


def quant_unpack_w4(q, s, z):
    N = q.shape[0]; K = q.shape[1] * 2; W = np.empty((N, K), np.float16)
    lib().orc_quant_unpack_w4(N, K, _p(np.ascontiguousarray(q)), _p(_h(s)), _p(_h(z)), _p(W))
    return W


def linear_w8a16(x, q, s, epi=EPI_NONE):
    x = _h(x); M, K = x.shape; N = q.shape[0]; y = np.empty((M, N), np.float16)
    lib().orc_linear_w8a16(M, K, N, _p(x), _p(np.ascontiguousarray(q)), _p(_h(s)), _p(y), epi)
    return y


def linear_w4a16(x, q, s, z, epi=EPI_NONE):
    x = _h(x); M, K = x.shape; N = q.shape[0]; y = np.empty((M, N), np.float16)
    lib().orc_linear_w4a16(M, K, N, _p(x), _p(np.ascontiguousarray(q)), _p(_h(s)), _p(_h(z)), _p(y), epi)
    return y


def wkv_fp32(B, T, H, state, r, w, k, v, a, b):
    """state float32 [B,H,64,64] updated in place; returns y [B*T, C] float16."""
    Cc = H * 64
    assert state.dtype == np.float32 and state.flags["C_CONTIGUOUS"]
    y = np.empty((B * T, Cc), np.float16)
    lib().orc_wkv_fp32(B, T, Cc, H, _p(state), _p(_h(r)), _p(_h(w)), _p(_h(k)), _p(_h(v)), _p(_h(a)), _p(_h(b)), _p(y))
    return y


def wkv_fp16(B, T, H, state, r, w, w0, k, v, a, b, elapsed):
    """state float16 [B,H,64,64] updated in place; w0 may be None; elapsed int32 [B]."""
    Cc = H * 64
    assert state.dtype == np.float16 and state.flags["C_CONTIGUOUS"]
    elapsed = np.ascontiguousarray(elapsed, np.int32)
    y = np.empty((B * T, Cc), np.float16)
    lib().orc_wkv_fp16(B, T, Cc, H, _p(state), _p(_h(r)), _p(_h(w)), _p(_h(w0)) if w0 is not None else None,
                       _p(_h(k)), _p(_h(v)), _p(_h(a)), _p(_h(b)), _p(y), _p(elapsed))
    return y


def greedy_pick(logits, penalties=None, presence=0.0, repetition=0.0, decay=1.0):
    """The reference sampler's greedy case (top_p == 0 => top_k = 1, src/utils/sampling.cu:507-512) restated in numpy.

    Per row: value = finite(logit) - penalty (:253 with :139-142: NaN -> 0, +-inf -> +-FLT_MAX; the temperature is a
    positive factor and drops out of an argmax), token = the largest value's index (the lowest index among equal
    values -- the reference draws among them at random), then penalty = fma(penalty, decay, chosen ? (penalty == 0 ?
    presence : repetition) : 0) (:460-469).  ``penalties`` (fp32 [B, V]) is updated in place.  Returns int32 [B].
    """
    lg = np.asarray(logits, dtype=np.float32)
    fmax = np.finfo(np.float32).max
    val = np.where(np.isnan(lg), np.float32(0), np.clip(lg, -fmax, fmax)).astype(np.float32)
    if penalties is not None:
        with np.errstate(invalid="ignore", over="ignore"):
            val = (val - penalties).astype(np.float32)
    out = np.zeros(lg.shape[0], dtype=np.int32)
    for b in range(lg.shape[0]):
        row = val[b]
        ok = ~np.isnan(row)
        if ok.any():
            out[b] = int(np.flatnonzero(ok & (row == row[ok].max()))[0])
        if penalties is not None:
            p = penalties[b].astype(np.float64)
            add = np.zeros_like(p)
            add[out[b]] = presence if penalties[b, out[b]] == 0 else repetition
            with np.errstate(invalid="ignore", over="ignore"):
                penalties[b] = (p * float(np.float32(decay)) + add.astype(np.float32)).astype(np.float32)
    return out


class Model:
    """Whole-model oracle; tensors are set by checkpoint name as float16 arrays."""

    def __init__(self, L, Cc, F, V, Rw, Ra, Rv, Rg, fmt=FMT_F16):
        self.L, self.C, self.F, self.V, self.H = L, Cc, F, V, Cc // 64
        self.h = lib().orc_model_create(L, Cc, F, V, Rw, Ra, Rv, Rg, fmt)

    def set(self, name: str, arr) -> None:
        arr = _h(arr)
        ok = lib().orc_model_set(self.h, name.encode(), _p(arr), arr.size)
        if not ok:
            raise KeyError(f"oracle: tensor {name} not accepted")

    def new_state(self, B, wkv32):
        shift = np.zeros((self.L, 2, B, self.C), np.float16)
        wkv = np.zeros((self.L, B, self.H, 64, 64), np.float32 if wkv32 else np.float16)
        elapsed = np.zeros((B,), np.int32)
        return shift, wkv, elapsed

    def forward(self, tokens, shift, wkv, elapsed, lora_round_act=0):
        tokens = np.ascontiguousarray(tokens, np.int64)
        B, T = tokens.shape
        logits = np.empty((B, self.V), np.float32)
        wkv32 = 1 if wkv.dtype == np.float32 else 0
        rc = lib().orc_forward(C.c_void_p(self.h), _p(tokens), B, T, wkv32, lora_round_act, _p(shift), _p(wkv), _p(elapsed), _p(logits))
        if rc != 0:
            raise ValueError("token id out of range")
        return logits

    def __del__(self):
        try:
            lib().orc_model_destroy(self.h)
        except Exception:
            pass


def philox4x32_first(c0, c1, c2, c3, k0, k1):
    """First output word of Philox-4x32-10 (Salmon et al. 2011), plain Python integers."""
    M = 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = 0xD2511F53 * c0, 0xCD9E8D57 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & M, p1 & M, ((p0 >> 32) ^ c3 ^ k1) & M, p0 & M
        k0, k1 = (k0 + 0x9E3779B9) & M, (k1 + 0xBB67AE85) & M
    return c0


def sample_weights(logits, penalties=None, temperature=1.0, top_k=0, top_p=1.0):
    """What the sampler keeps of every token's probability, [B, V] float64: the reference's rule
    (src/utils/sampling.cu:205-399, argument rules :504-512) restated -- softmax of (finite(logit) - penalty) / T, the
    smallest threshold t whose strictly-greater tokens stay strictly inside both budgets, tokens on the threshold scaled to fill them."""
    lg = np.asarray(logits, dtype=np.float32)
    B, V = lg.shape
    if top_k <= 0 or top_k > V:
        top_k = V
    if not (0.0 <= top_p <= 1.0):
        top_p = 1.0
    if top_p == 0.0:
        top_k, top_p = 1, 1.0
    big = np.float32(np.finfo(np.float32).max)
    fin = lambda x: np.clip(np.nan_to_num(x, nan=0.0, posinf=big, neginf=-big), -big, big)
    pen = np.zeros_like(lg) if penalties is None else np.asarray(penalties, dtype=np.float32)
    z = fin((fin(lg) - pen).astype(np.float32) * np.float32(1.4426950408889634 / temperature)).astype(np.float64)
    p = np.exp2(z - z.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    w = np.zeros_like(p)
    for b in range(B):
        vals = np.unique(p[b])[::-1]                     # distinct values, descending
        thr = vals[-1]
        for v in vals:                                   # the first value at which a budget is reached: everything
            keep = p[b] >= v                             # strictly above it is still strictly inside both budgets
            if keep.sum() >= top_k or p[b][keep].sum() >= top_p:
                thr = v
                break
        above, on = p[b] > thr, p[b] == thr
        n = on.sum()
        comp = 1.0
        if n:
            comp = min(comp, (top_p - p[b][above].sum()) / (thr * n), (top_k - above.sum()) / n)
            comp = max(comp, 0.0)
        w[b] = np.where(above, p[b], np.where(on, p[b] * comp, 0.0))
    return w


def sample(logits, penalties=None, presence=0.0, repetition=0.0, decay=1.0, temperature=1.0, top_k=0, top_p=1.0, seed=0, offset=0):
    """Tokens [B] drawn with the counter-based uniform number of (seed, offset, row): the first token whose cumulative kept
    weight reaches u * total.  `penalties` ([B, V] float32) is updated in place like greedy_pick does."""
    w = sample_weights(logits, penalties, temperature, top_k, top_p)
    B, V = w.shape
    out = np.zeros(B, dtype=np.int64)
    for b in range(B):
        bits = philox4x32_first(offset & 0xFFFFFFFF, (offset >> 32) & 0xFFFFFFFF, b, 0, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
        u = ((bits >> 8) + 0.5) / 16777216.0
        cum = np.cumsum(w[b])
        idx = int(np.searchsorted(cum, u * cum[-1], side="left"))
        idx = min(idx, V - 1)
        while w[b][idx] == 0.0 and idx > 0:              # (cannot happen for side="left" unless rounding: stay on a kept token)
            idx -= 1
        out[b] = idx
    if penalties is not None:
        for b in range(B):
            hit = penalties[b, out[b]]
            add = np.float32(presence if hit == 0 else repetition)
            penalties[b] = (penalties[b].astype(np.float32) * np.float32(decay)).astype(np.float32)
            penalties[b, out[b]] = np.float32(np.float32(hit) * np.float32(decay) + add)
    return out
