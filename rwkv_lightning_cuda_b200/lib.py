"""ctypes declarations of every entry point in ``include/rwkv7_b200.h``."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

FMT_F16, FMT_W8A16, FMT_W4A16 = 0, 1, 2
DT_F16, DT_BF16 = 0, 1
ACT_NONE, ACT_TANH, ACT_SIGMOID = 0, 1, 2
EPI_NONE, EPI_RELU2, EPI_F32 = 0, 1, 3

STATUS_NAMES = {0: "OK", 1: "BAD_ARG", 2: "SHAPE", 3: "PRECISION", 4: "CUDA", 5: "NCCL", 6: "TIMEOUT", 7: "NOT_READY"}


class Rwkv7B200Error(RuntimeError):
    """Raised when a library call returns a non-zero status (the reference throws std::runtime_error)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"rwkv7_b200 [{STATUS_NAMES.get(status, status)}]: {message}")
        self.status = status


class Config(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "layers", "channels", "ffn", "vocab", "rank_w", "rank_a", "rank_v", "rank_g",
        "weight_format", "wkv32", "device", "tp_rank", "tp_size")]


class Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("seed", C.c_ulonglong), ("offset", C.c_ulonglong)]


class Capacity(C.Structure):
    _fields_ = [("free_vram_bytes", C.c_size_t), ("total_vram_bytes", C.c_size_t), ("reserve_vram_bytes", C.c_size_t),
                ("bytes_per_batch", C.c_size_t), ("max_batch_size", C.c_int)]


_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float

# name -> argtypes; every function returns int unless listed in _RESTYPES
SIGNATURES = {
    "rwkv7_b200_last_error": [],
    "rwkv7_b200_abi_version": [],
    "rwkv7_b200_model_create": [C.POINTER(Config), C.POINTER(_vp)],
    "rwkv7_b200_model_set_tensor": [_vp, C.c_char_p, _vp, _i, _ll, _i],
    "rwkv7_b200_model_finalize": [_vp],
    "rwkv7_b200_tp_unique_id": [_vp],
    "rwkv7_b200_model_tp_init": [_vp, _vp],
    "rwkv7_b200_model_destroy": [_vp],
    "rwkv7_b200_vocab_size": [_vp],
    "rwkv7_b200_state_sizes": [_vp, _i, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)],
    "rwkv7_b200_state_init": [_vp, _i, _vp, _vp, _vp, _vp],
    "rwkv7_b200_forward": [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp],
    "rwkv7_b200_forward_to_host": [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "rwkv7_b200_decode_greedy": [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _f, _f, _f, _vp, _vp, _vp],
    "rwkv7_b200_greedy_pick": [_vp, _i, _i, _vp, _vp, _f, _f, _f, _vp, _vp],
    "rwkv7_b200_decode_sample": [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _f, _f, _f, C.POINTER(Sampling), _vp, _vp, _vp],
    "rwkv7_b200_sample": [_vp, _i, _i, _vp, _vp, _vp, _f, _f, _f, C.POINTER(Sampling), _vp, _vp],
    "rwkv7_b200_copy_state_slice": [_vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp],
    "rwkv7_b200_state_blob_sizes": [_vp, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)],
    "rwkv7_b200_state_export": [_vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp],
    "rwkv7_b200_state_import": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "rwkv7_b200_state_convert_wkv": [_vp, _vp, _vp, _ll, _i],
    "rwkv7_b200_query_capacity": [_vp, _i, C.POINTER(Capacity)],
    "rwkv7_b200_kernel_launches": [_vp],
    "rwkv7_b200_model_workspace_bytes": [_vp, C.POINTER(C.c_size_t)],
    "rwkv7_b200_timeout_flags": [_i, C.POINTER(_i)],
    "rwkv7_b200_debug_wait_probe": [_vp, C.c_uint],
    "rwkv7_b200_debug_timeout_detail": [C.POINTER(_i), _i],
    "rwkv7_b200_debug_last_gemm_splits": [],
    "rwkv7_b200_set_option": [C.c_char_p, _i],
    "rwkv7_b200_wkv_fp16_seq": [_vp, _i, _i, _i, _i] + [_vp] * 9,
    "rwkv7_b200_wkv_fp16_seq_w0": [_vp, _i, _i, _i, _i] + [_vp] * 10,
    "rwkv7_b200_wkv_fp32io16": [_vp, _i, _i, _i, _i] + [_vp] * 8,
    "rwkv7_b200_tmix_mix6": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp],
    "rwkv7_b200_cmix_mix": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp],
    "rwkv7_b200_tmix_kk_a_gate": [_vp, _i, _i, _i, _i] + [_vp] * 8,
    "rwkv7_b200_tmix_lnx_rkvres_xg": [_vp, _i, _i, _i, _i] + [_vp] * 9,
    "rwkv7_b200_tmix_vres_gate": [_vp, _i, _i, _i] + [_vp] * 5,
    "rwkv7_b200_layer_norm_f16": [_vp, _i, _i, _vp, _vp, _vp, _vp, _f],
    "rwkv7_b200_add_layer_norm_f16": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _f],
    "rwkv7_b200_add_last_layer_norm_f16": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _f],
    "rwkv7_b200_add_layer_norm_cmix_mix_f16": [_vp, _i, _i, _i] + [_vp] * 8 + [_f],
    "rwkv7_b200_add_layer_norm_tmix_mix6_f16": [_vp, _i, _i, _i] + [_vp] * 8 + [_f],
    "rwkv7_b200_emb_ln0": [_vp, _i, _i, _vp, _vp, _vp, _i, _vp, _f],
    "rwkv7_b200_relu_square": [_vp, _vp, _vp, _ll],
    "rwkv7_b200_advance_i32": [_vp, _vp, _i, _ll],
    "rwkv7_b200_linear_f16_orig": [_vp, _i, _i, _i, _vp, _vp, _i, _i, _vp],
    "rwkv7_b200_linear_f16_orig_static": [_vp, _i, _i, _i, _vp, _vp, _i, _vp],
    "rwkv7_b200_linear_w8a16": [_vp, _i, _i, _i, _vp, _vp, _vp, _i, _vp],
    "rwkv7_b200_linear_w4a16": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp],
    "rwkv7_b200_quant_pack_w8": [_vp, _i, _i, _vp, _vp, _vp],
    "rwkv7_b200_quant_unpack_w8": [_vp, _i, _i, _vp, _vp, _vp],
    "rwkv7_b200_quant_pack_w4": [_vp, _i, _i, _vp, _vp, _vp, _vp],
    "rwkv7_b200_quant_unpack_w4": [_vp, _i, _i, _vp, _vp, _vp, _vp],
}
_RESTYPES = {"rwkv7_b200_last_error": C.c_char_p, "rwkv7_b200_kernel_launches": C.c_longlong}


def library_path() -> str:
    return os.path.join(_HERE, "librwkv7_b200.so")


def load_library() -> C.CDLL:
    """Loads the CUDA library; raises (never falls back) when it is missing or incomplete."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m rwkv_lightning_cuda_b200.build` "
            "(nvcc, sm_100a). There is no CPU fallback.")
    lib = C.CDLL(path)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the export is missing
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, C.c_int)
    _LIB = lib
    return lib


def set_option(name: str, value: int) -> None:
    """rwkv7_b200_set_option: process-wide switches for measurements and tests (see the header)."""
    check(load_library().rwkv7_b200_set_option(name.encode(), int(value)))


def timeout_detail(clear: bool = True):
    """The record of the first expired GEMM wait (see the header); a list of 15 ints, all zero when nothing expired."""
    buf = (C.c_int * 15)()
    check(load_library().rwkv7_b200_debug_timeout_detail(buf, int(clear)))
    return list(buf)


def timeout_flags(clear: bool = True) -> int:
    """The current device's failure word (bits: 1 GEMV, 2 GEMM, 4 time-mix, 8 probe, 16 peer all-reduce)."""
    v = C.c_int(0)
    check(load_library().rwkv7_b200_timeout_flags(int(clear), C.byref(v)))
    return v.value


def check(status: int) -> None:
    if status != 0:
        msg = load_library().rwkv7_b200_last_error()
        raise Rwkv7B200Error(status, msg.decode() if msg else "")
