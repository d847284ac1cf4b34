"""CPU-only checks of the drop-in boundary: the library loads, exports exactly what
include/rwkv7_b200.h declares, and rejects bad arguments with a status code before touching CUDA."""
import ctypes as C
import os
import re

import pytest

from tests.helpers import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "rwkv7_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rwkv7_b200_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from rwkv_lightning_cuda_b200 import build, lib as L
    build.build()
    return L.load_library()


def test_every_declared_symbol_is_exported_and_bound(lib):
    from rwkv_lightning_cuda_b200 import lib as L
    names = declared_functions()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(L.SIGNATURES) == names, "python binding table and header disagree"
    assert lib.rwkv7_b200_abi_version() == 1


def test_bad_config_is_rejected_without_a_gpu(lib):
    from rwkv_lightning_cuda_b200 import lib as L
    h = C.c_void_p()
    good = dict(layers=2, channels=128, ffn=512, vocab=64, rank_w=32, rank_a=32, rank_v=16, rank_g=64,
                weight_format=0, wkv32=0, device=-1, tp_rank=0, tp_size=1)
    for patch, status in ((dict(channels=100), 2), (dict(layers=0), 2), (dict(rank_g=520), 2), (dict(weight_format=7), 1),
                          (dict(weight_format=2, channels=192), 2)):
        cfg = L.Config(**{**good, **patch})
        assert lib.rwkv7_b200_model_create(C.byref(cfg), C.byref(h)) == status
        assert lib.rwkv7_b200_last_error()
    assert lib.rwkv7_b200_model_create(None, C.byref(h)) == 1
    cfg = L.Config(**good)
    assert lib.rwkv7_b200_model_create(C.byref(cfg), C.byref(h)) == 0
    ns, nw, ne = C.c_size_t(), C.c_size_t(), C.c_size_t()
    assert lib.rwkv7_b200_state_sizes(h, 3, C.byref(ns), C.byref(nw), C.byref(ne)) == 0
    # GenerationState layout: shift [L][2][B][C], wkv [L][B][H][64][64], elapsed [B]
    assert (ns.value, nw.value, ne.value) == (2 * 2 * 3 * 128, 2 * 3 * 2 * 64 * 64, 3)
    assert lib.rwkv7_b200_state_sizes(h, 0, None, None, None) == 1
    assert b"positive" in lib.rwkv7_b200_last_error()
    # forward before finalize / with bad shapes fails with a status, it never exits the process
    assert lib.rwkv7_b200_forward(h, None, 1, 1, None, None, None, None, None) == 7
    assert lib.rwkv7_b200_model_destroy(h) == 0


def test_options_are_named_ranged_and_documented(lib):
    """rwkv7_b200_set_option: every switch the header documents is accepted at its documented default, values outside
    its range and unknown names are refused with BAD_ARG (no GPU involved: the switches are host-side state)."""
    import re
    text = open(os.path.join(ROOT, "include", "rwkv7_b200.h")).read()
    end = text.index("int rwkv7_b200_set_option")
    block = text[text.rindex("/*", 0, end):end]
    documented = re.findall(r'^ \*   "([a-z0-9_]+)"', block, flags=re.M)
    defaults = dict(gemm_cta_pair=0, quant_tc_rows=0, fp16_tc_rows=0, decode_graphs=1, wkv_chunked=1, tp_peer_ranks=2,
                    gemv_mma_tall=2, gemv_mma=3)
    assert sorted(documented) == sorted(defaults), (documented, "header and test disagree about the options")
    for name, value in defaults.items():
        assert lib.rwkv7_b200_set_option(name.encode(), value) == 0, name
    assert lib.rwkv7_b200_set_option(b"gemv_mma", 5) == 1 and b"gemv_mma" in lib.rwkv7_b200_last_error()
    assert lib.rwkv7_b200_set_option(b"decode_graphs", -1) == 1
    assert lib.rwkv7_b200_set_option(b"no_such_option", 0) == 1
    assert lib.rwkv7_b200_set_option(None, 0) == 1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from rwkv_lightning_cuda_b200 import lib as L
    monkeypatch.setattr(L, "_LIB", None)
    monkeypatch.setattr(L, "_HERE", str(tmp_path))
    with pytest.raises(ImportError, match="no CPU fallback"):
        L.load_library()


def test_adapter_compiles_against_the_unmodified_reference_headers():
    """The C++ IModelBackend adapter must build against the reference's own headers (drop-in proof)."""
    import shutil
    import subprocess
    from oracle.oracle import reference_dir
    ref = os.path.join(reference_dir(), "include")
    if not os.path.isdir(ref) or shutil.which("g++") is None:
        pytest.skip("reference tree or g++ not present")
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-I" + ref, "-I/usr/local/cuda/include", "-I" + os.path.join(ROOT, "include"),
           os.path.join(ROOT, "rwkv_lightning_cuda_b200", "adapter", "b200_model_backend.cpp")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def test_infer_model_dims_follows_the_reference_rule():
    """Dimensions and LoRA ranks come from the checkpoint's tensor shapes as in the reference
    (include/rwkv7_fast_v4_common.hpp:262-288); its three failure messages are kept."""
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic
    d = bk.ModelDims(3, 128, 512, 320, 32, 24, 16, 64)
    shapes = synthetic.tensor_shapes(d)
    assert bk.infer_model_dims(shapes) == d
    one = {k: v for k, v in shapes.items() if not k.startswith(("blocks.1.", "blocks.2."))}
    assert bk.infer_model_dims(one) == bk.ModelDims(1, 128, 512, 320, 32, 24, 8, 64)
    with pytest.raises(ValueError, match="could not infer model dimensions"):
        bk.infer_model_dims({k: v for k, v in shapes.items() if k != "emb.weight"})
    with pytest.raises(ValueError, match="C must equal H\\*N"):
        bk.infer_model_dims({**shapes, "blocks.0.att.r_k": (3, 64)})
    with pytest.raises(ValueError, match="head size 64"):
        bk.infer_model_dims({**shapes, "blocks.0.att.r_k": (4, 32)})
