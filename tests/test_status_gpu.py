"""The TIMEOUT status and the model's single grow-only workspace.

A kernel of this library never waits without a poll limit; when a limit runs out the kernel sets a bit in a
per-device failure word and returns.  The test makes such a wait run out without losing a copy or stalling
anything (a one-thread kernel polling a barrier that nothing completes) and checks that the calls which
synchronise report status 6, that the word is reset, and that the next call works."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_becomes_status_timeout_and_the_next_call_is_clean():
    from rwkv_lightning_cuda_b200 import backend as bk, lib as L
    from oracle.parity import build_pair
    lib = L.load_library()
    assert L.timeout_flags(clear=True) == 0 or True          # start from a clean word
    d, om, gm = build_pair(orc.FMT_F16, False)
    st = gm.create_state(1); lg = bk.DeviceLogits()
    out = torch.empty((1, d.vocab), dtype=torch.float32).pin_memory()
    toks = torch.tensor([[3]], dtype=torch.int64)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        gm.forward_to_host(toks, st, lg, out)                 # a normal call: status 0
        good = out.clone()
        L.check(lib.rwkv7_b200_debug_wait_probe(C.c_void_p(s.cuda_stream), 2000))
        with pytest.raises(L.Rwkv7B200Error) as e:
            gm.forward_to_host(toks, st, lg, out)
        assert e.value.status == 6 and "bounded wait" in str(e.value)
        assert L.timeout_flags(clear=False) == 0              # reported once, then reset
        st2 = gm.create_state(1)
        gm.forward_to_host(toks, st2, lg, out)                # the context is intact: same result as the first call
        assert torch.equal(out, good)
        # asynchronous callers read the word themselves
        L.check(lib.rwkv7_b200_debug_wait_probe(C.c_void_p(s.cuda_stream), 10))
        s.synchronize()
        assert L.timeout_flags(clear=True) == 8 and L.timeout_flags(clear=True) == 0
        # decode_greedy with a host buffer synchronises too
        L.check(lib.rwkv7_b200_debug_wait_probe(C.c_void_p(s.cuda_stream), 10))
        host = torch.empty((2, 1), dtype=torch.int32).pin_memory()
        with pytest.raises(L.Rwkv7B200Error) as e:
            gm.decode_greedy([5], 2, st2, lg, out_host=host)
        assert e.value.status == 6
        gm.decode_greedy([5], 2, st2, lg, out_host=host)
    with pytest.raises(L.Rwkv7B200Error, match="unknown option"):
        L.set_option("no_such_switch", 1)
    with pytest.raises(L.Rwkv7B200Error, match="must be in"):
        L.set_option("decode_graphs", 7)


def test_the_workspace_is_one_grow_only_arena_whatever_shapes_are_called():
    """The reference's engine calls forward_prefill with whatever (active sequences, chunk) pair is left
    (src/rwkv_inference_engine.cpp:288-329).  Device memory must stop falling once the largest shape has been seen,
    results must not depend on the order of shapes, and calls on different streams must not trample each other."""
    from rwkv_lightning_cuda_b200 import backend as bk, lib as L
    from oracle.parity import build_pair
    lib = L.load_library()
    d, om, gm = build_pair(orc.FMT_F16, False)

    def ws_bytes():
        v = C.c_size_t(0)
        L.check(lib.rwkv7_b200_model_workspace_bytes(gm._h, C.byref(v)))
        return v.value

    rng = np.random.default_rng(3)
    lg = bk.DeviceLogits()
    states = {B: gm.create_state(B) for B in (1, 2, 3, 5, 8)}
    big = gm.create_state(8)
    gm.forward_prefill(rng.integers(0, d.vocab, (8, 40)).tolist(), big, lg)       # the largest call
    held = ws_bytes()
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    shapes = [(B, T) for B in (1, 2, 3, 5, 8) for T in (1, 2, 7, 16, 33, 40)]
    for B, T in shapes:
        gm.forward_prefill(rng.integers(0, d.vocab, (B, T)).tolist(), states[B], lg)
    torch.cuda.synchronize()
    assert ws_bytes() == held, "smaller shapes must reuse the arena"
    assert torch.cuda.mem_get_info()[0] >= free0 - (8 << 20), "device memory kept falling with new shapes"
    # same tokens, same state history -> same logits, whether or not other shapes ran in between, on either stream
    toks = rng.integers(0, d.vocab, (2, 5))
    outs = []
    for other in (False, True):
        st = gm.create_state(2)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            gm.forward_prefill(toks.tolist(), st, lg, sync=False)
            first = lg.values
        if other:      # a call on another stream right behind it: must wait for the first one's kernels
            lg2 = bk.DeviceLogits()
            s2 = torch.cuda.Stream()
            with torch.cuda.stream(s2):
                gm.forward_prefill(rng.integers(0, d.vocab, (3, 9)).tolist(), states[3], lg2, sync=False)
        torch.cuda.synchronize()
        outs.append(first.clone())
    assert torch.equal(outs[0], outs[1])
    cap = gm.query_prefill_capacity(128)
    assert cap.max_batch_size > 0 and cap.reserve_vram_bytes >= (512 << 20)
