"""The allocation-free linear entry point (collected last on purpose: if it fails under `-x`, every
other test has already run).

Some hosts of this library cannot allocate device memory around a forward call: an inference server
whose memory budget is fixed once the model is resident, or a plugin host that forbids cudaMalloc
inside its callbacks.  `rwkv7_b200_linear_f16_orig_static` serves them: the split-K partial sums of the
tensor-core GEMM live in a fixed device array inside the library instead of caller-provided scratch.
The test calls it through the C ABI twice in a row (the array keeps the previous call's contents, so the
second call must not be disturbed by them) and checks both results against the ordinary entry point."""
import numpy as np
import pytest
import torch

from tests.helpers import h16, ulp_diff16

pytestmark = pytest.mark.gpu


def test_static_scratch_linear_matches_the_ordinary_entry_point_twice():
    from rwkv_lightning_cuda_b200 import lib as L, ops
    rng = np.random.default_rng(42)
    for M, K, N in ((64, 1024, 256), (200, 2048, 128)):        # second shape after the first: stale partial sums in the array
        x = torch.from_numpy(h16(rng.standard_normal((M, K)))).cuda()
        W = torch.from_numpy(h16(rng.standard_normal((N, K)) * 0.02)).cuda()
        want = ops.linear_f16_orig(x, W).cpu().numpy()            # existing entry point (unsplit)
        out = torch.empty((M, N), dtype=torch.float16, device="cuda")
        for call in range(2):
            out.fill_(float("nan"))
            ops.linear_f16_orig_static(x, W, out=out)
            got = out.cpu().numpy()
            d = ulp_diff16(got, want)
            d = np.where(np.abs(got.astype(np.float32) - want.astype(np.float32)) <= 1e-5, np.minimum(d, 1), d)
            assert d.max() <= 2, f"call {call}: max ulp {d.max()}"      # the tolerance of the other tensor-path tests
            assert (d == 0).mean() >= 0.97
    # sizes beyond the built-in scratch are refused with a clear error, not truncated
    x = torch.zeros((4096, 64), dtype=torch.float16, device="cuda")
    W = torch.zeros((1024, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(L.Rwkv7B200Error, match="exceeds the built-in scratch"):
        ops.linear_f16_orig_static(x, W)
    with pytest.raises(L.Rwkv7B200Error):
        ops.linear_f16_orig_static(x[:2], W)                      # the weight-streaming path (rows <= 4) needs no scratch at all
