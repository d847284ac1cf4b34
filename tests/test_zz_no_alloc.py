"""The allocation-free linear entry point (collected last on purpose: if it fails under `-x`, every
other test has already run).

Some hosts of this library cannot allocate device memory around a forward call: an inference server
whose memory budget is fixed once the model is resident, or a plugin host that forbids cudaMalloc
inside its callbacks.  `rwkv7_b200_linear_f16_orig_static` serves them: the split-K partial sums of the
tensor-core GEMM live in a fixed device array inside the library instead of caller-provided scratch.
The test calls it through the C ABI twice in a row (the array keeps the previous call's contents, so the
second call must not be disturbed by them) and checks both results against the ordinary entry point and against
the CPU oracle, on shapes that do split K (so the array really is used) and at the largest size it accepts."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import h16, ulp_diff16

pytestmark = pytest.mark.gpu


def test_static_scratch_linear_matches_the_ordinary_entry_point_twice():
    from rwkv_lightning_cuda_b200 import lib as L, ops
    lib = L.load_library()
    rng = np.random.default_rng(42)
    # (M, K, N, must the K split be used?).  Later shapes run over the earlier ones' stale partial sums in the array;
    # the last one is the largest the entry point accepts (M*N = 2,097,152: two splits would fill the array exactly).
    shapes = ((64, 1024, 256, False), (64, 8192, 128, True), (200, 2048, 128, False), (40, 4096, 64, True), (512, 256, 4096, False))
    for M, K, N, must_split in shapes:
        xh, Wh = h16(rng.standard_normal((M, K))), h16(rng.standard_normal((N, K)) * 0.02)
        x, W = torch.from_numpy(xh).cuda(), torch.from_numpy(Wh).cuda()
        want = ops.linear_f16_orig(x, W).cpu().numpy()            # existing entry point (no scratch given: unsplit)
        exact = orc.linear_orig(xh, Wh)                           # CPU oracle
        out = torch.empty((M, N), dtype=torch.float16, device="cuda")
        for call in range(2):
            out.fill_(float("nan"))
            ops.linear_f16_orig_static(x, W, out=out)
            splits = lib.rwkv7_b200_debug_last_gemm_splits()
            assert splits > 1 or not must_split, f"{(M, K, N)}: expected the K split (and so the built-in array) to be used"
            got = out.cpu().numpy()
            # next to zero an fp16 ulp is far smaller than the rounding error of an fp32 sum over K products taken in
            # another order (the K split), so differences below that error never count for more than one ulp
            atol = 1e-5 * (K / 1024) ** 0.5 * 4
            for ref, name in ((want, "ordinary entry point"), (exact, "oracle")):
                d = ulp_diff16(got, ref)
                d = np.where(np.abs(got.astype(np.float32) - ref.astype(np.float32)) <= atol, np.minimum(d, 1), d)
                assert d.max() <= 2, f"{(M, K, N)} call {call} vs {name}: max ulp {d.max()}"      # the tolerance of the other tensor-path tests
                assert (d == 0).mean() >= (0.95 if must_split else 0.97)      # 32 partial sums added in split order round a few more results the other way
    # sizes beyond the built-in scratch are refused with a clear error, not truncated
    x = torch.zeros((4096, 64), dtype=torch.float16, device="cuda")
    W = torch.zeros((1024, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(L.Rwkv7B200Error, match="exceeds the built-in scratch"):
        ops.linear_f16_orig_static(x, W)
    with pytest.raises(L.Rwkv7B200Error):
        ops.linear_f16_orig_static(x[:2], W)                      # the weight-streaming path (rows <= 4) needs no scratch at all
