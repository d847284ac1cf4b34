"""Single-kernel timings of the library's operators on the current GPU.

    python -m rwkv_lightning_cuda_b200.microbench linear --fmt w4 --n 16384 --k 4096 --m 1
    python -m rwkv_lightning_cuda_b200.microbench wkv --tokens 128 --heads 64
    python -m rwkv_lightning_cuda_b200.microbench linear --fmt f16 --n 16384 --k 4096 --m 1 --launches 3   # for a profiler

`linear`: y = x W^T through the C-ABI entry points (fp16 / W8A16 / W4A16), weights drawn at random, rotating over
enough copies of W to exceed the L2 cache; the calls are captured into one CUDA graph and the replay is timed with
CUDA events, so the figure is the kernel (plus its hand-over to the next launch), not the host's launch rate.
`--launches N` instead issues N plain launches and exits (a small, fixed workload to capture with a profiler).
`wkv`: the fp32-state WKV-7 over a chunk of tokens, matrix form against the per-token scan.
"""
import argparse
import json

import numpy as np
import torch

from . import lib as L, ops

L2_BYTES = 126 << 20


def _weights(fmt, n, k, gen):
    if fmt == "f16":
        return ((torch.randn(n, k, device="cuda", generator=gen) * 0.02).half(),)
    if fmt == "w8":
        return (torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8, generator=gen),
                (torch.rand(n, device="cuda", generator=gen) * 0.01).half())
    return (torch.randint(0, 256, (n, k // 2), device="cuda", dtype=torch.uint8, generator=gen),
            (torch.rand(n, k // 128, device="cuda", generator=gen) * 0.01).half(),
            torch.randint(0, 16, (n, k // 128), device="cuda", generator=gen).half())


def _call(fmt, x, w):
    if fmt == "f16":
        return ops.linear_f16_orig(x, w[0])
    if fmt == "w8":
        return ops.linear_w8a16(x, w[0], w[1])
    return ops.linear_w4a16(x, w[0], w[1], w[2])


def linear(args):
    gen = torch.Generator(device="cuda").manual_seed(1)
    per = args.n * args.k * {"f16": 2.0, "w8": 1.0, "w4": 0.5}[args.fmt]
    copies = 1 if args.launches else max(2, int(2 * L2_BYTES / per) + 1)
    x = torch.randn(args.m, args.k, device="cuda", generator=gen).half()
    ws = [_weights(args.fmt, args.n, args.k, gen) for _ in range(copies)]
    if args.launches:
        for i in range(args.launches):
            _call(args.fmt, x, ws[0])
        torch.cuda.synchronize()
        return {"op": "linear", "launches": args.launches}
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(st):
        for i in range(3):
            _call(args.fmt, x, ws[i % copies])
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            keep = [_call(args.fmt, x, ws[i % copies]) for i in range(args.iters)]
        graph.replay()
        torch.cuda.synchronize()
        e0.record(st)
        graph.replay()
        e1.record(st)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.iters
    del keep
    return {"op": "linear", "fmt": args.fmt, "n": args.n, "k": args.k, "m": args.m, "us": round(us, 2),
            "weight_gb_per_s": round(per / us / 1e3, 1), "weight_copies": copies, "timed": "CUDA graph replay, CUDA events"}


def wkv(args):
    rng = np.random.default_rng(1)
    B, T, H = args.batch, args.tokens, args.heads
    C = H * 64

    def t(x):
        return torch.from_numpy(x.astype(np.float16)).cuda()
    # r, k, v ~ N(0,1); decay exp(-exp(x)), x ~ U(-6,-0.5), as the pre-activation the kernel consumes; kk a unit vector per
    # head, a = -kk, b = kk * sigmoid(U(-3,3))
    shape = (B * T, C)
    r, k, v = (t(rng.standard_normal(shape)) for _ in range(3))
    p = np.clip(np.exp(rng.uniform(-6.0, -0.5, shape) + 0.5), 1e-6, 1 - 1e-6)
    w = t(np.clip(np.log(p / (1 - p)), -12, 12))
    kk = rng.standard_normal((B * T, H, 64)); kk /= np.linalg.norm(kk, axis=-1, keepdims=True)
    a = t(-kk.reshape(shape))
    b = t((kk / (1 + np.exp(-rng.uniform(-3, 3, kk.shape)))).reshape(shape))
    out = {"op": "wkv_fp32", "batch": B, "tokens": T, "heads": H}
    for name, mode in (("matrix_form_us", 1), ("scan_us", 0)):
        L.set_option("wkv_chunked", mode)
        state = torch.zeros((B, H, 64, 64), dtype=torch.float32, device="cuda")
        for _ in range(3):
            ops.wkv_fp32io16(B, T, H, state, r, w, k, v, a, b)
        torch.cuda.synchronize()
        if args.launches:
            continue
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            ops.wkv_fp32io16(B, T, H, state, r, w, k, v, a, b)
        e1.record()
        torch.cuda.synchronize()
        out[name] = round(e0.elapsed_time(e1) * 1e3 / args.iters, 2)
    L.set_option("wkv_chunked", 1)
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="op", required=True)
    a = sub.add_parser("linear")
    a.add_argument("--fmt", choices=("f16", "w8", "w4"), default="f16")
    a.add_argument("--n", type=int, default=16384)
    a.add_argument("--k", type=int, default=4096)
    a.add_argument("--m", type=int, default=1)
    a.add_argument("--iters", type=int, default=40)
    a.add_argument("--launches", type=int, default=0)
    a.add_argument("--gemv-mma", type=int, default=None, help="the library's gemv_mma option (0, 1, 2)")
    a.add_argument("--option", action="append", default=[], metavar="NAME=VALUE", help="any switch of rwkv7_b200_set_option")
    b = sub.add_parser("wkv")
    b.add_argument("--batch", type=int, default=1)
    b.add_argument("--tokens", type=int, default=128)
    b.add_argument("--heads", type=int, default=64)
    b.add_argument("--iters", type=int, default=20)
    b.add_argument("--launches", type=int, default=0)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    torch.cuda.set_device(0)
    if getattr(args, "gemv_mma", None) is not None:
        L.set_option("gemv_mma", args.gemv_mma)
    for item in getattr(args, "option", []):
        name, _, value = item.partition("=")
        L.set_option(name, int(value))
    print(json.dumps(linear(args) if args.op == "linear" else wkv(args)))


if __name__ == "__main__":
    main()
