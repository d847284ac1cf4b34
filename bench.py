"""Benchmark of the RWKV-7 forward hot path: decode tokens/s on the 7.2B configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model 7.2B] [--batch 1]

One step = one decode forward of `batch` sequences (one new token each) through the whole model.
Weights are random-init N(0, 0.02) of the named architecture, generated on the device; token ids
are uniform random.  With N > 1 (torchrun, one rank per GPU) every rank runs an independent
replica on its own sequences: the path shards by batch with no data-path collective, so the
figure is weak scaling (batch per GPU fixed).  Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np
import torch
import torch.distributed as dist


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        rows = [l.strip().split(", ") for l in open(self.f.name) if l.strip()]
        os.unlink(self.f.name)
        rows = [r for r in rows if len(r) >= 9]
        if not rows:
            return out
        sm = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        out["sm_mhz"] = statistics.median(sm) if sm else None
        out["sm_max_mhz"] = float(rows[0][2]) if rows[0][2].replace(".", "").isdigit() else None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for i, n in enumerate(names):
            if any(r[5 + i].strip() == "Active" for r in rows):
                out["reasons"].append(n)
        out["samples"] = len(rows)
        return out


def algorithmic_bytes(d, B, wkv32, fmt):
    """Bytes one decode step must move: every weight once, the recurrent state read + written per
    sequence, the embedding rows and the fp32 logits.  Dense weight counts (no sparsity discount)."""
    C, F, V, L = d.channels, d.ffn, d.vocab, d.layers
    big_layer = 4 * C * C + 2 * C * F
    lora = 2 * C * (d.rank_w + d.rank_a + d.rank_g)
    vec = 20 * C
    small = L * (lora + vec) + (L - 1) * 2 * C * d.rank_v + 2 * C
    big = L * big_layer + V * C
    if fmt == 0:
        wbytes = 2 * big
    elif fmt == 1:
        wbytes = big + 2 * (L * (4 * C + F + C) + V)
    else:
        wbytes = big // 2 + 4 * (big // 128)
    wbytes += 2 * small
    state = 2 * L * (C // 64) * 64 * 64 * (4 if wkv32 else 2) + 2 * L * 2 * C * 2
    act = V * 4 + C * 2
    return wbytes + B * (state + act), wbytes, state


def max_over_ranks(values, world, device):
    """Per-rank step times -> the slowest rank's (what a whole-job rate must be computed from)."""
    t = torch.tensor(values, device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def whole_job_rate(world, batch_per_gpu, ms_per_step):
    """Tokens per second of all replicas together: every rank decodes batch_per_gpu tokens per step."""
    return world * batch_per_gpu / (ms_per_step * 1e-3)


def build_model(args, dev_index, seed, tp_rank=0, tp_size=1):
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic, lib as L
    d = synthetic.CONFIGS[args.model]
    if args.layers or args.vocab:          # reduced-depth timing aid for per-layer work; never a bench line
        d = bk.ModelDims(args.layers or d.layers, d.channels, d.ffn, args.vocab or d.vocab, d.rank_w, d.rank_a, d.rank_v, d.rank_g)
    fmt = {"f16": L.FMT_F16, "w8a16": L.FMT_W8A16, "w4a16": L.FMT_W4A16}[args.fmt]
    ident = None
    if tp_size > 1:                       # rank 0 makes the communicator id, the others receive it
        box = [bk.tp_unique_id() if tp_rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ident = box[0]
    gm = bk.ModelBackend(d, None, use_wkv32=bool(args.wkv32), weight_format=fmt, device=dev_index, finalize=False,
                         tp_rank=tp_rank, tp_size=tp_size, tp_unique_id=ident)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    for name, shape in synthetic.tensor_shapes(d).items():
        t = synthetic._draw(name, shape, gen, "cuda").to(torch.bfloat16)
        gm.set_tensor(name, t)
        del t
    gm.finalize()
    torch.cuda.empty_cache()
    return d, gm, fmt


def cpu_baseline(args):
    """The CPU oracle timed on this host's cores: 2 layers + lm-head of one B=1 decode token of the
    same architecture, layer time extrapolated to the full depth."""
    from oracle import oracle as orc
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic
    full = synthetic.CONFIGS[args.model]
    vocab = min(full.vocab, 8192)      # the table is only gathered from; the head is timed on its own
    d = bk.ModelDims(2, full.channels, full.ffn, vocab, full.rank_w, full.rank_a, full.rank_v, full.rank_g)
    ck = synthetic.make_checkpoint(d, seed=0, device="cpu")
    om = orc.Model(d.layers, d.channels, d.ffn, d.vocab, d.rank_w, d.rank_a, d.rank_v, d.rank_g)
    om.set("emb_ln0", ck["emb.weight"].numpy())
    for name, t in ck.items():
        if name in ("emb.weight", "blocks.0.ln0.weight", "blocks.0.ln0.bias"):
            continue
        om.set(name, t.numpy())
    shift, wkv, elapsed = om.new_state(1, bool(args.wkv32))
    om.forward(np.array([[1]]), shift, wkv, elapsed)
    t0 = time.perf_counter(); reps = 2
    for i in range(reps):
        om.forward(np.array([[2 + i]]), shift, wkv, elapsed)
    t_small = (time.perf_counter() - t0) / reps
    x = ck["ln_out.weight"].numpy().reshape(1, -1)
    t0 = time.perf_counter()
    orc.linear_orig(x, ck["head.weight"].numpy())
    t_head_small = time.perf_counter() - t0
    per_layer = (t_small - t_head_small) / 2
    t_token = per_layer * full.layers + t_head_small * (full.vocab / vocab)
    cores = os.cpu_count() or 1
    return {"value": 1.0 / t_token, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"2 of {full.layers} layers + lm-head rows of one B=1 decode token of {args.model}, extrapolated to full depth and vocab"}


def run_ours(args, rank, world, local_rank):
    from rwkv_lightning_cuda_b200 import backend as bk
    hbm_peak, peak_kind = measured_peaks()
    d, gm, fmt = build_model(args, local_rank, seed=rank)
    B = args.batch
    st = gm.create_state(B)
    lg = bk.DeviceLogits()
    rng = np.random.default_rng(1234 + rank)
    total = args.warmup + args.steps
    toks = torch.from_numpy(rng.integers(0, d.vocab, (2 * total + 8, B, 1)))
    stream = torch.cuda.Stream()
    out_host = torch.empty((B, d.vocab), dtype=torch.float32).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for i in range(args.warmup):                                            # also makes the state non-zero
            gm._forward(toks[1 + i], st, lg, sync=False)
        barrier()
        sampler = ClockSampler(local_rank)
        launches0 = gm.kernel_launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(args.steps):
            gm._forward(toks[1 + args.warmup + i], st, lg, sync=False)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1) / args.steps
        launches = gm.kernel_launches() - launches0
        # end to end through the host-buffer call: token ids in host memory in, logits in host memory out
        for i in range(min(args.warmup, 3)):
            gm.forward_to_host(toks[1 + total + i], st, lg, out_host)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            gm.forward_to_host(toks[1 + total + 3 + i], st, lg, out_host)
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        # the same steps with the greedy choice of the next token on the device: first ids in, chosen ids out, one call
        ids_host = torch.empty((args.steps, B), dtype=torch.int32).pin_memory()
        gm.decode_greedy(toks[0].reshape(-1), min(args.warmup, 3), st, lg)
        barrier()
        launches_g0 = gm.kernel_launches()
        t0 = time.perf_counter()
        gm.decode_greedy(toks[0].reshape(-1), args.steps, st, lg, out_host=ids_host)
        greedy_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        launches_g = gm.kernel_launches() - launches_g0
        clocks = sampler.stop()

    ms, e2e_ms, greedy_ms = max_over_ranks([ms, e2e_ms, greedy_ms], world, "cuda")
    if rank != 0:
        return
    abytes, wbytes, sbytes = algorithmic_bytes(d, B, bool(args.wkv32), fmt)
    achieved = abytes / (ms * 1e-3) / 1e9
    # DRAM traffic of the dominant kernel (gemv_tma_kernel) per algorithmic byte, from the ncu capture summarised in
    # profiles/gemv_tma_16384x4096_ncu_full.md: 134.28 MB read + 3.58 MB written for 134.26 MB; scaled to the step
    traffic = abytes * (137.86 / 134.26) if (fmt == 0 and B == 1) else None
    line = {
        "metric": "decode_tokens_per_s", "value": whole_job_rate(world, B, ms), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16" if fmt == 0 else args.fmt, "data": "synthetic",
        "config": {"reduced": {"layers": args.layers, "vocab": args.vocab} if (args.layers or args.vocab) else None,
                   "workload": f"RWKV-7 {args.model} random-init, decode, batch {B} per GPU, {'fp32' if args.wkv32 else 'fp16'} WKV state, weights {args.fmt}",
                   "batch_per_gpu": B, "parallelism": f"replicas x{world} (batch-sharded, no collective)",
                   "l2": "inputs larger than L2 (every step streams all weights)"},
        "clocks": clocks,
        "e2e": {"value": whole_job_rate(world, B, e2e_ms), "unit": "tok/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * d.vocab * 4},
        "e2e_greedy": {"value": whole_job_rate(world, B, greedy_ms), "unit": "tok/s", "ms_per_step": greedy_ms,
                       "what": "decode steps + greedy token choice on the device, one host call for all steps",
                       "h2d_bytes_per_call": B * 8, "d2h_bytes_per_call": args.steps * B * 4, "gpu_launches": int(launches_g)},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": traffic, "peak_kind": peak_kind, "frac_of_nominal_8000": achieved / 8000.0,
                     "algorithmic_bytes_per_step": abytes, "weight_bytes": wbytes, "state_bytes_per_seq": sbytes,
                     "scope": "whole decode step (weight-streaming GEMV kernels dominate)"},
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args)
    print(json.dumps(line))


def run_prefill(args, rank, world, local_rank):
    """Secondary line (not the headline metric): chunked prefill of one long prompt.  With --tp the ranks form one
    head-sharded tensor-parallel group working on the same prompt (strong scaling); without it every rank prefills
    its own prompt (weak scaling)."""
    from rwkv_lightning_cuda_b200 import backend as bk
    tp = world if args.tp else 1
    seed = 0 if tp > 1 else rank           # tensor-parallel ranks must draw the same checkpoint
    d, gm, fmt = build_model(args, local_rank, seed, tp_rank=rank if tp > 1 else 0, tp_size=tp)
    B, T, n_chunks = args.batch, args.chunk, args.prefill // args.chunk
    st = gm.create_state(B)
    lg = bk.DeviceLogits()
    rng = np.random.default_rng(99 if tp > 1 else 99 + rank)
    toks = torch.from_numpy(rng.integers(0, d.vocab, (n_chunks, B, T)))
    stream = torch.cuda.Stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for i in range(min(args.warmup, n_chunks)):
            gm._forward(toks[i], st, lg, sync=False)
        barrier()
        sampler = ClockSampler(local_rank)
        launches0 = gm.kernel_launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(n_chunks):
            gm._forward(toks[i], st, lg, sync=False)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        launches = gm.kernel_launches() - launches0
        clocks = sampler.stop()
    (ms,) = max_over_ranks([ms], world, "cuda")
    if rank != 0:
        return
    prompts = B * (1 if tp > 1 else world)
    tokens = prompts * n_chunks * T
    C, F, L_ = d.channels, d.ffn, d.layers
    p_layer = 4 * C * C + 2 * C * F + 2 * C * (d.rank_w + d.rank_a + d.rank_g + d.rank_v)
    flops = 2.0 * (p_layer * L_ * tokens + d.vocab * C * prompts * n_chunks)      # the head runs on each chunk's last row
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            tf_peak, kind = float(json.load(fh)["bf16_tflops_sustained"]), "measured (sustained)"
    except Exception:
        tf_peak, kind = 1400.0, "fallback"
    achieved = flops / (ms * 1e-3) / 1e12 / world
    print(json.dumps({
        "metric": "prefill_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": n_chunks,
        "warmup": min(args.warmup, n_chunks), "ms_per_step": ms / n_chunks, "higher_is_better": True,
        "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"reduced": {"layers": args.layers, "vocab": args.vocab} if (args.layers or args.vocab) else None,
                   "workload": f"RWKV-7 {args.model} random-init, prefill {n_chunks * T} tokens x {B} prompt(s) in chunks of {T}, "
                               f"{'fp32' if args.wkv32 else 'fp16'} WKV state, weights {args.fmt}",
                   "parallelism": f"tp{tp} (head-sharded, fp32 all-reduce after att.output and ffn.value)" if tp > 1 else f"replicas x{world}",
                   "l2": "inputs larger than L2 (every chunk streams all weights)"},
        "clocks": clocks, "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf_peak, "unit": "TFLOP/s", "frac": achieved / tf_peak,
                     "traffic": None, "peak_kind": kind, "scope": "whole prefill, per GPU"},
    }))


def micro_gemv(args):
    """Isolated GEMV timing (not the benchmark line): y = x W^T for the 7.2B layer shapes on rotating weight
    copies larger than L2, replayed from a CUDA graph so that launches are back to back.  `--micro gemv-small`
    runs a handful of eager launches of the 16384x4096 case only (the command the ncu captures use)."""
    from rwkv_lightning_cuda_b200 import ops
    if args.micro.startswith("gemm"):
        return micro_gemm(args)
    small = args.micro == "gemv-small"
    shapes = [(16384, 4096)] if small else [(4096, 4096), (13120, 4096), (16384, 4096), (4096, 16384), (65536, 4096)]
    for N, K in shapes:
        copies = max(2, min(6, int(2e9 // (N * K * 2))))
        Ws = [torch.randn(N, K, device="cuda", dtype=torch.float16) * 0.02 for _ in range(copies)]
        x = torch.randn(1, K, device="cuda", dtype=torch.float16)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            for W in Ws:
                ops.linear_f16_orig(x, W)
            torch.cuda.synchronize()
            if small:
                for i in range(4):
                    ops.linear_f16_orig(x, Ws[i % copies])
                torch.cuda.synchronize()
                print(json.dumps({"micro": "gemv-small", "N": N, "K": K, "launches": copies + 4}))
                continue
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                for _ in range(4):
                    for W in Ws:
                        ops.linear_f16_orig(x, W)
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            for _ in range(5):
                g.replay()
            e1.record(s)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (5 * 4 * copies)
        print(json.dumps({"micro": "gemv", "N": N, "K": K, "us_per_launch": us, "GB_per_s": N * K * 2 / us / 1e3}))


def micro_gemm(args):
    """Isolated tensor-core GEMM timing: y[M,N] = x[M,K] W[N,K]^T for batched-decode / prefill shapes of the 7.2B
    model, graph-replayed on rotating weights.  `--micro gemm-small` runs a few eager launches of two shapes."""
    from rwkv_lightning_cuda_b200 import ops
    small = args.micro == "gemm-small"
    shapes = [(256, 4096, 16384), (128, 4096, 16384)] if small else \
        [(256, 128, 4096), (256, 4096, 128), (256, 4096, 4096), (256, 4096, 16384), (256, 16384, 4096), (128, 4096, 4096), (2048, 4096, 4096)]
    for M, K, N in shapes:
        copies = max(2, min(6, int(1e9 // (N * K * 2))))
        Ws = [torch.randn(N, K, device="cuda", dtype=torch.float16) * 0.02 for _ in range(copies)]
        x = torch.randn(M, K, device="cuda", dtype=torch.float16)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            for W in Ws:
                ops.linear_f16_orig(x, W)
            torch.cuda.synchronize()
            if small:
                continue
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                for _ in range(4):
                    for W in Ws:
                        ops.linear_f16_orig(x, W)
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            for _ in range(5):
                g.replay()
            e1.record(s)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (5 * 4 * copies)
        print(json.dumps({"micro": "gemm", "M": M, "K": K, "N": N, "us_per_launch": us, "TFLOP_per_s": 2.0 * M * N * K / us / 1e6,
                          "weight_GB_per_s": N * K * 2 / us / 1e3}))
    if small:
        print(json.dumps({"micro": "gemm-small", "shapes": shapes}))


def write_reference_checkpoint(args, path):
    from rwkv_lightning_cuda_b200 import synthetic
    d = synthetic.CONFIGS[args.model]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    sd = {}
    for name, shape in synthetic.tensor_shapes(d).items():
        sd[name] = synthetic._draw(name, shape, gen, "cuda").to(torch.bfloat16).cpu().clone()
    torch.save(sd, path)
    return d


def run_reference(args, rank, world):
    """The reference's own CUDA backend (built unmodified into oracle/_ref) on the same workload."""
    if rank != 0:
        return
    import ctypes as C
    from tests.helpers import ref_lib
    lib = ref_lib()
    if lib is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libref_rwkv7.so was not built (reference tree absent at build time)"}))
        return
    tmpdir = tempfile.mkdtemp(prefix="rwkv7_ref_")
    path = os.path.join(tmpdir, "model.pth")
    try:
        d = write_reference_checkpoint(args, path)
        be = lib.ref_backend_create(path.encode(), int(args.wkv32))
    finally:
        if os.path.exists(path):
            os.unlink(path)
        os.rmdir(tmpdir)
    if not be:
        print(json.dumps({"impl": "reference", "unavailable": "reference backend failed to load: " + lib.ref_last_error().decode()}))
        return
    B = args.batch
    st = lib.ref_state_create(be, B)
    rng = np.random.default_rng(1234)
    toks = rng.integers(0, d.vocab, (args.warmup + args.steps + 1, B)).astype(np.int64)
    out = np.empty((B, d.vocab), np.float32)
    prompt = np.ascontiguousarray(np.repeat(toks[0][:, None], 4, axis=1))
    lib.ref_forward(be, st, prompt.ctypes.data_as(C.c_void_p), B, 4, None)
    for i in range(args.warmup):
        lib.ref_forward(be, st, toks[1 + i].ctypes.data_as(C.c_void_p), B, 1, out.ctypes.data_as(C.c_void_p))
    sampler = ClockSampler(0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        rc = lib.ref_forward(be, st, toks[1 + args.warmup + i].ctypes.data_as(C.c_void_p), B, 1, out.ctypes.data_as(C.c_void_p))
        assert rc == 0, lib.ref_last_error()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop()
    v = B / (ms * 1e-3)
    print(json.dumps({
        "impl": "reference", "metric": "decode_tokens_per_s", "value": v, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"RWKV-7 {args.model} random-init, decode, batch {B}, {'fp32' if args.wkv32 else 'fp16'} WKV state, weights f16",
                   "note": "the reference's own CUDA ModelBackend (it has no CPU implementation of this path), host token ids in, logits copied to host; wall clock including its per-call allocation and synchronisation"},
        "clocks": clocks,
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": 1, "kind": "reference", "sample": f"{args.steps} decode steps of the reference CUDA backend driven by one host thread"},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="7.2B")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--fmt", default="f16", choices=["f16", "w8a16", "w4a16"])
    ap.add_argument("--wkv32", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prefill", type=int, default=0, help="secondary line: prefill this many tokens in chunks instead of decoding")
    ap.add_argument("--chunk", type=int, default=128)
    ap.add_argument("--layers", type=int, default=0, help="timing aid: override the depth (the line then says so)")
    ap.add_argument("--vocab", type=int, default=0, help="timing aid: override the vocabulary size")
    ap.add_argument("--tp", action="store_true", help="with --prefill: the ranks form one head-sharded tensor-parallel group")
    ap.add_argument("--micro", default="", choices=["", "gemv", "gemv-small", "gemm", "gemm-small"], help="kernel micro-benchmark instead of the bench line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if args.micro:
        micro_gemv(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.prefill:
            run_prefill(args, rank, world, local_rank)
        else:
            run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
