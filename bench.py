"""Benchmark of the RWKV-7 forward hot path: decode tokens/s on the 7.2B configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one decode forward of `batch` sequences (one new token each) through the whole model.
Weights are random-init N(0, 0.02) of the named architecture, generated on the device; token ids
are uniform random.  With N > 1 (torchrun, one rank per GPU) every rank runs an independent
replica on its own sequences: the path shards by batch with no data-path collective, so the
figure is weak scaling (batch per GPU fixed).  Prints ONE JSON line on rank 0.

The headline (`value`, `e2e`, `roofline`) is the 7.2B fp16 model at B=1.  The same line carries, timed in the
same run, the other workloads of the benchmark definition under their own keys: `b256` (7.2B, 256 sequences),
`b2` / `b4`, `w8a16_1p5B` (B = 1, 8, 32, 64), `w4a16_2p9B_b256`, `w4a16_7p2B` (B = 1, 2, 4), `prefill_16k` (7.2B, 16384 tokens in chunks of 128, fp32
state) and, with N > 1, `tp_prefill` (the ranks as one head-sharded group, with a parity check of that path against
the CPU oracle on a small model first).  `--only headline` skips them.  `check` compares a fixed short run's logits
with what the reference arm (`--impl reference`, run before on the same machine) left for it.
"""
import argparse
import json
import os
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np
import torch
import torch.distributed as dist

HANDOFF = os.path.join(ROOT, ".bench_handoff")     # the reference arm leaves its check logits here for the other arm
CHECK_PROMPT = [11, 4099, 65000, 7]                # fixed ids of the correctness run: a 4-token chunk ...
CHECK_NEXT = 123                                   # ... and one decode step


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", 1400.0)), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """SM clock and throttle reasons of one GPU, read through NVML every 20 ms on a host thread while a timed region
    runs (reading only; nothing is set)."""

    def __init__(self, index):
        self.rows = []
        self.stop_flag = threading.Event()
        self.max_mhz = None
        self.thread = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[index]) if vis and all(v.strip().isdigit() for v in vis.split(",")) else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None

    def _run(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                self.rows.append((nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM),
                                  nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                                  if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons")
                                  else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)))
            except Exception:
                pass
            time.sleep(0.02)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        if self.thread is None:
            return out
        self.stop_flag.set()
        self.thread.join(timeout=2)
        if not self.rows:
            return out
        clocks = sorted(r[0] for r in self.rows)
        out["sm_mhz"] = float(clocks[len(clocks) // 2])
        out["samples"] = len(clocks)
        bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
        for name, bit in bits.items():
            if any(r[1] & bit for r in self.rows):
                out["reasons"].append(name)
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


def step_flops(d, rows, heads_rows):
    """Multiply-adds x 2 of the dense products of one forward: `rows` rows through the layers, `heads_rows` through the head."""
    C, F = d.channels, d.ffn
    p_layer = 4 * C * C + 2 * C * F + 2 * C * (d.rank_w + d.rank_a + d.rank_g + d.rank_v)
    return 2.0 * (p_layer * d.layers * rows + d.vocab * C * heads_rows)


def max_over_ranks(values, world, device="cuda"):
    """Per-rank times -> the slowest rank's (what a whole-job rate must be computed from)."""
    t = torch.tensor(values, device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def whole_job_rate(world, batch_per_gpu, ms_per_step):
    """Tokens per second of all replicas together: every rank decodes batch_per_gpu tokens per step."""
    return world * batch_per_gpu / (ms_per_step * 1e-3)


def barrier(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def build_model(model, fmt_name, wkv32, dev_index, seed, tp_rank=0, tp_size=1, layers=0, vocab=0):
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic, lib as L
    d = synthetic.CONFIGS[model]
    if layers or vocab:          # reduced-depth timing aid for per-layer work; never a bench line
        d = bk.ModelDims(layers or d.layers, d.channels, d.ffn, vocab or d.vocab, d.rank_w, d.rank_a, d.rank_v, d.rank_g)
    fmt = {"f16": L.FMT_F16, "w8a16": L.FMT_W8A16, "w4a16": L.FMT_W4A16}[fmt_name]
    ident = None
    if tp_size > 1:                       # rank 0 makes the communicator id, the others receive it
        box = [bk.tp_unique_id() if tp_rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ident = box[0]
    gm = bk.ModelBackend(d, None, use_wkv32=bool(wkv32), weight_format=fmt, device=dev_index, finalize=False,
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


def cpu_baseline(model, wkv32):
    """The CPU oracle timed on this host's cores: 2 layers + lm-head of one B=1 decode token of the
    same architecture, layer time extrapolated to the full depth."""
    from oracle import oracle as orc
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic
    full = synthetic.CONFIGS[model]
    vocab = min(full.vocab, 8192)      # the table is only gathered from; the head is timed on its own
    d = bk.ModelDims(2, full.channels, full.ffn, vocab, full.rank_w, full.rank_a, full.rank_v, full.rank_g)
    ck = synthetic.make_checkpoint(d, seed=0, device="cpu")
    om = orc.Model(d.layers, d.channels, d.ffn, d.vocab, d.rank_w, d.rank_a, d.rank_v, d.rank_g)
    om.set("emb_ln0", ck["emb.weight"].numpy())
    for name, t in ck.items():
        if name in ("emb.weight", "blocks.0.ln0.weight", "blocks.0.ln0.bias"):
            continue
        om.set(name, t.numpy())
    shift, wkv, elapsed = om.new_state(1, bool(wkv32))
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
            "sample": f"2 of {full.layers} layers + lm-head rows of one B=1 decode token of {model}, extrapolated to full depth and vocab"}


def check_logits_ours(gm, d):
    """The fixed short run both arms make from a zero state: a 4-token chunk, then one decode step."""
    from rwkv_lightning_cuda_b200 import backend as bk
    st = gm.create_state(1)
    lg = bk.DeviceLogits()
    gm.forward_prefill([[t % d.vocab for t in CHECK_PROMPT]], st, lg)
    gm.forward_decode([CHECK_NEXT % d.vocab], st, lg)
    return lg.values[0].cpu().numpy()


def correctness_check(gm, d, model, wkv32):
    path = os.path.join(HANDOFF, f"ref_logits_{model}_{int(bool(wkv32))}.npy")
    mine = check_logits_ours(gm, d)
    if not os.path.exists(path):
        return {"against": None, "note": "no logits from the reference arm on this machine (run bench.py --impl reference first)",
                "finite": bool(np.isfinite(mine).all())}
    both = np.load(path)
    if both.ndim != 2 or both.shape[1:] != mine.shape:
        return {"against": None, "note": "the reference arm ran another configuration"}
    ref = both[0]
    top2 = np.sort(ref)[-2:]
    return {"against": "reference arm on this machine: same seeded checkpoint, 4-token chunk + 1 decode step from a zero state",
            "max_abs_diff": float(np.abs(mine - ref).max()), "rms_diff": float(np.sqrt(np.mean((mine - ref) ** 2))),
            "argmax_equal": bool(mine.argmax() == ref.argmax()),
            "ref_run_to_run_max_abs_diff": float(np.abs(both[0] - both[1]).max()),
            "ref_run_to_run_rms_diff": float(np.sqrt(np.mean((both[0] - both[1]) ** 2))),
            "ref_top2_margin": float(top2[1] - top2[0]), "max_abs_logit": float(np.abs(ref).max()), "tolerance": 2e-2}


def time_decode(gm, d, B, steps, warmup, world, rank, e2e=True, greedy=True):
    """Device-timed decode steps (graph replays, CUDA events on the launching stream), then the same steps through
    the host-buffer call and through the on-device greedy loop (wall clock, synchronised)."""
    from rwkv_lightning_cuda_b200 import backend as bk
    st = gm.create_state(B)
    lg = bk.DeviceLogits()
    rng = np.random.default_rng(1234 + rank)
    total = warmup + steps
    toks = torch.from_numpy(rng.integers(0, d.vocab, (2 * total + 8, B, 1)))
    stream = torch.cuda.Stream()
    out = {}
    with torch.cuda.stream(stream):
        for i in range(warmup):                                            # also makes the state non-zero
            gm._forward(toks[1 + i], st, lg, sync=False)
        barrier(world)
        launches0 = gm.kernel_launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            gm._forward(toks[1 + warmup + i], st, lg, sync=False)
        e1.record(stream)
        barrier(world)
        out["ms"] = e0.elapsed_time(e1) / steps
        out["launches"] = gm.kernel_launches() - launches0
        if e2e:   # token ids in host memory in, logits in (pinned) host memory out, synchronised every step
            out_host = torch.empty((B, d.vocab), dtype=torch.float32).pin_memory()
            for i in range(min(warmup, 3)):
                gm.forward_to_host(toks[1 + total + i], st, lg, out_host)
            barrier(world)
            t0 = time.perf_counter()
            for i in range(steps):
                gm.forward_to_host(toks[1 + total + 3 + i], st, lg, out_host)
            torch.cuda.synchronize()
            out["e2e_ms"] = (time.perf_counter() - t0) * 1e3 / steps
            del out_host
        if greedy:  # the greedy choice of the next token on the device: first ids in, chosen ids out, one call
            ids_host = torch.empty((steps, B), dtype=torch.int32).pin_memory()
            gm.decode_greedy(toks[0].reshape(-1), min(warmup, 3), st, lg)
            barrier(world)
            l0 = gm.kernel_launches()
            t0 = time.perf_counter()
            gm.decode_greedy(toks[0].reshape(-1), steps, st, lg, out_host=ids_host)
            out["greedy_ms"] = (time.perf_counter() - t0) * 1e3 / steps
            out["greedy_launches"] = gm.kernel_launches() - l0
    del st, lg
    return out


def decode_entry(d, fmt, B, wkv32, t, world, hbm_peak, tf_peak):
    """One secondary workload's figures."""
    ms = t["ms"]
    abytes, wbytes, sbytes = algorithmic_bytes(d, B, bool(wkv32), fmt)
    gbs = abytes / (ms * 1e-3) / 1e9
    tfs = step_flops(d, B, B) / (ms * 1e-3) / 1e12
    e = {"value": whole_job_rate(world, B, ms), "unit": "tok/s", "ms_per_step": ms, "batch_per_gpu": B, "gpu_launches": int(t["launches"]),
         "algorithmic_bytes_per_step": abytes, "hbm_gbs": gbs, "hbm_frac": gbs / hbm_peak, "tensor_tflops": tfs, "tensor_frac": tfs / tf_peak}
    if "e2e_ms" in t:
        e["e2e"] = {"value": whole_job_rate(world, B, t["e2e_ms"]), "unit": "tok/s", "ms_per_step": t["e2e_ms"],
                    "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * d.vocab * 4}
    if "greedy_ms" in t:
        e["e2e_greedy"] = {"value": whole_job_rate(world, B, t["greedy_ms"]), "unit": "tok/s", "ms_per_step": t["greedy_ms"],
                           "h2d_bytes_per_call": B * 8, "d2h_bytes_per_step": B * 4}
    return e


def time_prefill(gm, d, B, T, n_chunks, warmup, world, rank, same_tokens):
    from rwkv_lightning_cuda_b200 import backend as bk
    st = gm.create_state(B)
    lg = bk.DeviceLogits()
    rng = np.random.default_rng(99 if same_tokens else 99 + rank)
    toks = torch.from_numpy(rng.integers(0, d.vocab, (n_chunks, B, T)))
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(min(warmup, n_chunks)):
            gm._forward(toks[i], st, lg, sync=False)
        barrier(world)
        launches0 = gm.kernel_launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(n_chunks):
            gm._forward(toks[i], st, lg, sync=False)
        e1.record(stream)
        barrier(world)
        ms = e0.elapsed_time(e1)
        launches = gm.kernel_launches() - launches0
    del st, lg
    return ms, launches


def prefill_entry(d, B, T, n_chunks, ms, launches, prompts, gpus_sharing, tf_peak):
    tokens = prompts * n_chunks * T
    flops = step_flops(d, tokens, prompts * n_chunks)      # the head runs on each chunk's last row
    tfs = flops / (ms * 1e-3) / 1e12 / gpus_sharing
    return {"value": tokens / (ms * 1e-3), "unit": "tok/s", "tokens": tokens, "chunk": T, "ms_per_chunk": ms / n_chunks,
            "gpu_launches": int(launches), "tensor_tflops_per_gpu": tfs, "tensor_frac": tfs / tf_peak}


def tp_parity(rank, world):
    """The head-sharded path against the CPU oracle on a small model (both state precisions, tensor-core and GEMV row
    counts), run by all ranks before the tensor-parallel timing.  Returns (ok, worst fp16-state error, worst fp32-state error)."""
    from oracle import oracle as orc
    from rwkv_lightning_cuda_b200 import backend as bk
    from oracle.parity import build_pair, run_both
    from oracle.parity import FP32_STATE_REL
    dims = dict(layers=2, channels=64 * 2 * world, ffn=256 * world, vocab=64 * world, rank_w=32, rank_a=32, rank_v=16, rank_g=64)
    ok, worst = True, [0.0, 0.0]
    for wkv32 in (False, True):
        box = [bk.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        d, om, gm = build_pair(orc.FMT_F16, wkv32, dims=dims, tp_rank=rank, tp_size=world, tp_unique_id=box[0])
        for B, chunks, n_decode in ((2, (24, 7), 2), (1, (3,), 2)):
            w, ids_ok, (shift, wkv, elapsed), st = run_both(d, om, gm, wkv32, B, chunks, n_decode)
            worst[int(wkv32)] = max(worst[int(wkv32)], float(w))
            Hl = d.heads // world
            mine = wkv.astype(np.float32)[:, :, rank * Hl:(rank + 1) * Hl]
            got = st.wkv_state.cpu().numpy().astype(np.float32)
            ok = ok and ids_ok and w < (FP32_STATE_REL if wkv32 else 2e-2) and \
                bool(np.abs(got - mine).max() <= 2e-2 * max(1.0, np.abs(mine).max()))
        gm.close()
    flag = torch.tensor([0.0 if ok else 1.0, worst[0], worst[1]], device="cuda", dtype=torch.float64)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return bool(flag[0].item() == 0.0), float(flag[1].item()), float(flag[2].item())


def run_ours(args, rank, world, local_rank):
    hbm_peak, tf_peak, peak_kind = measured_peaks()
    d, gm, fmt = build_model(args.model, args.fmt, args.wkv32, local_rank, seed=rank, layers=args.layers, vocab=args.vocab)
    B = args.batch
    check = correctness_check(gm, d, args.model, args.wkv32) if (rank == 0 and fmt == 0 and not (args.layers or args.vocab)) else None
    sampler = ClockSampler(local_rank)
    t = time_decode(gm, d, B, args.steps, args.warmup, world, rank)
    clocks = sampler.stop()
    ms, e2e_ms, greedy_ms = max_over_ranks([t["ms"], t["e2e_ms"], t["greedy_ms"]], world)
    abytes, wbytes, sbytes = algorithmic_bytes(d, B, bool(args.wkv32), fmt)
    achieved = abytes / (ms * 1e-3) / 1e9
    # DRAM traffic of the dominant kernel (gemv_mma_kernel, one row of fp16) per algorithmic byte, from an ncu capture of one launch
    # (16384 x 4096 fp16): 134.27 MB read + 4.85 MB written for 134.26 MB of weights; scaled to the step
    traffic = abytes * (139.12 / 134.26) if (fmt == 0 and B == 1) else None
    line = {
        "metric": "decode_tokens_per_s", "value": whole_job_rate(world, B, ms), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16" if fmt == 0 else args.fmt, "data": "synthetic",
        "config": {"reduced": {"layers": args.layers, "vocab": args.vocab} if (args.layers or args.vocab) else None,
                   "workload": f"RWKV-7 {args.model} random-init, decode, batch {B} per GPU, {'fp32' if args.wkv32 else 'fp16'} WKV state, weights {args.fmt}",
                   "options": args.option or None,
                   "batch_per_gpu": B, "parallelism": f"replicas x{world} (batch-sharded, no collective)",
                   "l2": "inputs larger than L2 (every step streams all weights)",
                   "quantised_parity": None if fmt == 0 else "unpinned against the reference (it has no quantised weights); format and kernels checked against this repository's oracle"},
        "clocks": clocks,
        "e2e": {"value": whole_job_rate(world, B, e2e_ms), "unit": "tok/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * d.vocab * 4},
        "e2e_greedy": {"value": whole_job_rate(world, B, greedy_ms), "unit": "tok/s", "ms_per_step": greedy_ms,
                       "what": "decode steps + greedy token choice on the device, one host call for all steps",
                       "h2d_bytes_per_call": B * 8, "d2h_bytes_per_call": args.steps * B * 4, "gpu_launches": int(t["greedy_launches"])},
        "gpu_launches": int(t["launches"]),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": traffic, "peak_kind": peak_kind, "frac_of_nominal_8000": achieved / 8000.0,
                     "algorithmic_bytes_per_step": abytes, "weight_bytes": wbytes, "state_bytes_per_seq": sbytes,
                     "scope": "whole decode step (the weight-streaming linear kernel is 92 % of it)"},
        "check": check,
    }
    extras = args.only == "all" and not (args.layers or args.vocab) and args.model == "7.2B" and fmt == 0 and B == 1
    if extras:
        steps2, warm2 = max(8, args.steps // 2), 3
        # the other half of the metric: 256 sequences per GPU on the same model, fp16 state
        t256 = time_decode(gm, d, 256, steps2, warm2, world, rank)
        t256["ms"], t256["e2e_ms"], t256["greedy_ms"] = max_over_ranks([t256["ms"], t256["e2e_ms"], t256["greedy_ms"]], world)
        line["b256"] = decode_entry(d, fmt, 256, 0, t256, world, hbm_peak, tf_peak)
        if world == 1:
            for b in (2, 4):   # a few sequences: the same weight stream as one sequence
                tb = time_decode(gm, d, b, steps2, warm2, world, rank, e2e=False, greedy=False)
                line[f"b{b}"] = decode_entry(d, fmt, b, 0, tb, world, hbm_peak, tf_peak)
        gm.close()
        torch.cuda.empty_cache()
        if world == 1:
            # long prompt on one GPU: 16384 tokens in chunks of 128, fp32 state (the configuration's prefill half)
            d2, gm2, _ = build_model("7.2B", "f16", 1, local_rank, seed=0)
            ms_p, launches_p = time_prefill(gm2, d2, 1, 128, 128, 3, world, rank, same_tokens=True)
            line["prefill_16k"] = prefill_entry(d2, 1, 128, 128, ms_p, launches_p, 1, 1, tf_peak)
            gm2.close()
            torch.cuda.empty_cache()
            d3, gm3, f3 = build_model("1.5B", "w8a16", 0, local_rank, seed=0)
            sweep = {}
            for b in (1, 8, 32, 64):
                tb = time_decode(gm3, d3, b, steps2, warm2, world, rank, e2e=False, greedy=False)
                sweep[f"b{b}"] = decode_entry(d3, f3, b, 0, tb, world, hbm_peak, tf_peak)
            line["w8a16_1p5B"] = sweep
            gm3.close()
            torch.cuda.empty_cache()
            d4, gm4, f4 = build_model("2.9B", "w4a16", 0, local_rank, seed=0)
            tb = time_decode(gm4, d4, 256, steps2, warm2, world, rank, e2e=False, greedy=False)
            line["w4a16_2p9B_b256"] = decode_entry(d4, f4, 256, 0, tb, world, hbm_peak, tf_peak)
            gm4.close()
            torch.cuda.empty_cache()
            # the quantised row of the headline model: 7.2B W4A16 at 1, 2 and 4 sequences
            d5, gm5, f5 = build_model("7.2B", "w4a16", 0, local_rank, seed=0)
            sweep = {}
            for b in (1, 2, 4):
                tb = time_decode(gm5, d5, b, steps2, warm2, world, rank, e2e=False, greedy=False)
                sweep[f"b{b}"] = decode_entry(d5, f5, b, 0, tb, world, hbm_peak, tf_peak)
            line["w4a16_7p2B"] = sweep
            gm5.close()
            torch.cuda.empty_cache()
            line["quantised_parity"] = "unpinned against the reference (it has no quantised weights); format and kernels checked against this repository's oracle"
        else:
            # the one path with a collective: all ranks as ONE head-sharded group on one 2048-token prompt
            ok, w16, w32 = tp_parity(rank, world)
            d2, gm2, _ = build_model("7.2B", "f16", 1, local_rank, seed=0, tp_rank=rank, tp_size=world)
            ms_p, launches_p = time_prefill(gm2, d2, 1, 128, 16, 3, world, rank, same_tokens=True)
            (ms_p,) = max_over_ranks([ms_p], world)
            e = prefill_entry(d2, 1, 128, 16, ms_p, launches_p, 1, world, tf_peak)
            e.update({"scaling": "strong", "parallelism": f"tp{world}: heads sharded, fp32 all-reduce after att.output and ffn.value",
                      "parity_vs_oracle": {"ok": ok, "worst_logit_err_fp16_state": w16, "worst_rel_logit_err_fp32_state": w32}})
            line["tp_prefill"] = e
            gm2.close()
            torch.cuda.empty_cache()
    if rank != 0:
        return
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.model, args.wkv32)
    # bounded waits inside the kernels that ran out during any of the timed work (0 = none; bits as in the header)
    from rwkv_lightning_cuda_b200 import lib as _L
    line["timeout_flags"] = int(_L.timeout_flags(clear=True))
    print(json.dumps(line))


def run_prefill(args, rank, world, local_rank):
    """Secondary line (not the headline metric): chunked prefill of one long prompt.  With --tp the ranks form one
    head-sharded tensor-parallel group working on the same prompt (strong scaling); without it every rank prefills
    its own prompt (weak scaling)."""
    _, tf_peak, kind = measured_peaks()
    tp = world if args.tp else 1
    seed = 0 if tp > 1 else rank           # tensor-parallel ranks must draw the same checkpoint
    d, gm, fmt = build_model(args.model, args.fmt, args.wkv32, local_rank, seed, tp_rank=rank if tp > 1 else 0, tp_size=tp,
                             layers=args.layers, vocab=args.vocab)
    B, T, n_chunks = args.batch, args.chunk, args.prefill // args.chunk
    sampler = ClockSampler(local_rank)
    ms, launches = time_prefill(gm, d, B, T, n_chunks, args.warmup, world, rank, same_tokens=tp > 1)
    clocks = sampler.stop()
    (ms,) = max_over_ranks([ms], world)
    if rank != 0:
        return
    prompts = B * (1 if tp > 1 else world)
    e = prefill_entry(d, B, T, n_chunks, ms, launches, prompts, tp if tp > 1 else world, tf_peak)
    print(json.dumps({
        "metric": "prefill_tokens_per_s", "value": e["value"], "unit": "tok/s", "n_gpus": world, "steps": n_chunks,
        "warmup": min(args.warmup, n_chunks), "ms_per_step": ms / n_chunks, "higher_is_better": True,
        "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"reduced": {"layers": args.layers, "vocab": args.vocab} if (args.layers or args.vocab) else None,
                   "options": args.option or None,
                   "workload": f"RWKV-7 {args.model} random-init, prefill {n_chunks * T} tokens x {B} prompt(s) in chunks of {T}, "
                               f"{'fp32' if args.wkv32 else 'fp16'} WKV state, weights {args.fmt}",
                   "parallelism": f"tp{tp} (head-sharded, fp32 all-reduce after att.output and ffn.value)" if tp > 1 else f"replicas x{world}",
                   "l2": "inputs larger than L2 (every chunk streams all weights)"},
        "clocks": clocks, "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "achieved": e["tensor_tflops_per_gpu"], "peak": tf_peak, "unit": "TFLOP/s", "frac": e["tensor_frac"],
                     "traffic": None, "peak_kind": kind + " (sustained)", "scope": "whole prefill, per GPU"},
    }))


def write_reference_checkpoint(model, path):
    from rwkv_lightning_cuda_b200 import synthetic
    d = synthetic.CONFIGS[model]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    sd = {}
    for name, shape in synthetic.tensor_shapes(d).items():
        sd[name] = synthetic._draw(name, shape, gen, "cuda").to(torch.bfloat16).cpu().clone()
    torch.save(sd, path)
    return d


def reference_kernel_times(lib):
    """CUDA-event time of two of the reference's own kernels alone (no host work, no allocation): its one-row GEMV on
    a 16384 x 4096 fp16 matrix (cuda/rwkv7_v3a_ops.cu:464-560) and its fp16-state WKV step for 256 sequences x 64 heads
    (cuda/rwkv7_wkv_fp16_v2.cu:676-742), with the same two shapes through this repository's kernels beside them.
    Weights rotate over copies larger than L2."""
    import ctypes as C
    from rwkv_lightning_cuda_b200 import ops
    p = lambda t: C.c_void_p(t.data_ptr())
    N, K = 16384, 4096
    Ws = [torch.randn(N, K, device="cuda", dtype=torch.float16) * 0.02 for _ in range(3)]
    x = torch.randn(1, K, device="cuda", dtype=torch.float16)
    y = torch.empty(1, N, device="cuda", dtype=torch.float16)
    B, Cc, H = 256, 4096, 64
    state = torch.zeros(B, H, 64, 64, device="cuda", dtype=torch.float16)
    r, w, k, v, a, b = (torch.randn(B, Cc, device="cuda", dtype=torch.float16) * 0.1 for _ in range(6))
    yy = torch.empty(B, Cc, device="cuda", dtype=torch.float16)
    elapsed = torch.zeros(B, device="cuda", dtype=torch.int32)

    def timed(fn, reps):
        fn(0); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    lib.ref_set_sync(0)
    out = {}
    try:
        us = timed(lambda i: lib.ref_linear_orig(1, K, N, p(x), p(Ws[i % 3]), p(y), 1), 30)
        out["ref_linear_orig_1x4096x16384"] = {"us": us, "GB_per_s": N * K * 2 / us / 1e3}
        us = timed(lambda i: lib.ref_wkv_fp16_seq(B, 1, Cc, H, p(state), p(r), p(w), p(k), p(v), p(a), p(b), p(yy), p(elapsed)), 30)
        out["ref_wkv_fp16_seq_b256"] = {"us": us, "GB_per_s": 2 * state.numel() * 2 / us / 1e3}
    finally:
        lib.ref_set_sync(1)
    us = timed(lambda i: ops.linear_f16_orig(x, Ws[i % 3]), 30)
    out["ours_linear_1x4096x16384"] = {"us": us, "GB_per_s": N * K * 2 / us / 1e3}
    us = timed(lambda i: ops.wkv_fp16_seq(B, 1, H, state, r, w, k, v, a, b, elapsed), 30)
    out["ours_wkv_fp16_seq_b256"] = {"us": us, "GB_per_s": 2 * state.numel() * 2 / us / 1e3}
    out["note"] = "back-to-back eager launches on one stream, CUDA events around 30 of them"
    return out


def run_reference(args, rank, world):
    """The reference's own CUDA backend (built unmodified into oracle/_ref) on the same workload."""
    if rank != 0:
        return
    import ctypes as C
    from oracle.oracle import ref_lib
    lib = ref_lib()
    if lib is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libref_rwkv7.so was not built (reference tree absent at build time)"}))
        return
    tmpdir = tempfile.mkdtemp(prefix="rwkv7_ref_")
    path = os.path.join(tmpdir, "model.pth")
    try:
        d = write_reference_checkpoint(args.model, path)
        be = lib.ref_backend_create(path.encode(), int(args.wkv32))
    finally:
        if os.path.exists(path):
            os.unlink(path)
        os.rmdir(tmpdir)
    if not be:
        print(json.dumps({"impl": "reference", "unavailable": "reference backend failed to load: " + lib.ref_last_error().decode()}))
        return
    B = args.batch
    out = np.empty((B, d.vocab), np.float32)
    # the fixed short run whose logits the other arm compares its own with
    # (run twice: the reference's FFN down-projection for few rows adds fp16 partial sums with atomics in arbitrary
    # order, cuda/rwkv7_fast_ops_fp16.cu:618-679, so its own run-to-run difference is the floor of any comparison)
    prompt = np.array([[t % d.vocab for t in CHECK_PROMPT]], dtype=np.int64)
    nxt = np.array([[CHECK_NEXT % d.vocab]], dtype=np.int64)
    runs = []
    for _ in range(2):
        st1 = lib.ref_state_create(be, 1)
        one = np.empty((1, d.vocab), np.float32)
        lib.ref_forward(be, st1, prompt.ctypes.data_as(C.c_void_p), 1, prompt.shape[1], None)
        rc = lib.ref_forward(be, st1, nxt.ctypes.data_as(C.c_void_p), 1, 1, one.ctypes.data_as(C.c_void_p))
        lib.ref_state_destroy(st1)
        if rc == 0:
            runs.append(one[0].copy())
    if len(runs) == 2:
        os.makedirs(HANDOFF, exist_ok=True)
        np.save(os.path.join(HANDOFF, f"ref_logits_{args.model}_{int(bool(args.wkv32))}.npy"), np.stack(runs))
    st = lib.ref_state_create(be, B)
    rng = np.random.default_rng(1234)
    toks = rng.integers(0, d.vocab, (args.warmup + args.steps + 1, B)).astype(np.int64)
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
    try:
        kernels = reference_kernel_times(lib)
    except Exception as e:      # the headline of this arm does not depend on it
        kernels = {"unavailable": repr(e)[:200]}
    print(json.dumps({
        "impl": "reference", "metric": "decode_tokens_per_s", "value": v, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"RWKV-7 {args.model} random-init, decode, batch {B} per GPU, {'fp32' if args.wkv32 else 'fp16'} WKV state, weights f16",
                   "note": "the reference's own CUDA ModelBackend (it has no CPU implementation of this path), host token ids in, logits copied to host; wall clock including its per-call allocation and synchronisation"},
        "clocks": clocks,
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": 1, "kind": "reference", "sample": f"{args.steps} decode steps of the reference CUDA backend driven by one host thread"},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": B * d.channels * 2, "d2h_bytes_per_step": B * d.vocab * 4,
                "note": "the reference gathers embedding rows on the host and copies them in; its logits are copied back every step"},
        "kernel_only": kernels,
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
    ap.add_argument("--only", default="all", choices=["all", "headline"], help="headline: skip the secondary workloads of the line")
    ap.add_argument("--prefill", type=int, default=0, help="secondary line: prefill this many tokens in chunks instead of decoding")
    ap.add_argument("--chunk", type=int, default=128)
    ap.add_argument("--layers", type=int, default=0, help="timing aid: override the depth (the line then says so)")
    ap.add_argument("--vocab", type=int, default=0, help="timing aid: override the vocabulary size")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="measurement aid: a switch of rwkv7_b200_set_option (the line then lists it under config.options)")
    ap.add_argument("--tp", action="store_true", help="with --prefill: the ranks form one head-sharded tensor-parallel group")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.option:
        from rwkv_lightning_cuda_b200 import lib as _L
        for item in args.option:
            name, _, value = item.partition("=")
            _L.set_option(name, int(value))
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
