"""world_size-2 checks (gloo, CPU) of the benchmark's multi-rank logic: the path shards by batch with no
data-path collective, so the only cross-rank step is taking the slowest rank's time."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import bench
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ms, e2e = bench.max_over_ranks([2.0 + rank, 5.0 - rank], world, "cpu")
    out[rank] = (ms, e2e, bench.whole_job_rate(world, 4, ms))
    dist.barrier()
    dist.destroy_process_group()


def test_slowest_rank_sets_the_whole_job_rate():
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, 29531, out), nprocs=world, join=True)
        assert out[0] == out[1]
        ms, e2e, rate = out[0]
        assert ms == 3.0 and e2e == 5.0            # max over ranks of each time
        assert rate == world * 4 / 3.0e-3          # both replicas' tokens over the slowest rank's step time


def _tp_worker(rank, world, port, out):
    """Each rank evaluates its share of a (projection -> per-head op -> output projection) chain and of the FFN on
    its slice of the weights; the sum over ranks must equal the unsharded result."""
    sys.path.insert(0, ROOT)
    import numpy as np
    from rwkv_lightning_cuda_b200 import tp
    from rwkv_lightning_cuda_b200.backend import ModelDims
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    d = ModelDims(layers=1, channels=256, ffn=512, vocab=64, rank_w=8, rank_a=8, rank_v=8, rank_g=8)
    rng = np.random.default_rng(7)           # same seed on every rank: the "checkpoint"
    C, F = d.channels, d.ffn
    full = {"blocks.0.att.receptance.weight": rng.standard_normal((C, C)), "blocks.0.att.output.weight": rng.standard_normal((C, C)),
            "blocks.0.att.w2": rng.standard_normal((8, C)), "blocks.0.att.r_k": rng.standard_normal((d.heads, 64)),
            "blocks.0.att.k_k": rng.standard_normal(C), "blocks.0.ffn.key.weight": rng.standard_normal((F, C)),
            "blocks.0.ffn.value.weight": rng.standard_normal((C, F)), "head.weight": rng.standard_normal((d.vocab, C)),
            "blocks.0.ln1.weight": rng.standard_normal(C)}
    x = rng.standard_normal((3, C)); low = rng.standard_normal((3, 8))

    def chain(w):
        r = x @ w["blocks.0.att.receptance.weight"].T                     # [3, Cl]
        r = r * w["blocks.0.att.k_k"] + low @ w["blocks.0.att.w2"]        # per-channel vector and LoRA up follow the heads
        hl = w["blocks.0.att.r_k"].shape[0]
        r = (r.reshape(3, hl, 64) * w["blocks.0.att.r_k"]).reshape(3, -1)  # per-head parameter
        att = r @ w["blocks.0.att.output.weight"].T                       # partial sum over this rank's channels
        hid = np.maximum(x @ w["blocks.0.ffn.key.weight"].T, 0) ** 2
        return att, hid @ w["blocks.0.ffn.value.weight"].T, x @ w["head.weight"].T

    mine = {k: tp.take_shard(k, v, d, rank, world) for k, v in full.items()}
    assert mine["blocks.0.ln1.weight"] is full["blocks.0.ln1.weight"]     # replicated
    att, ffn, logits = chain(mine)
    att_t, ffn_t = torch.from_numpy(att.copy()), torch.from_numpy(ffn.copy())
    dist.all_reduce(att_t); dist.all_reduce(ffn_t)
    parts = [torch.zeros(3, d.vocab // world, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(logits.copy()))
    want_att, want_ffn, want_logits = chain(full)
    out[rank] = (float(np.abs(att_t.numpy() - want_att).max()), float(np.abs(ffn_t.numpy() - want_ffn).max()),
                 float(np.abs(torch.cat(parts, 1).numpy() - want_logits).max()))
    dist.barrier()
    dist.destroy_process_group()


def test_head_sharded_partial_sums_add_up():
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_tp_worker, args=(world, 29533, out), nprocs=world, join=True)
        for rank in range(world):
            assert max(out[rank]) < 1e-9, out[rank]


def test_shard_rule_partitions_every_split_tensor():
    """For every checkpoint tensor the ranks' slices are disjoint, in rank order, and together cover the split axis; tensors
    the rule does not split come back whole.  Bad rank / indivisible sizes are refused."""
    import numpy as np
    import pytest
    from rwkv_lightning_cuda_b200 import synthetic, tp
    from rwkv_lightning_cuda_b200.backend import ModelDims
    d = ModelDims(layers=2, channels=256, ffn=1024, vocab=512, rank_w=32, rank_a=32, rank_v=16, rank_g=64)
    split_names = 0
    for name, shape in synthetic.tensor_shapes(d).items():
        full = np.arange(int(np.prod(shape)), dtype=np.int64).reshape(shape)
        for world in (2, 4):
            parts = [tp.take_shard(name, full, d, r, world) for r in range(world)]
            plan = tp.shard_of(name, d, 0, world)
            if plan is None:
                assert all(p is full for p in parts), name
                continue
            split_names += world == 2
            axis = plan[0]
            assert np.array_equal(np.concatenate(parts, axis=axis), full), name
            assert all(p.shape[axis] * world == full.shape[axis] for p in parts), name
        assert tp.shard_of(name, d, 0, 1) is None
    assert split_names == 2 * 18 - 2 + 1          # 18 split tensors per layer (layer 0 has no v0 and no v2) + the head
    with pytest.raises(ValueError):
        tp.shard_of("head.weight", d, 2, 2)
    with pytest.raises(ValueError):
        tp.shard_of("head.weight", ModelDims(layers=1, channels=192, ffn=512, vocab=512), 0, 2)   # 3 heads over 2 ranks
