"""One rank of the 2-GPU tensor-parallel parity check; launched by tests/test_tp_gpu.py through
``python -m torch.distributed.run``.  Every rank builds the head-sharded model from the same seeded
checkpoint, runs the same prefill chunks and decode steps, and compares the gathered logits and its own
slice of the WKV state with the CPU oracle's full-model result."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

DIMS = dict(layers=3, channels=256, ffn=1024, vocab=512, rank_w=32, rank_a=32, rank_v=16, rank_g=64)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")         # host channel for the communicator id only
    from oracle import oracle as orc
    from rwkv_lightning_cuda_b200 import backend as bk
    from oracle.parity import build_pair, run_both
    from oracle.parity import FP32_STATE_REL

    for wkv32 in (False, True):
        d, om, gm = build_pair(orc.FMT_F16, wkv32, dims=DIMS, tp_rank=rank, tp_size=world,
                               tp_unique_id=_fresh_id(rank))
        for B, chunks, n_decode in ((2, (24, 7), 3), (1, (3,), 4)):     # tensor-core rows, then GEMV rows
            worst, ids_ok, (shift, wkv, elapsed), st = run_both(d, om, gm, wkv32, B, chunks, n_decode)
            print(f"[parity] tensor-parallel rank {rank}/{world} wkv32={wkv32} B={B} chunks={chunks}: "
                  f"worst logit err {worst:.3e}", flush=True)
            assert worst < (FP32_STATE_REL if wkv32 else 2e-2), worst
            assert ids_ok
            Hl = d.heads // world
            mine = wkv.astype(np.float32)[:, :, rank * Hl:(rank + 1) * Hl]
            got = st.wkv_state.cpu().numpy().astype(np.float32)
            assert got.shape == mine.shape
            assert np.abs(got - mine).max() <= 2e-2 * max(1.0, np.abs(mine).max())
            assert np.abs(st.shift.cpu().numpy().astype(np.float32) - shift.astype(np.float32)).max() < 2e-2
            assert (st.elapsed.cpu().numpy() == elapsed).all()
        gm.close()
    dist.barrier()
    dist.destroy_process_group()


def _fresh_id(rank):
    from rwkv_lightning_cuda_b200 import backend as bk
    ident = [bk.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ident, src=0)
    return ident[0]


if __name__ == "__main__":
    main()
