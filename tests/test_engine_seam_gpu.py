"""The drop-in seam, run: the reference's unmodified inference engine (batch_generate, batch_generate_state), sampler,
tokenizer and checkpoint reader drive a model through IModelBackend -- once the reference's own ModelBackend, once
B200ModelBackend, the adapter over this library -- in the test program oracle/_ref/engine_seam (built by
`make -C oracle engine` where the reference sources are; skipped where that build is absent).

Both runs read the same bf16 checkpoint and the same prompts (two prompts of different length: the engine's chunked
prefill then splits the batch and exercises copy_state_slice / copy_logits_slice of the backend).  Generation is the
sampler's greedy case.  The engine feeds each backend its OWN tokens, so after a near-tie the two texts may part; what
must hold: the adapter's run is deterministic, the first generated token of every prompt is the same for both backends,
and the stateful batch-1 path agrees on its first token too."""
import itertools
import os
import string
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "oracle", "_ref", "engine_seam")
DIMS = dict(layers=2, channels=768, ffn=3072, vocab=1024, rank_w=64, rank_a=64, rank_v=32, rank_g=128)


def write_vocab(path, n):
    """A vocabulary in the tokenizer's file format (index, Python literal, byte length): ids 1..26 are the letters, the
    following ids two- and three-letter strings."""
    words = list(string.ascii_lowercase)
    for k in (2, 3):
        words += ["".join(t) for t in itertools.product(string.ascii_lowercase, repeat=k)]
    with open(path, "w") as f:
        for i in range(1, n):
            f.write(f"{i} '{words[i - 1]}' {len(words[i - 1])}\n")


def run(which, pth, vocab, wkv32, prompts, max_tokens=12):
    res = subprocess.run([BINARY, which, pth, vocab, str(int(wkv32)), str(max_tokens), *prompts], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith(("out ", "state"))]
    outs = [bytes.fromhex(l.split(" ")[2]) if len(l.split(" ")) > 2 else b"" for l in lines if l.startswith("out ")]
    state = [bytes.fromhex(l.split(" ")[1]) if len(l.split(" ")) > 1 else b"" for l in lines if l.startswith("state")]
    return outs, state[0]


@pytest.mark.parametrize("wkv32", [False, True])
def test_reference_engine_runs_on_the_adapter_and_agrees_with_the_reference_backend(tmp_path, wkv32):
    if not os.path.exists(BINARY):
        pytest.skip("oracle/_ref/engine_seam is not built here")
    from rwkv_lightning_cuda_b200 import backend as bk, synthetic
    d = bk.ModelDims(**DIMS)
    ck = synthetic.make_checkpoint(d, seed=0, device="cpu", dtype=torch.bfloat16)
    pth, vocab = str(tmp_path / "m.pth"), str(tmp_path / "vocab.txt")
    torch.save({k: v.clone() for k, v in ck.items()}, pth)
    write_vocab(vocab, d.vocab)
    prompts = ["thequickbrownfoxjumpsoverthelazydog" * 3, "hello"]
    ours_a, st_a = run("b200", pth, vocab, wkv32, prompts)
    ours_b, st_b = run("b200", pth, vocab, wkv32, prompts)
    ref, st_r = run("ref", pth, vocab, wkv32, prompts)
    assert ours_a == ours_b and st_a == st_b, "the adapter's run is not deterministic"
    assert all(len(o) > 0 for o in ours_a) and len(ours_a) == len(prompts)

    def common(a, b):
        n = 0
        while n < min(len(a), len(b)) and a[n] == b[n]:
            n += 1
        return n
    prefix = [common(a, b) for a, b in zip(ours_a, ref)]
    print(f"[parity] engine through the adapter vs through the reference backend (wkv32={wkv32}): texts {[o.decode() for o in ours_a]} / "
          f"{[o.decode() for o in ref]}, common prefix lengths {prefix}")
    for a, b in zip(ours_a, ref):
        assert a[:1] == b[:1]              # the first generated token depends on the prefill alone
    assert st_a[:1] == st_r[:1]
