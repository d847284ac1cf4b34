"""Seeded random-init RWKV-7 ("x070") checkpoints with the tensor names and shapes the
reference loader expects (src/rwkv7_fast_v4.cu:574-596), for tests and benchmarks.

Matrices, LoRA factors and the embedding are N(0, 0.02); LayerNorm / GroupNorm weights are
1 + N(0, 0.02) with N(0, 0.02) biases (all-N(0, 0.02) norm weights would collapse the
activations); token-shift coefficients and k_a are U(0, 1); k_k is U(0.5, 1.5); the decay bias
w0 is U(-6, 2); a0, v0 are N(0, 1); r_k is N(0, 0.1).  Values are drawn in fp32, rounded to
bf16 (the checkpoint dtype) and then to fp16 exactly as the reference's loader does.
"""
from __future__ import annotations

from typing import Dict

import torch

from .backend import ModelDims

# the configurations named by the benchmark definition
CONFIGS = {
    "0.1B": ModelDims(12, 768, 3072, 65536, 64, 64, 32, 128),
    "1.5B": ModelDims(24, 2048, 8192, 65536, 96, 96, 64, 256),
    "2.9B": ModelDims(32, 2560, 10240, 65536, 96, 96, 64, 320),
    "7.2B": ModelDims(32, 4096, 16384, 65536, 128, 128, 96, 480),
}


def tensor_shapes(d: ModelDims) -> Dict[str, tuple]:
    C, F, V, H = d.channels, d.ffn, d.vocab, d.heads
    shapes = {"emb.weight": (V, C), "blocks.0.ln0.weight": (C,), "blocks.0.ln0.bias": (C,),
              "ln_out.weight": (C,), "ln_out.bias": (C,), "head.weight": (V, C)}
    for i in range(d.layers):
        p = f"blocks.{i}."
        for n in ("ln1.weight", "ln1.bias", "ln2.weight", "ln2.bias", "att.x_r", "att.x_w", "att.x_k", "att.x_v",
                  "att.x_a", "att.x_g", "att.w0", "att.a0", "att.k_k", "att.k_a", "att.ln_x.weight", "att.ln_x.bias", "ffn.x_k"):
            shapes[p + n] = (C,)
        shapes[p + "att.r_k"] = (H, 64)
        for n in ("receptance", "key", "value", "output"):
            shapes[p + f"att.{n}.weight"] = (C, C)
        shapes[p + "att.w1"] = (C, d.rank_w); shapes[p + "att.w2"] = (d.rank_w, C)
        shapes[p + "att.a1"] = (C, d.rank_a); shapes[p + "att.a2"] = (d.rank_a, C)
        shapes[p + "att.g1"] = (C, d.rank_g); shapes[p + "att.g2"] = (d.rank_g, C)
        if i > 0:
            shapes[p + "att.v0"] = (C,)
            shapes[p + "att.v1"] = (C, d.rank_v); shapes[p + "att.v2"] = (d.rank_v, C)
        shapes[p + "ffn.key.weight"] = (F, C)
        shapes[p + "ffn.value.weight"] = (C, F)
    return shapes


def _draw(name: str, shape, gen: torch.Generator, device) -> torch.Tensor:
    def normal(std, mean=0.0):
        return torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std + mean

    def uniform(lo, hi):
        return torch.rand(shape, generator=gen, device=device, dtype=torch.float32) * (hi - lo) + lo

    leaf = name.split(".", 2)[-1] if name.startswith("blocks.") else name
    if leaf.endswith("ln_x.weight") or (leaf.endswith(".weight") and (leaf.startswith("ln") or name.startswith("ln_out"))):
        return normal(0.02, 1.0)
    if leaf.endswith(".bias"):
        return normal(0.02)
    if leaf in ("att.x_r", "att.x_w", "att.x_k", "att.x_v", "att.x_a", "att.x_g", "ffn.x_k", "att.k_a"):
        return uniform(0.0, 1.0)
    if leaf == "att.k_k":
        return uniform(0.5, 1.5)
    if leaf == "att.w0":
        return uniform(-6.0, 2.0)
    if leaf in ("att.a0", "att.v0"):
        return normal(1.0)
    if leaf == "att.r_k":
        return normal(0.1)
    return normal(0.02)


def make_checkpoint(d: ModelDims, seed: int = 0, device="cpu", dtype=torch.float16) -> Dict[str, torch.Tensor]:
    """Returns name -> tensor.  dtype float16 gives half_rn(float(bf16(value))) -- the canonical
    device value of a bf16 checkpoint; dtype bfloat16 gives the checkpoint values themselves."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(d).items():
        t = _draw(name, shape, gen, device).to(torch.bfloat16)
        out[name] = t if dtype == torch.bfloat16 else t.to(torch.float32).to(torch.float16)
    return out
