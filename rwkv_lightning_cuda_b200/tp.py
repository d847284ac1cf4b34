"""Which part of each checkpoint tensor a tensor-parallel rank keeps.

The library slices the full tensors itself (``rwkv7_b200_model_set_tensor`` on a model created with
``tp_size`` > 1); this module states the same rule in Python so that loaders can read only their share from
disk and tests can check the decomposition.  Rank ``g`` of ``G`` owns heads ``[g*H/G, (g+1)*H/G)``, ffn
hidden units ``[g*F/G, ...)`` and vocabulary rows ``[g*V/G, ...)``.
"""
from __future__ import annotations

from typing import Optional, Tuple

# tensor leaf name -> (axis that is split, which extent it follows); everything else is replicated
_SPLIT = {
    "att.receptance.weight": (0, "C"), "att.key.weight": (0, "C"), "att.value.weight": (0, "C"),
    "att.output.weight": (1, "C"),
    "att.w2": (1, "C"), "att.a2": (1, "C"), "att.g2": (1, "C"), "att.v2": (1, "C"),
    "att.w0": (0, "C"), "att.a0": (0, "C"), "att.v0": (0, "C"), "att.k_k": (0, "C"), "att.k_a": (0, "C"),
    "att.r_k": (0, "H"), "att.ln_x.weight": (0, "C"), "att.ln_x.bias": (0, "C"),
    "ffn.key.weight": (0, "F"), "ffn.value.weight": (1, "F"),
}


def shard_of(name: str, dims, rank: int, size: int) -> Optional[Tuple[int, int, int]]:
    """Returns (axis, lo, hi) of the slice rank ``rank`` keeps of tensor ``name``, or None if it is replicated."""
    if size <= 1:
        return None
    if not 0 <= rank < size:
        raise ValueError(f"rank {rank} outside [0, {size})")
    if dims.heads % size or dims.ffn % size or dims.vocab % size:
        raise ValueError("heads, ffn and vocab must divide by the number of ranks")
    extent = {"C": dims.channels, "H": dims.heads, "F": dims.ffn, "V": dims.vocab}
    if name == "head.weight":
        axis, which = 0, "V"
    else:
        leaf = name.split(".", 2)[-1] if name.startswith("blocks.") else name
        if leaf not in _SPLIT:
            return None
        axis, which = _SPLIT[leaf]
    n = extent[which] // size
    return axis, rank * n, (rank + 1) * n


def take_shard(name: str, tensor, dims, rank: int, size: int):
    """The slice of ``tensor`` (anything indexable like a numpy array or torch tensor) rank ``rank`` keeps."""
    part = shard_of(name, dims, rank, size)
    if part is None:
        return tensor
    axis, lo, hi = part
    index = [slice(None)] * tensor.ndim
    index[axis] = slice(lo, hi)
    return tensor[tuple(index)]
