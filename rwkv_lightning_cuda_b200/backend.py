"""Python mirror of the reference's ``rwkv7_server::ModelBackend`` on top of the C ABI.

Same method names, argument meaning and error behaviour as the reference class
(include/rwkv_server_backend.hpp:72-147, src/rwkv7_fast_v4.cu:1373-1592): argument errors raise
(``Rwkv7B200Error`` here, ``std::runtime_error`` there) with the same messages; ``forward_*`` is
synchronous on return.  torch is used only to own device memory and streams.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, Optional, Sequence

import torch

from . import lib as L


@dataclass
class ModelDims:
    """Mirror of rwkv7_fast_v4::ModelDims (include/rwkv7_fast_v4_common.hpp:29-36) plus LoRA ranks."""
    layers: int
    channels: int
    ffn: int
    vocab: int
    rank_w: int = 64
    rank_a: int = 64
    rank_v: int = 32
    rank_g: int = 128

    @property
    def heads(self) -> int:
        return self.channels // 64


def infer_model_dims(shapes: Dict[str, Sequence[int]]) -> ModelDims:
    """Model dimensions from a checkpoint's tensor names and shapes, by the reference's rule
    (infer_model_dims, include/rwkv7_fast_v4_common.hpp:262-288; LoRA ranks from the shapes as in
    src/rwkv7_fast_v4.cu:1168-1171).  Raises ValueError with the reference's messages."""
    vocab = channels = heads = head_size = ffn = layers = 0
    for name, shape in shapes.items():
        shape = tuple(shape)
        if name == "emb.weight" and len(shape) == 2:
            vocab, channels = shape
        elif name == "blocks.0.att.r_k" and len(shape) == 2:
            heads, head_size = shape
        elif name == "blocks.0.ffn.key.weight" and len(shape) == 2:
            ffn = shape[0]
        if name.startswith("blocks."):
            idx = name[7:].split(".", 1)
            if len(idx) == 2 and idx[0].isdigit():
                layers = max(layers, int(idx[0]) + 1)
    if not (layers > 0 and channels > 0 and heads > 0 and head_size > 0 and vocab > 0 and ffn > 0):
        raise ValueError("could not infer model dimensions")
    if channels != heads * head_size:
        raise ValueError("C must equal H*N")
    if head_size != 64:
        raise ValueError("current kernels require head size 64")

    def rank(name, default):
        shape = tuple(shapes.get(name, ()))
        return int(shape[1]) if len(shape) == 2 else default
    return ModelDims(layers, channels, ffn, vocab, rank("blocks.0.att.w1", 0), rank("blocks.0.att.a1", 0),
                     rank("blocks.1.att.v1", 8), rank("blocks.0.att.g1", 0))    # one layer: the value residual is unused


class GenerationState:
    """Mirror of rwkv7_server::GenerationState: the four device buffers and their layouts."""

    def __init__(self, batch_size: int, wkv32: bool, shift: torch.Tensor, wkv: torch.Tensor, elapsed: torch.Tensor):
        self.batch_size = batch_size
        self.wkv32 = wkv32
        self.shift = shift        # half  [L, 2, B, C]
        self.wkv_state = wkv      # half or float [L, B, H, 64, 64]
        self.elapsed = elapsed    # int32 [B]


class DeviceLogits:
    """Mirror of rwkv7_server::DeviceLogits: fp32 [rows, vocab] on the device."""

    def __init__(self):
        self.rows = 0
        self.vocab_size = 0
        self.values: Optional[torch.Tensor] = None


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def tp_unique_id() -> bytes:
    """128 bytes identifying a new tensor-parallel group; call on rank 0 and send to the other ranks."""
    buf = C.create_string_buffer(128)
    L.check(L.load_library().rwkv7_b200_tp_unique_id(buf))
    return buf.raw


class ModelBackend:
    """Drop-in counterpart of the reference ``ModelBackend`` (weights given as named tensors)."""

    def __init__(self, dims: ModelDims, tensors: Optional[Dict[str, torch.Tensor]] = None, use_wkv32: bool = False,
                 weight_format: int = L.FMT_F16, device: Optional[int] = None, model_path: str = "<synthetic>",
                 finalize: bool = True, tp_rank: int = 0, tp_size: int = 1, tp_unique_id: Optional[bytes] = None):
        """``tp_size`` > 1: head-sharded tensor parallelism, one ModelBackend per GPU/process.  Every rank passes
        the full ``tensors`` (its slice is kept), the 128-byte ``tp_unique_id`` made by :func:`tp_unique_id` on
        rank 0 and shared over any host channel, and afterwards makes the same forward calls."""
        self._lib = L.load_library()
        self.tp_rank, self.tp_size = (tp_rank, tp_size) if tp_size > 1 else (0, 1)
        self.dims = dims
        self.use_wkv32 = bool(use_wkv32)
        self._model_path = model_path
        self.device = torch.cuda.current_device() if device is None else device
        cfg = L.Config(dims.layers, dims.channels, dims.ffn, dims.vocab, dims.rank_w, dims.rank_a, dims.rank_v,
                       dims.rank_g, weight_format, int(self.use_wkv32), self.device, self.tp_rank, self.tp_size)
        handle = C.c_void_p()
        L.check(self._lib.rwkv7_b200_model_create(C.byref(cfg), C.byref(handle)))
        self._h = handle
        if self.tp_size > 1:
            if tp_unique_id is None or len(tp_unique_id) != 128:
                raise ValueError("tp_size > 1 needs the 128-byte tp_unique_id shared by rank 0")
            buf = C.create_string_buffer(bytes(tp_unique_id), 128)
            with torch.cuda.device(self.device):
                L.check(self._lib.rwkv7_b200_model_tp_init(self._h, buf))
        for name, t in (tensors or {}).items():
            self.set_tensor(name, t)
        if finalize:
            self.finalize()

    @classmethod
    def from_pth(cls, model_path: str, use_wkv32: bool = False, weight_format: int = L.FMT_F16, **kw) -> "ModelBackend":
        """The reference's constructor (ModelBackend(model_path, use_wkv32, ...), include/rwkv_server_backend.hpp:106-109):
        reads a torch ``.pth`` checkpoint with the reference's tensor names (bf16 or fp16), infers the dimensions as
        the reference does and uploads tensor by tensor; layer 0's unused v0/v1/v2 are skipped
        (include/rwkv7_fast_v4_common.hpp:323-328)."""
        ck = torch.load(model_path, map_location="cpu", mmap=True, weights_only=True)
        dims = infer_model_dims({k: tuple(v.shape) for k, v in ck.items()})
        self = cls(dims, None, use_wkv32=use_wkv32, weight_format=weight_format, model_path=model_path, finalize=False, **kw)
        for name, t in ck.items():
            if name in ("blocks.0.att.v0", "blocks.0.att.v1", "blocks.0.att.v2"):
                continue
            self.set_tensor(name, t)
        self.finalize()
        return self

    def finalize(self) -> None:
        """Builds the device layouts once every tensor has been set (streaming loaders call
        set_tensor per tensor and this at the end)."""
        L.check(self._lib.rwkv7_b200_model_finalize(self._h))

    def set_tensor(self, name: str, t: torch.Tensor) -> None:
        if t.dtype == torch.float16:
            dt = L.DT_F16
        elif t.dtype == torch.bfloat16:
            dt = L.DT_BF16
        else:
            raise TypeError(f"{name}: dtype {t.dtype} not supported (float16 or bfloat16)")
        t = t.contiguous()
        L.check(self._lib.rwkv7_b200_model_set_tensor(self._h, name.encode(), _ptr(t), dt, t.numel(), int(t.is_cuda)))

    # ---- IModelBackend surface -------------------------------------------------------------
    def create_state(self, batch_size: int) -> GenerationState:
        ns, nw, ne = C.c_size_t(), C.c_size_t(), C.c_size_t()
        L.check(self._lib.rwkv7_b200_state_sizes(self._h, batch_size, C.byref(ns), C.byref(nw), C.byref(ne)))
        d = self.dims
        dev = torch.device("cuda", self.device)
        shift = torch.empty((d.layers, 2, batch_size, d.channels), dtype=torch.float16, device=dev)
        wkv = torch.empty((d.layers, batch_size, d.heads // self.tp_size, 64, 64), dtype=torch.float32 if self.use_wkv32 else torch.float16, device=dev)
        elapsed = torch.empty((batch_size,), dtype=torch.int32, device=dev)
        assert shift.numel() == ns.value and wkv.numel() == nw.value and elapsed.numel() == ne.value
        stream = torch.cuda.current_stream(dev).cuda_stream
        L.check(self._lib.rwkv7_b200_state_init(self._h, batch_size, _ptr(shift), _ptr(wkv), _ptr(elapsed), C.c_void_p(stream)))
        torch.cuda.synchronize(dev)
        return GenerationState(batch_size, self.use_wkv32, shift, wkv, elapsed)

    def _forward(self, tokens: torch.Tensor, state: GenerationState, logits: DeviceLogits, sync: bool) -> None:
        B, T = tokens.shape
        if state.batch_size != B:
            raise L.Rwkv7B200Error(1, "state batch size mismatch")
        if state.wkv32 != self.use_wkv32:
            raise L.Rwkv7B200Error(3, "state wkv precision mismatch")
        dev = torch.device("cuda", self.device)
        if logits.values is None or logits.values.numel() < B * self.dims.vocab:
            logits.values = torch.empty((B, self.dims.vocab), dtype=torch.float32, device=dev)
        logits.rows, logits.vocab_size = B, self.dims.vocab
        stream = torch.cuda.current_stream(dev).cuda_stream
        L.check(self._lib.rwkv7_b200_forward(self._h, C.c_void_p(tokens.data_ptr()), B, T, _ptr(state.shift), _ptr(state.wkv_state),
                                             _ptr(state.elapsed), _ptr(logits.values), C.c_void_p(stream)))
        if sync:
            torch.cuda.current_stream(dev).synchronize()

    @staticmethod
    def _as_tokens(token_batches) -> torch.Tensor:
        if isinstance(token_batches, torch.Tensor):
            t = token_batches.to(dtype=torch.int64, device="cpu").contiguous()
        else:
            if len(token_batches) == 0:
                raise L.Rwkv7B200Error(1, "token_batches must not be empty")
            n = len(token_batches[0])
            if n == 0:
                raise L.Rwkv7B200Error(1, "token batch length must be positive")
            if any(len(b) != n for b in token_batches):
                raise L.Rwkv7B200Error(1, "all token batches must share the same length")
            t = torch.tensor(token_batches, dtype=torch.int64)
        return t

    def forward_prefill(self, token_batches: Sequence[Sequence[int]], state: GenerationState, logits: DeviceLogits,
                        sync: bool = True) -> None:
        self._forward(self._as_tokens(token_batches), state, logits, sync)

    def forward_decode(self, token_batch: Sequence[int], state: GenerationState, logits: DeviceLogits, sync: bool = True) -> None:
        t = self._as_tokens(token_batch) if isinstance(token_batch, torch.Tensor) else torch.tensor(list(token_batch), dtype=torch.int64)
        if t.numel() == 0:
            raise L.Rwkv7B200Error(1, "token_batches must not be empty")
        self._forward(t.reshape(-1, 1), state, logits, sync)

    def forward_to_host(self, tokens: torch.Tensor, state: GenerationState, logits: DeviceLogits, out_host: torch.Tensor) -> None:
        """Host-buffer call: token ids from host memory in, fp32 logits in (pinned) host memory out."""
        B, T = tokens.shape
        dev = torch.device("cuda", self.device)
        if logits.values is None or logits.values.numel() < B * self.dims.vocab:
            logits.values = torch.empty((B, self.dims.vocab), dtype=torch.float32, device=dev)
        logits.rows, logits.vocab_size = B, self.dims.vocab
        stream = torch.cuda.current_stream(dev).cuda_stream
        L.check(self._lib.rwkv7_b200_forward_to_host(self._h, C.c_void_p(tokens.data_ptr()), B, T, _ptr(state.shift),
                                                     _ptr(state.wkv_state), _ptr(state.elapsed), _ptr(logits.values),
                                                     C.c_void_p(out_host.data_ptr()), C.c_void_p(stream)))

    def decode_greedy(self, first_tokens: Sequence[int], steps: int, state: GenerationState, logits: DeviceLogits,
                      penalties: Optional[torch.Tensor] = None, presence_penalty: float = 0.0, repetition_penalty: float = 0.0,
                      penalty_decay: float = 1.0, out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``steps`` decode steps with the greedy choice of the next token on the device (the reference's sampler with
        top_p == 0, src/utils/sampling.cu:507-512) and no host round trip in between.  Returns the chosen ids as a
        device tensor int32 [steps, B]; with ``out_host`` (int32, pinned) they are also copied there and the stream is
        synchronised.  ``penalties`` (fp32 [B, vocab], device) is subtracted from the logits and updated in place."""
        t = first_tokens.to(dtype=torch.int64, device="cpu").contiguous() if isinstance(first_tokens, torch.Tensor) \
            else torch.tensor(list(first_tokens), dtype=torch.int64)
        B = t.numel()
        if B == 0:
            raise L.Rwkv7B200Error(1, "token_batches must not be empty")
        if state.batch_size != B:
            raise L.Rwkv7B200Error(1, "state batch size mismatch")
        if state.wkv32 != self.use_wkv32:
            raise L.Rwkv7B200Error(3, "state wkv precision mismatch")
        dev = torch.device("cuda", self.device)
        if penalties is not None and (penalties.dtype != torch.float32 or penalties.numel() != B * self.dims.vocab
                                      or not penalties.is_cuda or not penalties.is_contiguous()):
            raise L.Rwkv7B200Error(1, "penalties must be a contiguous fp32 device tensor [B, vocab]")
        if logits.values is None or logits.values.numel() < B * self.dims.vocab:
            logits.values = torch.empty((B, self.dims.vocab), dtype=torch.float32, device=dev)
        logits.rows, logits.vocab_size = B, self.dims.vocab
        out = torch.empty((max(steps, 0), B), dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        L.check(self._lib.rwkv7_b200_decode_greedy(
            self._h, C.c_void_p(t.data_ptr()), B, steps, _ptr(state.shift), _ptr(state.wkv_state), _ptr(state.elapsed),
            _ptr(logits.values), _ptr(penalties), presence_penalty, repetition_penalty, penalty_decay, _ptr(out),
            C.c_void_p(out_host.data_ptr()) if out_host is not None else None, C.c_void_p(stream)))
        return out

    def decode_sample(self, first_tokens: Sequence[int], steps: int, state: GenerationState, logits: DeviceLogits,
                      temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0, offset: int = 0,
                      penalties: Optional[torch.Tensor] = None, presence_penalty: float = 0.0, repetition_penalty: float = 0.0,
                      penalty_decay: float = 1.0, out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """decode_greedy with the sampler's general case (temperature / top-k / top-p; src/utils/sampling.cu:205-512): step i
        draws with the counter-based random number of (seed, offset + i, sequence).  Returns the ids, int32 [steps, B]."""
        t = first_tokens.to(dtype=torch.int64, device="cpu").contiguous() if isinstance(first_tokens, torch.Tensor) \
            else torch.tensor(list(first_tokens), dtype=torch.int64)
        B = t.numel()
        if B == 0:
            raise L.Rwkv7B200Error(1, "token_batches must not be empty")
        if state.batch_size != B:
            raise L.Rwkv7B200Error(1, "state batch size mismatch")
        if state.wkv32 != self.use_wkv32:
            raise L.Rwkv7B200Error(3, "state wkv precision mismatch")
        dev = torch.device("cuda", self.device)
        if logits.values is None or logits.values.numel() < B * self.dims.vocab:
            logits.values = torch.empty((B, self.dims.vocab), dtype=torch.float32, device=dev)
        logits.rows, logits.vocab_size = B, self.dims.vocab
        out = torch.empty((max(steps, 0), B), dtype=torch.int32, device=dev)
        sp = L.Sampling(temperature, top_k, top_p, seed, offset)
        stream = torch.cuda.current_stream(dev).cuda_stream
        L.check(self._lib.rwkv7_b200_decode_sample(
            self._h, C.c_void_p(t.data_ptr()), B, steps, _ptr(state.shift), _ptr(state.wkv_state), _ptr(state.elapsed),
            _ptr(logits.values), _ptr(penalties), presence_penalty, repetition_penalty, penalty_decay, C.byref(sp), _ptr(out),
            C.c_void_p(out_host.data_ptr()) if out_host is not None else None, C.c_void_p(stream)))
        return out

    def copy_state_slice(self, src: GenerationState, src_offset: int, dst: GenerationState, dst_offset: int, count: int) -> None:
        if src.wkv32 != dst.wkv32 or src.wkv32 != self.use_wkv32:
            raise L.Rwkv7B200Error(3, "state slice wkv precision mismatch")
        dev = torch.device("cuda", self.device)
        stream = torch.cuda.current_stream(dev).cuda_stream
        L.check(self._lib.rwkv7_b200_copy_state_slice(
            self._h, _ptr(src.shift), _ptr(src.wkv_state), _ptr(src.elapsed), src.batch_size, src_offset,
            _ptr(dst.shift), _ptr(dst.wkv_state), _ptr(dst.elapsed), dst.batch_size, dst_offset, count, C.c_void_p(stream)))
        torch.cuda.current_stream(dev).synchronize()

    def export_sequence(self, state: GenerationState, index: int):
        """One sequence's state as the reference's session record (src/rwkv_state_cache.cpp:268-292): pinned host tensors
        (shift half [L, 2, C], wkv half|float [L, H, 64, 64], elapsed int32 [1]), filled by asynchronous copies; synchronised
        on return."""
        d = self.dims
        shift = torch.empty((d.layers, 2, d.channels), dtype=torch.float16).pin_memory()
        wkv = torch.empty((d.layers, d.heads // self.tp_size, 64, 64), dtype=torch.float32 if self.use_wkv32 else torch.float16).pin_memory()
        elapsed = torch.empty((1,), dtype=torch.int32).pin_memory()
        dev = torch.device("cuda", self.device)
        stream = torch.cuda.current_stream(dev)
        L.check(self._lib.rwkv7_b200_state_export(self._h, _ptr(state.shift), _ptr(state.wkv_state), _ptr(state.elapsed), state.batch_size,
                                                  index, _ptr(shift), _ptr(wkv), _ptr(elapsed), C.c_void_p(stream.cuda_stream)))
        stream.synchronize()
        return shift, wkv, elapsed

    def import_sequence(self, blobs, state: GenerationState, index: int) -> None:
        """The inverse of export_sequence: writes a session record into sequence `index` of `state`."""
        shift, wkv, elapsed = (t.contiguous() for t in blobs)
        dev = torch.device("cuda", self.device)
        stream = torch.cuda.current_stream(dev)
        L.check(self._lib.rwkv7_b200_state_import(self._h, _ptr(shift), _ptr(wkv), _ptr(elapsed), _ptr(state.shift), _ptr(state.wkv_state),
                                                  _ptr(state.elapsed), state.batch_size, index, C.c_void_p(stream.cuda_stream)))
        stream.synchronize()

    def copy_logits_slice(self, src: DeviceLogits, src_offset: int, dst: DeviceLogits, dst_offset: int, count: int) -> None:
        if src_offset < 0 or dst_offset < 0 or count <= 0:
            raise L.Rwkv7B200Error(1, "invalid backend logits slice range")
        if src.rows <= 0 or src.vocab_size <= 0 or src.values is None:
            raise L.Rwkv7B200Error(1, "logits slice requires non-empty source")
        if dst.rows <= 0 or dst.vocab_size != src.vocab_size or dst.values is None:
            raise L.Rwkv7B200Error(1, "logits slice destination shape mismatch")
        if src_offset + count > src.rows or dst_offset + count > dst.rows:
            raise L.Rwkv7B200Error(1, "logits slice range exceeds row count")
        dst.values[dst_offset:dst_offset + count].copy_(src.values[src_offset:src_offset + count])

    def query_prefill_capacity(self, prefill_chunk_size: int) -> L.Capacity:
        cap = L.Capacity()
        L.check(self._lib.rwkv7_b200_query_capacity(self._h, prefill_chunk_size, C.byref(cap)))
        return cap

    def vocab_size(self) -> int:
        return self._lib.rwkv7_b200_vocab_size(self._h)

    def model_path(self) -> str:
        return self._model_path

    def kernel_launches(self) -> int:
        return int(self._lib.rwkv7_b200_kernel_launches(self._h))

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.rwkv7_b200_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
