"""Host-side mirror of the reference's layer interface for the attention hot path.

The reference's host language is C++20 built with Bazel/Abseil, neither of which is available to
this build, so the layer objects that sit above the C ABI are written here with the reference's
names, argument meaning, saved-state layout and error behaviour:

    AttentionLayer          src/llm/layers/attention.h:25-77, attention.cc:400-596
    Layer.fwd / Layer.bwd   src/llm/layer.cc:35-84 (state identity check, hook dispatch)
    LayerHooks              src/llm/layer_hooks.h:46-109 (attention_probabilities_hook only)

torch is used for device memory and streams only: every arithmetic operation goes through the C
ABI into the CUDA engine, on the current torch stream (the reference's Executor::stream()).
Errors are `PlutoStatusError` with absl::StatusCode names instead of absl::Status values.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from . import _capi
from ._capi import PlutoStatusError, check


class DataType(enum.Enum):
    """src/llm/layer.h:25-31.  FP16 is a compute policy whose activations are stored as fp32."""
    FP16 = 0
    BF16 = 1
    FP8 = 2
    FP32 = 3
    INT32 = 4


def activation_torch_dtype(data_type: DataType) -> torch.dtype:
    """ActivationDataType, src/llm/layer.h:86-88."""
    return torch.bfloat16 if data_type == DataType.BF16 else torch.float32


@dataclass
class ActivationType:
    """src/llm/layer.h:33-80: storage dtype plus logical dimensions; -2 is the symbolic batch."""
    data_type: DataType
    dimensions: tuple
    kBatchDimension = -2


@dataclass
class BackwardState:
    """src/llm/layer.h:96-106."""
    layer: object = None
    intermediates: List[torch.Tensor] = field(default_factory=list)
    children: list = field(default_factory=list)


@dataclass
class FwdResult:
    """src/llm/layer.h:108-114."""
    outputs: List[torch.Tensor]
    state: BackwardState


@dataclass
class LayerHooks:
    """The one hook the attention path consumes (src/llm/layer_hooks.h:104-108): called with
    (layer name, ActivationType, probabilities tensor) before the output is published; raising
    cancels the forward."""
    attention_probabilities_hook: Optional[Callable] = None


def _invalid(message: str) -> PlutoStatusError:
    return PlutoStatusError("InvalidArgument", message, -1)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class Layer:
    """Public fwd/bwd wrappers of src/llm/layer.cc:35-84."""

    def name(self) -> str:
        raise NotImplementedError

    def fwd(self, inputs: Sequence[torch.Tensor], hooks: Optional[LayerHooks] = None) -> FwdResult:
        result = self.fwd_impl(list(inputs), hooks)
        result.state.layer = self
        return result

    def bwd(self, output_gradients: Sequence[torch.Tensor], state: BackwardState,
            hooks: Optional[LayerHooks] = None) -> List[torch.Tensor]:
        if state.layer is not self:
            raise _invalid("bwd requires a state from this layer's successful fwd")
        return self.bwd_impl(list(output_gradients), state, hooks)

    def weights(self):
        return []

    def gradients(self):
        return []


def _activation_rows(buffer: torch.Tensor, columns: int, data_type: DataType, what: str) -> int:
    """internal::ActivationRows (src/llm/layers/util.h): byte size must be a whole matrix."""
    element = 2 if data_type == DataType.BF16 else 4
    size = buffer.numel() * buffer.element_size()
    if not buffer.is_cuda:
        raise _invalid(f"{what} belongs to a different Executor")
    if size == 0 or size % element != 0:
        raise _invalid(f"{what} has an invalid byte size")
    count = size // element
    if count % columns != 0:
        raise _invalid(f"{what} is not an activation matrix")
    return count // columns


def _validate_buffer(buffer: torch.Tensor, expected_bytes: int, what: str) -> None:
    size = buffer.numel() * buffer.element_size()
    if size != expected_bytes:
        raise _invalid(f"{what} has {size} bytes; expected {expected_bytes}")


class AttentionLayer(Layer):
    """Causal multi-head attention over packed [Q, K, V] (src/llm/layers/attention.h:25-77)."""

    def __init__(self, context_length, num_heads, embedding_dim, data_type):
        self.context_length_ = context_length
        self.num_heads_ = num_heads
        self.embedding_dim_ = embedding_dim
        self.output_type_ = data_type

    @staticmethod
    def Create(context_length: int, num_heads: int, embedding_dim: int,
               data_type: DataType) -> "AttentionLayer":
        # src/llm/layers/attention.cc:400-416
        if data_type not in (DataType.FP16, DataType.BF16):
            raise PlutoStatusError("Unimplemented",
                                   "backend supports only FP16 and BF16 compute policies", -2)
        if context_length <= 0 or num_heads <= 0 or embedding_dim <= 0:
            raise _invalid("attention dimensions must all be positive")
        if embedding_dim % num_heads != 0:
            raise _invalid("embedding_dim must be divisible by num_heads")
        _capi.lib()  # fail now, loudly, if the CUDA engine is not built
        return AttentionLayer(context_length, num_heads, embedding_dim, data_type)

    def name(self) -> str:
        return "AttentionLayer"

    def output_type(self) -> DataType:
        return self.output_type_

    def input_types(self):
        storage = DataType.BF16 if self.output_type_ == DataType.BF16 else DataType.FP32
        return [ActivationType(storage, (-2, self.context_length_, 3 * self.embedding_dim_))]

    def output_types(self):
        storage = DataType.BF16 if self.output_type_ == DataType.BF16 else DataType.FP32
        return [ActivationType(storage, (-2, self.context_length_, self.embedding_dim_))]

    def _dtype_code(self) -> int:
        return 1 if self.output_type_ == DataType.BF16 else 0

    def fwd_impl(self, inputs, hooks) -> FwdResult:
        # src/llm/layers/attention.cc:418-507
        if len(inputs) != 1:
            raise _invalid("AttentionLayer fwd expects packed Q/K/V")
        qkv = inputs[0]
        E, H, S = self.embedding_dim_, self.num_heads_, self.context_length_
        rows = _activation_rows(qkv, 3 * E, self.output_type_, "attention packed Q/K/V input")
        if rows % S != 0:
            raise _invalid("attention rows must be divisible by context_length")
        inspect = hooks is not None and hooks.attention_probabilities_hook is not None
        dtype = activation_torch_dtype(self.output_type_)
        out = torch.empty((rows, E), dtype=dtype, device=qkv.device)
        maxima = torch.empty((rows * H,), dtype=torch.float32, device=qkv.device)
        normalizers = torch.empty_like(maxima)
        L = _capi.lib()
        check(L.pluto_attn_fwd(_stream(), _ptr(qkv), _ptr(out), _ptr(maxima), _ptr(normalizers),
                               rows // S, S, H, E // H, self._dtype_code()))
        if inspect:
            probs = torch.empty((rows // S, H, S, S), dtype=torch.float32, device=qkv.device)
            check(L.pluto_attn_probs(_stream(), _ptr(qkv), _ptr(maxima), _ptr(normalizers),
                                     _ptr(probs), rows // S, S, H, E // H, self._dtype_code()))
            hooks.attention_probabilities_hook(
                self.name(), ActivationType(DataType.FP32, (rows // S, H, S, S)), probs)
        state = BackwardState(intermediates=[qkv, out, maxima, normalizers])
        return FwdResult([out], state)

    def bwd_impl(self, output_gradients, state, hooks) -> List[torch.Tensor]:
        # src/llm/layers/attention.cc:509-596
        if len(output_gradients) != 1 or len(state.intermediates) != 4:
            raise _invalid("AttentionLayer bwd received an incompatible gradient or state")
        d_out = output_gradients[0]
        E, H, S = self.embedding_dim_, self.num_heads_, self.context_length_
        rows = _activation_rows(d_out, E, DataType.FP32, "attention output gradient")
        if rows % S != 0:
            raise _invalid("attention gradient rows must be divisible by context_length")
        element = 2 if self.output_type_ == DataType.BF16 else 4
        qkv, out, maxima, normalizers = state.intermediates
        _validate_buffer(qkv, rows * 3 * E * element, "attention saved Q/K/V")
        _validate_buffer(out, rows * E * element, "attention saved output")
        _validate_buffer(maxima, rows * H * 4, "attention saved maxima")
        _validate_buffer(normalizers, rows * H * 4, "attention saved normalizers")
        d_qkv = torch.empty((rows, 3 * E), dtype=torch.float32, device=d_out.device)
        deltas = torch.empty((rows * H,), dtype=torch.float32, device=d_out.device)
        check(_capi.lib().pluto_attn_bwd(_stream(), _ptr(qkv), _ptr(out), _ptr(d_out),
                                         _ptr(maxima), _ptr(normalizers), _ptr(d_qkv),
                                         _ptr(deltas), rows // S, S, H, E // H,
                                         self._dtype_code()))
        return [d_qkv]


def gqa_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                gate: Optional[torch.Tensor] = None, round_to_bfloat16: bool = True,
                want_core: bool = False, want_stats: bool = False):
    """Attention core of QwenAttentionLayer::SequenceForward (qwen_attention.cc:414-448) for
    already prepared q [B,T,Hq,D] (any token/head strides with a contiguous last dim), k, v
    [B,T,Hkv,D] bf16.  Returns dict(out[, core, maxima, normalizers])."""
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    if q.stride(3) != 1 or q.stride(0) != T * q.stride(1):
        raise _invalid("attention query must have a contiguous head dimension and batch")
    k, v = k.contiguous(), v.contiguous()
    out = torch.empty((B, T, Hq, D), dtype=torch.bfloat16, device=q.device)
    core = torch.empty((B, T, Hq, D), dtype=torch.float32, device=q.device) if want_core else None
    maxima = normalizers = None
    if want_stats:
        maxima = torch.empty((B * Hq * T,), dtype=torch.float32, device=q.device)
        normalizers = torch.empty_like(maxima)
    if gate is not None and (gate.stride(1) != q.stride(1) or gate.stride(2) != q.stride(2)):
        raise _invalid("attention gate must share the query's strides")
    check(_capi.lib().pluto_gqa_prefill_fwd(
        _stream(), _ptr(q), _ptr(gate), _ptr(k), _ptr(v), _ptr(out), _ptr(core), _ptr(maxima),
        _ptr(normalizers), B, T, Hq, Hkv, D, q.stride(1), q.stride(2), int(round_to_bfloat16)))
    result = {"out": out}
    if want_core:
        result["core"] = core
    if want_stats:
        result["maxima"], result["normalizers"] = maxima, normalizers
    return result
