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


class BlockParameter:
    """A trainable or frozen fp32 parameter shared between a layer and its optimizer
    (src/llm/block_parameter.h): `value()`, `active()`, `Activate()` (allocates a zeroed gradient),
    `gradient()`.  Backward passes ACCUMULATE into the gradient of an active parameter."""

    def __init__(self, value: torch.Tensor):
        self.value_ = value
        self.gradient_ = None

    @staticmethod
    def Create(value: torch.Tensor) -> "BlockParameter":
        if value is None or value.dtype not in (torch.float32, torch.bfloat16) or not value.is_cuda:
            raise _invalid("BlockParameter requires an FP32 or BF16 device buffer")
        return BlockParameter(value)

    def value(self) -> torch.Tensor:
        return self.value_

    def active(self) -> bool:
        return self.gradient_ is not None

    def Activate(self) -> None:
        if self.gradient_ is None:   # the gradient (optimizer storage) is fp32 whatever the value is
            self.gradient_ = torch.zeros(self.value_.shape, dtype=torch.float32, device=self.value_.device)

    def Deactivate(self) -> None:
        self.gradient_ = None

    def gradient(self) -> Optional[torch.Tensor]:
        return self.gradient_


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
        # bf16 layers with head width 64/128 run backward on the tensor cores; set False to force
        # the exact fp32 kernels (every shape has them)
        self.tensor_core_backward = True

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
        L = _capi.lib()
        ws_ptr, ws_bytes = None, 0
        need = L.pluto_attn_bwd_workspace_bytes(rows // S, S, H, E // H, self._dtype_code())
        if need and self.tensor_core_backward:
            ws = torch.empty((need + 256,), dtype=torch.uint8, device=d_out.device)
            ws_ptr = (ws.data_ptr() + 255) // 256 * 256
            ws_bytes = need
        check(L.pluto_attn_bwd(_stream(), _ptr(qkv), _ptr(out), _ptr(d_out), _ptr(maxima),
                               _ptr(normalizers), _ptr(d_qkv), _ptr(deltas), rows // S, S, H, E // H,
                               self._dtype_code(), ws_ptr, ws_bytes))
        return [d_qkv]


def gqa_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                gate: Optional[torch.Tensor] = None, round_to_bfloat16: bool = True,
                want_core: bool = False, want_stats: bool = False,
                workspace: Optional[torch.Tensor] = None):
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
    gts = ghs = 0
    if gate is not None:
        if gate.stride(3) != 1 or gate.stride(0) != T * gate.stride(1):
            raise _invalid("attention gate must have a contiguous head dimension and batch")
        gts, ghs = gate.stride(1), gate.stride(2)
    # a few heads of a long prompt cannot load the SMs evenly with whole query tiles: the kernel
    # then cuts the longest tile pairs along their keys and needs scratch for the partial results
    # (the query returns 0 for shapes it would not cut); pass `workspace` to reuse one across calls
    L = _capi.lib()
    ws_ptr, ws_bytes = None, 0
    if D in (64, 128):
        ws_bytes = L.pluto_gqa_prefill_fwd_workspace_bytes(B, T, Hq, D)
    if ws_bytes > 0:
        if workspace is None or workspace.numel() < ws_bytes + 16:
            workspace = torch.empty((ws_bytes + 16,), dtype=torch.uint8, device=q.device)
        ws_ptr = (workspace.data_ptr() + 15) // 16 * 16
    check(L.pluto_gqa_prefill_fwd(
        _stream(), _ptr(q), _ptr(gate), _ptr(k), _ptr(v), _ptr(out), _ptr(core), _ptr(maxima),
        _ptr(normalizers), B, T, Hq, Hkv, D, q.stride(1), q.stride(2), gts, ghs,
        int(round_to_bfloat16), ws_ptr, ws_bytes))
    result = {"out": out}
    if ws_ptr is not None:
        result["workspace"] = workspace   # hand it back in to skip the allocation next time
    if want_core:
        result["core"] = core
    if want_stats:
        result["maxima"], result["normalizers"] = maxima, normalizers
    return result


def gqa_prefill_host(q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
                     out_host: torch.Tensor, kv_heads_per_group: int = 1,
                     workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """gqa_prefill for activations in pinned host memory (bf16, dense [B,T,Hq,D] / [B,T,Hkv,D]):
    the copies in both directions and the kernels of successive key/value-head groups overlap
    (pluto_gqa_prefill_fwd_host).  kv_heads_per_group = 0 cuts the prompt by query tokens instead
    (contiguous copies, the whole Q / K / V / output on the device).  Writes out_host; the caller
    synchronises the current stream before reading it.  Pass `workspace` (uint8 device tensor) to
    reuse one across calls."""
    B, T, Hq, D = q_host.shape
    Hkv = k_host.shape[2]
    for t in (q_host, k_host, v_host, out_host):
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.is_cuda or not t.is_pinned():
            raise _invalid("host prefill requires dense bf16 tensors in pinned host memory")
    L = _capi.lib()
    need = L.pluto_gqa_prefill_host_workspace_bytes(B, T, Hq, Hkv, D, kv_heads_per_group)
    if need == 0:
        raise _invalid("invalid full-attention dimensions or parameters")
    if workspace is None or workspace.numel() < need + 256:
        workspace = torch.empty((need + 256,), dtype=torch.uint8, device="cuda")
    ws_ptr = (workspace.data_ptr() + 255) // 256 * 256
    check(L.pluto_gqa_prefill_fwd_host(_stream(), q_host.data_ptr(), k_host.data_ptr(),
                                       v_host.data_ptr(), out_host.data_ptr(), ws_ptr,
                                       workspace.numel() - (ws_ptr - workspace.data_ptr()), B, T, Hq,
                                       Hkv, D, kv_heads_per_group))
    return workspace


# =================================================================================================
# Qwen cached attention: KeyValueCache, FullAttentionParameters, CachedAttentionStep
# =================================================================================================
def _resource_exhausted(message: str) -> PlutoStatusError:
    return PlutoStatusError("ResourceExhausted", message, -3)


@dataclass
class FullAttentionParameters:
    """src/llm/layers/util/cached_attention_ops.h:13-22, field for field."""
    query_heads: int = 24
    key_value_heads: int = 4
    head_dim: int = 256
    rotary_dim: int = 64
    capacity: int = 4096
    rms_norm_epsilon: float = 1e-6
    rope_theta: float = 10000000.0
    round_to_bfloat16: bool = True


class KeyValueCache:
    """Per-sequence K/V storage [capacity, kv_heads, head_dim] with a position counter
    (src/llm/key_value_cache.h:25-57).  The reference stores fp32; every value it writes is already
    bf16-rounded when rounding is on, so `dtype=torch.bfloat16` (default) holds the same numbers
    in half the bytes.  `torch.float32` keeps the reference's storage."""

    def __init__(self, capacity, key_value_heads, head_dim, dtype, device):
        self.capacity_ = capacity
        self.key_value_heads_ = key_value_heads
        self.head_dim_ = head_dim
        self.keys_ = torch.zeros((capacity, key_value_heads, head_dim), dtype=dtype, device=device)
        self.values_ = torch.zeros_like(self.keys_)
        self.position_ = 0

    @staticmethod
    def Create(capacity: int, key_value_heads: int, head_dim: int,
               dtype: torch.dtype = torch.bfloat16, device="cuda") -> "KeyValueCache":
        # src/llm/key_value_cache.cc:20-36
        if capacity <= 0 or key_value_heads <= 0 or head_dim <= 0:
            raise _invalid("key-value cache dimensions must be positive")
        if dtype not in (torch.bfloat16, torch.float32):
            raise _invalid("key-value cache stores bf16 or fp32")
        return KeyValueCache(capacity, key_value_heads, head_dim, dtype, device)

    def capacity(self): return self.capacity_
    def key_value_heads(self): return self.key_value_heads_
    def head_dim(self): return self.head_dim_
    def position(self): return self.position_
    def keys(self): return self.keys_
    def values(self): return self.values_

    def Advance(self) -> None:
        if self.position_ >= self.capacity_:
            raise _resource_exhausted("key-value cache capacity reached")
        self.position_ += 1

    def Reset(self) -> None:
        self.position_ = 0  # contents are not cleared, as in the reference

    def layout(self) -> "_capi.KvCacheStruct":
        return kv_layout(self.keys_, self.values_, None, self.capacity_,
                         self.capacity_ * self.key_value_heads_ * self.head_dim_,
                         self.key_value_heads_ * self.head_dim_)


def kv_layout(k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: Optional[torch.Tensor],
              page_size: int, page_stride: int, token_stride: int) -> "_capi.KvCacheStruct":
    s = _capi.KvCacheStruct()
    s.k_base, s.v_base = k_pool.data_ptr(), v_pool.data_ptr()
    s.block_table = None if block_table is None else block_table.data_ptr()
    s.max_blocks = 0 if block_table is None else block_table.shape[1]
    s.page_size, s.page_stride, s.token_stride = page_size, page_stride, token_stride
    s.dtype = 1 if k_pool.dtype == torch.bfloat16 else 0
    s.num_pages = k_pool.shape[0] if k_pool.dim() == 4 else 1
    return s


def gqa_decode_separate_caches(q: torch.Tensor, caches, seq_lens: torch.Tensor, *,
                               round_to_bfloat16: bool = True, want_lse: bool = False):
    """Batched decode over independently allocated per-sequence caches (one KeyValueCache object
    per sequence, as the reference keeps them, src/llm/key_value_cache.h:25-57): the cache
    descriptor carries two device arrays of base pointers instead of one pool.  q [B,Hq,D];
    `caches` B KeyValueCache objects of equal shape and dtype; seq_lens int32 [B]."""
    B, Hq, D = q.shape
    first = caches[0]
    if len(caches) != B or any(c.keys().shape != first.keys().shape or c.keys().dtype != first.keys().dtype
                               for c in caches):
        raise _invalid("one cache per sequence, all of one shape and dtype")
    capacity, Hkv = first.capacity(), first.key_value_heads()
    k_bases = torch.tensor([c.keys().data_ptr() for c in caches], dtype=torch.int64, device=q.device)
    v_bases = torch.tensor([c.values().data_ptr() for c in caches], dtype=torch.int64, device=q.device)
    layout = _capi.KvCacheStruct()
    layout.k_base = layout.v_base = layout.block_table = None
    layout.max_blocks, layout.page_size = 0, capacity
    layout.page_stride = layout.token_stride = Hkv * D
    layout.page_stride *= capacity
    layout.dtype = 1 if first.keys().dtype == torch.bfloat16 else 0
    layout.num_pages = 0
    layout.k_bases, layout.v_bases = k_bases.data_ptr(), v_bases.data_ptr()
    L = _capi.lib()
    out = torch.empty_like(q)
    nbytes = L.pluto_gqa_decode_workspace_bytes(B, Hq, Hkv, D, capacity)
    ws = _workspace(q.device, nbytes)
    lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device) if want_lse else None
    check(L.pluto_gqa_decode(_stream(), _ptr(q), _dt(q), None, 0, 0, 0, C_byref(layout), _ptr(seq_lens),
                             capacity, _ptr(out), _dt(out), _ptr(lse), _ptr(ws), ws.numel(), B, Hq, Hkv, D,
                             int(round_to_bfloat16)))
    return (out, lse) if want_lse else out


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise _invalid("tensor must be bf16 or fp32")


def ValidateCachedAttention(p: FullAttentionParameters, cache: KeyValueCache) -> None:
    """src/llm/layers/util/cached_attention_ops.cc:283-306.  No GPU work."""
    import math
    imax = 2 ** 31 - 1
    if (p.query_heads <= 0 or p.key_value_heads <= 0 or p.query_heads % p.key_value_heads != 0
            or p.head_dim <= 0 or p.head_dim > 256 or p.rotary_dim <= 0
            or p.rotary_dim > p.head_dim or p.rotary_dim % 2 != 0 or p.capacity <= 0
            or p.capacity > imax - 32 or not math.isfinite(p.rope_theta) or p.rope_theta <= 0.0
            or not math.isfinite(p.rms_norm_epsilon) or p.rms_norm_epsilon <= 0.0
            or p.query_heads > imax // (2 * p.head_dim)
            or p.query_heads > imax - p.key_value_heads):
        raise _invalid("invalid full-attention dimensions or parameters")
    if (cache.capacity() != p.capacity or cache.key_value_heads() != p.key_value_heads
            or cache.head_dim() != p.head_dim):
        raise _invalid("attention cache shape or capacity does not match parameters")


_decode_workspaces = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    key = (str(device), torch.cuda.current_stream().cuda_stream)
    ws = _decode_workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty((max(nbytes, 1 << 20),), dtype=torch.uint8, device=device)
        _decode_workspaces[key] = ws
    return ws


def CachedAttentionStep(p: FullAttentionParameters, cache: KeyValueCache, q_gate: torch.Tensor,
                        k: torch.Tensor, v: torch.Tensor, q_norm: torch.Tensor,
                        k_norm: torch.Tensor, output: torch.Tensor,
                        probabilities: Optional[torch.Tensor] = None) -> None:
    """One token of batch-one causal attention against `cache`
    (src/llm/layers/util/cached_attention_ops.cc:308-353): validate everything, prepare
    (norm + RoPE + append), attend, optional probabilities, then advance the cache -- the position
    moves only after every launch succeeded.  q_gate [Hq,2,D], k,v [Hkv,D], output [Hq,D];
    fp32 (the reference's pointer type) or bf16."""
    ValidateCachedAttention(p, cache)
    for t in (q_gate, k, v, q_norm, k_norm, output):
        if t is None:
            raise _invalid("attention requires non-null device pointers")
    if cache.position() >= cache.capacity():
        raise _resource_exhausted("full-attention cache capacity reached")
    L = _capi.lib()
    device = output.device
    position = cache.position()
    D, Hq, Hkv = p.head_dim, p.query_heads, p.key_value_heads
    queries = torch.empty((Hq, D), dtype=torch.bfloat16 if p.round_to_bfloat16 else torch.float32,
                          device=device)
    positions = torch.tensor([position], dtype=torch.int32, device=device)
    layout = cache.layout()
    check(L.pluto_qk_prepare(_stream(), _ptr(q_gate), _ptr(k), _ptr(v), _dt(q_gate), 2 * Hq * D,
                             2 * D, _ptr(q_norm), _ptr(k_norm), _ptr(positions), _ptr(queries),
                             _dt(queries), C_byref(layout), 1, 1, Hq, Hkv, D, p.rotary_dim,
                             p.rms_norm_epsilon, p.rope_theta, int(p.round_to_bfloat16)))
    lens = positions + 1
    nbytes = L.pluto_gqa_decode_workspace_bytes(1, Hq, Hkv, D, position + 1)
    ws = _workspace(device, nbytes)
    gate = q_gate.reshape(-1)[D:]
    check(L.pluto_gqa_decode(_stream(), _ptr(queries), _dt(queries), _ptr(gate), _dt(q_gate),
                             2 * Hq * D, 2 * D, C_byref(layout), _ptr(lens), position + 1,
                             _ptr(output), _dt(output), None, _ptr(ws), ws.numel(), 1, Hq, Hkv, D,
                             int(p.round_to_bfloat16)))
    if probabilities is not None:
        check(L.pluto_gqa_decode_probs(_stream(), _ptr(queries), _dt(queries), C_byref(layout),
                                       _ptr(lens), _ptr(probabilities), 0, position + 1, 1, Hq, Hkv,
                                       D))
    cache.Advance()


def C_byref(struct):
    import ctypes
    return ctypes.cast(ctypes.pointer(struct), ctypes.c_void_p)


def gqa_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, seq_lens: torch.Tensor,
               max_seq_len: int, *, block_table: Optional[torch.Tensor] = None,
               page_size: Optional[int] = None, gate: Optional[torch.Tensor] = None,
               round_to_bfloat16: bool = True, out: Optional[torch.Tensor] = None,
               workspace: Optional[torch.Tensor] = None, want_lse: bool = False):
    """Batched decode over a page pool.  q [B,Hq,D] prepared queries; k_pool/v_pool
    [pages, page_size, Hkv, D]; without a block table sequence b owns page b.  Returns out
    [B,Hq,D] (and lse [B,Hq])."""
    B, Hq, D = q.shape
    pages, psize, Hkv, _ = k_pool.shape
    page_size = psize if page_size is None else page_size
    layout = kv_layout(k_pool, v_pool, block_table, page_size, k_pool.stride(0), k_pool.stride(1))
    L = _capi.lib()
    if out is None:
        out = torch.empty_like(q)
    nbytes = L.pluto_gqa_decode_workspace_bytes(B, Hq, Hkv, D, max_seq_len)
    ws = workspace if workspace is not None else _workspace(q.device, nbytes)
    lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device) if want_lse else None
    gts = ghs = 0
    if gate is not None:
        gts, ghs = gate.stride(0), gate.stride(1)
    check(L.pluto_gqa_decode(_stream(), _ptr(q), _dt(q), _ptr(gate),
                             _dt(gate) if gate is not None else 0, gts, ghs, C_byref(layout),
                             _ptr(seq_lens), max_seq_len, _ptr(out), _dt(out), _ptr(lse), _ptr(ws),
                             ws.numel(), B, Hq, Hkv, D, int(round_to_bfloat16)))
    return (out, lse) if want_lse else out


# =================================================================================================
# Gated delta-net
# =================================================================================================
@dataclass
class DeltaNetParameters:
    """src/llm/layers/util/cached_attention_ops.h:49-57, field for field."""
    key_heads: int = 16
    value_heads: int = 48
    key_head_dim: int = 128
    value_head_dim: int = 128
    conv_kernel_dim: int = 4
    rms_norm_epsilon: float = 1e-6
    round_to_bfloat16: bool = True


class DeltaNetState:
    """Single-token causal depthwise convolution + gated delta recurrence with an fp32 recurrent
    matrix (src/llm/layers/util/cached_attention_ops.h:59-89, .cc:355-442)."""

    def __init__(self, p: DeltaNetParameters, device):
        self.parameters_ = p
        self.channels_ = 2 * p.key_heads * p.key_head_dim + p.value_heads * p.value_head_dim
        f32 = dict(dtype=torch.float32, device=device)
        self.convolution_state_ = torch.empty((1, self.channels_, p.conv_kernel_dim), **f32)
        self.recurrent_state_ = torch.empty((1, p.value_heads, p.key_head_dim, p.value_head_dim),
                                            **f32)
        self.convolved_qkv_ = torch.empty((self.channels_,), **f32)
        self.core_output_ = torch.empty((p.value_heads, p.value_head_dim), **f32)
        self.g_ = torch.empty((p.value_heads,), **f32)
        self.beta_ = torch.empty((p.value_heads,), **f32)

    @staticmethod
    def Create(p: DeltaNetParameters, device="cuda") -> "DeltaNetState":
        import math
        if (p.key_heads <= 0 or p.value_heads <= 0 or p.value_heads % p.key_heads != 0
                or p.key_head_dim <= 0 or p.key_head_dim > 128 or p.value_head_dim <= 0
                or p.value_head_dim > 256 or p.conv_kernel_dim <= 0 or p.conv_kernel_dim > 32
                or not math.isfinite(p.rms_norm_epsilon) or p.rms_norm_epsilon <= 0.0):
            raise _invalid("invalid DeltaNet dimensions or parameters")
        _capi.lib()
        state = DeltaNetState(p, device)
        state.Reset()
        return state

    def Reset(self) -> None:
        self.convolution_state_.zero_()
        self.recurrent_state_.zero_()

    def Step(self, qkv, z, a, b, conv_weight, a_log, dt_bias, norm_weight, output) -> None:
        """qkv packed [all Q, all K, all V]; z [Hv,dv]; a, b, A_log, dt_bias [Hv]; conv weights
        [channels, kernel] oldest to newest; norm_weight [dv] plain multiplier; output [Hv,dv]."""
        for t in (qkv, z, a, b, conv_weight, a_log, dt_bias, norm_weight, output):
            if t is None:
                raise _invalid("DeltaNet requires non-null device pointers")
        p, L, rnd = self.parameters_, _capi.lib(), int(self.parameters_.round_to_bfloat16)
        check(L.pluto_gdn_conv_silu(_stream(), _ptr(qkv), _ptr(conv_weight), _dt(qkv), 1, 1,
                                    self.channels_, p.conv_kernel_dim, rnd,
                                    _ptr(self.convolution_state_), _ptr(self.convolved_qkv_), 0))
        check(L.pluto_gdn_gates(_stream(), _ptr(a), _ptr(b), _ptr(a_log), _ptr(dt_bias), _dt(a), 1,
                                p.value_heads, rnd, _ptr(self.g_), _ptr(self.beta_)))
        kq = p.key_heads * p.key_head_dim
        conv = self.convolved_qkv_
        check(L.pluto_gdn_step(_stream(), _ptr(conv[:kq]), _ptr(conv[kq:2 * kq]),
                               _ptr(conv[2 * kq:]), 0, _ptr(self.g_), _ptr(self.beta_),
                               _ptr(self.recurrent_state_), _ptr(self.core_output_), 0, 1,
                               p.key_heads, p.value_heads, p.key_head_dim, p.value_head_dim, 1,
                               1.0, rnd))
        check(L.pluto_gdn_out_norm_gate(_stream(), _ptr(self.core_output_), 0, _ptr(z), _dt(z),
                                        _ptr(norm_weight), p.value_heads, p.value_head_dim,
                                        p.rms_norm_epsilon, rnd, 1, _ptr(output), _dt(output)))


def gdn_prefill(q, k, v, g, beta, state, normalize_qk=True, q_scale=1.0, round_to_bfloat16=True,
                out=None, chunked=None, workspace=None):
    """Recurrence over a whole sequence from `state` (updated in place).  q,k [B,T,Hk,dk];
    v [B,T,Hv,dv]; g,beta fp32 [B,T,Hv]; state fp32 [B,Hv,dk,dv].  Returns out like v.
    chunked=None picks the 64-token chunked tensor-core form when the shape has one (bf16 inputs,
    key width 128, T >= 64) and the token-sequential kernel otherwise; False forces the latter."""
    B, T, Hk, dk = q.shape
    Hv, dv = v.shape[2], v.shape[3]
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if out is None:
        out = torch.empty_like(v)
    L = _capi.lib()
    ws_ptr, ws_bytes = None, 0
    if chunked is None or chunked:
        need = L.pluto_gdn_prefill_workspace_bytes(B, T, Hk, Hv, dk, dv, _dt(v))
        if need == 0 and chunked:
            raise _invalid("DeltaNet shape has no chunked prefill path")
        if need:
            ws = workspace if workspace is not None else _workspace(q.device, need + 256)
            ws_ptr = (ws.data_ptr() + 255) // 256 * 256
            ws_bytes = ws.numel() - (ws_ptr - ws.data_ptr())
    check(L.pluto_gdn_prefill(_stream(), _ptr(q), _ptr(k), _ptr(v), _dt(v), _ptr(g), _ptr(beta),
                              _ptr(state), _ptr(out), _dt(out), B, T, Hk, Hv, dk, dv, 0, 0,
                              int(normalize_qk), float(q_scale), int(round_to_bfloat16), ws_ptr,
                              ws_bytes))
    return out


def gdn_step(q, k, v, g, beta, state, normalize_qk=True, q_scale=1.0, round_to_bfloat16=True,
             out=None):
    """Single-token update: q,k [B,Hk,dk]; v [B,Hv,dv]; g,beta [B,Hv]."""
    B, Hk, dk = q.shape
    Hv, dv = v.shape[1], v.shape[2]
    if out is None:
        out = torch.empty_like(v)
    check(_capi.lib().pluto_gdn_step(_stream(), _ptr(q), _ptr(k), _ptr(v), _dt(v), _ptr(g),
                                     _ptr(beta), _ptr(state), _ptr(out), _dt(out), B, Hk, Hv, dk,
                                     dv, int(normalize_qk), float(q_scale), int(round_to_bfloat16)))
    return out


def gqa_decode_noalloc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                       seq_lens: torch.Tensor, max_seq_len: int, out: torch.Tensor, *,
                       block_table: Optional[torch.Tensor] = None,
                       gate: Optional[torch.Tensor] = None,
                       round_to_bfloat16: bool = True,
                       lse: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`gqa_decode` for callers that may not allocate device memory (a fixed, fully committed
    memory plan; a sandbox that forbids cudaMalloc to plugins; a decode loop that must stay off
    the allocator lock).  Nothing is allocated here or in the library: `out` comes from the
    caller and the split-KV partials use the 32 MiB area built into the library, which every
    call shares -- keep calls on one stream.  Raises ResourceExhausted when the shape needs more
    scratch than the area holds."""
    B, Hq, D = q.shape
    _, psize, Hkv, _ = k_pool.shape
    layout = kv_layout(k_pool, v_pool, block_table, psize, k_pool.stride(0), k_pool.stride(1))
    gts = ghs = 0
    if gate is not None:
        gts, ghs = gate.stride(0), gate.stride(1)
    check(_capi.lib().pluto_gqa_decode_noalloc(
        _stream(), _ptr(q), _dt(q), _ptr(gate), _dt(gate) if gate is not None else 0, gts, ghs,
        C_byref(layout), _ptr(seq_lens), max_seq_len, _ptr(out), _dt(out), _ptr(lse), B, Hq, Hkv, D,
        int(round_to_bfloat16)))
    return out


# =================================================================================================
# Layer objects of the Qwen decoder: QwenAttentionLayer, DeltaNetLayer, SequenceDeltaNetLayer
# =================================================================================================
def _unimplemented(message: str) -> PlutoStatusError:
    return PlutoStatusError("Unimplemented", message, -2)


def _validate_bf16_inputs(inputs, counts, what: str) -> None:
    """internal::ValidateBFloat16Inputs (src/llm/layers/util.cc): count and exact byte sizes."""
    if len(inputs) != len(counts):
        raise _invalid(f"{what} expects {len(counts)} inputs")
    for tensor, count in zip(inputs, counts):
        if not tensor.is_cuda:
            raise _invalid(f"{what} input belongs to a different Executor")
        if tensor.dtype != torch.bfloat16 or tensor.numel() != count:
            raise _invalid(f"{what} input has {tensor.numel() * tensor.element_size()} bytes; "
                           f"expected {2 * count}")


class QwenAttentionLayer(Layer):
    """Qwen grouped-query attention: per-head Q/K RMSNorm, partial RoPE, causal attention, sigmoid
    output gate (src/llm/layers/qwen_attention.h:14-99, .cc:291-448).  Inputs are bf16
    [T, query_heads, 2, head_dim] query/gate and [T, kv_heads, head_dim] K and V; the output is
    bf16 [T, query_heads, head_dim].  A cache selects single-token inference (sequence_length 1,
    backward rejected); without one the layer is the stateless sequence forward.  The reference
    limits the sequence form to 128 positions because it materialises all probabilities; here any
    length runs (the probabilities exist only when a hook asks for them)."""

    kMaximumDimension = 1048576

    def __init__(self, parameters, q_norm, k_norm, sequence_length, cache):
        self.parameters_ = parameters
        self.norms_ = [q_norm, k_norm]                       # BlockParameter
        # head widths 64/128 run the backward attention core on the tensor cores; set False to
        # force the exact fp32 kernels (every shape has them)
        self.tensor_core_backward = True
        self.weights_ = [q_norm.value(), k_norm.value()]
        self.sequence_length_ = sequence_length
        self.cache_ = cache

    @staticmethod
    def Create(parameters: FullAttentionParameters, q_norm, k_norm,
               sequence_length: int, cache: Optional[KeyValueCache] = None) -> "QwenAttentionLayer":
        """q_norm / k_norm: a BlockParameter (shared, possibly active) or a raw fp32 tensor (the
        reference's Buffer overload, qwen_attention.h:42-47: a frozen parameter)."""
        import math
        p = parameters
        q_norm = q_norm if isinstance(q_norm, BlockParameter) or q_norm is None else BlockParameter(q_norm)
        k_norm = k_norm if isinstance(k_norm, BlockParameter) or k_norm is None else BlockParameter(k_norm)
        if cache is not None:
            if sequence_length != 1:
                raise _invalid("cached Qwen attention requires sequence_length == 1")
            if p.query_heads <= 0 or p.key_value_heads <= 0 or p.head_dim <= 0:
                raise _invalid("QwenAttentionLayer dimensions must be positive")
            if (p.query_heads * p.head_dim > QwenAttentionLayer.kMaximumDimension // 2
                    or p.key_value_heads * p.head_dim > QwenAttentionLayer.kMaximumDimension):
                raise _invalid("QwenAttentionLayer activation exceeds the layer dimension limit")
            ValidateCachedAttention(p, cache)
        else:
            if (p.query_heads <= 0 or p.query_heads > 256 or p.key_value_heads <= 0
                    or p.query_heads % p.key_value_heads or p.head_dim <= 0 or p.head_dim > 256
                    or p.rotary_dim <= 0 or p.rotary_dim > p.head_dim or p.rotary_dim % 2
                    or sequence_length <= 0 or not (p.rms_norm_epsilon > 0)
                    or not math.isfinite(p.rms_norm_epsilon) or not (p.rope_theta > 0)
                    or not math.isfinite(p.rope_theta)):
                raise _invalid("sequence Qwen attention requires valid GQA dimensions and D<=256")
        for parameter in (q_norm, k_norm):
            norm = None if parameter is None else parameter.value()
            if norm is None or norm.dtype != torch.float32 or norm.numel() != p.head_dim or not norm.is_cuda:
                raise _invalid("Qwen attention norms must be FP32 head-width parameters on its Executor")
        _capi.lib()
        return QwenAttentionLayer(p, q_norm, k_norm, sequence_length, cache)

    def name(self) -> str:
        return "QwenAttentionLayer"

    def output_type(self) -> DataType:
        return DataType.BF16

    def weights(self):
        return self.weights_

    def gradients(self):
        return [n.gradient() for n in self.norms_ if n.active()]

    def input_types(self):
        p, t = self.parameters_, self.sequence_length_
        return [ActivationType(DataType.BF16, (-2, t, 2 * p.query_heads * p.head_dim)),
                ActivationType(DataType.BF16, (-2, t, p.key_value_heads * p.head_dim)),
                ActivationType(DataType.BF16, (-2, t, p.key_value_heads * p.head_dim))]

    def output_types(self):
        p = self.parameters_
        return [ActivationType(DataType.BF16, (-2, self.sequence_length_, p.query_heads * p.head_dim))]

    def fwd_impl(self, inputs, hooks) -> FwdResult:
        return self._cached_forward(inputs, hooks) if self.cache_ is not None else \
            self._sequence_forward(inputs, hooks)

    def bwd_impl(self, output_gradients, state, hooks):
        if self.cache_ is not None:
            raise _unimplemented("QwenAttentionLayer with a KV cache supports inference only")
        return self._sequence_backward(output_gradients, state)

    def _cached_forward(self, inputs, hooks) -> FwdResult:
        # src/llm/layers/qwen_attention.cc:370-412, minus the bf16<->fp32 cast launches
        p = self.parameters_
        width = p.query_heads * p.head_dim
        kv = p.key_value_heads * p.head_dim
        _validate_bf16_inputs(inputs, [2 * width, kv, kv], "QwenAttentionLayer")
        if self.cache_.position() >= self.cache_.capacity():
            raise _resource_exhausted("full-attention cache capacity reached")
        output = torch.empty((1, width), dtype=torch.bfloat16, device=inputs[0].device)
        length = self.cache_.position() + 1
        inspect = hooks is not None and hooks.attention_probabilities_hook is not None
        probabilities = torch.empty((p.query_heads, length), dtype=torch.float32,
                                    device=inputs[0].device) if inspect else None
        CachedAttentionStep(p, self.cache_, inputs[0].view(p.query_heads, 2, p.head_dim),
                            inputs[1].view(p.key_value_heads, p.head_dim),
                            inputs[2].view(p.key_value_heads, p.head_dim), self.weights_[0],
                            self.weights_[1], output.view(p.query_heads, p.head_dim), probabilities)
        if inspect:
            hooks.attention_probabilities_hook(
                self.name(), ActivationType(DataType.FP32, (1, p.query_heads, 1, length)), probabilities)
        return FwdResult([output], BackwardState())

    def _sequence_forward(self, inputs, hooks) -> FwdResult:
        # src/llm/layers/qwen_attention.cc:414-448: PrepareKernel + ForwardKernel
        p, t = self.parameters_, self.sequence_length_
        hq, hkv, d = p.query_heads, p.key_value_heads, p.head_dim
        _validate_bf16_inputs(inputs, [2 * t * hq * d, t * hkv * d, t * hkv * d], "QwenAttentionLayer")
        if not p.round_to_bfloat16:
            raise _unimplemented("sequence Qwen attention without bf16 rounding is not built")
        L = _capi.lib()
        device = inputs[0].device
        q = torch.empty((1, t, hq, d), dtype=torch.bfloat16, device=device)
        k = torch.empty((1, t, hkv, d), dtype=torch.bfloat16, device=device)
        v = torch.empty_like(k)
        layout = kv_layout(k, v, None, t, t * hkv * d, hkv * d)
        check(L.pluto_qk_prepare(_stream(), _ptr(inputs[0]), _ptr(inputs[1]), _ptr(inputs[2]), 1,
                                 2 * hq * d, 2 * d, _ptr(self.weights_[0]), _ptr(self.weights_[1]),
                                 None, _ptr(q), 1, C_byref(layout), 1, t, hq, hkv, d, p.rotary_dim,
                                 p.rms_norm_epsilon, p.rope_theta, 1))
        qg = inputs[0].view(1, t, hq, 2, d)
        result = gqa_prefill(q, k, v, gate=qg[:, :, :, 1], round_to_bfloat16=True, want_core=True,
                             want_stats=True)
        output = result["out"].view(t, hq * d)
        probabilities = torch.empty((0,), dtype=torch.float32, device=device)
        if hooks is not None and hooks.attention_probabilities_hook is not None:
            probabilities = torch.zeros((hq, t, t), dtype=torch.float32, device=device)
            rows = torch.arange(1, t + 1, dtype=torch.int32, device=device)
            table = torch.zeros((t, 1), dtype=torch.int32, device=device)
            paged = kv_layout(k, v, table, t, t * hkv * d, hkv * d)
            check(L.pluto_gqa_decode_probs(_stream(), _ptr(q), 1, C_byref(paged), _ptr(rows),
                                           _ptr(probabilities), t, t * t, t, hq, hkv, d))
            hooks.attention_probabilities_hook(
                self.name(), ActivationType(DataType.FP32, (1, hq, t, t)), probabilities)
        # the reference's seven saved buffers (its probabilities are empty here unless a hook asked
        # for them) plus what replaces them for backward: the softmax statistics and the value rows
        state = BackwardState(intermediates=[inputs[0], inputs[1], inputs[2], q, k, probabilities,
                                             result["core"], result["maxima"],
                                             result["normalizers"], v])
        return FwdResult([output], state)

    def _sequence_backward(self, output_gradients, state):
        # src/llm/layers/qwen_attention.cc:450-499: gate -> attention core -> RoPE^-1 + RMSNorm
        p, t = self.parameters_, self.sequence_length_
        hq, hkv, d = p.query_heads, p.key_value_heads, p.head_dim
        if len(state.intermediates) != 10:
            raise _invalid("sequence attention backward Executor/state mismatch")
        if len(output_gradients) != 1:
            raise _invalid("sequence attention received an unexpected number of buffers")
        dy = output_gradients[0]
        if dy is None or not dy.is_cuda or dy.dtype != torch.float32 or dy.numel() != t * hq * d:
            raise _invalid("sequence attention buffer has an invalid size or Executor")
        qg_in, k_in, _, q, k, _, core, maxima, normalizers, v = state.intermediates
        L = _capi.lib()
        device = dy.device
        f32 = dict(dtype=torch.float32, device=device)
        dqg = torch.empty((t, hq, 2, d), **f32)
        dk = torch.empty((t, hkv, d), **f32)
        dv = torch.empty((t, hkv, d), **f32)
        dq_rope = torch.empty((t, hq, d), **f32)
        dk_rope = torch.empty((t, hkv, d), **f32)
        dc = torch.empty((t, hq, d), **f32)
        deltas = torch.empty((hq * t,), **f32)
        check(L.pluto_gqa_gate_bwd(_stream(), qg_in.data_ptr() + 2 * d, 2 * hq * d, 2 * d, _ptr(core),
                                   _ptr(dy), _ptr(dc), dqg.data_ptr() + 4 * d, 2 * hq * d, 2 * d,
                                   _ptr(deltas), 1, t, hq, d, int(p.round_to_bfloat16)))
        size = L.pluto_gqa_prefill_bwd_workspace_bytes(1, t, hq, d, 1) if self.tensor_core_backward else 0
        workspace = torch.empty((size,), dtype=torch.uint8, device=device) if size else None
        check(L.pluto_gqa_prefill_bwd(_stream(), _ptr(q), _ptr(k), _ptr(v), 1, hq * d, d, _ptr(dc),
                                      _ptr(maxima), _ptr(normalizers), _ptr(deltas), _ptr(dq_rope),
                                      _ptr(dk_rope), _ptr(dv), _ptr(workspace), size, 1, t, hq, hkv, d))
        for x, x_token, x_head, norm, grad, dx, heads in (
                (qg_in, 2 * hq * d, 2 * d, self.norms_[0], dq_rope, dqg, hq),
                (k_in, hkv * d, d, self.norms_[1], dk_rope, dk, hkv)):
            workspace, size = None, 0
            if norm.active():
                size = L.pluto_qk_prepare_bwd_workspace_bytes(1, t, heads, d)
                workspace = torch.empty((size,), dtype=torch.uint8, device=device)
            check(L.pluto_qk_prepare_bwd(_stream(), _ptr(x), x_token, x_head, _ptr(norm.value()),
                                         _ptr(grad), None, _ptr(dx), x_token, x_head,
                                         _ptr(norm.gradient()), _ptr(workspace), size, 1, t, heads, d,
                                         p.rotary_dim, p.rms_norm_epsilon, p.rope_theta,
                                         int(p.round_to_bfloat16)))
        return [dqg, dk, dv]


class DeltaNetLayer(Layer):
    """Single-token gated delta-net layer over a DeltaNetState (src/llm/layers/delta_net.h:20-60,
    .cc:38-110).  Inputs bf16 [1, QKV channels], [1, Hv*dv] (z), [1, Hv] (a), [1, Hv] (b); output
    bf16 [1, Hv*dv].  Weights fp32: convolution [channels, kernel], A_log [Hv], dt_bias [Hv], RMS
    multiplier [dv].  Inference only."""

    kMaximumDimension = 1048576

    def __init__(self, parameters, weights, state):
        self.parameters_ = parameters
        self.weights_ = weights
        self.cache_ = state

    @staticmethod
    def Create(parameters: DeltaNetParameters, convolution, a_log, dt_bias, norm) -> "DeltaNetLayer":
        p = parameters
        if min(p.key_heads, p.value_heads, p.key_head_dim, p.value_head_dim, p.conv_kernel_dim) <= 0:
            raise _invalid("DeltaNetLayer dimensions must be positive")
        key_width, value_width = p.key_heads * p.key_head_dim, p.value_heads * p.value_head_dim
        limit = DeltaNetLayer.kMaximumDimension
        if key_width > limit // 2 or value_width > limit or 2 * key_width + value_width > limit:
            raise _invalid("DeltaNetLayer activation exceeds the layer dimension limit")
        channels = 2 * key_width + value_width
        counts = [channels * p.conv_kernel_dim, p.value_heads, p.value_heads, p.value_head_dim]
        for weight, count in zip((convolution, a_log, dt_bias, norm), counts):
            if weight is None or not weight.is_cuda or weight.dtype != torch.float32 or weight.numel() != count:
                raise _invalid("DeltaNetLayer weight has incorrect FP32 size or Executor")
        return DeltaNetLayer(p, [convolution, a_log, dt_bias, norm], DeltaNetState.Create(p, convolution.device))

    def name(self) -> str:
        return "DeltaNetLayer"

    def output_type(self) -> DataType:
        return DataType.BF16

    def weights(self):
        return self.weights_

    def Reset(self) -> None:
        self.cache_.Reset()

    def fwd_impl(self, inputs, hooks) -> FwdResult:
        p = self.parameters_
        width = p.value_heads * p.value_head_dim
        channels = 2 * p.key_heads * p.key_head_dim + width
        _validate_bf16_inputs(inputs, [channels, width, p.value_heads, p.value_heads], "DeltaNetLayer")
        output = torch.empty((1, width), dtype=torch.bfloat16, device=inputs[0].device)
        self.cache_.Step(inputs[0].view(-1), inputs[1].view(p.value_heads, p.value_head_dim),
                         inputs[2].view(-1), inputs[3].view(-1), *self.weights_,
                         output.view(p.value_heads, p.value_head_dim))
        return FwdResult([output], BackwardState())

    def bwd_impl(self, output_gradients, state, hooks):
        raise _unimplemented("DeltaNetLayer supports cached inference only")


class SequenceDeltaNetLayer(Layer):
    """Full-sequence gated delta-net forward from a zero state
    (src/llm/layers/sequence_delta_net.h:20-67, .cc:396-480): causal depthwise convolution + SiLU,
    the recurrence, RMSNorm * weight * SiLU(z).  Inputs bf16 QKV [1,T,channels], Z [1,T,Hv*dv],
    A and B [1,T,Hv]; output bf16 [1,T,Hv*dv].  The reference caps T at 128 because it stores every
    intermediate state; here the forward recurrence is chunked, the backward keeps one state per
    64 tokens and recomputes inside a chunk, and any T runs.  Each of the four parameters is a
    BlockParameter (or a raw fp32 tensor = frozen); backward accumulates into active ones."""

    def __init__(self, parameters, owned, sequence_length):
        self.parameters_ = parameters
        self.parameters_owned_ = owned                    # convolution, A_log, dt_bias, norm
        self.weights_ = [p.value() for p in owned]
        self.sequence_length_ = sequence_length

    @staticmethod
    def Create(parameters: DeltaNetParameters, convolution, a_log, dt_bias, norm,
               sequence_length: int) -> "SequenceDeltaNetLayer":
        import math
        p = parameters
        if (sequence_length < 1 or p.key_heads < 1 or p.value_heads < 1 or p.value_heads % p.key_heads
                or p.key_head_dim < 1 or p.key_head_dim > 128 or p.value_head_dim < 1
                or p.value_head_dim > 256 or p.conv_kernel_dim < 1 or p.conv_kernel_dim > 32
                or not math.isfinite(p.rms_norm_epsilon) or p.rms_norm_epsilon <= 0):
            raise _invalid("unsupported SequenceDeltaNetLayer shape")
        channels = 2 * p.key_heads * p.key_head_dim + p.value_heads * p.value_head_dim
        counts = [channels * p.conv_kernel_dim, p.value_heads, p.value_heads, p.value_head_dim]
        owned = []
        for parameter, count in zip((convolution, a_log, dt_bias, norm), counts):
            weight = parameter.value() if isinstance(parameter, BlockParameter) else parameter
            if weight is None or weight.dtype != torch.float32:
                raise _invalid("DeltaNet parameters must be FP32")
            if not weight.is_cuda or weight.numel() != count:
                raise _invalid(f"DeltaNet parameter has {weight.numel() * 4} bytes; expected {count * 4}")
            owned.append(parameter if isinstance(parameter, BlockParameter) else BlockParameter(weight))
        _capi.lib()
        return SequenceDeltaNetLayer(p, owned, sequence_length)

    def name(self) -> str:
        return "SequenceDeltaNetLayer"

    def output_type(self) -> DataType:
        return DataType.BF16

    def weights(self):
        return self.weights_

    def fwd_impl(self, inputs, hooks) -> FwdResult:
        p, t = self.parameters_, self.sequence_length_
        width = p.value_heads * p.value_head_dim
        kq = p.key_heads * p.key_head_dim
        channels = 2 * kq + width
        if len(inputs) != 4:
            raise _invalid("DeltaNet expects four inputs on its Executor")
        _validate_bf16_inputs(inputs, [t * channels, t * width, t * p.value_heads, t * p.value_heads],
                              "SequenceDeltaNetLayer")
        L, rnd = _capi.lib(), int(p.round_to_bfloat16)
        device = inputs[0].device
        if not p.round_to_bfloat16:
            raise _unimplemented("sequence delta-net without bf16 rounding is not built")
        post = torch.empty((t, channels), dtype=torch.bfloat16, device=device)
        conv_state = torch.zeros((1, channels, p.conv_kernel_dim), dtype=torch.float32, device=device)
        check(L.pluto_gdn_conv_silu(_stream(), _ptr(inputs[0]), _ptr(self.weights_[0]), 1, 1, t,
                                    channels, p.conv_kernel_dim, rnd, _ptr(conv_state), _ptr(post), 1))
        g = torch.empty((t, p.value_heads), dtype=torch.float32, device=device)
        beta = torch.empty_like(g)
        check(L.pluto_gdn_gates(_stream(), _ptr(inputs[2]), _ptr(inputs[3]), _ptr(self.weights_[1]),
                                _ptr(self.weights_[2]), 1, t, p.value_heads, rnd, _ptr(g), _ptr(beta)))
        state = torch.zeros((1, p.value_heads, p.key_head_dim, p.value_head_dim), dtype=torch.float32,
                            device=device)
        core = torch.empty((t, width), dtype=torch.bfloat16, device=device)
        flat = post.view(-1)
        need = L.pluto_gdn_prefill_workspace_bytes(1, t, p.key_heads, p.value_heads, p.key_head_dim,
                                                   p.value_head_dim, 1)
        ws_ptr, ws_bytes = None, 0
        if need and channels % 8 == 0 and kq % 8 == 0:
            ws = _workspace(device, need + 256)
            ws_ptr = (ws.data_ptr() + 255) // 256 * 256
            ws_bytes = ws.numel() - (ws_ptr - ws.data_ptr())
        check(L.pluto_gdn_prefill(_stream(), _ptr(flat), _ptr(flat[kq:]), _ptr(flat[2 * kq:]), 1,
                                  _ptr(g), _ptr(beta), _ptr(state), _ptr(core), 1, 1, t, p.key_heads,
                                  p.value_heads, p.key_head_dim, p.value_head_dim, channels, channels,
                                  1, 1.0, rnd, ws_ptr, ws_bytes))
        output = torch.empty((t, width), dtype=torch.bfloat16, device=device)
        check(L.pluto_gdn_out_norm_gate(_stream(), _ptr(core), 1, _ptr(inputs[1]), 1,
                                        _ptr(self.weights_[3]), t * p.value_heads, p.value_head_dim,
                                        p.rms_norm_epsilon, rnd, 0, _ptr(output), 1))
        saved = BackwardState(intermediates=[inputs[0], inputs[1], inputs[2], inputs[3], post, core, state])
        return FwdResult([output], saved)

    def gradients(self):
        return [p.gradient() for p in self.parameters_owned_ if p.active()]

    def bwd_impl(self, output_gradients, state, hooks):
        # src/llm/layers/sequence_delta_net.cc:482-561
        p, t = self.parameters_, self.sequence_length_
        width = p.value_heads * p.value_head_dim
        kq = p.key_heads * p.key_head_dim
        channels = 2 * kq + width
        if len(output_gradients) != 1 or len(state.intermediates) != 7:
            raise _invalid("invalid DeltaNet backward state or gradient")
        dy = output_gradients[0]
        if dy is None or not dy.is_cuda or dy.dtype != torch.float32 or dy.numel() != t * width:
            raise _invalid("SequenceDeltaNetLayer requires batch-one buffers of the declared shape")
        qkv_in, z, a, b, post, core, _ = state.intermediates
        L, rnd = _capi.lib(), int(p.round_to_bfloat16)
        device = dy.device
        f32 = dict(dtype=torch.float32, device=device)
        conv_p, a_log_p, dt_bias_p, norm_p = self.parameters_owned_
        dqkv = torch.empty((t, channels), **f32)
        dz = torch.empty((t, width), **f32)
        da = torch.empty((t, p.value_heads), **f32)
        db = torch.empty((t, p.value_heads), **f32)
        dcore = torch.empty((t, width), **f32)
        dpost = torch.empty((t, channels), **f32)
        rows = t * p.value_heads
        ws, size = None, 0
        if norm_p.active():
            size = L.pluto_gdn_out_norm_gate_bwd_workspace_bytes(rows, p.value_head_dim)
            ws = torch.empty((size,), dtype=torch.uint8, device=device)
        check(L.pluto_gdn_out_norm_gate_bwd(_stream(), _ptr(core), 1, _ptr(z), 1, _ptr(norm_p.value()),
                                            _ptr(dy), _ptr(dcore), _ptr(dz), _ptr(norm_p.gradient()),
                                            _ptr(ws), size, rows, p.value_head_dim,
                                            p.rms_norm_epsilon, rnd))
        size = L.pluto_gdn_recurrence_bwd_workspace_bytes(1, t, p.key_heads, p.value_heads,
                                                          p.key_head_dim, p.value_head_dim)
        ws = torch.empty((size,), dtype=torch.uint8, device=device)
        flat, dflat = post.view(-1), dpost.view(-1)
        check(L.pluto_gdn_recurrence_bwd(
            _stream(), _ptr(flat), _ptr(flat[kq:]), _ptr(flat[2 * kq:]), 1, channels, channels,
            _ptr(a), _ptr(b), 1, _ptr(a_log_p.value()), _ptr(dt_bias_p.value()), _ptr(dcore),
            _ptr(dflat), _ptr(dflat[kq:]), channels, _ptr(dflat[2 * kq:]), channels, _ptr(da), _ptr(db),
            _ptr(a_log_p.gradient()), _ptr(dt_bias_p.gradient()), _ptr(ws), size, 1, t, p.key_heads,
            p.value_heads, p.key_head_dim, p.value_head_dim, rnd))
        check(L.pluto_gdn_conv_silu_bwd(_stream(), _ptr(qkv_in), 1, _ptr(conv_p.value()), _ptr(dpost),
                                        _ptr(dqkv), _ptr(conv_p.gradient()), 1, t, channels,
                                        p.conv_kernel_dim, rnd))
        return [dqkv, dz, da, db]


# =================================================================================================
# Imported projections (FullyConnectedLayer, frozen checkpoint form)
# =================================================================================================
class MatrixStorage(enum.Enum):
    """src/llm/layers/matrix_common.h:11."""
    kBFloat16 = 0
    kFloat32 = 1
    kFp8E4M3 = 2


def _matrix_element_bytes(storage: MatrixStorage) -> int:
    return {MatrixStorage.kBFloat16: 2, MatrixStorage.kFloat32: 4, MatrixStorage.kFp8E4M3: 1}[storage]


class FullyConnectedLayer(Layer):
    """The imported form of FullyConnectedLayer (src/llm/layers/fully_connected.h:36-49,
    .cc:267-341): a frozen, biasless [output_dim, input_dim] matrix shared with the checkpoint
    (bf16, fp32, or FP8 E4M3 bytes with fp32 128x128 block scales), bf16 activations in and out,
    no gradients; initialisation and backward are rejected.  The reference runs one token per
    call; `tokens` > 1 rows are accepted here and share one pass over the weights.

    The trainable form is DenseLayer below (same reference class, :343-520)."""

    kMaximumDimension = 1048576

    def __init__(self, weights, storage, input_dim, output_dim, scales):
        self.weights_ = [weights] + ([scales] if scales is not None else [])
        self.imported_storage_ = storage
        self.input_dim_, self.output_dim_ = input_dim, output_dim

    @staticmethod
    def Create(weights: torch.Tensor, storage: MatrixStorage, input_dim: int, output_dim: int,
               scales: Optional[torch.Tensor] = None) -> "FullyConnectedLayer":
        limit = FullyConnectedLayer.kMaximumDimension
        if input_dim <= 0 or input_dim > limit or output_dim <= 0 or output_dim > limit:
            raise _invalid("imported linear dimensions must be in [1, 1048576]")
        if not isinstance(storage, MatrixStorage):
            raise _invalid("unknown matrix storage")
        expected = input_dim * output_dim * _matrix_element_bytes(storage)
        if weights is None or not weights.is_cuda:
            raise _invalid("imported linear weights belong to a different Executor")
        _validate_buffer(weights, expected, "imported linear weights")
        if (storage == MatrixStorage.kFp8E4M3) != (scales is not None):
            raise _invalid("only FP8 linear weights require block scales")
        if scales is not None:
            if not scales.is_cuda:
                raise _invalid("imported linear block scales belong to a different Executor")
            _validate_buffer(scales, ((input_dim + 127) // 128) * ((output_dim + 127) // 128) * 4,
                             "imported linear block scales")
        _capi.lib()
        return FullyConnectedLayer(weights, storage, input_dim, output_dim, scales)

    def name(self) -> str:
        return "FullyConnectedLayer"

    def output_type(self) -> DataType:
        return DataType.BF16

    def input_dim(self) -> int:
        return self.input_dim_

    def output_dim(self) -> int:
        return self.output_dim_

    def weights(self):
        return self.weights_

    def input_types(self):
        return [ActivationType(DataType.BF16, (-2, 1, self.input_dim_))]

    def output_types(self):
        return [ActivationType(DataType.BF16, (-2, 1, self.output_dim_))]

    def InitializeIdentity(self, scale: float = 1.0):
        raise PlutoStatusError("FailedPrecondition", "imported linear weights are frozen", -1)

    def InitializeNormal(self, standard_deviation: float, seed: int):
        raise PlutoStatusError("FailedPrecondition", "imported linear weights are frozen", -1)

    def fwd_impl(self, inputs, hooks) -> FwdResult:
        if len(inputs) != 1 or inputs[0] is None or not inputs[0].is_cuda or \
                inputs[0].dtype != torch.bfloat16 or inputs[0].numel() == 0 or \
                inputs[0].numel() % self.input_dim_ != 0:
            raise _invalid("FullyConnectedLayer expects one BF16 activation of its input width")
        tokens = inputs[0].numel() // self.input_dim_
        output = torch.empty((tokens, self.output_dim_), dtype=torch.bfloat16, device=inputs[0].device)
        scales = self.weights_[1] if len(self.weights_) == 2 else None
        check(_capi.lib().pluto_linear_imported_fwd(
            _stream(), _ptr(self.weights_[0]), self.imported_storage_.value, _ptr(scales),
            _ptr(inputs[0]), _ptr(output), tokens, self.input_dim_, self.output_dim_))
        return FwdResult([output], BackwardState())

    def bwd_impl(self, output_gradients, state, hooks):
        raise _unimplemented("imported FullyConnectedLayer has no backward")


class DenseLayer(Layer):
    """The trainable form of FullyConnectedLayer (src/llm/layers/fully_connected.h:27-35,
    .cc:343-520): fp32 master matrix [input_dim, output_dim] and bias, fp32 gradients (overwritten
    by every backward), activations bf16 (DataType.BF16) or fp32 (DataType.FP16 compute policy),
    MMA operands cast to bf16 / fp16 with fp32 accumulation.  Runs as tcgen05 GEMMs."""

    def __init__(self, input_dim, output_dim, data_type, sequence_length, device):
        self.input_dim_, self.output_dim_ = input_dim, output_dim
        self.output_type_, self.sequence_length_ = data_type, sequence_length
        f32 = dict(dtype=torch.float32, device=device)
        self.weights_ = [torch.zeros((input_dim, output_dim), **f32), torch.zeros((output_dim,), **f32)]
        self.gradients_ = [torch.zeros((input_dim, output_dim), **f32), torch.zeros((output_dim,), **f32)]

    @staticmethod
    def Create(input_dim: int, output_dim: Optional[int] = None, data_type: DataType = DataType.BF16,
               sequence_length: int = 1, device="cuda") -> "DenseLayer":
        output_dim = input_dim if output_dim is None else output_dim
        if sequence_length <= 0:
            raise _invalid("sequence_length must be positive")
        if data_type not in (DataType.FP16, DataType.BF16):
            raise _unimplemented("dense layers compute in FP16 or BF16")
        if input_dim <= 0:
            raise _invalid("input_dim must be positive")
        if output_dim <= 0:
            raise _invalid("output_dim must be positive")
        _capi.lib()
        return DenseLayer(input_dim, output_dim, data_type, sequence_length, device)

    def name(self) -> str:
        return "FullyConnectedLayer"

    def output_type(self) -> DataType:
        return self.output_type_

    def input_dim(self) -> int:
        return self.input_dim_

    def output_dim(self) -> int:
        return self.output_dim_

    def weights(self):
        return self.weights_

    def gradients(self):
        return self.gradients_

    def input_types(self):
        return [ActivationType(self.output_type_, (-2, self.sequence_length_, self.input_dim_))]

    def output_types(self):
        return [ActivationType(self.output_type_, (-2, self.sequence_length_, self.output_dim_))]

    def InitializeIdentity(self, scale: float = 1.0) -> None:
        matrix = torch.zeros((self.input_dim_, self.output_dim_), dtype=torch.float32)
        n = min(self.input_dim_, self.output_dim_)
        matrix[torch.arange(n), torch.arange(n)] = scale
        self.weights_[0].copy_(matrix)
        self.weights_[1].zero_()

    def InitializeNormal(self, standard_deviation: float, seed: int) -> None:
        if not standard_deviation > 0.0:
            raise _invalid("dense initialization standard deviation must be positive")
        gen = torch.Generator().manual_seed(seed)
        self.weights_[0].copy_(torch.randn((self.input_dim_, self.output_dim_), generator=gen)
                               * standard_deviation)

    def _workspace(self, rows, device):
        need = _capi.lib().pluto_dense_workspace_bytes(rows, self.input_dim_, self.output_dim_)
        ws = torch.empty((need + 256,), dtype=torch.uint8, device=device)
        ptr = (ws.data_ptr() + 255) // 256 * 256
        return ws, ptr, need

    def fwd_impl(self, inputs, hooks) -> FwdResult:
        if len(inputs) != 1:
            raise _invalid("FullyConnectedLayer fwd expects one input")
        rows = _activation_rows(inputs[0], self.input_dim_, self.output_type_, "dense input")
        dtype = activation_torch_dtype(self.output_type_)
        output = torch.empty((rows, self.output_dim_), dtype=dtype, device=inputs[0].device)
        ws, ptr, need = self._workspace(rows, inputs[0].device)
        check(_capi.lib().pluto_dense_fwd(
            _stream(), _ptr(inputs[0]), 1 if self.output_type_ == DataType.BF16 else 0,
            _ptr(self.weights_[0]), _ptr(self.weights_[1]), _ptr(output), rows, self.input_dim_,
            self.output_dim_, ptr, need))
        return FwdResult([output], BackwardState(intermediates=[inputs[0]]))

    def bwd_impl(self, output_gradients, state, hooks):
        if len(output_gradients) != 1 or len(state.intermediates) != 1:
            raise _invalid("FullyConnectedLayer bwd received an incompatible gradient or state")
        dy = output_gradients[0]
        if dy.dtype != torch.float32:
            raise _invalid("dense output gradient must be FP32")
        rows = _activation_rows(dy, self.output_dim_, DataType.FP32, "dense output gradient")
        x = state.intermediates[0]
        element = 2 if self.output_type_ == DataType.BF16 else 4
        _validate_buffer(x, rows * self.input_dim_ * element, "dense saved input")
        dx = torch.empty((rows, self.input_dim_), dtype=torch.float32, device=dy.device)
        ws, ptr, need = self._workspace(rows, dy.device)
        check(_capi.lib().pluto_dense_bwd(
            _stream(), _ptr(x), 1 if self.output_type_ == DataType.BF16 else 0, _ptr(self.weights_[0]),
            _ptr(dy), _ptr(dx), _ptr(self.gradients_[0]), _ptr(self.gradients_[1]), rows,
            self.input_dim_, self.output_dim_, ptr, need))
        return [dx]


def DequantizeMatrix(input: torch.Tensor, storage: MatrixStorage, scales: Optional[torch.Tensor],
                     rows: int, cols: int) -> torch.Tensor:
    """src/llm/layers/block_training.cc:281-319: an imported matrix as resident bf16 storage.
    bf16 inputs are shared, fp32 and FP8 (with block scales) are converted."""
    if rows <= 0 or cols <= 0 or rows > 1048576 or cols > 1048576:
        raise _invalid("invalid imported matrix shape")
    if not isinstance(storage, MatrixStorage):
        raise _invalid("unknown matrix storage")
    if input is None or not input.is_cuda or \
            input.numel() * input.element_size() != rows * cols * _matrix_element_bytes(storage):
        raise _invalid("block training requires the owning executor, exact dimensions and batch size one")
    if storage == MatrixStorage.kFp8E4M3:
        if scales is None:
            raise _invalid("FP8 matrix requires scales")
        if not scales.is_cuda or scales.numel() * scales.element_size() != \
                ((rows + 127) // 128) * ((cols + 127) // 128) * 4:
            raise _invalid("block training requires the owning executor, exact dimensions and batch size one")
    elif scales is not None:
        raise _invalid("non-FP8 matrix must not have scales")
    if storage == MatrixStorage.kBFloat16:
        return input
    output = torch.empty((rows, cols), dtype=torch.bfloat16, device=input.device)
    check(_capi.lib().pluto_dequantize_matrix(_stream(), _ptr(input), storage.value, _ptr(scales),
                                              _ptr(output), rows, cols))
    return output


class BlockLinearLayer(Layer):
    """Bias-free [output, input] bf16 matrix with bf16 forward and fp32 backward
    (src/llm/layers/block_training.h:49-83, .cc:321-399).  A frozen weight still propagates input
    gradients but never accumulates a weight gradient; an active BlockParameter's gradient is
    accumulated into.  One sample of sequence_length tokens."""

    def __init__(self, weight, input_dim, output_dim, sequence_length, output_float32):
        self.parameter_ = weight
        self.weights_ = [weight.value()]
        self.input_dim_, self.output_dim_ = input_dim, output_dim
        self.sequence_length_, self.output_float32_ = sequence_length, output_float32

    @staticmethod
    def Create(weight: BlockParameter, input_dim: int, output_dim: int, sequence_length: int,
               output_float32: bool = False) -> "BlockLinearLayer":
        if (weight is None or input_dim <= 0 or output_dim <= 0 or sequence_length <= 0
                or input_dim > 1048576 or output_dim > 1048576
                or sequence_length * input_dim > 2 ** 31 - 1 or sequence_length * output_dim > 2 ** 31 - 1
                or weight.value().dtype != torch.bfloat16 or not weight.value().is_cuda
                or weight.value().numel() != input_dim * output_dim):
            raise _invalid("invalid block parameter dimensions, storage or executor")
        _capi.lib()
        return BlockLinearLayer(weight, input_dim, output_dim, sequence_length, output_float32)

    def name(self) -> str:
        return "BlockLinearLayer"

    def output_type(self) -> DataType:
        return DataType.FP32 if self.output_float32_ else DataType.BF16

    def weights(self):
        return self.weights_

    def gradients(self):
        return [self.parameter_.gradient()] if self.parameter_.active() else []

    def input_types(self):
        return [ActivationType(DataType.BF16, (-2, self.sequence_length_, self.input_dim_))]

    def output_types(self):
        return [ActivationType(self.output_type(), (-2, self.sequence_length_, self.output_dim_))]

    def _check(self, buffer, elements, element_size):
        if buffer is None or not buffer.is_cuda or buffer.numel() * buffer.element_size() != elements * element_size:
            raise _invalid("block training requires the owning executor, exact dimensions and batch size one")

    def _workspace(self, device):
        need = _capi.lib().pluto_block_linear_workspace_bytes(self.sequence_length_, self.input_dim_,
                                                              self.output_dim_)
        ws = torch.empty((need + 256,), dtype=torch.uint8, device=device)
        return ws, (ws.data_ptr() + 255) // 256 * 256, need

    def fwd_impl(self, inputs, hooks) -> FwdResult:
        if len(inputs) != 1:
            raise _invalid("linear requires one input")
        t = self.sequence_length_
        self._check(inputs[0], t * self.input_dim_, 2)
        output = torch.empty((t, self.output_dim_), device=inputs[0].device,
                             dtype=torch.float32 if self.output_float32_ else torch.bfloat16)
        ws, ptr, need = self._workspace(inputs[0].device)
        check(_capi.lib().pluto_block_linear_fwd(
            _stream(), _ptr(self.weights_[0]), _ptr(inputs[0]), _ptr(output),
            0 if self.output_float32_ else 1, t, self.input_dim_, self.output_dim_, ptr, need))
        return FwdResult([output], BackwardState(intermediates=[inputs[0]]))

    def bwd_impl(self, output_gradients, state, hooks):
        if len(output_gradients) != 1 or len(state.intermediates) != 1:
            raise _invalid("invalid linear backward state/gradient")
        t = self.sequence_length_
        dy = output_gradients[0]
        self._check(dy, t * self.output_dim_, 4)
        self._check(state.intermediates[0], t * self.input_dim_, 2)
        dx = torch.empty((t, self.input_dim_), dtype=torch.float32, device=dy.device)
        ws, ptr, need = self._workspace(dy.device)
        check(_capi.lib().pluto_block_linear_bwd(
            _stream(), _ptr(self.weights_[0]), _ptr(state.intermediates[0]), _ptr(dy), _ptr(dx),
            _ptr(self.parameter_.gradient()), t, self.input_dim_, self.output_dim_, ptr, need))
        return [dx]
