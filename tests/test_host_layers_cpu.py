"""Host-side layer objects: factory validation and state checks that the reference performs
before touching the GPU (attention_test.cc:549-626, key_value_cache_test.cc:37-133,
cached_attention_ops_test.cc:505-636)."""
import pytest
import torch

from pluto_b200 import PlutoStatusError
from pluto_b200.layers import (AttentionLayer, BackwardState, DataType, DeltaNetParameters,
                               DeltaNetState, FullAttentionParameters, KeyValueCache,
                               ValidateCachedAttention)


def code_of(fn, *args, **kwargs):
    with pytest.raises(PlutoStatusError) as info:
        fn(*args, **kwargs)
    return info.value.code, info.value.message


def test_attention_create_validation(engine):
    assert code_of(AttentionLayer.Create, 8, 2, 32, DataType.FP8)[0] == "Unimplemented"
    assert code_of(AttentionLayer.Create, 0, 2, 32, DataType.FP16)[0] == "InvalidArgument"
    assert "divisible by num_heads" in code_of(AttentionLayer.Create, 8, 3, 32, DataType.BF16)[1]
    layer = AttentionLayer.Create(17, 2, 32, DataType.BF16)
    assert layer.name() == "AttentionLayer"
    assert layer.input_types()[0].dimensions == (-2, 17, 96)
    assert layer.output_types()[0].dimensions == (-2, 17, 32)
    assert layer.input_types()[0].data_type == DataType.BF16
    assert AttentionLayer.Create(1, 2, 32, DataType.FP16).input_types()[0].data_type == DataType.FP32
    assert layer.weights() == [] and layer.gradients() == []


def test_backward_rejects_foreign_state(engine):
    a = AttentionLayer.Create(4, 2, 32, DataType.FP16)
    b = AttentionLayer.Create(4, 2, 32, DataType.FP16)
    state = BackwardState(layer=b, intermediates=[torch.zeros(1)] * 4)
    assert code_of(a.bwd, [torch.zeros(4, 32)], state)[0] == "InvalidArgument"
    assert code_of(a.bwd, [torch.zeros(4, 32)], BackwardState())[0] == "InvalidArgument"


def test_forward_rejects_bad_inputs_before_launch(engine):
    layer = AttentionLayer.Create(4, 2, 32, DataType.FP16)
    assert "expects packed Q/K/V" in code_of(layer.fwd, [])[1]
    # CPU tensor stands for "a buffer of another Executor"
    assert code_of(layer.fwd, [torch.zeros(4, 96)])[0] == "InvalidArgument"


def test_key_value_cache_counter():
    assert code_of(KeyValueCache.Create, 0, 1, 4, torch.float32, "cpu")[0] == "InvalidArgument"
    cache = KeyValueCache.Create(2, 1, 4, torch.float32, "cpu")
    assert (cache.capacity(), cache.key_value_heads(), cache.head_dim(), cache.position()) == (2, 1, 4, 0)
    cache.Advance()
    cache.Advance()
    assert code_of(cache.Advance)[0] == "ResourceExhausted"
    assert cache.position() == 2
    cache.keys()[0, 0, 0] = 3.0
    cache.Reset()
    assert cache.position() == 0 and cache.keys()[0, 0, 0] == 3.0  # Reset does not clear


def test_validate_cached_attention():
    good = FullAttentionParameters(query_heads=4, key_value_heads=2, head_dim=8, rotary_dim=4, capacity=6)
    cache = KeyValueCache.Create(6, 2, 8, torch.float32, "cpu")
    ValidateCachedAttention(good, cache)
    for change in (dict(query_heads=3), dict(head_dim=257), dict(rotary_dim=3), dict(rotary_dim=10),
                   dict(rope_theta=float("inf")), dict(rms_norm_epsilon=0.0), dict(capacity=0)):
        bad = FullAttentionParameters(**{**good.__dict__, **change})
        assert code_of(ValidateCachedAttention, bad, cache)[0] == "InvalidArgument"
    other = KeyValueCache.Create(7, 2, 8, torch.float32, "cpu")
    assert "does not match" in code_of(ValidateCachedAttention, good, other)[1]


def test_delta_net_create_validation(engine):
    for change in (dict(key_heads=0), dict(value_heads=5, key_heads=2), dict(key_head_dim=129),
                   dict(value_head_dim=257), dict(conv_kernel_dim=33), dict(rms_norm_epsilon=-1.0)):
        bad = DeltaNetParameters(**{**DeltaNetParameters().__dict__, **change})
        assert code_of(DeltaNetState.Create, bad, "cpu")[0] == "InvalidArgument"
