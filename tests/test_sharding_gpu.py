"""The local half of the head all-gather on the GPU: pluto_interleave_heads against a torch
permute, on the 16-byte vector path and on the byte path."""
import pytest
import torch

from pluto_b200 import _capi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ranks,rows,cols,dtype", [(8, 8192, 5 * 128, torch.bfloat16), (2, 64, 40 * 128, torch.bfloat16),
                                                   (4, 33, 7, torch.bfloat16), (3, 5, 3, torch.float32),
                                                   (2, 1, 1, torch.uint8)])
def test_interleave_heads_matches_permute(ranks, rows, cols, dtype):
    if dtype == torch.uint8:
        gathered = torch.randint(0, 255, (ranks, rows, cols), dtype=dtype, device="cuda")
    else:
        gathered = torch.randn(ranks, rows, cols, device="cuda").to(dtype)
    out = torch.zeros(rows, ranks * cols, dtype=dtype, device="cuda")
    _capi.check(_capi.lib().pluto_interleave_heads(torch.cuda.current_stream().cuda_stream, gathered.data_ptr(),
                                                   out.data_ptr(), ranks, rows, cols * gathered.element_size()))
    want = gathered.permute(1, 0, 2).reshape(rows, ranks * cols)
    assert torch.equal(out, want)


def test_allgather_heads_rejects_a_missing_communicator():
    x = torch.zeros(16, device="cuda")
    with pytest.raises(_capi.PlutoStatusError) as info:
        _capi.check(_capi.lib().pluto_allgather_heads(torch.cuda.current_stream().cuda_stream, None, x.data_ptr(),
                                                      x.data_ptr(), x.data_ptr(), 2, 1, 8))
    assert info.value.code == "InvalidArgument"
