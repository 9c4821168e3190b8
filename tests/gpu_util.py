"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def to_device_bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def near(actual, expected, absolute, relative):
    """VectorsNear of the reference tests (reference_test_util.h:151-174)."""
    actual, expected = np.asarray(actual, np.float64), np.asarray(expected, np.float64)
    tol = absolute + relative * np.maximum(np.abs(actual), np.abs(expected))
    return bool(np.all(np.abs(actual - expected) <= tol))
