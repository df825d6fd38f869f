"""The torch-facing wrappers (the reference binding's matmul / cast / adam_step, binds/python/csrc/
e5m2effma_torch.cpp:127-274) refuse host tensors with the binding's own errors: there is no CPU path to fall
back to.  Checks that precede the device check (rank, operand dtypes) are exercised too."""
import pytest
import torch

from e5m2effma_b200 import functional as F


def fp8(shape, dtype=torch.float8_e5m2):
    return torch.zeros(shape, dtype=torch.uint8).view(dtype)


def test_matmul_argument_checks_and_no_cpu_path():
    with pytest.raises(ValueError, match="2-D"):
        F.matmul(torch.zeros(16, dtype=torch.bfloat16), torch.zeros(16, 16, dtype=torch.bfloat16))
    with pytest.raises(TypeError, match="float8_e5m2, float8_e4m3fn, bfloat16 or float32"):
        F.matmul(torch.zeros(16, 16, dtype=torch.float16), torch.zeros(16, 16, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="CUDA tensor is required"):
        F.matmul(fp8((16, 16)), fp8((16, 16), torch.float8_e4m3fn))


def test_cast_and_adam_have_no_cpu_path():
    with pytest.raises(ValueError, match="x must be a CUDA tensor"):
        F.cast(torch.zeros(8), torch.float8_e5m2)
    p = torch.zeros(8)
    with pytest.raises(ValueError, match="param must be a CUDA tensor"):
        F.adam_step(p, torch.zeros(8), torch.zeros(8), torch.zeros(8), lr=1e-3, step=1)
