"""The benchmark's CPU reference arm builds its inputs without loading the library: same seeds, same torch
generator calls, but quantised by the oracle's encoder instead of e5ma_cast.  Both routes must give the same bytes,
or the two arms of the benchmark would not run on identical inputs."""
import numpy as np
import pytest

import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["c1", "c2_bf16", "c3n8", "c4"])
def test_oracle_quantised_inputs_equal_library_quantised_inputs(name):
    import torch
    from e5m2effma_b200 import workloads
    dev = torch.device("cuda", 0)

    def cpu_quantizer(x32, dtype, scale=None):
        codes = orc.encode(dtype, x32.detach().float().cpu().contiguous().numpy().reshape(-1), 1.0 if scale is None else float(scale))
        return torch.from_numpy(codes.reshape(tuple(x32.shape))).to(x32.device)

    a = workloads.make(name, dev, 8)
    workloads.QUANTIZER = cpu_quantizer
    try:
        b = workloads.make(name, dev, 8)
    finally:
        workloads.QUANTIZER = None
    for field in ("A", "B", "sa", "sb", "bias"):
        x, y = getattr(a, field), getattr(b, field)
        assert (x is None) == (y is None)
        if x is not None:
            assert torch.equal(x.view(torch.uint8), y.view(torch.uint8)), field
