"""Every one of the 2^32 FP32 bit patterns through e5ma_cast to E5M2, E4M3, BF16 and FP16, compared with
the oracle bit for bit (the reference's tests/test_e5m2effma.cu:194-213 sweeps the same space against
its own definitions).  Inputs are generated on the GPU, 2^26 patterns per call; E5MA_TEST_QUICK=1 visits
every 16th block only."""
import os

import numpy as np
import pytest

import oracle as orc
from harness import BF16, E4M3, E5M2, FP16, FP32

pytestmark = pytest.mark.gpu
BLOCK = 1 << 26


@pytest.mark.parametrize("ddt", [E5M2, E4M3, BF16, FP16])
def test_all_fp32_patterns(ddt):
    import torch
    from e5m2effma_b200 import capi
    dev = torch.device("cuda", 0)
    es = orc.esize(ddt)
    src = torch.empty(BLOCK, dtype=torch.int32, device=dev)
    dst = torch.empty(BLOCK * es, dtype=torch.uint8, device=dev)
    base = torch.arange(BLOCK, dtype=torch.int64, device=dev)
    host = np.arange(BLOCK, dtype=np.uint32)
    step = 16 if os.environ.get("E5MA_TEST_QUICK") == "1" else 1
    stream = torch.cuda.current_stream().cuda_stream
    for blk in range(0, 64, step):
        u = base + blk * BLOCK                       # the bit patterns of this block as unsigned values
        src.copy_(torch.where(u >= 2 ** 31, u - 2 ** 32, u).to(torch.int32))
        st = capi.cast(capi.tensor(src.data_ptr(), FP32), capi.tensor(dst.data_ptr(), ddt), BLOCK, stream)
        assert st == capi.OK, capi.last_error()
        got = dst.cpu().numpy().view(orc.NP_STORAGE[ddt])
        exp = orc.encode(ddt, (host + np.uint32(blk * BLOCK)).view(np.float32))
        bad = np.flatnonzero(got != exp)
        assert bad.size == 0, (f"block {blk}: {bad.size} mismatches, first input {int(host[bad[0]]) + blk * BLOCK:#010x} "
                               f"got {int(got[bad[0]]):#x} expected {int(exp[bad[0]]):#x}")
