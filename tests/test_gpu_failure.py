"""Device-side failure detection: a wait on a flag that nothing sets runs out, the kernel records a
status code and returns, and the CUDA context stays usable.  No fault, trap or hang is provoked."""
import time

import pytest
import torch

from tinyinfinitrain_b200._lib import C
from tinyinfinitrain_b200.parallel.health import PeerFailure, check_device_status

pytestmark = pytest.mark.gpu


def test_barrier_wait_times_out_with_status_and_context_survives():
    assert C.status_read(True) == 0
    # two "ranks" whose signal pads are plain local buffers; rank 1 does not exist, so its slot is never written
    pad0 = torch.zeros(8 * 16, dtype=torch.int32, device="cuda")
    pad1 = torch.zeros(8 * 16, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.time()
    C.comm_barrier([pad0.data_ptr(), pad1.data_ptr()], 0, 0, epoch, 0.25)   # 0.25 s budget
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert int(epoch.item()) == 1
    assert int(pad1[0].item()) == 1            # this rank did signal its peer
    with pytest.raises(PeerFailure):
        check_device_status()
    assert C.status_read(True) == 0            # cleared
    # the context is intact: run a tensor-core GEMM afterwards
    a = torch.randn(128, 64, device="cuda").bfloat16()
    out = C.gemm(a, a)[0]
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), a.float() @ a.float().t(), atol=0.5, rtol=2e-2)
    assert C.status_read(True) == 0
