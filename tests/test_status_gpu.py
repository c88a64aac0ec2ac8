"""Failure reporting of device-side waits: a wait on a peer flag that nothing ever sets runs out
after its clock limit (about a second), the kernel records the reason in the status word and
returns, the host turns that into an exception, and the CUDA context stays usable (GPU)."""
import time
from ctypes import c_int, c_uint

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_wait_runs_out_with_a_status_and_the_context_survives():
    from allie_b200.ops import _lib
    from allie_b200.ops._lib import ptr, stream_ptr

    lib = _lib.cuda()
    flags = torch.zeros(4 * 32, dtype=torch.int32, device="cuda")       # phase slots no peer will write
    st = _lib.status_word()
    st.zero_()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    assert lib.ab_nvl_wait(ptr(flags), c_int(0), c_int(1), c_uint(1), ptr(st), stream_ptr()) == 0
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.2 < waited < 10, waited
    with pytest.raises(RuntimeError, match="peer"):
        _lib.check_status()
    assert int(st[0]) == 0                                               # reading the status clears it
    x = torch.ones(1024, device="cuda")
    assert float(x.sum()) == 1024.0                                      # the context still works
    flags[0] = 1                                                         # the "peer" has signalled epoch 1
    t0 = time.perf_counter()
    assert lib.ab_nvl_wait(ptr(flags), c_int(0), c_int(1), c_uint(1), ptr(st), stream_ptr()) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.2
    _lib.check_status()
