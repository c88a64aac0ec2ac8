"""The allocation-free attention backward (``ab_attn_bwd_static``), called through its exported C
symbol, against the regular entry point.

Some embedders of the kernel library cannot call cudaMalloc where they run attention backward (a
process whose device memory is owned by another allocator, a plugin whose host lends it only
streams and buffers, a latency-critical serving loop).  For them the library keeps the kernel's scratch in a static device array.  This
test checks that the variant returns what the regular entry returns, twice in a row (the scratch
is shared between calls and must not leak state from one into the next), and that oversize
problems are rejected instead of overrunning the array.  It is collected last on purpose.
"""
from ctypes import c_float, c_int, c_uint, c_ulonglong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, qkv, out, lse, dout, dqkv, B, T, H, hd, status):
    fn = lib.ab_attn_bwd_static
    fn.restype = c_int
    return fn(c_void_p(qkv.data_ptr()), c_void_p(out.data_ptr()), c_void_p(lse.data_ptr()),
              c_void_p(dout.data_ptr()), c_void_p(dqkv.data_ptr()), c_void_p(0), c_int(B), c_int(T),
              c_int(H), c_int(hd), c_float(1.0 / hd ** 0.5), c_ulonglong(0), c_uint(0), c_uint(0),
              c_void_p(status.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_attention_backward_matches_regular_entry():
    from allie_b200.ops import _lib
    from allie_b200.ops.attention import attention_bwd, attention_fwd

    lib = _lib.cuda()
    dev = "cuda"
    status = _lib.status_word()
    # two head sizes, a sequence length that is not a multiple of the 128-row tile, and a problem
    # that uses the static array to its last row (B * H * T == AB_ATTN_STATIC_MAX_ROWS)
    for call, (B, T, H, hd) in enumerate([(2, 256, 3, 64), (1, 384, 2, 128), (3, 200, 2, 64), (128, 512, 16, 64)]):
        assert B * H * T <= 1 << 20
        torch.manual_seed(call)
        d = H * hd
        qkv = (torch.randn(B * T, 3 * d, device=dev) * 0.6).bfloat16()
        out = torch.zeros(B * T, d, device=dev, dtype=torch.bfloat16)
        lse = torch.zeros(B, H, T, device=dev)
        attention_fwd(qkv, out, lse, B, T, H, hd, 0.0, 0, 0)
        dout = (torch.randn(B * T, d, device=dev) * 0.5).bfloat16()
        want = torch.zeros(B * T, 3 * d, device=dev, dtype=torch.bfloat16)
        attention_bwd(qkv, out, lse, dout, want, torch.zeros(B, H, T, device=dev), B, T, H, hd, 0.0, 0, 0)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call_static(lib, qkv, out, lse, dout, got, B, T, H, hd, status)
        torch.cuda.synchronize()
        assert rc == 0
        # neither through torch's allocator nor behind its back (a raw cudaMalloc inside the
        # library would show up as less free device memory); the very first call of a process may
        # load the kernels' code lazily, which is not an allocation of this entry point
        assert torch.cuda.memory_allocated() == before
        if call > 0:
            assert torch.cuda.mem_get_info()[0] >= free_before
        _lib.check_status()
        # same kernels, same inputs: the tolerance of the other attention tests is more than enough
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(got, want)


def test_static_scratch_rejects_oversize():
    from allie_b200.ops import _lib

    lib = _lib.cuda()
    t = torch.zeros(8, device="cuda")
    rc = _call_static(lib, t, t, t, t, t, 4096, 512, 16, 64, _lib.status_word())   # 32 Mi rows > limit
    assert rc == -10
