"""The allocation-free attention-backward entry point, called through its exported C symbol.

Some callers of these kernels cannot allocate device memory at the moment they need a backward
pass: code replaying a frozen region, hosts with a strict memory accountant, latency-critical
serving loops, C programs without PyTorch's allocator. ``ob_flash_attn_bwd_noalloc`` serves them
by keeping its scratch (fp32 dQ accumulators and the per-row delta) in a static device array
inside the library. This test checks that it computes what the regular, allocating entry point
computes, twice in a row (the second call starts from a dirty scratch array), and that it refuses
problems larger than the built-in scratch.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from ohara_b200 import build_ext
    from ohara_b200.ops._ext import ext

    ext()  # make sure the shared object (and libtorch, which it links) is loaded
    lib = ctypes.CDLL(str(build_ext.ext_path()))
    fn = lib.ob_flash_attn_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = (
        [ctypes.c_void_p] * 9
        + [ctypes.c_int] * 7
        + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    )
    return fn


def _call(fn, q, k, v, out, dout, lse, causal, scale):
    b, t, h, d = q.shape
    s, hk = k.shape[1], k.shape[2]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
            lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), b, t, s, h, hk, d,
            int(causal), scale, stream, None, err, len(err))
    return rc, err.value.decode(), (dq, dk, dv)


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-12)


@pytest.mark.parametrize("shape", [(2, 256, 256, 4, 2, 128, True), (1, 200, 328, 4, 4, 64, True)])
def test_noalloc_backward_matches_allocating_entry_point_twice(shape):
    from ohara_b200.ops._ext import ext

    b, t, s, h, hk, d, causal = shape
    fn = _library()
    C = ext()
    scale = 1.0 / math.sqrt(d)
    for attempt in range(2):  # the second pass runs over the first pass's leftovers
        torch.manual_seed(attempt)
        q = torch.randn(b, t, h, d, device="cuda").bfloat16()
        k = torch.randn(b, s, hk, d, device="cuda").bfloat16()
        v = torch.randn(b, s, hk, d, device="cuda").bfloat16()
        dout = torch.randn(b, t, h, d, device="cuda").bfloat16()
        out, lse = C.flash_attn_fwd(q, k, v, causal, scale)
        ref_dq, ref_dk, ref_dv = C.flash_attn_bwd(dout, q, k, v, out, lse, causal, scale)
        rc, message, (dq, dk, dv) = _call(fn, q, k, v, out, dout, lse, causal, scale)
        assert rc == 0, message
        torch.cuda.synchronize()
        assert _rel(dq, ref_dq) < 2e-2
        assert _rel(dk, ref_dk) < 2e-2
        assert _rel(dv, ref_dv) < 2e-2
    assert C.status(True)[0] == 0


def test_noalloc_rejects_problems_beyond_the_scratch():
    fn = _library()
    # 4 * 2048 * 16 * 128 = 16 Mi dQ elements: twice what the built-in scratch holds. The size
    # check runs before anything touches the tensors, so small placeholders are enough here.
    dummy = torch.zeros(16, device="cuda", dtype=torch.bfloat16)
    lse = torch.zeros(16, device="cuda")
    err = ctypes.create_string_buffer(256)
    rc = fn(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
            dummy.data_ptr(), lse.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
            4, 2048, 2048, 16, 16, 128, 1, 0.1, None, None, err, len(err))
    assert rc == -2
    assert b"scratch" in err.value
    rc = fn(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
            dummy.data_ptr(), lse.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
            1, 128, 128, 3, 2, 128, 1, 0.1, None, None, err, len(err))
    assert rc == -1
