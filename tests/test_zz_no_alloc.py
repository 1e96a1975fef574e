"""The entry point that allocates nothing: decode attention with its scratch inside the library.

Some programs that link this library may not call cudaMalloc where they call us (a plug-in
inside another program's real-time loop, a host that gave all device memory to one arena).
For them ``dk_attention_decode_static`` keeps the partial results of the split-key kernel
in an 8 MiB array that is part of the library image.  Here it is called through its exported
C symbol, twice in a row with different requests (the array keeps the first call's contents
when the second one starts), and compared with the ordinary entry point, whose scratch the
caller allocates.  This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
STATIC_FLOATS = 2 * 1024 * 1024


def entry_point():
    from delta_b200.kernels import lib
    l = lib.load()
    fn = l.dk_attention_decode_static
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(lib.AttnParams), C.c_void_p]
    return l, fn


def test_static_scratch_gives_the_same_attention_twice_in_a_row():
    from delta_b200.kernels import ops
    from test_gpu_kernels import PagedCase
    l, static = entry_point()
    stream = torch.cuda.current_stream().cuda_stream
    H, KV, hd, ps = 32, 4, 128, 16
    for call, (seq_lens, splits, seed) in enumerate([([700, 64, 1, 333, 1000, 17, 256, 90], 9, 1),
                                                     ([129, 500, 2, 65], 16, 2)]):
        case = PagedCase(torch.bfloat16, H, KV, hd, ps, seq_lens, [1] * len(seq_lens), seed=seed)
        ref, ref_lse, _ = case.reference()
        # the ordinary entry point, scratch allocated by the caller
        want = torch.zeros(case.T, H * hd, dtype=torch.bfloat16, device=DEV)
        want_lse = torch.zeros(case.T, H, device=DEV)
        scratch = torch.empty(ops.attention_decode_scratch_floats(case.T, H, hd, splits), device=DEV)
        ops.attention_decode(case.params(want, lse=want_lse, scratch=scratch, splits=splits))
        # the entry point without allocation: no scratch is passed
        got = torch.zeros_like(want)
        got_lse = torch.zeros_like(want_lse)
        p = case.params(got, lse=got_lse, splits=splits)
        assert not p.scratch
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = static(C.byref(p), stream)
        assert rc == 0, l.dk_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if call > 0:    # the driver's own count of free bytes too (the first call may load the kernel's code)
            assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2), f"call {call}"
        assert torch.equal(got, want), f"call {call}: the same kernels in the same order give the same bits"
        assert torch.allclose(got_lse, want_lse, atol=2e-2, rtol=1e-3)
        assert torch.allclose(got.float().cpu(), ref, atol=2e-2, rtol=2e-2)


def test_static_scratch_refuses_what_does_not_fit():
    from delta_b200.kernels import ops
    from test_gpu_kernels import PagedCase
    l, static = entry_point()
    H, KV, hd, ps = 32, 4, 128, 16
    rows = 40
    splits = 16
    assert ops.attention_decode_scratch_floats(rows, H, hd, splits) > STATIC_FLOATS
    case = PagedCase(torch.bfloat16, H, KV, hd, ps, [40] * rows, [1] * rows, seed=3)
    out = torch.zeros(case.T, H * hd, dtype=torch.bfloat16, device=DEV)
    rc = static(C.byref(case.params(out, splits=splits)), torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    msg = l.dk_last_error().decode()
    assert "floats of scratch" in msg and str(STATIC_FLOATS) in msg
    torch.cuda.synchronize()
    assert out.abs().sum() == 0          # nothing was launched
    # one split needs no scratch at all and is taken whatever the size
    rc = static(C.byref(case.params(out, splits=1)), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, l.dk_last_error().decode()
    ref, _, _ = case.reference()
    assert torch.allclose(out.float().cpu(), ref, atol=2e-2, rtol=2e-2)
