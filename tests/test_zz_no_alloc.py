"""The allocation-free greedy selection, called through its exported C symbol.

Some users of the kernel library are handed their input and output buffers by
a host application and may not allocate anything themselves - cudaMalloc
synchronises the device, and with the GPU full of cache pages it may fail - so
``ib_argmax_noalloc`` keeps its scratch in a fixed array inside the library.
This file checks it against the ordinary entry point on two calls in a row
(the second must not be disturbed by what the first left in the shared
array), and that sizes beyond its stated maximum are refused.  It is named to
be collected last, and passes alone in a fresh process as well as after the
other tests.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def symbol():
    from infernum_b200.ops import core
    lib = core.core_lib()
    fn = lib.ib_argmax_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.ib_argmax_noalloc_max_rows.restype = ctypes.c_int
    return core, lib, fn


def call(fn, logits, out):
    stream = torch.cuda.current_stream(logits.device).cuda_stream
    return fn(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], out.data_ptr(),
              stream)


def test_noalloc_argmax_equals_the_ordinary_entry_point_twice_in_a_row():
    core, lib, fn = symbol()
    assert lib.ib_argmax_noalloc_max_rows() == 256
    g = torch.Generator().manual_seed(0)
    cases = [(40, 128256), (3, 50000), (256, 5000), (1, 17)]  # the second call is smaller than the first
    inputs = []
    for rows, vocab in cases:
        logits = torch.randn(rows, vocab, generator=g).to(DEV)
        logits[0, vocab - 1] = logits[0, vocab // 3] = 50.0  # equal maxima: the lower index wins
        want = torch.empty(rows, dtype=torch.int32, device=DEV)
        core.argmax(logits, want)
        inputs.append((logits, want, torch.full((rows,), -1, dtype=torch.int32, device=DEV)))
    # the first call on the device looks up the scratch array's address; after it, the calls
    # must leave the device's free memory as the driver reports it untouched (torch's own
    # counters would not see a cudaMalloc inside the library)
    assert call(fn, inputs[0][0], inputs[0][2]) == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(DEV)[0]
    for logits, want, got in inputs:
        got.fill_(-1)
        assert call(fn, logits, got) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(DEV)[0] == free_before
    for (rows, vocab), (logits, want, got) in zip(cases, inputs):
        assert torch.equal(got, want)
        assert got[0].item() == vocab // 3
        # and independently of the sibling entry point, on the rows that have no tie
        assert got[1:].tolist() == logits[1:].argmax(dim=1).tolist()


def test_noalloc_argmax_refuses_what_it_cannot_hold():
    core, lib, fn = symbol()
    logits = torch.zeros(257, 64, device=DEV)
    out = torch.zeros(257, dtype=torch.int32, device=DEV)
    assert call(fn, logits, out) == -3  # beyond the stated maximum
    assert fn(None, 64, 4, 64, out.data_ptr(), None) == -1
    assert fn(logits.data_ptr(), 32, 4, 64, out.data_ptr(), None) == -1  # rows shorter than V
