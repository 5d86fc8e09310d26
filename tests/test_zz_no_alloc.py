"""The allocation-free greedy choice (csrc/argmax_static.h), called through its exported C
symbol the way a host that cannot use the Python layer would call it. Its callers are code
that may not allocate device memory (a plug-in inside another program's CUDA context, a
real-time loop, a host whose pool already owns all memory), so the test hands it only
buffers that exist already and checks that it gives the same tokens as the library's usual
argmax, twice in a row on the same fixed scratch, and that it refuses more rows than that
scratch holds. This file is named to be collected last."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ROWS = 4096            # CML_ARGMAX_STATIC_MAX_ROWS
TOO_MANY_ROWS = -10        # CML_ARGMAX_STATIC_TOO_MANY_ROWS


def _entry():
    from camelid_b200.csrc import build
    lib = ctypes.CDLL(build.compile_module("sampling"))
    fn = lib.cml_argmax_rows_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    fn.restype = ctypes.c_int
    return fn


def test_static_argmax_matches_the_usual_one_twice(cuda):
    from camelid_b200.csrc import ops
    fn = _entry()
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(3)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    msg = ctypes.create_string_buffer(256)
    for call, (rows, vocab) in enumerate([(9, 128256), (70, 5003)]):
        logits = torch.tensor(rng.normal(size=(rows, vocab)).astype(np.float32), device=cuda)
        logits[1, 77] = logits[1, vocab - 5] = 50.0                 # equal maxima: the lower index wins
        want = torch.empty(rows, dtype=torch.int32, device=cuda)
        ops.argmax_rows(logits, want, err)
        got = torch.full((rows,), -1, dtype=torch.int32, device=cuda)
        before = torch.cuda.memory_allocated()
        rc = fn(logits.data_ptr(), logits.stride(0), rows, vocab, got.data_ptr(), err.data_ptr(), stream, msg, 256)
        torch.cuda.synchronize()
        assert rc == 0, (rc, msg.value)
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(got, want), f"call {call}"
        assert int(got[1]) == 77 and int(err) == 0


def test_static_argmax_refuses_more_rows_than_its_scratch(cuda):
    fn = _entry()
    msg = ctypes.create_string_buffer(256)
    dummy = torch.zeros(4, device=cuda)
    out = torch.zeros(4, dtype=torch.int32, device=cuda)
    rc = fn(dummy.data_ptr(), 4, MAX_ROWS + 1, 4, out.data_ptr(), out.data_ptr(),
            torch.cuda.current_stream().cuda_stream, msg, 256)
    assert rc == TOO_MANY_ROWS and b"exceed" in msg.value and str(MAX_ROWS).encode() in msg.value
