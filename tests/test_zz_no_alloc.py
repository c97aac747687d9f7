"""The allocation-free argmax entry point (``owl_argmax_noalloc``), called through its exported C
symbol, must agree with the regular ``owl_argmax`` that takes caller-provided scratch.

Some users of the library cannot hand it scratch memory: they run inside a device-memory budget
that is already fully committed, or embed the C ABI without any allocator. For them the partial
results live in a fixed array inside the library; this test checks two calls in a row (the array
keeps the previous call's contents) against the existing entry point.

The file name sorts last so a run that stops at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

from owl_engine_b200 import _native
from owl_engine_b200.ops import kernels as K

pytestmark = pytest.mark.gpu


def _noalloc():
    lib = _native.cuda()
    f = lib.owl_argmax_noalloc
    f.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                  ctypes.c_void_p]
    f.restype = ctypes.c_int
    return f


def test_noalloc_argmax_matches_regular_entry_point_twice():
    f = _noalloc()
    dev = "cuda"
    g = torch.Generator().manual_seed(7)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, vocab, off) in enumerate([(3, 151936, 0), (32, 4099, 1000)]):
        logits = torch.randn(rows, vocab, generator=g).to(torch.bfloat16).to(dev)
        want = torch.empty(rows, dtype=torch.int32, device=dev)
        sv = torch.empty(rows * 64, dtype=torch.float32, device=dev)
        si = torch.empty(rows * 64, dtype=torch.int32, device=dev)
        K.argmax(logits, rows, vocab, vocab, sv, si, 64, want, off)
        got = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        rc = f(logits.data_ptr(), rows, vocab, vocab, got.data_ptr(), off, stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.equal(got, want), call
        assert got.cpu().tolist() == (logits.float().argmax(-1) + off).cpu().tolist()


def test_noalloc_rejects_oversize_without_launching():
    f = _noalloc()
    x = torch.zeros(1, 16, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(64, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert f(x.data_ptr(), 33, 16, 16, out.data_ptr(), 0, stream) == -1
    assert f(x.data_ptr(), 0, 16, 16, out.data_ptr(), 0, stream) == -1
    assert f(x.data_ptr(), 1, 16, 8, out.data_ptr(), 0, stream) == -1
    torch.cuda.synchronize()
