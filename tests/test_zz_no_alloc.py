"""The sampler variant for callers that cannot allocate device memory (csrc/noalloc.h): called
through its exported C symbol, it must pick the same tokens as the regular sampler, on two calls
in a row that share its built-in scratch array.  Runs last; passes alone in a fresh process too."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from glint_b200.csrc import build
    lib = ctypes.CDLL(build.build_library("core"))
    fn = lib.glint_sample_noalloc
    P = ctypes.c_void_p
    fn.argtypes = [P, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, P, P, P, P, P, P, P]
    fn.restype = ctypes.c_int
    return fn


def _case(rows, vocab, seed, top_k):
    g = torch.Generator().manual_seed(seed)
    dev = "cuda:0"
    return {
        "logits": (torch.randn(rows, vocab, generator=g) * 3.0).to(dev),
        "temperature": (0.5 + torch.rand(rows, generator=g)).to(dev),
        "top_k": torch.full((rows,), top_k, dtype=torch.int32, device=dev),
        "top_p": torch.ones(rows, device=dev),
        "min_p": torch.zeros(rows, device=dev),
        "uniform": torch.rand(rows, generator=g).to(dev),
    }


def _regular(c):
    from glint_b200 import ops
    rows, vocab = c["logits"].shape
    work = torch.empty(rows, vocab, device=c["logits"].device)
    out = torch.empty(rows, dtype=torch.int32, device=c["logits"].device)
    ops.sample(c["logits"], work, c["temperature"], c["top_k"], c["top_p"], c["min_p"], c["uniform"], out)
    return out.cpu()


def _no_alloc(fn, c):
    rows, vocab = c["logits"].shape
    out = torch.full((rows,), -1, dtype=torch.int32, device=c["logits"].device)
    before = torch.cuda.memory_allocated()
    rc = fn(c["logits"].data_ptr(), c["logits"].stride(0), rows, vocab, c["temperature"].data_ptr(),
            c["top_k"].data_ptr(), c["top_p"].data_ptr(), c["min_p"].data_ptr(), c["uniform"].data_ptr(),
            out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    return out.cpu()


def test_no_alloc_sampler_matches_the_regular_one_twice_in_a_row():
    fn = _entry()
    first = _case(8, 50000, seed=1, top_k=0)       # fills most of the shared array
    second = _case(3, 777, seed=2, top_k=40)       # a smaller call right after must not see leftovers
    for c in (first, second):
        want = _regular(c)
        got = _no_alloc(fn, c)
        assert torch.equal(got, want), (got, want)
        assert int(got.min()) >= 0 and int(got.max()) < c["logits"].shape[1]


def test_no_alloc_sampler_refuses_sizes_beyond_its_array():
    fn = _entry()
    c = _case(2, 64, seed=3, top_k=0)
    args = lambda rows, vocab: (c["logits"].data_ptr(), 64, rows, vocab, c["temperature"].data_ptr(),
                                c["top_k"].data_ptr(), c["top_p"].data_ptr(), c["min_p"].data_ptr(),
                                c["uniform"].data_ptr(), c["top_k"].data_ptr(),
                                torch.cuda.current_stream().cuda_stream)
    assert fn(*args(9, 64)) == -2
    assert fn(*args(2, 262145)) == -2
    assert fn(*args(0, 64)) == 0
