"""arle_sample_static, the sampling entry point that allocates nothing, called
through its exported C symbol and compared with the ordinary entry point.

Some users of the library may not allocate device memory when they need a token
(they run inside another allocator's callback, or under a harness that has
already handed out all memory, or they are bare C/FFI clients without an
allocator): for them the probabilities go into an array built into the library
instead of a scratch buffer from the caller.  The file is named so that pytest
collects it last; it passes alone in a fresh process and after the other tests.
"""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from arle_b200.ops import build

    lib = ctypes.CDLL(build.library_path())
    P, I = c_void_p, c_int
    lib.arle_sample_static.argtypes = [P, I, I, I, P, P, P, P, P, P, P]
    lib.arle_sample_static.restype = c_int
    lib.arle_sample.argtypes = [P, I, I, I, P, P, P, P, P, P, P, P]
    lib.arle_sample.restype = c_int
    lib.arle_sample_static_max_floats.restype = c_longlong
    lib.arle_no_alloc_error_string.argtypes = [c_int]
    lib.arle_no_alloc_error_string.restype = ctypes.c_char_p
    return lib


def _case(rows, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    dev = "cuda"
    return dict(
        logits=(torch.randn(rows, vocab, generator=g) * 3).to(dev),
        temp=torch.tensor([0.0, 0.8, 1.2, 1.0, 0.6, 0.0][:rows], device=dev),
        top_k=torch.tensor([-1, -1, 20, 1, 50, 3][:rows], dtype=torch.int32, device=dev),
        top_p=torch.tensor([1.0, 0.9, 1.0, 1.0, 0.7, 1.0][:rows], device=dev),
        min_p=torch.tensor([0.0, 0.0, 0.05, 0.0, 0.0, 0.0][:rows], device=dev),
        u=torch.rand(rows, generator=g).to(dev))


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    lib = _lib()
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.arle_sample_static_max_floats() == 1 << 20
    # two calls in a row with different sizes and contents: the second finds the
    # first one's leftovers in the built-in array and must not be disturbed by them
    for rows, vocab, seed in ((6, 151936, 1), (5, 30011, 2)):
        c = _case(rows, vocab, seed)
        want = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        got = torch.full((rows,), -2, dtype=torch.int32, device="cuda")
        scratch = torch.empty(rows, vocab, device="cuda")
        args = [c["logits"].data_ptr(), vocab, rows, vocab, c["temp"].data_ptr(), c["top_k"].data_ptr(),
                c["top_p"].data_ptr(), c["min_p"].data_ptr(), c["u"].data_ptr()]
        assert lib.arle_sample(*args, scratch.data_ptr(), want.data_ptr(), stream) == 0
        # free bytes as the driver counts them: an allocation inside the call, by whatever
        # route, would lower the figure (torch's own counters only see torch's allocator)
        torch.cuda.synchronize()
        before = torch.cuda.mem_get_info()[0]
        assert lib.arle_sample_static(*args, got.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == before
        # token ids: the same kernel on the same numbers, so equality is the tolerance
        assert got.tolist() == want.tolist()
        assert all(0 <= t < vocab for t in got.tolist())
    # all rows greedy: no parameter arrays at all
    lg = c["logits"]
    got = torch.empty(rows, dtype=torch.int32, device="cuda")
    assert lib.arle_sample_static(lg.data_ptr(), vocab, rows, vocab, None, None, None, None, None, got.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert got.tolist() == lg.argmax(dim=1).tolist()


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _lib()
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    rows, vocab = 8, 151936                      # 1,215,488 floats > 1,048,576
    lg = torch.randn(rows, vocab, device="cuda")
    out = torch.full((rows,), 7, dtype=torch.int32, device="cuda")
    temp = torch.full((rows,), 0.9, device="cuda")
    u = torch.full((rows,), 0.5, device="cuda")
    code = lib.arle_sample_static(lg.data_ptr(), vocab, rows, vocab, temp.data_ptr(), None, None, None, u.data_ptr(),
                                  out.data_ptr(), stream)
    assert code == -4
    assert b"ARLE_SAMPLE_STATIC_MAX_FLOATS" in lib.arle_no_alloc_error_string(code)
    torch.cuda.synchronize()
    assert out.tolist() == [7] * rows            # nothing was launched
    # without temperatures every row is an argmax, which does not use the array: the same size is taken
    assert lib.arle_sample_static(lg.data_ptr(), vocab, rows, vocab, None, None, None, None, None, out.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert out.tolist() == lg.argmax(dim=1).tolist()
    assert lib.arle_sample_static(lg.data_ptr(), vocab - 1, 1, vocab, None, None, None, None, None, out.data_ptr(), stream) == -3
