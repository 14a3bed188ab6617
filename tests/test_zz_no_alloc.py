"""The decode-attention entry point that allocates nothing (csrc/no_alloc.h), called through
its exported C symbol as a host program would call it.

Some programs that embed this library own all device memory themselves or run loops in
which cudaMalloc (which synchronises the device) is not acceptable; they can hand in their
own inputs and outputs but not the scratch that the split decode kernel needs.  The entry
point keeps that scratch in an array inside the library.  The test checks two calls in a
row, with different data, against the ordinary entry point that takes caller scratch (the
array keeps the first call's contents, so a slot that the second call failed to overwrite
would show) and against the plain implementation, with and without context splits and with
a window; and it checks the property the entry point exists for: the device's free memory
is the same before and after a call.  The file sorts last so that a run stopping at the
first failure has already run everything else.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64
MAX_FLOATS = 1 << 20  # MLL_NO_ALLOC_SCRATCH_FLOATS


def _library():
    from cpp_minilamma_b200.csrc.build import load_library
    lib = ctypes.CDLL(str(load_library()._name))  # the exported symbols, as any C caller sees them
    lib.mll_last_error.restype = ctypes.c_char_p
    ptr, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.mll_attn_decode_no_alloc.argtypes = [ptr] * 7 + [i32] * 8 + [f32, ptr]
    lib.mll_attn_decode_no_alloc.restype = i32
    lib.mll_attn_decode.argtypes = [ptr] * 8 + [i32] * 8 + [f32, ptr]
    lib.mll_attn_decode.restype = i32
    return lib


def _case(seed, dtype, ctx_lens, hq, hk, d):
    g = torch.Generator().manual_seed(seed)
    n_seqs = len(ctx_lens)
    blocks = [(c + PAGE - 1) // PAGE for c in ctx_lens]
    n_pages = sum(blocks) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_seqs, max(blocks)), -1, dtype=torch.int32)
    at = 0
    for b, nb in enumerate(blocks):
        for i in range(nb):
            table[b, i] = order[at]
            at += 1
    rnd = lambda *shape: torch.randn(*shape, generator=g).to(dtype).to(DEV)
    return dict(q=rnd(n_seqs, hq * d), k=rnd(n_pages, hk, PAGE, d), v=rnd(n_pages, hk, PAGE, d),
                slot=torch.arange(n_seqs, dtype=torch.int32, device=DEV),
                ctx=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), table=table.to(DEV))


def _plain(case, ctx_lens, hq, hk, d, window):
    """The plain implementation on the same pages: one query at the last position of each sequence."""
    rows = []
    for b, c in enumerate(ctx_lens):
        pages = case["table"][b, :(c + PAGE - 1) // PAGE].cpu().long()
        k = case["k"].cpu().float()[pages].permute(0, 2, 1, 3).reshape(-1, hk, d)[:c].numpy().astype(np.float64)
        v = case["v"].cpu().float()[pages].permute(0, 2, 1, 3).reshape(-1, hk, d)[:c].numpy().astype(np.float64)
        q = case["q"][b].cpu().float().reshape(1, hq, d).numpy().astype(np.float64)
        rows.append(pl.causal_attention(q, k, v, window=window or None, q_positions=[c - 1]).reshape(hq * d))
    return np.stack(rows)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("splits,window", [(4, 0), (1, 0), (4, 70)])
def test_two_calls_in_a_row_match_the_entry_point_with_caller_scratch(dtype, splits, window):
    lib = _library()
    hq, hk, d = 8, 2, 64
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = 0 if dtype == torch.float32 else 1
    tol = dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-3)
    for call, ctx_lens in enumerate(([300, 1, 65, 129], [64, 257, 30, 500])):
        c = _case(10 + call, dtype, ctx_lens, hq, hk, d)
        n = len(ctx_lens)
        args = [c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), c["slot"].data_ptr(), c["ctx"].data_ptr(),
                c["table"].data_ptr()]
        sizes = [code, n, hq, hk, d, c["table"].shape[1], splits, window]
        scale = ctypes.c_float(1.0 / math.sqrt(d))
        expected = torch.full((n, hq * d), float("nan"), dtype=dtype, device=DEV)
        scratch = torch.empty(n * hq * splits * (d + 2), dtype=torch.float32, device=DEV)
        rc = lib.mll_attn_decode(*args, scratch.data_ptr(), expected.data_ptr(), *sizes, scale, stream)
        assert rc == 0, lib.mll_last_error()
        got = torch.full((n, hq * d), float("nan"), dtype=dtype, device=DEV)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.mll_attn_decode_no_alloc(*args, got.data_ptr(), *sizes, scale, stream)
        assert rc == 0, lib.mll_last_error()
        torch.cuda.synchronize()
        if call == 1:  # the first call on a device looks the array's address up; after that nothing may move
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        np.testing.assert_allclose(got.float().cpu().numpy(), expected.float().cpu().numpy(), **tol,
                                   err_msg=f"call {call}")
        assert torch.isfinite(got.float()).all()
        plain_tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
        np.testing.assert_allclose(got.float().cpu().numpy(), _plain(c, ctx_lens, hq, hk, d, window), **plain_tol,
                                   err_msg=f"call {call} against the plain implementation")


def test_sizes_beyond_the_built_in_scratch_are_refused():
    lib = _library()
    c = _case(3, torch.float32, [10], 4, 2, 64)
    out = torch.zeros((1, 4 * 64), dtype=torch.float32, device=DEV)
    n_seqs = MAX_FLOATS // (4 * 8 * 66) + 1  # one sequence too many for 8 splits of 4 heads
    rc = lib.mll_attn_decode_no_alloc(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), c["slot"].data_ptr(),
                                      c["ctx"].data_ptr(), c["table"].data_ptr(), out.data_ptr(), 0, n_seqs, 4, 2, 64,
                                      1, 8, 0, ctypes.c_float(0.125), None)
    assert rc != 0
    message = lib.mll_last_error().decode()
    assert "exceed the built-in" in message and str(MAX_FLOATS) in message
    torch.cuda.synchronize()  # nothing was launched, nothing faulted
