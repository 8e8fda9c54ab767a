"""The allocation-free GEMM entry point, driven the way a non-Python caller would drive it.

``cs_gemm_skinny_noalloc`` is meant for processes that cannot allocate GPU memory when they need a small-M GEMM
(an executor that gave the whole device to its KV cache, a serving loop where an allocation would stall the
device): its split-K scratch is a static array inside the library.  This test reaches the function through its
exported C symbol with ctypes only, hands it caller-owned buffers, and checks it against the regular entry point
(``cs_gemm_skinny`` behind ``ops.linear(..., skinny=True)``), twice in a row on the same shared scratch, plus the
refusal of a problem that does not fit the built-in array.  The file name sorts last so that a run that stops
at the first failure has already run every other test.
"""

import ctypes
from ctypes import c_char_p, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = -20


def _lib():
    from cornserve.ops import _lib as loader

    lib = ctypes.CDLL(str(loader.lib_path()))  # plain dlopen + dlsym, no Python-side wrapper
    fn = lib.cs_gemm_skinny_noalloc
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    fn.restype = c_int
    lib.cs_noalloc_last_message.restype = c_char_p
    lib.cs_gemm_skinny_noalloc_kernel_error.restype = c_int
    lib.cs_gemm_skinny_noalloc_need_bytes.argtypes = [c_int] * 5
    lib.cs_gemm_skinny_noalloc_need_bytes.restype = c_longlong
    return lib


def _call(lib, x, w, out, bias=None, residual=None, act=0, swiglu=0, splits=0):
    M, K = x.shape
    N = out.shape[1]
    return lib.cs_gemm_skinny_noalloc(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
        None if bias is None else bias.data_ptr(), None if residual is None else residual.data_ptr(),
        0 if residual is None else residual.stride(0), M, N, K, act, swiglu, 0, splits,
        torch.cuda.current_stream().cuda_stream)


def _close(a, b):
    a, b = a.float(), b.float()
    bad = ((a - b).abs() > 2e-2 + 2e-2 * b.abs()).float().mean().item()
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert bad < 1e-3 and cos > 0.999, (bad, cos)


def test_noalloc_gemm_matches_regular_entry_point_twice():
    from cornserve import ops
    from cornserve.ops.reference import ACTS

    lib = _lib()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, std=1.0: (torch.randn(*s, device=dev, generator=g) * std).bfloat16()  # noqa: E731
    # two different problems back to back: they share the built-in scratch, the second must not see the first
    cases = [(48, 3584, 3584, 5, None), (7, 1024, 18944, 0, "silu")]
    for rep in range(2):
        for M, N, K, splits, act in cases:
            x, w, b, r = rnd(M, K), rnd(N, K, std=K ** -0.5), rnd(N), rnd(M, N)
            want = ops.linear(x, w, b, act=act, residual=r, skinny=True, splits=splits)
            got = torch.full((M, N), float("nan"), device=dev, dtype=torch.bfloat16)
            if rep == 1:
                free_before = torch.cuda.mem_get_info()[0]
            rc = _call(lib, x, w, got, b, r, ACTS[act or "none"], 0, splits)
            assert rc == 0, lib.cs_noalloc_last_message().decode()
            torch.cuda.synchronize()
            if rep == 1:
                assert torch.cuda.mem_get_info()[0] == free_before  # the call took no device memory
            _close(got, want)
            # and against the fp32 restatement, with the tolerance the other GEMM tests use
            _close(got, ops.reference.linear(x, w, b, act, r, out_dtype=torch.float32))
    assert lib.cs_gemm_skinny_noalloc_kernel_error() == 0
    ops.check_error("no-alloc test")


def test_noalloc_gemm_refuses_what_does_not_fit():
    lib = _lib()
    M, N, K, splits = 256, 16384, 4096, 16
    assert lib.cs_gemm_skinny_noalloc_need_bytes(M, N, K, 0, splits) > (8 << 20)
    x = torch.zeros(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    assert _call(lib, x, w, out, splits=splits) == TOO_LARGE
    msg = lib.cs_noalloc_last_message().decode()
    assert "built-in scratch" in msg and "splits" in msg
    # without a split there is nothing to store in the scratch, so the same problem is accepted
    assert _call(lib, x, w, out, splits=1) == 0
    torch.cuda.synchronize()
