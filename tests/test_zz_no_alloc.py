"""The allocation-free decode-attention entry point against the regular one.

``ab2_paged_decode_noalloc`` is for callers that must not allocate device memory when they
call into the library (inside a CUDA-graph capture or a serving loop where an allocation
would stall the device, under a host runtime that owns the allocator, or without PyTorch).
It keeps its split-KV workspace inside the library image. The test loads the exported C
symbol directly with ctypes, runs it twice in a row on different inputs (the workspace is
shared and keeps old contents, so the second call checks that stale data does not leak) and
compares with ``ab2_paged_decode`` fed a caller-allocated workspace. It also checks that an
oversized request is refused. The file name sorts last so a failure here cannot hide other
tests under ``-x``.
"""
import ctypes

import pytest
import torch

from areal_b200.ops import lib as oplib

pytestmark = pytest.mark.gpu

c_void_p, c_int, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _raw_lib():
    lib = ctypes.CDLL(str(oplib.lib_path()))
    lib.ab2_paged_decode_noalloc.argtypes = [c_void_p] * 6 + [c_int] * 7 + [c_float, c_void_p]
    lib.ab2_paged_decode_noalloc.restype = c_int
    lib.ab2_paged_decode.argtypes = [c_void_p] * 8 + [c_int] * 7 + [c_float, c_void_p]
    lib.ab2_paged_decode.restype = c_int
    return lib


def _case(seed, B, Hq, Hkv, D, page_size, max_len):
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_pages = B * ((max_len + page_size - 1) // page_size) + 3
    kc = torch.randn(n_pages * page_size, Hkv, D, device="cuda", generator=g).bfloat16()
    vc = torch.randn(n_pages * page_size, Hkv, D, device="cuda", generator=g).bfloat16()
    q = torch.randn(B, Hq, D, device="cuda", generator=g).bfloat16()
    lens = torch.randint(1, max_len + 1, (B,), device="cuda", generator=g).int()
    max_pages = (max_len + page_size - 1) // page_size
    perm = torch.randperm(n_pages, device="cuda", generator=g)[: B * max_pages].int()
    pt = perm.view(B, max_pages).contiguous()
    return q, kc, vc, pt, lens, max_pages


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 8, 2), (64, 4, 2)])
def test_noalloc_decode_matches_regular_entry_point(D, Hq, Hkv):
    lib = _raw_lib()
    stream = torch.cuda.current_stream().cuda_stream
    splits, page_size, scale = 4, 16, D ** -0.5
    for call, (seed, B, max_len) in enumerate([(1, 7, 300), (2, 5, 90)]):
        q, kc, vc, pt, lens, max_pages = _case(seed, B, Hq, Hkv, D, page_size, max_len)
        ref = torch.empty_like(q)
        po = torch.empty(B * Hq * splits * D, device="cuda")
        pml = torch.empty(B * Hq * splits * 2, device="cuda")
        rc = lib.ab2_paged_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pt.data_ptr(), lens.data_ptr(),
                                  po.data_ptr(), pml.data_ptr(), ref.data_ptr(), B, Hq, Hkv, D, page_size, max_pages,
                                  splits, scale, stream)
        assert rc == 0
        out = torch.full_like(q, float("nan"))
        rc = lib.ab2_paged_decode_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pt.data_ptr(), lens.data_ptr(),
                                          out.data_ptr(), B, Hq, Hkv, D, page_size, max_pages, splits, scale, stream)
        assert rc == 0, f"call {call} returned {rc}"
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        err = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
        assert err < 1e-2, f"call {call}: relative error {err}"


def test_noalloc_decode_rejects_oversized_request():
    lib = _raw_lib()
    q, kc, vc, pt, lens, max_pages = _case(3, 4, 8, 2, 128, 16, 64)
    out = torch.empty_like(q)
    # B * Hq * splits = 600 * 32 * 4 rows would not fit the built-in workspace
    rc = lib.ab2_paged_decode_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pt.data_ptr(), lens.data_ptr(),
                                      out.data_ptr(), 600, 32, 8, 128, 16, max_pages, 4, 0.1,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 20
