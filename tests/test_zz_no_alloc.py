"""The decode-attention entry point that allocates nothing (csrc/no_alloc.h), called through its
exported C symbol, against the ordinary entry point.

It is for callers that must not allocate device memory while serving: the engine has given the free
memory to the page pool, so a late cudaMalloc can fail, and cudaMalloc/cudaFree stall the whole
device.  The test makes two calls in a row (they share the library's one scratch array, which keeps
the first call's contents) and checks both results, and checks that a call too large for the array
is refused.  This file sorts last on purpose: a run that stops at the first failure has then run
every other test already."""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _setup(lens, Hq, Hkv, D, page, seed):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((n + page - 1) // page for n in lens) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    max_blocks = max((n + page - 1) // page for n in lens)
    bt = torch.full((len(lens), max_blocks), -1, dtype=torch.int32)
    for i, n in enumerate(lens):
        for b in range((n + page - 1) // page):
            bt[i, b] = order.pop()
    kc = (torch.randn(n_pages, Hkv, page, D, generator=g)).to(torch.bfloat16).to(DEV)
    vc = (torch.randn(n_pages, Hkv, page, D, generator=g)).to(torch.bfloat16).to(DEV)
    qkv = torch.randn(len(lens), (Hq + 2 * Hkv) * D, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    ent = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    return qkv, kc, vc, bt.to(DEV), ent, pos


def _call(lib, name, qkv, kc, vc, bt, ent, pos, out, Hq, Hkv, D, page, splits, scratch=None):
    fn = getattr(lib, name)
    fn.restype = c_int
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [c_void_p(qkv.data_ptr()), c_int(1), c_int(qkv.shape[1]), c_void_p(kc.data_ptr()), c_void_p(vc.data_ptr()),
            c_int(1), c_void_p(bt.data_ptr()), c_int(bt.shape[1]), c_void_p(ent.data_ptr()), c_void_p(pos.data_ptr()),
            c_void_p(0), c_int(qkv.shape[0]), c_float(1.0 / math.sqrt(D)), c_int(0), c_void_p(out.data_ptr()), c_int(1),
            c_int(Hq), c_int(Hkv), c_int(D), c_int(page), c_int(kc.shape[0]), c_int(splits)]
    if scratch is not None:
        args.append(c_void_p(scratch.data_ptr()))
        args.append(c_void_p(0))            # the ordinary entry point also takes an error flag; none here
        args += [c_void_p(0), c_int(0)]     # ... and counters for adding the splits up in the kernel itself; none
    args.append(stream)
    return fn(*args)


def test_no_alloc_decode_attention_matches_the_ordinary_entry_point():
    from nano_vllm_cpp_b200.csrc import ops
    lib = ops.lib()
    Hq, Hkv, D, page, splits = 8, 2, 64, 16, 3
    for call, lens in enumerate(([300, 17, 1024, 63], [90, 700])):        # two calls in a row, different sizes
        qkv, kc, vc, bt, ent, pos = _setup(lens, Hq, Hkv, D, page, seed=call)
        R = len(lens)
        want = torch.zeros(R, Hq * D, dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(R * Hq * splits * (D + 2), dtype=torch.float32, device=DEV)
        assert _call(lib, "nv_attention_decode", qkv, kc, vc, bt, ent, pos, want, Hq, Hkv, D, page, splits, scratch) == 0
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        rc = _call(lib, "nv_attention_decode_noalloc", qkv, kc, vc, bt, ent, pos, got, Hq, Hkv, D, page, splits)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        err = float((got.float() - want.float()).abs().max())
        assert err <= 1.5e-2 * float(want.float().abs().max()), f"call {call}: max error {err}"
    # a call whose partial results exceed the library's array is refused and launches nothing
    lib.nv_attention_decode_noalloc_max_rows.restype = c_int
    most = lib.nv_attention_decode_noalloc_max_rows(c_int(Hq), c_int(D), c_int(splits))
    assert most == (1 << 20) // (Hq * splits * (D + 2))
    lens = [5] * (most + 1)
    qkv, kc, vc, bt, ent, pos = _setup(lens, Hq, Hkv, D, page, seed=9)
    out = torch.zeros(len(lens), Hq * D, dtype=torch.bfloat16, device=DEV)
    assert _call(lib, "nv_attention_decode_noalloc", qkv, kc, vc, bt, ent, pos, out, Hq, Hkv, D, page, splits) == -6
    assert float(out.abs().max()) == 0.0
    assert _call(lib, "nv_attention_decode_noalloc", qkv[:most], kc, vc, bt, ent, pos, out[:most], Hq, Hkv, D, page,
                 splits) == 0
    torch.cuda.synchronize()
    lib.nv_attention_decode_noalloc_status.restype = c_int
    assert lib.nv_attention_decode_noalloc_status() == 0
    # sizes the kernel does not take are refused before the size test, and fit no row
    assert lib.nv_attention_decode_noalloc_max_rows(c_int(Hq), c_int(20), c_int(splits)) == 0
    assert lib.nv_attention_decode_noalloc_max_rows(c_int(Hq), c_int(264), c_int(splits)) == 0
    assert lib.nv_attention_decode_noalloc_max_rows(c_int(0), c_int(D), c_int(splits)) == 0
    assert _call(lib, "nv_attention_decode_noalloc", qkv[:2], kc, vc, bt, ent, pos, out[:2], Hq, Hkv, 20, page, splits) == -4
    assert _call(lib, "nv_attention_decode_noalloc", qkv[:2], kc, vc, bt, ent, pos, out[:2], Hq, 0, D, page, splits) == -4
    assert _call(lib, "nv_attention_decode_noalloc", qkv[:2], kc, vc, bt, ent, pos, out[:2], -Hq, -Hkv, D, page, splits) == -4
