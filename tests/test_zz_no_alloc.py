"""lf_decode_bf16_static: decode for hosts that cannot allocate.

A serving loop whose memory pool is frozen, or a plugin that is called from inside another
runtime, may hold nothing but its input and output buffers and may not call cudaMalloc when it
launches decode. For such callers the library keeps the split-KV partials in a fixed device array
of LF_STATIC_SCRATCH_BYTES that belongs to the library image. This test calls the entry point
through the C ABI, twice in a row with different inputs (the array is shared and keeps the
previous call's contents), and checks each result against lf_decode_bf16 with a caller-owned
workspace - bit for bit: at the same split count the two run the same kernels on the same
numbers, only the address of the partials differs. It also checks that the call itself leaves
the device's free memory and the allocator's books untouched, and that a problem whose partials
exceed the fixed array is refused.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import pytest
import torch

from loopfuse_b200 import _native

pytestmark = pytest.mark.gpu


def _args(q, k, v, out, splits, workspace=None):
    a = _native.LfDecodeArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.B, a.Hkv, a.G, a.D = q.shape
    a.Skv = k.shape[2]
    for i in range(3):
        a.q_stride[i], a.o_stride[i] = q.stride(i), out.stride(i)
        a.k_stride[i], a.v_stride[i] = k.stride(i), v.stride(i)
    a.scale = q.shape[-1] ** -0.5
    a.splits = splits
    if workspace is not None:
        a.workspace = workspace.data_ptr()
        a.workspace_bytes = workspace.numel()
    return a


def _inputs(seed, B=4, Hkv=8, G=4, Skv=2048, D=128):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()
    return mk(B, Hkv, G, D), mk(B, Hkv, Skv, D), mk(B, Hkv, Skv, D)


def test_static_scratch_decode_matches_workspace_decode_twice():
    lib = _native.load()
    stream = torch.cuda.current_stream().cuda_stream
    for seed, splits in ((11, 4), (12, 8)):          # two calls in a row, shared scratch
        q, k, v = _inputs(seed)
        B, Hkv, G, D = q.shape
        nbytes = lib.lf_decode_workspace_bytes(B, Hkv, G, D, splits)
        assert 0 < nbytes <= _native.LF_STATIC_SCRATCH_BYTES
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        want = torch.empty_like(q)
        got = torch.full_like(q, float("nan"))
        rc = lib.lf_decode_bf16(C.byref(_args(q, k, v, want, splits, ws)), stream)
        assert rc == 0, lib.lf_strerror(rc)
        static_args = _args(q, k, v, got, splits)
        if seed == 11:   # the first call on a device looks up the array's address: do it once
            rc = lib.lf_decode_bf16_static(C.byref(static_args), stream)
            assert rc == 0, lib.lf_strerror(rc)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        booked_before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
        rc = lib.lf_decode_bf16_static(C.byref(static_args), stream)
        assert rc == 0, lib.lf_strerror(rc)
        torch.cuda.synchronize()
        # nothing was allocated or freed: the driver's free memory and torch's allocator
        # statistics are what they were before the call
        assert torch.cuda.mem_get_info()[0] == free_before
        assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == booked_before
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got, want)


def test_static_scratch_refuses_oversized_problem():
    lib = _native.load()
    q, k, v = _inputs(13, B=16, Hkv=32, G=8, Skv=2048)
    out = torch.empty_like(q)
    need = lib.lf_decode_workspace_bytes(16, 32, 8, 128, 8)
    assert need > _native.LF_STATIC_SCRATCH_BYTES
    rc = lib.lf_decode_bf16_static(C.byref(_args(q, k, v, out, 8)),
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == -7 and b"limit" in lib.lf_strerror(rc)
    torch.cuda.synchronize()
