"""The allocation-free flash-decode entry point against the regular one.

Some callers of this library may not allocate device memory while they run (a server that fixed its memory
budget at start-up, an embedder whose own runtime owns the allocator); for them the split kernel's scratch
lives in an array built into the library. This file is named so that pytest collects it last.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(lib, handle, fn_noalloc, B, H, KV, D, ctx, seed):
    import torch

    gen = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, H, D, device="cuda", generator=gen).bfloat16()
    k = torch.randn(B, KV, ctx, D, device="cuda", generator=gen).bfloat16()
    v = torch.randn(B, KV, ctx, D, device="cuda", generator=gen).bfloat16()
    ref = torch.empty(B, H, D, device="cuda", dtype=torch.bfloat16)
    out = torch.full((B, H, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    scratch = torch.empty(lib.swlm_op_flash_decode_scratch_bytes(B, H, KV, D, ctx), device="cuda", dtype=torch.uint8)
    torch.cuda.synchronize()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    scale = 1.0 / np.sqrt(D)
    lib.check(lib.swlm_op_flash_decode_dev(handle, B, H, KV, D, ctx, ctx, scale, q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                           ref.data_ptr(), scratch.data_ptr(), stream))
    lib.check(fn_noalloc(handle, B, H, KV, D, ctx, ctx, scale, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), stream))
    torch.cuda.synchronize()
    # fp32 reference of the same attention (softmax(q k^T * scale) v per GQA group), independent of both entry points
    G = H // KV
    qf = q.float().view(B, KV, G, D)
    scores = torch.einsum("bkgd,bktd->bkgt", qf, k.float()) * scale
    exact = torch.einsum("bkgt,bktd->bkgd", torch.softmax(scores, dim=-1), v.float()).reshape(B, H, D)
    return out.float().cpu().numpy(), ref.float().cpu().numpy(), exact.cpu().numpy()


def test_noalloc_flash_decode_matches_regular_entry_point(pkg):
    from swlm_helpers import rel_err

    store = pkg.WeightStore(0)
    lib = store.lib
    assert lib.swlm_op_flash_decode_noalloc_capacity() == 8 << 20
    # two calls in a row with different shapes and data: the shared array keeps the first call's contents,
    # the second must not be disturbed by them
    for seed, (B, H, KV, D, ctx) in enumerate([(2, 32, 8, 128, 3000), (4, 32, 8, 128, 1500), (1, 8, 2, 64, 777)]):
        out, ref, exact = _run(lib, store.handle, lib.swlm_op_flash_decode_noalloc_dev, B, H, KV, D, ctx, seed)
        assert np.isfinite(out).all()
        assert rel_err(out.reshape(B * H, D), ref.reshape(B * H, D)).max() <= 1e-2
        # and against the fp32 reference, so that a fault common to both entry points cannot pass
        assert rel_err(out.reshape(B * H, D), exact.reshape(B * H, D)).max() <= 1e-2
        assert rel_err(ref.reshape(B * H, D), exact.reshape(B * H, D)).max() <= 1e-2
    # a request beyond the built-in scratch is refused, not truncated
    import torch

    # (checked before anything is launched: 16 x 1024 heads x 130 floats is 8.1 MiB of partials)
    B, H, KV, D, ctx = 16, 1024, 128, 128, 4096
    assert lib.swlm_op_flash_decode_scratch_bytes(B, H, KV, D, ctx) > lib.swlm_op_flash_decode_noalloc_capacity()
    t = torch.empty(1, device="cuda", dtype=torch.bfloat16)
    rc = lib.swlm_op_flash_decode_noalloc_dev(store.handle, B, H, KV, D, ctx, ctx, 0.1, t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                              t.data_ptr(), None)
    assert rc == -1 and b"built-in scratch" in lib.swlm_last_error()
    # arguments that would fault on the GPU or divide by zero on the host are refused before anything is launched:
    # a pointer that is not 16-byte aligned (the kernel uses 128-bit loads), no KV heads, a non-positive head_dim
    buf = torch.zeros(4096, device="cuda", dtype=torch.bfloat16)
    good, odd = buf.data_ptr(), buf.data_ptr() + 2
    for args in [(1, 8, 2, 64, 16, 16, 0.1, good, odd, good, good), (1, 8, 2, 64, 16, 16, 0.1, good, good, odd, good),
                 (1, 8, 0, 64, 16, 16, 0.1, good, good, good, good), (1, 8, 2, 0, 16, 16, 0.1, good, good, good, good),
                 (1, 7, 2, 64, 16, 16, 0.1, good, good, good, good)]:
        assert lib.swlm_op_flash_decode_noalloc_dev(store.handle, *args, None) == -1
        assert lib.swlm_op_flash_decode_dev(store.handle, *args, good, None) == -1
    assert lib.swlm_op_flash_decode_dev(store.handle, 1, 8, 2, 64, 16, 16, 0.1, good, good, good, good, odd, None) == -1
    assert lib.swlm_op_flash_decode_scratch_bytes(1, 8, 0, 64, 16) == 0
    store.close()
