"""cn_absmax_f32_noalloc — the absmax entry point for callers that cannot allocate (no context, scratch in a fixed
array inside the library) — must give exactly what cn_absmax_f32 gives.  Collected last on purpose: if it fails, a
run that stops at the first failure has already run every other test.  Works alone in a fresh process and after the
other tests (it does not depend on their state: the shared scratch array cleans up after itself)."""
import ctypes

import numpy as np
import pytest
import torch

import clusternet_b200 as cn
from clusternet_b200 import _lib

pytestmark = pytest.mark.gpu


def test_noalloc_absmax_matches_context_absmax_on_consecutive_calls(ctx):
    lib = ctx.lib
    rng = np.random.default_rng(123)
    out_ref = torch.empty(1, dtype=torch.float32, device="cuda")
    out_new = torch.full((1,), -7.0, dtype=torch.float32, device="cuda")
    sp = ctx.stream_ptr()
    # two calls in a row (then more, with awkward sizes): the ticket in the shared array must be back at zero each time
    for n in (1 << 20, 3_000_001, 1, 0, 513, (1 << 22) + 7):
        x = torch.from_numpy((rng.standard_normal(n) * rng.uniform(0.1, 50)).astype(np.float32)).cuda()
        cn.check(lib.cn_absmax_f32(ctx.h, x.data_ptr(), n, out_ref.data_ptr(), sp))
        cn.check(lib.cn_absmax_f32_noalloc(x.data_ptr(), n, out_new.data_ptr(), sp))
        torch.cuda.synchronize()
        assert out_new.item() == out_ref.item(), n                     # bit-exact: same kernel, same reduction order
        if n:
            assert out_new.item() == float(x.abs().max().item())
        else:
            assert out_new.item() == -1.0
    # unaligned input takes the scalar path in both
    big = torch.randn(10_000, device="cuda")
    view = big[1:9_000]
    cn.check(lib.cn_absmax_f32(ctx.h, view.data_ptr(), view.numel(), out_ref.data_ptr(), sp))
    cn.check(lib.cn_absmax_f32_noalloc(view.data_ptr(), view.numel(), out_new.data_ptr(), sp))
    torch.cuda.synchronize()
    assert out_new.item() == out_ref.item()


def test_noalloc_absmax_rejects_oversize_and_null(ctx):
    lib = ctx.lib
    x = torch.zeros(16, device="cuda")
    out = torch.zeros(1, device="cuda")
    st = lib.cn_absmax_f32_noalloc(x.data_ptr(), (1 << 32) + 1, out.data_ptr(), None)   # refused before any launch
    assert st == _lib.CN_ERR_ARG and b"exceed the limit" in lib.cn_last_error()
    assert lib.cn_absmax_f32_noalloc(x.data_ptr(), 16, None, None) == _lib.CN_ERR_ARG
    assert lib.cn_absmax_f32_noalloc(None, 16, out.data_ptr(), None) == _lib.CN_ERR_ARG
    torch.cuda.synchronize()
