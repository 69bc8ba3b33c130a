"""The workspace-free attention entry point, called straight through the C ABI.

For hosts that cannot create device memory at call time (engine plugins with a frozen memory
plan, processes whose device memory belongs to a broker) the library keeps the attention
kernel's 256-byte scratch block in a static array of its own. This file checks that entry
point against the regular one on two calls in a row, so that the second call runs on a block
that still holds what the first one left behind. It is named to be collected last: a run that
stops at the first failure has then already executed every other test.
"""
import ctypes

import pytest
import torch

from trinix_b200 import _lib
from trinix_b200._lib import I64x3

pytestmark = pytest.mark.gpu
TOL = 2e-2  # the attention tolerance used throughout the suite (max abs, bf16)


def _call(lib, fn_name, q, k, v, causal, window, slopes, extra, out=None):
    B, Sq, Hq, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    if out is None:
        out = torch.empty_like(q)
    P = ctypes.c_void_p
    wl, wr = window if window is not None else (-1, -1)
    args = [P(q.data_ptr()), P(k.data_ptr()), P(v.data_ptr()), P(out.data_ptr()), None,
            P(slopes.data_ptr()) if slopes is not None else None, B, Sq, Sk, Hq, Hk, D,
            I64x3(*q.stride()[:3]), I64x3(*k.stride()[:3]), I64x3(*v.stride()[:3]),
            I64x3(*out.stride()[:3]), float(D ** -0.5), int(causal), wl, wr, _lib.TRX_BF16]
    stream = P(torch.cuda.current_stream(q.device).cuda_stream)
    rc = getattr(lib, fn_name)(*args, *extra, stream)
    assert rc == 0, lib.trx_status_string(rc)
    return out


def test_static_scratch_attention_matches_workspace_attention_twice(cuda):
    lib = _lib.load()
    g = torch.Generator().manual_seed(0)
    ws = torch.zeros(int(lib.trx_attn_workspace_bytes()), dtype=torch.uint8, device=cuda)
    status = torch.full((1,), 7, dtype=torch.int32, device=cuda)
    P = ctypes.c_void_p
    cases = [  # (Sq, Sk, Hq, Hk, D, causal, window, alibi)
        (700, 700, 8, 2, 128, True, None, False),
        (520, 520, 4, 1, 64, False, (100, 0), True),
    ]
    free_before = None
    with torch.cuda.device(cuda):
        for Sq, Sk, Hq, Hk, D, causal, window, alibi in cases:  # two calls in a row
            q = torch.randn(2, Sq, Hq, D, generator=g).bfloat16().to(cuda)
            k = torch.randn(2, Sk, Hk, D, generator=g).bfloat16().to(cuda)
            v = torch.randn(2, Sk, Hk, D, generator=g).bfloat16().to(cuda)
            slopes = None
            if alibi:
                slopes = torch.tensor([2.0 ** (-(i + 1)) for i in range(Hq)], device=cuda)
            ref = _call(lib, "trx_attn_fwd", q, k, v, causal, window, slopes,
                        [P(ws.data_ptr()), ws.numel()])
            if free_before is None:
                # the first call on a device looks up the block's address; device memory in use
                # is compared around every call after that one
                _call(lib, "trx_attn_fwd_static_scratch", q, k, v, causal, window, slopes,
                      [P(status.data_ptr())])
            got = torch.empty_like(q)   # the caller's output buffer exists before the call
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info(cuda)[0]   # cudaMemGetInfo: the driver's view
            _call(lib, "trx_attn_fwd_static_scratch", q, k, v, causal, window, slopes,
                  [P(status.data_ptr())], out=got)
            torch.cuda.synchronize()
            # "allocates nothing": the device has exactly as much free memory after the call
            assert torch.cuda.mem_get_info(cuda)[0] >= free_before
            assert int(status.item()) == 0, "the kernel recorded a bounded-wait timeout"
            assert int(ws[:4].view(torch.int32).item()) == 0
            assert not torch.isnan(got.float()).any()
            assert float((got.float() - ref.float()).abs().max()) <= TOL
            # and against plain math, so that "both wrong in the same way" cannot pass
            kf, vf = (t.float().repeat_interleave(Hq // Hk, 2) for t in (k, v))
            s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf) * D ** -0.5
            i = torch.arange(Sq, device=cuda)[:, None]
            j = torch.arange(Sk, device=cuda)[None, :]
            if alibi:
                s = s - slopes.view(1, -1, 1, 1) * (i - j).abs()
            keep = torch.ones(Sq, Sk, dtype=torch.bool, device=cuda)
            if causal:
                keep &= j <= i
            if window is not None:
                keep &= (j - i >= -window[0]) & (j - i <= window[1])
            s = s.masked_fill(~keep, float("-inf"))
            exact = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vf)
            assert float((got.float() - exact).abs().max()) <= TOL


def test_static_scratch_reports_the_same_argument_errors(cuda):
    lib = _lib.load()
    P = ctypes.c_void_p
    one = P(4096)
    st = I64x3(64, 8, 8)
    with torch.cuda.device(cuda):
        rc = lib.trx_attn_fwd_static_scratch(one, one, one, one, None, None, 1, 8, 8, 4, 3, 128, st,
                                             st, st, st, 1.0, 0, -1, -1, 2, None, None)
    assert rc == -3  # Hq % Hk != 0, same code as trx_attn_fwd
