"""The allocation-free attention entry point, called through the C ABI.

Some callers of this library have no way to allocate device memory when they run a layer (a fixed memory
plan, a host process that owns the allocator). et_attention_static_scores serves them from a score buffer
built into the library. This file checks it against et_attention_otf on two calls in a row, the second with
other inputs and a shorter sequence so that whatever the first call left in the shared buffer cannot help.
Both are also compared with the fp32 CPU oracle. It is collected last so that a run stopping at the first failure has already executed every other test.
"""
import ctypes

import numpy as np
import pytest

from tests import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _p(t):
    return ctypes.c_void_p(None if t is None else t.data_ptr())


def test_static_score_attention_matches_on_the_fly_twice():
    import et_b200 as et
    L = et.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    d, H = 768, 12
    for call, (seq, seed) in enumerate([(256, 1), (100, 2)]):
        q, k, v = (torch.from_numpy(util.activations(seed * 10 + i, (seq, d))).cuda() for i in range(3))
        mask = torch.from_numpy((util.rng(seed).standard_normal((seq, seq)) * 0.5).astype(np.float16)).cuda()
        want = torch.full((seq, d), float("nan"), dtype=torch.float16, device="cuda")
        got = torch.full((seq, d), float("nan"), dtype=torch.float16, device="cuda")
        et.check(L.et_attention_otf(_p(want), _p(q), _p(k), _p(v), _p(mask), seq, d, H, stream))
        et.check(L.et_attention_static_scores(_p(got), _p(q), _p(k), _p(v), _p(mask), seq, d, H, stream))
        torch.cuda.synchronize()
        # the scores pass through fp16 once more than in the on-the-fly kernel; same tolerance as every
        # fp16-vs-oracle comparison of this suite
        util.assert_close(got.float().cpu().numpy(), want.float().cpu().numpy(),
                          what=f"static-score attention, call {call}")
        from tests import oracle_lib
        ref = oracle_lib.load().attention(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), [seq], d, H,
                                          mask=mask.float().cpu().numpy())
        util.assert_close(got.float().cpu().numpy(), ref, what=f"static-score attention vs the oracle, call {call}")


def test_static_score_attention_rejects_oversize():
    import et_b200 as et
    L = et.lib()
    x = torch.zeros((8, 64), dtype=torch.float16, device="cuda")
    rc = L.et_attention_static_scores(_p(x), _p(x), _p(x), _p(x), None, 1024, 1024, 16, None)
    assert rc == 3   # ET_ERR_UNSUPPORTED: 16 * 1024 * 1024 elements do not fit the built-in buffer
    assert b"exceeds" in L.et_last_error()
