"""The allocation-free estimator entry point (minf_vs_estimate_static).

It exists for callers that cannot give the library scratch memory: an attention plugin living in
a process whose device memory is one pre-carved arena, or code on a path where calling an
allocator is forbidden.  Its scratch is a fixed array inside the library's device image, so the
test (a) calls it through the C ABI exactly like the buffer-taking entry point, (b) checks that
both produce the same index lists, and (c) does so twice in a row with different sizes, because
the second call sees whatever the first one left in the shared array.

This file is collected last on purpose (run `pytest --collect-only`): a run that stops at the
first failure has then already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _estimate(lib, cabi, q, k, vsize, ssize, static: bool):
    B, H, N, D = q.shape
    dev = q.device
    cap_v, cap_s = min(N, max(vsize, 30)), min(N, max(ssize, 50))
    vs = torch.full((B * H,), vsize, dtype=torch.int32, device=dev)
    ss = torch.full((B * H,), ssize, dtype=torch.int32, device=dev)
    v_idx = torch.full((B, H, cap_v), -7, dtype=torch.int32, device=dev)
    s_idx = torch.full((B, H, cap_s), -7, dtype=torch.int32, device=dev)
    nnz_v = torch.zeros(B * H, dtype=torch.int32, device=dev)
    nnz_s = torch.zeros(B * H, dtype=torch.int32, device=dev)
    status = cabi.new_status(dev)
    common = [cabi.ptr(q), cabi.ptr(k), cabi.strides3(q), cabi.strides3(k), B, H, k.shape[1], N, D,
              cabi.ptr(vs), cabi.ptr(ss), cap_v, cap_s, cabi.ptr(v_idx), cabi.ptr(s_idx), cabi.ptr(nnz_v), cabi.ptr(nnz_s)]
    stream = cabi.stream_ptr(dev)
    if static:
        rc = lib.minf_vs_estimate_static(*common, cabi.ptr(status), stream)
    else:
        scratch = torch.empty(lib.minf_vs_estimate_scratch_bytes(B, H, N), dtype=torch.uint8, device=dev)
        rc = lib.minf_vs_estimate(*common, None, None, cabi.ptr(scratch), cabi.ptr(status), stream)
    cabi.check(rc)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    return v_idx.cpu(), s_idx.cpu(), nnz_v.cpu(), nnz_s.cpu()


def test_static_scratch_estimator_matches_buffer_version_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from minference_b200 import _cabi
    from minference_b200.synthetic import make_qkv

    lib = _cabi.lib()
    limit = lib.minf_vs_estimate_static_scratch_limit()
    assert limit == 16 << 20
    # two calls in a row; the second is smaller, so stale scores of the first lie beyond and inside its range
    for (n, hq, hkv, vsize, ssize, seed) in [(4096, 4, 2, 200, 500, 21), (1500, 2, 1, 64, 128, 22)]:
        q, k, _ = make_qkv(n, hq, hkv, seed=seed, dtype=torch.bfloat16)
        q, k = q.cuda(), k.cuda()
        assert lib.minf_vs_estimate_scratch_bytes(1, hq, n) <= limit
        want = _estimate(lib, _cabi, q, k, vsize, ssize, static=False)
        got = _estimate(lib, _cabi, q, k, vsize, ssize, static=True)
        for a, b in zip(got, want):
            assert torch.equal(a, b)        # same kernels, same arithmetic: identical index lists
    # a problem beyond the built-in scratch is refused with a clear message, nothing runs
    n_big = 1 << 20
    assert lib.minf_vs_estimate_scratch_bytes(1, 8, n_big) > limit
    one = ctypes.c_void_p(256)
    st = (ctypes.c_int64 * 3)(n_big * 128 * 8, n_big * 128, 128)
    rc = lib.minf_vs_estimate_static(one, one, st, st, 1, 8, 8, n_big, 128, one, one, 1000, 6096,
                                     one, one, one, one, one, None)
    assert rc == -3 and b"built-in scratch" in lib.minf_last_error()
