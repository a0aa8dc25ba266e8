"""The backward entry point for callers that cannot allocate (att3_sg_backward_static).

Some hosts of the library cannot give the backward a scratch buffer because they may not
call an allocator where the kernel is launched: code inside a framework's capture-private
memory pool, a real-time loop with a fixed device-memory plan, a sandboxed worker.  For them
the scratch is a fixed 32 MiB array inside the library.  This test calls that entry point
through the C ABI twice in a row and checks both results against the regular entry point
(which takes a caller-allocated workspace) on the same inputs: they must be bit-identical,
the second call must not be disturbed by what the first left in the shared array, and sizes
beyond the array must be refused with a clear message.  Collected last on purpose, so a run
that stops at the first failure has already run everything else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, Hq, Hkv, N, D, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    Q = torch.randn(B, Hq, N, D, generator=g).to(torch.bfloat16).cuda()
    kv = [torch.randn(B, Hkv, N, D, generator=g).to(torch.bfloat16).cuda() for _ in range(4)]
    dY = torch.randn(B, Hq, N, D, generator=g).to(torch.bfloat16).cuda()
    return Q, kv, dY


def _static_backward(lib, dY, Q, kv, Y, m, l, mask, window):
    B, Hq, N, D = Q.shape
    outs = [torch.full_like(Q, float("nan"))] + [torch.full_like(kv[0], float("nan")) for _ in range(4)]
    rc = lib.att3_sg_backward_static(dY.data_ptr(), Q.data_ptr(), *[t.data_ptr() for t in kv], Y.data_ptr(),
                                     m.data_ptr(), l.data_ptr(), None if mask is None else mask.data_ptr(),
                                     *[o.data_ptr() for o in outs], B, Hq, kv[0].shape[1], N, D, window, 0,
                                     torch.cuda.current_stream().cuda_stream)
    return rc, outs


def test_static_scratch_backward_matches_workspace_backward_twice():
    from att3ntion_b200 import _cabi, _cuda_kernels as ck
    lib = _cabi.lib
    assert lib.att3_sg_backward_static_max_bytes() == 32 << 20
    # two different problems back to back: the second must not see the first one's leftovers
    for (B, Hq, Hkv, N, D, w, seed) in [(2, 8, 1, 400, 128, 128, 1), (1, 4, 2, 272, 64, 32, 2)]:
        Q, kv, dY = _inputs(B, Hq, Hkv, N, D, seed)
        Y, m, l = ck.sg_forward_raw(Q, *kv, None, w)
        ref = ck.sg_backward_raw(dY, Q, *kv, Y, m, l, None, w)
        for _ in range(2):
            rc, outs = _static_backward(lib, dY, Q, kv, Y, m, l, None, w)
            assert rc == _cabi.OK, _cabi.last_error()
            ck.device_status()
            for a, b in zip(outs, ref):
                assert torch.equal(a, b)


def test_static_scratch_rejects_sizes_beyond_the_array():
    from att3ntion_b200 import _cabi
    lib = _cabi.lib
    Q, kv, dY = _inputs(1, 1, 1, 16, 128, 0)
    Y, m, l = torch.empty_like(Q), torch.empty(1, 1, 16, device="cuda"), torch.empty(1, 1, 16, device="cuda")
    # declared sizes only matter for the check: 16 * 4 * 8192 * 128 bytes = 64 MiB > 32 MiB, refused before any launch
    rc = lib.att3_sg_backward_static(dY.data_ptr(), Q.data_ptr(), *[t.data_ptr() for t in kv], Y.data_ptr(),
                                     m.data_ptr(), l.data_ptr(), None, *[Q.data_ptr()] * 5,
                                     4, 8, 1, 8192, 128, 128, 0, None)
    assert rc == _cabi.ERR_WORKSPACE
    assert "built-in array" in _cabi.last_error() and "33554432" in _cabi.last_error()
    rc = lib.att3_sg_backward_static(dY.data_ptr(), Q.data_ptr(), *[t.data_ptr() for t in kv], Y.data_ptr(),
                                     m.data_ptr(), l.data_ptr(), None, *[Q.data_ptr()] * 5,
                                     1, 1, 1, 16, 128, 0, 0, None)
    assert rc == _cabi.ERR_INVALID and "windowed" in _cabi.last_error()
