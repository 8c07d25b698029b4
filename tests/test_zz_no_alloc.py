"""dism_hard_readout_static, the readout for callers that have no scratch memory to give.

A host that calls the operator with only input and output buffers (a serving hook, a process whose
pool already owns the GPU) cannot pass a workspace and must not trigger cudaMalloc in the call.
This entry point keeps its scratch inside the library; the test calls it through the C ABI twice in
a row and expects exactly the output of dism_hard_readout, which is given a caller-owned workspace.
The file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def operands(seed, b, n, h, r, dv):
    g = torch.Generator().manual_seed(seed)
    sq, sk = [(torch.nn.functional.silu(torch.randn(b, n, h, r, generator=g)) * .4).bfloat16().cuda() for _ in range(2)]
    v = torch.randn(b, n, h, dv, generator=g).bfloat16().cuda()
    iq, ik = [torch.randint(0, 24, (b, h, n), generator=g, dtype=torch.int32).cuda() for _ in range(2)]
    ik[:, :, 300:420] = iq[:, :, 310:430]  # a run longer than a strip
    hard = torch.ones(b, h, dtype=torch.bool).cuda()
    hard[0, 1] = False
    tau = torch.linspace(-.4, .6, h).cuda()
    return sq, sk, v, iq, ik, hard, tau


def test_static_readout_matches_workspace_readout_twice():
    from dism_b200 import _lib
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, b, n, h) in enumerate(((3, 2, 512, 3), (4, 1, 1024, 2))):
        r, dv = 32, 64
        sq, sk, v, iq, ik, hard, tau = operands(seed, b, n, h, r, dv)
        lut = torch.empty(h, n + 1, dtype=torch.float32, device='cuda')
        _lib.check(lib.dism_hard_log_weights(tau.data_ptr(), h, n, lut.data_ptr(), stream))
        want, want_norm = torch.empty(b, n, h, dv, dtype=torch.bfloat16, device='cuda'), torch.empty(b, h, n, device='cuda')
        size = lib.dism_hard_readout_workspace(b, h, n)
        workspace = torch.empty(size, dtype=torch.uint8, device='cuda')
        _lib.check(lib.dism_hard_readout(sq.data_ptr(), sk.data_ptr(), v.data_ptr(), iq.data_ptr(), ik.data_ptr(),
                                         hard.data_ptr(), None, None, b, n, lut.data_ptr(), n + 1, b, n, h, r, dv, 0,
                                         want.data_ptr(), want_norm.data_ptr(), workspace.data_ptr(), size, stream))
        got, got_norm = torch.full_like(want, float('nan')), torch.full_like(want_norm, float('nan'))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0] if call else None  # the first call on a device may load the array
        status = lib.dism_hard_readout_static(sq.data_ptr(), sk.data_ptr(), v.data_ptr(), iq.data_ptr(), ik.data_ptr(),
                                              hard.data_ptr(), None, lut.data_ptr(), n + 1, b, n, h, r, dv, 0,
                                              got.data_ptr(), got_norm.data_ptr(), stream)
        assert status == 0, lib.dism_hard_readout_static_error().decode()
        torch.cuda.synchronize()
        if call:  # a later call leaves the device's free memory exactly as it found it
            assert torch.cuda.mem_get_info()[0] == free_before
        # the same kernels on the same inputs: the hard-path tests compare such runs bit for bit
        assert torch.equal(got, want), f'call {call}: output differs'
        assert torch.equal(got_norm, want_norm), f'call {call}: normaliser differs'
        assert got.count_nonzero() and not got[0, :, 1].count_nonzero()
        # and against the CPU oracle, at the tolerances of the forward tests
        from oracle import dism_oracle
        f = lambda t: t.float().cpu().numpy()
        expected, lse2 = dism_oracle.forward(f(sq), f(sk), f(v), iq.cpu().numpy(), ik.cpu().numpy(), hard.cpu().numpy(), f(tau))
        torch.testing.assert_close(got.double().cpu(), torch.from_numpy(expected), atol=.008, rtol=.025)
        torch.testing.assert_close(got_norm.double().cpu(), torch.from_numpy(lse2), atol=2e-5, rtol=2e-6)


def test_static_readout_rejects_shapes_beyond_its_scratch():
    from dism_b200 import _lib
    lib = _lib.load()
    p = ctypes.c_void_p(4096)  # never dereferenced: the size check comes first
    status = lib.dism_hard_readout_static(p, p, p, p, p, p, None, p, 8193, 8, 8192, 16, 32, 64, 0, p, p, None)
    assert status == 1
    message = lib.dism_hard_readout_static_error().decode()
    assert 'built-in scratch' in message and 'dism_hard_readout' in message
