"""Full-size checks at the benchmark shape (B8 H16 N8192 R32 DV64, labels over 512 symbols).

The dense oracle is run on a few (batch, head) slices; the rest is covered by size-independent
properties: sign-flip antisymmetry, grid-size invariance, and linearity of the gradients in dO.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def workload():
    import dism_b200
    dism_b200.install_dropin()
    from flash_dism import hard_forward, hard_backward
    b, h, n, r, dv = 8, 16, 8192, 32, 64
    g = torch.Generator(device='cuda').manual_seed(0)
    sq, sk = [(torch.nn.functional.silu(torch.randn(b, n, h, r, generator=g, device='cuda')) * .4).bfloat16()
              for _ in range(2)]
    v, dout = [torch.randn(b, n, h, dv, generator=g, device='cuda').bfloat16() for _ in range(2)]
    iq, ik = [torch.randint(0, 512, (b, h, n), generator=g, device='cuda', dtype=torch.int32) for _ in range(2)]
    # plant a long copy so that run lengths beyond one strip are exercised
    ik[:, :, 5000:6000] = iq[:, :, 5100:6100]
    hard = torch.ones(b, h, dtype=torch.bool, device='cuda')
    hard[1, 2] = False
    tau = torch.full((h,), .5, device='cuda')
    return dict(fwd=hard_forward, bwd=hard_backward, x=[sq, sk, v, iq, ik, hard], tau=tau, dout=dout)


def test_full_size_forward_and_backward(workload, oracle):
    w = workload
    sq, sk, v, iq, ik, hard = w['x']
    out, norm = w['fwd'].forward_hard(*w['x'], w['tau'])
    lut = w['fwd'].hard_log_weights(w['tau'], sq.shape[1])
    grads = w['bwd'].backward_hard(sq, sk, v, w['dout'], iq, ik, hard, norm, dict(boundary=None, log_weights=lut))
    f = lambda t, b, h: t[b:b + 1, :, h:h + 1].float().cpu().numpy()
    for b, h in ((0, 0), (7, 15), (1, 2)):
        lab = lambda t: t[b:b + 1, h:h + 1].cpu().numpy()
        flags = hard[b:b + 1, h:h + 1].cpu().numpy()
        tau = w['tau'][h:h + 1].cpu().numpy()
        expected, lse2 = oracle.forward(f(sq, b, h), f(sk, b, h), f(v, b, h), lab(iq), lab(ik), flags, tau)
        got = out[b:b + 1, :, h:h + 1].double().cpu()
        torch.testing.assert_close(got, torch.from_numpy(expected), atol=.008, rtol=.025)
        torch.testing.assert_close(norm[b:b + 1, h:h + 1].double().cpu(), torch.from_numpy(lse2), atol=2e-5, rtol=2e-6)
        want = oracle.backward(f(sq, b, h), f(sk, b, h), f(v, b, h), f(w['dout'], b, h), lab(iq), lab(ik), flags, tau)
        for a, e in zip(grads[:3], want[:3]):
            a = a[b:b + 1, :, h:h + 1].double().cpu()
            torch.testing.assert_close(a, torch.from_numpy(e), atol=.008, rtol=.025)
            assert (a - torch.from_numpy(e)).norm() / torch.from_numpy(e).norm().clamp_min(1e-8) < .01
    assert not out[1, :, 2].count_nonzero() and not grads[2][1, :, 2].count_nonzero()
    # properties over the whole tensor
    flipped, flipped_norm = w['fwd'].forward_hard(-sq, sk, v, iq, ik, hard, w['tau'], ctas=64)
    assert torch.equal(flipped, -out) and torch.equal(flipped_norm, norm)
    doubled = w['bwd'].backward_hard(sq, sk, v, (w['dout'].float() * 2).bfloat16(), iq, ik, hard, norm,
                                     dict(boundary=None, log_weights=lut), ctas=100)
    # scaling dO by a power of two scales dSQ and dV exactly, except where FP32 partial sums are subnormal
    assert (doubled[0] - grads[0] * 2).abs().max() < 1e-30
    assert (doubled[2].float() - grads[2].float() * 2).abs().max() < 1e-30


def test_long_context_with_planted_runs(oracle):
    """Long-context shape in miniature: N = 32768, and every 4096 positions a 1024-long window of
    query labels repeats an earlier window of key labels, so run lengths reach 1024."""
    import dism_b200
    dism_b200.install_dropin()
    from flash_dism import hard_forward
    b, h, n, r, dv = 1, 2, 32768, 32, 64
    g = torch.Generator().manual_seed(4)
    sq, sk = [(torch.nn.functional.silu(torch.randn(b, n, h, r, generator=g)) * .4).bfloat16() for _ in range(2)]
    v = torch.randn(b, n, h, dv, generator=g).bfloat16()
    iq, ik = [torch.randint(0, 512, (b, h, n), generator=g, dtype=torch.int32) for _ in range(2)]
    rng = np.random.default_rng(4)
    for start in range(4096, n, 4096):
        target = start + int(rng.integers(0, 3072))
        source = int(rng.integers(0, target - 1024))
        iq[:, :, target:target + 1024] = ik[:, :, source:source + 1024]
    hard = torch.ones(b, h, dtype=torch.bool)
    tau = torch.tensor([.05, -.2])
    out, norm = hard_forward.forward_hard(sq.cuda(), sk.cuda(), v.cuda(), iq.cuda(), ik.cuda(), hard.cuda(), tau.cuda())
    f = lambda t: t.float().numpy()
    expected, lse2 = oracle.forward(f(sq), f(sk), f(v), iq.numpy(), ik.numpy(), hard.numpy(), tau.numpy(), threads=2)
    torch.testing.assert_close(out.double().cpu(), torch.from_numpy(expected), atol=.008, rtol=.025)
    torch.testing.assert_close(norm.double().cpu(), torch.from_numpy(lse2), atol=2e-5, rtol=2e-6)
    assert lse2.max() > 30  # the planted runs dominate their rows' normalisers


def test_full_size_discretiser(oracle):
    """The tcgen05 discretiser at the benchmark shape: the oracle on three (batch, head) slices; over the whole
    tensor, agreement with an fp32 arg-max up to near ties, and three exact properties: the same labels
    on a second call, under scaling of x by a power of two (every logit scales exactly in both summation
    orders), and under a permutation of the codebook (labels map through the permutation)."""
    import ctypes
    import dism_b200
    dism_b200.install_dropin()
    import cu_flash_dism as cu
    from dism_b200 import _lib
    b, n, h, d, v = 8, 8192, 16, 64, 512
    g = torch.Generator(device='cuda').manual_seed(3)
    x = torch.randn(b, n, h, d, generator=g, device='cuda').bfloat16()
    e = torch.nn.functional.silu(torch.randn(h, v, d, generator=g, device='cuda')).bfloat16()
    got = cu.labels(x, e)
    code = ctypes.c_int(-1)
    _lib.check(_lib.load().dism_labels_fault(ctypes.byref(code)))
    assert code.value == 0
    for bi, hi in ((0, 0), (7, 15), (3, 9)):
        want = oracle.labels(x[bi:bi + 1, :, hi:hi + 1].float().cpu().numpy(), e[hi:hi + 1].float().cpu().numpy())
        assert np.array_equal(got[bi:bi + 1, hi:hi + 1].cpu().numpy(), want)
    mismatches = 0
    for bi in range(b):
        reference = torch.argmax(torch.einsum('nhd,hvd->hnv', x[bi].float(), e.float()), -1)
        mismatches += int((reference != got[bi]).sum())
    assert mismatches < 1e-3 * got.numel()
    assert torch.equal(cu.labels(x, e), got)
    assert torch.equal(cu.labels((x.float() * 4).bfloat16(), e), got)
    permutation = torch.randperm(v, generator=torch.Generator().manual_seed(4)).cuda()
    permuted = cu.labels(x, e[:, permutation].contiguous())
    assert int((permutation[permuted.long()] != got).sum()) <= 2  # exact ties between two codes may resolve differently
