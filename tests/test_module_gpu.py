"""The operator under autograd and the nanochat-shaped model built on it."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def flash():
    import dism_b200
    dism_b200.install_dropin()
    import flash_dism
    return flash_dism


def test_voc_dism_gradients_match_the_oracle(flash, oracle):
    """Output and the sq/sk/v/tau gradients against the CPU oracle on the kernel's own labels; q, k and both
    codebooks get exactly zero, as on the reference's hard rows (dism_v3/tests/test_hard_training.py:69-71)."""
    import cu_flash_dism as cu
    b, n, h, d, r, dv, vocab = 2, 512, 3, 64, 32, 64, 256
    g = torch.Generator().manual_seed(21)
    leaf = lambda t: t.cuda().requires_grad_()
    q, k = (leaf(torch.randn(b, n, h, d, generator=g).bfloat16()) for _ in range(2))
    sq, sk = (leaf((torch.nn.functional.silu(torch.randn(b, n, h, r, generator=g)) * .4).bfloat16()) for _ in range(2))
    v = leaf(torch.randn(b, n, h, dv, generator=g).bfloat16())
    eq, ek = (leaf(torch.nn.functional.silu(torch.randn(h, vocab, d, generator=g))) for _ in range(2))
    tau = leaf(torch.tensor([.5, -.25, .1]))
    hard = torch.ones(b, h, dtype=torch.bool, device='cuda')
    out = flash.voc_dism(q, k, sq, sk, v, eq, ek, tau, direction=None, hard=hard)
    dout = torch.randn(b, n, h, dv, generator=g).bfloat16().cuda()
    grads = torch.autograd.grad(out, (q, k, sq, sk, v, eq, ek, tau), dout)
    f = lambda t: t.detach().float().cpu().numpy()
    iq, ik = cu.labels_pair(q.detach(), eq.detach().bfloat16(), k.detach(), ek.detach().bfloat16())
    expected, _ = oracle.forward(f(sq), f(sk), f(v), iq.cpu().numpy(), ik.cpu().numpy(), hard.cpu().numpy(), f(tau))
    torch.testing.assert_close(out.double().cpu(), torch.from_numpy(expected), atol=.008, rtol=.025)
    dsq, dsk, dvv, dtau = oracle.backward(f(sq), f(sk), f(v), f(dout), iq.cpu().numpy(), ik.cpu().numpy(), hard.cpu().numpy(), f(tau))
    for got, want in zip(grads[2:5], (dsq, dsk, dvv)):
        torch.testing.assert_close(got.double().cpu(), torch.from_numpy(want), atol=.008, rtol=.025)
    torch.testing.assert_close(grads[7].double().cpu(), torch.from_numpy(dtau), atol=.003, rtol=.01)
    for index in (0, 1, 5, 6):
        assert grads[index].shape == (q, k, sq, sk, v, eq, ek, tau)[index].shape and not grads[index].count_nonzero()
    with pytest.raises(NotImplementedError, match='soft'):
        flash.voc_dism(q, k, sq, sk, v, eq, ek, tau, direction=None, hard=torch.zeros_like(hard))


def test_model_step_updates_every_trained_parameter(flash):
    """One fwd+bwd of a small model of the benchmark's architecture: finite loss, gradients on the mixer's
    readout projections, value projection, tau and the MLP, zeros on the q/k projections and codebooks."""
    from dism_b200.model import DismLM
    torch.manual_seed(3)
    model = DismLM(depth=2, width=256, heads=2, head_dim=128, vocab=1024).cuda().bfloat16()
    tokens = torch.randint(0, 1024, (2, 512), device='cuda')
    loss = model(tokens, tokens.roll(-1, 1))
    loss.backward()
    assert torch.isfinite(loss) and abs(loss.item() - np.log(1024)) < 1.5
    mixer = model.blocks[0].mixer
    for name in ('sq_proj', 'sk_proj', 'c_v', 'c_proj'):
        grad = getattr(mixer, name).weight.grad
        assert grad is not None and torch.isfinite(grad).all() and grad.count_nonzero()
    assert mixer.log_sel_tau.grad is not None and torch.isfinite(mixer.log_sel_tau.grad).all()
    assert not mixer.q_vocab.grad.count_nonzero() and not mixer.c_q.weight.grad.count_nonzero()
    assert model.blocks[1].c_fc.weight.grad.count_nonzero() and model.embed.weight.grad.count_nonzero()
