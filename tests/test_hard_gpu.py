"""Parity of the CUDA hard path with the CPU oracle and the reference's golden vectors.

Every call goes through the drop-in modules, which forward to the C ABI of libdism_b200.so.
Tolerances are the ones the reference's own tests use (dism_v3/tests/test_hard_forward.py:54-57,80;
dism_v3/tests/test_hard_backward.py:32-38); integer stages and labels are compared bit for bit.
"""
import numpy as np
import pytest
import torch

from conftest import golden, reference_labels

pytestmark = pytest.mark.gpu

PATTERNS = ['random', 'equal', 'disjoint', 'periodic', 'boundary']


@pytest.fixture(scope='module')
def api():
    import dism_b200
    dism_b200.install_dropin()
    import cu_flash_dism as cu
    from flash_dism import summary, hard_forward, hard_backward
    return dict(cu=cu, summary=summary, fwd=hard_forward, bwd=hard_backward)


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def vectors(seed, b, n, h, r, dv):
    g = torch.Generator().manual_seed(seed)
    sq, sk = [(torch.nn.functional.silu(torch.randn(b, n, h, r, generator=g)) * .4).bfloat16() for _ in range(2)]
    v, dout = [torch.randn(b, n, h, dv, generator=g).bfloat16() for _ in range(2)]
    return sq, sk, v, dout


def assert_vectors(actual, expected, atol=.008, rtol=.025, l2=.01):
    actual, expected = actual.double().cpu(), torch.as_tensor(expected).double()
    torch.testing.assert_close(actual, expected, atol=atol, rtol=rtol)
    assert (actual - expected).norm() / expected.norm().clamp_min(1e-8) < l2


# ---- integer stages: bit-exact -----------------------------------------------------------------
@pytest.mark.parametrize('pattern', PATTERNS)
@pytest.mark.parametrize('n', [256, 512])
def test_summary_and_boundary_match_golden(api, pattern, n):
    g = golden(f'pattern_{pattern}.npz')
    iq, ik, hard = dev(g[f'iq{n}']), dev(g[f'ik{n}']), dev(g['hard'])
    for ctas in (1, 2, 0):
        summary = api['summary'].summarize_hard(iq, ik, hard, ctas=ctas)
        assert np.array_equal(summary.cpu().numpy(), g[f'summary{n}'])
    boundary = api['summary'].hard_chunk_scan(summary)
    assert np.array_equal(boundary.cpu().numpy(), g[f'boundary{n}'])
    assert np.array_equal(summary.cpu().numpy(), g[f'summary{n}'])  # input preserved
    inplace = api['summary'].hard_chunk_scan(summary, inplace=True)
    assert inplace.data_ptr() == summary.data_ptr()
    assert np.array_equal(inplace.cpu().numpy(), g[f'boundary{n}'])


@pytest.mark.parametrize('pattern', PATTERNS)
@pytest.mark.parametrize('n', [1024, 2048])
def test_summary_and_boundary_match_oracle(api, oracle, pattern, n):
    q, k = reference_labels(n, pattern)
    hard = np.array([[True, False, True], [False, True, True]])
    summary = api['summary'].summarize_hard(dev(q), dev(k), dev(hard))
    expected = oracle.summary(q, k, hard)
    assert np.array_equal(summary.cpu().numpy(), expected)
    assert np.array_equal(api['summary'].hard_chunk_scan(summary).cpu().numpy(), oracle.chunk(expected))


@pytest.mark.parametrize('n', [256, 2048])
def test_chunk_ignores_poisoned_noncausal_entries(api, oracle, n):
    rng = np.random.default_rng(63)
    source = rng.integers(-1, n, (2, 3, (n - 1) // 32, n), dtype=np.int32)
    for c in range(source.shape[2]):
        source[:, :, c, 32 * c + 32:] = np.iinfo(np.int32).max
    expected = oracle.chunk(source)
    for inplace in (False, True):
        actual = api['summary'].hard_chunk_scan(dev(source), inplace=inplace)
        assert np.array_equal(actual.cpu().numpy(), expected)


# ---- forward ---------------------------------------------------------------------------------------
@pytest.mark.parametrize('pattern', PATTERNS)
def test_forward_matches_golden(api, pattern):
    g = golden(f'pattern_{pattern}.npz')
    x = [dev(g['sq'], torch.bfloat16), dev(g['sk'], torch.bfloat16), dev(g['v'], torch.bfloat16),
         dev(g['iq256']), dev(g['ik256']), dev(g['hard']), dev(g['tau'])]
    out, norm = api['fwd'].forward_hard(*x, ctas=1)
    assert out.dtype == torch.bfloat16 and norm.dtype == torch.float32
    assert_vectors(out, g['out'])
    torch.testing.assert_close(norm.double().cpu(), torch.from_numpy(g['lse2']), atol=2e-5, rtol=2e-6)
    # the saved-state route (summary + boundary rectangle) gives the same bits as the label-only route
    out2, norm2, state = api['fwd'].forward_hard(*x, save_state=True)
    assert torch.equal(out, out2) and torch.equal(norm, norm2)
    assert np.array_equal(state['boundary'].cpu().numpy(), g['boundary256'])


@pytest.mark.parametrize('pattern', PATTERNS)
@pytest.mark.parametrize('n', [512, 1024])
def test_forward_matches_oracle(api, oracle, pattern, n):
    q, k = reference_labels(n, pattern)
    hard = np.array([[True, False, True], [False, True, True]])
    sq, sk, v, _ = vectors(417 + n, 2, n, 3, 32, 64)
    tau = torch.linspace(-.5, .5, 3)
    out, norm = api['fwd'].forward_hard(sq.cuda(), sk.cuda(), v.cuda(), dev(q), dev(k), dev(hard), tau.cuda())
    expected, lse2 = oracle.forward(sq.float().numpy(), sk.float().numpy(), v.float().numpy(), q, k, hard, tau.numpy())
    assert_vectors(out, expected)
    torch.testing.assert_close(norm.double().cpu(), torch.from_numpy(lse2), atol=2e-5, rtol=2e-6)


@pytest.mark.parametrize('n,r,dv', [(1024, 32, 64), (2048, 16, 128), (4096, 32, 32)])
def test_dense_labels_take_the_consecutive_tile_kernels(api, oracle, n, r, dv):
    """Slices where at least a tenth of all pairs match go to the dense kernel: all labels equal, a period of
    seven, two symbols at random; a slice of sparse labels and a slice that is not hard sit in the same call.  The
    reference tests these patterns for its strip stages (dism_v3/tests/test_hard_summary.py:70,
    tests/test_hard_chunk.py:39) and benchmarks equal labels (tools/bench_hard_forward.py:24-28)."""
    rng = np.random.default_rng(n)
    q, k = np.empty((2, 3, n), np.int32), np.empty((2, 3, n), np.int32)
    q[0, 0], k[0, 0] = 5, 5
    q[0, 1] = k[0, 1] = np.arange(n) % 7
    q[0, 2], k[0, 2] = rng.integers(0, 2, n), rng.integers(0, 2, n)
    q[1, 0], k[1, 0] = rng.integers(0, 300, n), rng.integers(0, 300, n)   # sparse: stays with the label-block kernel
    q[1, 1], k[1, 1] = 9, 9                                                  # dense but not hard: zeros
    q[1, 2] = np.arange(n) % 3
    k[1, 2] = (np.arange(n) + 1) % 3
    hard = np.array([[True, True, True], [True, False, True]])
    sq, sk, v, _ = vectors(n, 2, n, 3, r, dv)
    tau = torch.tensor([-.02, .3, -.6])
    out, norm = api['fwd'].forward_hard(sq.cuda(), sk.cuda(), v.cuda(), dev(q), dev(k), dev(hard), tau.cuda())
    expected, lse2 = oracle.forward(sq.float().numpy(), sk.float().numpy(), v.float().numpy(), q, k, hard, tau.numpy(), threads=8)
    assert_vectors(out, expected)
    torch.testing.assert_close(norm.double().cpu(), torch.from_numpy(lse2), atol=2e-5, rtol=2e-6)
    assert not out[1, :, 1].count_nonzero() and not norm[1, 1].count_nonzero()
    # the backward takes the same route per slice: dSQ and the tau terms by query rows, dV and dSK by key columns
    dout = vectors(n + 1, 2, n, 3, r, dv)[3]
    state = dict(boundary=None, log_weights=api['fwd'].hard_log_weights(tau.cuda(), n))
    got = api['bwd'].backward_hard(sq.cuda(), sk.cuda(), v.cuda(), dout.cuda(), dev(q), dev(k), dev(hard), norm, state)
    f = lambda t: t.float().numpy()
    want = oracle.backward(f(sq), f(sk), f(v), f(dout), q, k, hard, tau.numpy(), threads=8)
    for a, e in zip(got[:3], want[:3]):
        assert_vectors(a, e)
    torch.testing.assert_close(got[3].double().cpu(), torch.from_numpy(want[3]), atol=.003, rtol=.01)
    for gradient in got[:3]:
        assert not gradient[1, :, 1].count_nonzero()


@pytest.mark.parametrize('seed', range(16))
def test_mixed_label_kinds_against_oracle(api, oracle, seed):
    """Every (batch, head) slice of a call draws its own kind of labels: all equal, two symbols, a period of 2 to 8 with
    a shift between the sides, 12 symbols (around the dense-route threshold), 400 symbols, 5000 symbols with the keys a
    rolled copy of the queries (buckets shared by several labels, long runs).  Slices of one call so take different
    routes; forward and backward against the oracle."""
    rng = np.random.default_rng(5000 + seed)
    b, h = int(rng.integers(1, 3)), int(rng.integers(1, 4))
    n = int(rng.choice([256, 512, 768, 1024, 2048]))
    r, dv = int(rng.choice([16, 32])), int(rng.choice([32, 64, 128]))
    q, k = np.empty((b, h, n), np.int32), np.empty((b, h, n), np.int32)
    for slice_q, slice_k in zip(q.reshape(-1, n), k.reshape(-1, n)):
        kind = rng.choice(['equal', 'two', 'period', 'sparse', 'threshold', 'rolled'])
        if kind == 'equal':
            slice_q[:] = slice_k[:] = 7
        elif kind == 'two':
            slice_q[:], slice_k[:] = rng.integers(0, 2, n), rng.integers(0, 2, n)
        elif kind == 'period':
            period = int(rng.integers(2, 9))
            slice_q[:], slice_k[:] = np.arange(n) % period, (np.arange(n) + int(rng.integers(0, period))) % period
        elif kind == 'sparse':
            slice_q[:], slice_k[:] = rng.integers(0, 400, n), rng.integers(0, 400, n)
        elif kind == 'threshold':
            slice_q[:], slice_k[:] = rng.integers(0, 12, n), rng.integers(0, 12, n)
        else:
            slice_q[:] = rng.integers(0, 5000, n)
            slice_k[:] = np.roll(slice_q, int(rng.integers(0, 5)))
    hard = rng.random((b, h)) < .85
    hard[0, 0] = True
    sq, sk, v, dout = vectors(3000 + seed, b, n, h, r, dv)
    tau = torch.from_numpy(rng.uniform(-.6, .6, h).astype(np.float32))
    x = [sq.cuda(), sk.cuda(), v.cuda(), dev(q), dev(k), dev(hard)]
    out, norm = api['fwd'].forward_hard(*x, tau.cuda())
    state = dict(boundary=None, log_weights=api['fwd'].hard_log_weights(tau.cuda(), n))
    got = api['bwd'].backward_hard(*x[:3], dout.cuda(), *x[3:], norm, state)
    f = lambda t: t.float().numpy()
    expected, lse2 = oracle.forward(f(sq), f(sk), f(v), q, k, hard, tau.numpy(), threads=8)
    want = oracle.backward(f(sq), f(sk), f(v), f(dout), q, k, hard, tau.numpy(), threads=8)
    assert_vectors(out, expected)
    torch.testing.assert_close(norm.double().cpu(), torch.from_numpy(lse2), atol=2e-5, rtol=2e-6)
    for a, e in zip(got[:3], want[:3]):
        assert_vectors(a, e)
    torch.testing.assert_close(got[3].double().cpu(), torch.from_numpy(want[3]), atol=.003, rtol=.01)


def test_forward_long_chain_tau_sweep(api):
    g = golden('chain_equal.npz')
    x = [dev(g['sq'], torch.bfloat16), dev(g['sk'], torch.bfloat16), dev(g['v'], torch.bfloat16),
         dev(g['iq']), dev(g['ik']), torch.ones(1, 1, dtype=torch.bool, device='cuda')]
    for index, tau in enumerate(g['taus']):
        out, norm = api['fwd'].forward_hard(*x, torch.tensor([tau], dtype=torch.float32, device='cuda'))
        assert_vectors(out, g[f'out{index}'])
        torch.testing.assert_close(norm.double().cpu(), torch.from_numpy(g[f'lse2_{index}']), atol=2e-5, rtol=2e-6)


@pytest.mark.parametrize('r,dv', [(16, 32), (16, 64), (32, 32), (32, 64), (32, 128), (16, 128)])
def test_forward_backward_dimensions(api, oracle, r, dv):
    n = 512
    q, k = reference_labels(n, 'periodic')
    hard = np.array([[True, False, True], [False, True, True]])
    sq, sk, v, dout = vectors(5 + r + dv, 2, n, 3, r, dv)
    tau = torch.linspace(-.5, .5, 3)
    x = [sq.cuda(), sk.cuda(), v.cuda(), dev(q), dev(k), dev(hard)]
    out, norm, state = api['fwd'].forward_hard(*x, tau.cuda(), ctas=2, save_state=True)
    f = lambda t: t.float().numpy()
    expected, lse2 = oracle.forward(f(sq), f(sk), f(v), q, k, hard, tau.numpy())
    assert_vectors(out, expected)
    torch.testing.assert_close(norm.double().cpu(), torch.from_numpy(lse2), atol=2e-5, rtol=2e-6)
    got = api['bwd'].backward_hard(*x[:3], dout.cuda(), *x[3:], norm, state)
    want = oracle.backward(f(sq), f(sk), f(v), f(dout), q, k, hard, tau.numpy())
    for a, e in zip(got[:3], want[:3]):
        assert_vectors(a, e)
    torch.testing.assert_close(got[3].double().cpu(), torch.from_numpy(want[3]), atol=.003, rtol=.01)


@pytest.mark.parametrize('seed', range(12))
def test_random_shapes_against_oracle(api, oracle, seed):
    """Seeded random shapes, label densities (2 to 600 symbols: dense buckets with many key steps and long
    runs, down to buckets of one position), hard flags and tau signs: forward and backward against the oracle,
    with and without the reference's boundary rectangle."""
    rng = np.random.default_rng(1000 + seed)
    b, h = int(rng.integers(1, 4)), int(rng.integers(1, 5))
    n = int(rng.choice([256, 512, 768]))
    r, dv = int(rng.choice([16, 32])), int(rng.choice([32, 64, 128]))
    symbols = int(rng.choice([2, 5, 40, 600]))
    q = rng.integers(0, symbols, (b, h, n)).astype(np.int32)
    k = rng.integers(0, symbols, (b, h, n)).astype(np.int32)
    start = int(rng.integers(0, n // 2))
    k[:, :, start:start + n // 4] = q[:, :, start + 3:start + 3 + n // 4]  # a planted run of n/4
    hard = rng.random((b, h)) < .8
    hard[0, 0] = True
    sq, sk, v, dout = vectors(2000 + seed, b, n, h, r, dv)
    tau = torch.from_numpy(rng.uniform(-.6, .6, h).astype(np.float32))
    x = [sq.cuda(), sk.cuda(), v.cuda(), dev(q), dev(k), dev(hard)]
    save = bool(seed % 2)
    result = api['fwd'].forward_hard(*x, tau.cuda(), ctas=int(rng.choice([0, 1, 7])), save_state=save)
    out, norm = result[0], result[1]
    state = result[2] if save else dict(boundary=None, log_weights=api['fwd'].hard_log_weights(tau.cuda(), n))
    f = lambda t: t.float().numpy()
    expected, lse2 = oracle.forward(f(sq), f(sk), f(v), q, k, hard, tau.numpy())
    assert_vectors(out, expected)
    torch.testing.assert_close(norm.double().cpu(), torch.from_numpy(lse2), atol=2e-5, rtol=2e-6)
    got = api['bwd'].backward_hard(*x[:3], dout.cuda(), *x[3:], norm, state)
    want = oracle.backward(f(sq), f(sk), f(v), f(dout), q, k, hard, tau.numpy())
    for a, e in zip(got[:3], want[:3]):
        assert_vectors(a, e)
    torch.testing.assert_close(got[3].double().cpu(), torch.from_numpy(want[3]), atol=.003, rtol=.01)


def test_forward_exactness_properties(api):
    g = golden('pattern_boundary.npz')
    x = [dev(g['sq'], torch.bfloat16), dev(g['sk'], torch.bfloat16), dev(g['v'], torch.bfloat16),
         dev(g['iq256']), dev(g['ik256']), dev(g['hard']), dev(g['tau'])]
    out, norm = api['fwd'].forward_hard(*x, ctas=1)
    for ctas in (2, 0, 7):  # grid size never changes a bit
        o, m = api['fwd'].forward_hard(*x, ctas=ctas)
        assert torch.equal(o, out) and torch.equal(m, norm)
    x[0] = -x[0]  # flipping sq flips the output exactly and leaves the normaliser alone
    flipped, flipped_norm = api['fwd'].forward_hard(*x, ctas=1)
    assert torch.equal(flipped, -out) and torch.equal(flipped_norm, norm)
    x[0] = torch.zeros_like(x[0])
    zero, zero_norm = api['fwd'].forward_hard(*x)
    assert not zero.count_nonzero() and torch.equal(zero_norm, norm)
    x[3], x[4] = torch.full_like(x[3], 1), torch.full_like(x[4], 2)  # disjoint labels: nothing matches
    zero, zero_norm = api['fwd'].forward_hard(*x)
    assert not zero.count_nonzero() and not zero_norm.count_nonzero()
    x[5] = torch.zeros_like(x[5])  # all soft: operands are never read
    for item in x[:3]:
        item.fill_(float('nan'))
    zero, zero_norm = api['fwd'].forward_hard(*x)
    assert not zero.count_nonzero() and not zero_norm.count_nonzero()


def test_forward_is_causal(api):
    n = 512
    q, k = reference_labels(n, 'equal')
    sq, sk, v, _ = vectors(3, 2, n, 3, 32, 64)
    hard, tau = torch.ones(2, 3, dtype=torch.bool, device='cuda'), torch.linspace(-.5, .5, 3).cuda()
    x = [sq.cuda(), sk.cuda(), v.cuda(), dev(q), dev(k), hard, tau]
    original, _ = api['fwd'].forward_hard(*x)
    x[2][:, 127:] = 20
    changed, _ = api['fwd'].forward_hard(*x)
    assert torch.equal(original[:, :127], changed[:, :127])


# ---- backward --------------------------------------------------------------------------------------
@pytest.mark.parametrize('pattern', PATTERNS)
def test_backward_matches_golden(api, pattern):
    g = golden(f'pattern_{pattern}.npz')
    x = [dev(g['sq'], torch.bfloat16), dev(g['sk'], torch.bfloat16), dev(g['v'], torch.bfloat16),
         dev(g['iq256']), dev(g['ik256']), dev(g['hard'])]
    dout = dev(g['dout'], torch.bfloat16)
    _, norm, state = api['fwd'].forward_hard(*x, dev(g['tau']), save_state=True, ctas=1)
    got = api['bwd'].backward_hard(*x[:3], dout, *x[3:], norm, state, ctas=1)
    assert got[0].dtype == torch.float32 and got[1].dtype == torch.bfloat16 and got[2].dtype == torch.bfloat16
    for a, name in zip(got[:3], ('dsq', 'dsk', 'dv')):
        assert torch.isfinite(a).all()
        assert_vectors(a, g[name])
        assert not a.masked_select(~x[5][:, None, :, None]).count_nonzero()  # soft rows: exact zeros
    torch.testing.assert_close(got[3].double().cpu(), torch.from_numpy(g['dtau']), atol=.003, rtol=.01)
    # label-only route (no rectangle) and any grid size give the same bits
    for ctas in (0, 3):
        again = api['bwd'].backward_hard(*x[:3], dout, *x[3:], norm, dict(boundary=None, log_weights=state['log_weights']),
                                         ctas=ctas)
        assert all(torch.equal(a, b) for a, b in zip(got, again))
    recomputed = api['bwd'].backward_hard_recompute(*x[:3], dout, *x[3:], dev(g['tau']))
    assert all(torch.equal(a, recomputed[key]) for a, key in zip(got, ('sq_vec', 'sk_vec', 'v', 'rtau')))


def test_backward_tau_long_chain(api):
    g = golden('chain_equal.npz')
    x = [dev(g['sq'], torch.bfloat16), dev(g['sk'], torch.bfloat16), dev(g['v'], torch.bfloat16),
         dev(g['iq']), dev(g['ik']), torch.ones(1, 1, dtype=torch.bool, device='cuda')]
    dout = dev(g['dout'], torch.bfloat16)
    for index, tau in enumerate(g['taus']):
        t = torch.tensor([tau], dtype=torch.float32, device='cuda')
        _, norm, state = api['fwd'].forward_hard(*x, t, save_state=True)
        got = api['bwd'].backward_hard(*x[:3], dout, *x[3:], norm, state)
        torch.testing.assert_close(got[3].double().cpu(), torch.from_numpy(g[f'dtau{index}']), atol=.003, rtol=.01)
        assert_vectors(got[0], g[f'dsq{index}'])


def test_backward_all_soft_is_zero(api):
    g = golden('pattern_random.npz')
    x = [dev(g['sq'], torch.bfloat16), dev(g['sk'], torch.bfloat16), dev(g['v'], torch.bfloat16),
         dev(g['iq256']), dev(g['ik256']), torch.zeros(2, 3, dtype=torch.bool, device='cuda')]
    _, norm, state = api['fwd'].forward_hard(*x, dev(g['tau']), save_state=True)
    got = api['bwd'].backward_hard(*x[:3], dev(g['dout'], torch.bfloat16), *x[3:], norm, state)
    assert all(not t.count_nonzero() for t in got)


def test_backward_reuses_the_forward_index(api):
    """The backward takes the position index that travels on the normaliser of the readout of the same label
    tensors: same bits as a rebuilt index; labels written in place, other label tensors or another forward's
    normaliser are not served."""
    b, n, h, r, dv = 2, 1024, 3, 32, 64
    sq, sk, v, dout = (t.cuda() for t in vectors(5, b, n, h, r, dv))
    g = torch.Generator().manual_seed(6)
    iq, ik = (torch.randint(0, 40, (b, h, n), generator=g, dtype=torch.int32).cuda() for _ in range(2))
    hard = torch.ones(b, h, dtype=torch.bool, device='cuda')
    tau = torch.full((h,), .3, device='cuda')
    cu = api['cu']

    def both(iq, ik):
        out, norm = api['fwd'].forward_hard(sq, sk, v, iq, ik, hard, tau)
        lut = api['fwd'].hard_log_weights(tau, n)
        return norm, api['bwd'].backward_hard(sq, sk, v, dout, iq, ik, hard, norm, dict(boundary=None, log_weights=lut))

    norm, shared = both(iq, ik)
    assert cu._recall_index(norm, iq, ik) is not None
    cu.share_index(False)
    try:
        unshared_norm, rebuilt = both(iq, ik)
        assert cu._recall_index(unshared_norm, iq, ik) is None
    finally:
        cu.share_index(True)
    assert all(torch.equal(a, e) for a, e in zip(shared, rebuilt))
    norm, _ = both(iq, ik)
    assert cu._recall_index(norm.clone(), iq, ik) is None  # the index belongs to one readout's normaliser
    iq[0, 1, 7] += 1                       # in place: the index that travelled with the normaliser is stale
    assert cu._recall_index(norm, iq, ik) is None
    norm, _ = both(iq, ik)
    assert cu._recall_index(norm, iq.clone(), ik) is None  # another tensor, even with the same values
    lut = api['fwd'].hard_log_weights(tau, n)
    _, fresh = both(iq, ik)
    again = api['bwd'].backward_hard(sq, sk, v, dout, iq.clone(), ik.clone(), hard, _, dict(boundary=None, log_weights=lut))
    assert all(torch.equal(a, e) for a, e in zip(fresh, again))


# ---- the route word of a captured graph ----------------------------------------------------------------
@pytest.mark.parametrize('kind', ['random', 'equal'])
def test_route_word_opens_and_closes_a_captured_graph(api, kind):
    """`_graph_choice` (dism_v3/include/common/graph_route.cuh:8-13): word 0 runs the path and gives the bits of a
    call without it; any other value makes every kernel return, which leaves the zero-filled outputs.  The word is
    read when the kernels run, so one captured graph follows what was written before each replay (the use in
    dism_v3/tests/test_planner_graph.py:403-433).  `equal` labels take the dense kernels, `random` the tile kernels."""
    b, n, h, r, dv = 2, 512, 2, 16, 64
    sq, sk, v, dout = (t.cuda() for t in vectors(21, b, n, h, r, dv))
    g = torch.Generator().manual_seed(22)
    if kind == 'random':
        iq, ik = (torch.randint(0, 9, (b, h, n), generator=g, dtype=torch.int32).cuda() for _ in range(2))
    else:
        iq, ik = (torch.full((b, h, n), 3, dtype=torch.int32, device='cuda') for _ in range(2))
    hard = torch.ones(b, h, dtype=torch.bool, device='cuda')
    tau = torch.tensor([.3, -.2], device='cuda')

    def call(choice):
        out, norm, state = api['fwd'].forward_hard(sq, sk, v, iq, ik, hard, tau, save_state=True, _graph_choice=choice)
        grads = api['bwd'].backward_hard(sq, sk, v, dout, iq, ik, hard, norm, state, _graph_choice=choice)
        return [out, norm, *grads], state['boundary']

    expected, boundary = call(None)
    choice = torch.zeros(1, dtype=torch.int32, device='cuda')
    opened, opened_boundary = call(choice)
    assert all(torch.equal(a, e) for a, e in zip(opened, expected)) and torch.equal(opened_boundary, boundary)
    choice.fill_(7)
    closed, _ = call(choice)
    assert all(not t.any() for t in closed)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call(choice)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        replayed, replayed_boundary = call(choice)
    for selected in (0, 5, 0, 1):
        choice.fill_(selected)
        graph.replay()
        torch.cuda.synchronize()
        if selected == 0:
            assert all(torch.equal(a, e) for a, e in zip(replayed, expected)) and torch.equal(replayed_boundary, boundary)
        else:
            assert all(not t.any() for t in replayed)

    for wrong in (torch.zeros(1, dtype=torch.int64, device='cuda'), torch.zeros(2, dtype=torch.int32, device='cuda'),
                  torch.zeros(1, dtype=torch.int32)):
        with pytest.raises(RuntimeError, match='graph choice'):
            api['fwd'].hard_log_weights(tau, n, _graph_choice=wrong)


# ---- the CPU-runnable reference configuration --------------------------------------------------------
def test_config1_reference_case(api, oracle):
    g = golden('config1.npz')
    bf = lambda a: dev(a, torch.bfloat16)
    # labels: the kernel's pinned accumulation order against the CPU restatement, bit for bit, and
    # against the reference's fp32 arg-max where the operands are bf16-exact
    q, k, eq, ek = bf(g['q']), bf(g['k']), bf(g['eq']), bf(g['ek'])
    f = lambda t: t.float().cpu().numpy()
    iq, ik = api['cu'].labels(q, eq), api['cu'].labels(k, ek)
    assert np.array_equal(iq.cpu().numpy(), oracle.labels(f(q), f(eq)))
    assert np.array_equal(ik.cpu().numpy(), oracle.labels(f(k), f(ek)))
    # hard path on the reference's own labels
    hard = torch.ones(1, 2, dtype=torch.bool, device='cuda')
    x = [bf(g['sq']), bf(g['sk']), bf(g['v']), dev(g['iq']), dev(g['ik']), hard]
    out, norm, state = api['fwd'].forward_hard(*x, dev(g['tau']), save_state=True)
    lengths = oracle.lengths(g['iq'][0, 0], g['ik'][0, 0])
    c = 3
    row = 32 * c + 31
    assert np.array_equal(np.arange(row + 1) - state['boundary'][0, 0, c, :row + 1].cpu().numpy(), lengths[row, :row + 1])
    # fp32 fixture inputs are rounded to bf16 for the kernel: compare with the oracle on the rounded values
    expected, lse2 = oracle.forward(f(x[0]), f(x[1]), f(x[2]), g['iq'], g['ik'], np.ones((1, 2), bool), g['tau'])
    assert_vectors(out, expected)
    torch.testing.assert_close(norm.double().cpu(), torch.from_numpy(lse2), atol=2e-5, rtol=2e-6)
    torch.testing.assert_close(norm.double().cpu(), torch.from_numpy(g['lse2']), atol=2e-5, rtol=2e-6)
    assert_vectors(out, g['out'], atol=.02, rtol=.05, l2=.02)  # vs the fp32-input reference run


def test_labels_bit_exact_and_ties(api, oracle):
    g = torch.Generator().manual_seed(11)
    x = torch.randn(2, 300, 3, 64, generator=g).bfloat16()
    e = torch.nn.functional.silu(torch.randn(3, 512, 64, generator=g)).bfloat16()
    got = api['cu'].labels(x.cuda(), e.cuda())
    assert np.array_equal(got.cpu().numpy(), oracle.labels(x.float().numpy(), e.float().numpy()))
    reference = torch.argmax(torch.einsum('bnhd,hvd->bnhv', x.float(), e.float()), -1).transpose(1, 2)
    assert (got.cpu() != reference).float().mean() < 1e-3  # near-ties only
    zero = api['cu'].labels(torch.zeros_like(x).cuda(), e.cuda())  # all ties: the lowest index wins
    assert not zero.count_nonzero()


def labels_fault():
    import ctypes
    from dism_b200 import _lib
    code = ctypes.c_int(-1)
    _lib.check(_lib.load().dism_labels_fault(ctypes.byref(code)))
    return code.value


@pytest.mark.parametrize('shape', [(2, 1024, 4, 64, 512), (1, 256, 2, 128, 256), (3, 128, 5, 64, 128),
                                   (1, 2048, 3, 64, 1024), (2, 640, 16, 128, 512), (1, 27 * 128, 7, 64, 384)])
def test_labels_tensor_memory_pipeline(api, oracle, shape):
    """Shapes the tcgen05 pipeline covers (D 64/128, V a multiple of 256, N a multiple of 128) and neighbours
    that fall back to the mma.sync kernel (V 128, 384): bit-exact labels, including duplicated codes (exact
    ties: the lowest index), near ties and zero rows."""
    b, n, h, d, v = shape
    g = torch.Generator().manual_seed(b * 1000 + n + v)
    x = torch.randn(b, n, h, d, generator=g).bfloat16()
    e = torch.nn.functional.silu(torch.randn(h, v, d, generator=g)).bfloat16()
    e[:, v // 2] = e[:, 3]          # exact duplicates
    e[:, v - 1] = e[:, 0]
    x[0, 5] = 0                     # all logits equal
    x[-1, n - 1, h - 1] = 0
    x[0, 7] = e[:, 3] * 4           # rows aligned with a duplicated code
    got = api['cu'].labels(x.cuda(), e.cuda())
    assert labels_fault() == 0
    assert np.array_equal(got.cpu().numpy(), oracle.labels(x.float().numpy(), e.float().numpy()))
    again = api['cu'].labels(x.cuda(), e.cuda())
    assert torch.equal(got, again)


@pytest.mark.parametrize('shape', [(2, 1024, 4, 64, 512), (1, 256, 2, 128, 256), (3, 128, 5, 64, 128), (1, 384, 3, 64, 512)])
def test_labels_pair_equals_two_calls(api, oracle, shape):
    """Two tensors of one shape in one launch (q with its codebook, k with its own): the bits of two single calls,
    on shapes the tensor-memory pipeline covers and on one it hands to the mma.sync kernel."""
    b, n, h, d, v = shape
    g = torch.Generator().manual_seed(b * 77 + n + v)
    xq, xk = (torch.randn(b, n, h, d, generator=g).bfloat16().cuda() for _ in range(2))
    eq, ek = (torch.nn.functional.silu(torch.randn(h, v, d, generator=g)).bfloat16().cuda() for _ in range(2))
    xk[0, 3] = 0                    # all logits equal: label 0
    ek[:, v - 1] = ek[:, 1]         # exact duplicate: the lower index wins
    iq, ik = api['cu'].labels_pair(xq, eq, xk, ek)
    assert labels_fault() == 0
    assert torch.equal(iq, api['cu'].labels(xq, eq)) and torch.equal(ik, api['cu'].labels(xk, ek))
    assert np.array_equal(ik.cpu().numpy(), oracle.labels(xk.float().cpu().numpy(), ek.float().cpu().numpy()))


def test_labels_tensor_memory_pipeline_all_ties(api):
    """Every row inside the margin bound: the per-warp lists overflow and rows are recomputed in place."""
    x = torch.zeros(1, 4096, 2, 64).bfloat16()
    e = torch.randn(2, 128, 64, generator=torch.Generator().manual_seed(5)).bfloat16()
    got = api['cu'].labels(x.cuda(), e.cuda())
    assert labels_fault() == 0 and not got.count_nonzero()
    # a scaled code as the row: the arg-max is that code or an earlier duplicate
    x = (e[:, :64].transpose(0, 1).reshape(1, 64, 2, 64) * 2).repeat(1, 2, 1, 1).contiguous()
    got = api['cu'].labels(x.cuda(), e.cuda()).cpu()
    reference = torch.argmax(torch.einsum('bnhd,hvd->bnhv', x.float(), e.float()), -1).transpose(1, 2)
    assert (got != reference).float().mean() < .02


def test_bounded_wait_gives_up_and_reports(api):
    """A wait that nothing satisfies runs out, reports its code, and leaves the context usable."""
    import ctypes
    from dism_b200 import _lib
    lib = _lib.load()
    assert labels_fault() == 0
    outcome = (ctypes.c_int * 2)(-1, -1)
    _lib.check(lib.dism_labels_wait_selftest(77, outcome, None))
    assert list(outcome) == [0, 0]
    assert labels_fault() == 77
    assert labels_fault() == 0  # reading clears it
    x = torch.randn(1, 256, 2, 64).bfloat16().cuda()
    e = torch.randn(2, 256, 64).bfloat16().cuda()
    reference = torch.argmax(torch.einsum('bnhd,hvd->bnhv', x.float(), e.float()), -1).transpose(1, 2)
    assert (api['cu'].labels(x, e) != reference).float().mean() < 1e-2 and labels_fault() == 0


# ---- the two weight tables by themselves -----------------------------------------------------------------
@pytest.mark.parametrize('n', [256, 2048])
def test_log_weight_table_against_the_closed_form(api, oracle, n):
    """lut[h, l] = log2 sum_{s=1..l} exp(s tau[h]) in FP64, at the reference's tolerance for the same table
    (dism_v3/tests/test_hard_forward.py:60-71), and against the oracle's FP32 restatement."""
    tau = torch.tensor([-4., -.5, -1e-6, -1e-12, 0., 1e-12, 1e-6, .5, 4.])
    table = api['fwd'].hard_log_weights(tau.cuda(), n).cpu()
    assert table.shape == (9, n + 1) and (table[:, 0] == -1e6).all()
    length = np.arange(1, n + 1, dtype=np.float64)
    t = tau.double().numpy()[:, None]
    with np.errstate(divide='ignore', invalid='ignore'):
        expected = (np.where(t > 0, length * t, t) + np.log(-np.expm1(-length * np.abs(t))) - np.log(-np.expm1(-np.abs(t)))) / np.log(2.)
    expected[tau.numpy() == 0] = np.log2(length)
    np.testing.assert_allclose(table[:, 1:].double().numpy(), expected, atol=2e-5, rtol=2e-6)
    np.testing.assert_allclose(table.numpy(), oracle.lut(tau.numpy(), n), atol=2e-5, rtol=2e-6)


def test_dlog_weight_table_against_the_moment_sums(api):
    """g[h, l] = d ln W_l / d tau = sum s e^{s tau} / sum e^{s tau}, summed directly in FP64 (the formula of
    dism_v3/docs/HARD_BACKWARD_QUADRATIC.md:60-75); the table the backward builds from the log2 table."""
    from dism_b200 import _lib
    n = 2048
    tau = torch.tensor([-4., -.5, -.01, -1e-4, -1e-6, 0., 1e-6, 1e-4, .01, .5, 4.])
    table = api['fwd'].hard_log_weights(tau.cuda(), n)
    out = torch.full_like(table, float('nan'))
    _lib.check(_lib.load().dism_hard_dlog_weights(table.data_ptr(), tau.numel(), n + 1, out.data_ptr(),
                                                  torch.cuda.current_stream().cuda_stream))
    got = out.cpu().double().numpy()
    assert (got[:, 0] == 0).all()
    s = np.arange(1, n + 1, dtype=np.float64)
    lower = np.tril(np.ones((n, n)))
    for row, t in enumerate(tau.double().numpy()):
        # weights of row l scaled by their largest (s = l for tau > 0, s = 1 otherwise): nothing overflows or vanishes
        scaled = np.exp(np.minimum((s[None, :] - (s[:, None] if t > 0 else 1.)) * t, 0.)) * lower
        expected = (scaled * s[None, :]).sum(1) / scaled.sum(1)
        np.testing.assert_allclose(got[row, 1:], expected, rtol=2e-4, atol=2e-4, err_msg=f'tau {t}')


# ---- symbol streams: single longest earlier match -----------------------------------------------------
def symbol_streams(batch, n, vocab, seed):
    rng = np.random.default_rng(seed)
    out = np.empty((batch, n), np.int32)
    for b in range(batch):
        s = list(rng.integers(0, vocab, 512))
        while len(s) < n:
            length = int(rng.integers(16, 513))
            if rng.random() < .5:
                start = int(rng.integers(0, len(s)))
                for t in range(length):  # may run into what it is writing, like a real self-copy
                    s.append(s[start + t])
            else:
                s.extend(rng.integers(0, vocab, length))
        out[b] = s[:n]
    return out


def test_longest_match_symbol_streams(api, oracle):
    streams = symbol_streams(4, 4096, 256, 0)
    end, length, nxt = api['cu'].longest_match(dev(streams))
    for b in range(4):
        e, l, x = oracle.longest(streams[b])
        assert np.array_equal(end[b].cpu().numpy(), e)
        assert np.array_equal(length[b].cpu().numpy(), l)
        assert np.array_equal(nxt[b].cpu().numpy(), x)


# ---- validation ------------------------------------------------------------------------------------------
def test_validation_errors(api):
    g = golden('pattern_random.npz')
    x = [dev(g['sq'], torch.bfloat16), dev(g['sk'], torch.bfloat16), dev(g['v'], torch.bfloat16),
         dev(g['iq256']), dev(g['ik256']), dev(g['hard']), dev(g['tau'])]
    out, norm, state = api['fwd'].forward_hard(*x, save_state=True)
    with pytest.raises(RuntimeError, match='too short'):
        api['fwd'].hard_readout(*x[:6], state['boundary'], state['log_weights'][:, :128].contiguous())
    with pytest.raises(RuntimeError, match='boundary'):
        api['fwd'].hard_readout(*x[:6], state['boundary'].float(), state['log_weights'])
    with pytest.raises(RuntimeError, match='token-level'):
        api['fwd'].forward_hard(*x[:5], x[5][:, :, None].expand(2, 3, 256), x[6])
    with pytest.raises(RuntimeError, match='CTA'):
        api['summary'].summarize_hard(x[3], x[4], x[5], ctas=-1)
    for bad in (x[3].long(), x[3].cpu(), x[3][:, :, :255], x[3][:, :, ::2]):
        with pytest.raises(RuntimeError):
            api['summary'].summarize_hard(bad, x[4], x[5])
    with pytest.raises(RuntimeError, match='sequence hard flags'):
        api['bwd'].backward_hard(*x[:3], x[2], *x[3:5], x[5][:, :, None].expand_as(x[3]).contiguous(), norm, state)
    with pytest.raises(RuntimeError, match='head'):
        api['summary'].hard_chunk_scan(state['summary'], heads=5)


# ---- packed documents ----------------------------------------------------------------------------------
def packed_case(api, pattern):
    from flash_dism.varlen import VarlenLayout
    n = 2048
    q, k = reference_labels(n, pattern, b=1, h=2)
    sq, sk, v, dout = vectors(77, 1, n, 2, 32, 64)
    x = [sq.cuda(), sk.cuda(), v.cuda(), dev(q), dev(k), torch.tensor([[True, False], [False, True]], device='cuda'),
         torch.tensor([.5, -.25], device='cuda')]
    offsets = [0, 0, 256, 512, 1024, 1024, 2048]
    layout = VarlenLayout.from_cu_seqlens(torch.tensor(offsets, dtype=torch.int32), n)
    return x, dout.cuda(), layout, [(a, z) for a, z in zip(offsets, offsets[1:]) if z > a]


def document(x, dout, start, end):
    return ([t[:, start:end].contiguous() for t in x[:3]] + [t[:, :, start:end].contiguous() for t in x[3:5]] +
            [x[5][start // 1024:start // 1024 + 1].contiguous(), x[6]], dout[:, start:end].contiguous())


@pytest.mark.parametrize('pattern', ['random', 'equal', 'periodic', 'boundary'])
def test_packed_documents_match_fixed_length(api, oracle, pattern):
    x, dout, layout, spans = packed_case(api, pattern)
    out, norm = api['fwd'].forward_hard(*x, layout=layout, ctas=1)
    grads = api['bwd'].backward_hard_recompute(*x[:3], dout, *x[3:], layout=layout)
    dtau = torch.zeros(2, device='cuda')
    # Dense label patterns take the consecutive-position kernels, packed or not; whether a slice does depends on its
    # share of matching pairs, which differs between the pack and a stand-alone document, so such patterns are
    # compared at the tolerance of the oracle tests.
    close = dict(atol=1e-3, rtol=2 ** -7) if pattern == 'random' else dict(atol=.008, rtol=.025)
    for start, end in spans:
        local, local_dout = document(x, dout, start, end)
        want, want_norm = api['fwd'].forward_hard(*local)
        # same pairs in the same order; only the grouping of keys into tensor-core steps differs between the
        # packed and the stand-alone run, so outputs agree to about one bf16 unit in the last place
        torch.testing.assert_close(out[:, start:end].float(), want.float(), **close)
        torch.testing.assert_close(norm[:, :, start:end], want_norm, atol=2e-5, rtol=2e-6)
        local_grads = api['bwd'].backward_hard_recompute(*local[:3], local_dout, *local[3:])
        for name in ('sq_vec', 'sk_vec', 'v'):  # the normalisers above differ in their last bits, so do these
            torch.testing.assert_close(grads[name][:, start:end].float(), local_grads[name].float(), **close)
        dtau += local_grads['rtau']
        f = lambda t: t.float().cpu().numpy()
        expected, _ = oracle.forward(f(local[0]), f(local[1]), f(local[2]), local[3].cpu().numpy(), local[4].cpu().numpy(),
                                     local[5].cpu().numpy(), f(local[6]))
        assert_vectors(want, expected)
    torch.testing.assert_close(grads['rtau'], dtau, atol=2e-3, rtol=1e-4)  # same terms, different summation tree
    # a change inside the first document leaves the later ones untouched
    x[2][:, :256] += 5
    changed, changed_norm = api['fwd'].forward_hard(*x, layout=layout)
    assert torch.equal(changed[:, 256:], out[:, 256:]) and torch.equal(changed_norm, norm)


@pytest.mark.parametrize('seed', range(8))
def test_packed_random_documents_match_stand_alone_runs(api, seed):
    """Random 256-aligned document splits of a pack, each head with its own kind of labels (equal, two symbols, a period,
    many symbols): forward and backward of the pack against every document run by itself."""
    from flash_dism.varlen import VarlenLayout
    rng = np.random.default_rng(7000 + seed)
    n, h, r, dv = 2048, 3, 32, 64
    q, k = np.empty((1, h, n), np.int32), np.empty((1, h, n), np.int32)
    for head in range(h):
        kind = rng.choice(['equal', 'two', 'period', 'sparse'])
        if kind == 'equal':
            q[0, head] = k[0, head] = 3
        elif kind == 'two':
            q[0, head], k[0, head] = rng.integers(0, 2, n), rng.integers(0, 2, n)
        elif kind == 'period':
            q[0, head], k[0, head] = np.arange(n) % 5, (np.arange(n) + 2) % 5
        else:
            q[0, head], k[0, head] = rng.integers(0, 300, n), rng.integers(0, 300, n)
    # documents end at the training rows' borders (1024) and at random multiples of 256 inside them
    cuts = sorted({0, 1024, 2048} | {int(c) * 256 for c in rng.integers(1, 8, 3)})
    layout = VarlenLayout.from_cu_seqlens(torch.tensor(cuts, dtype=torch.int32), n)
    sq, sk, v, dout = vectors(90 + seed, 1, n, h, r, dv)
    hard = torch.from_numpy(rng.random((2, h)) < .8).cuda()
    tau = torch.from_numpy(rng.uniform(-.5, .5, h).astype(np.float32)).cuda()
    x = [sq.cuda(), sk.cuda(), v.cuda(), dev(q), dev(k), hard, tau]
    out, norm = api['fwd'].forward_hard(*x, layout=layout)
    grads = api['bwd'].backward_hard_recompute(*x[:3], dout.cuda(), *x[3:], layout=layout)
    dtau = torch.zeros(h, device='cuda')
    for start, end in zip(cuts, cuts[1:]):
        local, local_dout = document(x, dout.cuda(), start, end)
        want, want_norm = api['fwd'].forward_hard(*local)
        torch.testing.assert_close(out[:, start:end].float(), want.float(), atol=.008, rtol=.025)
        torch.testing.assert_close(norm[:, :, start:end], want_norm, atol=2e-5, rtol=2e-6)
        local_grads = api['bwd'].backward_hard_recompute(*local[:3], local_dout, *local[3:])
        for name in ('sq_vec', 'sk_vec', 'v'):
            torch.testing.assert_close(grads[name][:, start:end].float(), local_grads[name].float(), atol=.008, rtol=.025)
        dtau += local_grads['rtau']
    torch.testing.assert_close(grads['rtau'], dtau, atol=3e-3, rtol=1e-3)


@pytest.mark.parametrize('n,symbols', [(8192, 12), (16384, 11)])
def test_packed_long_buckets_match_stand_alone_runs(api, n, symbols):
    """A long pack over few symbols (just under the share of matching pairs that would send it to the dense kernels):
    buckets hold hundreds to more than a thousand keys of many documents, so the warp-wide search for a tile's
    document range takes two and three rounds.  The pack against every document run by itself."""
    from flash_dism.varlen import VarlenLayout
    rng = np.random.default_rng(n + symbols)
    h, r, dv = 2, 16, 32
    q, k = (rng.integers(0, symbols, (1, h, n)).astype(np.int32) for _ in range(2))
    rows = n // 4096
    cuts = sorted({4096 * row for row in range(rows + 1)} | {int(c) * 256 for c in rng.integers(1, n // 256, 9)})
    layout = VarlenLayout.from_cu_seqlens(torch.tensor(cuts, dtype=torch.int32), n)
    sq, sk, v, dout = (t.cuda() for t in vectors(n, 1, n, h, r, dv))
    hard = torch.ones(rows, h, dtype=torch.bool, device='cuda')
    tau = torch.tensor([.2, -.3], device='cuda')
    x = [sq, sk, v, dev(q), dev(k), hard, tau]
    out, norm = api['fwd'].forward_hard(*x, layout=layout)
    grads = api['bwd'].backward_hard_recompute(*x[:3], dout, *x[3:], layout=layout)
    dtau = torch.zeros(h, device='cuda')
    for start, end in zip(cuts, cuts[1:]):
        local = ([t[:, start:end].contiguous() for t in x[:3]] + [t[:, :, start:end].contiguous() for t in x[3:5]] +
                 [hard[:1].contiguous(), tau])
        want, want_norm = api['fwd'].forward_hard(*local)
        torch.testing.assert_close(out[:, start:end].float(), want.float(), atol=.008, rtol=.025)
        torch.testing.assert_close(norm[:, :, start:end], want_norm, atol=2e-5, rtol=2e-6)
        local_grads = api['bwd'].backward_hard_recompute(*local[:3], dout[:, start:end].contiguous(), *local[3:])
        for name in ('sq_vec', 'sk_vec', 'v'):
            torch.testing.assert_close(grads[name][:, start:end].float(), local_grads[name].float(), atol=.008, rtol=.025)
        dtau += local_grads['rtau']
    torch.testing.assert_close(grads['rtau'], dtau, atol=3e-2, rtol=2e-3)


def test_packed_saved_state_gives_the_same_bits(api):
    """forward_hard(save_state=True) with a layout returns the packed rectangle (what the reference's forward always
    builds); readout and backward accept it and give the bits of the label-only route."""
    x, dout, layout, spans = packed_case(api, 'periodic')
    out, norm = api['fwd'].forward_hard(*x, layout=layout)
    out2, norm2, state = api['fwd'].forward_hard(*x, layout=layout, save_state=True)
    assert torch.equal(out, out2) and torch.equal(norm, norm2)
    assert state['boundary'].dim() == 1 and state['boundary'].numel() == sum(2 * ((z - a - 1) // 32) * (z - a) for a, z in spans)
    plain = api['bwd'].backward_hard(*x[:3], dout, *x[3:6], norm, dict(boundary=None, log_weights=state['log_weights']), layout=layout)
    saved = api['bwd'].backward_hard(*x[:3], dout, *x[3:6], norm2, state, layout=layout)
    assert all(torch.equal(a, e) for a, e in zip(plain, saved))
    with pytest.raises(RuntimeError, match='boundary'):
        api['fwd'].hard_readout(*x[:6], state['boundary'][:-1].contiguous(), state['log_weights'], layout=layout)


@pytest.mark.parametrize('seed', range(3))
def test_packed_summary_and_chunk_equal_the_documents_own(api, seed):
    """Many documents of random lengths in one pack, three heads with runs of different lengths, mixed hard flags: the
    packed summary and composition (one launch each) against the fixed-length kernels run document by document, bit
    for bit; in place and with a capped grid too."""
    from flash_dism.varlen import VarlenLayout
    rng = np.random.default_rng(400 + seed)
    n, h, rows = 8192, 3, 4
    q = np.stack([rng.integers(0, s, n) for s in (2, 3, 40)])[None].astype(np.int32)
    k = np.stack([rng.integers(0, s, n) for s in (2, 3, 40)])[None].astype(np.int32)
    cuts = sorted({2048 * row for row in range(rows + 1)} | {int(c) * 256 for c in rng.integers(1, n // 256, 14)})
    cuts = cuts[:3] + [cuts[2]] + cuts[3:]  # an empty document among them
    layout = VarlenLayout.from_cu_seqlens(torch.tensor(cuts, dtype=torch.int32), n)
    hard = torch.from_numpy(rng.random((rows, h)) < .7).cuda()
    iq, ik = dev(q), dev(k)
    summary = api['summary'].summarize_hard(iq, ik, hard, layout=layout)
    capped = api['summary'].summarize_hard(iq, ik, hard, layout=layout, ctas=3)
    boundary = api['summary'].hard_chunk_scan(summary, layout=layout, heads=h)
    want_summary, want_boundary = [], []
    for start, end in zip(cuts, cuts[1:]):
        if end > start:
            flags = hard[start // 2048:start // 2048 + 1].contiguous()
            local = api['summary'].summarize_hard(iq[:, :, start:end].contiguous(), ik[:, :, start:end].contiguous(), flags)
            want_summary.append(local.flatten())
            want_boundary.append(api['summary'].hard_chunk_scan(local).flatten())
    assert torch.equal(summary, torch.cat(want_summary)) and torch.equal(capped, summary)
    assert torch.equal(boundary, torch.cat(want_boundary))
    inplace = api['summary'].hard_chunk_scan(summary, layout=layout, heads=h, inplace=True)
    assert inplace.data_ptr() == summary.data_ptr() and torch.equal(inplace, boundary)


def test_packed_summary_chunk_and_errors(api, oracle):
    x, dout, layout, spans = packed_case(api, 'boundary')
    summary = api['summary'].summarize_hard(x[3], x[4], x[5], layout=layout)
    boundary = api['summary'].hard_chunk_scan(summary, layout=layout, heads=2)
    expected = []
    for start, end in spans:
        flags = x[5][start // 1024:start // 1024 + 1].cpu().numpy()
        expected.append(oracle.boundary_numpy(x[3][:, :, start:end].cpu().numpy(), x[4][:, :, start:end].cpu().numpy(),
                                              flags).ravel())
    assert np.array_equal(boundary.cpu().numpy(), np.concatenate(expected))
    from flash_dism.varlen import VarlenLayout
    whole = VarlenLayout.from_cu_seqlens(torch.tensor([0, 2048], dtype=torch.int32), 2048)
    with pytest.raises(RuntimeError, match='cross a hard training-row'):
        api['fwd'].forward_hard(*x, layout=whole)
    with pytest.raises(RuntimeError, match='aligned'):
        VarlenLayout.from_cu_seqlens(torch.tensor([0, 100, 2048], dtype=torch.int32), 2048)
    empty = VarlenLayout.from_cu_seqlens(torch.tensor([0, 0, 0], dtype=torch.int32), 0)
    assert api['summary'].hard_chunk_scan(torch.empty(0, device='cuda', dtype=torch.int32), layout=empty, heads=2).numel() == 0
