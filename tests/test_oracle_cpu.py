"""The CPU checker against the reference: golden vectors produced by the reference's own Python
(tests/golden/make_golden.py), the reference's native CPU forward when it was built, and
independent numpy restatements of the integer stages.  No GPU needed."""
import numpy as np
import pytest

from conftest import golden, reference_labels

PATTERNS = ['random', 'equal', 'disjoint', 'periodic', 'boundary']


@pytest.mark.parametrize('pattern', PATTERNS)
def test_integer_stages_match_reference_fixtures(oracle, pattern):
    g = golden(f'pattern_{pattern}.npz')
    for n in (256, 512):
        iq, ik = g[f'iq{n}'], g[f'ik{n}']
        summary = oracle.summary(iq, ik, g['hard'])
        assert np.array_equal(summary, g[f'summary{n}'])
        assert np.array_equal(oracle.chunk(summary), g[f'boundary{n}'])
        assert np.array_equal(oracle.summary_numpy(iq, ik, g['hard']), summary)
        assert np.array_equal(oracle.boundary_numpy(iq, ik, g['hard']), g[f'boundary{n}'])
        q, k = reference_labels(n, pattern)  # the recipe used for sizes that have no stored fixture
        assert np.array_equal(q, iq) and np.array_equal(k, ik)


@pytest.mark.parametrize('pattern', PATTERNS)
def test_forward_backward_match_reference_fixtures(oracle, pattern):
    g = golden(f'pattern_{pattern}.npz')
    iq, ik = g['iq256'], g['ik256']
    out, lse2 = oracle.forward(g['sq'], g['sk'], g['v'], iq, ik, g['hard'], g['tau'], threads=2)
    np.testing.assert_allclose(out, g['out'], atol=2e-6, rtol=1e-5)  # fixtures store float32
    np.testing.assert_allclose(lse2, g['lse2'], atol=1e-12)
    dsq, dsk, dv, dtau = oracle.backward(g['sq'], g['sk'], g['v'], g['dout'], iq, ik, g['hard'], g['tau'], threads=2)
    np.testing.assert_allclose(dsq, g['dsq'], atol=5e-6, rtol=1e-5)
    np.testing.assert_allclose(dsk, g['dsk'], atol=5e-6, rtol=1e-5)
    np.testing.assert_allclose(dv, g['dv'], atol=5e-6, rtol=1e-5)
    np.testing.assert_allclose(dtau, g['dtau'], atol=1e-6, rtol=1e-8)


def test_reference_cpu_case(oracle):
    """fp32 q,k,v [1,256,2,64] from seed 0, labels by the reference's arg-max, every row hard."""
    g = golden('config1.npz')
    hard = np.ones((1, 2), bool)
    assert np.array_equal(oracle.labels(g['q'], g['eq']), g['iq'])  # no near-tie in this fixture
    assert np.array_equal(oracle.labels(g['k'], g['ek']), g['ik'])
    out, lse2 = oracle.forward(g['sq'], g['sk'], g['v'], g['iq'], g['ik'], hard, g['tau'])
    np.testing.assert_allclose(out, g['out'], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(lse2, g['lse2'], atol=1e-12)
    dsq, dsk, dv, dtau = oracle.backward(g['sq'], g['sk'], g['v'], g['dout'], g['iq'], g['ik'], hard, g['tau'])
    np.testing.assert_allclose(dv, g['dv'], atol=5e-6, rtol=1e-5)
    np.testing.assert_allclose(dtau, g['dtau'], atol=1e-9, rtol=1e-9)
    lengths = oracle.lengths(g['iq'][0, 1], g['ik'][0, 1])
    boundary = oracle.chunk(oracle.summary(g['iq'], g['ik'], hard))
    for c in range(7):
        row = 32 * c + 31
        assert np.array_equal(np.arange(row + 1) - boundary[0, 1, c, :row + 1], lengths[row, :row + 1])


def test_long_chain_tau_sweep(oracle):
    g = golden('chain_equal.npz')
    hard = np.ones((1, 1), bool)
    for index, tau in enumerate(g['taus']):
        t = np.array([tau], np.float32)
        out, lse2 = oracle.forward(g['sq'], g['sk'], g['v'], g['iq'], g['ik'], hard, t)
        np.testing.assert_allclose(out, g[f'out{index}'], atol=2e-6, rtol=1e-5)
        np.testing.assert_allclose(lse2, g[f'lse2_{index}'], atol=1e-11)
        dtau = oracle.backward(g['sq'], g['sk'], g['v'], g['dout'], g['iq'], g['ik'], hard, t)[3]
        np.testing.assert_allclose(dtau, g[f'dtau{index}'], rtol=1e-7, atol=1e-9)


def test_lut_matches_closed_form(oracle):
    tau = np.array([-4., -.5, -1e-6, -1e-12, 0., 1e-12, 1e-6, .5, 4.], np.float32)
    n = 2048
    table = oracle.lut(tau, n)
    assert (table[:, 0] == -1e6).all()
    length = np.arange(1, n + 1, dtype=np.float64)
    t = tau.astype(np.float64)[:, None]
    a = np.abs(t)
    with np.errstate(divide='ignore', invalid='ignore'):
        expected = (np.where(t > 0, length * t, t) + np.log(-np.expm1(-length * a)) - np.log(-np.expm1(-a))) / np.log(2.)
    expected[tau == 0] = np.log2(length)
    np.testing.assert_allclose(table[:, 1:], expected, atol=2e-5, rtol=2e-6)


def test_against_reference_native_forward(oracle):
    if oracle.reference_lib() is None:
        pytest.skip('the reference native CPU forward was not built in this checkout')
    rng = np.random.default_rng(5)
    n, r, dv = 768, 32, 64
    iq, ik = rng.integers(0, 12, (1, 1, n), dtype=np.int32), rng.integers(0, 12, (1, 1, n), dtype=np.int32)
    ik[0, 0, 300:500] = iq[0, 0, 310:510]  # a long run
    sq, sk = [oracle.bf16_round(rng.standard_normal((1, n, 1, r)).astype(np.float32) * .3) for _ in range(2)]
    v = oracle.bf16_round(rng.standard_normal((1, n, 1, dv)).astype(np.float32))
    for tau in (-.7, 0., .4):
        out, lse2 = oracle.forward(sq, sk, v, iq, ik, np.ones((1, 1), bool), np.array([tau], np.float32))
        want, want_lse2 = oracle.reference_forward(sq[0, :, 0], sk[0, :, 0], v[0, :, 0], iq[0, 0], ik[0, 0],
                                                   float(np.float32(tau)))
        np.testing.assert_allclose(out[0, :, 0], want, atol=1e-11)
        np.testing.assert_allclose(lse2[0, 0], want_lse2, atol=1e-11)


def test_longest_match_against_brute_force(oracle):
    rng = np.random.default_rng(3)
    s = rng.integers(0, 4, 300).astype(np.int32)
    s[200:260] = s[50:110]
    end, length, nxt = oracle.longest(s)
    lengths = oracle.lengths(s, s)
    for i in range(len(s)):
        row = lengths[i, :i]
        best = row.max() if i else 0
        if best == 0:
            assert end[i] == -1 and length[i] == 0 and nxt[i] == -1
        else:
            j = int(np.nonzero(row == best)[0].max())
            assert (end[i], length[i], nxt[i]) == (j, best, s[j + 1])


def test_edge_cases(oracle):
    n = 256
    q = np.full((1, 1, n), np.iinfo(np.int32).min, np.int32)
    k = np.full((1, 1, n), np.iinfo(np.int32).max, np.int32)
    ones = np.ones((1, n, 1, 32), np.float32)
    out, lse2 = oracle.forward(ones, ones, np.ones((1, n, 1, 64), np.float32), q, k, np.ones((1, 1), bool),
                               np.array([.5], np.float32))
    assert not out.any() and not lse2.any()  # disjoint labels: only the unit fallback remains
    out, lse2 = oracle.forward(ones, ones, np.ones((1, n, 1, 64), np.float32), q, q, np.zeros((1, 1), bool),
                               np.array([.5], np.float32))
    assert not out.any() and not lse2.any()  # soft rows are skipped


def test_longest_match_length_against_reference_planner(oracle):
    """The one part of the single-longest-match quantity the reference defines: max_j L(i,j), which its decode
    planner keeps as max_length (inference/csrc/planner.hpp:132-149, :253-270: suffix-automaton match over the
    snapshot, diagonal band over the tail).  Self-matching streams exclude j = i, so the planner gets the stream
    delayed by one position as its keys; the two-sided form is checked against the dense L as well."""
    rng = np.random.default_rng(11)
    if oracle.reference_longest_lengths(np.zeros(4, np.int32), np.zeros(4, np.int32)) is None:
        pytest.skip('the reference planner was not built in this checkout')
    for n, vocab in ((300, 3), (2048, 4), (1000, 50), (512, 1)):
        s = rng.integers(0, vocab, n).astype(np.int32)
        if n == 2048:
            s[700:1200] = s[100:600]
        end, length, nxt = oracle.longest(s)
        delayed = np.concatenate([[-1], s[:-1]]).astype(np.int32)
        for interval in (16, 64):
            np.testing.assert_array_equal(oracle.reference_longest_lengths(delayed, s, interval), length)
        q, k = rng.integers(0, vocab, 384).astype(np.int32), rng.integers(0, vocab, 384).astype(np.int32)
        k[200:300] = q[210:310]
        np.testing.assert_array_equal(oracle.reference_longest_lengths(k, q, 32), oracle.lengths(q, k).max(1))
