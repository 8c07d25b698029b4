"""Generate the golden vectors under tests/golden/ by running the reference's own Python.

Run once in a container that has the reference checkout (the REFERENCE_ROOT environment variable, or
the default below); the resulting .npz files are committed and are what the test-suite reads, so
nothing at test time needs the checkout.  What is executed here is reference code only:
  * flash_dism/reference/dism_v3_ref.py  dism_ref / dism_ref_backward in float64 (forward output,
    dSQ/dSK/dV/dtau);
  * tests/test_hard_summary.py  labels() and oracle()  (label patterns, strip summaries);
  * tests/test_hard_chunk.py    dense_boundary()       (composed boundaries);
  * tests/test_hard_forward.py  normalizer_oracle()    (log2 normaliser).
The reference package imports its native extension at import time; a stub module of that name
is registered first (no native code of the reference runs), and Tensor.cuda is made the
identity because the reference's test helpers move their results to a GPU.
"""
import os
import sys
import types

import numpy as np
import torch

ROOT = os.environ.get('REFERENCE_ROOT', '/root/reference')
HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference():
    stub = types.ModuleType('cu_flash_dism')
    stub.fp32_enabled = lambda: False
    stub.configs = {}
    sys.modules['cu_flash_dism'] = stub
    sys.path.insert(0, os.path.join(ROOT, 'dism_v3', 'python'))
    sys.path.insert(0, os.path.join(ROOT, 'dism_v3', 'tests'))
    torch.Tensor.cuda = lambda self, *a, **k: self
    import test_hard_summary, test_hard_chunk, test_hard_forward
    from flash_dism.reference import dism_v3_ref
    return test_hard_summary, test_hard_chunk, test_hard_forward, dism_v3_ref


def bf16(x):
    return x.bfloat16().float()


def run_reference(ref, sq, sk, v, iq, ik, hard, tau, dout):
    """dism_ref / dism_ref_backward with every position hard, masked per (batch, head) afterwards."""
    b, n, h, _ = sq.shape
    zero = torch.zeros(b, n, h, 4, dtype=torch.float64)
    lse = torch.zeros(b, n, h, dtype=torch.float64)
    flags = torch.ones(b, h, n, dtype=torch.bool)
    direction = torch.ones(b, h, dtype=torch.bool)
    mask = hard[:, None, :, None]
    out = ref.dism_ref(zero, zero, sq.double(), sk.double(), lse, lse, iq.long(), ik.long(), direction, flags,
                       v.double(), tau.double()) * mask
    grads = ref.dism_ref_backward(zero, zero, sq.double(), sk.double(), lse, lse, iq.long(), ik.long(),
                                  direction, flags, v.double(), tau.double(), dout.double() * mask)
    return out, [grads[name] for name in ('sq_vec', 'sk_vec', 'v', 'rtau')]


def vectors(generator, b, n, h, r, dv):
    sq, sk = [bf16(torch.nn.functional.silu(torch.randn(b, n, h, r, generator=generator)) * .4) for _ in range(2)]
    v = bf16(torch.randn(b, n, h, dv, generator=generator))
    dout = bf16(torch.randn(b, n, h, dv, generator=generator))
    return sq, sk, v, dout


def main():
    ths, thc, thf, ref = load_reference()
    def save(name, **arrays):
        # Large float64 results are stored as float32 (the fixtures stay a few MB); the scalar-like
        # ones (dtau, log2 normaliser) keep float64.
        packed = {}
        for key, a in arrays.items():
            a = a.numpy() if torch.is_tensor(a) else np.asarray(a)
            if a.dtype == np.float64 and a.size > 8192:
                a = a.astype(np.float32)
            packed[key] = a
        np.savez_compressed(os.path.join(HERE, name), **packed)

    # 1. The CPU-runnable reference case: fp32 q,k,v [1,256,2,64] from seed 0, labels by arg-max
    #    against per-head codebooks exactly as dism_wrapper forms them (fp32 einsum + argmax).
    g = torch.Generator().manual_seed(0)
    b, n, h, d, r, vocab = 1, 256, 2, 64, 32, 512
    q, k, v = [torch.randn(b, n, h, d, generator=g) for _ in range(3)]
    sq, sk = [torch.nn.functional.silu(torch.randn(b, n, h, r, generator=g)) * .4 for _ in range(2)]
    eq, ek = [torch.nn.functional.silu(torch.randn(h, vocab, d, generator=g)) for _ in range(2)]
    dout = torch.randn(b, n, h, d, generator=g)
    iq = torch.argmax(torch.einsum('bnhd,hvd->bnhv', q, eq), -1).transpose(-1, -2).contiguous()
    ik = torch.argmax(torch.einsum('bnhd,hvd->bnhv', k, ek), -1).transpose(-1, -2).contiguous()
    hard = torch.ones(b, h, dtype=torch.bool)
    tau = torch.full((h,), .5)
    out, grads = run_reference(ref, sq, sk, v, iq, ik, hard, tau, dout)
    norm = thf.normalizer_oracle((None, None, None, iq, ik, hard, tau))
    save('config1.npz', q=q, k=k, v=v, sq=sq, sk=sk, eq=eq, ek=ek, dout=dout, iq=iq.int(), ik=ik.int(),
         tau=tau, out=out, lse2=norm, dsq=grads[0], dsk=grads[1], dv=grads[2], dtau=grads[3])

    # 2. The reference's label patterns: integer stages at two lengths, float stages at n=256.
    hard = torch.tensor([[True, False, True], [False, True, True]])
    for pattern in ('random', 'equal', 'disjoint', 'periodic', 'boundary'):
        arrays = {}
        for n in (256, 512):
            iq, ik = ths.labels(n, pattern)
            arrays[f'iq{n}'], arrays[f'ik{n}'] = iq, ik
            arrays[f'summary{n}'] = ths.oracle(iq, ik, hard)
            arrays[f'boundary{n}'] = thc.dense_boundary(iq, ik, hard)
        n = 256
        iq, ik = ths.labels(n, pattern)
        g = torch.Generator().manual_seed(417)
        sq, sk, v, dout = vectors(g, 2, n, 3, 32, 64)
        tau = torch.linspace(-.5, .5, 3)
        out, grads = run_reference(ref, sq, sk, v, iq, ik, hard, tau, dout)
        norm = thf.normalizer_oracle((None, None, None, iq, ik, hard, tau))
        arrays.update(hard=hard, sq=sq, sk=sk, v=v, dout=dout, tau=tau, out=out, lse2=norm,
                      dsq=grads[0], dsk=grads[1], dv=grads[2], dtau=grads[3])
        save(f'pattern_{pattern}.npz', **arrays)

    # 3. A 1024-long all-equal chain over the tau range the reference tests sweep.
    n = 1024
    iq, ik = ths.labels(n, 'equal', b=1, h=1)
    g = torch.Generator().manual_seed(918)
    sq, sk, v, dout = vectors(g, 1, n, 1, 32, 64)
    hard = torch.ones(1, 1, dtype=torch.bool)
    arrays = dict(sq=sq, sk=sk, v=v, dout=dout, iq=iq, ik=ik)
    taus = [-4., -1e-4, -1e-6, 0., 1e-6, 1e-4, .1, .5, 4.]
    arrays['taus'] = np.array(taus)
    for index, value in enumerate(taus):
        tau = torch.tensor([value])
        out, grads = run_reference(ref, sq, sk, v, iq, ik, hard, tau, dout)
        arrays[f'out{index}'] = out.float()
        arrays[f'lse2_{index}'] = thf.normalizer_oracle((None, None, None, iq, ik, hard, tau))
        arrays[f'dtau{index}'] = grads[3]
        arrays[f'dsq{index}'] = grads[0].float()
    save('chain_equal.npz', **arrays)


if __name__ == '__main__':
    main()
