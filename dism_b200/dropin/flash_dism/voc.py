"""Operator entry of the module call site: vocabulary labels, hard forward, hard backward under autograd.

Mirrors the reference's `voc_dism` (dism_v3/python/flash_dism/voc.py:7-40, dispatch in
dism_v3/python/flash_dism/__init__.py:43-56) for the sequences it sends down the hard path: every
(row, head) flag in `hard` must be set.  The soft path, which is where q, k and the codebooks get
their gradient in the reference, is not part of this library; a soft flag raises.
"""
import torch
import cu_flash_dism as cu

from .hard_forward import hard_readout, hard_log_weights
from .hard_backward import backward_hard


class _HardVocabulary(torch.autograd.Function):
    """labels -> log-weight table -> hard_readout in the forward; backward_hard in the backward.  On hard sequences the
    reference gives sq, sk, v and tau their gradient and q, k and both codebooks exactly zero
    (dism_v3/python/flash_dism/hard_backward.py:9-15, dism_v3/tests/test_hard_training.py:69-71)."""

    @staticmethod
    def forward(ctx, q, k, sq, sk, v, q_vocab, k_vocab, tau, hard, layout, ctas):
        codes_q, codes_k = (c.detach().to(torch.bfloat16).contiguous() for c in (q_vocab, k_vocab))
        if codes_q.dim() == 2:  # one codebook shared by the heads
            codes_q, codes_k = (c.expand(q.size(2), *c.shape).contiguous() for c in (codes_q, codes_k))
        idx_q, idx_k = cu.labels_pair(q.detach().contiguous(), codes_q, k.detach().contiguous(), codes_k)
        # the log-weight table is built once and kept for the backward, as forward_hard(save_state=True) keeps it
        longest = sq.size(1) if layout is None else (layout.max_length or max(layout.lengths))
        table = hard_log_weights(tau.detach().float().contiguous(), longest)
        out, norm = hard_readout(sq.detach().contiguous(), sk.detach().contiguous(), v.detach().contiguous(), idx_q, idx_k, hard,
                                 None, table, layout=layout, ctas=ctas)
        ctx.save_for_backward(q, k, sq, sk, v, q_vocab, k_vocab, tau, idx_q, idx_k, hard, norm, table)
        ctx.layout, ctx.ctas = layout, ctas
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, sq, sk, v, q_vocab, k_vocab, tau, idx_q, idx_k, hard, norm, table = ctx.saved_tensors
        state = dict(boundary=None, log_weights=table)
        dsq, dsk, dv, dtau = backward_hard(sq.detach().contiguous(), sk.detach().contiguous(), v.detach().contiguous(),
                                           dout.contiguous(), idx_q, idx_k, hard, norm, state, layout=ctx.layout, ctas=ctx.ctas)
        zero = lambda t, needed: torch.zeros_like(t) if needed else None
        needs = ctx.needs_input_grad
        return (zero(q, needs[0]), zero(k, needs[1]), dsq.to(sq.dtype), dsk, dv, zero(q_vocab, needs[5]), zero(k_vocab, needs[6]),
                dtau.to(tau.dtype), None, None, None)


def voc_dism(q, k, sq, sk, v, q_vocab, k_vocab, rtau, *, direction=None, hard, cu_seqlens=None, layout=None, ctas=0, beta=1.0,
             hard_planner=None):
    """BF16 [B,N,H,D] q and k, already-activated BF16 [B,N,H,R] sq and sk, BF16 [B,N,H,DV] v, codebooks [H,V,D] (or a
    shared [V,D]), rtau FP32 [H] -> BF16 [B,N,H,DV].  `direction` and `beta` only act on soft sequences and are accepted
    for signature compatibility; `hard` is bool [training_rows,H] and must be all true."""
    if hard_planner is not None:
        raise NotImplementedError('the asynchronous event planner of the reference is not part of this library')
    if not bool(hard.all()):
        raise NotImplementedError('soft sequences need the soft path, which this library does not build')
    if cu_seqlens is not None:
        if layout is not None:
            raise ValueError('provide either layout or cu_seqlens, not both')
        from .varlen import VarlenLayout
        layout = VarlenLayout.from_cu_seqlens(cu_seqlens, q.shape[1])
    if layout is not None and ctas:
        raise ValueError('ctas is only supported for fixed-length execution')
    return _HardVocabulary.apply(q, k, sq, sk, v, q_vocab, k_vocab, rtau, hard, layout, ctas)
