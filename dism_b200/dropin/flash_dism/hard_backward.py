"""Hard-only backward (mirrors dism_v3/python/flash_dism/hard_backward.py:6-59)."""
import torch
import cu_flash_dism as cu

from .hard_forward import forward_hard, hard_log_weights


@torch.no_grad()
def backward_hard(sq, sk, v, dout, idx_q, idx_k, hard, normalizer, state, *, layout=None, ctas=0, _graph_choice=None):
    """dSQ (FP32), dSK, dV (BF16) and dtau (FP32, natural-log coefficient) for hard rows; soft rows
    get zeros.  `state` needs 'log_weights'; 'boundary' is optional (None = derive from labels)."""
    table = None if layout is None else layout.table
    return cu.hard_backward((sq, sk, v, dout, idx_q, idx_k, hard), state.get('boundary'), state['log_weights'],
                            normalizer, ctas, table, _graph_choice)


@torch.no_grad()
def backward_hard_recompute(sq, sk, v, dout, iq, ik, hard, tau, *, layout=None, ctas=0, _graph_choice=None):
    """Backward without retained state: the forward is run again for the normaliser, nothing
    quadratic is materialised.  Returns a dict keyed sq_vec, sk_vec, v, rtau."""
    if layout is not None:
        n = sq.shape[1]
        if sq.shape[0] != 1 or hard.ndim != 2 or n % hard.shape[0] or layout.tokens != n:
            raise ValueError('invalid packed fallback rows')
        row_tokens = n // hard.shape[0]
        if any(length and begin // row_tokens != (begin + length - 1) // row_tokens
               for begin, length, *_ in layout.table.tolist()):
            raise ValueError('document crosses original hard row')
    sq, sk, v, dout = (t.contiguous() for t in (sq, sk, v, dout))
    iq, ik = (t.to(torch.int32).contiguous() for t in (iq, ik))
    hard, tau = hard.contiguous(), tau.contiguous()
    _, norm = forward_hard(sq, sk, v, iq, ik, hard, tau, layout=layout, ctas=ctas, _graph_choice=_graph_choice)
    longest = sq.shape[1] if layout is None else (layout.max_length or max(layout.lengths))
    state = dict(boundary=None, log_weights=hard_log_weights(tau, longest, _graph_choice=_graph_choice))
    grads = backward_hard(sq, sk, v, dout, iq, ik, hard, norm, state, layout=layout, ctas=ctas,
                          _graph_choice=_graph_choice)
    return dict(zip(('sq_vec', 'sk_vec', 'v', 'rtau'), grads))
