"""Integer stages (mirrors dism_v3/python/flash_dism/summary.py:8-31)."""
import cu_flash_dism as cu


def _table(layout):
    return None if layout is None else layout.table


def summarize_hard(idx_q, idx_k, hard, *, layout=None, ctas=0, _graph_choice=None):
    """Strip summaries R[c,j] of int32 labels [B,H,N]: int32 [B,H,(N-1)//32,N], -1 where nothing
    mismatches inside the strip, on non-causal entries and on soft (batch, head) rows."""
    return cu.hard_summary(idx_q, idx_k, hard, _table(layout), ctas, _graph_choice)


def hard_chunk_scan(summary, *, layout=None, heads=0, _graph_choice=None, inplace=False):
    """Inclusive boundaries max(R[c,j], boundary[c-1,j-32]); the match length on a causal hard
    entry is key coordinate minus boundary.  inplace=True reuses the summary's storage."""
    return cu.hard_chunk(summary, _table(layout), heads, _graph_choice, inplace)
