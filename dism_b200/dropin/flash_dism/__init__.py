"""Hard-path subset of the reference's `flash_dism` package, backed by libdism_b200.so.

Same module and function names as dism_v3/python/flash_dism/{summary,hard_forward,hard_backward,voc}.py
so callers and tests written against the reference import unchanged.
"""
from .summary import summarize_hard, hard_chunk_scan
from .hard_forward import forward_hard, hard_readout, hard_log_weights
from .hard_backward import backward_hard, backward_hard_recompute
from .varlen import VarlenLayout
from .voc import voc_dism
