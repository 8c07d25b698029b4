"""Packed single-batch layouts (mirrors the layout part of dism_v3/python/flash_dism/varlen.py:8-52)."""
from dataclasses import dataclass

import torch
import cu_flash_dism as cu


@dataclass(frozen=True)
class VarlenLayout:
    """A validated pack of 256-aligned documents; build once per pack and reuse.

    `table` is the CPU description the native side consumes; empty documents are allowed.
    """
    table: torch.Tensor
    lengths: tuple
    tokens: int
    padded_tokens: int
    forward_elements: int
    vertical_elements: int
    backward_elements: int
    max_length: int = 0

    @classmethod
    def from_cu_seqlens(cls, cu_seqlens, total_tokens):
        values = cu.make_varlen_layout(cu_seqlens, total_tokens)
        return cls(values[0], tuple(values[1]), *values[2:])

    def checkpoint_bytes(self, heads):
        return 4 * heads * (self.forward_elements + self.vertical_elements + 3 * self.backward_elements)
