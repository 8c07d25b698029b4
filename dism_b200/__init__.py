"""B200-native implementation of the flash_dism hard sequence-mixing path.

The product is the C-ABI library libdism_b200.so (built by `python -m dism_b200.build`) plus a
drop-in layer that keeps the reference's Python names: after `dism_b200.install_dropin()` the
modules `cu_flash_dism` and `flash_dism.{summary,hard_forward,hard_backward}` import from here.
"""
import os
import sys

DROPIN_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'dropin')


def install_dropin():
    """Put the drop-in `cu_flash_dism` / `flash_dism` modules first on sys.path."""
    if DROPIN_PATH not in sys.path:
        sys.path.insert(0, DROPIN_PATH)
    return DROPIN_PATH
