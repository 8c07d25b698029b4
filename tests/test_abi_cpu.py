"""The C-ABI library: it loads without a GPU, exports every symbol the header declares, and its
argument checks (which run before any CUDA call) report the reference's error words."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def lib():
    from dism_b200 import _lib, build
    build.build()
    return _lib.load()


def declared_symbols():
    header = open(os.path.join(ROOT, 'include', 'dism_b200.h')).read()
    header = re.sub(r'/\*.*?\*/', '', header, flags=re.S)
    return sorted(set(re.findall(r'\b(dism_[a-z_0-9]+)\s*\(', header)))


def test_every_declared_symbol_is_exported_and_typed(lib):
    from dism_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f'{name} is declared in include/dism_b200.h but not exported'
        assert name in _lib.SIGNATURES, f'{name} has no ctypes signature'
    assert lib.dism_abi_version() >= 9


def test_library_has_no_torch_dependency(lib):
    from dism_b200 import _lib
    needed = os.popen(f'ldd {_lib.LIBRARY_PATH}').read()
    assert 'torch' not in needed and 'c10' not in needed


def message(lib):
    return lib.dism_last_error().decode()


def test_argument_checks_run_without_a_device(lib):
    p = ctypes.c_void_p(4096)  # never dereferenced: every call below is rejected first
    assert lib.dism_hard_log_weights(p, 4, 100, p, None) == 1 and '256-aligned' in message(lib)
    assert lib.dism_hard_summary(p, p, p, 1, 2, 300, 0, p, None) == 1 and '256-aligned' in message(lib)
    assert lib.dism_hard_summary(p, p, p, 1, 2, 512, -1, p, None) == 1 and 'CTA' in message(lib)
    assert lib.dism_hard_readout(p, p, p, p, p, p, None, None, 1, 0, p, 512, 1, 512, 2, 32, 64, 0, p, p, p, 1 << 30, None) == 1
    assert 'too short' in message(lib)
    assert lib.dism_hard_readout(p, p, p, p, p, p, None, None, 1, 0, p, 513, 1, 512, 2, 24, 64, 0, p, p, p, 1 << 30, None) == 2
    assert 'unsupported' in message(lib)
    assert lib.dism_hard_readout(p, p, p, p, p, p, None, None, 1, 0, p, 513, 1, 512, 2, 32, 64, 0, p, p, p, 16, None) == 1
    assert 'workspace' in message(lib)
    assert lib.dism_hard_readout(p, p, p, p, p, p, None, p, 3, 256, p, 513, 1, 1024, 2, 32, 64, 0, p, p, p, 1 << 30, None) == 1
    assert 'training rows' in message(lib)
    assert lib.dism_hard_readout(p, p, p, p, p, p, None, p, 1, 256, p, 513, 2, 1024, 2, 32, 64, 0, p, p, p, 1 << 30, None) == 1
    assert 'packed' in message(lib)
    assert lib.dism_hard_backward(p, p, p, p, p, p, p, None, None, 1, 0, p, 513, p, 1, 512, 2, 32, 64, 0, p, p, p, p, p, 16,
                                  None, None) == 1
    assert 'workspace' in message(lib)
    # packed layouts: the tables are indexed up to the longest document, which the caller states
    assert lib.dism_hard_readout(p, p, p, p, p, p, None, p, 1, 1024, p, 513, 1, 1024, 2, 32, 64, 0, p, p, p, 1 << 30, None) == 1
    assert 'too short' in message(lib) and 'longest document' in message(lib)
    assert lib.dism_hard_readout(p, p, p, p, p, p, None, p, 1, 0, p, 2049, 1, 1024, 2, 32, 64, 0, p, p, p, 1 << 30, None) == 1
    assert 'longest document' in message(lib)
    assert lib.dism_hard_backward(p, p, p, p, p, p, p, None, p, 1, 768, p, 513, p, 1, 1024, 2, 32, 64, 0, p, p, p, p, p, 1 << 30,
                                  None, None) == 1
    assert 'too short' in message(lib)
    # (batch, head) slices are a grid dimension
    assert lib.dism_hard_readout(p, p, p, p, p, p, None, None, 4096, 0, p, 513, 4096, 512, 32, 32, 64, 0, p, p, p, 1 << 40, None) == 1
    assert '65535' in message(lib)
    assert lib.dism_labels(p, p, 1, 16, 2, 48, 512, p, None) == 2 and 'unsupported' in message(lib)
    assert lib.dism_labels(p, ctypes.c_void_p(4104), 1, 16, 2, 64, 512, p, None) == 1 and '16-byte aligned' in message(lib)
    assert lib.dism_longest_match(p, 1, 13, p, p, p, p, 1 << 20, None) == 1
    # packed summary / composition: the checks that need no look at the device table
    assert lib.dism_hard_summary_packed(p, p, p, p, 3, 40, 2, 1000, 1, 0, p, None) == 1 and '256-aligned' in message(lib)
    assert lib.dism_hard_summary_packed(p, p, p, p, 3, 40, 2, 1024, 3, 0, p, None) == 1 and 'training rows' in message(lib)
    assert lib.dism_hard_summary_packed(p, p, p, p, 5, 40, 2, 1024, 1, 0, p, None) == 1 and 'length mismatch' in message(lib)
    assert lib.dism_hard_summary_packed(p, p, p, p, 3, 40, 2, 1024, 1, -1, p, None) == 1 and 'CTA' in message(lib)
    assert lib.dism_hard_chunk_packed(p, p, p, 3, 1 << 40, 2, 1024, None) == 1 and 'exceed' in message(lib)
    assert lib.dism_hard_chunk_packed(p, ctypes.c_void_p(4100), p, 3, 10, 2, 1024, None) == 1 and '16-byte aligned' in message(lib)
    # the route word: one aligned device int32, or NULL to clear it (the pointer is only stored here)
    assert lib.dism_route_word(ctypes.c_void_p(4098)) == 1 and 'graph choice' in message(lib)
    assert lib.dism_route_word(p) == 0 and lib.dism_route_word(None) == 0
    assert lib.dism_hard_readout_workspace(8, 16, 8192) > 8 * 16 * 8192 * 8
    assert lib.dism_hard_backward_workspace(8, 16, 8192, 8193) > 2 * 8 * 16 * 8192 * 8


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    from dism_b200 import _lib
    monkeypatch.setattr(_lib, '_lib', None)
    monkeypatch.setattr(_lib, 'LIBRARY_PATH', str(tmp_path / 'absent.so'))
    with pytest.raises(ImportError, match='no CPU or PyTorch fallback'):
        _lib.load()
