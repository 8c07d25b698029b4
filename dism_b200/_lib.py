"""Loader of the C-ABI library.  There is no fallback: a missing library is an error."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, 'libdism_b200.so')
_lib = None

_c = ctypes
_P, _I, _Z = _c.c_void_p, _c.c_int, _c.c_size_t
SIGNATURES = {
    'dism_last_error': (_c.c_char_p, []),
    'dism_abi_version': (_I, []),
    'dism_route_word': (_I, [_P]),
    'dism_hard_dlog_weights': (_I, [_P, _I, _I, _P, _P]),
    'dism_labels': (_I, [_P, _P, _I, _I, _I, _I, _I, _P, _P]),
    'dism_labels_pair': (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    'dism_labels_fault': (_I, [_P]),
    'dism_labels_wait_selftest': (_I, [_I, _P, _P]),
    'dism_hard_summary': (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P]),
    'dism_hard_chunk': (_I, [_P, _P, _I, _I, _P]),
    'dism_hard_summary_packed': (_I, [_P, _P, _P, _P, _I, _c.c_int64, _I, _I, _I, _I, _P, _P]),
    'dism_hard_chunk_packed': (_I, [_P, _P, _P, _I, _c.c_int64, _I, _I, _P]),
    'dism_hard_log_weights': (_I, [_P, _I, _I, _P, _P]),
    'dism_hard_readout_workspace': (_Z, [_I, _I, _I]),
    'dism_hard_readout': (_I, [_P] * 8 + [_I, _I, _P] + [_I] * 7 + [_P, _P, _P, _Z, _P]),
    'dism_hard_readout_static': (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P]),
    'dism_hard_readout_static_error': (_c.c_char_p, []),
    'dism_hard_backward_workspace': (_Z, [_I, _I, _I, _I]),
    'dism_hard_backward': (_I, [_P] * 9 + [_I, _I, _P, _I, _P] + [_I] * 6 + [_P, _P, _P, _P, _P, _Z, _P, _P]),
    'dism_longest_match_workspace': (_Z, [_I, _I]),
    'dism_profile_enable': (_I, [_I]),
    'dism_profile_count': (_I, []),
    'dism_profile_read': (_I, [_I, _c.c_char_p, _I, _c.POINTER(_c.c_float)]),
    'dism_longest_match': (_I, [_P, _I, _I, _P, _P, _P, _P, _Z, _P]),
}


def load():
    """Return the ctypes handle of libdism_b200.so with every entry point typed."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY_PATH):
            raise ImportError(
                f'{LIBRARY_PATH} is missing: build it with `python -m dism_b200.build` '
                '(there is no CPU or PyTorch fallback for the hard path)')
        lib = ctypes.CDLL(LIBRARY_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            function = getattr(lib, name)
            function.restype, function.argtypes = restype, argtypes
        _lib = lib
    return _lib


def check(status):
    """Turn a non-zero status of the last call into RuntimeError with the library's message."""
    if status:
        raise RuntimeError(load().dism_last_error().decode())


def kernel_timings():
    """Records collected since dism_profile_enable(1): list of (kernel name, milliseconds)."""
    lib, out = load(), []
    name, ms = ctypes.create_string_buffer(64), ctypes.c_float()
    for index in range(lib.dism_profile_count()):
        check(lib.dism_profile_read(index, name, 64, ctypes.byref(ms)))
        out.append((name.value.decode(), ms.value))
    return out
