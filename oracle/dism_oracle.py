"""ctypes front end of the CPU checker (oracle/dism_oracle.c) plus numpy helpers.

Test infrastructure only: the test-suite, the smoke check and the CPU-baseline leg of the
benchmark import this module; the shipped package never does.  Arrays are numpy; vectors are
float32 holding values already rounded to their storage type, laid out [B,N,H,C]; labels are
int32 [B,H,N]; hard flags are bool [B,H].
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None


def build(force=False):
    """Compile the C restatement (and the reference shim when the reference checkout exists)."""
    target = os.path.join(_HERE, 'libdism_oracle.so')
    source = os.path.join(_HERE, 'dism_oracle.c')
    if force or not os.path.exists(target) or os.path.getmtime(target) < os.path.getmtime(source):
        subprocess.check_call(['make', '-C', _HERE, '-B', 'libdism_oracle.so'])
    subprocess.check_call(['make', '-C', _HERE, 'ref'], stdout=subprocess.DEVNULL)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, 'libdism_oracle.so')
        if not os.path.exists(path):
            build()
        _LIB = ctypes.CDLL(path)
    return _LIB


def reference_lib():
    """The reference's own native CPU forward, or None when it was not built."""
    global _REF
    path = os.path.join(_HERE, '_ref', 'libdism_ref.so')
    if _REF is None and os.path.exists(path):
        _REF = ctypes.CDLL(path)
    return _REF


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def labels(x, codebook):
    """x [B,N,H,D], codebook [H,V,D] (float32 values) -> int32 [B,H,N]."""
    x, codebook = _f32(x), _f32(codebook)
    b, n, h, d = x.shape
    v = codebook.shape[1]
    out = np.empty((b, h, n), np.int32)
    lib().dism_oracle_labels(_ptr(x), _ptr(codebook), b, n, h, d, v, _ptr(out))
    return out


def summary(iq, ik, hard):
    iq, ik, hard = _i32(iq), _i32(ik), _u8(hard)
    b, h, n = iq.shape
    out = np.empty((b, h, (n - 1) // 32, n), np.int32)
    lib().dism_oracle_summary(_ptr(iq), _ptr(ik), _ptr(hard), b, h, n, _ptr(out))
    return out


def chunk(summ):
    summ = _i32(summ)
    b, h, c, n = summ.shape
    out = np.empty_like(summ)
    lib().dism_oracle_chunk(_ptr(summ), b * h, n, _ptr(out))
    return out


def lengths(q, k):
    """Dense L[i,j] of one (batch, head): q, k int32 [N] -> int32 [N,N]."""
    q, k = _i32(q), _i32(k)
    out = np.empty((q.size, q.size), np.int32)
    lib().dism_oracle_lengths(_ptr(q), _ptr(k), q.size, _ptr(out))
    return out


def longest(stream):
    """Symbol stream int32 [N] -> (end index, length, next symbol), each int32 [N]."""
    s = _i32(stream)
    end, length, nxt = (np.empty(s.size, np.int32) for _ in range(3))
    lib().dism_oracle_longest(_ptr(s), s.size, _ptr(end), _ptr(length), _ptr(nxt))
    return end, length, nxt


def reference_longest_lengths(keys, queries, interval=64):
    """max_j<=i L(i,j) of one sequence from the reference's decode planner (suffix automaton + tail band), int32 [N];
    None when the reference was not built."""
    ref = reference_lib()
    if ref is None or not hasattr(ref, 'dism_ref_longest_lengths'):
        return None
    k, q = _i32(keys), _i32(queries)
    out = np.empty(k.size, np.int32)
    if ref.dism_ref_longest_lengths(_ptr(k), _ptr(q), k.size, int(interval), _ptr(out)):
        raise RuntimeError('the reference planner rejected the sequence')
    return out


def lut(tau, n):
    tau = _f32(tau)
    out = np.empty((tau.size, n + 1), np.float32)
    lib().dism_oracle_lut(_ptr(tau), tau.size, n, _ptr(out))
    return out


def forward(sq, sk, v, iq, ik, hard, tau, threads=1):
    """float64 output [B,N,H,DV] and log2 normaliser [B,H,N]."""
    sq, sk, v, iq, ik, hard, tau = _f32(sq), _f32(sk), _f32(v), _i32(iq), _i32(ik), _u8(hard), _f32(tau)
    b, n, h, r = sq.shape
    dv = v.shape[3]
    out = np.empty((b, n, h, dv), np.float64)
    lse2 = np.empty((b, h, n), np.float64)
    lib().dism_oracle_forward(_ptr(sq), _ptr(sk), _ptr(v), _ptr(iq), _ptr(ik), _ptr(hard), _ptr(tau),
                              b, n, h, r, dv, _ptr(out), _ptr(lse2), int(threads))
    return out, lse2


def backward(sq, sk, v, dout, iq, ik, hard, tau, threads=1):
    """float64 dSQ, dSK [B,N,H,R], dV [B,N,H,DV], dtau [H] (natural-log coefficient)."""
    sq, sk, v, dout = _f32(sq), _f32(sk), _f32(v), _f32(dout)
    iq, ik, hard, tau = _i32(iq), _i32(ik), _u8(hard), _f32(tau)
    b, n, h, r = sq.shape
    dv = v.shape[3]
    dsq, dsk = np.empty((b, n, h, r), np.float64), np.empty((b, n, h, r), np.float64)
    dvv, dtau = np.empty((b, n, h, dv), np.float64), np.empty(h, np.float64)
    lib().dism_oracle_backward(_ptr(sq), _ptr(sk), _ptr(v), _ptr(dout), _ptr(iq), _ptr(ik), _ptr(hard),
                               _ptr(tau), b, n, h, r, dv, _ptr(dsq), _ptr(dsk), _ptr(dvv), _ptr(dtau),
                               int(threads))
    return dsq, dsk, dvv, dtau


def reference_forward(sq, sk, v, iq, ik, tau):
    """One (batch, head) through the reference's native planner + executor in float64.

    sq, sk [N,R], v [N,DV], labels [N], tau scalar -> (out [N,DV], log2 normaliser [N]).
    """
    ref = reference_lib()
    if ref is None:
        raise RuntimeError('oracle/_ref/libdism_ref.so was not built')
    sq, sk, v = (np.ascontiguousarray(a, dtype=np.float64) for a in (sq, sk, v))
    iq, ik = _i32(iq), _i32(ik)
    n, r = sq.shape
    dv = v.shape[1]
    out, logden = np.empty((n, dv), np.float64), np.empty(n, np.float64)
    ref.dism_ref_forward_f64.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_double,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    status = ref.dism_ref_forward_f64(_ptr(iq), _ptr(ik), n, float(tau), _ptr(sq), _ptr(sk), _ptr(v), r, dv,
                                      _ptr(out), _ptr(logden))
    if status:
        raise RuntimeError('reference planner rejected the input')
    return out, logden / np.log(2.)


def reference_forward_many(sq, sk, v, iq, ik, tau, threads=1):
    """Many (batch, head) sequences through the reference's native planner + executor in float32, on `threads`
    host threads.  sq, sk [S,N,R], v [S,N,DV], labels [S,N], tau [S] -> out float32 [S,N,DV]."""
    ref = reference_lib()
    if ref is None:
        raise RuntimeError('oracle/_ref/libdism_ref.so was not built')
    sq, sk, v, iq, ik = _f32(sq), _f32(sk), _f32(v), _i32(iq), _i32(ik)
    tau = np.ascontiguousarray(tau, dtype=np.float64)
    s, n, r = sq.shape
    dv = v.shape[2]
    out = np.empty((s, n, dv), np.float32)
    ref.dism_ref_forward_f32_many.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                              ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_void_p, ctypes.c_int]
    if ref.dism_ref_forward_f32_many(_ptr(iq), _ptr(ik), s, n, _ptr(tau), _ptr(sq), _ptr(sk), _ptr(v), r, dv, _ptr(out),
                                     int(threads)):
        raise RuntimeError('reference planner rejected an input')
    return out


# ---- numpy restatements of the integer stages (independent of the C file) -------------------
def summary_numpy(iq, ik, hard):
    """Row-major recurrence restarted at every 32-row strip (dism_v3/tests/test_hard_summary.py:37-49)."""
    b, h, n = iq.shape
    out = np.full((b, h, (n - 1) // 32, n), -1, np.int32)
    col = np.arange(n, dtype=np.int32)
    for c in range(out.shape[2]):
        state = np.full((b, h, n), -1, np.int32)
        for row in range(32 * c, 32 * c + 32):
            shifted = np.concatenate((np.full((b, h, 1), -1, np.int32), state[:, :, :-1]), -1)
            state = np.maximum(shifted, np.where(iq[:, :, row, None] == ik, -1, col))
        out[:, :, c] = np.where(np.asarray(hard, bool)[:, :, None] & (col <= 32 * c + 31), state, -1)
    return out


def boundary_numpy(iq, ik, hard):
    """j - L(32c+31, j) from the full scalar recurrence (dism_v3/tests/test_hard_chunk.py:24-36)."""
    b, h, n = iq.shape
    length = np.zeros((b, h, n), np.int32)
    out = np.full((b, h, (n - 1) // 32, n), -1, np.int32)
    col = np.arange(n, dtype=np.int32)
    for row in range(n - 32):
        previous = np.concatenate((np.zeros((b, h, 1), np.int32), length[:, :, :-1]), -1)
        length = np.where(iq[:, :, row, None] == ik, previous + 1, 0)
        if row % 32 == 31:
            out[:, :, row // 32] = np.where(np.asarray(hard, bool)[:, :, None] & (col <= row), col - length, -1)
    return out


def bf16_round(a):
    """Round float32 values to bfloat16 (nearest even) and return them as float32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)
