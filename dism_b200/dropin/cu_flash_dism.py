"""Stand-in for the reference's native module `cu_flash_dism`, hard path only.

The reference binds its kernels with pybind11 (dism_v3/src/module.cpp:11-37,
dism_v3/src/frontend.cpp:282-403).  This module keeps those function names, argument orders,
return shapes and error words, allocates outputs as torch tensors on the inputs' device, and
forwards plain pointers to the C ABI of libdism_b200.so on the current CUDA stream.  It holds no
compute of its own and has no fallback: without the library, importing it fails.

Differences a caller can see: `hard_readout` and `hard_backward` accept `boundary=None` (run
lengths are then derived from the labels inside the kernel, nothing quadratic is stored); with a
packed `table` a boundary is checked for shape and otherwise left unread (same bits either way);
the soft path (`core_forward`, `core_backward`) is not
built and raises NotImplementedError.  The `choice` device word of the reference's CUDA-graph
router (one CUDA int32; 0 runs the hard path, anything else makes its kernels return at once) is
handed to the library for the calls of the operator it was given to.
"""
import contextlib

import torch

from dism_b200 import _lib

_abi = _lib.load()

# (R, D, DV) combinations the hard kernels are instantiated for; D is irrelevant to them.
configs = {(r, d, dv): None for r in (16, 32) for d in (32, 64, 128) for dv in (32, 64, 128)}


def fp32_enabled():
    return False


def get_config(r, d, dv):
    if (r, d, dv) not in configs:
        raise RuntimeError(f'unsupported configuration R={r} D={d} DV={dv}')
    return None


def _fail(message):
    raise RuntimeError(message)


def _stream(tensor):
    return torch.cuda.current_stream(tensor.device).cuda_stream


@contextlib.contextmanager
def _routed(choice, device):
    """Checks the route word as dism_v3/include/host/graph_route.h:4-10 does and sets it for the library calls inside."""
    if choice is None:
        yield
        return
    if not (torch.is_tensor(choice) and choice.device == device and choice.dtype == torch.int32
            and choice.numel() == 1 and choice.is_contiguous()):
        _fail('graph choice must be one contiguous CUDA int32 on the operand device')
    _lib.check(_abi.dism_route_word(choice.data_ptr()))
    try:
        yield
    finally:
        _abi.dism_route_word(None)


# ---- packed (varlen) layouts -------------------------------------------------------------------
# The reference describes a pack by a CPU int64 table [documents, 7] with the columns Begin, Length,
# PaddedBegin, PaddedLength, ForwardOffset, VerticalOffset, BackwardOffset
# (dism_v3/include/varlen/layout.cuh:17-20, built in dism_v3/src/frontend.cpp:259-280).
def make_varlen_layout(cu_seqlens, total):
    """cu_seqlens int32 [documents+1] -> (table, lengths, tokens, padded, forward, vertical, backward)."""
    if not (torch.is_tensor(cu_seqlens) and cu_seqlens.dim() == 1 and cu_seqlens.dtype == torch.int32
            and cu_seqlens.is_contiguous() and cu_seqlens.numel() > 0):
        _fail('cu_seqlens must be contiguous int32 [sequences+1]')
    offsets = cu_seqlens.cpu().tolist()
    if total < 0 or offsets[0] != 0 or offsets[-1] != total:
        _fail('invalid cu_seqlens endpoints')
    rows, lengths, forward, vertical, backward = [], [], 0, 0, 0
    for begin, end in zip(offsets, offsets[1:]):
        if begin < 0 or begin % 256 or end % 256:
            _fail('all varlen boundaries must be256-token aligned')
        n = end - begin
        if n < 0:
            _fail('cu_seqlens must be monotonic with supported lengths')
        rows.append([begin, n, begin, n, forward, vertical, backward])
        forward += ((n - 1) // 32 if n else 0) * n
        vertical += ((n - 1) // 16 if n else 0) * n
        backward += (n + 31) // 32 * n
        lengths.append(n)
    table = torch.tensor(rows, dtype=torch.int64).reshape(len(rows), 7)
    return table, lengths, total, total, forward, vertical, backward


def _documents(table, n, rows):
    """(begin, length) of the non-empty documents of a layout table, validated against N and the hard rows."""
    if not (torch.is_tensor(table) and table.device.type == 'cpu' and table.dtype == torch.int64 and table.dim() == 2
            and table.size(1) == 7 and table.is_contiguous()):
        _fail('layout must be CPU int64 [sequences,7]')
    spans, tokens = [], 0
    for begin, length, *_ in table.tolist():
        if length < 0 or length % 256 or begin != tokens:
            _fail('varlen boundaries including T must be256-token aligned; no input padding')
        tokens += length
        if length:
            spans.append((begin, length))
    if tokens != n:
        _fail('packed labels/layout length mismatch')
    if n % rows or (n // rows) % 256:
        _fail('packed hard rows must evenly divide tokens into 256-aligned training rows')
    row_tokens = n // rows
    for begin, length in spans:
        if begin // row_tokens != (begin + length - 1) // row_tokens:
            _fail('document cannot cross a hard training-row boundary')
    return spans


_document_tables = {}


def _document_table(spans, n, device):
    """Device int32 [N/256, 2]: for every 256-position block the [begin, end) of its document.
    Uploaded once per distinct pack and device (the reference caches its task tables the same way,
    dism_v3/include/host/metadata_upload.h:15-48)."""
    key = (tuple(spans), n, str(device))
    cached = _document_tables.get(key)
    if cached is None:
        if len(_document_tables) >= 32:
            _document_tables.pop(next(iter(_document_tables)))
        blocks = torch.zeros((n // 256, 2), dtype=torch.int32)
        for begin, length in spans:
            blocks[begin // 256:(begin + length) // 256, 0] = begin
            blocks[begin // 256:(begin + length) // 256, 1] = begin + length
        cached = _document_tables[key] = blocks.to(device)
    return cached


_row_tables = {}


def _row_table(spans, heads, device):
    """Device int64 [documents, 4] for the packed summary and composition kernels: per non-empty document its first
    position, its length, the (head, strip) rows before it and the rectangle elements before it; with the totals of
    the last two.  Uploaded once per distinct pack, head count and device."""
    key = (tuple(spans), heads, str(device))
    cached = _row_tables.get(key)
    if cached is None:
        if len(_row_tables) >= 32:
            _row_tables.pop(next(iter(_row_tables)))
        records, rows, elements = [], 0, 0
        for begin, length in spans:
            records.append([begin, length, rows, elements])
            rows += heads * ((length - 1) // 32)
            elements += heads * ((length - 1) // 32) * length
        table = torch.tensor(records, dtype=torch.int64).reshape(len(records), 4).to(device)
        cached = _row_tables[key] = (table, rows, elements)
    return cached


def _packed_hard(hard, device, heads):
    if not (torch.is_tensor(hard) and hard.device == device and hard.dtype == torch.bool and hard.dim() == 2
            and hard.size(0) > 0 and hard.size(1) == heads and hard.is_contiguous()):
        _fail('hard must be contiguous bool [training_rows,H]; token-level masks are unsupported '
              '(sequence hard flags only)')


def _check(tensor, dtype, shape, name):
    if not (torch.is_tensor(tensor) and tensor.is_cuda and tensor.dtype == dtype and tensor.is_contiguous()
            and (shape is None or tuple(tensor.shape) == tuple(shape))):
        _fail(f'{name}: invalid device, dtype, shape or stride')


def _check_hard(hard, device, batch, heads, what='hard'):
    if not (torch.is_tensor(hard) and hard.device == device and hard.dtype == torch.bool and hard.dim() == 2
            and hard.size(0) > 0 and hard.size(1) == heads and hard.is_contiguous()):
        _fail(f'{what} must be contiguous bool [training_rows,H]; token-level masks are unsupported '
              '(sequence hard flags only)')
    if hard.size(0) != batch:
        _fail('fixed hard must be [B,H]')


def hard_summary(query, key, hard, table=None, ctas=0, choice=None):
    """int32 labels [B,H,N] -> strip summaries int32 [B,H,(N-1)//32,N]; packed: the documents'
    [H,(length-1)//32,length] regions one after the other, flattened."""
    if table is not None:
        if not (torch.is_tensor(query) and query.is_cuda and query.dtype == torch.int32 and query.dim() == 3
                and query.is_contiguous()):
            _fail('query labels must be contiguous CUDA int32 [B,H,N]')
        if query.size(0) != 1:
            _fail('packed labels/layout length mismatch')
        h, n = query.size(1), query.size(2)
        if not (torch.is_tensor(key) and key.device == query.device and key.dtype == torch.int32
                and key.shape == query.shape and key.is_contiguous()):
            _fail('invalid key labels')
        _packed_hard(hard, query.device, h)
        spans = _documents(table, n, hard.size(0))
        if ctas < 0:
            _fail('invalid CTA count')
        records, rows, elements = _row_table(spans, h, query.device)
        with torch.cuda.device(query.device), _routed(choice, query.device):
            out = torch.empty((elements,), dtype=torch.int32, device=query.device)
            if rows:
                _lib.check(_abi.dism_hard_summary_packed(query.data_ptr(), key.data_ptr(), hard.data_ptr(), records.data_ptr(),
                                                         len(spans), rows, h, n, hard.size(0), int(ctas), out.data_ptr(),
                                                         _stream(query)))
        return out
    if not (torch.is_tensor(query) and query.is_cuda and query.dtype == torch.int32 and query.dim() == 3
            and query.is_contiguous()):
        _fail('query labels must be contiguous CUDA int32 [B,H,N]')
    b, h, n = query.shape
    if not (torch.is_tensor(key) and key.device == query.device and key.dtype == torch.int32
            and key.shape == query.shape and key.is_contiguous()):
        _fail('invalid key labels')
    if n <= 0 or n % 256:
        _fail('positive dimensions and 256-aligned sequence length required')
    _check_hard(hard, query.device, b, h)
    if ctas < 0:
        _fail('invalid CTA count')
    with torch.cuda.device(query.device), _routed(choice, query.device):
        out = torch.empty((b, h, (n - 1) // 32, n), dtype=torch.int32, device=query.device)
        _lib.check(_abi.dism_hard_summary(query.data_ptr(), key.data_ptr(), hard.data_ptr(), b, h, n, int(ctas),
                                          out.data_ptr(), _stream(query)))
    return out


def hard_chunk(summary, table=None, heads=0, choice=None, inplace=False):
    """Compose strip summaries into inclusive boundaries (same shape; aliases the input if inplace)."""
    if not (torch.is_tensor(summary) and summary.is_cuda and summary.dtype == torch.int32 and summary.is_contiguous()):
        _fail('hard summary must be contiguous CUDA int32')
    if table is not None:
        if not (torch.is_tensor(table) and table.device.type == 'cpu' and table.dtype == torch.int64 and table.dim() == 2
                and table.size(1) == 7):
            _fail('layout must be CPU int64 [sequences,7]')
        spans = [(begin, m) for begin, m, *_ in table.tolist() if m]
        tokens = sum(m for _, m in spans)
        expected = sum(heads * ((m - 1) // 32) * m for _, m in spans)
        if heads <= 0 or summary.dim() != 1 or summary.numel() != expected or tokens % 256 or any(m % 256 for _, m in spans):
            _fail('invalid packed hard summary/heads')
        records, rows, _ = _row_table(spans, heads, summary.device)
        with torch.cuda.device(summary.device), _routed(choice, summary.device):
            out = summary if inplace else torch.empty_like(summary)
            if rows:
                _lib.check(_abi.dism_hard_chunk_packed(summary.data_ptr(), out.data_ptr(), records.data_ptr(), len(spans), rows,
                                                       heads, tokens, _stream(summary)))
        return out
    if summary.dim() != 4:
        _fail('fixed hard summary must be [B,H,C,N]')
    b, h, c, n = summary.shape
    if b * h <= 0 or not (heads == 0 or heads == h):
        _fail('invalid fixed batch/head count')
    if n <= 0 or n % 256 or c != (n - 1) // 32:
        _fail('invalid hard checkpoint shape/alignment')
    with torch.cuda.device(summary.device), _routed(choice, summary.device):
        out = summary if inplace else torch.empty_like(summary)
        _lib.check(_abi.dism_hard_chunk(summary.data_ptr(), out.data_ptr(), b * h, n, _stream(summary)))
    return out


def hard_log_weights(tau, n, choice=None):
    """FP32 log2 geometric-sum table [H,n+1] for per-head tau."""
    if not (torch.is_tensor(tau) and tau.is_cuda and tau.dtype == torch.float32 and tau.dim() == 1
            and tau.is_contiguous() and 0 < tau.numel() <= 65535):
        _fail('tau must be contiguous CUDA FP32 [H]')
    if n <= 0 or n % 256:
        _fail('LUT maximum length must be positive and 256-aligned')
    with torch.cuda.device(tau.device), _routed(choice, tau.device):
        out = torch.empty((tau.numel(), n + 1), dtype=torch.float32, device=tau.device)
        _lib.check(_abi.dism_hard_log_weights(tau.data_ptr(), tau.numel(), int(n), out.data_ptr(), _stream(tau)))
    return out


def _vectors(x, count, names):
    if len(x) != count:
        _fail('expected ' + ','.join(names))
    sq = x[0]
    if not (torch.is_tensor(sq) and sq.is_cuda and sq.dim() == 4):
        _fail('SQ must be CUDA [B,N,H,R]')
    b, n, h, r = sq.shape
    if b <= 0 or h <= 0 or n <= 0 or n % 256:
        _fail('positive dimensions and 256-aligned length required')
    return b, n, h, r


def _check_boundary(boundary, b, h, n, device):
    if boundary is None:
        return 0
    if not (torch.is_tensor(boundary) and boundary.device == device and boundary.dtype == torch.int32
            and boundary.is_contiguous() and tuple(boundary.shape) == (b, h, (n - 1) // 32, n)):
        _fail('hard boundary: invalid device, dtype, shape or stride')
    return boundary.data_ptr()


def _check_lut(lut, h, n, device):
    if not (torch.is_tensor(lut) and lut.device == device and lut.dtype == torch.float32 and lut.dim() == 2
            and lut.size(0) == h and lut.is_contiguous()):
        _fail('invalid hard log-weight table')
    if lut.size(1) <= n:
        _fail('hard log-weight table is too short')


def _layout_arguments(table, hard, boundary, lut, b, h, n, device):
    """Validates hard flags and LUT for the fixed or the packed layout; returns the document-table
    pointer (0 = fixed), the number of hard rows and the longest document."""
    if table is None:
        _check_hard(hard, device, b, h)
        _check_lut(lut, h, n, device)
        return 0, b, n
    _packed_hard(hard, device, h)
    if b != 1:
        _fail('packed labels/layout length mismatch')
    spans = _documents(table, n, hard.size(0))
    if boundary is not None:
        # The reference's forward_hard always hands over the packed rectangle (the documents' [H,(m-1)//32,m] regions,
        # flattened).  It is checked for shape and then left unread: with a packed layout the kernels take run lengths
        # from the labels alone, which gives the same bits.
        expected = sum(h * ((m - 1) // 32) * m for _, m in spans)
        if not (torch.is_tensor(boundary) and boundary.device == device and boundary.dtype == torch.int32
                and boundary.is_contiguous() and boundary.dim() == 1 and boundary.numel() == expected):
            _fail('hard boundary: invalid device, dtype, shape or stride')
    longest = max([m for _, m in spans], default=0)
    _check_lut(lut, h, longest, device)
    return _document_table(spans, n, device).data_ptr(), hard.size(0), max(longest, 256)


# The readout's workspace starts with the position index of both label tensors; the backward of the same
# step can reuse it.  The reuse is explicit: the workspace travels on the normaliser that hard_readout
# returns (the tensor every caller hands to hard_backward), together with the two label tensors it was built
# from and their version counters.  hard_backward takes it only when it is given those same label tensors,
# unmodified as far as torch can tell; a writer that goes through a raw pointer (a custom kernel filling a
# preallocated label buffer) does not bump the counter, so such callers switch the reuse off with
# share_index(False) or pass fresh label tensors per step.
_share_index = True


def share_index(enabled):
    """Let hard_backward reuse the position index that hard_readout built for the same label tensors."""
    global _share_index
    _share_index = bool(enabled)


def _remember_index(norm, iq, ik, workspace):
    if _share_index:
        norm._dism_readout = (iq, ik, iq._version, ik._version, workspace)


def _recall_index(norm, iq, ik):
    entry = getattr(norm, '_dism_readout', None) if _share_index else None
    if entry is not None and entry[0] is iq and entry[1] is ik and entry[2] == iq._version and entry[3] == ik._version:
        return entry[4]
    return None


def hard_readout(x, boundary, lut, table=None, ctas=0, choice=None):
    """x = (sq, sk, v, query labels, key labels, hard) -> (bf16 [B,N,H,DV], FP32 log2 normaliser [B,H,N])."""
    b, n, h, r = _vectors(x, 6, ('SQ', 'SK', 'V', 'query labels', 'key labels', 'hard flags'))
    sq, sk, v, iq, ik, hard = x
    _check(sq, torch.bfloat16, (b, n, h, r), 'SQ')
    _check(sk, torch.bfloat16, (b, n, h, r), 'SK')
    _check(v, torch.bfloat16, None, 'V')
    if v.dim() != 4 or tuple(v.shape[:3]) != (b, n, h):
        _fail('V: invalid device, dtype, shape or stride')
    dv = v.size(3)
    _check(iq, torch.int32, (b, h, n), 'query labels')
    _check(ik, torch.int32, (b, h, n), 'key labels')
    documents_ptr, rows, longest = _layout_arguments(table, hard, boundary, lut, b, h, n, sq.device)
    if ctas < 0:
        _fail('invalid CTA count')
    boundary_ptr = _check_boundary(boundary, b, h, n, sq.device) if table is None else 0
    # The kernels write every row, so outputs start uninitialised; with a route word they start as zeros, which is
    # what a closed route returns (the reference zero-fills them always: dism_v3/src/host/hard_forward.cpp:92-93).
    fresh = torch.empty if choice is None else torch.zeros
    with torch.cuda.device(sq.device), _routed(choice, sq.device):
        out = fresh((b, n, h, dv), dtype=torch.bfloat16, device=sq.device)
        norm = fresh((b, h, n), dtype=torch.float32, device=sq.device)
        size = _abi.dism_hard_readout_workspace(b, h, n)
        workspace = torch.empty((size,), dtype=torch.uint8, device=sq.device)
        _lib.check(_abi.dism_hard_readout(sq.data_ptr(), sk.data_ptr(), v.data_ptr(), iq.data_ptr(), ik.data_ptr(),
                                          hard.data_ptr(), boundary_ptr, documents_ptr, rows, longest, lut.data_ptr(),
                                          lut.size(1), b, n, h, r, dv, int(ctas), out.data_ptr(), norm.data_ptr(),
                                          workspace.data_ptr(), size, _stream(sq)))
        _remember_index(norm, iq, ik, workspace)
    return out, norm


def hard_backward(x, boundary, lut, normalizer, ctas=0, table=None, choice=None):
    """x = (sq, sk, v, dO, query labels, key labels, hard) -> [dSQ f32, dSK bf16, dV bf16, dtau f32[H]]."""
    b, n, h, r = _vectors(x, 7, ('SQ', 'SK', 'V', 'dO', 'query labels', 'key labels', 'hard'))
    sq, sk, v, dout, iq, ik, hard = x
    _check(sq, torch.bfloat16, (b, n, h, r), 'SQ')
    _check(sk, torch.bfloat16, (b, n, h, r), 'SK')
    if not (torch.is_tensor(v) and v.dim() == 4):
        _fail('V: invalid device, dtype, shape or stride')
    dv = v.size(3)
    _check(v, torch.bfloat16, (b, n, h, dv), 'V')
    _check(dout, torch.bfloat16, (b, n, h, dv), 'dO')
    _check(iq, torch.int32, (b, h, n), 'query labels')
    _check(ik, torch.int32, (b, h, n), 'key labels')
    _check(normalizer, torch.float32, (b, h, n), 'log2 normalizer')
    if table is None and not (torch.is_tensor(hard) and hard.dtype == torch.bool and tuple(hard.shape) == (b, h)
                              and hard.is_contiguous() and hard.device == sq.device):
        _fail('sequence hard flags: invalid device, dtype, shape or stride')
    documents_ptr, rows, longest = _layout_arguments(table, hard, boundary, lut, b, h, n, sq.device)
    if ctas < 0:
        _fail('invalid CTA count')
    boundary_ptr = _check_boundary(boundary, b, h, n, sq.device) if table is None else 0
    # zeros under a route word: a closed route returns zero gradients (dism_v3/src/host/hard_backward.cpp:106-108)
    fresh = torch.empty if choice is None else torch.zeros
    with torch.cuda.device(sq.device), _routed(choice, sq.device):
        dsq = fresh((b, n, h, r), dtype=torch.float32, device=sq.device)
        dsk, dv_out = fresh(sk.shape, dtype=sk.dtype, device=sk.device), fresh(v.shape, dtype=v.dtype, device=v.device)
        dtau = fresh((h,), dtype=torch.float32, device=sq.device)
        size = _abi.dism_hard_backward_workspace(b, h, n, lut.size(1))
        workspace = torch.empty((size,), dtype=torch.uint8, device=sq.device)
        index = _recall_index(normalizer, iq, ik)
        if index is not None:
            index.record_stream(torch.cuda.current_stream(sq.device))  # read by this stream's kernels
        _lib.check(_abi.dism_hard_backward(sq.data_ptr(), sk.data_ptr(), v.data_ptr(), dout.data_ptr(),
                                           iq.data_ptr(), ik.data_ptr(), hard.data_ptr(), boundary_ptr,
                                           documents_ptr, rows, longest, lut.data_ptr(), lut.size(1), normalizer.data_ptr(),
                                           b, n, h, r, dv,
                                           int(ctas), dsq.data_ptr(), dsk.data_ptr(), dv_out.data_ptr(),
                                           dtau.data_ptr(), workspace.data_ptr(), size,
                                           index.data_ptr() if index is not None else None, _stream(sq)))
    return [dsq, dsk, dv_out, dtau]


def labels(x, codebook):
    """bf16 rows [B,N,H,D] against bf16 codebooks [H,V,D] -> int32 labels [B,H,N] (lowest index on ties)."""
    _check(x, torch.bfloat16, None, 'x')
    if x.dim() != 4:
        _fail('x must be [B,N,H,D]')
    b, n, h, d = x.shape
    _check(codebook, torch.bfloat16, None, 'codebook')
    if codebook.dim() != 3 or codebook.size(0) != h or codebook.size(2) != d or codebook.device != x.device:
        _fail('codebook must be [H,V,D] on the device of x')
    with torch.cuda.device(x.device):
        out = torch.empty((b, h, n), dtype=torch.int32, device=x.device)
        _lib.check(_abi.dism_labels(x.data_ptr(), codebook.data_ptr(), b, n, h, d, codebook.size(1), out.data_ptr(),
                                    _stream(x)))
    return out


def labels_pair(x0, codebook0, x1, codebook1):
    """labels(x0, codebook0) and labels(x1, codebook1) for two tensors of one shape (the q and k side of a step) in one launch."""
    for x, codebook in ((x0, codebook0), (x1, codebook1)):
        _check(x, torch.bfloat16, None, 'x')
        _check(codebook, torch.bfloat16, None, 'codebook')
    if x0.dim() != 4 or x1.shape != x0.shape or x1.device != x0.device:
        _fail('both x must be [B,N,H,D] on one device')
    b, n, h, d = x0.shape
    if (codebook0.dim() != 3 or codebook0.size(0) != h or codebook0.size(2) != d or codebook1.shape != codebook0.shape
            or codebook0.device != x0.device or codebook1.device != x0.device):
        _fail('both codebooks must be [H,V,D] on the device of x')
    with torch.cuda.device(x0.device):
        out0, out1 = (torch.empty((b, h, n), dtype=torch.int32, device=x0.device) for _ in range(2))
        _lib.check(_abi.dism_labels_pair(x0.data_ptr(), codebook0.data_ptr(), out0.data_ptr(), x1.data_ptr(), codebook1.data_ptr(),
                                         out1.data_ptr(), b, n, h, d, codebook0.size(1), _stream(x0)))
    return out0, out1


def longest_match(streams):
    """int32 symbol streams [B,N] -> (end index, run length, next symbol), each int32 [B,N]."""
    _check(streams, torch.int32, None, 'streams')
    if streams.dim() != 2:
        _fail('streams must be [B,N]')
    b, n = streams.shape
    with torch.cuda.device(streams.device):
        end, length, nxt = (torch.empty_like(streams) for _ in range(3))
        size = _abi.dism_longest_match_workspace(b, n)
        workspace = torch.empty((size,), dtype=torch.uint8, device=streams.device)
        _lib.check(_abi.dism_longest_match(streams.data_ptr(), b, n, end.data_ptr(), length.data_ptr(),
                                           nxt.data_ptr(), workspace.data_ptr(), size, _stream(streams)))
    return end, length, nxt


def core_forward(*args, **kwargs):
    raise NotImplementedError('the soft path is not built in this library')


def core_backward(*args, **kwargs):
    raise NotImplementedError('the soft path is not built in this library')
