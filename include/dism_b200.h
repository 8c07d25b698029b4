/*
 * dism_b200 — C ABI of the B200 (sm_100a) implementation of the flash_dism hard path.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its kernels on `stream`
 * (a cudaStream_t passed as void*; NULL = the legacy default stream), never synchronises the
 * host, and returns 0 on success or a DISM_E* code; dism_last_error() then holds a message for
 * the calling thread.  Layouts follow the reference: vectors are contiguous bf16 [B,N,H,C],
 * labels are contiguous int32 [B,H,N], hard flags are bytes [B,H] (non-zero = hard), N is a
 * positive multiple of 256.  `ctas` caps the grid (0 = fill the device); results never depend
 * on it.  Each declaration names the reference interface it stands in for.
 */
#ifndef DISM_B200_H
#define DISM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { DISM_OK = 0, DISM_EINVAL = 1, DISM_EUNSUPPORTED = 2, DISM_ECUDA = 3 };

/* Message of the last failing call on this thread ("" if none). */
const char *dism_last_error(void);
/* ABI revision; bumped on any signature change. */
int dism_abi_version(void);

/* Route word of a captured CUDA graph: the `choice` argument of the reference's hard operators
 * (dism_v3/include/host/graph_route.h:4-10 validates it, include/common/graph_route.cuh:8-13 reads it;
 * passed to the kernels in src/host/hard_summary.cpp, hard_forward.cpp, hard_backward.cpp).
 * `choice` is one int32 in device memory, or NULL.  While it is set, every kernel that this THREAD
 * launches through dism_hard_summary, dism_hard_chunk, dism_hard_log_weights, dism_hard_dlog_weights,
 * dism_hard_readout(_static) and dism_hard_backward reads the word with acquire semantics when it
 * starts and returns at once, unless the word is 0 (the backward's tile kernels instead find an
 * empty tile plan that its plan kernel wrote into the workspace).  No operand is read, no output written.  The word
 * is read at execution time, so a captured graph follows the value written before each replay.
 * Set it before the calls of one operator and clear it (NULL) afterwards; the discretiser and
 * dism_longest_match are not routed.  Outputs of a closed route are left as they were. */
int dism_route_word(const uint32_t *choice);

/* Discretiser: labels[b,h,n] = argmax_v <x[b,n,h,:], codebook[h,v,:]>, lowest index on ties,
 * FP32 accumulation in ascending d.  x bf16 [B,N,H,D], codebook bf16 [H,V,D], D in {32,64,128}.
 * Stands in for the label output of emb_fwd (dism_v3/python/flash_dism/emb_kernel.py:88-108,
 * 155-189) and of kernels/interp_true.py:8-65. */
int dism_labels(const void *x, const void *codebook, int batch, int n, int heads, int d, int vocab,
                int32_t *labels, void *stream);
/* The same for two tensors of one shape in one launch: the q and the k side of a step, each with its own codebook
 * and label output.  The reference discretises q and k with two launches of the same kernel
 * (dism_v3/python/flash_dism/kernels/interp_true.py:51-65); here they share one pipeline fill and drain. */
int dism_labels_pair(const void *x0, const void *codebook0, int32_t *labels0, const void *x1, const void *codebook1,
                     int32_t *labels1, int batch, int n, int heads, int d, int vocab, void *stream);
/* The discretiser's tensor-memory pipeline bounds every wait of its roles on one another; *code is
 * the first wait that ran out in any dism_labels launch on the current device since the last call
 * (0: none, the only value a correct run produces); the call clears it.  Synchronises the device.
 * No counterpart in the reference. */
int dism_labels_fault(int *code);
/* Exercises that bounded wait without the pipeline: one tiny kernel whose two warps wait (through the
 * pipeline's own wait routine) on a barrier that nothing ever completes.  The first to run out, after
 * about a second at most, records `code` (> 0) as the fault and releases the other.
 * outcome[0..1] (host memory) receive 1 if a wait came back satisfied, 0 if it gave up — both must be 0;
 * dism_labels_fault then returns `code`.  The call allocates 8 bytes, synchronises `stream`, and leaves the
 * context usable.  No counterpart in the reference. */
int dism_labels_wait_selftest(int code, int *outcome, void *stream);

/* Strip summaries: summary int32 [B,H,(N-1)/32,N]; non-causal and soft entries are -1.
 * Stands in for cu_flash_dism.hard_summary (dism_v3/src/frontend.cpp:309-312,
 * dism_v3/src/host/hard_summary.cpp:11-73), fixed-length layout.  ik and summary 16-byte aligned. */
int dism_hard_summary(const int32_t *iq, const int32_t *ik, const uint8_t *hard, int batch, int heads,
                      int n, int ctas, int32_t *summary, void *stream);

/* Boundary composition over [BH,(N-1)/32,N]; `boundary` may alias `summary` (in place).
 * Stands in for cu_flash_dism.hard_chunk (dism_v3/src/host/hard_chunk.cpp:10-68).  boundary 16-byte aligned. */
int dism_hard_chunk(const int32_t *summary, int32_t *boundary, int batch_heads, int n, void *stream);

/* The same two stages over a pack of documents (one batch row of n tokens): the `table` branches of
 * dism_v3/src/host/hard_summary.cpp:29-60 and dism_v3/src/host/hard_chunk.cpp:18-45.  The rectangle is the
 * documents' [H,(length-1)/32,length] regions one after the other (the reference's ForwardOffset * H layout,
 * dism_v3/include/varlen/layout.cuh:17-20).  `table` is DEVICE int64 [documents,4], one record per non-empty
 * document in order: first position, length (both multiples of 256), rows before the document (a row is
 * one (head, strip): H * (length-1)/32 per document), rectangle elements before it; `rows` is the total.
 * The caller builds and vouches for the table (the library cannot read it on the host); `hard` is
 * [hard_rows,H], a document lies inside one training row of n / hard_rows tokens. */
int dism_hard_summary_packed(const int32_t *iq, const int32_t *ik, const uint8_t *hard, const int64_t *table,
                             int documents, int64_t rows, int heads, int n, int hard_rows, int ctas,
                             int32_t *summary, void *stream);
int dism_hard_chunk_packed(const int32_t *summary, int32_t *boundary, const int64_t *table, int documents,
                           int64_t rows, int heads, int n, void *stream);

/* lut float [H, n+1]: log2 of sum_{s=1..l} exp(s*tau[h]); entry 0 is -1e6.
 * Stands in for cu_flash_dism.hard_log_weights (dism_v3/src/host/hard_forward.cpp:11-23). */
int dism_hard_log_weights(const float *tau, int heads, int n, float *lut, void *stream);

/* out float [H, lut_stride]: g[h,l] = d ln W_l / d tau[h] for W_l = sum_{s=1..l} exp(s*tau[h]), with tau recovered from
 * the table itself (lut[h,1] = tau[h] * log2 e); entry 0 is 0.  dism_hard_backward builds this table in its
 * workspace on every call; the entry point makes it testable and reusable by itself.
 * Stands in for hard_dlog_weights_kernel (dism_v3/src/hard_backward.cu:8-24), which the reference launches
 * inside cu_flash_dism.hard_backward (dism_v3/src/host/hard_backward.cpp). */
int dism_hard_dlog_weights(const float *lut, int heads, int lut_stride, float *out, void *stream);

/* Bytes of scratch dism_hard_readout needs for this shape (both position indices and the tile plan). */
size_t dism_hard_readout_workspace(int batch, int heads, int n);

/* Fused hard readout.  `boundary` is the rectangle of dism_hard_chunk or NULL (the kernel then
 * derives run lengths from the labels alone); lut has row stride lut_stride > N (packed: > the
 * longest document).  Packed layout (the reference's `table` argument, dism_v3/src/host/hard_forward.cpp:
 * 56-85): batch 1, `documents` is a device int32 [N/256, 2] table giving, for every 256-position
 * block, the [begin, end) of the 256-aligned document that contains it, and `hard` is
 * [hard_rows, H] over equal training rows of N / hard_rows positions, and `longest_document` is the
 * length of the longest document (the host knows it when it builds the table; lut_stride must exceed it);
 * fixed layout: documents NULL, hard_rows = batch, longest_document ignored.
 * out bf16 [B,N,H,DV], lse2 float [B,H,N]; soft (batch, head) rows are written as zeros.
 * R in {16,32}, DV in {32,64,128}; vectors 16-byte aligned.  `workspace` is caller-owned scratch of
 * dism_hard_readout_workspace bytes, 256-byte aligned; its contents are dead after the call.
 * Stands in for cu_flash_dism.hard_readout (dism_v3/src/host/hard_forward.cpp:25-113). */
int dism_hard_readout(const void *sq, const void *sk, const void *v, const int32_t *iq, const int32_t *ik,
                      const uint8_t *hard, const int32_t *boundary, const int32_t *documents, int hard_rows,
                      int longest_document, const float *lut, int lut_stride, int batch, int n, int heads, int r, int dv, int ctas,
                      void *out, float *lse2, void *workspace, size_t workspace_bytes, void *stream);

/* The same readout for callers that cannot supply scratch memory (an operator hook that only gets its
 * input and output buffers, a server whose memory pool already holds the whole GPU: cudaMalloc there
 * serialises the device and may fail).  It has no counterpart in the reference.  The position index
 * lives in a fixed array inside the library (DISM_READOUT_STATIC_BYTES, held on every GPU that loads
 * the library until the process exits); the call allocates nothing.  Limits: the shape's scratch
 * (dism_hard_readout_workspace: about 49 bytes per position plus 112 KiB per (batch, head)) must fit,
 * otherwise DISM_EINVAL; all calls on a
 * device share the array, so calls that overlap on the GPU race and must be serialised by the caller;
 * the first call on each device resolves the array's address, which may load the library image (and with it
 * the array) onto that device: make it at start-up, before the host's pool takes the remaining memory and
 * before any stream capture starts.  The message of a failing call is in dism_hard_readout_static_error(). */
#define DISM_READOUT_STATIC_BYTES 8388608 /* 8 MiB: e.g. 16 (batch x head) rows of 8192 positions */
int dism_hard_readout_static(const void *sq, const void *sk, const void *v, const int32_t *iq,
                             const int32_t *ik, const uint8_t *hard, const int32_t *boundary,
                             const float *lut, int lut_stride, int batch, int n, int heads, int r, int dv,
                             int ctas, void *out, float *lse2, void *stream);
const char *dism_hard_readout_static_error(void);

/* Bytes of scratch dism_hard_backward needs for this shape. */
size_t dism_hard_backward_workspace(int batch, int heads, int n, int lut_stride);

/* Hard backward: dsq float [B,N,H,R], dsk bf16 [B,N,H,R], dv bf16 [B,N,H,DV], dtau float [H]
 * (gradient of the natural-log coefficient).  lse2 is the normaliser the forward returned;
 * `boundary` may be NULL; `documents`/`hard_rows`/`longest_document` as in dism_hard_readout; `workspace` is caller-owned scratch of dism_hard_backward_workspace bytes.
 * `readout_workspace` is NULL, or the workspace a dism_hard_readout call filled for the same labels, batch,
 * heads and n and that nothing has written since: its position index is then reused instead of rebuilt
 * (the reference's backward likewise consumes state its forward saved).
 * Stands in for cu_flash_dism.hard_backward (dism_v3/src/host/hard_backward.cpp:13-141). */
int dism_hard_backward(const void *sq, const void *sk, const void *v, const void *dout, const int32_t *iq,
                       const int32_t *ik, const uint8_t *hard, const int32_t *boundary,
                       const int32_t *documents, int hard_rows, int longest_document, const float *lut, int lut_stride,
                       const float *lse2, int batch, int n, int heads, int r, int dv, int ctas, float *dsq,
                       void *dsk, void *dv_out, float *dtau, void *workspace, size_t workspace_bytes,
                       const void *readout_workspace, void *stream);

/* Single longest earlier match of symbol streams int32 [B,N] (labels of queries and keys are
 * the same stream): for every i the most recent j < i with the longest run L(i,j), its length,
 * and the symbol after it (-1 when nothing matches).  The reference defines L(i,j)
 * (dism_v3/python/flash_dism/summary.py:8-16) but no single winner: this reduction is ours. */
size_t dism_longest_match_workspace(int batch, int n);
int dism_longest_match(const int32_t *streams, int batch, int n, int32_t *end, int32_t *length,
                       int32_t *next, void *workspace, size_t workspace_bytes, void *stream);

/* Per-kernel device timing for benchmarks (no counterpart in the reference, which times whole
 * calls with CUDA events from Python).  dism_profile_enable(1) clears the records and makes every
 * later launch record CUDA events around each kernel on its launch stream;
 * dism_profile_read(i, ...) waits for record i and returns its kernel name and milliseconds.
 * Process-wide and not thread-safe: switch it on from one thread, around the calls to be timed. */
int dism_profile_enable(int on);
int dism_profile_count(void);
int dism_profile_read(int index, char *name, int capacity, float *milliseconds);

#ifdef __cplusplus
}
#endif
#endif
