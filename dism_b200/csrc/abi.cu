// C ABI of the library: argument validation, error reporting and dispatch to the launchers.
// The messages keep the key words the reference's checks use ("256-aligned", "CTA", "too short"),
// so callers that match on them keep working.
#include "../../include/dism_b200.h"
#include "dism_common.cuh"

#include <climits>
#include <cstdarg>
#include <cstdio>

namespace {
thread_local char last_error[512] = "";

int fail(int code, const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(last_error, sizeof(last_error), format, args);
    va_end(args);
    return code;
}
int cuda_status(cudaError_t status, const char* what) {
    if (status == cudaSuccess) return DISM_OK;
    return fail(DISM_ECUDA, "%s: %s", what, cudaGetErrorString(status));
}
bool aligned(const void* p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) & (bytes - 1)) == 0; }

int check_shape(int batch, int heads, int n) {
    if (batch <= 0 || heads <= 0 || n <= 0 || n > INT_MAX - 256 || n % 256)
        return fail(DISM_EINVAL, "positive dimensions and 256-aligned sequence length required");
    if (int64_t(batch) * heads > 65535)  // (batch, head) slices are one grid dimension of every kernel
        return fail(DISM_EINVAL, "batch * heads must not exceed 65535");
    return DISM_OK;
}
int check_dims(int r, int dv) {
    if ((r != 16 && r != 32) || (dv != 32 && dv != 64 && dv != 128))
        return fail(DISM_EUNSUPPORTED, "unsupported readout shape R=%d DV=%d (R in {16,32}, DV in {32,64,128})", r, dv);
    return DISM_OK;
}
}  // namespace

// ---- optional per-kernel timing ---------------------------------------------------------------------
namespace {
constexpr int MAX_RECORDS = 256;
struct Record {
    cudaEvent_t start, stop;
    char name[48];
};
bool timing_on = false;
int record_count = 0, events_made = 0;
Record records[MAX_RECORDS];
}  // namespace

namespace {
thread_local const unsigned* current_route = nullptr;
}  // namespace

namespace dism {
const unsigned* route_word() { return current_route; }

KernelTimer::KernelTimer(const char* name, cudaStream_t s) : slot(-1), stream(s) {
    if (!timing_on || record_count >= MAX_RECORDS) return;
    slot = record_count++;
    if (slot >= events_made) {
        cudaEventCreate(&records[slot].start);
        cudaEventCreate(&records[slot].stop);
        events_made = slot + 1;
    }
    snprintf(records[slot].name, sizeof(records[slot].name), "%s", name);
    cudaEventRecord(records[slot].start, stream);
}
KernelTimer::~KernelTimer() {
    if (slot >= 0) cudaEventRecord(records[slot].stop, stream);
}
}  // namespace dism

extern "C" {

int dism_profile_enable(int on) {
    timing_on = on != 0;
    record_count = 0;
    return DISM_OK;
}

int dism_profile_count(void) { return record_count; }

int dism_profile_read(int index, char* name, int capacity, float* milliseconds) {
    if (index < 0 || index >= record_count || !name || capacity <= 0 || !milliseconds)
        return fail(DISM_EINVAL, "no such timing record");
    if (cudaError_t status = cudaEventSynchronize(records[index].stop); status != cudaSuccess)
        return cuda_status(status, "profile_read");
    snprintf(name, size_t(capacity), "%s", records[index].name);
    return cuda_status(cudaEventElapsedTime(milliseconds, records[index].start, records[index].stop), "profile_read");
}

const char* dism_last_error(void) { return last_error; }
int dism_abi_version(void) { return 9; }

int dism_route_word(const uint32_t* choice) {
    if (choice && !aligned(choice, 4)) return fail(DISM_EINVAL, "graph choice must be one aligned device int32");
    current_route = choice;
    return DISM_OK;
}

int dism_labels(const void* x, const void* codebook, int batch, int n, int heads, int d, int vocab,
                int32_t* labels, void* stream) {
    if (!x || !codebook || !labels) return fail(DISM_EINVAL, "null pointer");
    if (batch <= 0 || n <= 0 || heads <= 0 || vocab <= 0 || int64_t(batch) * heads > 65535)
        return fail(DISM_EINVAL, "positive dimensions required (batch*heads <= 65535)");
    if (d != 32 && d != 64 && d != 128) return fail(DISM_EUNSUPPORTED, "unsupported label width D=%d", d);
    if (!aligned(x, 16) || !aligned(codebook, 16)) return fail(DISM_EINVAL, "x and codebook must be 16-byte aligned");
    return cuda_status(dism::launch_labels(static_cast<const __nv_bfloat16*>(x),
                                           static_cast<const __nv_bfloat16*>(codebook), batch, n, heads, d, vocab,
                                           labels, static_cast<cudaStream_t>(stream)), "labels");
}

int dism_labels_pair(const void* x0, const void* codebook0, int32_t* labels0, const void* x1, const void* codebook1,
                     int32_t* labels1, int batch, int n, int heads, int d, int vocab, void* stream) {
    if (!x0 || !codebook0 || !labels0 || !x1 || !codebook1 || !labels1) return fail(DISM_EINVAL, "null pointer");
    if (batch <= 0 || n <= 0 || heads <= 0 || vocab <= 0 || int64_t(batch) * heads > 65535)
        return fail(DISM_EINVAL, "positive dimensions required (batch*heads <= 65535)");
    if (d != 32 && d != 64 && d != 128) return fail(DISM_EUNSUPPORTED, "unsupported label width D=%d", d);
    if (!aligned(x0, 16) || !aligned(codebook0, 16) || !aligned(x1, 16) || !aligned(codebook1, 16))
        return fail(DISM_EINVAL, "x and codebook must be 16-byte aligned");
    using bf = __nv_bfloat16;
    return cuda_status(dism::launch_labels_pair(static_cast<const bf*>(x0), static_cast<const bf*>(codebook0), labels0,
                                                static_cast<const bf*>(x1), static_cast<const bf*>(codebook1), labels1, batch, n, heads,
                                                d, vocab, static_cast<cudaStream_t>(stream)), "labels");
}

int dism_labels_fault(int* code) {
    if (!code) return fail(DISM_EINVAL, "null pointer");
    return cuda_status(dism::read_labels_fault(code), "labels fault code");
}

int dism_labels_wait_selftest(int code, int* outcome, void* stream) {
    if (!outcome || code <= 0) return fail(DISM_EINVAL, "outcome array and a positive code required");
    return cuda_status(dism::run_wait_selftest(code, outcome, static_cast<cudaStream_t>(stream)), "wait self-test");
}

int dism_hard_summary(const int32_t* iq, const int32_t* ik, const uint8_t* hard, int batch, int heads, int n,
                      int ctas, int32_t* summary, void* stream) {
    if (int status = check_shape(batch, heads, n)) return status;
    if (!iq || !ik || !hard || (!summary && n > 32)) return fail(DISM_EINVAL, "null pointer");
    if (ctas < 0) return fail(DISM_EINVAL, "invalid CTA count");
    if (!aligned(summary, 16) || !aligned(ik, 16)) return fail(DISM_EINVAL, "key labels and hard summary must be 16-byte aligned");
    return cuda_status(dism::launch_hard_summary(iq, ik, hard, batch, heads, n, ctas, summary,
                                                 static_cast<cudaStream_t>(stream)), "hard_summary");
}

int dism_hard_chunk(const int32_t* summary, int32_t* boundary, int batch_heads, int n, void* stream) {
    if (int status = check_shape(1, batch_heads, n)) return status;
    if (!summary || !boundary) return fail(DISM_EINVAL, "null pointer");
    if (!aligned(boundary, 16)) return fail(DISM_EINVAL, "hard boundary must be 16-byte aligned");
    if (int64_t(n) + int64_t((n - 1) / 32) * 32 > INT_MAX) return fail(DISM_EINVAL, "invalid hard checkpoint shape");
    return cuda_status(dism::launch_hard_chunk(summary, boundary, batch_heads, n, static_cast<cudaStream_t>(stream)),
                       "hard_chunk");
}

static int check_pack(const int64_t* table, int documents, int64_t rows, int heads, int n) {
    if (int status = check_shape(1, heads, n)) return status;
    if (documents < 0 || rows < 0 || (documents > 0 && !table)) return fail(DISM_EINVAL, "invalid packed document table");
    if (documents > n / 256) return fail(DISM_EINVAL, "more documents than 256-token blocks: packed labels/layout length mismatch");
    if (rows > int64_t(heads) * ((n - 1) / 32 + 1)) return fail(DISM_EINVAL, "packed rows exceed the layout");
    return DISM_OK;
}

int dism_hard_summary_packed(const int32_t* iq, const int32_t* ik, const uint8_t* hard, const int64_t* table, int documents,
                             int64_t rows, int heads, int n, int hard_rows, int ctas, int32_t* summary, void* stream) {
    if (int status = check_pack(table, documents, rows, heads, n)) return status;
    if (!iq || !ik || !hard || (!summary && rows)) return fail(DISM_EINVAL, "null pointer");
    if (hard_rows <= 0 || n % hard_rows || (n / hard_rows) % 256)
        return fail(DISM_EINVAL, "packed hard rows must evenly divide tokens into 256-aligned training rows");
    if (ctas < 0) return fail(DISM_EINVAL, "invalid CTA count");
    if (!aligned(summary, 16) || !aligned(ik, 16)) return fail(DISM_EINVAL, "key labels and hard summary must be 16-byte aligned");
    return cuda_status(dism::launch_hard_summary_packed(iq, ik, hard, reinterpret_cast<const long long*>(table), documents, rows,
                                                        heads, n, hard_rows, ctas, summary, static_cast<cudaStream_t>(stream)),
                       "hard_summary");
}

int dism_hard_chunk_packed(const int32_t* summary, int32_t* boundary, const int64_t* table, int documents, int64_t rows,
                           int heads, int n, void* stream) {
    if (int status = check_pack(table, documents, rows, heads, n)) return status;
    if ((!summary || !boundary) && rows) return fail(DISM_EINVAL, "null pointer");
    if (!aligned(boundary, 16)) return fail(DISM_EINVAL, "hard boundary must be 16-byte aligned");
    return cuda_status(dism::launch_hard_chunk_packed(summary, boundary, reinterpret_cast<const long long*>(table), documents, rows,
                                                      static_cast<cudaStream_t>(stream)), "hard_chunk");
}

int dism_hard_log_weights(const float* tau, int heads, int n, float* lut, void* stream) {
    if (!tau || !lut) return fail(DISM_EINVAL, "null pointer");
    if (heads <= 0 || heads > 65535) return fail(DISM_EINVAL, "tau must hold 1..65535 heads");
    if (n <= 0 || n > INT_MAX - 256 || n % 256)
        return fail(DISM_EINVAL, "LUT maximum length must be positive and 256-aligned");
    return cuda_status(dism::launch_log_weights(tau, heads, n, lut, static_cast<cudaStream_t>(stream)),
                       "hard_log_weights");
}

int dism_hard_dlog_weights(const float* lut, int heads, int lut_stride, float* out, void* stream) {
    if (!lut || !out) return fail(DISM_EINVAL, "null pointer");
    if (heads <= 0 || heads > 65535) return fail(DISM_EINVAL, "the table must hold 1..65535 heads");
    if (lut_stride < 2) return fail(DISM_EINVAL, "the table must hold lengths 0 and 1 at least");
    return cuda_status(dism::launch_dlog_weights(lut, heads, lut_stride, out, static_cast<cudaStream_t>(stream)),
                       "hard_dlog_weights");
}

static int check_documents(const int32_t* documents, int hard_rows, int longest_document, int lut_stride, const int32_t* boundary,
                           int batch, int n) {
    if (!documents) {
        if (hard_rows != batch) return fail(DISM_EINVAL, "fixed hard must be [B,H]");
        if (lut_stride <= n) return fail(DISM_EINVAL, "hard log-weight table is too short");
        return DISM_OK;
    }
    // the kernels index the tables with run lengths up to the longest document
    if (longest_document <= 0 || longest_document > n || longest_document % 256)
        return fail(DISM_EINVAL, "longest document must be a positive 256-aligned length within the pack");
    if (lut_stride <= longest_document) return fail(DISM_EINVAL, "hard log-weight table is too short for the longest document");
    if (batch != 1) return fail(DISM_EINVAL, "packed labels/layout length mismatch: packed layouts use one batch row");
    if (boundary) return fail(DISM_EUNSUPPORTED, "the boundary rectangle is not used with packed layouts; pass NULL");
    if (hard_rows <= 0 || n % hard_rows || (n / hard_rows) % 256)
        return fail(DISM_EINVAL, "packed hard rows must evenly divide tokens into 256-aligned training rows");
    if (!aligned(documents, 8)) return fail(DISM_EINVAL, "document table must be 8-byte aligned");
    return DISM_OK;
}

int dism_hard_readout(const void* sq, const void* sk, const void* v, const int32_t* iq, const int32_t* ik,
                      const uint8_t* hard, const int32_t* boundary, const int32_t* documents, int hard_rows,
                      int longest_document, const float* lut, int lut_stride, int batch,
                      int n, int heads, int r, int dv, int ctas, void* out, float* lse2, void* workspace,
                      size_t workspace_bytes, void* stream) {
    if (int status = check_shape(batch, heads, n)) return status;
    if (int status = check_dims(r, dv)) return status;
    if (!sq || !sk || !v || !iq || !ik || !hard || !lut || !out || !lse2) return fail(DISM_EINVAL, "null pointer");
    if (ctas < 0) return fail(DISM_EINVAL, "invalid CTA count");
    if (int status = check_documents(documents, hard_rows, longest_document, lut_stride, boundary, batch, n)) return status;
    if (!aligned(sq, 16) || !aligned(sk, 16) || !aligned(v, 16) || !aligned(out, 16))
        return fail(DISM_EINVAL, "vector tensors must be 16-byte aligned");
    if (!workspace || workspace_bytes < dism::hard_forward_workspace_bytes(batch, heads, n) || !aligned(workspace, 256))
        return fail(DISM_EINVAL, "workspace missing, too small or misaligned (see dism_hard_readout_workspace)");
    dism::HardShape shape{batch, heads, n, r, dv};
    using bf = __nv_bfloat16;
    return cuda_status(dism::launch_hard_forward(shape, static_cast<const bf*>(sq), static_cast<const bf*>(sk),
                                                 static_cast<const bf*>(v), iq, ik, hard, boundary,
                                                 reinterpret_cast<const int2*>(documents), hard_rows, lut, lut_stride,
                                                 ctas, static_cast<bf*>(out), lse2, workspace,
                                                 static_cast<cudaStream_t>(stream)),
                       "hard_readout");
}

size_t dism_hard_readout_workspace(int batch, int heads, int n) {
    if (batch <= 0 || heads <= 0 || n <= 0) return 0;
    return dism::hard_forward_workspace_bytes(batch, heads, n);
}

size_t dism_hard_backward_workspace(int batch, int heads, int n, int lut_stride) {
    if (batch <= 0 || heads <= 0 || n <= 0 || lut_stride <= 0) return 0;
    return dism::hard_backward_workspace_bytes(batch, heads, n, lut_stride);
}

int dism_hard_backward(const void* sq, const void* sk, const void* v, const void* dout, const int32_t* iq,
                       const int32_t* ik, const uint8_t* hard, const int32_t* boundary, const int32_t* documents,
                       int hard_rows, int longest_document, const float* lut, int lut_stride, const float* lse2, int batch, int n, int heads,
                       int r, int dv, int ctas,
                       float* dsq, void* dsk, void* dv_out, float* dtau, void* workspace, size_t workspace_bytes,
                       const void* readout_workspace, void* stream) {
    if (int status = check_shape(batch, heads, n)) return status;
    if (int status = check_dims(r, dv)) return status;
    if (!sq || !sk || !v || !dout || !iq || !ik || !hard || !lut || !lse2 || !dsq || !dsk || !dv_out || !dtau ||
        !workspace)
        return fail(DISM_EINVAL, "null pointer");
    if (ctas < 0) return fail(DISM_EINVAL, "invalid CTA count");
    if (int status = check_documents(documents, hard_rows, longest_document, lut_stride, boundary, batch, n)) return status;
    if (workspace_bytes < dism::hard_backward_workspace_bytes(batch, heads, n, lut_stride) || !aligned(workspace, 256))
        return fail(DISM_EINVAL, "workspace too small or misaligned (see dism_hard_backward_workspace)");
    if (readout_workspace && !aligned(readout_workspace, 256)) return fail(DISM_EINVAL, "readout workspace misaligned");
    if (!aligned(sq, 16) || !aligned(sk, 16) || !aligned(v, 16) || !aligned(dout, 16) || !aligned(dsq, 16) ||
        !aligned(dsk, 16) || !aligned(dv_out, 16))
        return fail(DISM_EINVAL, "vector tensors must be 16-byte aligned");
    dism::HardShape shape{batch, heads, n, r, dv};
    using bf = __nv_bfloat16;
    return cuda_status(dism::launch_hard_backward(shape, static_cast<const bf*>(sq), static_cast<const bf*>(sk),
                                                  static_cast<const bf*>(v), static_cast<const bf*>(dout), iq, ik,
                                                  hard, boundary, reinterpret_cast<const int2*>(documents), hard_rows, lut,
                                                  lut_stride, lse2, ctas, dsq,
                                                  static_cast<bf*>(dsk), static_cast<bf*>(dv_out), dtau, workspace,
                                                  readout_workspace, static_cast<cudaStream_t>(stream)), "hard_backward");
}

size_t dism_longest_match_workspace(int batch, int n) {
    if (batch <= 0 || n <= 0) return 0;
    return dism::longest_match_workspace_bytes(batch, n);
}

int dism_longest_match(const int32_t* streams, int batch, int n, int32_t* end, int32_t* length, int32_t* next,
                       void* workspace, size_t workspace_bytes, void* stream) {
    if (!streams || !end || !length || !next) return fail(DISM_EINVAL, "null pointer");
    if (batch <= 0 || n <= 0 || n % 8) return fail(DISM_EINVAL, "positive batch and a stream length divisible by 8 required");
    if (!workspace || workspace_bytes < dism::longest_match_workspace_bytes(batch, n) || !aligned(workspace, 256))
        return fail(DISM_EINVAL, "workspace missing, too small or misaligned (see dism_longest_match_workspace)");
    return cuda_status(dism::launch_longest_match(streams, batch, n, end, length, next, workspace,
                                                  static_cast<cudaStream_t>(stream)), "longest_match");
}

}  // extern "C"
