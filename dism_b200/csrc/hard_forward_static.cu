// dism_hard_readout_static: the fused hard readout for callers that cannot give the library any
// scratch memory.
//
// Some hosts call an operator with nothing but its input and output buffers: the request path of
// an inference server whose memory was handed to the server's own pool at start-up, or a plugin
// hook whose contract forbids device allocation because cudaMalloc serialises the whole device
// and can fail once that pool holds everything.  Such a caller has no workspace to pass to
// dism_hard_readout.  This entry point keeps the scratch the readout needs (the position indices
// of both sides and the tile plan) in a fixed array that is part of the library image, so the call
// allocates nothing: no cudaMalloc, no cudaFree, no allocating library routine.
//
// The price is a fixed ceiling and shared state.  Every GPU that loads the library holds the
// array (DISM_READOUT_STATIC_BYTES) until the process exits; shapes whose index does not fit are
// rejected; all calls on a device use the same array, so two calls that overlap on the GPU (two
// streams, two threads) race and must be serialised by the caller.  Nothing in the array has to
// start at zero: each call rebuilds every entry it later reads.
#include "../../include/dism_b200.h"
#include "dism_common.cuh"

#include <atomic>
#include <cstdio>

namespace {

// In host code this name is only a handle for the runtime, not a device address: the address a
// kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
static __device__ __align__(256) unsigned char static_index[DISM_READOUT_STATIC_BYTES];

constexpr int MAX_DEVICES = 64;
std::atomic<void*> device_address[MAX_DEVICES] = {};  // written once per device; threads may race to resolve the same value
thread_local char static_error[256] = "";

}  // namespace

extern "C" {

const char* dism_hard_readout_static_error(void) { return static_error; }

int dism_hard_readout_static(const void* sq, const void* sk, const void* v, const int32_t* iq, const int32_t* ik,
                             const uint8_t* hard, const int32_t* boundary, const float* lut, int lut_stride,
                             int batch, int n, int heads, int r, int dv, int ctas, void* out, float* lse2,
                             void* stream) {
    static_error[0] = 0;
    if (batch <= 0 || heads <= 0 || n <= 0) {
        snprintf(static_error, sizeof(static_error), "positive dimensions required");
        return DISM_EINVAL;
    }
    const size_t needed = dism_hard_readout_workspace(batch, heads, n);
    if (needed > size_t(DISM_READOUT_STATIC_BYTES)) {
        snprintf(static_error, sizeof(static_error),
                 "shape needs %zu bytes of scratch but the built-in scratch holds %zu; "
                 "use dism_hard_readout with a caller-owned workspace",
                 needed, size_t(DISM_READOUT_STATIC_BYTES));
        return DISM_EINVAL;
    }
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status == cudaSuccess && (device < 0 || device >= MAX_DEVICES)) status = cudaErrorInvalidDevice;
    void* address = status == cudaSuccess ? device_address[device].load(std::memory_order_acquire) : nullptr;
    if (status == cudaSuccess && !address) {
        // First call on this device: resolve the array's device address.  This is a set-up step: it may load the
        // library's image on the device (which takes device memory for the array), so make the first call on each
        // device at start-up, before the host's pool takes the remaining memory and before any stream capture begins.
        status = cudaGetSymbolAddress(&address, static_index);
        if (status == cudaSuccess) device_address[device].store(address, std::memory_order_release);
    }
    if (status != cudaSuccess) {
        snprintf(static_error, sizeof(static_error), "built-in scratch unavailable: %s", cudaGetErrorString(status));
        return DISM_ECUDA;
    }
    const int code = dism_hard_readout(sq, sk, v, iq, ik, hard, boundary, nullptr, batch, n, lut, lut_stride, batch, n, heads, r, dv, ctas,
                                       out, lse2, address, size_t(DISM_READOUT_STATIC_BYTES), stream);
    if (code) snprintf(static_error, sizeof(static_error), "%s", dism_last_error());
    return code;
}

}  // extern "C"
