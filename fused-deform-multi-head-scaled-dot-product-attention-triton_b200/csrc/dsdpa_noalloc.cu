// dsdpa_backward_static_scratch: the backward for callers that must not allocate.
//
// Who needs it.  dsdpa_backward leaves the scratch to its caller, which in practice means a
// cudaMalloc or a framework allocator call per backward (or a pool that has to be sized and
// owned by somebody).  Some callers cannot do either: code running inside a region where
// device allocation is forbidden (a real-time inference loop with a fixed memory budget, a
// plugin whose host framework owns all device memory and hands none out, a callback that
// may not call into the allocator because the allocator's lock is held further up the
// stack).  For them the scratch lives inside the library: one fixed array in device memory,
// part of the loaded module, present on every GPU that loads the library until the process
// exits.
//
// What it costs.  DSDPA_STATIC_SCRATCH_BYTES of device memory per GPU whether the entry
// point is ever called or not, a hard upper limit on the problem size (a larger problem is
// refused with DSDPA_ERR_TOO_LARGE, nothing is truncated), and no concurrency: every call
// on a device uses the same array, so two calls whose GPU work overlaps (different streams,
// or different host threads) corrupt each other's scratch.  Serialise them on one stream.
//
// The array keeps whatever the previous call left in it.  Nothing here relies on its
// contents: the parts that must start from zero (the fp32 dK/dV accumulators) are cleared
// on the stream at the start of every call, the rest is written before it is read.
#include <cuda_runtime.h>

#include "../../include/dsdpa.h"

namespace dsdpa {
int report_cuda_failure(int cuda_error);   // dsdpa_api.cu: what dsdpa_last_cuda_error() returns
}

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime's symbol
// table, not a device address: passing it (or its host address) to a kernel would make the
// kernel read and write the wrong memory.  The device address is asked for once per device
// with cudaGetSymbolAddress, below.
static __device__ __align__(256) unsigned char g_static_scratch[DSDPA_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
// (Filled without a lock: two threads that race here look the same address up twice and store
// the same value.)
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the array on `device`, looked up on first use while `device` is the
// current device (the address differs from device to device).
cudaError_t scratch_address(int device, void** out) {
    if (device >= 0 && device < kMaxDevices && g_scratch_addr[device] != nullptr) {
        *out = g_scratch_addr[device];
        return cudaSuccess;
    }
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return e;
    if (prev != device) {
        e = cudaSetDevice(device);
        if (e != cudaSuccess) return e;
    }
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (prev != device) (void)cudaSetDevice(prev);
    if (e != cudaSuccess) return e;
    if (ptr == nullptr) return cudaErrorInvalidSymbol;
    if (device >= 0 && device < kMaxDevices) g_scratch_addr[device] = ptr;
    *out = ptr;
    return cudaSuccess;
}

}  // namespace

extern "C" int dsdpa_backward_static_scratch(const dsdpa_problem* p, const void* q, const void* k, const void* v,
                                             const float* coords, const void* out, const float* lse,
                                             const void* dout, void* dq, void* dk, void* dv, int device,
                                             void* stream) {
    if (!p) return DSDPA_ERR_NULL_POINTER;
    // 0 both for "needs none" and for an invalid problem; the latter is reported by the
    // backward itself
    const size_t need = dsdpa_backward_workspace_bytes(p);
    if (need > (size_t)DSDPA_STATIC_SCRATCH_BYTES) return DSDPA_ERR_TOO_LARGE;
    void* scratch = nullptr;
    if (need > 0) {
        // First call on a device: symbol lookup.  The array is part of the library's device
        // image; with CUDA's lazy module loading the driver may only place that image (and so
        // reserve the array's memory) now, which is why this call belongs into initialisation.
        const cudaError_t e = scratch_address(device, &scratch);
        if (e != cudaSuccess) return dsdpa::report_cuda_failure((int)e);
    }
    // Same kernels, same order, same checks as dsdpa_backward; only the owner of the scratch
    // differs.  The accumulators inside the scratch are zero-filled there on `stream`.
    return dsdpa_backward(p, q, k, v, coords, out, lse, dout, dq, dk, dv, /*dcoords=*/nullptr, scratch, need, device,
                          stream);
}
