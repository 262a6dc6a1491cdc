// fkda_fwd_noalloc: the forward pass for callers that cannot allocate device memory.
//
// Who needs this: code that runs where cudaMalloc (or a framework allocator built on it) is not
// available or not allowed at call time -- for example a serving loop that has handed all device
// memory to a pool it does not control, a plugin invoked from inside another library's callback, or
// a host thread that must never take the allocator's locks or trigger its implicit device
// synchronisation.  Such callers still own their input and output tensors; what they lack is a
// place for the per-chunk operand records that the prepare kernel hands to the recurrence kernel.
//
// Here that scratch is a fixed array in the library's own device image.  It exists once per GPU that
// loads the library (FKDA_NOALLOC_SCRATCH_BYTES, held until the process exits) and is shared by every
// call: two calls whose kernels overlap on the GPU (different streams, or different host threads)
// race on it, so callers must serialise their use of this entry point per device.  The array keeps
// the previous call's contents; the only part that has to start from zero (the work-queue counter
// and the device status word in its header) is cleared by every call before the kernels run.
#include <atomic>

#include "fkda_internal.h"

namespace {

// File-scope device array.  In host code this name is only a stand-in for the symbol: its device
// address has to be asked for with cudaGetSymbolAddress, per device, and that address is what the
// kernels receive.
static __device__ __align__(256) unsigned char g_noalloc_scratch[FKDA_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_addr[kMaxDevices];   // zero-initialised; every thread that resolves an address stores the same value

// One-time set-up for the current device: resolves the device address of the array.
// Runs on the first call per device; that call should happen outside any stream capture.  (A first call that
// takes the slab pipeline -- a fixed batch of few long sequences -- also creates that pipeline's side stream and
// events, once per device: driver objects, no device memory.)
int scratch_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FKDA_ERR_LAUNCH;
    void* ptr = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr) return FKDA_ERR_LAUNCH;
        g_scratch_addr[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return FKDA_OK;
}

}  // namespace

namespace fkda {
void* noalloc_scratch_or_null() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    return g_scratch_addr[dev].load(std::memory_order_acquire);
}
}  // namespace fkda

extern "C" {

size_t fkda_noalloc_scratch_bytes(void) { return (size_t)FKDA_NOALLOC_SCRATCH_BYTES; }

int fkda_fwd_noalloc(const fkda_fwd_params* p, void* stream_v) {
    if (p == nullptr) return FKDA_ERR_NULL_POINTER;
    if (p->B <= 0 || p->T < 0 || p->H <= 0 || p->N <= 0) return FKDA_ERR_BAD_SHAPE;
    const size_t need = fkda_workspace_bytes_for(p);  // by the path this call takes: a decode step needs 256 bytes
    if (need > (size_t)FKDA_NOALLOC_SCRATCH_BYTES) return FKDA_ERR_NOALLOC_TOO_LARGE;
    void* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc != FKDA_OK) return rc;
    fkda_fwd_params q = *p;  // same call, with the built-in scratch in place of a caller workspace
    q.workspace = scratch;
    q.workspace_bytes = (size_t)FKDA_NOALLOC_SCRATCH_BYTES;
    return fkda_fwd(&q, stream_v);
}

}  // extern "C"
