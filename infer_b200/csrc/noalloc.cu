// FP8 linear for callers that must not allocate device memory.
//
// The tensor-core decode path splits K and parks partial sums in a scratch buffer that the ordinary entry
// point (fth_b200_fp8_linear) expects from its caller.  Some callers have no way to provide one: a Feather node
// built with a workspace limit of zero (KernelRequest::workspace_limit, include/core/kernel.h:50) may not
// acquire temporary device buffers, and a session whose device memory was planned and frozen when the plan was
// compiled has nowhere to put a buffer that was not in the plan.  For them the scratch lives in this library's
// own image: a fixed array in device global memory that every GPU loading the library carries until the
// process exits.
#include <mutex>

#include <cuda_runtime.h>

#include "../../include/fth_b200.h"

namespace {

constexpr size_t kStaticScratchBytes = size_t{4} << 20;  // FTH_B200_NOALLOC_SCRATCH_BYTES

}  // namespace

// In host code this name is only a handle for the runtime's symbol table, not a device address: the address is
// looked up per device below and travels to the kernels inside the descriptor.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kStaticScratchBytes];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_address[kMaxDevices] = {};

// Device address of the array on the current device; resolved on the first call per device.
int ScratchAddress(void** out) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return FTH_B200_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr) return FTH_B200_ERR_CUDA;
        g_scratch_address[device] = ptr;
    }
    *out = g_scratch_address[device];
    return FTH_B200_OK;
}

}  // namespace

extern "C" size_t fth_b200_noalloc_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int fth_b200_fp8_linear_noalloc(const fth_b200_fp8_linear_desc* desc, fth_b200_stream_t stream) {
    if (desc == nullptr) return FTH_B200_ERR_INVALID;
    fth_b200_fp8_linear_desc d = *desc;
    d.variant = FTH_B200_VARIANT_TCGEN05;  // the kernel family whose scratch this entry point replaces
    d.workspace = nullptr;
    d.workspace_bytes = 0;
    // how much scratch the request needs; 0 also covers invalid descriptors, which the call below reports
    const size_t need = fth_b200_fp8_linear_workspace_bytes(&d);
    if (need > kStaticScratchBytes) return FTH_B200_ERR_SCRATCH_LIMIT;
    void* scratch = nullptr;
    const int rc = ScratchAddress(&scratch);
    if (rc != FTH_B200_OK) return rc;
    d.workspace = scratch;
    d.workspace_bytes = kStaticScratchBytes;
    return fth_b200_fp8_linear(&d, stream);
}
