// Host side of tma.cuh: tensor-map encoding through the driver entry point (no link-time dependency on
// libcuda, so the library loads on machines without a driver) and the device status word.
#include <mutex>

#include <cudaTypedefs.h>

#include "common.cuh"
#include "tma.cuh"

namespace fth {

namespace {

__device__ int g_device_status = 0;

PFN_cuTensorMapEncodeTiled_v12000 EncodeFn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
        }
    });
    return fn;
}

CUtensorMapSwizzle ToDriver(TmaSwizzle s) {
    switch (s) {
        case TmaSwizzle::k32B: return CU_TENSOR_MAP_SWIZZLE_32B;
        case TmaSwizzle::k64B: return CU_TENSOR_MAP_SWIZZLE_64B;
        case TmaSwizzle::k128B: return CU_TENSOR_MAP_SWIZZLE_128B;
        default: return CU_TENSOR_MAP_SWIZZLE_NONE;
    }
}

}  // namespace

int* DeviceStatusPtr() {
    // One address per device; looked up on first use while that device is current.
    static int* ptrs[64] = {};
    static std::mutex mutex;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mutex);
    if (ptrs[device] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        ptrs[device] = static_cast<int*>(p);
    }
    return ptrs[device];
}

bool MakeTensorMap2D(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t row_pitch_bytes,
                     uint32_t box_cols, uint32_t box_rows, TmaSwizzle swizzle) {
    auto fn = EncodeFn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {row_pitch_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, ToDriver(swizzle), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool MakeTensorMap4D(CUtensorMap* map, const void* base, const uint64_t dims_[4], const uint64_t strides_bytes[3],
                     const uint32_t box_[4], TmaSwizzle swizzle) {
    auto fn = EncodeFn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[4] = {dims_[0], dims_[1], dims_[2], dims_[3]};
    const cuuint64_t strides[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
    const cuuint32_t box[4] = {box_[0], box_[1], box_[2], box_[3]};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, ToDriver(swizzle), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace fth

// Reads and clears the device status word (synchronises the device).  0 = no bounded wait ever gave up;
// otherwise (site << 16) | detail of the first one that did.
extern "C" int fth_b200_device_status(void) {
    int value = 0;
    int* ptr = fth::DeviceStatusPtr();
    if (ptr == nullptr || cudaDeviceSynchronize() != cudaSuccess) return FTH_B200_ERR_CUDA;
    if (cudaMemcpy(&value, ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return FTH_B200_ERR_CUDA;
    if (value != 0) cudaMemset(ptr, 0, sizeof(int));
    return value;
}
