// Multi-GPU plumbing for column-sharded projections: peer-mapped output buffers (CUDA IPC), the block copy used by
// kernels that do not write the peer replicas themselves, and the signal / wait step that ends a gather.
//
// A gather works without a collective library: every rank's linear kernel stores its columns into all ranks'
// output buffers (plain peer stores over NVLink), then each rank raises a flag in every rank's flag array and
// waits — bounded — for everybody's flag.  Flags carry the caller's step number, so nothing is ever reset.
#include <string.h>

#include "common.cuh"
#include "linear_internal.h"
#include "linear_tc.cuh"
#include "tma.cuh"

namespace fth {
namespace {

__global__ void __launch_bounds__(256) PeerCopyKernel(const uint8_t* __restrict__ out, int64_t rows, int64_t row_bytes, int64_t pitch_bytes,
                                                      PeerOut peers) {
    const int64_t total = rows * row_bytes;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t offset = (i / row_bytes) * pitch_bytes + i % row_bytes;
        const uint8_t v = out[offset];
        for (int r = 0; r < peers.count; ++r) const_cast<uint8_t*>(out)[offset + peers.delta[r]] = v;
    }
}

struct FlagPtrs { uint32_t* rank_flags[kMaxPeers + 1]; };

// Thread r tells rank r "rank `self` has finished step `epoch`" and then waits until rank r has said the same here.
// The kernels whose stores this publishes ran earlier on the same stream, so they are complete; the release at
// system scope orders them before the flag for a peer that acquires it.
__global__ void GatherSyncKernel(FlagPtrs flags, int world, int self, uint32_t epoch, int* status) {
    // Launched with programmatic stream serialization: the next kernel in the stream (the next step's linear, which
    // writes the other pair of buffers) may set up and fetch static weights while this one waits for the peers; this
    // kernel itself starts only after the kernels whose stores it publishes have completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ uint32_t step;
    if (threadIdx.x == 0) {
        // epoch 0: the step number lives on the device (slot [world] of this rank's own flag array) and grows by one
        // per call, so the same launch can be replayed from a CUDA graph
        uint32_t e = epoch;
        if (e == 0) {
            e = flags.rank_flags[self][world] + 1;
            if (e == 0) e = 1;
            flags.rank_flags[self][world] = e;
        }
        step = e;
    }
    __syncthreads();
    const int r = threadIdx.x;
    if (r >= world) return;
    const uint32_t e = step;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.rank_flags[r] + self), "r"(e) : "memory");
    const uint32_t* mine = flags.rank_flags[self] + r;
    const uint64_t start = GlobalTimerNs();
    for (;;) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if (static_cast<int32_t>(seen - e) >= 0) break;  // steps only grow (wrap-around safe)
        if (GlobalTimerNs() - start > kWaitBudgetNs) { ReportTimeout(status, 40, r); break; }
        __nanosleep(100);
    }
}

// The halves of a folded gather step as kernels of their own (for kernel families without the in-kernel path), and the
// consumer-side wait.  mode 1: count this step and publish it; otherwise wait until every rank has published the step
// this rank's counter stands at.
__global__ void GatherStepKernel(GatherSignal g, int mode, int* status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = threadIdx.x;
    if (mode == 1) {
        if (r == 0) tc::GatherArriveAndPublish(g, tc::GatherStep(g), 1u);
        return;
    }
    if (r >= g.world) return;
    // Both waits are for the value of this rank's step counter: in front of a step's kernel that is the previous step;
    // behind the kernel (which advanced the counter) it is the step itself.
    tc::GatherWaitPrevious(g, r, tc::GatherStep(g), status);
}

__global__ void ArgmaxFinalizeKernel(unsigned long long* keys, int64_t m, long long none_value) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= m) return;
    const unsigned long long key = keys[i];
    reinterpret_cast<long long*>(keys)[i] = key == 0 ? none_value : static_cast<long long>(0xffffffffu - static_cast<uint32_t>(key & 0xffffffffu));
}

}  // namespace

int LaunchArgmaxFinalize(unsigned long long* keys, int64_t m, int64_t none_value, cudaStream_t stream) {
    ArgmaxFinalizeKernel<<<static_cast<unsigned>((m + 127) / 128), 128, 0, stream>>>(keys, m, static_cast<long long>(none_value));
    NoteLaunch("argmax_finalize");
    return CheckLaunch();
}

static int LaunchGatherStep(const GatherSignal& signal, int mode, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, GatherStepKernel, signal, mode, DeviceStatusPtr()) != cudaSuccess) return FTH_B200_ERR_CUDA;
    NoteLaunch(mode == 1 ? "gather_publish" : "gather_wait");
    return CheckLaunch();
}
int LaunchGatherWaitPrevious(const GatherSignal& signal, cudaStream_t stream) { return LaunchGatherStep(signal, 0, stream); }
int LaunchGatherPublish(const GatherSignal& signal, cudaStream_t stream) { return LaunchGatherStep(signal, 1, stream); }

int LaunchPeerCopy(const void* out, int64_t m, int64_t n, int64_t ldo, int elem_bytes, const PeerOut& peers, cudaStream_t stream) {
    if (peers.count <= 0 || m <= 0 || n <= 0) return FTH_B200_OK;
    const int64_t total = m * n * elem_bytes;
    const int64_t blocks = (total + 255) / 256;
    PeerCopyKernel<<<static_cast<unsigned>(blocks < 1184 ? blocks : 1184), 256, 0, stream>>>(static_cast<const uint8_t*>(out), m, n * elem_bytes,
                                                                                           ldo * elem_bytes, peers);
    NoteLaunch("peer_copy");
    return CheckLaunch();
}

}  // namespace fth

using namespace fth;

extern "C" int fth_b200_peer_buffer_create(size_t bytes, void** ptr, unsigned char* handle) {
    if (ptr == nullptr || handle == nullptr || bytes == 0) return FTH_B200_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == FTH_B200_PEER_HANDLE_BYTES, "IPC handle size");
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return FTH_B200_ERR_CUDA;
    cudaIpcMemHandle_t h;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess || cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaFree(p);
        return FTH_B200_ERR_CUDA;
    }
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return FTH_B200_OK;
}

extern "C" int fth_b200_peer_buffer_open(const unsigned char* handle, void** ptr) {
    if (ptr == nullptr || handle == nullptr) return FTH_B200_ERR_INVALID;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? FTH_B200_OK : FTH_B200_ERR_CUDA;
}

extern "C" int fth_b200_peer_buffer_close(void* ptr) {
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? FTH_B200_OK : FTH_B200_ERR_CUDA;
}

extern "C" int fth_b200_peer_buffer_destroy(void* ptr) { return cudaFree(ptr) == cudaSuccess ? FTH_B200_OK : FTH_B200_ERR_CUDA; }

extern "C" int fth_b200_gather_sync(void* const* rank_flags, int32_t world, int32_t rank, uint32_t epoch, fth_b200_stream_t stream_) {
    ClearStaleError();
    if (rank_flags == nullptr || world < 1 || world > kMaxPeers + 1 || rank < 0 || rank >= world) return FTH_B200_ERR_INVALID;
    FlagPtrs flags = {};
    for (int r = 0; r < world; ++r) {
        if (rank_flags[r] == nullptr) return FTH_B200_ERR_INVALID;
        flags.rank_flags[r] = static_cast<uint32_t*>(rank_flags[r]);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = static_cast<cudaStream_t>(stream_);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int world_arg = world, rank_arg = rank;
    if (cudaLaunchKernelEx(&cfg, GatherSyncKernel, flags, world_arg, rank_arg, epoch, DeviceStatusPtr()) != cudaSuccess) return FTH_B200_ERR_CUDA;
    NoteLaunch("gather_sync");
    return CheckLaunch();
}

extern "C" int fth_b200_gather_wait(void* const* rank_flags, int32_t world, int32_t rank, fth_b200_stream_t stream_) {
    ClearStaleError();
    if (rank_flags == nullptr || world < 1 || world > kMaxPeers + 1 || rank < 0 || rank >= world) return FTH_B200_ERR_INVALID;
    GatherSignal signal = {};
    for (int r = 0; r < world; ++r) {
        if (rank_flags[r] == nullptr) return FTH_B200_ERR_INVALID;
        signal.flags[r] = static_cast<uint32_t*>(rank_flags[r]);
    }
    signal.world = world;
    signal.rank = rank;
    return LaunchGatherStep(signal, 2, static_cast<cudaStream_t>(stream_));
}
