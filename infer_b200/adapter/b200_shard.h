// Column-sharded projections over several GPUs driven by ONE process — Feather's own layout for more than one device:
// one CudaExecutionContext (and ExecutionSession) per GPU, each created while that GPU is current
// (src/kernel/cuda/runtime.cu:318-321, 453-472).  The reference has no multi-device code; this is what an embedding
// host adds next to its per-GPU sessions.
//
// A ShardGroup owns what the ranks share: per GPU two gathered [M, N] output buffers (used by step parity) and the
// flag array of the step signalling that the linear kernels do themselves, every GPU mapped into every other
// (cudaDeviceEnablePeerAccess: one process, so no IPC handles).  While a ShardBindingScope is alive on a thread, a B200
// FP8 / INT8 linear candidate whose node is this rank's column slice stores its outputs into all ranks' buffers from
// its own epilogue and publishes the step (fth_b200.h: gather_out, gather_world, gather_flags); the node's own output
// tensor still receives the rank's block.  No collective library is involved.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <utility>
#include <vector>

#include "fth_b200.h"

namespace feather {
namespace kernel {
namespace b200 {

class ShardGroup {
   public:
    // devices: the CUDA ordinals of the ranks, in rank order (2 .. 8 of them).  Returns null when a buffer cannot be
    // allocated or a pair of GPUs cannot reach each other.
    static std::shared_ptr<ShardGroup> Create(const std::vector<int>& devices, int64_t m, int64_t n, int64_t elem_bytes = 1) {
        if (devices.size() < 2 || devices.size() > 8 || m <= 0 || n <= 0 || elem_bytes <= 0) return nullptr;
        std::shared_ptr<ShardGroup> g(new ShardGroup());
        g->devices_ = devices;
        g->m_ = m; g->n_ = n; g->elem_ = elem_bytes;
        g->block_ = (static_cast<size_t>(m * n * elem_bytes) + 255) / 256 * 256;
        int previous = 0;
        if (cudaGetDevice(&previous) != cudaSuccess) return nullptr;
        bool ok = true;
        for (size_t r = 0; r < devices.size() && ok; ++r) {
            ok = cudaSetDevice(devices[r]) == cudaSuccess;
            for (size_t q = 0; q < devices.size() && ok; ++q) {
                if (q == r) continue;
                int can = 0;
                ok = cudaDeviceCanAccessPeer(&can, devices[r], devices[q]) == cudaSuccess && can != 0;
                if (ok) {
                    const cudaError_t e = cudaDeviceEnablePeerAccess(devices[q], 0);
                    if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
                    else ok = e == cudaSuccess;
                }
            }
            void* base = nullptr;
            ok = ok && cudaMalloc(&base, 2 * g->block_ + 256) == cudaSuccess && cudaMemset(base, 0, 2 * g->block_ + 256) == cudaSuccess &&
                 cudaDeviceSynchronize() == cudaSuccess;
            g->base_.push_back(static_cast<uint8_t*>(base));
        }
        (void)cudaSetDevice(previous);
        return ok ? g : nullptr;
    }

    ~ShardGroup() {
        int previous = 0;
        (void)cudaGetDevice(&previous);
        for (size_t r = 0; r < base_.size(); ++r) {
            if (base_[r] != nullptr && cudaSetDevice(devices_[r]) == cudaSuccess) (void)cudaFree(base_[r]);
        }
        (void)cudaSetDevice(previous);
    }

    int world() const { return static_cast<int>(devices_.size()); }
    int device(int rank) const { return devices_[static_cast<size_t>(rank)]; }
    int64_t m() const { return m_; }
    int64_t n() const { return n_; }
    int64_t elem_bytes() const { return elem_; }

    // Columns [n0, n1) of `rank`: equal runs of 128-column blocks, the remainder spread over the first ranks.
    std::pair<int64_t, int64_t> Columns(int rank) const {
        const int64_t blocks = (n_ + 127) / 128, base = blocks / world(), extra = blocks % world();
        const int64_t b0 = rank * base + (rank < extra ? rank : extra);
        const int64_t b1 = b0 + base + (rank < extra ? 1 : 0);
        return {b0 * 128 < n_ ? b0 * 128 : n_, b1 * 128 < n_ ? b1 * 128 : n_};
    }

    // Rank r's gathered [M, N] buffer for steps of this parity (an address every rank's GPU can use).
    uint8_t* Buffer(int rank, int parity) const { return base_[static_cast<size_t>(rank)] + static_cast<size_t>(parity) * block_; }
    void* Flags(int rank) const { return base_[static_cast<size_t>(rank)] + 2 * block_; }

    // One call per step, before any rank launches it: the buffers of the new step's parity are the ones nobody reads
    // any more (a rank cannot pass step s before every rank has published s - 1).
    void NextStep() { ++epoch_; }
    int Parity() const { return static_cast<int>(epoch_ & 1); }

    // Points a linear descriptor (FP8 or INT8: the gather fields have the same names) at this step's buffers: the
    // rank's own block in its own buffer as `out`, the same block in every other rank's, and the flag arrays.
    template <typename Desc>
    void Point(Desc* d, int rank) const {
        const int64_t offset = Columns(rank).first * elem_;
        d->out = Buffer(rank, Parity()) + offset;
        d->ldo = n_;
        int peers = 0;
        for (int r = 0; r < world(); ++r) {
            if (r != rank) d->gather_out[peers++] = Buffer(r, Parity()) + offset;
            d->gather_flags[r] = Flags(r);
        }
        d->gather_peers = peers;
        d->gather_world = world();
        d->gather_rank = rank;
        d->gather_multicast_out = nullptr;
    }

    // Consumer side, on `stream` of rank's GPU: returns once every rank has published the step this rank published
    // last (bounded on the device; read fth_b200_device_status() before trusting the buffer).
    int Wait(int rank, cudaStream_t stream) const {
        void* flags[8] = {};
        for (int r = 0; r < world(); ++r) flags[r] = Flags(r);
        return fth_b200_gather_wait(flags, world(), rank, stream);
    }

   private:
    ShardGroup() = default;
    std::vector<int> devices_;
    std::vector<uint8_t*> base_;
    int64_t m_{0}, n_{0}, elem_{1};
    size_t block_{0};
    uint64_t epoch_{0};
};

// The rank a thread is driving.  Candidates consult Current() in compute().
class ShardBindingScope {
   public:
    ShardBindingScope(std::shared_ptr<ShardGroup> group, int rank) : group_(std::move(group)), rank_(rank), previous_(Slot()) { Slot() = this; }
    ~ShardBindingScope() { Slot() = previous_; }
    ShardBindingScope(const ShardBindingScope&) = delete;
    ShardBindingScope& operator=(const ShardBindingScope&) = delete;

    static const ShardBindingScope* Current() { return Slot(); }
    const ShardGroup& group() const { return *group_; }
    int rank() const { return rank_; }
    // True when an [m, n] node output with this element size is this rank's column block of the group's projection.
    bool Matches(int64_t m, int64_t n, int64_t elem_bytes) const {
        const auto cols = group_->Columns(rank_);
        return m == group_->m() && n == cols.second - cols.first && elem_bytes == group_->elem_bytes();
    }

   private:
    static const ShardBindingScope*& Slot() {
        static thread_local const ShardBindingScope* current = nullptr;
        return current;
    }
    std::shared_ptr<ShardGroup> group_;
    int rank_;
    const ShardBindingScope* previous_;
};

}  // namespace b200
}  // namespace kernel
}  // namespace feather
