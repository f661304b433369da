// Weight-streaming GEMV / skinny GEMM for decode shapes (M <= 16): the HBM-bound half of the linear path.
//
// Every weight byte is read exactly once per block of up to 4 activation rows, with 16-byte coalesced
// streaming loads (ld.global.nc, no L1 allocation) and many loads in flight per thread.  Arithmetic stays
// on the CUDA cores: FP8 codes are decoded to FP32 and accumulated with FP32 FMAs, INT8 uses dp4a into
// int32 — both reproduce the reference's accumulation types exactly.
//
//  * weights [K,N] ("KN", FC / MatMul layout): a CTA owns a 256-column tile and one K chunk.  Thread
//    (column group, row lane) walks rows row_lane, row_lane+16, … of its chunk, keeping 16 columns x MB rows
//    of accumulators.  Row lanes are combined through shared memory; the S CTAs of a thread-block cluster
//    (one per K chunk) are then combined through distributed shared memory in rank order, so no global
//    scratch buffer and no atomics are needed.
//  * weights [N,K] ("NK", Gemm trans_b / lm-head layout): a warp owns R output columns, its lanes stride
//    along K 16 bytes at a time, and the partial dot products are combined with warp shuffles.
//
// The split of K (S chunks, 16 row lanes, 8 warps) depends on K alone, never on N or the grid, so a
// column shard of a weight produces bit-identical outputs to the same columns of the full weight.
#include <cooperative_groups.h>

#include "common.cuh"
#include "linear_internal.h"

namespace cg = cooperative_groups;

namespace fth {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kTileN = 256;              // columns per CTA (KN kernel)
constexpr int kColGroups = kTileN / 16;  // 16 threads across a tile row, 16 bytes each
constexpr int kRowLanes = kThreads / kColGroups;  // 16
constexpr int kSubK = 2048;              // activation rows staged in shared memory at a time (KN kernel)
constexpr int kPadK = 128;               // zero rows behind them: unrolled tail iterations multiply by zero
constexpr int kMaxSplit = 8;             // portable cluster size limit

template <int DTYPE>
struct Acc { using type = float; };
template <>
struct Acc<FTH_B200_INT8> { using type = int32_t; };

__host__ __device__ inline int SplitForK(int64_t k) {
    int64_t s = k / 128;
    if (s < 1) s = 1;
    if (s > kMaxSplit) s = kMaxSplit;
    // power of two so that cluster shapes stay regular
    int p = 1;
    while (p * 2 <= s) p *= 2;
    return p;
}

template <int DTYPE>
__device__ __forceinline__ void Decode16(const uint4& v, float (&out)[16]) {
    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 lo = DecodePair<DTYPE>(static_cast<uint16_t>(words[i] & 0xffffu));
        const float2 hi = DecodePair<DTYPE>(static_cast<uint16_t>(words[i] >> 16));
        out[4 * i + 0] = lo.x; out[4 * i + 1] = lo.y; out[4 * i + 2] = hi.x; out[4 * i + 3] = hi.y;
    }
}

// Transposes a 4x4 byte block held as four row words into four column words.
__device__ __forceinline__ void Transpose4x4(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t (&c)[4]) {
    const uint32_t t0 = __byte_perm(r0, r1, 0x5140);  // r0.b0 r1.b0 r0.b1 r1.b1
    const uint32_t t1 = __byte_perm(r2, r3, 0x5140);
    const uint32_t t2 = __byte_perm(r0, r1, 0x7362);  // r0.b2 r1.b2 r0.b3 r1.b3
    const uint32_t t3 = __byte_perm(r2, r3, 0x7362);
    c[0] = __byte_perm(t0, t1, 0x5410);
    c[1] = __byte_perm(t0, t1, 0x7632);
    c[2] = __byte_perm(t2, t3, 0x5410);
    c[3] = __byte_perm(t2, t3, 0x7632);
}

// ---------------------------------------------------------------------------------------------------
// KN kernel
// ---------------------------------------------------------------------------------------------------
template <int DTYPE, int MB>
__global__ void __launch_bounds__(kThreads) SkinnyKnKernel(LinearArgs args, Fp8Epilogue fe, Int8Epilogue ie, int split,
                                                           int64_t chunk) {
    using T = typename Acc<DTYPE>::type;
    constexpr bool kInt8 = DTYPE == FTH_B200_INT8;
    extern __shared__ __align__(16) uint8_t smem[];
    // layout: activations | cross-warp reduction | CTA partial | (int8) column sums, row sums
    constexpr int kActBytes = kInt8 ? MB * (kSubK + kPadK) : MB * (kSubK + kPadK) * 4;
    T* red = reinterpret_cast<T*>(smem + kActBytes);                 // [kWarps][MB][kTileN]
    T* partial = red + kWarps * MB * kTileN;                         // [MB][kTileN]
    int32_t* col_sum_s = reinterpret_cast<int32_t*>(partial + MB * kTileN);  // [kTileN]   (int8 only)
    int32_t* row_sum_s = col_sum_s + kTileN;                         // [MB]       (int8 only)

    const int tid = threadIdx.x;
    const int cgp = tid % kColGroups;
    const int row_lane = tid / kColGroups;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kTileN;
    const int64_t m0 = static_cast<int64_t>(blockIdx.z) * MB;
    const int rank = blockIdx.y;  // K chunk index == cluster rank
    const int64_t k_begin = rank * chunk;
    const int64_t k_end = (k_begin + chunk < args.k) ? k_begin + chunk : args.k;
    const int64_t col = n0 + cgp * 16;
    const bool col_ok = col < args.n;  // N is a multiple of 16, so a group is all-in or all-out
    const uint8_t* wbase = static_cast<const uint8_t*>(args.w) + col;

    T acc[MB][16];
    int32_t csum[16];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[m][j] = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) csum[j] = 0;
    const bool need_sums = kInt8 && (ie.a_zp != 0 || ie.w_zps != nullptr);
    if (kInt8 && tid < MB) row_sum_s[tid] = 0;

    for (int64_t sub = k_begin; sub < k_end; sub += kSubK) {
        const int rows = static_cast<int>((k_end - sub < kSubK) ? (k_end - sub) : kSubK);
        const int fill = rows + kPadK;  // staged rows plus the zero tail
        __syncthreads();  // previous sub-chunk fully consumed
        // ---- stage activations (zero padded by kPadK so tail rows multiply by zero) ----
        if constexpr (kInt8) {
            int8_t* a_s = reinterpret_cast<int8_t*>(smem);
            for (int idx = tid; idx < MB * fill; idx += kThreads) {
                const int m = idx / fill, r = idx % fill;
                int8_t v = 0;
                if (r < rows && m0 + m < args.m) {
                    v = LoadInt8Activation(args.a, (m0 + m) * args.k + sub + r, args.a_dtype, ie.a_scale, ie.a_zp);
                    if (need_sums) atomicAdd(&row_sum_s[m], static_cast<int32_t>(v));
                }
                a_s[m * (kSubK + kPadK) + r] = v;
            }
        } else {
            float* a_s = reinterpret_cast<float*>(smem);
            for (int idx = tid; idx < MB * fill; idx += kThreads) {
                const int m = idx / fill, r = idx % fill;
                float v = 0.0f;
                if (r < rows && m0 + m < args.m) v = LoadActivation<DTYPE>(args.a, (m0 + m) * args.k + sub + r, args.a_dtype, args.a_scale);
                a_s[m * (kSubK + kPadK) + r] = v;
            }
        }
        __syncthreads();

        if (col_ok) {
            if constexpr (kInt8) {
                const int32_t* a_w = reinterpret_cast<const int32_t*>(smem);  // 4 consecutive k per word
                const int quads = (rows + 3) / 4;
                for (int q = row_lane; q < quads; q += kRowLanes * 2) {
                    uint4 v[2][4];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int qq = q + u * kRowLanes;
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const int row = qq * 4 + r;
                            v[u][r] = (row < rows) ? LoadStream16(wbase + (sub + row) * args.n) : make_uint4(0, 0, 0, 0);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int qq = q + u * kRowLanes;
                        int32_t aw[MB];
#pragma unroll
                        for (int m = 0; m < MB; ++m) aw[m] = a_w[m * ((kSubK + kPadK) / 4) + qq];
                        const uint32_t* r0 = reinterpret_cast<const uint32_t*>(&v[u][0]);
                        const uint32_t* r1 = reinterpret_cast<const uint32_t*>(&v[u][1]);
                        const uint32_t* r2 = reinterpret_cast<const uint32_t*>(&v[u][2]);
                        const uint32_t* r3 = reinterpret_cast<const uint32_t*>(&v[u][3]);
#pragma unroll
                        for (int c4 = 0; c4 < 4; ++c4) {
                            uint32_t cw[4];
                            Transpose4x4(r0[c4], r1[c4], r2[c4], r3[c4], cw);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
#pragma unroll
                                for (int m = 0; m < MB; ++m) acc[m][c4 * 4 + j] = __dp4a(static_cast<int32_t>(cw[j]), aw[m], acc[m][c4 * 4 + j]);
                                if (need_sums) csum[c4 * 4 + j] = __dp4a(static_cast<int32_t>(cw[j]), 0x01010101, csum[c4 * 4 + j]);
                            }
                        }
                    }
                }
            } else {
                const float* a_s = reinterpret_cast<const float*>(smem);
                constexpr int kUnroll = MB <= 2 ? 8 : 4;
                for (int r = row_lane; r < rows; r += kRowLanes * kUnroll) {
                    uint4 v[kUnroll];
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const int row = r + u * kRowLanes;
                        v[u] = (row < rows) ? LoadStream16(wbase + (sub + row) * args.n) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const int row = r + u * kRowLanes;  // < kSubK + kPadK by construction
                        float wv[16];
                        Decode16<DTYPE>(v[u], wv);
#pragma unroll
                        for (int m = 0; m < MB; ++m) {
                            const float av = a_s[m * (kSubK + kPadK) + row];
#pragma unroll
                            for (int j = 0; j < 16; ++j) acc[m][j] = fmaf(av, wv[j], acc[m][j]);
                        }
                    }
                }
            }
        }
    }

    // ---- combine the two row lanes of each warp, then the 8 warps, in a fixed order ----
    const int warp = tid / 32, lane = tid % 32;
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const T other = __shfl_xor_sync(0xffffffffu, acc[m][j], 16);
            acc[m][j] = (lane < 16) ? acc[m][j] + other : other + acc[m][j];
        }
    if (need_sums) {
#pragma unroll
        for (int j = 0; j < 16; ++j) csum[j] += __shfl_xor_sync(0xffffffffu, csum[j], 16);
    }
    if (lane < 16) {
#pragma unroll
        for (int m = 0; m < MB; ++m)
#pragma unroll
            for (int j = 0; j < 16; ++j) red[(warp * MB + m) * kTileN + lane * 16 + j] = acc[m][j];
    }
    __syncthreads();
    for (int idx = tid; idx < MB * kTileN; idx += kThreads) {
        const int m = idx / kTileN, c = idx % kTileN;
        T sum = red[(0 * MB + m) * kTileN + c];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) sum += red[(w * MB + m) * kTileN + c];
        partial[idx] = sum;
    }
    if (need_sums) {
        __syncthreads();
        if (lane < 16) {
#pragma unroll
            for (int j = 0; j < 16; ++j) reinterpret_cast<int32_t*>(red)[warp * kTileN + lane * 16 + j] = csum[j];
        }
        __syncthreads();
        if (tid < kTileN) {
            int32_t s = 0;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += reinterpret_cast<int32_t*>(red)[w * kTileN + tid];
            col_sum_s[tid] = s;
        }
    }

    // ---- combine the K chunks (cluster ranks) through distributed shared memory and write out ----
    if (split > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const int cols_per_rank = kTileN / split;
        for (int idx = tid; idx < MB * cols_per_rank; idx += kThreads) {
            const int m = idx / cols_per_rank, c = rank * cols_per_rank + idx % cols_per_rank;
            if (m0 + m >= args.m || n0 + c >= args.n) continue;
            T sum = 0;
            int32_t cs = 0, rs = 0;
            for (int r = 0; r < split; ++r) {
                const T* peer = cluster.map_shared_rank(partial, r);
                sum += peer[m * kTileN + c];
                if (need_sums) {
                    cs += cluster.map_shared_rank(col_sum_s, r)[c];
                    rs += cluster.map_shared_rank(row_sum_s, r)[m];
                }
            }
            if constexpr (kInt8) StoreInt8Result(ie, m0 + m, n0 + c, sum, rs, cs);
            else StoreFp8Result<DTYPE>(fe, m0 + m, n0 + c, sum);
        }
        cluster.sync();  // peers may still be reading this CTA's shared memory
    } else {
        __syncthreads();
        for (int idx = tid; idx < MB * kTileN; idx += kThreads) {
            const int m = idx / kTileN, c = idx % kTileN;
            if (m0 + m >= args.m || n0 + c >= args.n) continue;
            if constexpr (kInt8) StoreInt8Result(ie, m0 + m, n0 + c, partial[idx], need_sums ? row_sum_s[m] : 0, need_sums ? col_sum_s[c] : 0);
            else StoreFp8Result<DTYPE>(fe, m0 + m, n0 + c, partial[idx]);
        }
    }
}

template <int DTYPE, int MB>
constexpr size_t KnSmemBytes() {
    constexpr bool kInt8 = DTYPE == FTH_B200_INT8;
    return (kInt8 ? MB * (kSubK + kPadK) : MB * (kSubK + kPadK) * 4) + (kWarps * MB * kTileN + MB * kTileN) * 4 +
           (kTileN + MB + 4) * 4;
}

template <int DTYPE, int MB>
int LaunchKn(const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    const int split = SplitForK(args.k);
    // chunk: rows per cluster rank, a multiple of 64 so INT8 quads and row lanes never straddle chunks
    int64_t chunk = (args.k + split - 1) / split;
    chunk = (chunk + 63) / 64 * 64;
    const size_t smem = KnSmemBytes<DTYPE, MB>();
    auto kernel = SkinnyKnKernel<DTYPE, MB>;
    if (EnsureDynamicSmem(reinterpret_cast<const void*>(kernel), smem) != FTH_B200_OK) return FTH_B200_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((args.n + kTileN - 1) / kTileN), static_cast<unsigned>(split),
                       static_cast<unsigned>((args.m + MB - 1) / MB));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = static_cast<unsigned>(split);
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, args, fe, ie, split, chunk) != cudaSuccess) return FTH_B200_ERR_CUDA;
    NoteLaunch("skinny");
    return CheckLaunch();
}

// ---------------------------------------------------------------------------------------------------
// NK kernel
// ---------------------------------------------------------------------------------------------------
template <int DTYPE, int MB, int R>
__global__ void __launch_bounds__(kThreads) SkinnyNkKernel(LinearArgs args, Fp8Epilogue fe, Int8Epilogue ie) {
    constexpr bool kInt8 = DTYPE == FTH_B200_INT8;
    using T = typename Acc<DTYPE>::type;
    extern __shared__ __align__(16) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * MB;
    const int64_t n_base = (static_cast<int64_t>(blockIdx.x) * kWarps + warp) * R;
    const int64_t k = args.k;  // multiple of 16

    if constexpr (kInt8) {
        int8_t* a_s = reinterpret_cast<int8_t*>(smem);
        for (int64_t idx = tid; idx < MB * k; idx += kThreads) {
            const int64_t m = idx / k, kk = idx % k;
            a_s[idx] = (m0 + m < args.m) ? LoadInt8Activation(args.a, (m0 + m) * k + kk, args.a_dtype, ie.a_scale, ie.a_zp) : int8_t(0);
        }
    } else {
        float* a_s = reinterpret_cast<float*>(smem);
        for (int64_t idx = tid; idx < MB * k; idx += kThreads) {
            const int64_t m = idx / k, kk = idx % k;
            a_s[idx] = (m0 + m < args.m) ? LoadActivation<DTYPE>(args.a, (m0 + m) * k + kk, args.a_dtype, args.a_scale) : 0.0f;
        }
    }
    __syncthreads();
    if (n_base >= args.n) return;

    T acc[R][MB];
    int32_t csum[R], rsum[MB];
#pragma unroll
    for (int r = 0; r < R; ++r) { csum[r] = 0;
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[r][m] = 0; }
#pragma unroll
    for (int m = 0; m < MB; ++m) rsum[m] = 0;
    const bool need_sums = kInt8 && (ie.a_zp != 0 || ie.w_zps != nullptr);
    const uint8_t* wbase = static_cast<const uint8_t*>(args.w) + n_base * k;

    constexpr int kU = 2;
    for (int64_t kk0 = static_cast<int64_t>(lane) * 16; kk0 < k; kk0 += 512 * kU) {
        uint4 v[kU][R];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int64_t kk = kk0 + u * 512;
#pragma unroll
            for (int r = 0; r < R; ++r)
                v[u][r] = (kk < k && n_base + r < args.n) ? LoadStream16(wbase + r * k + kk) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int64_t kk = kk0 + u * 512;
            if (kk >= k) break;
            if constexpr (kInt8) {
                const int8_t* a_s = reinterpret_cast<const int8_t*>(smem);
                uint4 av[MB];
#pragma unroll
                for (int m = 0; m < MB; ++m) av[m] = *reinterpret_cast<const uint4*>(a_s + m * k + kk);
                if (need_sums) {
#pragma unroll
                    for (int m = 0; m < MB; ++m) {
                        const int32_t* aw = reinterpret_cast<const int32_t*>(&av[m]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) rsum[m] = __dp4a(aw[i], 0x01010101, rsum[m]);
                    }
                }
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int32_t* ww = reinterpret_cast<const int32_t*>(&v[u][r]);
#pragma unroll
                    for (int m = 0; m < MB; ++m) {
                        const int32_t* aw = reinterpret_cast<const int32_t*>(&av[m]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[r][m] = __dp4a(ww[i], aw[i], acc[r][m]);
                    }
                    if (need_sums) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) csum[r] = __dp4a(ww[i], 0x01010101, csum[r]);
                    }
                }
            } else {
                const float* a_s = reinterpret_cast<const float*>(smem);
                float wv[R][16];
#pragma unroll
                for (int r = 0; r < R; ++r) Decode16<DTYPE>(v[u][r], wv[r]);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    float av[16];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 t = *reinterpret_cast<const float4*>(a_s + m * k + kk + q * 4);
                        av[4 * q] = t.x; av[4 * q + 1] = t.y; av[4 * q + 2] = t.z; av[4 * q + 3] = t.w;
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[r][m] = fmaf(av[j], wv[r][j], acc[r][m]);
                }
            }
        }
    }

    // warp-shuffle reduction of the K split across lanes (xor tree: the same order on every lane)
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int m = 0; m < MB; ++m) acc[r][m] += __shfl_xor_sync(0xffffffffu, acc[r][m], off);
            if (need_sums) csum[r] += __shfl_xor_sync(0xffffffffu, csum[r], off);
        }
        if (need_sums) {
#pragma unroll
            for (int m = 0; m < MB; ++m) rsum[m] += __shfl_xor_sync(0xffffffffu, rsum[m], off);
        }
    }
    // lanes 0 .. R*MB-1 each write one output
    if (lane < R * MB) {
        const int r = lane / MB, m = lane % MB;
        T value = 0;
        int32_t cs = 0, rs = 0;
#pragma unroll
        for (int rr = 0; rr < R; ++rr)
#pragma unroll
            for (int mm = 0; mm < MB; ++mm)
                if (rr == r && mm == m) { value = acc[rr][mm]; cs = csum[rr]; rs = rsum[mm]; }
        if (n_base + r < args.n && m0 + m < args.m) {
            if constexpr (kInt8) StoreInt8Result(ie, m0 + m, n_base + r, value, rs, cs);
            else StoreFp8Result<DTYPE>(fe, m0 + m, n_base + r, value);
        }
    }
}

template <int DTYPE, int MB, int R>
int LaunchNk(const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    constexpr bool kInt8 = DTYPE == FTH_B200_INT8;
    const size_t smem = static_cast<size_t>(MB) * args.k * (kInt8 ? 1 : 4);
    auto kernel = SkinnyNkKernel<DTYPE, MB, R>;
    if (EnsureDynamicSmem(reinterpret_cast<const void*>(kernel), smem) != FTH_B200_OK) return FTH_B200_ERR_CUDA;
    const dim3 grid(static_cast<unsigned>((args.n + kWarps * R - 1) / (kWarps * R)), static_cast<unsigned>((args.m + MB - 1) / MB));
    kernel<<<grid, kThreads, smem, stream>>>(args, fe, ie);
    NoteLaunch("skinny");
    return CheckLaunch();
}

constexpr size_t kNkSmemLimit = 200 * 1024;

template <int DTYPE>
int LaunchSkinnyTyped(const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    const int mb = args.m >= 4 ? 4 : (args.m >= 2 ? 2 : 1);
    if (args.trans_b) {
        switch (mb) {
            case 1: return LaunchNk<DTYPE, 1, 4>(args, fe, ie, stream);
            case 2: return LaunchNk<DTYPE, 2, 4>(args, fe, ie, stream);
            default: return LaunchNk<DTYPE, 4, 2>(args, fe, ie, stream);
        }
    }
    switch (mb) {
        case 1: return LaunchKn<DTYPE, 1>(args, fe, ie, stream);
        case 2: return LaunchKn<DTYPE, 2>(args, fe, ie, stream);
        default: return LaunchKn<DTYPE, 4>(args, fe, ie, stream);
    }
}

}  // namespace

bool SkinnySupported(int dtype, const LinearArgs& args) {
    if (args.m < 1 || args.m > kSkinnyMaxM) return false;
    if (reinterpret_cast<uintptr_t>(args.w) % 16 != 0) return false;
    if (args.trans_b) {
        if (args.k % 16 != 0) return false;
        const size_t mb = args.m >= 4 ? 4 : (args.m >= 2 ? 2 : 1);
        const size_t smem = mb * static_cast<size_t>(args.k) * (dtype == FTH_B200_INT8 ? 1 : 4);
        return smem <= kNkSmemLimit;
    }
    return args.n % 16 == 0 && (args.n + kTileN - 1) / kTileN <= 0x7fffffff;
}

int LaunchLinearSkinny(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie,
                       cudaStream_t stream) {
    if (!SkinnySupported(dtype, args)) return FTH_B200_ERR_UNSUPPORTED;
    switch (dtype) {
        case FTH_B200_FP8E4M3: return LaunchSkinnyTyped<FTH_B200_FP8E4M3>(args, fe, ie, stream);
        case FTH_B200_FP8E5M2: return LaunchSkinnyTyped<FTH_B200_FP8E5M2>(args, fe, ie, stream);
        case FTH_B200_INT8: return LaunchSkinnyTyped<FTH_B200_INT8>(args, fe, ie, stream);
        default: return FTH_B200_ERR_INVALID;
    }
}

}  // namespace fth
