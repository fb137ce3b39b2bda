// Peer-memory halves of the two matmul + collective operators the reference ships:
//   npu_mm_reduce_scatter_base: the matmul's epilogue has stored every rank's fp32 partial rows into
//     the OWNER's region (slot [source rank][rows_per][N] of the first half, see dense_gemm.cuh);
//     peer_reduce_scatter_kernel adds the W slots of this rank's rows in rank order, adds the bias,
//     rounds once and writes the [rows_per, N] result: the golden of
//     test/test_custom_ops/test_mm_reduce_scatter_base.py:69-81 (fp32 matmul per rank, summed, cast,
//     sliced) operation by operation.
//   npu_all_gather_base_mm: every rank has copied its x1 shard into its own region;
//     peer_all_gather_kernel pulls the other ranks' shards over NVLink into the gathered [W * M, K]
//     matrix that the matmul then consumes (test_all_gather_base_mm.py:72-78).
// Both kernels end with a second flag round ("I have finished reading"), after which a rank may
// overwrite what its peers read - the next call's pushes or copies - without further synchronisation.
// Flags live in the regions' flag area behind those of the allreduce kernel, carry the communicator's
// call epoch (which only grows) and are never reset; every wait is bounded like the allreduce's.
#pragma once

#include "peer_all_reduce.cuh"

namespace qmm {

constexpr size_t kPeerSgFlagOffset = 32 * 1024;  // reduce-scatter: ready [W] at +0, done [W] at +64, counter at +128
constexpr size_t kPeerAgFlagOffset = kPeerSgFlagOffset + 256;  // all-gather: the same three, 256 bytes further

struct PeerSgParams {
    uint8_t *base[kPeerMaxRanks];
    int world, rank;
    uint32_t epoch;
    uint32_t done_target;   // value of this rank's CTA counter once every CTA of this launch has finished
    size_t flag_off;        // kPeerSgFlagOffset or kPeerAgFlagOffset
    size_t area_off;        // the first half of a region
    int64_t rows, cols;     // reduce-scatter: rows_per x N (fp32 slots); all-gather: M x K of the 16-bit shard
    const void *bias;       // reduce-scatter only
    void *out;              // reduce-scatter: [rows, cols] 16-bit; all-gather: gathered [W * rows, cols]
    int64_t ld_out;
    uint32_t *status;
    uint32_t status_at_launch;
};

// "ready" round at the start (block 0 announces, every CTA waits), shared by both kernels
__device__ __forceinline__ bool peer_sg_ready_round(const PeerSgParams &p, int *s_ok) {
    uint32_t *my_flags = reinterpret_cast<uint32_t *>(p.base[p.rank] + p.flag_off);
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t *>(p.base[threadIdx.x] + p.flag_off) + p.rank, p.epoch);
    }
    if (threadIdx.x == 0) *s_ok = 1;
    __syncthreads();
    if (threadIdx.x < p.world && !peer_wait_flag(my_flags + threadIdx.x, p.epoch, p.status, p.status_at_launch, 0x11))
        *s_ok = 0;
    __syncthreads();
    return *s_ok != 0;
}

// "done" round at the end: the CTA that finishes last tells every peer, then waits for every peer
__device__ __forceinline__ void peer_sg_done_round(const PeerSgParams &p, int *s_last) {
    uint32_t *my_flags = reinterpret_cast<uint32_t *>(p.base[p.rank] + p.flag_off);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t old = atomicAdd(my_flags + 32, 1u);
        *s_last = (old + 1 == p.done_target) ? 1 : 0;
    }
    __syncthreads();
    if (*s_last == 0) return;
    if (threadIdx.x < p.world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t *>(p.base[threadIdx.x] + p.flag_off) + 16 + p.rank, p.epoch);
        (void)peer_wait_flag(my_flags + 16 + threadIdx.x, p.epoch, p.status, p.status_at_launch, 0x12);
    }
}

template <typename T>
__global__ void __launch_bounds__(kPeerThreads, 1) peer_reduce_scatter_kernel(PeerSgParams p) {
    __shared__ int s_ok, s_last;
    if (!peer_sg_ready_round(p, &s_ok)) return;
    const int W = p.world;
    const T *bias = static_cast<const T *>(p.bias);
    const float *slots = reinterpret_cast<const float *>(p.base[p.rank] + p.area_off);
    const int64_t slot_elems = p.rows * p.cols;
    T *out = static_cast<T *>(p.out);
    if ((p.cols & 3) == 0 && (p.ld_out & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 7) == 0) {
        const int64_t vec_per_row = p.cols / 4;
        const int64_t nvec = p.rows * vec_per_row;
        for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
             v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < W; ++r) {  // rank order: the sum does not depend on timing
                const float4 x = __ldcg(reinterpret_cast<const float4 *>(slots + r * slot_elems) + v);
                acc.x += x.x;
                acc.y += x.y;
                acc.z += x.z;
                acc.w += x.w;
            }
            const int64_t row = v / vec_per_row, col = (v - row * vec_per_row) * 4;
            if (bias != nullptr) {
                acc.x += to_float(bias[col]);
                acc.y += to_float(bias[col + 1]);
                acc.z += to_float(bias[col + 2]);
                acc.w += to_float(bias[col + 3]);
            }
            *reinterpret_cast<uint2 *>(out + row * p.ld_out + col) = make_uint2(pack2<T>(acc.x, acc.y), pack2<T>(acc.z, acc.w));
        }
    } else {
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < slot_elems;
             i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
            float acc = 0.f;
            for (int r = 0; r < W; ++r) acc += __ldcg(slots + r * slot_elems + i);
            const int64_t row = i / p.cols, col = i - row * p.cols;
            if (bias != nullptr) acc += to_float(bias[col]);
            out[row * p.ld_out + col] = from_float<T>(acc);
        }
    }
    peer_sg_done_round(p, &s_last);
}

// 16-byte vectors where the shard allows, single elements otherwise
__global__ void __launch_bounds__(kPeerThreads, 1) peer_all_gather_kernel(PeerSgParams p) {
    __shared__ int s_ok, s_last;
    if (!peer_sg_ready_round(p, &s_ok)) return;
    const int W = p.world;
    const int64_t row_bytes = p.cols * 2;
    uint8_t *out = static_cast<uint8_t *>(p.out);
    const bool vec = (row_bytes & 15) == 0 && ((p.ld_out * 2) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
    for (int i = 1; i < W; ++i) {
        const int src = (p.rank + i) % W;  // every rank starts with its right-hand neighbour
        const uint8_t *from = p.base[src] + p.area_off;
        uint8_t *to = out + static_cast<int64_t>(src) * p.rows * p.ld_out * 2;
        if (vec) {
            const int64_t vec_per_row = row_bytes / 16;
            const int64_t nvec = p.rows * vec_per_row;
            for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
                 v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
                const int64_t row = v / vec_per_row, c = v - row * vec_per_row;
                reinterpret_cast<uint4 *>(to + row * p.ld_out * 2)[c] = __ldcg(reinterpret_cast<const uint4 *>(from) + v);
            }
        } else {
            const int64_t n = p.rows * p.cols;
            for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < n;
                 e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
                const int64_t row = e / p.cols, c = e - row * p.cols;
                reinterpret_cast<uint16_t *>(to + row * p.ld_out * 2)[c] = __ldcg(reinterpret_cast<const uint16_t *>(from) + e);
            }
        }
    }
    peer_sg_done_round(p, &s_last);
}

// out[rows, cols] = cast(in_fp32 + bias): the tail of the NCCL reduce-scatter path
template <typename T>
__global__ void __launch_bounds__(256) cast_rows_kernel(const float *__restrict__ in, const T *__restrict__ bias,
                                                       T *__restrict__ out, int64_t ld_out, int64_t rows, int64_t cols) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * cols) return;
    const int64_t row = i / cols, col = i - row * cols;
    out[row * ld_out + col] = from_float<T>(in[i] + (bias != nullptr ? to_float(bias[col]) : 0.0f));
}

}  // namespace qmm
