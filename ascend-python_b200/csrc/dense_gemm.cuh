// Dense bf16/f16 matmul on tcgen05 (kind::f16, fp32 accumulator in tensor memory) for the two fused
// matmul + collective operators the reference ships (npu_mm_reduce_scatter_base,
// npu_all_gather_base_mm; op_plugin/ops/base_ops/opapi/MatmulReduceScatterBaseKernelNpuOpApi.cpp:22-42,
// AllGatherBaseMatmulKernelNpuOpApi.cpp:37-60).  Interface of dense_gemm.cu.
#pragma once

#include "qmm_common.cuh"

namespace qmm {

// Where the fp32 accumulator of an output element goes.
//   kDenseOutCast:  out[m, n] = cast(acc + bias[n]), 16-bit, row pitch ld_out.
//   kDenseOutPush:  the reduce-scatter form: row m belongs to rank o = m / rows_per, and the raw fp32
//                   accumulator is stored into o's peer region at
//                   base[o] + area_off + ((rank * rows_per + m - o * rows_per) * N + n) * 4
//                   (plain stores; for o != rank they cross NVLink while the tensor pipe works on).
enum { kDenseOutCast = 0, kDenseOutPush = 1 };

struct DenseParams {
    const void *a;   // [M, K] 16-bit, row pitch ld_a
    int64_t ld_a;
    const void *b;   // [K, N] addressed as b[k * b_sk + n * b_sn]; one of the strides is 1
    int64_t b_sk, b_sn;
    int dtype;       // QMM_DTYPE_BF16 or QMM_DTYPE_F16 (both operands, and the output of kDenseOutCast)
    int64_t M, N, K;
    int mode;
    void *out;       // kDenseOutCast
    int64_t ld_out;
    const void *bias;  // [N] of dtype, or nullptr (kDenseOutCast only)
    uint8_t *base[8];  // kDenseOutPush
    size_t area_off;
    int world, rank;
    int64_t rows_per;
};

// Launches the tcgen05 kernel when the operands meet TMA's 16-byte rules, a CUDA-core kernel otherwise.
int launch_dense_gemm(const DenseParams &p, cudaStream_t stream);

}  // namespace qmm
