/*
 * qmm_b200.h — C ABI of the B200 quantized-matmul library (libqmm_b200.so).
 *
 * This is the launch boundary the operator host code binds to.  In the
 * reference plugin the same role is played by the `aclnn*` symbols that
 * `EXEC_NPU_CMD` resolves with dlsym and calls in two phases
 * (op_plugin/utils/op_api_common.h:62, :520-570): a `...GetWorkspaceSize`
 * query followed by the launch on an explicit stream, `0` meaning success and
 * any other value being turned into a TORCH_CHECK failure that quotes the
 * library's last error text (op_api_common.h:546,555).  The functions below
 * keep that convention: plain pointers and sizes, an explicit stream, an `int`
 * status, `qmm_last_error()` for the message.  No torch types, no exceptions.
 *
 * All device pointers must belong to the device that is current on the calling
 * thread.  Every launch is asynchronous on `stream` (a `cudaStream_t`, passed
 * as `void*` so that this header needs no CUDA include).
 */
#ifndef QMM_B200_H_
#define QMM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define QMM_API __attribute__((visibility("default")))
#else
#define QMM_API
#endif

/* Status codes (0 = success, like the aclnn convention). */
enum {
    QMM_OK = 0,
    QMM_ERR_INVALID_ARGUMENT = 1,
    QMM_ERR_UNSUPPORTED = 2,
    QMM_ERR_CUDA = 3,
    QMM_ERR_NCCL = 4,
    QMM_ERR_NOT_FOUND = 5,
    QMM_ERR_WORKSPACE = 6,
    QMM_ERR_DEVICE_TIMEOUT = 7
};

/* Element types of activations, biases and outputs. */
enum {
    QMM_DTYPE_BF16 = 0,
    QMM_DTYPE_F16 = 1,
    QMM_DTYPE_F32 = 2,
    QMM_DTYPE_I32 = 3,
    QMM_DTYPE_NONE = -1
};

/* Kernel selection for qmm_quant_matmul (QMM_ALGO_AUTO in production). */
enum {
    QMM_ALGO_AUTO = 0,
    QMM_ALGO_TCGEN05_TILE = 1,   /* 128x256 output tiles, one CTA per tile (prefill) */
    QMM_ALGO_TCGEN05_STREAMK = 2, /* weights as the MMA's M operand, K split over CTAs (decode) */
    QMM_ALGO_SIMT = 3,           /* dp4a kernel: any alignment, any stride */
    QMM_ALGO_TCGEN05_PAIR = 4,   /* 256x256 output tiles on CTA pairs, cta_group::2 MMA (prefill) */
    QMM_ALGO_TCGEN05_SPLITK = 5  /* the one-CTA tile kernel over K slices + a reduce kernel (M <= 128, few tiles) */
};

/* Text of the last error raised on the calling thread ("" if none). */
QMM_API const char *qmm_last_error(void);

/* Library version: major*10000 + minor*100 + patch. */
QMM_API int qmm_version(void);

/*
 * Status word written by kernels whose bounded device-side waits gave up
 * (0 = no wait ever timed out on this device).  Reads host-mapped memory: call
 * after synchronizing the stream.  `reset` != 0 clears it.
 */
QMM_API int qmm_device_status(int reset);

/*
 * Measurement utility (no counterpart in the reference): the rate at which this GPU's tensor pipe executes
 * tcgen05.mma.kind::i8 when nothing else limits it (operands resident in shared memory, one CTA per SM,
 * `batches` x 64 MMAs of 128 x 256 x 32 per CTA; runs on the default stream and synchronizes).  Returns
 * int8 operations per clock and SM (from the SMs' cycle counters), TOPS over the run (CUDA events) and
 * the SM clock the run saw.  It is the denominator of the W8A8 roofline fractions.
 */
QMM_API int qmm_int8_mma_peak(int batches, double *ops_per_clk_per_sm, double *tops, double *sm_mhz);

/*
 * Per-token dynamic quantization (torch op `npu_dynamic_quant`; the op is not
 * in the reference snapshot, its host conventions follow
 * op_plugin/ops/base_ops/aclops/QuantizePerChannelKernelNpu.cpp:69-92).
 *   amax[r]  = max_c |x[r,c]|            (fp32)
 *   scale[r] = amax[r] / 127             (fp32 division)
 *   q[r,c]   = clamp(rint(x[r,c] / scale[r]), -128, 127), rows with amax==0 -> 0
 * x: [rows, cols] bf16/f16, row stride ld_x elements; q: int8 row stride ld_q;
 * scale: [rows] fp32.
 */
QMM_API int qmm_dynamic_quant(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld_x,
                              int8_t *q, int64_t ld_q, float *scale, void *stream);

/*
 * RMS normalisation (torch op `npu_rms_norm`; host function
 * op_plugin/ops/base_ops/opapi/RmsNormKernelOpApi.cpp:24-35, numpy golden
 * test/test_custom_ops/test_npu_rms_norm.py:10-18):
 *   variance[r] = mean_c x[r,c]^2;  rstd[r] = 1 / sqrt(variance[r] + epsilon);
 *   y[r,c] = (x[r,c] * rstd[r]) * gamma[c]        fp32, one rounding per operation, y rounded to x's dtype
 * x, y: [rows, cols] of x_dtype (BF16, F16 or F32), row strides ld_x / ld_y; gamma: [cols] of x_dtype;
 * rstd: [rows] fp32.
 */
QMM_API int qmm_rms_norm(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld_x, const void *gamma,
                         double epsilon, void *y, int64_t ld_y, float *rstd, void *stream);

/*
 * qmm_rms_norm followed by qmm_dynamic_quant of its output, in one pass over HBM (torch op
 * `npu_rms_norm_dynamic_quant`, which has no counterpart in the reference: it fuses the reference's
 * npu_rms_norm, RmsNormKernelOpApi.cpp:24-35, with the quantization step that consumes it).  q and scale
 * are bit-identical to qmm_dynamic_quant(qmm_rms_norm(x)): the normalised row is rounded to x_dtype
 * (BF16 or F16) in registers before its absmax is taken.
 */
QMM_API int qmm_rms_norm_dynamic_quant(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld_x,
                                       const void *gamma, double epsilon, int8_t *q, int64_t ld_q, float *scale,
                                       float *rstd, void *stream);

/*
 * Bytes of scratch memory qmm_quant_matmul needs for a problem (first phase
 * of the two-phase call, cf. `aclnnXGetWorkspaceSize`, op_api_common.h:543-546).
 * May be 0.  The scratch must be zero-filled before its FIRST use only; the
 * kernels leave it zeroed again.
 */
QMM_API int qmm_quant_matmul_workspace_size(int64_t M, int64_t N, int64_t K, int algo, size_t *bytes);

/*
 * W8A8 matmul with fused dequantization (torch op `npu_quant_matmul`; host
 * conventions follow op_plugin/ops/base_ops/opapi/MmKernelNpuOpApi.cpp:24-42).
 *   acc[m,n] = sum_k x1[m,k] * x2[k,n]                       (int32, exact)
 *   out_dtype == I32 : out = acc (+ bias if bias_dtype == I32)
 *   else             : out = cast(float(acc) * scale[n] * pertoken_scale[m] + bias[n])
 * x1: int8 [M,K], row stride ld_x1.  x2: int8 [K,N] addressed as
 * x2[k*x2_stride_k + n*x2_stride_n]; one of the two strides must be 1
 * (row-major [K,N], or the transposed view of a row-major [N,K]).
 * scale: fp32, scale_len is N or 1.  pertoken_scale: fp32 [M] or NULL.
 * bias: [N] of bias_dtype, or NULL with QMM_DTYPE_NONE.
 * out: [M,N] of out_dtype (BF16, F16 or I32), row stride ld_out.
 * workspace: at least the queried size (may be NULL when that is 0).
 */
QMM_API int qmm_quant_matmul(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_stride_k,
                             int64_t x2_stride_n, const float *scale, int64_t scale_len,
                             const float *pertoken_scale, const void *bias, int bias_dtype, void *out,
                             int out_dtype, int64_t ld_out, int64_t M, int64_t N, int64_t K, int algo,
                             void *workspace, size_t workspace_bytes, void *stream);

/*
 * W8A8 matmul with an int8 (requantized) output: torch op `npu_quant_matmul` with output_dtype = int8 and the
 * optional `offset` (neither the operator nor this arithmetic is in the reference snapshot; the form is this
 * library's stated choice):
 *   acc = x1 @ x2 + bias (int32, exact);  v = float(acc) * scale[n] (* pertoken_scale[m]) (+ offset[n])  in fp32,
 *   one rounding per operation;  out = clamp(rint(v), -128, 127), ties to even.
 * scale / offset: fp32 with N elements or one; offset, pertoken_scale and bias (int32 [N]) may be NULL.
 * workspace: 256-byte aligned, qmm_quant_matmul_int8_workspace_size bytes; it holds the matmul kernels' own
 * scratch (cleared by the call) and the int32 accumulator, and needs no preparation by the caller.
 */
QMM_API int qmm_quant_matmul_int8_workspace_size(int64_t M, int64_t N, int64_t K, size_t *bytes);
QMM_API int qmm_quant_matmul_int8(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_stride_k,
                                  int64_t x2_stride_n, const float *scale, int64_t scale_len, const float *offset,
                                  int64_t offset_len, const float *pertoken_scale, const int32_t *bias, int8_t *out,
                                  int64_t ld_out, int64_t M, int64_t N, int64_t K, void *workspace,
                                  size_t workspace_bytes, void *stream);

/*
 * Decode-shape W8A8 matmul that allocates nothing.  It has no counterpart in
 * the reference: it exists for hosts that may not call cudaMalloc (or any
 * allocator) once they are running — a server whose device memory was split up
 * at start-up, a plugin bound by a no-allocation-after-init contract, a
 * latency-critical thread that must stay off allocator locks.  Where
 * qmm_quant_matmul takes its split-K scratch from the caller, this entry point
 * uses a QMM_NOALLOC_SCRATCH_BYTES array that is part of the library image
 * (each GPU that loads the library holds it until the process exits).
 * Arguments and results are those of qmm_quant_matmul; the result is
 * bit-identical to qmm_quant_matmul with QMM_ALGO_TCGEN05_STREAMK.
 *   - 1 <= M <= 128, and ceil(N/128) * (round_up(M,16) * 512 + 4) + 252 bytes
 *     must fit the array (e.g. M=128 up to N=32640, M=16 up to N=262016);
 *     larger problems are refused with QMM_ERR_WORKSPACE.
 *   - operands need 16-byte aligned addresses and row pitches.
 *   - the first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call before any stream capture.
 *   - all calls on a device share the one array: calls that may overlap on the
 *     GPU (different streams without ordering) race on it; keep them ordered.
 *   - the array keeps what the last call left.  The kernel hands it back zeroed, which
 *     is what the next call needs; a small kernel in front of every call clears it
 *     after a call that was cut short (no per-call memset of the 16 MiB).
 *   - a bounded device-side wait that gives up on this path is recorded in a status word
 *     inside the library image, read with qmm_noalloc_status (qmm_device_status reads
 *     allocated host memory, which this path never creates).
 */
#define QMM_NOALLOC_SCRATCH_BYTES (16u << 20)
QMM_API int qmm_quant_matmul_decode_noalloc(const int8_t *x1, int64_t ld_x1, const int8_t *x2,
                                            int64_t x2_stride_k, int64_t x2_stride_n, const float *scale,
                                            int64_t scale_len, const float *pertoken_scale, const void *bias,
                                            int bias_dtype, void *out, int out_dtype, int64_t ld_out, int64_t M,
                                            int64_t N, int64_t K, void *stream);
/* Status word of the entry point above on the current device (0 = no wait gave up, -1 = the read failed);
 * synchronizes with the device; `reset` != 0 clears the codes whose clean-up has already run.  Allocates nothing. */
QMM_API int qmm_noalloc_status(int reset);

/*
 * W4A16 matmul (torch op `npu_weight_quant_batchmatmul`; host conventions as
 * above plus the bias handling of
 * op_plugin/ops/base_ops/aclops/LinearKernelNpu.cpp:29-45).
 *   W[k,n]  = (w4[k,n] + offset[k/group, n]) * scale[k/group, n]
 *   out     = cast(x @ W + bias)
 * x: [M,K] bf16/f16 (x_dtype), row stride ld_x.  weight: int32 [K, N/8], row
 * stride ld_w words; nibble j of word i holds column 8*i+j as a two's
 * complement 4-bit integer.  antiquant_scale / antiquant_offset:
 * [K/group, N] of x_dtype (offset may be NULL = 0).  group must divide K and
 * be a multiple of 32; group == K gives per-channel quantization.
 * out: [M,N] of x_dtype, row stride ld_out.
 * workspace: scratch of at least qmm_weight_quant_batchmatmul_workspace_size bytes, 256-byte
 * aligned, zero-filled before its first use only (the kernel leaves it reusable).  Without it
 * (NULL), or with operands that break the 16-byte rules of TMA, a CUDA-core kernel runs.
 */
QMM_API int qmm_weight_quant_batchmatmul_workspace_size(int64_t M, int64_t N, int64_t K, int64_t group,
                                                        size_t *bytes);
QMM_API int qmm_weight_quant_batchmatmul(const void *x, int x_dtype, int64_t ld_x, const int32_t *weight,
                                         int64_t ld_w, const void *antiquant_scale,
                                         const void *antiquant_offset, int64_t group, const void *bias,
                                         void *out, int64_t ld_out, int64_t M, int64_t N, int64_t K,
                                         void *workspace, size_t workspace_bytes, void *stream);

/*
 * Prepacked W4A16 weights.  The reference keeps matmul operands in a private device format and
 * casts to and from the plain layout around the matmul (ND <-> FRACTAL_NZ,
 * op_plugin/ops/base_ops/aclops/MmKernelNpu.cpp:80-94, :301-316); this is the same step for the
 * int4 weights of npu_weight_quant_batchmatmul.  qmm_w4a16_prepack rewrites weight [K, N/8] with
 * its antiquant scale and offset ONCE into a k-major stream (128 columns x 128 k per block, scale
 * and offset*scale of the block's group behind its nibbles); qmm_weight_quant_batchmatmul_prepacked
 * then computes the same product as qmm_weight_quant_batchmatmul from that buffer alone, with the
 * weight W = fma(w, scale, offset*scale) rounded once to the activation dtype before the
 * tensor-core product (fp32 accumulation).
 *   - supported: N % 8 == 0, K % 128 == 0, group a multiple of 128 that divides K (group <= 0 means K);
 *     qmm_w4a16_prepack_size returns 0 bytes for anything else and the stock entry point remains.
 *   - sdtype (BF16/F16) is the dtype of scale and offset and must equal the x_dtype used later.
 *   - packed: 16-byte aligned, at least qmm_w4a16_prepack_size bytes.
 *   - qmm_w4a16_unpack_weight restores the stock int32 [K, N/8] words exactly.
 *   - workspace of the matmul: 256-byte aligned, zero-filled before its first use only.
 */
QMM_API int qmm_w4a16_prepack_size(int64_t N, int64_t K, int64_t group, size_t *bytes);
QMM_API int qmm_w4a16_prepack(const int32_t *weight, int64_t ld_w, const void *antiquant_scale,
                              const void *antiquant_offset, int sdtype, int64_t group, int64_t N, int64_t K,
                              void *packed, size_t packed_bytes, void *stream);
QMM_API int qmm_w4a16_unpack_weight(const void *packed, int64_t N, int64_t K, int32_t *weight, int64_t ld_w,
                                    void *stream);
QMM_API int qmm_weight_quant_batchmatmul_prepacked_workspace_size(int64_t M, int64_t N, int64_t K, size_t *bytes);
QMM_API int qmm_weight_quant_batchmatmul_prepacked(const void *x, int x_dtype, int64_t ld_x, const void *packed,
                                                   size_t packed_bytes, const void *bias, void *out,
                                                   int64_t ld_out, int64_t M, int64_t N, int64_t K,
                                                   void *workspace, size_t workspace_bytes, void *stream);

/*
 * Communicator registry.  The reference passes a communicator NAME into its
 * fused matmul+collective kernels (`hcom`,
 * op_plugin/ops/base_ops/opapi/MatmulReduceScatterBaseKernelNpuOpApi.cpp:35-40)
 * which the device library resolves.  Here the name resolves to an NCCL
 * communicator created by qmm_comm_init_rank (all ranks call it with the id
 * rank 0 obtained from qmm_comm_unique_id) or adopted with qmm_comm_register.
 */
#define QMM_UNIQUE_ID_BYTES 128
QMM_API int qmm_comm_unique_id(void *id_out /* QMM_UNIQUE_ID_BYTES */);
QMM_API int qmm_comm_init_rank(const char *name, const void *id, int nranks, int rank);
QMM_API int qmm_comm_register(const char *name, void *nccl_comm, int nranks, int rank);
QMM_API int qmm_comm_info(const char *name, int *nranks, int *rank);
QMM_API int qmm_comm_destroy(const char *name);
/* Calls of qmm_mm_all_reduce made through the communicator so far, by the path their allreduce took:
 * the library's own kernels over peer memory (of those, calls whose matmul pushed its output tiles to the
 * owning ranks itself; and, of those again, calls whose matmul kernel also reduced and gathered the output, so
 * that no second kernel ran), or NCCL.  Any pointer may be NULL.  No counterpart in the reference. */
QMM_API int qmm_comm_stats(const char *name, int64_t *peer_calls, int64_t *peer_pushed_calls,
                           int64_t *peer_fused_calls, int64_t *nccl_calls);

/* Peer memory for the allreduce of qmm_mm_all_reduce (no counterpart in the reference: its device
 * library owns the communication buffers behind the communicator name,
 * op_plugin/ops/base_ops/opapi/MatmulReduceScatterBaseKernelNpuOpApi.cpp:35-40).
 * Every rank of the node allocates a region of the same size, zero-filled, that all ranks map
 * (CUDA IPC / symmetric memory), and hands the library the W addresses under which this process
 * sees them, in rank order (its own included), plus - where the regions are bound to an NVLink
 * multicast object - the multicast address (else NULL).  qmm_comm_peer_memory_size gives the size an
 * allreduce of [M][N] 16-bit values needs.  While regions are attached and large enough, calls
 * with comm_turn == 0 reduce and gather over NVLink in the library's own kernels instead of NCCL
 * (for prefill-sized M on two ranks inside the matmul kernel itself, otherwise in one more kernel per
 * rank); the environment variable QMM_ALLREDUCE=nccl switches that off, QMM_PEER_FUSED=0|1 forces the
 * exchange out of / into the matmul kernel (set them on every rank or on none).  The choice depends
 * only on M, N, comm_turn, the rank count, the attached size and those variables, which all ranks share; on
 * that path `out` must be 16-byte aligned and the stream must not be capturing (both are errors, not a
 * switch to NCCL that the other ranks would not follow).  Calls of different shapes may follow one
 * another without synchronisation in between.  bytes == 0 detaches. */
QMM_API int qmm_comm_peer_memory_size(int64_t M, int64_t N, int nranks, size_t *bytes);
QMM_API int qmm_comm_attach_peer_memory(const char *name, const void *const *regions, const void *multicast,
                                        size_t bytes);

/*
 * Row-parallel W8A8 matmul + allreduce (torch op `npu_mm_all_reduce_base`;
 * modelled on `npu_mm_reduce_scatter_base`,
 * MatmulReduceScatterBaseKernelNpuOpApi.cpp:22-42).  Each rank holds a K shard
 * of x1/x2 and its own pertoken_scale; the per-rank result is rounded to
 * out_dtype (BF16/F16) and summed over the communicator `hcom`.  bias is added
 * on rank 0 only, so it enters the sum once.  `comm_turn` > 0 sets the number
 * of M chunks whose allreduce overlaps the matmul of the next chunk (0 = let
 * the library choose).  Arguments otherwise as qmm_quant_matmul.  The call
 * returns with all work ordered on `stream`.
 */
QMM_API int qmm_mm_all_reduce(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_stride_k,
                              int64_t x2_stride_n, const float *scale, int64_t scale_len,
                              const float *pertoken_scale, const void *bias, int bias_dtype, void *out,
                              int out_dtype, int64_t ld_out, int64_t M, int64_t N, int64_t K,
                              const char *hcom, const char *reduce_op, int64_t comm_turn, void *workspace,
                              size_t workspace_bytes, void *stream);

/*
 * Matmul + reduce-scatter (torch op `npu_mm_reduce_scatter_base`,
 * op_plugin/ops/base_ops/opapi/MatmulReduceScatterBaseKernelNpuOpApi.cpp:22-42; golden formula
 * test/test_custom_ops/test_mm_reduce_scatter_base.py:69-81):
 *   out = rows [rank * M/W, (rank+1) * M/W) of cast( sum_r float(x1_r) @ float(x2_r) + bias )
 * x1: [M, K] bf16/f16 (dtype), row pitch ld_x1; x2: [K, N] of dtype addressed as in qmm_quant_matmul (row-major or
 * the transposed view of a row-major [N, K]); bias: [N] of dtype or NULL; out: [M/W, N] of dtype.  M must be
 * divisible by the communicator's size W.  Every rank's products are accumulated in fp32 and added in fp32 in rank
 * order before the single rounding.  With peer memory attached (qmm_comm_attach_peer_memory; the first half of a
 * region must hold M*N*4 bytes) the matmul's epilogue stores its fp32 rows straight into the owning rank's region
 * and one kernel per rank adds them; otherwise the fp32 partial goes through ncclReduceScatter and needs the
 * workspace (256-byte aligned).  comm_turn is accepted for signature compatibility.
 */
QMM_API int qmm_mm_reduce_scatter_workspace_size(int64_t M, int64_t N, int64_t K, int nranks, size_t *bytes);
QMM_API int qmm_mm_reduce_scatter(const void *x1, int dtype, int64_t ld_x1, const void *x2, int64_t x2_stride_k,
                                  int64_t x2_stride_n, const void *bias, void *out, int64_t ld_out, int64_t M,
                                  int64_t N, int64_t K, const char *hcom, const char *reduce_op, int64_t comm_turn,
                                  void *workspace, size_t workspace_bytes, void *stream);

/*
 * All-gather + matmul (torch op `npu_all_gather_base_mm`,
 * op_plugin/ops/base_ops/opapi/AllGatherBaseMatmulKernelNpuOpApi.cpp:22-60; golden formula
 * test/test_custom_ops/test_all_gather_base_mm.py:72-78):
 *   gathered = concat_r x1_r  ([W * M, K]);   out = cast( float(gathered) @ float(x2) + bias )   ([W * M, N])
 * M is this rank's row count.  gather_out ([W * M, K], row pitch ld_gather) receives the gathered matrix, or is
 * NULL, in which case the workspace holds it.  Only gather_index == 0 is supported.  With peer memory attached
 * (first half >= M*K*2 bytes) the shards are pulled over NVLink by the library's own kernel, otherwise by
 * ncclAllGather (contiguous x1 and gather_out required).
 */
QMM_API int qmm_all_gather_mm_workspace_size(int64_t M, int64_t N, int64_t K, int nranks, size_t *bytes);
QMM_API int qmm_all_gather_mm(const void *x1, int dtype, int64_t ld_x1, const void *x2, int64_t x2_stride_k,
                              int64_t x2_stride_n, const void *bias, void *out, int64_t ld_out, void *gather_out,
                              int64_t ld_gather, int64_t M, int64_t N, int64_t K, const char *hcom,
                              int64_t gather_index, int64_t comm_turn, void *workspace, size_t workspace_bytes,
                              void *stream);

#ifdef __cplusplus
}
#endif
#endif /* QMM_B200_H_ */
