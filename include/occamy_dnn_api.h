/*
 * occamy_dnn_api.h -- the flat C ABI of the Occamy DNN operator runtime.
 *
 * These are the symbols the LLVM lowering of Occamy's `dnn` dialect emits calls
 * to (reference: src/Conversion/DNNToLLVM/DNNAPISpecs.inc:2-129) and that the
 * reference resolves from its static library `cd_dnn_wrapper`
 * (src/Tools/dnn-wrapper/).  liboccamy_dnn.so / libcd_dnn_wrapper.a export every
 * one of them with the reference's names, argument order and meaning; behind
 * them sit hand-written sm_100a kernels instead of cuDNN / cuBLASLt.
 *
 * Conventions shared by all entry points (reference behaviour, kept):
 *   - tensors are fp32, NCHW, dense; shapes arrive as host int64_t arrays that
 *     are only valid during the call;
 *   - the caller owns every buffer (obtained from wrapDNNMalloc or
 *     wrapDNNMemPoolInit + wrapDNNMemOffset) and pre-allocates the output;
 *   - compute entry points return the output device pointer;
 *   - memory entry points return cudaError_t 0, or print and exit(-1).
 *   - `workspace`, `workspaceSize` and `algoValue` are accepted and ignored.
 *
 * Each declaration cites the reference definition it replaces
 * (path relative to src/Tools/dnn-wrapper/).
 */
#ifndef OCCAMY_DNN_API_H
#define OCCAMY_DNN_API_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef OCCAMY_NO_VENDOR_TYPES
struct cudnnContext;
typedef struct cudnnContext *cudnnHandle_t;
struct CUstream_st;
typedef struct CUstream_st *cudaStream_t;
typedef int occamy_cuda_error_t; /* cudaError_t by value */
#endif

/* ---- memory pool (the Occamy arena at run time) ---------------------------- */
/* cuda/wrapDNNMalloc.cpp:19 -- cudaMalloc + zero fill. */
occamy_cuda_error_t wrapDNNMalloc(void **devPtr, size_t size);
/* cuda/wrapDNNMemPoolInit.cpp:18 -- one allocation holding the whole planned pool. */
occamy_cuda_error_t wrapDNNMemPoolInit(void **devPtr, size_t size);
/* cuda/wrapDNNMemOffset.cpp:18 -- *devPtr = basePtr + offset; the tensor reads as zero. */
occamy_cuda_error_t wrapDNNMemOffset(void **devPtr, void *basePtr, size_t offset, size_t mallocSize);
/* cuda/wrapDNNMemcpy.cpp:16 -- kind 1 host->device, 2 device->host (complete on return). */
occamy_cuda_error_t wrapDNNMemcpy(void *dst, const void *src, size_t count, int kind, cudaStream_t stream);
/* cuda/wrapDNNDealloc.cpp:15 -- cudaFree. */
occamy_cuda_error_t wrapDNNDealloc(void *devPtr);

/* ---- vendor symbols the generated code calls directly ----------------------- */
/* DNNAPISpecs.inc:92-93; emitted at DNNToLLVMCommon.cpp:176-184.  The handle is an
 * opaque context owned by this library (no cuDNN is loaded).  cudaStreamCreate /
 * cudaStreamDestroy (DNNAPISpecs.inc:94-95) come from libcudart unchanged. */
int cudnnCreate(cudnnHandle_t *handle);
int cudnnDestroy(cudnnHandle_t handle);

/* ---- convolution ------------------------------------------------------------ */
/* cudnn/CUDNNConvFunc.cpp:8 -- y = x (*) w, KCRS filter, cross-correlation, dilation 1,
 * pads = (h, w) symmetric, `groups` channel groups (groups == C: depthwise). */
float *DNNConvFunc(cudnnHandle_t h, float *x, int64_t dimX[4], float *w, int64_t dimW[4],
                   float *workspace, int64_t workspaceSize, int64_t algoValue, int64_t groups,
                   int64_t pads[2], int64_t strides[2], float *y);
/* cudnn/fusedOp/CUDNNConvBiasReluFunc.cpp:7 -- y = act(x (*) w + b), bias [1,K,1,1];
 * activMode 1 ReLU, 5 identity (as in the reference), and additionally 3 = clipped
 * ReLU with ceiling 6 (ReLU6), which the reference never emits. */
float *DNNConvBiasActivFunc(cudnnHandle_t h, float *x, int64_t dimX[4], float *w, int64_t dimW[4],
                            float *bias, int64_t dimB[4], float *workspace, int64_t workspaceSize,
                            int64_t algoValue, int64_t pads[2], int64_t strides[2],
                            int64_t activMode, float *y);

/* ---- element-wise ----------------------------------------------------------- */
/* cudnn/CUDNNActiveFunc.cpp:7 -- mode 0 sigmoid, 1 ReLU, 2 tanh. */
float *DNNActiveFunc(cudnnHandle_t h, float *x, int64_t dimX[4], int32_t mode, float *y);
/* cudnn/CUDNNTensorOpFunc.cpp:7 -- out = A op (bias*B); opMode 0 add, 1 mul, 4 sqrt(A);
 * B is broadcast along dimensions where its extent is 1. */
float *DNNTensorOpFunc(cudnnHandle_t h, int64_t opMode, float *A, int64_t *dimA, int32_t rankA,
                       float *B, int64_t *dimB, int32_t rankB, float *out, int64_t *dimOut,
                       int32_t rankOut, float bias);
/* cuda/CUDAClipFunc.cu:13 -- y = min(max(x, lo), hi). */
float *CUDAClipFunc(float *x, float *y, int64_t *dimOut, float lo, float hi, int64_t rank);

/* ---- pooling / reduction ---------------------------------------------------- */
/* cudnn/CUDNNMaxPoolFunc.cpp:7 -- window kernel[0..1], pads (padding[0], padding[2]). */
float *DNNMaxPoolFunc(cudnnHandle_t h, float *x, int64_t dimIn[4], float *y, int64_t dimOut[4],
                      int64_t kernel[2], int64_t padding[4], int64_t stride[2]);
/* cudnn/CUDNNAveragePoolFunc.cpp:7 -- divisor counts padding. */
float *DNNAveragePoolFunc(cudnnHandle_t h, float *x, int64_t dimIn[4], float *y, int64_t dimOut[4],
                          int64_t kernel[2], int64_t padding[4], int64_t stride[2]);
/* cudnn/CUDNNReduceFunc.cpp:7 -- mode 5: mean over axes whose output extent is 1. */
float *DNNReduceFunc(cudnnHandle_t h, int32_t rank, float *x, int64_t *dimIn, float *y,
                     int64_t *dimOut, int32_t mode);

/* ---- classifier head -------------------------------------------------------- */
/* cublas/CUBLASMatmul2dFunc.cu:8 -- out = alpha*op(A)*op(B) + beta*out, row-major. */
float *CUBLASMatmul2dFunc(int64_t rank, float *A, int64_t dimA[2], float *B, int64_t dimB[2],
                          float *C, int64_t dimC[2], float *out, int64_t dimOut[2], float alpha,
                          float beta, int64_t transA, int64_t transB);
/* cuda/CUDASoftmaxFunc.cu:68 -- softmax along `axis`. */
float *CUDASoftmaxFunc(float *x, int64_t *dimIn, float *y, int64_t *dimOut, int64_t axis,
                       int64_t rank);
/* cuda/CUDAFlattenFunc.cpp:7, cuda/CUDAReshapeFunc.cpp:7 -- contiguous copy. */
float *CUDAFlattenFunc(float *x, int64_t *dimIn, float *y, int64_t *dimOut, int32_t axis,
                       int64_t rank);
float *CUDAReshapeFunc(float *x, int64_t *dimIn, int64_t rank, float *y);

/* ---- operators outside the CNN hot path (correct, not tuned) ------------------ */
/* cuda/CUDACastI64toFloatFunc.cu:12 -- returns the INPUT pointer, as the reference does. */
int64_t *CUDACastI64toFloatFunc(int64_t *in, float *out, int64_t *dimOut, int64_t rank);
/* cuda/CUDAConcatFloatFunc.cu:64, cuda/CUDAConcatInt64Func.cu:65 */
float *CUDAConcatFloatFunc(float **inList, int64_t **dimInList, float *out, int64_t *dimOut,
                           int64_t axis, int64_t inputNum, int32_t inputRank);
int64_t *CUDAConcatInt64Func(int64_t **inList, int64_t **dimInList, int64_t *out,
                             int64_t *dimOut, int64_t axis, int64_t inputNum, int32_t inputRank);
/* cuda/CUDAErfFunc.cu:12 */
float *CUDAErfFunc(float *in, float *out, int64_t *dimOut, int64_t rank);
/* cuda/CUDAExpandInt64Func.cu:4 -- plain copy of the input elements. */
int64_t *CUDAExpandInt64Func(int64_t *in, int64_t *dimIn, int64_t inRank, int64_t *out,
                             int64_t *dimOut, int64_t *shape_d, int64_t *dimShape);
/* cuda/CUDAGatherFloatFunc.cu:61, cuda/CUDAGatherInt64Func.cu:63 */
float *CUDAGatherFloatFunc(float *in, int64_t *dimIn, int64_t inRank, float *out, int64_t *dimOut,
                           int64_t outRank, int64_t *indices_d, int64_t *dimIdx, int64_t idxRank,
                           int64_t axis);
int64_t *CUDAGatherInt64Func(int64_t *in, int64_t *dimIn, int64_t inRank, int64_t *out,
                             int64_t *dimOut, int64_t outRank, int64_t *indices_d,
                             int64_t *dimIdx, int64_t idxRank, int64_t axis);
/* cuda/CUDALeakyReluFunc.cu:17 */
float *CUDALeakyReluFunc(float *in, float *out, int64_t *dimOut, float alpha, int64_t rank);
/* cuda/CUDAMatmulNdFunc.cu:85 -- batched matmul, leading dimensions of B broadcast. */
float *CUDAMatmulNdFunc(float *A, int64_t *dimA, int32_t rankA, float *B, int64_t *dimB,
                        int32_t rankB, float *out, int64_t *dimOut, int32_t rankOut);
/* cuda/CUDANegativeFunc.cu:13, cuda/CUDAReciprocalFunc.cu:13 */
float *CUDANegativeFunc(float *in, float *out, int64_t *dimIn, int64_t rank);
float *CUDAReciprocalFunc(float *in, float *out, int64_t *dimIn, int64_t rank);
/* cuda/CUDANonZeroFloatFunc.cu:19, cuda/CUDANonZeroInt64Func.cu:19 */
float *CUDANonZeroFloatFunc(float *in, int64_t *dimIn, float *out, int64_t *dimOut, int64_t rank);
int64_t *CUDANonZeroInt64Func(int64_t *in, int64_t *dimIn, int64_t *out, int64_t *dimOut,
                              int64_t rank);
/* cuda/CUDAPReluFunc.cu:17 (uses slope[0] only), cuda/CUDAPowFunc.cu:16 (scalar exponent) */
float *CUDAPReluFunc(float *in, float *out, int64_t *dimOut, float *slope, int64_t rank);
float *CUDAPowFunc(float *in, float *exponent_d, float *out, int64_t *dimOut, int64_t rank);
/* cuda/CUDASqueeze{Float,Int64}Func.cpp:5, cuda/CUDAUnsqueeze{Float,Int64}Func.cpp:5 -- copies. */
float *CUDASqueezeFloatFunc(float *in, int64_t *dimIn, float *out, int64_t *dimOut, int32_t axis,
                            int64_t rank);
int64_t *CUDASqueezeInt64Func(int64_t *in, int64_t *dimIn, int64_t *out, int64_t *dimOut,
                              int32_t axis, int64_t rank);
float *CUDAUnsqueezeFloatFunc(float *in, int64_t *dimIn, float *out, int64_t *dimOut,
                              int32_t axis, int64_t rank);
int64_t *CUDAUnsqueezeInt64Func(int64_t *in, int64_t *dimIn, int64_t *out, int64_t *dimOut,
                                int32_t axis, int64_t rank);
/* cuda/CUDATranspose{2,3,4,6}D{Float,Int64}Func.cu -- out = permute(in, perm). */
float *CUDATranspose2DFloatFunc(float *in, int64_t *dimIn, float *out, int64_t *dimOut,
                                int64_t *perm, int64_t rank);
float *CUDATranspose3DFloatFunc(float *in, int64_t *dimIn, float *out, int64_t *dimOut,
                                int64_t *perm, int64_t rank);
float *CUDATranspose4DFloatFunc(float *in, int64_t *dimIn, float *out, int64_t *dimOut,
                                int64_t *perm, int64_t rank);
float *CUDATranspose6DFloatFunc(float *in, int64_t *dimIn, float *out, int64_t *dimOut,
                                int64_t *perm, int64_t rank);
int64_t *CUDATranspose2DInt64Func(int64_t *in, int64_t *dimIn, int64_t *out, int64_t *dimOut,
                                  int64_t *perm, int64_t rank);
int64_t *CUDATranspose3DInt64Func(int64_t *in, int64_t *dimIn, int64_t *out, int64_t *dimOut,
                                  int64_t *perm, int64_t rank);
int64_t *CUDATranspose4DInt64Func(int64_t *in, int64_t *dimIn, int64_t *out, int64_t *dimOut,
                                  int64_t *perm, int64_t rank);
int64_t *CUDATranspose6DInt64Func(int64_t *in, int64_t *dimIn, int64_t *out, int64_t *dimOut,
                                  int64_t *perm, int64_t rank);

/* ---- controls that have no counterpart in the reference ----------------------- */
/* Arithmetic mode of the convolution / GEMM kernels:
 * 0 = fp32 CUDA-core kernels on the ABI's NCHW fp32 tensors (max rel. error <= 1e-4 against
 *     the CPU semantics);
 * 1 = bf16 tcgen05 tensor-core kernels with fp32 accumulation, activations kept as NHWC bf16
 *     between operators (default; <= 2e-2 on the logits of ResNet-50 and VGG-16);
 * 2 = the same kernels on fp16 operands and fp16 NHWC activations: three more mantissa bits
 *     than bf16 (the precision of TF32) at the same speed and bytes, for networks whose
 *     activations stay below 65504 in magnitude -- MobileNetV2, whose ReLU6 bounds them, needs
 *     it to stay within 2e-2.  A value beyond that range becomes infinity, never a silently
 *     wrong finite number.  In this mode the 3x3 depthwise convolution also keeps its sums of
 *     nine products in fp16 (all other kernels accumulate in fp32 in both 16-bit modes).
 * Also settable with the environment variable OCCAMY_MATH=fp32|bf16|fp16 before the first
 * call. */
void occamy_set_math_mode(int mode);
int occamy_get_math_mode(void);
/* 0 if every call so far succeeded; otherwise a sticky code (CUDA error, or 1000 + a
 * kernel-side watchdog code).  `clear` != 0 resets it. */
int occamy_last_error(int clear);
/* Block until all work enqueued by this library has finished; returns cudaError_t. */
int occamy_synchronize(void);
/* Self-test of the kernels' watchdog: enqueues a one-thread kernel that waits on a barrier
 * nothing will ever signal.  Its wait is the bounded wait of the convolution kernels, so
 * after about two seconds it gives up and reports; the next occamy_synchronize() then makes
 * occamy_last_error() return 1099.  Nothing hangs and the context stays usable. */
void occamy_selftest_bounded_wait(void);
/* Stream all kernels of this library are launched on (for CUDA-event timing). */
cudaStream_t occamy_stream(void);
/* Counters since load: [0] kernel launches, [1] bytes uploaded host->device,
 * [2] bytes of uploads skipped because the packed weight was already resident,
 * [3] pool high-water mark in bytes, [4] tensor-core conv/GEMM launches,
 * [5] layout materialisations (NHWC bf16 -> NCHW fp32), [6] tensor-map encodes,
 * [7] fp32 CUDA-core conv/GEMM launches. */
void occamy_get_counters(int64_t out[8]);
/* Per-launch timing of the tensor-core convolution / GEMM kernel: after _begin, every such
 * launch is bracketed by a CUDA-event pair on the launch stream; _end waits for the stream,
 * writes the elapsed milliseconds of up to `cap` launches in call order and returns how
 * many launches were recorded. */
void occamy_profile_begin(void);
int occamy_profile_end(float *ms, int cap);
/* Number of convolution -> add / activation chains that arrived as separate calls and were
 * executed as one kernel (cross-call fusion; OCCAMY_FUSE_ACROSS_CALLS=0 turns it off). */
int64_t occamy_fused_chains(void);
void occamy_set_cross_call_fusion(int on);
/* Drop the resident packed-weight cache (forces re-upload and re-pack). */
void occamy_clear_weight_cache(void);
/* fp32 mode: 1 (default) runs dense convolutions (1x1 and 3x3, stride <= 2) and GEMMs on the
 * tensor cores with every fp32 value carried as three bf16 parts and fp32 accumulation --
 * the result stays within the fp32 mode's 1e-4 bound; 0 leaves the CUDA-core kernels.
 * Same switch as the environment variable OCCAMY_FP32_TC=0|1. */
void occamy_set_fp32_tensor_cores(int on);
/* 0: keep no packed constants between calls (every filter is packed again on every use and
 * every constant upload crosses PCIe, as in the reference); 1 (default): keep them.  Same
 * switch as the environment variable OCCAMY_CACHE_WEIGHTS=0|1. */
void occamy_set_weight_cache(int on);

/* ---- fused convolution for callers that must not allocate ---------------------- */
/* No counterpart in the reference.  Same arithmetic as DNNConvBiasActivFunc in the bf16
 * tensor-core mode (y = act(x (*) w + b), fp32 NCHW in and out, activMode 1 / 3 / 5), for
 * hosts that cannot call cudaMalloc where they call the runtime: processes that run inside
 * a device-memory budget fixed before start-up, and latency-critical loops that must stay
 * out of the driver's allocator (it takes process-wide locks and may synchronise the
 * device).  All working copies live in a fixed 32 MiB device array that is part of the
 * library image (so every GPU that loads the library carries it until exit); a problem
 * whose copies (NHWC bf16 forms of x and y plus the packed filter) do not fit is refused
 * with -2 and nothing is launched.  Needs C % 16 == 0 and K % 8 == 0 (-3 otherwise).
 * Work is enqueued on `stream`; the call does not wait for it.  All calls share the one
 * array: calls whose kernels may overlap on the GPU race, so keep them on one stream or
 * order them with events.  The first call on each device also looks up the array's device
 * address (guarded: once per device even if two host threads race to it); make it outside
 * any stream capture.  Returns 0, a negative code as above (-3 also for extents beyond
 * INT_MAX, negative pads, or a filter larger than the padded image), or a cudaError_t
 * value.  A return of 0 says the work was enqueued: a kernel whose bounded waits ran out
 * afterwards leaves garbage in y and a code in the array's error word, which
 * occamy_noalloc_last_error() below (and occamy_last_error / occamy_synchronize) report. */
int occamy_conv_bias_act_noalloc(const float *x, const int64_t dimX[4], const float *w,
                                 const int64_t dimW[4], const float *bias, const int64_t pads[2],
                                 const int64_t strides[2], int64_t activMode, float *y,
                                 cudaStream_t stream);
/* No counterpart in the reference.  0, or the code (1001..1006) a kernel of an earlier
 * occamy_conv_bias_act_noalloc call on the current device left when one of its bounded
 * waits ran out; `clear` != 0 resets it.  Reads one word with a blocking copy and allocates
 * nothing; synchronise the stream the calls went to before asking. */
int occamy_noalloc_last_error(int clear);
/* Bytes of the fixed array available to one call's working copies. */
int64_t occamy_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
#endif /* OCCAMY_DNN_API_H */
