// Launchers of the device kernels.  Every launcher enqueues on the given stream and
// returns immediately; none allocates.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace occ {

// Activation codes shared by host and device (cuDNN's numbering, which is what crosses
// the ABI): 0 sigmoid, 1 ReLU, 2 tanh, 3 clipped ReLU [lo, hi], 5 identity.
enum Act { ACT_SIGMOID = 0, ACT_RELU = 1, ACT_TANH = 2, ACT_CLIP = 3, ACT_IDENTITY = 5 };

struct ConvGeom {
  int N, C, H, W;       // input, NCHW logical dims
  int K, R, S;          // filter [K, C/groups, R, S]
  int P, Q;             // output spatial dims
  int groups;
  int pad_h, pad_w, stride_h, stride_w;
  int act;              // Act
  float lo, hi;         // bounds for ACT_CLIP
};

// ---- fp32 NCHW kernels (ABI layout) ------------------------------------------
void launch_conv_f32(const float *x, const float *w, const float *bias, float *y,
                     const ConvGeom &g, cudaStream_t s);
void launch_depthwise_f32(const float *x, const float *w, const float *bias, float *y,
                          const ConvGeom &g, cudaStream_t s);
// out = A op (biasB*B); dimB has extent 1 where B is broadcast; rank <= 8.
void launch_tensor_op_f32(int mode, const float *A, const float *B, float *out, int rank,
                          const int64_t *dimA, const int64_t *dimB, float biasB, cudaStream_t s);
void launch_act_f32(const float *x, float *y, int64_t n, int act, float lo, float hi,
                    cudaStream_t s);
void launch_pool_f32(const float *x, float *y, int N, int C, int H, int W, int P, int Q, int kh,
                     int kw, int pad_h, int pad_w, int sh, int sw, bool avg, cudaStream_t s);
// Mean over the axes where dimOut is 1 and dimIn is not; rank <= 8.
void launch_reduce_mean_f32(const float *x, float *y, int rank, const int64_t *dimIn,
                            const int64_t *dimOut, cudaStream_t s);
// out[M,N] = alpha * op(A) * op(B) + beta * out, row-major; lda/ldb are the stored row lengths.
void launch_gemm_f32(const float *A, const float *B, float *out, int M, int N, int K, int lda,
                     int ldb, float alpha, float beta, bool transA, bool transB, cudaStream_t s);
void launch_softmax_f32(const float *x, float *y, int64_t outer, int64_t len, int64_t inner,
                        cudaStream_t s);

// ---- 16-bit NHWC kernels (tensor-core mode activations) -----------------------
// `bf16 *` is the pointer type of every 16-bit tensor, whichever of the two element types it
// holds; the `f16` argument of a launcher says which: false = bf16, true = fp16.
typedef __nv_bfloat16 bf16;
void launch_nchw_f32_to_nhwc_bf16(const float *x, bf16 *y, int N, int C, int H, int W, bool f16,
                                  cudaStream_t s);
void launch_nhwc_bf16_to_nchw_f32(const bf16 *x, float *y, int N, int C, int H, int W, bool f16,
                                  cudaStream_t s);
void launch_f32_to_bf16(const float *x, bf16 *y, int64_t n, bool f16, cudaStream_t s);
// out = act(a + b) over n elements (b may be null); c-periodic fp32 bias may be added.
void launch_add_act_bf16(const bf16 *a, const bf16 *b, const float *bias_c, int C, bf16 *out,
                         int64_t n, int act, float lo, float hi, bool f16, cudaStream_t s);
void launch_pool_bf16(const bf16 *x, bf16 *y, int N, int C, int H, int W, int P, int Q, int kh,
                      int kw, int pad_h, int pad_w, int sh, int sw, bool avg, bool f16,
                      cudaStream_t s);
// Global average pool: x [N, HW, C] 16-bit -> y [N, C] fp32.
void launch_gap_bf16(const bf16 *x, float *y, int N, int HW, int C, bool f16, cudaStream_t s);
// Depthwise RxS convolution on 16-bit NHWC, weights fp32 packed [R*S][C], fused bias + act.
void launch_depthwise_bf16(const bf16 *x, const float *w_rsc, const float *bias, bf16 *y,
                           const ConvGeom &g, bool f16, cudaStream_t s);
// Weight packing: fp32 KCRS -> 16-bit [R*S][K][C] (dense conv) ...
void launch_pack_krsc_bf16(const float *w, bf16 *out, int K, int C, int R, int S, int Cp, bool f16,
                           cudaStream_t s);
void launch_pad_channels_bf16(const bf16 *x, bf16 *y, int64_t pixels, int C, int Cp, cudaStream_t s);
// ... fp32 [C,1,R,S] -> fp32 [R*S][C] (depthwise) ...
void launch_pack_dw_f32(const float *w, float *out, int C, int R, int S, cudaStream_t s);
// ... and fp32 KCRS with tiny C -> bf16 [R][K][Sp*Cp] (width taps folded into channels).
void launch_pack_fold_bf16(const float *w, bf16 *out, int K, int C, int R, int S, int Sp, int Cp,
                           bool f16, cudaStream_t s);
// Input side of the folded form: x fp32 NCHW (C <= Cp) -> bf16 [N][H][Wp][Cp] with pad_w zero
// pixels on the left of every row and zeros up to Wp on the right.  The A vector of output
// column q, Cf = Sp*Cp elements starting at pixel q*stride_w, is then a window of the row;
// windows of neighbouring columns overlap and a tensor map with a pixel stride shorter than
// its innermost extent reads them in place.
void launch_pad_input_bf16(const float *x, bf16 *out, int N, int C, int H, int W, int Wp, int Cp,
                           int pad_w, bool f16, cudaStream_t s);

// ---- fp32 carried as three bf16 parts (fp32 mode on the tensor cores) ----------
// x fp32 NCHW -> three consecutive NHWC planes [N][H][W][Cp] (hi, mid, lo), zero channels up to Cp
void launch_split3_nchw(const float *x, bf16 *y, int N, int C, int Cp, int H, int W, cudaStream_t s);
// x fp32 [M][K], rows `ld` floats apart -> three consecutive planes [M][Kp]
void launch_split3_rows(const float *x, bf16 *y, int M, int K, int Kp, int ld, cudaStream_t s);
// fp32 KCRS -> bf16 [R*S*6][K][Cp]: six filter parts per tap, in the order the kernel pairs
// them with the activation parts
void launch_pack_krsc_split(const float *w, bf16 *out, int K, int C, int R, int S, int Cp,
                            cudaStream_t s);

// ---- tcgen05 implicit-GEMM convolution / GEMM --------------------------------
struct TcConvArgs {
  const bf16 *x;         // A operand: NHWC bf16 [N][H][W][C] (or folded rows, see w_step)
  const bf16 *w;         // B operand: packed [T][K][Cf]
  const float *bias;     // [K] or null
  const bf16 *residual;  // NHWC bf16 like the output, or null
  bf16 *y;               // NHWC bf16 [N][P][Q][K]      (when out_f32 == null)
  float *out_f32;        // fp32 output (else null): row-major [N*P*Q][ldo] (GEMM head) ...
  int ldo;
  int out_nchw;          // ... or, when set, the NCHW tensor [N][K][P][Q] itself
  int split;             // fp32 operands as bf16 parts: x points at three planes (hi, mid, lo) of
                         // N*H*W*Cf elements each, w holds six parts per tap (launch_pack_krsc_split)
  int N, H, W, Cf;       // A tensor dims (W already = Q for the folded form)
  int K, P, Q;
  int R, S;              // taps looped over (S = 1 for the folded form)
  int pad_h, pad_w, stride_h, stride_w;  // stride_w = 1, pad_w = 0 for the folded form
  int act;
  float lo, hi;
  // Folded form only (else 0): elements between the A vectors of neighbouring output
  // columns, and elements per input row; the vectors overlap when w_step < Cf.
  int w_step, row_elems;
  int f16;               // operands and bf16-typed pointers hold fp16 (else bf16)
  // Filter (and bias) were resident on the device before this call was made, i.e. no work
  // enqueued earlier in the stream produces them.
  int consts_ready;
};
// ---- few-channel convolution fused with the 3x3 / stride 2 / pad 1 max pool after it -----
struct StemPoolArgs {
  const bf16 *x;      // padded channels-last rows [N][H][row_bytes / 2] (launch_pad_input_bf16)
  const bf16 *w;      // launch_pack_stem_bf16 layout
  const float *bias;  // [K] or null
  bf16 *y;            // pooled output, NHWC bf16 [N][PP][QP][K]
  int N, H, row_bytes, w_step_bytes;
  int P, Q, K;        // convolution output rows / columns / channels
  int R, Cf;          // filter rows, Sp*Cp folded channels
  int pad_h, stride_h;
  int PP, QP;         // pooled rows / columns
  float lo, hi;       // clamp applied before the pool
};
bool stem_pool_supported(const StemPoolArgs &a);
size_t stem_pool_weight_bytes(int R, int Cf);
// fp32 KCRS (C <= Cp) -> the weight layout of the fused kernel
void launch_pack_stem_bf16(const float *w, bf16 *out, int C, int R, int S, int Cp, int Cf,
                           cudaStream_t s);
bool launch_stem_pool(const StemPoolArgs &a, int *err_word, int num_sms, cudaStream_t s);

// Enqueues a one-thread kernel whose bounded mbarrier wait must run out (see conv_tc.cu).
void launch_selftest_bounded_wait(cudaStream_t s);

// Returns false when the shape is outside what the kernel supports (caller falls back).
bool tc_conv_supported(const TcConvArgs &a);
void launch_tc_conv(const TcConvArgs &a, cudaStream_t s);
// Same kernel, no runtime state, no caches, no allocation; false when the plan fails.
bool launch_tc_conv_stateless(const TcConvArgs &a, int *err_word, int num_sms, cudaStream_t s);

}  // namespace occ
