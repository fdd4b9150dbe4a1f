/*
 * CPU oracle for the Occamy DNN operator runtime -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic each hot-path runtime symbol of the
 * reference (corelab-src/occamy, src/Tools/dnn-wrapper) must produce, written
 * as straightforward loop nests over fp32 NCHW data.  It is the checker the GPU
 * kernels are compared against and the timed CPU baseline; nothing the product
 * ships may call into it.
 *
 * PARITY UNPINNED: the reference holds no golden vectors, known-answer tests or
 * fixtures for this path (its tests compare live against onnxruntime/PyTorch
 * with downloaded weights), and its CPU lowering lives in the un-vendored
 * onnx-mlir submodule, which cannot be built offline.  The restatement is
 * therefore pinned only against an independent implementation of the same ONNX
 * operator semantics (torch.nn.functional on CPU) by the CPU test-suite.
 *
 * Every function cites the reference file:line whose semantics it follows.
 * Accumulation is fp32 in (c, r, s) order, vectorised only across independent
 * outputs, compiled with -ffp-contract=off so results are bit-reproducible
 * across x86-64 hosts.  The *_f64 variants accumulate in double and bound the
 * oracle's own rounding error.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define OCC_ACT_SIGMOID 0
#define OCC_ACT_RELU 1
#define OCC_ACT_TANH 2
#define OCC_ACT_CLIPPED_RELU 3
#define OCC_ACT_IDENTITY 5

static inline float apply_act(float v, int mode, float lo, float hi) {
  /* cudnn/CUDNNActiveFunc.cpp:37-62 (mode passed straight to cuDNN: 0 sigmoid,
   * 1 ReLU, 2 tanh, NaN-propagating); fusedOp/CUDNNConvBiasReluFunc.cpp:62-68
   * (1 ReLU, 5 identity).  Mode 3 (clipped ReLU with [lo, hi]) is the fused
   * form of cuda/CUDAClipFunc.cu:5-11. */
  switch (mode) {
  case OCC_ACT_SIGMOID: return 1.0f / (1.0f + expf(-v));
  case OCC_ACT_RELU: return v != v ? v : (v > 0.0f ? v : 0.0f);
  case OCC_ACT_TANH: return tanhf(v);
  case OCC_ACT_CLIPPED_RELU: return fminf(fmaxf(v, lo), hi);
  default: return v;
  }
}

/* y = act(x (*) w + b).  NCHW input, KCRS filter, cross-correlation, dilation
 * 1, symmetric zero padding, floor output size, `groups` channel groups.
 * Follows cudnn/CUDNNConvFunc.cpp:48-82 (geometry, groups) and
 * cudnn/fusedOp/CUDNNConvBiasReluFunc.cpp:70-112 (bias [1,K,1,1] + activation);
 * output size per ONNXToDNN/Ops/cudnn/Conv.cpp:40-57.  bias may be NULL. */
void occ_conv2d(const float *x, const float *w, const float *bias, float *y,
                int64_t N, int64_t C, int64_t H, int64_t W, int64_t K,
                int64_t R, int64_t S, int64_t groups, int64_t pad_h,
                int64_t pad_w, int64_t stride_h, int64_t stride_w, int act,
                float lo, float hi) {
  const int64_t P = (H + 2 * pad_h - R) / stride_h + 1;
  const int64_t Q = (W + 2 * pad_w - S) / stride_w + 1;
  const int64_t Cg = C / groups, Kg = K / groups;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t k = 0; k < K; ++k) {
      const int64_t g = k / Kg;
      float *yk = y + (n * K + k) * P * Q;
      for (int64_t i = 0; i < P * Q; ++i) yk[i] = 0.0f;
      for (int64_t c = 0; c < Cg; ++c) {
        const float *xc = x + (n * C + g * Cg + c) * H * W;
        for (int64_t r = 0; r < R; ++r)
          for (int64_t s = 0; s < S; ++s) {
            const float wv = w[((k * Cg + c) * R + r) * S + s];
            for (int64_t p = 0; p < P; ++p) {
              const int64_t h = p * stride_h - pad_h + r;
              if (h < 0 || h >= H) continue;
              /* valid q range: 0 <= q*stride_w - pad_w + s < W */
              int64_t q0 = 0, q1 = Q;
              const int64_t off = s - pad_w;
              if (off < 0) q0 = (-off + stride_w - 1) / stride_w;
              const int64_t lim = W - off; /* q*stride_w < lim */
              const int64_t qmax = (lim + stride_w - 1) / stride_w;
              if (qmax < q1) q1 = qmax;
              const float *xr = xc + h * W + off;
              float *yr = yk + p * Q;
              for (int64_t q = q0; q < q1; ++q) yr[q] += wv * xr[q * stride_w];
            }
          }
      }
      const float b = bias ? bias[k] : 0.0f;
      for (int64_t i = 0; i < P * Q; ++i) yk[i] = apply_act(yk[i] + b, act, lo, hi);
    }
}

/* Same operator, double accumulation: bounds the fp32 oracle's own rounding. */
void occ_conv2d_f64(const float *x, const float *w, const float *bias, float *y,
                    int64_t N, int64_t C, int64_t H, int64_t W, int64_t K,
                    int64_t R, int64_t S, int64_t groups, int64_t pad_h,
                    int64_t pad_w, int64_t stride_h, int64_t stride_w, int act,
                    float lo, float hi) {
  const int64_t P = (H + 2 * pad_h - R) / stride_h + 1;
  const int64_t Q = (W + 2 * pad_w - S) / stride_w + 1;
  const int64_t Cg = C / groups, Kg = K / groups;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t k = 0; k < K; ++k) {
      const int64_t g = k / Kg;
      for (int64_t p = 0; p < P; ++p)
        for (int64_t q = 0; q < Q; ++q) {
          double acc = 0.0;
          for (int64_t c = 0; c < Cg; ++c)
            for (int64_t r = 0; r < R; ++r) {
              const int64_t h = p * stride_h - pad_h + r;
              if (h < 0 || h >= H) continue;
              for (int64_t s = 0; s < S; ++s) {
                const int64_t ww = q * stride_w - pad_w + s;
                if (ww < 0 || ww >= W) continue;
                acc += (double)x[((n * C + g * Cg + c) * H + h) * W + ww] *
                       (double)w[((k * Cg + c) * R + r) * S + s];
              }
            }
          acc += bias ? (double)bias[k] : 0.0;
          y[((n * K + k) * P + p) * Q + q] = apply_act((float)acc, act, lo, hi);
        }
    }
}

/* out = A op (biasB * B); op 0 add, 1 mul, 4 sqrt(A).  B is broadcast along every
 * dimension where its extent is 1; ranks are equal (the lowering pads B's shape
 * with leading 1s, ONNXToDNN/Ops/cudnn/Conv.cpp:118-147).  Follows
 * cudnn/CUDNNTensorOpFunc.cpp:102-124 (alpha1 = 1, alpha2 = biasB, beta = 0). */
void occ_tensor_op(int64_t mode, const float *A, const int64_t *dimA,
                   const float *B, const int64_t *dimB, float *out, int rank,
                   float biasB) {
  int64_t total = 1, strideB[8], sb = 1;
  for (int i = 0; i < rank; ++i) total *= dimA[i];
  for (int i = rank - 1; i >= 0; --i) {
    strideB[i] = dimB[i] == 1 ? 0 : sb;
    sb *= dimB[i];
  }
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < total; ++i) {
    int64_t rem = i, ib = 0;
    for (int d = rank - 1; d >= 0; --d) {
      ib += (rem % dimA[d]) * strideB[d];
      rem /= dimA[d];
    }
    const float a = A[i];
    if (mode == 0) out[i] = a + biasB * B[ib];
    else if (mode == 1) out[i] = a * (biasB * B[ib]);
    else out[i] = sqrtf(a);
  }
}

/* y = act(x) elementwise.  cudnn/CUDNNActiveFunc.cpp:37-82. */
void occ_activation(const float *x, float *y, int64_t n, int mode) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = apply_act(x[i], mode, 0.0f, 0.0f);
}

/* y = min(max(x, lo), hi).  cuda/CUDAClipFunc.cu:5-11. */
void occ_clip(const float *x, float *y, int64_t n, float lo, float hi) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = fminf(fmaxf(x[i], lo), hi);
}

/* 2-D pooling over NCHW.  is_avg = 0: max pooling, padding never wins
 * (cudnn/CUDNNMaxPoolFunc.cpp:43-60).  is_avg = 1: average pooling; with
 * count_include_pad = 1 the divisor is always kh*kw, which is what the GPU
 * wrapper asks cuDNN for (cudnn/CUDNNAveragePoolFunc.cpp:43-48); 0 divides by
 * the number of in-range taps (the ONNX default the CPU lowering uses).  Only
 * the begin pads (pads[0], pads[2] of the ONNX attribute) reach the wrapper. */
void occ_pool2d(const float *x, float *y, int64_t N, int64_t C, int64_t H,
                int64_t W, int64_t P, int64_t Q, int64_t kh, int64_t kw,
                int64_t pad_h, int64_t pad_w, int64_t stride_h,
                int64_t stride_w, int is_avg, int count_include_pad) {
#pragma omp parallel for schedule(static)
  for (int64_t nc = 0; nc < N * C; ++nc) {
    const float *xc = x + nc * H * W;
    float *yc = y + nc * P * Q;
    for (int64_t p = 0; p < P; ++p)
      for (int64_t q = 0; q < Q; ++q) {
        float m = -INFINITY, sum = 0.0f;
        int64_t cnt = 0;
        for (int64_t r = 0; r < kh; ++r) {
          const int64_t h = p * stride_h - pad_h + r;
          if (h < 0 || h >= H) continue;
          for (int64_t s = 0; s < kw; ++s) {
            const int64_t ww = q * stride_w - pad_w + s;
            if (ww < 0 || ww >= W) continue;
            const float v = xc[h * W + ww];
            if (v > m || v != v) m = v;
            sum += v;
            ++cnt;
          }
        }
        if (is_avg) yc[p * Q + q] = sum / (float)(count_include_pad ? kh * kw : (cnt ? cnt : 1));
        else yc[p * Q + q] = m;
      }
  }
}

/* Mean over every axis whose output extent is 1 (keepdims).  Global average
 * pooling arrives here (ONNXToDNN/Ops/cudnn/ReduceMeanV13.cpp:37-77;
 * cudnn/CUDNNReduceFunc.cpp:60-125, CUDNN_REDUCE_TENSOR_AVG = mode 5). */
void occ_reduce_mean(const float *x, const int64_t *dimIn, float *y,
                     const int64_t *dimOut, int rank) {
  int64_t total_in = 1, total_out = 1, strideOut[8], so = 1;
  for (int i = 0; i < rank; ++i) { total_in *= dimIn[i]; total_out *= dimOut[i]; }
  for (int i = rank - 1; i >= 0; --i) {
    strideOut[i] = dimOut[i] == 1 && dimIn[i] != 1 ? 0 : so;
    so *= dimOut[i];
  }
  double *acc = (double *)calloc((size_t)total_out, sizeof(double));
  for (int64_t i = 0; i < total_in; ++i) {
    int64_t rem = i, io = 0;
    for (int d = rank - 1; d >= 0; --d) {
      io += (rem % dimIn[d]) * strideOut[d];
      rem /= dimIn[d];
    }
    acc[io] += (double)x[i];
  }
  const double cnt = (double)(total_in / total_out);
  for (int64_t i = 0; i < total_out; ++i) y[i] = (float)(acc[i] / cnt);
  free(acc);
}

/* out = alpha * op(A) * op(B) + beta * out, row-major 2-D.
 * cublas/CUBLASMatmul2dFunc.cu:57-123 (CUBLAS_COMPUTE_32F, C == out).  The Gemm
 * lowering then adds ONNX input C with weight 1 through the tensor-op symbol
 * (ONNXToDNN/Ops/cublas/Gemm.cpp:60-78).  dimA/dimB are the stored shapes. */
void occ_matmul2d(const float *A, const int64_t *dimA, const float *B,
                  const int64_t *dimB, float *out, float alpha, float beta,
                  int64_t transA, int64_t transB) {
  const int64_t M = transA ? dimA[1] : dimA[0];
  const int64_t Kd = transA ? dimA[0] : dimA[1];
  const int64_t Nn = transB ? dimB[0] : dimB[1];
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < Nn; ++n) {
      float acc = 0.0f;
      for (int64_t k = 0; k < Kd; ++k) {
        const float a = transA ? A[k * dimA[1] + m] : A[m * dimA[1] + k];
        const float b = transB ? B[n * dimB[1] + k] : B[k * dimB[1] + n];
        acc += a * b;
      }
      float *o = out + m * Nn + n;
      *o = alpha * acc + (beta != 0.0f ? beta * *o : 0.0f);
    }
}

/* Softmax along `axis`, shifted by the per-slice maximum.  The reference
 * subtracts the whole-tensor maximum instead (cuda/CUDASoftmaxFunc.cu:56-65),
 * which is the same function by shift invariance; cuda/CUDASoftmaxFunc.cu:7-36
 * for the indexing. */
void occ_softmax(const float *x, float *y, const int64_t *dim, int rank,
                 int64_t axis) {
  int64_t outer = 1, inner = 1;
  const int64_t len = dim[axis];
  for (int i = 0; i < axis; ++i) outer *= dim[i];
  for (int i = (int)axis + 1; i < rank; ++i) inner *= dim[i];
#pragma omp parallel for schedule(static)
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t in = 0; in < inner; ++in) {
      const float *xs = x + o * len * inner + in;
      float *ys = y + o * len * inner + in;
      float m = -INFINITY, sum = 0.0f;
      for (int64_t j = 0; j < len; ++j) m = fmaxf(m, xs[j * inner]);
      for (int64_t j = 0; j < len; ++j) {
        const float e = expf(xs[j * inner] - m);
        ys[j * inner] = e;
        sum += e;
      }
      for (int64_t j = 0; j < len; ++j) ys[j * inner] = ys[j * inner] / sum;
    }
}

/* Flatten / reshape: contiguous copy (cuda/CUDAFlattenFunc.cpp:24-32,
 * cuda/CUDAReshapeFunc.cpp:22-30). */
void occ_copy(const float *x, float *y, int64_t n) {
  memcpy(y, x, (size_t)n * sizeof(float));
}
