// fp32 kernels on the ABI's own layout (dense NCHW).  They serve OCCAMY_MATH=fp32
// (bit-for-bit the reference's data types, CUDA-core FMA, error <= 1e-4 against the CPU
// semantics) and every shape the tensor-core path does not take.
#include "kernels.h"
#include "runtime.h"

namespace occ {

__device__ __forceinline__ float act_apply(float v, int act, float lo, float hi) {
  switch (act) {
    case ACT_SIGMOID: return 1.0f / (1.0f + __expf(-v));
    case ACT_RELU: return v != v ? v : fmaxf(v, 0.0f);
    case ACT_TANH: return tanhf(v);
    case ACT_CLIP: return fminf(fmaxf(v, lo), hi);
    default: return v;
  }
}

static inline int grid_for(int64_t n, int threads, int per_thread = 1) {
  int64_t b = (n + (int64_t)threads * per_thread - 1) / ((int64_t)threads * per_thread);
  const int64_t cap = (int64_t)rt().num_sms * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

// ---------------------------------------------------------------------------
// Dense / grouped convolution as an implicit GEMM on CUDA cores.
// Per group: Y[k, m] = sum_j Wt[k, j] * im2col(X)[j, m],  j over (c, r, s), m over
// (n, p, q).  64x64 output tile per CTA, 16-deep reduction slices through shared memory,
// 4x4 outputs per thread.
// ---------------------------------------------------------------------------
constexpr int CT_M = 64, CT_N = 64, CT_K = 16;

__global__ void __launch_bounds__(256) conv_f32_kernel(const float *__restrict__ x,
                                                       const float *__restrict__ w,
                                                       const float *__restrict__ bias,
                                                       float *__restrict__ y, ConvGeom g) {
  __shared__ float sW[CT_K][CT_M + 4];
  __shared__ float sX[CT_K][CT_N + 4];
  const int Cg = g.C / g.groups, Kg = g.K / g.groups;
  const int CRS = Cg * g.R * g.S, RS = g.R * g.S;
  const int64_t PQ = (int64_t)g.P * g.Q, Mtot = (int64_t)g.N * PQ;
  const int grp = blockIdx.z;
  const int k0 = blockIdx.y * CT_M;
  const int64_t m0 = (int64_t)blockIdx.x * CT_N;
  const int t = threadIdx.x;
  const int tx = t % 16, ty = t / 16;

  // this thread's im2col column for the shared-memory fill: one pixel, 4 reduction rows
  const int fill_m = t % CT_N, fill_j = t / CT_N;  // j rows fill_j, +4, +8, +12
  const int64_t pm = m0 + fill_m;
  const bool pm_ok = pm < Mtot;
  int pn = 0, pp = 0, pq = 0;
  if (pm_ok) {
    pn = (int)(pm / PQ);
    const int rem = (int)(pm % PQ);
    pp = rem / g.Q;
    pq = rem % g.Q;
  }
  const int h0 = pp * g.stride_h - g.pad_h, w0 = pq * g.stride_w - g.pad_w;
  const float *xn = x + ((int64_t)pn * g.C + (int64_t)grp * Cg) * g.H * g.W;
  // weight fill: row = t / 4 (0..63), 4 consecutive j
  const int wrow = t / 4, wj = (t % 4) * 4;
  const int kglob_fill = k0 + wrow;
  const float *wk = w + ((int64_t)grp * Kg + kglob_fill) * CRS;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int j0 = 0; j0 < CRS; j0 += CT_K) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + wj + u;
      sW[wj + u][wrow] = (kglob_fill < Kg && j < CRS) ? wk[j] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int jj = fill_j + u * 4;
      const int j = j0 + jj;
      float v = 0.0f;
      if (pm_ok && j < CRS) {
        const int c = j / RS, rs = j % RS;
        const int r = rs / g.S, s2 = rs % g.S;
        const int h = h0 + r, ww = w0 + s2;
        if (h >= 0 && h < g.H && ww >= 0 && ww < g.W) v = xn[((int64_t)c * g.H + h) * g.W + ww];
      }
      sX[jj][fill_m] = v;
    }
    __syncthreads();
#pragma unroll
    for (int jj = 0; jj < CT_K; ++jj) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sW[jj][ty * 4 + i];
#pragma unroll
      for (int i = 0; i < 4; ++i) b[i] = sX[jj][tx * 4 + i];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int jx = 0; jx < 4; ++jx) acc[i][jx] = fmaf(a[i], b[jx], acc[i][jx]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int kl = k0 + ty * 4 + i;
    if (kl >= Kg) continue;
    const int kg = grp * Kg + kl;
    const float b = bias ? bias[kg] : 0.0f;
#pragma unroll
    for (int jx = 0; jx < 4; ++jx) {
      const int64_t m = m0 + tx * 4 + jx;
      if (m >= Mtot) continue;
      const int64_t n = m / PQ, rem = m % PQ;
      y[(n * g.K + kg) * PQ + rem] = act_apply(acc[i][jx] + b, g.act, g.lo, g.hi);
    }
  }
}

void launch_conv_f32(const float *x, const float *w, const float *bias, float *y,
                     const ConvGeom &g, cudaStream_t s) {
  const int Kg = g.K / g.groups;
  const int64_t Mtot = (int64_t)g.N * g.P * g.Q;
  dim3 grid((unsigned)((Mtot + CT_N - 1) / CT_N), (unsigned)((Kg + CT_M - 1) / CT_M),
            (unsigned)g.groups);
  conv_f32_kernel<<<grid, 256, 0, s>>>(x, w, bias, y, g);
  count(CNT_LAUNCHES);
  count(CNT_SIMT_LAUNCHES);
}

// Depthwise (groups == C == K): one thread per output element, q fastest so a warp reads
// and writes contiguous rows.
__global__ void depthwise_f32_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                     const float *__restrict__ bias, float *__restrict__ y,
                                     ConvGeom g, int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int q = (int)(i % g.Q);
    const int p = (int)((i / g.Q) % g.P);
    const int64_t nc = i / ((int64_t)g.P * g.Q);
    const int c = (int)(nc % g.C);
    const float *xc = x + nc * g.H * g.W;
    const float *wc = w + (int64_t)c * g.R * g.S;
    float acc = 0.0f;
    for (int r = 0; r < g.R; ++r) {
      const int h = p * g.stride_h - g.pad_h + r;
      if (h < 0 || h >= g.H) continue;
      for (int s2 = 0; s2 < g.S; ++s2) {
        const int ww = q * g.stride_w - g.pad_w + s2;
        if (ww < 0 || ww >= g.W) continue;
        acc = fmaf(xc[h * g.W + ww], wc[r * g.S + s2], acc);
      }
    }
    y[i] = act_apply(acc + (bias ? bias[c] : 0.0f), g.act, g.lo, g.hi);
  }
}

void launch_depthwise_f32(const float *x, const float *w, const float *bias, float *y,
                          const ConvGeom &g, cudaStream_t s) {
  const int64_t total = (int64_t)g.N * g.C * g.P * g.Q;
  depthwise_f32_kernel<<<grid_for(total, 256), 256, 0, s>>>(x, w, bias, y, g, total);
  count(CNT_LAUNCHES);
}

// ---------------------------------------------------------------------------
// Element-wise
// ---------------------------------------------------------------------------
struct Bcast {
  int rank;
  int64_t dimA[8];
  int64_t strideB[8];
};

__global__ void tensor_op_f32_kernel(int mode, const float *A,
                                     const float *B, float *out,
                                     Bcast bc, float biasB, int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, ib = 0;
    for (int d = bc.rank - 1; d >= 0; --d) {
      ib += (rem % bc.dimA[d]) * bc.strideB[d];
      rem /= bc.dimA[d];
    }
    const float a = A[i];
    float r;
    if (mode == 0) r = a + biasB * B[ib];
    else if (mode == 1) r = a * (biasB * B[ib]);
    else r = sqrtf(a);
    out[i] = r;
  }
}

// Same shape, no broadcast: 128-bit accesses.
__global__ void tensor_op_same_f32_kernel(int mode, const float4 *A,
                                          const float4 *B, float4 *out,
                                          float biasB, int64_t n4) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float4 a = A[i], b = B[i];
    float4 r;
    if (mode == 0) {
      r.x = a.x + biasB * b.x; r.y = a.y + biasB * b.y;
      r.z = a.z + biasB * b.z; r.w = a.w + biasB * b.w;
    } else if (mode == 1) {
      r.x = a.x * (biasB * b.x); r.y = a.y * (biasB * b.y);
      r.z = a.z * (biasB * b.z); r.w = a.w * (biasB * b.w);
    } else {
      r.x = sqrtf(a.x); r.y = sqrtf(a.y); r.z = sqrtf(a.z); r.w = sqrtf(a.w);
    }
    out[i] = r;
  }
}

// B = [1, C, 1, 1] added to A = [N, C, H, W]: one (n, c) plane per blockIdx.y.
__global__ void bias_plane_f32_kernel(int mode, const float *A,
                                      const float *B, float *out, int C,
                                      int64_t HW, float biasB) {
  const int64_t plane = blockIdx.x;
  const float b = biasB * B[plane % C];
  const float *a = A + plane * HW;
  float *o = out + plane * HW;
  for (int64_t i = blockIdx.y * (int64_t)blockDim.x + threadIdx.x; i < HW;
       i += (int64_t)gridDim.y * blockDim.x)
    o[i] = mode == 0 ? a[i] + b : a[i] * b;
}

void launch_tensor_op_f32(int mode, const float *A, const float *B, float *out, int rank,
                          const int64_t *dimA, const int64_t *dimB, float biasB, cudaStream_t s) {
  int64_t total = 1;
  bool same = true;
  for (int i = 0; i < rank; ++i) {
    total *= dimA[i];
    if (dimA[i] != dimB[i]) same = false;
  }
  if (total == 0) return;
  const bool aligned = (((uintptr_t)A | (uintptr_t)B | (uintptr_t)out) & 15) == 0;
  if ((same || mode == 4) && aligned && total % 4 == 0) {
    tensor_op_same_f32_kernel<<<grid_for(total / 4, 256, 2), 256, 0, s>>>(
        mode, (const float4 *)A, (const float4 *)(mode == 4 ? A : B), (float4 *)out, biasB,
        total / 4);
  } else if (mode != 4 && rank == 4 && dimB[0] == 1 && dimB[2] == 1 && dimB[3] == 1 &&
             dimB[1] == dimA[1] && dimA[2] * dimA[3] < 65535 * 1024) {
    const int64_t HW = dimA[2] * dimA[3];
    dim3 grid((unsigned)(dimA[0] * dimA[1]), (unsigned)((HW + 1023) / 1024));
    bias_plane_f32_kernel<<<grid, 256, 0, s>>>(mode, A, B, out, (int)dimA[1], HW, biasB);
  } else {
    Bcast bc;
    bc.rank = rank;
    int64_t sb = 1;
    for (int i = rank - 1; i >= 0; --i) {
      bc.dimA[i] = dimA[i];
      bc.strideB[i] = dimB[i] == 1 ? 0 : sb;
      sb *= dimB[i];
    }
    tensor_op_f32_kernel<<<grid_for(total, 256), 256, 0, s>>>(mode, A, mode == 4 ? A : B, out, bc,
                                                               biasB, total);
  }
  count(CNT_LAUNCHES);
}

__global__ void act_f32_kernel(const float *x, float *y, int64_t n,
                               int act, float lo, float hi) {
  const int64_t n4 = n / 4;
  const float4 *x4 = (const float4 *)x;
  float4 *y4 = (float4 *)y;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 v = x4[i];
    v.x = act_apply(v.x, act, lo, hi); v.y = act_apply(v.y, act, lo, hi);
    v.z = act_apply(v.z, act, lo, hi); v.w = act_apply(v.w, act, lo, hi);
    y4[i] = v;
  }
  for (int64_t i = n4 * 4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    y[i] = act_apply(x[i], act, lo, hi);
}

__global__ void act_f32_scalar_kernel(const float *x, float *y,
                                      int64_t n, int act, float lo, float hi) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    y[i] = act_apply(x[i], act, lo, hi);
}

void launch_act_f32(const float *x, float *y, int64_t n, int act, float lo, float hi,
                    cudaStream_t s) {
  if (n == 0) return;
  if ((((uintptr_t)x | (uintptr_t)y) & 15) == 0)
    act_f32_kernel<<<grid_for(n / 4 + 1, 256, 2), 256, 0, s>>>(x, y, n, act, lo, hi);
  else
    act_f32_scalar_kernel<<<grid_for(n, 256), 256, 0, s>>>(x, y, n, act, lo, hi);
  count(CNT_LAUNCHES);
}

// ---------------------------------------------------------------------------
// Pooling (NCHW): one thread per output, q fastest.
// ---------------------------------------------------------------------------
__global__ void pool_f32_kernel(const float *__restrict__ x, float *__restrict__ y, int H, int W,
                                int P, int Q, int kh, int kw, int pad_h, int pad_w, int sh,
                                int sw, bool avg, int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int q = (int)(i % Q);
    const int p = (int)((i / Q) % P);
    const int64_t nc = i / ((int64_t)P * Q);
    const float *xc = x + nc * H * W;
    float m = -INFINITY, sum = 0.0f;
    for (int r = 0; r < kh; ++r) {
      const int h = p * sh - pad_h + r;
      if (h < 0 || h >= H) continue;
      for (int s2 = 0; s2 < kw; ++s2) {
        const int ww = q * sw - pad_w + s2;
        if (ww < 0 || ww >= W) continue;
        const float v = xc[h * W + ww];
        if (v > m || v != v) m = v;
        sum += v;
      }
    }
    y[i] = avg ? sum / (float)(kh * kw) : m;
  }
}

void launch_pool_f32(const float *x, float *y, int N, int C, int H, int W, int P, int Q, int kh,
                     int kw, int pad_h, int pad_w, int sh, int sw, bool avg, cudaStream_t s) {
  const int64_t total = (int64_t)N * C * P * Q;
  if (total == 0) return;
  pool_f32_kernel<<<grid_for(total, 256), 256, 0, s>>>(x, y, H, W, P, Q, kh, kw, pad_h, pad_w, sh,
                                                       sw, avg, total);
  count(CNT_LAUNCHES);
}

// ---------------------------------------------------------------------------
// Mean over a set of axes: one warp per output element, lanes stride over the reduced
// index space (contiguous for the global-average-pool case), shuffle reduction.
// ---------------------------------------------------------------------------
struct ReduceShape {
  int nk, nr;            // number of kept / reduced axes
  int64_t kdim[8], kstride[8];
  int64_t rdim[8], rstride[8];
};

__global__ void reduce_mean_f32_kernel(const float *__restrict__ x, float *__restrict__ y,
                                       ReduceShape rs, int64_t n_out, int64_t n_red) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t o = warp; o < n_out; o += nwarps) {
    int64_t rem = o, base = 0;
    for (int d = rs.nk - 1; d >= 0; --d) {
      base += (rem % rs.kdim[d]) * rs.kstride[d];
      rem /= rs.kdim[d];
    }
    float acc = 0.0f;
    for (int64_t r = lane; r < n_red; r += 32) {
      int64_t rr = r, off = 0;
      for (int d = rs.nr - 1; d >= 0; --d) {
        off += (rr % rs.rdim[d]) * rs.rstride[d];
        rr /= rs.rdim[d];
      }
      acc += x[base + off];
    }
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sft);
    if (lane == 0) y[o] = acc / (float)n_red;
  }
}

void launch_reduce_mean_f32(const float *x, float *y, int rank, const int64_t *dimIn,
                            const int64_t *dimOut, cudaStream_t s) {
  ReduceShape rs;
  rs.nk = rs.nr = 0;
  int64_t stride = 1, n_out = 1, n_red = 1;
  int64_t strides[8];
  for (int i = rank - 1; i >= 0; --i) {
    strides[i] = stride;
    stride *= dimIn[i];
  }
  for (int i = 0; i < rank; ++i) {
    if (dimOut[i] == 1 && dimIn[i] != 1) {
      rs.rdim[rs.nr] = dimIn[i];
      rs.rstride[rs.nr++] = strides[i];
      n_red *= dimIn[i];
    } else {
      rs.kdim[rs.nk] = dimIn[i];
      rs.kstride[rs.nk++] = strides[i];
      n_out *= dimIn[i];
    }
  }
  if (n_out == 0) return;
  reduce_mean_f32_kernel<<<grid_for(n_out * 32, 256), 256, 0, s>>>(x, y, rs, n_out, n_red);
  count(CNT_LAUNCHES);
}

// ---------------------------------------------------------------------------
// GEMM on CUDA cores: 64x64 tile, 16-deep slices, 4x4 per thread, strided operands.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float *__restrict__ A,
                                                       const float *__restrict__ B,
                                                       float *__restrict__ out, int M, int N,
                                                       int K, int64_t sam, int64_t sak,
                                                       int64_t sbk, int64_t sbn, float alpha,
                                                       float beta) {
  __shared__ float sA[CT_K][CT_M + 4];
  __shared__ float sB[CT_K][CT_N + 4];
  const int t = threadIdx.x, tx = t % 16, ty = t / 16;
  const int m0 = blockIdx.y * CT_M, n0 = blockIdx.x * CT_N;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int kk0 = 0; kk0 < K; kk0 += CT_K) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int idx = t + u * 256;       // 0..1023 over 64 x 16
      const int row = idx / CT_K, kk = idx % CT_K;
      const int m = m0 + row, k = kk0 + kk;
      sA[kk][row] = (m < M && k < K) ? A[m * sam + k * sak] : 0.0f;
      const int n = n0 + row;
      sB[kk][row] = (n < N && k < K) ? B[k * sbk + n * sbn] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < CT_K; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
      for (int i = 0; i < 4; ++i) b[i] = sB[kk][tx * 4 + i];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float *o = out + (int64_t)m * N + n;
      *o = alpha * acc[i][j] + (beta != 0.0f ? beta * *o : 0.0f);
    }
  }
}

void launch_gemm_f32(const float *A, const float *B, float *out, int M, int N, int K, int lda,
                     int ldb, float alpha, float beta, bool transA, bool transB, cudaStream_t s) {
  if (M == 0 || N == 0) return;
  const int64_t sam = transA ? 1 : lda, sak = transA ? lda : 1;
  const int64_t sbk = transB ? 1 : ldb, sbn = transB ? ldb : 1;
  dim3 grid((N + CT_N - 1) / CT_N, (M + CT_M - 1) / CT_M);
  gemm_f32_kernel<<<grid, 256, 0, s>>>(A, B, out, M, N, K, sam, sak, sbk, sbn, alpha, beta);
  count(CNT_LAUNCHES);
  count(CNT_SIMT_LAUNCHES);
}

// ---------------------------------------------------------------------------
// Softmax along one axis: one CTA per (outer, inner) slice; three strided passes with
// warp-shuffle + shared-memory reductions (max, sum of exp, normalise).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float block_reduce(float v, bool is_max, float *sh) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int sft = 16; sft > 0; sft >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, v, sft);
    v = is_max ? fmaxf(v, o) : v + o;
  }
  __syncthreads();
  if (lane == 0) sh[wid] = v;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  float r = is_max ? -INFINITY : 0.0f;
  for (int i = 0; i < nw; ++i) r = is_max ? fmaxf(r, sh[i]) : r + sh[i];
  return r;
}

__global__ void softmax_f32_kernel(const float *x, float *y,
                                   int64_t len, int64_t inner) {
  __shared__ float sh[32];
  const int64_t slice = blockIdx.x;
  const int64_t base = (slice / inner) * len * inner + slice % inner;
  const float *xs = x + base;
  float *ys = y + base;
  float m = -INFINITY;
  for (int64_t j = threadIdx.x; j < len; j += blockDim.x) m = fmaxf(m, xs[j * inner]);
  m = block_reduce(m, true, sh);
  float sum = 0.0f;
  for (int64_t j = threadIdx.x; j < len; j += blockDim.x) sum += expf(xs[j * inner] - m);
  sum = block_reduce(sum, false, sh);
  for (int64_t j = threadIdx.x; j < len; j += blockDim.x)
    ys[j * inner] = expf(xs[j * inner] - m) / sum;
}

void launch_softmax_f32(const float *x, float *y, int64_t outer, int64_t len, int64_t inner,
                        cudaStream_t s) {
  if (outer * inner == 0) return;
  softmax_f32_kernel<<<(unsigned)(outer * inner), 128, 0, s>>>(x, y, len, inner);
  count(CNT_LAUNCHES);
}

}  // namespace occ
