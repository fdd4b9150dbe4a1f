// Kernels on the tensor-core modes' activation format: 16-bit elements (bf16 or fp16, the
// template parameter F16 says which), NHWC, C a multiple of 8 so that every thread moves 128
// bits (8 channels) per access.  All are HBM-bound; they are written so that consecutive
// threads touch consecutive 16-byte channel groups.  Pointers to either element type travel
// as `bf16 *`; the launchers' `f16` argument names the type behind them.
#include <cuda_fp16.h>

#include <cstring>

#include "kernels.h"
#include "runtime.h"

namespace occ {

__device__ __forceinline__ float act_apply_b(float v, int act, float lo, float hi) {
  switch (act) {
    case ACT_SIGMOID: return 1.0f / (1.0f + __expf(-v));
    case ACT_RELU: return v != v ? v : fmaxf(v, 0.0f);
    case ACT_TANH: return tanhf(v);
    case ACT_CLIP: return fminf(fmaxf(v, lo), hi);
    default: return v;
  }
}

static inline int grid_for(int64_t n, int threads) {
  int64_t b = (n + threads - 1) / threads;
  const int64_t cap = (int64_t)rt().num_sms * 64;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

// ---- conversions between fp32 and the two 16-bit element types ----------------------
// A pair of 16-bit values in one 32-bit word, first element in the low half.
template <bool F16>
__device__ __forceinline__ float2 pair_to_f32(uint32_t v) {
  if constexpr (F16) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&v));
  } else {   // a bf16 is the top half of the fp32 of its value
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
  }
}
template <bool F16>
__device__ __forceinline__ uint32_t f32_to_pair(float a, float b) {
  uint32_t r;
  if constexpr (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
// the same with negative values clamped to zero by the conversion itself
template <bool F16>
__device__ __forceinline__ uint32_t f32_to_pair_relu(float a, float b) {
  uint32_t r;
  if constexpr (F16) asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  else asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
template <bool F16>
__device__ __forceinline__ uint32_t pair_max_nan(uint32_t a, uint32_t b) {
  uint32_t r;
  if constexpr (F16) asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  else asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <bool F16>
__device__ __forceinline__ uint32_t pair_min(uint32_t a, uint32_t b) {
  uint32_t r;
  if constexpr (F16) asm("min.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  else asm("min.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
template <bool F16>
__device__ __forceinline__ uint16_t f32_to_elem(float v) {
  if constexpr (F16) return __half_as_ushort(__float2half_rn(v));
  else return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
template <bool F16>
__device__ __forceinline__ float elem_to_f32(uint16_t v) {
  if constexpr (F16) return __half2float(__ushort_as_half(v));
  else return __uint_as_float((uint32_t)v << 16);
}
// host side: the bits of `v` rounded to the element type, and back
static uint16_t host_elem_bits(float v, bool f16) {
  if (f16) {
    const __half h = __float2half_rn(v);
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
  }
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  uint16_t b;
  memcpy(&b, &h, 2);
  return b;
}
static float host_elem_value(uint16_t bits, bool f16) {
  if (f16) {
    __half h;
    memcpy(&h, &bits, 2);
    return __half2float(h);
  }
  __nv_bfloat16 h;
  memcpy(&h, &bits, 2);
  return __bfloat162float(h);
}

// Eight 16-bit values moved as one 16-byte word: the copy operations go through the uint4
// member, so a load or store is a single 128-bit access (a member-wise copy of the four pairs
// compiles to four 32-bit accesses, which costs four times the L1 wavefronts).
struct alignas(16) bf16x8 {
  union {
    uint4 u;
    uint32_t v[4];
  };
  __device__ __forceinline__ bf16x8() {}
  __device__ __forceinline__ bf16x8(const bf16x8 &o) : u(o.u) {}
  __device__ __forceinline__ bf16x8 &operator=(const bf16x8 &o) {
    u = o.u;
    return *this;
  }
};

template <bool F16>
__device__ __forceinline__ void unpack8(const bf16x8 &p, float *f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = pair_to_f32<F16>(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <bool F16>
__device__ __forceinline__ bf16x8 pack8(const float *f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = f32_to_pair<F16>(f[2 * i], f[2 * i + 1]);
  return p;
}

// ---------------------------------------------------------------------------
// Layout conversion, per image: [C][HW] fp32 <-> [HW][C] bf16 through a 32x32 tile.
// ---------------------------------------------------------------------------
template <bool F16>
__global__ void nchw_to_nhwc_kernel(const float *__restrict__ x, uint16_t *__restrict__ y, int C,
                                    int HW) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 32;
  const float *xn = x + (int64_t)n * C * HW;
  uint16_t *yn = y + (int64_t)n * C * HW;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, p = p0 + threadIdx.x;
    tile[i][threadIdx.x] = (c < C && p < HW) ? xn[(int64_t)c * HW + p] : 0.0f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int p = p0 + i, c = c0 + threadIdx.x;
    if (p < HW && c < C) yn[(int64_t)p * C + c] = f32_to_elem<F16>(tile[threadIdx.x][i]);
  }
}

template <bool F16>
__global__ void nhwc_to_nchw_kernel(const uint16_t *__restrict__ x, float *__restrict__ y, int C,
                                    int HW) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 32;
  const uint16_t *xn = x + (int64_t)n * C * HW;
  float *yn = y + (int64_t)n * C * HW;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int p = p0 + i, c = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (p < HW && c < C) ? elem_to_f32<F16>(xn[(int64_t)p * C + c]) : 0.0f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, p = p0 + threadIdx.x;
    if (c < C && p < HW) yn[(int64_t)c * HW + p] = tile[threadIdx.x][i];
  }
}

void launch_nchw_f32_to_nhwc_bf16(const float *x, bf16 *y, int N, int C, int H, int W, bool f16,
                                  cudaStream_t s) {
  const int HW = H * W;
  if ((int64_t)N * C * HW == 0) return;
  dim3 grid((HW + 31) / 32, (C + 31) / 32, N), block(32, 8);
  if (f16) nchw_to_nhwc_kernel<true><<<grid, block, 0, s>>>(x, (uint16_t *)y, C, HW);
  else nchw_to_nhwc_kernel<false><<<grid, block, 0, s>>>(x, (uint16_t *)y, C, HW);
  count(CNT_LAUNCHES);
}

void launch_nhwc_bf16_to_nchw_f32(const bf16 *x, float *y, int N, int C, int H, int W, bool f16,
                                  cudaStream_t s) {
  const int HW = H * W;
  if ((int64_t)N * C * HW == 0) return;
  dim3 grid((HW + 31) / 32, (C + 31) / 32, N), block(32, 8);
  if (f16) nhwc_to_nchw_kernel<true><<<grid, block, 0, s>>>((const uint16_t *)x, y, C, HW);
  else nhwc_to_nchw_kernel<false><<<grid, block, 0, s>>>((const uint16_t *)x, y, C, HW);
  count(CNT_LAUNCHES);
}

template <bool F16>
__global__ void f32_to_bf16_kernel(const float *__restrict__ x, uint16_t *__restrict__ y, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    y[i] = f32_to_elem<F16>(x[i]);
}

void launch_f32_to_bf16(const float *x, bf16 *y, int64_t n, bool f16, cudaStream_t s) {
  if (n == 0) return;
  if (f16) f32_to_bf16_kernel<true><<<grid_for(n, 256), 256, 0, s>>>(x, (uint16_t *)y, n);
  else f32_to_bf16_kernel<false><<<grid_for(n, 256), 256, 0, s>>>(x, (uint16_t *)y, n);
  count(CNT_LAUNCHES);
}

// ---------------------------------------------------------------------------
// out = act(a + b + bias[c]);  b and bias optional.  8 channels per thread.
// ---------------------------------------------------------------------------
template <bool F16>
__global__ void add_act_bf16_kernel(const bf16x8 *a, const bf16x8 *b, const float *bias_c, int C8,
                                    bf16x8 *out, int64_t n8, int act, float lo, float hi) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8;
       i += (int64_t)gridDim.x * blockDim.x) {
    float f[8], g2[8];
    unpack8<F16>(a[i], f);
    if (b) {
      unpack8<F16>(b[i], g2);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] += g2[k];
    }
    if (bias_c) {
      const float4 *bp = (const float4 *)(bias_c + (i % C8) * 8);
      const float4 b0 = bp[0], b1 = bp[1];
      f[0] += b0.x; f[1] += b0.y; f[2] += b0.z; f[3] += b0.w;
      f[4] += b1.x; f[5] += b1.y; f[6] += b1.z; f[7] += b1.w;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = act_apply_b(f[k], act, lo, hi);
    out[i] = pack8<F16>(f);
  }
}

void launch_add_act_bf16(const bf16 *a, const bf16 *b, const float *bias_c, int C, bf16 *out,
                         int64_t n, int act, float lo, float hi, bool f16, cudaStream_t s) {
  if (n == 0) return;
  if (f16)
    add_act_bf16_kernel<true><<<grid_for(n / 8, 256), 256, 0, s>>>(
        (const bf16x8 *)a, (const bf16x8 *)b, bias_c, C / 8, (bf16x8 *)out, n / 8, act, lo, hi);
  else
    add_act_bf16_kernel<false><<<grid_for(n / 8, 256), 256, 0, s>>>(
        (const bf16x8 *)a, (const bf16x8 *)b, bias_c, C / 8, (bf16x8 *)out, n / 8, act, lo, hi);
  count(CNT_LAUNCHES);
}

// ---------------------------------------------------------------------------
// Pooling on NHWC: one thread per (n, p, q, 8 channels); consecutive threads take
// consecutive channel groups, so every access of a warp is one contiguous run.
// ---------------------------------------------------------------------------
template <bool AVG, bool F16>
__global__ void __launch_bounds__(256) pool_bf16_kernel(const bf16x8 *__restrict__ x,
                                                        bf16x8 *__restrict__ y, int C8, int H,
                                                        int W, int P, int Q, int kh, int kw,
                                                        int pad_h, int pad_w, int sh, int sw,
                                                        int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c8 = (int)(i % C8);
    int64_t rest = i / C8;
    const int q = (int)(rest % Q);
    rest /= Q;
    const int p = (int)(rest % P);
    const int64_t n = rest / P;
    const int h0 = max(p * sh - pad_h, 0), h1 = min(p * sh - pad_h + kh, H);
    const int w0 = max(q * sw - pad_w, 0), w1 = min(q * sw - pad_w + kw, W);
    if (AVG) {
      float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int h = h0; h < h1; ++h)
        for (int ww = w0; ww < w1; ++ww) {
          float f[8];
          unpack8<F16>(x[((n * H + h) * W + ww) * C8 + c8], f);
#pragma unroll
          for (int k = 0; k < 8; ++k) sum[k] += f[k];
        }
      const float inv = 1.0f / (float)(kh * kw);
#pragma unroll
      for (int k = 0; k < 8; ++k) sum[k] *= inv;
      y[i] = pack8<F16>(sum);
    } else {
      // max of 16-bit pairs directly (NaN-propagating), no conversion round trip
      const uint32_t ninf = f32_to_pair<F16>(-INFINITY, -INFINITY);
      bf16x8 m;
#pragma unroll
      for (int k = 0; k < 4; ++k) m.v[k] = ninf;
      for (int h = h0; h < h1; ++h)
        for (int ww = w0; ww < w1; ++ww) {
          const bf16x8 v = x[((n * H + h) * W + ww) * C8 + c8];
#pragma unroll
          for (int k = 0; k < 4; ++k) m.v[k] = pair_max_nan<F16>(m.v[k], v.v[k]);
        }
      y[i] = m;
    }
  }
}

// Pooling with a compile-time square window K and stride S: one thread per (n, p, q, 8 channels).
// All K*K 16-byte loads of a thread are issued before the first is used: their addresses are
// clamped into the image instead of being skipped (a clamped element lies inside the window, so the
// maximum is unchanged; the average masks it to zero), which leaves no branch between the loads.
// Neighbouring windows overlap in the L1.  The grid is (chunks of one image's outputs) x images, so
// a thread needs two short divisions only.
template <int K, int S, bool AVG, bool F16>
__global__ void __launch_bounds__(256) pool_win_bf16_kernel(const bf16x8 *__restrict__ x,
                                                            bf16x8 *__restrict__ y, int C8, int H,
                                                            int W, int Q, int pad_h, int pad_w,
                                                            unsigned per_image, unsigned chunks) {
  const unsigned n = blockIdx.x / chunks;
  const unsigned j = (blockIdx.x - n * chunks) * 256u + threadIdx.x;
  if (j >= per_image) return;
  const unsigned pq = j / (unsigned)C8;
  const int c8 = (int)(j - pq * (unsigned)C8);
  const int p = (int)(pq / (unsigned)Q), q = (int)(pq - (unsigned)p * (unsigned)Q);
  const bf16x8 *xin = x + (int64_t)n * H * W * C8 + c8;
  const int h0 = p * S - pad_h, w0 = q * S - pad_w;
  bf16x8 v[K][K];
#pragma unroll
  for (int r = 0; r < K; ++r) {
    const int h = min(max(h0 + r, 0), H - 1);
#pragma unroll
    for (int c = 0; c < K; ++c) {
      const int w = min(max(w0 + c, 0), W - 1);
      v[r][c] = xin[((int64_t)h * W + w) * C8];
    }
  }
  bf16x8 out;
  if (AVG) {
    float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int r = 0; r < K; ++r)
#pragma unroll
      for (int c = 0; c < K; ++c) {
        const bool in = (unsigned)(h0 + r) < (unsigned)H && (unsigned)(w0 + c) < (unsigned)W;
        float f[8];
        unpack8<F16>(v[r][c], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) sum[k] += in ? f[k] : 0.0f;
      }
#pragma unroll
    for (int k = 0; k < 8; ++k) sum[k] *= 1.0f / (float)(K * K);
    out = pack8<F16>(sum);
  } else {
    out = v[0][0];
#pragma unroll
    for (int r = 0; r < K; ++r)
#pragma unroll
      for (int c = 0; c < K; ++c)
#pragma unroll
        for (int k = 0; k < 4; ++k) out.v[k] = pair_max_nan<F16>(out.v[k], v[r][c].v[k]);
  }
  y[(int64_t)n * per_image + j] = out;
}

template <int K, int S>
static void launch_pool_win(const bf16 *x, bf16 *y, int N, int C, int H, int W, int P, int Q,
                            int pad_h, int pad_w, bool avg, bool f16, cudaStream_t s) {
  const unsigned per_image = (unsigned)((int64_t)P * Q * (C / 8));
  const unsigned chunks = (per_image + 255u) / 256u;
  const unsigned grid = chunks * (unsigned)N;
  auto go = [&](auto kern) {
    kern<<<grid, 256, 0, s>>>((const bf16x8 *)x, (bf16x8 *)y, C / 8, H, W, Q, pad_h, pad_w, per_image,
                              chunks);
  };
  if (avg && f16) go(pool_win_bf16_kernel<K, S, true, true>);
  else if (avg) go(pool_win_bf16_kernel<K, S, true, false>);
  else if (f16) go(pool_win_bf16_kernel<K, S, false, true>);
  else go(pool_win_bf16_kernel<K, S, false, false>);
  count(CNT_LAUNCHES);
}

void launch_pool_bf16(const bf16 *x, bf16 *y, int N, int C, int H, int W, int P, int Q, int kh,
                      int kw, int pad_h, int pad_w, int sh, int sw, bool avg, bool f16,
                      cudaStream_t s) {
  const int64_t total = (int64_t)N * P * Q * (C / 8);
  if (total == 0) return;
  // every window lies at least partly inside the image and the per-image index fits 32 bits
  if (kh == kw && sh == sw && pad_h < kh && pad_w < kw && (P - 1) * sh - pad_h < H &&
      (Q - 1) * sw - pad_w < W && (int64_t)P * Q * (C / 8) < (1ll << 31) - 256 &&
      ((int64_t)P * Q * (C / 8) + 255) / 256 * N < (1ll << 31)) {
    if (kh == 3 && sh == 2) return launch_pool_win<3, 2>(x, y, N, C, H, W, P, Q, pad_h, pad_w, avg, f16, s);
    if (kh == 2 && sh == 2) return launch_pool_win<2, 2>(x, y, N, C, H, W, P, Q, pad_h, pad_w, avg, f16, s);
    if (kh == 3 && sh == 1) return launch_pool_win<3, 1>(x, y, N, C, H, W, P, Q, pad_h, pad_w, avg, f16, s);
    if (kh == 2 && sh == 1) return launch_pool_win<2, 1>(x, y, N, C, H, W, P, Q, pad_h, pad_w, avg, f16, s);
  }
  const int grid = grid_for(total, 256);
  auto go = [&](auto kern) {
    kern<<<grid, 256, 0, s>>>((const bf16x8 *)x, (bf16x8 *)y, C / 8, H, W, P, Q, kh, kw, pad_h, pad_w, sh,
                              sw, total);
  };
  if (avg && f16) go(pool_bf16_kernel<true, true>);
  else if (avg) go(pool_bf16_kernel<true, false>);
  else if (f16) go(pool_bf16_kernel<false, true>);
  else go(pool_bf16_kernel<false, false>);
  count(CNT_LAUNCHES);
}

// Global average pool: [N][HW][C] bf16 -> [N][C] fp32.  One CTA per (image, 64-channel group
// of 8 threads): the GAP_ROWS thread rows split the pixels, each thread sums 8 channels of its
// pixels with 16-byte loads (a warp covers 4 pixels x 128 bytes), partial sums meet in shared
// memory.
constexpr int GAP_ROWS = 16;
template <bool F16>
__global__ void __launch_bounds__(8 * GAP_ROWS) gap_bf16_kernel(const bf16x8 *__restrict__ x,
                                                               float *__restrict__ y, int HW, int C8) {
  __shared__ float part[GAP_ROWS][8][8];
  const int lane8 = threadIdx.x & 7, prow = threadIdx.x >> 3;
  const int c8 = blockIdx.x * 8 + lane8;
  const int64_t n = blockIdx.y;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c8 < C8) {
    const bf16x8 *xp = x + n * HW * C8 + c8;
    for (int p = prow; p < HW; p += GAP_ROWS) {
      float f[8];
      unpack8<F16>(xp[(int64_t)p * C8], f);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += f[k];
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) part[prow][lane8][k] = acc[k];
  __syncthreads();
  if (threadIdx.x < 64) {            // thread = (channel group lane, channel within it)
    const int l = threadIdx.x >> 3, k = threadIdx.x & 7;
    float s = 0.0f;
#pragma unroll
    for (int r = 0; r < GAP_ROWS; ++r) s += part[r][l][k];
    const int c = (blockIdx.x * 8 + l) * 8 + k;
    if (blockIdx.x * 8 + l < C8) y[n * C8 * 8 + c] = s * (1.0f / (float)HW);
  }
}

void launch_gap_bf16(const bf16 *x, float *y, int N, int HW, int C, bool f16, cudaStream_t s) {
  if ((int64_t)N * C == 0) return;
  const int C8 = C / 8;
  const dim3 grid((unsigned)((C8 + 7) / 8), (unsigned)N);
  if (f16) gap_bf16_kernel<true><<<grid, 8 * GAP_ROWS, 0, s>>>((const bf16x8 *)x, y, HW, C8);
  else gap_bf16_kernel<false><<<grid, 8 * GAP_ROWS, 0, s>>>((const bf16x8 *)x, y, HW, C8);
  count(CNT_LAUNCHES);
}

// ---------------------------------------------------------------------------
// Depthwise convolution on NHWC: thread per (n, p, q, 8 channels); the R*S taps of a
// channel group are 2 float4 loads each from the [R*S][C] fp32 filter (L1-resident).
// ---------------------------------------------------------------------------
// CLAMP: the activation is identity / ReLU / Clip, applied as a clamp to [lo, hi] (the general
// switch drags the transcendental activations' code into the loop).
template <bool CLAMP, bool F16>
__global__ void depthwise_bf16_kernel(const bf16x8 *__restrict__ x, const float *__restrict__ w,
                                      const float *__restrict__ bias, bf16x8 *__restrict__ y,
                                      ConvGeom g, int64_t total, float lo, float hi) {
  const int C8 = g.C / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c8 = (int)(i % C8);
    int64_t rest = i / C8;
    const int q = (int)(rest % g.Q);
    rest /= g.Q;
    const int p = (int)(rest % g.P);
    const int64_t n = rest / g.P;
    float acc[8];
    if (bias) {
      const float4 *bp = (const float4 *)(bias + c8 * 8);
      const float4 b0 = bp[0], b1 = bp[1];
      acc[0] = b0.x; acc[1] = b0.y; acc[2] = b0.z; acc[3] = b0.w;
      acc[4] = b1.x; acc[5] = b1.y; acc[6] = b1.z; acc[7] = b1.w;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
    }
    for (int r = 0; r < g.R; ++r) {
      const int h = p * g.stride_h - g.pad_h + r;
      if (h < 0 || h >= g.H) continue;
      for (int s2 = 0; s2 < g.S; ++s2) {
        const int ww = q * g.stride_w - g.pad_w + s2;
        if (ww < 0 || ww >= g.W) continue;
        float f[8];
        unpack8<F16>(x[((n * g.H + h) * g.W + ww) * C8 + c8], f);
        const float4 *wp = (const float4 *)(w + (int64_t)(r * g.S + s2) * g.C + c8 * 8);
        const float4 w0 = wp[0], w1 = wp[1];
        acc[0] = fmaf(f[0], w0.x, acc[0]); acc[1] = fmaf(f[1], w0.y, acc[1]);
        acc[2] = fmaf(f[2], w0.z, acc[2]); acc[3] = fmaf(f[3], w0.w, acc[3]);
        acc[4] = fmaf(f[4], w1.x, acc[4]); acc[5] = fmaf(f[5], w1.y, acc[5]);
        acc[6] = fmaf(f[6], w1.z, acc[6]); acc[7] = fmaf(f[7], w1.w, acc[7]);
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k)
      acc[k] = CLAMP ? fminf(fmaxf(acc[k], lo), hi) : act_apply_b(acc[k], g.act, g.lo, g.hi);
    y[i] = pack8<F16>(acc);
  }
}

// 3x3 depthwise convolution, stride ST (1 or 2), tiled.
// A CTA owns G 8-channel groups (G * 16 bytes of every pixel) of a strip of `cols` output columns
// and works through a run of row tiles (TH output rows each) that continues from one image into
// the next, so the grid is cut into equal runs whatever the image size.  The input tile with its
// halo is staged in shared memory by 16-byte cp.async copies, two tiles ahead; what lies outside
// the image is stored as zeros.  A thread owns FOUR channels of one output column: its nine taps
// (18 packed fp32 pairs) and the three input rows of the current window, already converted to
// fp32 pairs, stay in registers, so an input value is converted once and an output row costs
// ST * 3 eight-byte shared-memory loads and 18 packed FMAs (fma.rn.f32x2).  The kernel is bound by
// instruction issue as much as by memory, which is why the work per output is kept this small.
__device__ __forceinline__ uint64_t dw_pair(uint32_t lo_bits, uint32_t hi_bits) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo_bits), "r"(hi_bits));
  return r;
}
__device__ __forceinline__ uint64_t dw_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t dw_mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t dw_add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// two 16-bit values in one word -> the fp32 pair
template <bool F16>
__device__ __forceinline__ uint64_t dw_unpack(uint32_t v) {
  const float2 t = pair_to_f32<F16>(v);
  return dw_pair(__float_as_uint(t.x), __float_as_uint(t.y));
}
// fp32 pair -> clamp -> two 16-bit values in one word
template <bool F16>
__device__ __forceinline__ uint32_t dw_finish(uint64_t acc, float lo, float hi) {
  float a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(acc));
  a = fminf(fmaxf(a, lo), hi);
  b = fminf(fmaxf(b, lo), hi);
  return f32_to_pair<F16>(a, b);
}
// The same for bounds that the element type holds exactly (lower bound 0 or none): the lower
// bound rides on the conversion, the upper one is a packed minimum after it.  flags: 1 = lower
// bound 0, 2 = upper bound present (hi2 holds it twice).
template <bool F16>
__device__ __forceinline__ uint32_t dw_finish_packed(uint64_t acc, int flags, uint32_t hi2) {
  float a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(acc));
  uint32_t r = (flags & 1) ? f32_to_pair_relu<F16>(a, b) : f32_to_pair<F16>(a, b);
  if (flags & 2) r = pair_min<F16>(r, hi2);
  return r;
}
template <int NP>
struct DwRow {
  uint64_t v[3][NP];   // three columns x NP channel pairs as fp32 pairs
};
// packed fp16 arithmetic (fp16 mode): two channels per 32-bit word, no conversions
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t h2_max_nan(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t h2_min_nan(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("min.NaN.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t h2_from_floats(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// CH = channels per thread: 4 (two CTAs per SM); 2 also compiles (four CTAs per SM) but is slower.
template <int ST, bool PACKED_ACT, int CH, bool F16>
__global__ void __launch_bounds__(256, CH == 2 ? 4 : 2) depthwise3x3_tile_kernel(
    const uint4 *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias,
    uint32_t *__restrict__ y, ConvGeom g, int G, int cols, int TH, int tiles_q, int tiles_c, int ntiles,
    int run_len, int run_total, float act_lo, float act_hi, int act_flags, uint32_t act_hi2) {
  constexpr int NP = CH / 2;      // channel pairs (32-bit words of bf16) per thread
  constexpr int LG = 8 / CH;      // threads per 16-byte channel group
  extern __shared__ uint4 dw_smem[];
  const int C8 = g.C / 8;
  int b = blockIdx.x;
  const int cb = b % tiles_c;
  b /= tiles_c;
  const int qt = b % tiles_q;
  const int run = b / tiles_q;
  const int s0 = run * run_len, s1 = min(s0 + run_len, run_total);   // (image, row tile) pairs
  if (s0 >= s1) return;
  const int q0 = qt * cols;
  const int IW = (cols - 1) * ST + 3, IH = (TH - 1) * ST + 3;
  const int row_vecs = IW * G, stage_vecs = IH * row_vecs;
  const int tid = threadIdx.x;
  const int sub = tid % LG, gl = (tid / LG) % G, col = tid / (LG * G);
  const int q = q0 + col;
  const bool active = col < cols && q < g.Q;
  const int c8 = cb * G + gl;
  const int w_in0 = q0 * ST - g.pad_w;

  // Staging: a thread always copies the same 16-byte pieces of a tile row (piece j = tid + 256 k
  // of the IW * G pieces, at most 2 * 128 + G of them), so their arithmetic is done once.  A piece
  // outside the image is a copy of zero source bytes, which fills the 16 bytes with zeros: the
  // loop over the rows has no branch.
  // When a tile row has at most 128 pieces, the threads split into groups that take every
  // `ngroups`-th row each, so that all warps share the copy work.
  constexpr int KMAX = 2;
  const int ngroups = row_vecs <= 128 ? 256 / row_vecs : 1;
  const int grp = ngroups > 1 ? tid / row_vecs : 0;
  const int jbase = ngroups > 1 ? tid - grp * row_vecs : tid;
  int src_off[KMAX];                            // offset of the piece inside an input row, or -1
#pragma unroll
  for (int k = 0; k < KMAX; ++k) {
    const int j = jbase + 256 * k;
    const int gg = j % G, ww = w_in0 + j / G;
    src_off[k] = (j < row_vecs && ww >= 0 && ww < g.W) ? ww * C8 + cb * G + gg : -1;
  }
  const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(dw_smem);
  const int row_elems = g.W * C8;
  auto stage = [&](int sidx, int into) {
    if (grp < ngroups) {
      const int n = sidx / ntiles, t = sidx - n * ntiles;
      const uint32_t dst = smem0 + (uint32_t)((into * stage_vecs + jbase) * 16);
      const uint4 *xin = x + (int64_t)n * g.H * row_elems;
      const int h_in0 = t * TH * ST - g.pad_h;
#pragma unroll
      for (int k = 0; k < KMAX; ++k) {
        if (jbase + 256 * k >= row_vecs) break;
        const uint4 *colp = xin + max(src_off[k], 0);
        for (int ih = grp; ih < IH; ih += ngroups) {
          const int h = h_in0 + ih;
          const bool ok = (unsigned)h < (unsigned)g.H && src_off[k] >= 0;
          const uint4 *src = ok ? colp + (int64_t)h * row_elems : x;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                           dst + (uint32_t)((ih * row_vecs + 256 * k) * 16)),
                       "l"(src), "r"(ok ? 16 : 0)
                       : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  uint64_t wv[9][NP];
  uint64_t bv[NP];
#pragma unroll
  for (int j = 0; j < NP; ++j) bv[j] = 0;
  if (active) {
#pragma unroll
    for (int t = 0; t < 9; ++t) {
      const float2 *wp = (const float2 *)(w + (int64_t)t * g.C + c8 * 8 + sub * CH);
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const float2 a = wp[j];
        wv[t][j] = dw_pair(__float_as_uint(a.x), __float_as_uint(a.y));
      }
    }
    if (bias) {
      const float2 *bp = (const float2 *)(bias + c8 * 8 + sub * CH);
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const float2 a = bp[j];
        bv[j] = dw_pair(__float_as_uint(a.x), __float_as_uint(a.y));
      }
    }
  } else {
#pragma unroll
    for (int t = 0; t < 9; ++t)
#pragma unroll
      for (int j = 0; j < NP; ++j) wv[t][j] = 0;
  }
  // Three buffers, one barrier per tile: after the barrier of tile i every thread has finished
  // tile i - 1, whose buffer then takes tile i + 2.  A group is committed every iteration (an empty
  // one past the end), so "all but the newest group" always means "tile i has landed".
  stage(s0, 0);
  if (s0 + 1 < s1) stage(s0 + 1, 1);
  else asm volatile("cp.async.commit_group;" ::: "memory");
  int buf = 0;
  for (int sidx = s0; sidx < s1; ++sidx) {
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    if (sidx + 2 < s1) stage(sidx + 2, buf == 0 ? 2 : buf - 1);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    if (active) {
      const int n = sidx / ntiles, t = sidx - n * ntiles;
      // shared-memory and output positions in 32-bit words (NP words per thread)
      const uint32_t *src = reinterpret_cast<const uint32_t *>(dw_smem + buf * stage_vecs) +
                            ((col * ST) * G + gl) * 4 + sub * NP;
      uint32_t *yout = y + ((int64_t)n * g.P * g.Q + q) * C8 * 4 + c8 * 4 + sub * NP;
      auto load_row = [&](int ih, DwRow<NP> &r) {
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          const uint32_t *sp = src + (ih * IW + k) * G * 4;
          if (NP == 2) {
            const uint2 v = *reinterpret_cast<const uint2 *>(sp);
            r.v[k][0] = dw_unpack<F16>(v.x);
            r.v[k][NP - 1] = dw_unpack<F16>(v.y);
          } else {
            r.v[k][0] = dw_unpack<F16>(*sp);
          }
        }
      };
      auto emit = [&](int p, const DwRow<NP> &a, const DwRow<NP> &bq, const DwRow<NP> &cq) {
        if (p >= g.P) return;
        // one accumulation chain per filter row and channel pair
        uint32_t o[NP];
#pragma unroll
        for (int j = 0; j < NP; ++j) {
          uint64_t fa = dw_fma2(a.v[0][j], wv[0][j], bv[j]);
          uint64_t fb = dw_mul2(bq.v[0][j], wv[3][j]);
          uint64_t fc = dw_mul2(cq.v[0][j], wv[6][j]);
#pragma unroll
          for (int k = 1; k < 3; ++k) {
            fa = dw_fma2(a.v[k][j], wv[k][j], fa);
            fb = dw_fma2(bq.v[k][j], wv[3 + k][j], fb);
            fc = dw_fma2(cq.v[k][j], wv[6 + k][j], fc);
          }
          const uint64_t f = dw_add2(dw_add2(fa, fb), fc);
          // the activations this kernel takes are all a clamp (a switch over every activation,
          // inlined into each unrolled copy of this body, would not fit the instruction cache)
          o[j] = PACKED_ACT ? dw_finish_packed<F16>(f, act_flags, act_hi2)
                            : dw_finish<F16>(f, act_lo, act_hi);
        }
        uint32_t *yp = yout + (int64_t)p * g.Q * C8 * 4;
        if (NP == 2) *reinterpret_cast<uint2 *>(yp) = make_uint2(o[0], o[NP - 1]);
        else *yp = o[0];
      };
      DwRow<NP> r0, r1, r2;
      const int pbase = t * TH;
      if (ST == 1) {
        load_row(0, r0);
        load_row(1, r1);
        for (int pl = 0; pl < TH; pl += 3) {
          load_row(pl + 2, r2);
          emit(pbase + pl, r0, r1, r2);
          load_row(pl + 3, r0);
          emit(pbase + pl + 1, r1, r2, r0);
          load_row(pl + 4, r1);
          emit(pbase + pl + 2, r2, r0, r1);
        }
      } else {
        load_row(0, r0);
        for (int pl = 0; pl < TH; pl += 3) {
          load_row(2 * pl + 1, r1);
          load_row(2 * pl + 2, r2);
          emit(pbase + pl, r0, r1, r2);
          load_row(2 * pl + 3, r0);
          load_row(2 * pl + 4, r1);
          emit(pbase + pl + 1, r2, r0, r1);
          load_row(2 * pl + 5, r2);
          load_row(2 * pl + 6, r0);
          emit(pbase + pl + 2, r1, r2, r0);
        }
      }
    }
    buf = buf == 2 ? 0 : buf + 1;
  }
}

// 3x3 depthwise convolution in packed fp16 arithmetic without shared memory.  A thread owns the
// eight channels of one 16-byte piece in one output column and walks down a strip of output
// rows: the input rows of its window stay in registers (each is loaded once per thread), the
// three columns of a row are three 16-byte loads that the neighbouring threads' loads overlap
// (L1 serves the overlap), and the rows of the next two outputs are requested before the
// current output is computed.  Lanes run over the channel pieces of a pixel first, then over columns, so every
// load and store of a warp is one contiguous run of bytes.  About 7 instructions per output
// (nine fma.rn.f16x2 per channel pair) against about 20 for the staged tile kernel.
struct DwRow8 {
  uint4 c[3];   // three input columns x eight channels (fp16 pairs)
};
__device__ __forceinline__ uint32_t dw_word(const uint4 &v, int j) {
  return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w));
}
__device__ __forceinline__ uint4 dw_ldg16(const uint4 *p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
template <int ST>
__global__ void __launch_bounds__(128, 4)
    depthwise3x3_strip_h2_kernel(const uint4 *__restrict__ x, const float *__restrict__ w,
                                 const float *__restrict__ bias, uint4 *__restrict__ y, ConvGeom g,
                                 int strips, int strip_rows, int64_t total, int act_flags,
                                 uint32_t act_hi2, int ahead) {
  const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;   // the launcher keeps total < 2^31
  if (idx >= (uint32_t)total) return;
  const int C8 = g.C / 8;
  const int c8 = (int)(idx % (uint32_t)C8);
  uint32_t r = idx / (uint32_t)C8;
  const int q = (int)(r % (uint32_t)g.Q);
  r /= (uint32_t)g.Q;
  const int sidx = (int)(r % (uint32_t)strips);
  const int n = (int)(r / (uint32_t)strips);
  const int p0 = sidx * strip_rows;
  const int p1 = min(p0 + strip_rows, g.P);
  if (p0 >= p1) return;

  uint32_t wh[9][4], bh[4] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int t = 0; t < 9; ++t) {
    const float4 *wp = reinterpret_cast<const float4 *>(w + (int64_t)t * g.C + c8 * 8);
    const float4 a = wp[0], b = wp[1];
    wh[t][0] = h2_from_floats(a.x, a.y);
    wh[t][1] = h2_from_floats(a.z, a.w);
    wh[t][2] = h2_from_floats(b.x, b.y);
    wh[t][3] = h2_from_floats(b.z, b.w);
  }
  if (bias) {
    const float4 *bp = reinterpret_cast<const float4 *>(bias + c8 * 8);
    const float4 a = bp[0], b = bp[1];
    bh[0] = h2_from_floats(a.x, a.y);
    bh[1] = h2_from_floats(a.z, a.w);
    bh[2] = h2_from_floats(b.x, b.y);
    bh[3] = h2_from_floats(b.z, b.w);
  }
  // Input columns of the window.  A column outside the image (first and last output column
  // only) is read from the middle column instead and its three taps get weight zero, so the
  // loop has no per-column test.
  const int w0 = q * ST - g.pad_w;
  const bool cok0 = w0 >= 0 && w0 < g.W, cok2 = w0 + 2 >= 0 && w0 + 2 < g.W;
#pragma unroll
  for (int t = 0; t < 9; t += 3)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (!cok0) wh[t][j] = 0u;
      if (!cok2) wh[t + 2][j] = 0u;
    }
  const int64_t row_pieces = (int64_t)g.W * C8;
  const int off0 = cok0 ? 0 : C8, off2 = cok2 ? 2 * C8 : C8;   // piece offsets inside a row
  const int h_first = p0 * ST - g.pad_h;                 // first input row of the strip
  const int h_last = min((p1 - 1) * ST - g.pad_h + 2, g.H - 1);   // last one it reads
  // next row to load: rows are loaded strictly in order, so the pointer just steps
  const uint4 *rp = x + (((int64_t)n * g.H + h_first) * g.W + w0) * C8 + c8;
  int h_next = h_first;
  // Rows further down are asked into L2 ahead of time (one request per thread for its middle
  // column; a warp's requests cover its contiguous run of the row): the register window then
  // only has to cover the L2 latency, not the DRAM latency.  Stride 2 has enough in flight.
  auto load = [&](DwRow8 &row) {
    if (h_next >= 0 && h_next <= h_last) {   // the same for all threads of a warp
      row.c[0] = dw_ldg16(rp + off0);
      row.c[1] = dw_ldg16(rp + C8);
      row.c[2] = dw_ldg16(rp + off2);
      if (ST == 1 && h_next + ahead <= h_last)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(rp + (int64_t)ahead * row_pieces + C8));
    } else {
      row.c[0] = row.c[1] = row.c[2] = make_uint4(0u, 0u, 0u, 0u);
    }
    rp += row_pieces;
    ++h_next;
  };
  // bounds as packed halves; "none" is -inf / +inf, so that both are always applied
  const uint32_t lo2 = (act_flags & 1) ? 0u : 0xFC00FC00u;
  const uint32_t hi2 = (act_flags & 2) ? act_hi2 : 0x7C007C00u;
  uint4 *yp = y + (((int64_t)n * g.P + p0) * g.Q + q) * C8 + c8;
  const int64_t out_row = (int64_t)g.Q * C8;
  auto emit = [&](const DwRow8 &a, const DwRow8 &b, const DwRow8 &c) {
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t f = bh[j];
#pragma unroll
      for (int k = 0; k < 3; ++k) f = h2_fma(dw_word(a.c[k], j), wh[k][j], f);
#pragma unroll
      for (int k = 0; k < 3; ++k) f = h2_fma(dw_word(b.c[k], j), wh[3 + k][j], f);
#pragma unroll
      for (int k = 0; k < 3; ++k) f = h2_fma(dw_word(c.c[k], j), wh[6 + k][j], f);
      o[j] = h2_min_nan(h2_max_nan(f, lo2), hi2);
    }
    *yp = make_uint4(o[0], o[1], o[2], o[3]);
    yp += out_row;
  };
  const int nout = p1 - p0;
  if (ST == 1) {
    // one new row per output, requested two outputs ahead: five row buffers in rotation
    DwRow8 A, B, C, D, E;
    load(A);
    load(B);
    load(C);
    load(D);
    for (int i = 0; i < nout; i += 5) {
      load(E);
      emit(A, B, C);
      if (i + 1 >= nout) break;
      load(A);
      emit(B, C, D);
      if (i + 2 >= nout) break;
      load(B);
      emit(C, D, E);
      if (i + 3 >= nout) break;
      load(C);
      emit(D, E, A);
      if (i + 4 >= nout) break;
      load(D);
      emit(E, A, B);
    }
  } else {
    // stride 2: an output shares one input row with the next; two new rows per output
    DwRow8 A, B, C, D, E;
    load(A);
    load(B);
    load(C);
    for (int i = 0; i < nout; i += 5) {
      load(D);
      load(E);
      emit(A, B, C);
      if (i + 1 >= nout) break;
      load(A);
      load(B);
      emit(C, D, E);
      if (i + 2 >= nout) break;
      load(C);
      load(D);
      emit(E, A, B);
      if (i + 3 >= nout) break;
      load(E);
      load(A);
      emit(B, C, D);
      if (i + 4 >= nout) break;
      load(B);
      load(C);
      emit(D, E, A);
    }
  }
}

void launch_depthwise_bf16(const bf16 *x, const float *w_rsc, const float *bias, bf16 *y,
                           const ConvGeom &g, bool f16, cudaStream_t s) {
  const int64_t total = (int64_t)g.N * g.P * g.Q * (g.C / 8);
  if (total == 0) return;
  const int C8 = g.C / 8;
  if (g.R == 3 && g.S == 3 && g.stride_h == g.stride_w && (g.stride_h == 1 || g.stride_h == 2) &&
      (g.act == ACT_IDENTITY || g.act == ACT_RELU || g.act == ACT_CLIP)) {
    const int ST = g.stride_h;
    // Channel groups per CTA (a divisor of C / 8, at most 16) and columns per CTA (128 / G at
    // most: two threads per channel group and column): the pair that keeps most of the 256
    // threads busy; among near-equal ones the widest channel run, for contiguous 16-byte pieces.
    const float act_lo = g.act == ACT_RELU ? 0.0f : (g.act == ACT_CLIP ? g.lo : -INFINITY);
    const float act_hi = g.act == ACT_CLIP ? g.hi : INFINITY;
    // bounds that the element type holds exactly go through the packed conversion
    const uint16_t hbits = host_elem_bits(act_hi, f16);
    const bool packed = (act_lo == 0.0f || act_lo == -INFINITY) &&
                        (act_hi == INFINITY || host_elem_value(hbits, f16) == act_hi);
    // Channels per thread: 4.  (2 halves the registers and doubles the resident CTAs, but the
    // kernel is bound by its instruction count, which grows: measured 1.4x slower.)
    // fp16 mode with bounds fp16 holds: 8, computed on packed fp16 pairs (see the kernel).
    bool h2 = f16 && packed;
#ifdef OCCAMY_TUNING
    if (const char *f = getenv("OCCAMY_DW_H2")) h2 = h2 && atoi(f) != 0;
#endif
    // the kernel relies on a valid middle column and on 32-bit thread numbers
    bool strip = h2 && g.pad_w >= 0 && g.pad_w <= 1 && total * 16 < (int64_t)1 << 31;
#ifdef OCCAMY_TUNING
    if (const char *f = getenv("OCCAMY_DW_STRIP")) strip = strip && atoi(f) != 0;
#endif
    if (strip) {
      // Register strips (see the kernel): enough strips per column for a few waves of threads,
      // but at least seven output rows each, so that the two halo rows and the weights a
      // thread fetches stay a small part of its traffic.
      const int64_t base = (int64_t)g.N * g.Q * C8;
      // waves of threads the strips are cut for (measured: 2 best at stride 1, 4 at stride 2;
      // 8 and 16 are 10 to 25 % slower) and rows ahead of the loads that are asked into L2
      int waves = ST == 1 ? 2 : 4, ahead = 4;
#ifdef OCCAMY_TUNING
      if (const char *f = getenv("OCCAMY_DW_WAVES")) waves = atoi(f) > 0 ? atoi(f) : waves;
      if (const char *f = getenv("OCCAMY_DW_AHEAD")) ahead = atoi(f) > 0 ? atoi(f) : ahead;
#endif
      const int64_t want = (int64_t)rt().num_sms * 512 * waves;
      int strips = (int)((want + base - 1) / base);
      const int most = g.P / 7 > 1 ? g.P / 7 : 1;
      if (strips > most) strips = most;
      if (strips < 1) strips = 1;
      const int strip_rows = (g.P + strips - 1) / strips;
      strips = (g.P + strip_rows - 1) / strip_rows;
      const int64_t threads = base * strips;
      const unsigned grid = (unsigned)((threads + 127) / 128);
      const int act_flags = (act_lo == 0.0f ? 1 : 0) | (act_hi != INFINITY ? 2 : 0);
      const uint32_t act_hi2 = (uint32_t)hbits * 0x10001u;
      if (ST == 1)
        depthwise3x3_strip_h2_kernel<1><<<grid, 128, 0, s>>>((const uint4 *)x, w_rsc, bias, (uint4 *)y, g,
                                                            strips, strip_rows, threads, act_flags, act_hi2, ahead);
      else
        depthwise3x3_strip_h2_kernel<2><<<grid, 128, 0, s>>>((const uint4 *)x, w_rsc, bias, (uint4 *)y, g,
                                                            strips, strip_rows, threads, act_flags, act_hi2, ahead);
      count(CNT_LAUNCHES);
      return;
    }
    const int CH = 4;
    const int LG = 8 / CH;
    // Geometry: G channel groups x `cols` columns per CTA (G * cols * LG <= 256 threads) and TH
    // output rows per staged tile (a multiple of 3, the register rotation; three buffers within
    // the CTA's share of the shared memory).  Scored by the share of threads with work times the
    // share of the staged input that is not halo; a tile row may have at most 512 pieces (two per
    // thread in the staging loop).
    int G = 0, cols = 0, tiles_q = 0, TH = 0, ntiles = 0;
    double best = 0.0;
    const size_t smem_cap = (size_t)(CH == 2 ? 50 : 100) * 1024;
    for (int cand = 16; cand >= 1; --cand) {
      if (C8 % cand) continue;
      const int cmax = 256 / (LG * cand);
      if (cmax < 1) continue;
      const int tq0 = (g.Q + cmax - 1) / cmax;
      for (int tq = tq0; tq <= tq0 + 3 && tq <= g.Q; ++tq) {
        const int cl = (g.Q + tq - 1) / tq;
        const int iw = (cl - 1) * ST + 3;
        if (iw * cand > 512) continue;
        int th_best = 0;
        int64_t rows_best = 0;
        for (int th = 3; th <= 18; th += 3) {
          const int ih = (th - 1) * ST + 3;
          if ((size_t)3 * ih * iw * cand * 16 > smem_cap) break;
          const int64_t rows = (int64_t)((g.P + th - 1) / th) * ih;
          if (th_best == 0 || rows < rows_best) {
            th_best = th;
            rows_best = rows;
          }
        }
        if (th_best == 0) continue;
        const double util = (double)(cl * cand * LG) / 256.0 * (double)g.Q / (double)(cl * tq);
        const double fresh = (double)(g.P * ST) / (double)rows_best * (double)(cl * ST) / (double)iw;
        const double score = util * (fresh < 1.0 ? fresh : 1.0);
        if (score > best * 1.03) {
          best = score;
          G = cand;
          cols = cl;
          tiles_q = tq;
          TH = th_best;
          ntiles = (g.P + th_best - 1) / th_best;
        }
      }
    }
    const int IW = (cols - 1) * ST + 3;
    if (G > 0 && TH > 0 && best >= 0.25) {
      const size_t smem = (size_t)3 * ((TH - 1) * ST + 3) * IW * G * 16;
      const int tiles_c = C8 / G;
      // Runs of (image, row tile) pairs: one wave of equal runs over the CTA slots when the
      // strips alone do not fill them, else one run per strip.
      const int run_total = g.N * ntiles;
      const int base = tiles_q * tiles_c;
      const int slots = rt().num_sms * (CH == 2 ? 4 : 2);
      int runs = slots / base;
      if (runs < 1) runs = 1;
      if (runs > run_total) runs = run_total;
      const int run_len = (run_total + runs - 1) / runs;
      runs = (run_total + run_len - 1) / run_len;
      const unsigned grid = (unsigned)((int64_t)runs * base);
      const int act_flags = (act_lo == 0.0f ? 1 : 0) | (act_hi != INFINITY ? 2 : 0);
      const uint32_t act_hi2 = (uint32_t)hbits * 0x10001u;
      static unsigned char attr_done[64] = {};
      int dev = 0;
      cudaGetDevice(&dev);
      if (dev >= 0 && dev < 64 && !attr_done[dev]) {   // function attributes are per device
        attr_done[dev] = 1;
        const int lim = 100 * 1024;
        const auto attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
        cudaFuncSetAttribute(depthwise3x3_tile_kernel<1, true, 4, false>, attr, lim);
        cudaFuncSetAttribute(depthwise3x3_tile_kernel<1, false, 4, false>, attr, lim);
        cudaFuncSetAttribute(depthwise3x3_tile_kernel<2, true, 4, false>, attr, lim);
        cudaFuncSetAttribute(depthwise3x3_tile_kernel<2, false, 4, false>, attr, lim);
        cudaFuncSetAttribute(depthwise3x3_tile_kernel<1, true, 4, true>, attr, lim);
        cudaFuncSetAttribute(depthwise3x3_tile_kernel<1, false, 4, true>, attr, lim);
        cudaFuncSetAttribute(depthwise3x3_tile_kernel<2, true, 4, true>, attr, lim);
        cudaFuncSetAttribute(depthwise3x3_tile_kernel<2, false, 4, true>, attr, lim);
      }
      auto go = [&](auto kern) {
        kern<<<grid, 256, smem, s>>>((const uint4 *)x, w_rsc, bias, (uint32_t *)y, g, G, cols, TH, tiles_q,
                                     tiles_c, ntiles, run_len, run_total, act_lo, act_hi, act_flags,
                                     act_hi2);
      };
      if (f16) {
        if (ST == 1 && packed) go(depthwise3x3_tile_kernel<1, true, 4, true>);
        else if (ST == 1) go(depthwise3x3_tile_kernel<1, false, 4, true>);
        else if (packed) go(depthwise3x3_tile_kernel<2, true, 4, true>);
        else go(depthwise3x3_tile_kernel<2, false, 4, true>);
      } else {
        if (ST == 1 && packed) go(depthwise3x3_tile_kernel<1, true, 4, false>);
        else if (ST == 1) go(depthwise3x3_tile_kernel<1, false, 4, false>);
        else if (packed) go(depthwise3x3_tile_kernel<2, true, 4, false>);
        else go(depthwise3x3_tile_kernel<2, false, 4, false>);
      }
      count(CNT_LAUNCHES);
      return;
    }
  }
  if (g.act == ACT_IDENTITY || g.act == ACT_RELU || g.act == ACT_CLIP) {
    const float lo = g.act == ACT_RELU ? 0.0f : (g.act == ACT_CLIP ? g.lo : -INFINITY);
    const float hi = g.act == ACT_CLIP ? g.hi : INFINITY;
    if (f16)
      depthwise_bf16_kernel<true, true><<<grid_for(total, 256), 256, 0, s>>>(
          (const bf16x8 *)x, w_rsc, bias, (bf16x8 *)y, g, total, lo, hi);
    else
      depthwise_bf16_kernel<true, false><<<grid_for(total, 256), 256, 0, s>>>(
          (const bf16x8 *)x, w_rsc, bias, (bf16x8 *)y, g, total, lo, hi);
  } else if (f16) {
    depthwise_bf16_kernel<false, true><<<grid_for(total, 256), 256, 0, s>>>(
        (const bf16x8 *)x, w_rsc, bias, (bf16x8 *)y, g, total, 0.f, 0.f);
  } else {
    depthwise_bf16_kernel<false, false><<<grid_for(total, 256), 256, 0, s>>>(
        (const bf16x8 *)x, w_rsc, bias, (bf16x8 *)y, g, total, 0.f, 0.f);
  }
  count(CNT_LAUNCHES);
}

// ---------------------------------------------------------------------------
// fp32 on the tensor cores: a value is carried as three bf16 parts, hi + mid + lo, which
// together hold its 24 mantissa bits.  A product a * w is then the sum of the six part
// products that matter (hi*hi, hi*mid, hi*lo, mid*hi, mid*mid, lo*hi; the three left out are
// below 2^-24 of it), each exact in the fp32 accumulator.  These kernels make the parts: the
// activation as three NHWC planes, the filter with six parts per tap in the matching order.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void split3(float v, uint16_t &hi, uint16_t &mid, uint16_t &lo) {
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  const float r1 = v - __bfloat162float(h);            // exact: the part bf16 dropped
  const __nv_bfloat16 m = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(m);
  hi = __bfloat16_as_ushort(h);
  mid = __bfloat16_as_ushort(m);
  lo = __bfloat16_as_ushort(__float2bfloat16_rn(r2));
}

// x fp32 [N][C][HW] -> three planes [N][HW][Cp] bf16 (channels C..Cp-1 zero), `plane` elements
// apart, through a 32 x 32 tile like the plain layout conversion.
__global__ void split3_nchw_kernel(const float *__restrict__ x, uint16_t *__restrict__ y, int C, int Cp,
                                   int HW, int64_t plane) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 32;
  const float *xn = x + (int64_t)n * C * HW;
  uint16_t *yn = y + (int64_t)n * Cp * HW;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, p = p0 + threadIdx.x;
    tile[i][threadIdx.x] = (c < C && p < HW) ? xn[(int64_t)c * HW + p] : 0.0f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int p = p0 + i, c = c0 + threadIdx.x;
    if (p < HW && c < Cp) {
      uint16_t h, m, l;
      split3(tile[threadIdx.x][i], h, m, l);
      const int64_t at = (int64_t)p * Cp + c;
      yn[at] = h;
      yn[at + plane] = m;
      yn[at + 2 * plane] = l;
    }
  }
}

void launch_split3_nchw(const float *x, bf16 *y, int N, int C, int Cp, int H, int W, cudaStream_t s) {
  const int HW = H * W;
  if ((int64_t)N * C * HW == 0) return;
  dim3 grid((HW + 31) / 32, (Cp + 31) / 32, N), block(32, 8);
  split3_nchw_kernel<<<grid, block, 0, s>>>(x, (uint16_t *)y, C, Cp, HW, (int64_t)N * HW * Cp);
  count(CNT_LAUNCHES);
}

// x fp32 [M][K] (row length ld) -> three planes [M][Kp] bf16
__global__ void split3_rows_kernel(const float *__restrict__ x, uint16_t *__restrict__ y, int K, int Kp,
                                   int ld, int64_t total, int64_t plane) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int k = (int)(i % Kp);
    const int64_t m = i / Kp;
    uint16_t h, md, l;
    split3(k < K ? x[m * ld + k] : 0.0f, h, md, l);
    y[i] = h;
    y[i + plane] = md;
    y[i + 2 * plane] = l;
  }
}

void launch_split3_rows(const float *x, bf16 *y, int M, int K, int Kp, int ld, cudaStream_t s) {
  const int64_t total = (int64_t)M * Kp;
  if (total == 0) return;
  split3_rows_kernel<<<grid_for(total, 256), 256, 0, s>>>(x, (uint16_t *)y, K, Kp, ld, total, total);
  count(CNT_LAUNCHES);
}

// [K][C][R*S] fp32 -> [R*S * 6][K][Cp] bf16: per tap the parts (hi, mid, lo, hi, mid, hi), to be
// multiplied with the activation parts (hi, hi, hi, mid, mid, lo).
__global__ void pack_krsc_split_kernel(const float *__restrict__ w, uint16_t *__restrict__ out, int K,
                                       int C, int Cp, int RS, int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cp);
    const int k = (int)((i / Cp) % K);
    const int tj = (int)(i / ((int64_t)Cp * K));
    const int t = tj / 6, j = tj % 6;
    uint16_t part[3];
    split3(c < C ? w[((int64_t)k * C + c) * RS + t] : 0.0f, part[0], part[1], part[2]);
    const int which = j == 0 ? 0 : (j == 1 ? 1 : (j == 2 ? 2 : (j == 3 ? 0 : (j == 4 ? 1 : 0))));
    out[i] = part[which];
  }
}

void launch_pack_krsc_split(const float *w, bf16 *out, int K, int C, int R, int S, int Cp,
                            cudaStream_t s) {
  const int64_t total = (int64_t)K * Cp * R * S * 6;
  if (total == 0) return;
  pack_krsc_split_kernel<<<grid_for(total, 256), 256, 0, s>>>(w, (uint16_t *)out, K, C, Cp, R * S, total);
  count(CNT_LAUNCHES);
}

// ---------------------------------------------------------------------------
// Weight packing (runs once per constant; results stay resident)
// ---------------------------------------------------------------------------
// [K][C][R*S] fp32 -> [R*S][K][Cp] bf16, channels c >= C (padding up to Cp) zero.
template <bool F16>
__global__ void pack_krsc_kernel(const float *__restrict__ w, uint16_t *__restrict__ out, int K, int C,
                                 int Cp, int RS, int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cp);
    const int k = (int)((i / Cp) % K);
    const int t = (int)(i / ((int64_t)Cp * K));
    out[i] = f32_to_elem<F16>(c < C ? w[((int64_t)k * C + c) * RS + t] : 0.0f);
  }
}

void launch_pack_krsc_bf16(const float *w, bf16 *out, int K, int C, int R, int S, int Cp, bool f16,
                           cudaStream_t s) {
  if (Cp < C) Cp = C;
  const int64_t total = (int64_t)K * Cp * R * S;
  if (total == 0) return;
  if (f16)
    pack_krsc_kernel<true><<<grid_for(total, 256), 256, 0, s>>>(w, (uint16_t *)out, K, C, Cp, R * S, total);
  else
    pack_krsc_kernel<false><<<grid_for(total, 256), 256, 0, s>>>(w, (uint16_t *)out, K, C, Cp, R * S, total);
  count(CNT_LAUNCHES);
}

// [pixels][C8 * 8] bf16 -> [pixels][Cp8 * 8] bf16 with zero channels appended (a channel count
// that is not a multiple of the MMA's 16 is padded before the tensor-core convolution).
__global__ void pad_channels_kernel(const bf16x8 *__restrict__ x, bf16x8 *__restrict__ y, int C8,
                                    int Cp8, int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cp8);
    const int64_t px = i / Cp8;
    bf16x8 v;
    v.u = make_uint4(0, 0, 0, 0);
    if (c < C8) v = x[px * C8 + c];
    y[i] = v;
  }
}

void launch_pad_channels_bf16(const bf16 *x, bf16 *y, int64_t pixels, int C, int Cp, cudaStream_t s) {
  const int64_t total = pixels * (Cp / 8);
  if (total == 0) return;
  pad_channels_kernel<<<grid_for(total, 256), 256, 0, s>>>((const bf16x8 *)x, (bf16x8 *)y, C / 8, Cp / 8,
                                                        total);
  count(CNT_LAUNCHES);
}

__global__ void pack_dw_kernel(const float *__restrict__ w, float *__restrict__ out, int C, int RS,
                               int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int t = (int)(i / C);
    out[i] = w[(int64_t)c * RS + t];
  }
}

void launch_pack_dw_f32(const float *w, float *out, int C, int R, int S, cudaStream_t s) {
  const int64_t total = (int64_t)C * R * S;
  if (total == 0) return;
  pack_dw_kernel<<<grid_for(total, 256), 256, 0, s>>>(w, out, C, R * S, total);
  count(CNT_LAUNCHES);
}

// Folded form for convolutions with very few input channels (the RGB stems): the S width
// taps and the C channels of one filter row become Sp*Cp "channels" of a Rx1 convolution.
template <bool F16>
__global__ void pack_fold_kernel(const float *__restrict__ w, uint16_t *__restrict__ out, int K, int C,
                                 int R, int S, int Sp, int Cp, int64_t total) {
  const int Cf = Sp * Cp;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int cf = (int)(i % Cf);
    const int k = (int)((i / Cf) % K);
    const int r = (int)(i / ((int64_t)Cf * K));
    const int s2 = cf / Cp, c = cf % Cp;
    float v = 0.0f;
    if (s2 < S && c < C) v = w[(((int64_t)k * C + c) * R + r) * S + s2];
    out[i] = f32_to_elem<F16>(v);
  }
}

void launch_pack_fold_bf16(const float *w, bf16 *out, int K, int C, int R, int S, int Sp, int Cp,
                           bool f16, cudaStream_t s) {
  const int64_t total = (int64_t)R * K * Sp * Cp;
  if (total == 0) return;
  if (f16)
    pack_fold_kernel<true><<<grid_for(total, 256), 256, 0, s>>>(w, (uint16_t *)out, K, C, R, S, Sp, Cp, total);
  else
    pack_fold_kernel<false><<<grid_for(total, 256), 256, 0, s>>>(w, (uint16_t *)out, K, C, R, S, Sp, Cp, total);
  count(CNT_LAUNCHES);
}

// x fp32 NCHW -> bf16 [N][H][Wp][Cp], image shifted right by pad_w pixels, zeros elsewhere.
// One thread per 16-byte piece of an output row, eight image rows per CTA; CP is a template
// parameter so that the index arithmetic is shifts, and reads of one channel are contiguous
// along w.
template <int CP, bool F16>
__global__ void __launch_bounds__(256) pad_input_kernel(const float *__restrict__ x, bf16 *__restrict__ out, int C,
                                 int H, int W, int Wp, int pad_w, int64_t rows_total) {
  constexpr int ROWS = 8;                        // image rows per CTA
  const int pieces_row = Wp * CP / 8;
  const int64_t plane = (int64_t)H * W;
  for (int pc = threadIdx.x; pc < pieces_row; pc += blockDim.x) {
    // source column and channel of the piece's eight values (the same for every row)
    int col[8];
    bool on[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int e = pc * 8 + u;
      const int c = e % CP, w = e / CP - pad_w;
      on[u] = c < C && w >= 0 && w < W;
      col[u] = on[u] ? (int)(c * plane + w) : 0;
    }
#pragma unroll 4
    for (int rr = 0; rr < ROWS; ++rr) {
      const int64_t nh = (int64_t)blockIdx.x * ROWS + rr;     // n * H + h
      if (nh >= rows_total) break;
      const int64_t n = nh / H;
      const int h = (int)(nh - n * H);
      const float *xin = x + (n * C * H + h) * (int64_t)W;
      float f[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) f[u] = on[u] ? xin[col[u]] : 0.0f;
      uint4 pk;
      pk.x = f32_to_pair<F16>(f[0], f[1]);
      pk.y = f32_to_pair<F16>(f[2], f[3]);
      pk.z = f32_to_pair<F16>(f[4], f[5]);
      pk.w = f32_to_pair<F16>(f[6], f[7]);
      *reinterpret_cast<uint4 *>(out + (nh * Wp * CP) + (int64_t)pc * 8) = pk;
    }
  }
}

void launch_pad_input_bf16(const float *x, bf16 *out, int N, int C, int H, int W, int Wp, int Cp,
                           int pad_w, bool f16, cudaStream_t s) {
  const int pieces_row = Wp * Cp / 8;
  if ((int64_t)N * H * pieces_row == 0) return;
  const int threads = pieces_row >= 256 ? 256 : (pieces_row + 31) / 32 * 32;
  const int64_t rows = (int64_t)N * H;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  auto go = [&](auto kern) { kern<<<grid, threads, 0, s>>>(x, out, C, H, W, Wp, pad_w, rows); };
  if (f16) {
    if (Cp == 4) go(pad_input_kernel<4, true>);
    else if (Cp == 8) go(pad_input_kernel<8, true>);
    else go(pad_input_kernel<16, true>);
  } else {
    if (Cp == 4) go(pad_input_kernel<4, false>);
    else if (Cp == 8) go(pad_input_kernel<8, false>);
    else go(pad_input_kernel<16, false>);
  }
  count(CNT_LAUNCHES);
}

}  // namespace occ
