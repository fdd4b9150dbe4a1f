// Entry points of the ABI that the CNN graphs (ResNet / MobileNet / VGG) never reach:
// transposes, concat, gather, N-d matmul, casts and a few unary maps.  They exist so that
// any graph the Occamy compiler emits links and runs; they are correct and allocation-free
// (shapes travel as kernel arguments) but not tuned.
#include <cstring>

#include "kernels.h"
#include "runtime.h"

using namespace occ;

extern "C" void occamy_internal_opaque_call(void);

namespace {

inline int64_t prod(const int64_t *d, int64_t rank) {
  int64_t n = 1;
  for (int64_t i = 0; i < rank; ++i) n *= d[i];
  return n;
}
inline int blocks_for(int64_t n) {
  int64_t b = (n + 255) / 256;
  const int64_t cap = (int64_t)rt().num_sms * 32;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

enum Unary { U_ERF, U_LEAKY, U_NEG, U_RECIP, U_PRELU, U_POW };

__global__ void unary_kernel(const float *x, float *y, int64_t n, int op, float a,
                             const float *dev_scalar) {
  const float s = dev_scalar ? *dev_scalar : a;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float v = x[i];
    float r;
    switch (op) {
      case U_ERF: r = erff(v); break;
      case U_LEAKY: r = v >= 0.0f ? v : v * s; break;
      case U_PRELU: r = v >= 0.0f ? v : v * s; break;
      case U_NEG: r = -v; break;
      case U_RECIP: r = 1.0f / v; break;
      default: r = powf(v, s); break;
    }
    y[i] = r;
  }
}

float *unary(float *in, float *out, const int64_t *dim, int64_t rank, int op, float a,
             const float *dev_scalar) {
  occamy_internal_opaque_call();
  Runtime &r = rt();
  const int64_t n = prod(dim, rank);
  ensure_f32(in);
  if (dev_scalar) ensure_f32(dev_scalar);
  if (n) {
    unary_kernel<<<blocks_for(n), 256, 0, r.stream>>>(in, out, n, op, a, dev_scalar);
    count(CNT_LAUNCHES);
  }
  mark_f32(out);
  return out;
}

__global__ void cast_i64_f32_kernel(const int64_t *x, float *y, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    y[i] = (float)x[i];
}

struct PermShape {
  int rank;
  int64_t out_dim[8];
  int64_t in_stride[8];  // stride in the input of the axis that output axis d walks
};

template <typename T>
__global__ void permute_kernel(const T *x, T *y, PermShape ps, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, src = 0;
    for (int d = ps.rank - 1; d >= 0; --d) {
      src += (rem % ps.out_dim[d]) * ps.in_stride[d];
      rem /= ps.out_dim[d];
    }
    y[i] = x[src];
  }
}

template <typename T>
T *transpose(T *in, const int64_t *dimIn, T *out, const int64_t *perm, int64_t rank) {
  occamy_internal_opaque_call();
  Runtime &r = rt();
  if (rank > 8) {
    set_error(994, "transpose: rank > 8");
    return out;
  }
  ensure_f32(in);
  int64_t stride[8], s = 1;
  for (int i = (int)rank - 1; i >= 0; --i) {
    stride[i] = s;
    s *= dimIn[i];
  }
  PermShape ps;
  ps.rank = (int)rank;
  for (int d = 0; d < rank; ++d) {
    ps.out_dim[d] = dimIn[perm[d]];
    ps.in_stride[d] = stride[perm[d]];
  }
  if (s) {
    permute_kernel<T><<<blocks_for(s), 256, 0, r.stream>>>(in, out, ps, s);
    count(CNT_LAUNCHES);
  }
  mark_f32(out);
  return out;
}

// Copies one concat operand: rows of `inner_in` elements into rows of `inner_out`.
template <typename T>
__global__ void concat_copy_kernel(const T *x, T *y, int64_t inner_in, int64_t inner_out,
                                   int64_t offset, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    y[(i / inner_in) * inner_out + offset + i % inner_in] = x[i];
}

template <typename T>
T *concat(T **inList, int64_t **dimInList, T *out, const int64_t *dimOut, int64_t axis,
          int64_t inputNum, int32_t rank) {
  occamy_internal_opaque_call();
  Runtime &r = rt();
  if (axis < 0) axis += rank;
  int64_t inner_out = 1;
  for (int i = (int)axis; i < rank; ++i) inner_out *= dimOut[i];
  int64_t offset = 0;
  for (int64_t k = 0; k < inputNum; ++k) {
    const int64_t *d = dimInList[k];
    int64_t inner_in = 1;
    for (int i = (int)axis; i < rank; ++i) inner_in *= d[i];
    const int64_t n = prod(d, rank);
    ensure_f32(inList[k]);
    if (n) {
      concat_copy_kernel<T><<<blocks_for(n), 256, 0, r.stream>>>(inList[k], out, inner_in,
                                                                inner_out, offset, n);
      count(CNT_LAUNCHES);
    }
    offset += inner_in;
  }
  mark_f32(out);
  return out;
}

// out[o, j, i] = in[o, idx[j], i]   (o over dims before `axis`, i over dims after it)
template <typename T>
__global__ void gather_kernel(const T *x, const int64_t *idx, T *y, int64_t axis_dim,
                              int64_t nidx, int64_t inner, int64_t n) {
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = t % inner, j = (t / inner) % nidx, o = t / (inner * nidx);
    int64_t k = idx[j];
    if (k < 0) k += axis_dim;
    y[t] = x[(o * axis_dim + k) * inner + i];
  }
}

template <typename T>
T *gather(T *in, const int64_t *dimIn, int64_t inRank, T *out, int64_t *indices,
          const int64_t *dimIdx, int64_t idxRank, int64_t axis) {
  occamy_internal_opaque_call();
  Runtime &r = rt();
  if (axis < 0) axis += inRank;
  int64_t outer = 1, inner = 1;
  for (int64_t i = 0; i < axis; ++i) outer *= dimIn[i];
  for (int64_t i = axis + 1; i < inRank; ++i) inner *= dimIn[i];
  const int64_t nidx = prod(dimIdx, idxRank);
  const int64_t n = outer * nidx * inner;
  ensure_f32(in);
  ensure_f32(indices);
  if (n) {
    gather_kernel<T><<<blocks_for(n), 256, 0, r.stream>>>(in, indices, out, dimIn[axis], nidx,
                                                         inner, n);
    count(CNT_LAUNCHES);
  }
  mark_f32(out);
  return out;
}

// Indices (as T) of the non-zero elements, in order: one CTA walks the tensor in chunks of
// blockDim.x, ranks the non-zeros of a chunk with a ballot / popcount scan.
template <typename T>
__global__ void nonzero_kernel(const T *x, T *y, int64_t n) {
  __shared__ int warp_cnt[32];
  __shared__ int64_t base;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  for (int64_t c0 = 0; c0 < n; c0 += blockDim.x) {
    const int64_t i = c0 + threadIdx.x;
    const bool nz = i < n && x[i] != (T)0;
    const unsigned m = __ballot_sync(0xffffffffu, nz);
    if (lane == 0) warp_cnt[wid] = __popc(m);
    __syncthreads();
    int before = 0, total = 0;
    for (int w = 0; w < nw; ++w) {
      if (w < wid) before += warp_cnt[w];
      total += warp_cnt[w];
    }
    if (nz) y[base + before + __popc(m & ((1u << lane) - 1u))] = (T)i;
    __syncthreads();
    if (threadIdx.x == 0) base += total;
    __syncthreads();
  }
}

template <typename T>
T *nonzero(T *in, const int64_t *dimIn, T *out, int64_t rank) {
  occamy_internal_opaque_call();
  Runtime &r = rt();
  const int64_t n = prod(dimIn, rank);
  ensure_f32(in);
  ensure_f32(out);  // entries past the number of non-zeros keep the buffer's zero fill
  if (n) {
    nonzero_kernel<T><<<1, 1024, 0, r.stream>>>(in, out, n);
    count(CNT_LAUNCHES);
  }
  return out;
}

template <typename T>
T *plain_copy(T *in, const int64_t *dimIn, int64_t rank, T *out) {
  occamy_internal_opaque_call();
  Runtime &r = rt();
  const int64_t n = prod(dimIn, rank);
  ensure_f32(in);
  if (n) OCC_CUDA(cudaMemcpyAsync(out, in, (size_t)n * sizeof(T), cudaMemcpyDeviceToDevice, r.stream));
  mark_f32(out);
  return out;
}

// Batched row-major matmul.  An operand with fewer leading (batch) dimensions than the output
// is indexed by the trailing batch indices only, i.e. its batch index wraps - the broadcast
// rule of the reference kernel (cuda/CUDAMatmulNdFunc.cu:49-58).
__global__ void matmul_nd_kernel(const float *A, const float *B, float *out, int M, int N, int K,
                                 int64_t batchA, int64_t batchB, int64_t total) {
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int n = (int)(t % N), m = (int)((t / N) % M);
    const int64_t b = t / ((int64_t)M * N);
    const float *a = A + ((b % batchA) * M + m) * (int64_t)K;
    const float *bb = B + (b % batchB) * (int64_t)K * N + n;
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) acc = fmaf(a[k], bb[(int64_t)k * N], acc);
    out[t] = acc;
  }
}

}  // namespace

extern "C" {

int64_t *CUDACastI64toFloatFunc(int64_t *in, float *out, int64_t *dimOut, int64_t rank) {
  occamy_internal_opaque_call();
  Runtime &r = rt();
  const int64_t n = prod(dimOut, rank);
  ensure_f32(in);
  if (n) {
    cast_i64_f32_kernel<<<blocks_for(n), 256, 0, r.stream>>>(in, out, n);
    count(CNT_LAUNCHES);
  }
  mark_f32(out);
  return in;  // as the reference does
}

float *CUDAErfFunc(float *in, float *out, int64_t *dimOut, int64_t rank) {
  return unary(in, out, dimOut, rank, U_ERF, 0.f, nullptr);
}
float *CUDALeakyReluFunc(float *in, float *out, int64_t *dimOut, float alpha, int64_t rank) {
  return unary(in, out, dimOut, rank, U_LEAKY, alpha, nullptr);
}
float *CUDANegativeFunc(float *in, float *out, int64_t *dimIn, int64_t rank) {
  return unary(in, out, dimIn, rank, U_NEG, 0.f, nullptr);
}
float *CUDAReciprocalFunc(float *in, float *out, int64_t *dimIn, int64_t rank) {
  return unary(in, out, dimIn, rank, U_RECIP, 0.f, nullptr);
}
float *CUDAPReluFunc(float *in, float *out, int64_t *dimOut, float *slope, int64_t rank) {
  return unary(in, out, dimOut, rank, U_PRELU, 0.f, slope);
}
float *CUDAPowFunc(float *in, float *exponent_d, float *out, int64_t *dimOut, int64_t rank) {
  return unary(in, out, dimOut, rank, U_POW, 0.f, exponent_d);
}

float *CUDAConcatFloatFunc(float **inList, int64_t **dimInList, float *out, int64_t *dimOut,
                           int64_t axis, int64_t inputNum, int32_t inputRank) {
  return concat<float>(inList, dimInList, out, dimOut, axis, inputNum, inputRank);
}
int64_t *CUDAConcatInt64Func(int64_t **inList, int64_t **dimInList, int64_t *out, int64_t *dimOut,
                             int64_t axis, int64_t inputNum, int32_t inputRank) {
  return concat<int64_t>(inList, dimInList, out, dimOut, axis, inputNum, inputRank);
}

int64_t *CUDAExpandInt64Func(int64_t *in, int64_t *dimIn, int64_t inRank, int64_t *out,
                             int64_t * /*dimOut*/, int64_t * /*shape_d*/, int64_t * /*dimShape*/) {
  return plain_copy<int64_t>(in, dimIn, inRank, out);
}

float *CUDAGatherFloatFunc(float *in, int64_t *dimIn, int64_t inRank, float *out,
                           int64_t * /*dimOut*/, int64_t /*outRank*/, int64_t *indices_d,
                           int64_t *dimIdx, int64_t idxRank, int64_t axis) {
  return gather<float>(in, dimIn, inRank, out, indices_d, dimIdx, idxRank, axis);
}
int64_t *CUDAGatherInt64Func(int64_t *in, int64_t *dimIn, int64_t inRank, int64_t *out,
                             int64_t * /*dimOut*/, int64_t /*outRank*/, int64_t *indices_d,
                             int64_t *dimIdx, int64_t idxRank, int64_t axis) {
  return gather<int64_t>(in, dimIn, inRank, out, indices_d, dimIdx, idxRank, axis);
}

float *CUDAMatmulNdFunc(float *A, int64_t *dimA, int32_t rankA, float *B, int64_t *dimB,
                        int32_t rankB, float *out, int64_t *dimOut, int32_t rankOut) {
  occamy_internal_opaque_call();
  Runtime &r = rt();
  if (rankA < 2 || rankB < 2) {
    set_error(993, "matmulNd: rank < 2");
    return out;
  }
  const int M = (int)dimA[rankA - 2], K = (int)dimA[rankA - 1], N = (int)dimB[rankB - 1];
  int64_t batchA = prod(dimA, rankA - 2), batchB = prod(dimB, rankB - 2);
  if (batchA < 1) batchA = 1;
  if (batchB < 1) batchB = 1;
  const int64_t total = prod(dimOut, rankOut);
  ensure_f32(A);
  ensure_f32(B);
  if (total) {
    matmul_nd_kernel<<<blocks_for(total), 256, 0, r.stream>>>(A, B, out, M, N, K, batchA, batchB, total);
    count(CNT_LAUNCHES);
  }
  mark_f32(out);
  return out;
}

float *CUDANonZeroFloatFunc(float *in, int64_t *dimIn, float *out, int64_t * /*dimOut*/,
                            int64_t rank) {
  return nonzero<float>(in, dimIn, out, rank);
}
int64_t *CUDANonZeroInt64Func(int64_t *in, int64_t *dimIn, int64_t *out, int64_t * /*dimOut*/,
                              int64_t rank) {
  return nonzero<int64_t>(in, dimIn, out, rank);
}

float *CUDASqueezeFloatFunc(float *in, int64_t *dimIn, float *out, int64_t *, int32_t,
                            int64_t rank) {
  return plain_copy<float>(in, dimIn, rank, out);
}
int64_t *CUDASqueezeInt64Func(int64_t *in, int64_t *dimIn, int64_t *out, int64_t *, int32_t,
                              int64_t rank) {
  return plain_copy<int64_t>(in, dimIn, rank, out);
}
float *CUDAUnsqueezeFloatFunc(float *in, int64_t *dimIn, float *out, int64_t *, int32_t,
                              int64_t rank) {
  return plain_copy<float>(in, dimIn, rank, out);
}
int64_t *CUDAUnsqueezeInt64Func(int64_t *in, int64_t *dimIn, int64_t *out, int64_t *, int32_t,
                                int64_t rank) {
  return plain_copy<int64_t>(in, dimIn, rank, out);
}

#define OCC_TRANSPOSE(NAME, T)                                                               \
  T *NAME(T *in, int64_t *dimIn, T *out, int64_t * /*dimOut*/, int64_t *perm, int64_t rank) { \
    return transpose<T>(in, dimIn, out, perm, rank);                                          \
  }
OCC_TRANSPOSE(CUDATranspose2DFloatFunc, float)
OCC_TRANSPOSE(CUDATranspose3DFloatFunc, float)
OCC_TRANSPOSE(CUDATranspose4DFloatFunc, float)
OCC_TRANSPOSE(CUDATranspose6DFloatFunc, float)
OCC_TRANSPOSE(CUDATranspose2DInt64Func, int64_t)
OCC_TRANSPOSE(CUDATranspose3DInt64Func, int64_t)
OCC_TRANSPOSE(CUDATranspose4DInt64Func, int64_t)
OCC_TRANSPOSE(CUDATranspose6DInt64Func, int64_t)

}  // extern "C"
