// occamy_conv_bias_act_noalloc: the fused convolution for callers that must not allocate.
//
// The regular DNNConvBiasActivFunc keeps its working copies (the NHWC bf16 form of an
// fp32 NCHW input, the packed filter, the NHWC bf16 result before it is turned back into
// the ABI's layout) in scratch blocks that it obtains from cudaMalloc and grows on demand.
// Some hosts cannot do that at the point where they call us: code running inside a
// pre-sized memory budget where every device byte is accounted for before start-up, and
// latency-critical loops that may not enter the driver's allocator (cudaMalloc takes
// process-wide locks and can synchronise the device).  For them this file holds the same
// computation with its scratch in a fixed array that is part of the library image.
//
// Limits and rules:
//   * the scratch is OCCAMY_NOALLOC_SCRATCH_BYTES (32 MiB) per GPU that loads the library,
//     held from load to exit whether or not the entry point is ever called;
//   * a problem whose working copies do not fit is rejected with code -2 and a message;
//     nothing is launched in that case;
//   * every call uses the same array: two calls whose kernels can overlap on the GPU
//     (different streams, no dependency between them) race on it.  Issue them on one stream
//     or order them with events;
//   * the first call on a device looks up the array's device address
//     (cudaGetSymbolAddress) and the SM count; make that first call outside any stream
//     capture.  That set-up is guarded (once per device, safe against two host threads making
//     the first call together); the calls themselves share one array, so serialise them;
//   * a kernel whose bounded waits ran out (codes 1001..1006) reports into a word kept in the
//     last 256 bytes of the array.  A call never clears that word, so a report survives
//     until occamy_noalloc_last_error() - or occamy_last_error() / occamy_synchronize() of the
//     regular API - has read it; after such a report y holds garbage;
//   * no cudaMalloc / cudaFree / allocating library call is made, by any call.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <climits>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "kernels.h"
#include "runtime.h"

#define OCCAMY_NOALLOC_SCRATCH_BYTES (32u << 20)
#define OCCAMY_NOALLOC_MAX_DEVICES 16
// The kernels' error word sits at a fixed place, the last 256 bytes of the array; the working
// copies are carved out of the bytes before it.
#define OCCAMY_NOALLOC_ERR_OFFSET (OCCAMY_NOALLOC_SCRATCH_BYTES - 256u)

// File-scope device array.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is never passed to a kernel or used as an address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[OCCAMY_NOALLOC_SCRATCH_BYTES];

namespace {

using occ::bf16;

struct DeviceSetup {
  std::once_flag once;
  bool ready = false;
  unsigned char *scratch = nullptr;  // device address of g_noalloc_scratch on this device
  int num_sms = 0;
};
DeviceSetup g_setup[OCCAMY_NOALLOC_MAX_DEVICES];

// Once per device, with that device current: ask the runtime where this device's copy of
// the array lives.  The host-side symbol itself is not a device address.
void setup_device(DeviceSetup &su, int dev) {
  void *ptr = nullptr;
  cudaError_t ce = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
  if (ce != cudaSuccess || !ptr) {
    fprintf(stderr, "[occamy_b200] noalloc conv: cudaGetSymbolAddress failed (%s)\n",
            cudaGetErrorString(ce));
    return;
  }
  int sms = 0;
  ce = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (ce != cudaSuccess || sms <= 0) {
    fprintf(stderr, "[occamy_b200] noalloc conv: cannot read the SM count (%s)\n",
            cudaGetErrorString(ce));
    return;
  }
  su.scratch = static_cast<unsigned char *>(ptr);
  su.num_sms = sms;
  su.ready = true;
}

// fp32 NCHW -> bf16 NHWC, one thread per output element (c fastest: coalesced writes).
__global__ void na_nchw_to_nhwc(const float *__restrict__ x, bf16 *__restrict__ y, int C, int HW,
                                int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int64_t np = i / C;
    const int64_t n = np / HW, p = np % HW;
    y[i] = __float2bfloat16_rn(x[(n * C + c) * HW + p]);
  }
}

// bf16 NHWC -> fp32 NCHW, one thread per output element (pixel fastest: coalesced writes).
__global__ void na_nhwc_to_nchw(const bf16 *__restrict__ x, float *__restrict__ y, int C, int HW,
                                int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = i % HW;
    const int64_t nc = i / HW;
    const int64_t n = nc / C, c = nc % C;
    y[i] = __bfloat162float(x[(n * HW + p) * C + c]);
  }
}

// fp32 KCRS -> bf16 [R*S][K][C]
__global__ void na_pack_krsc(const float *__restrict__ w, bf16 *__restrict__ out, int K, int C,
                             int RS, int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const int k = (int)((i / C) % K);
    const int t = (int)(i / ((int64_t)C * K));
    out[i] = __float2bfloat16_rn(w[((int64_t)k * C + c) * RS + t]);
  }
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline int blocks_for(int64_t n, int num_sms) {
  int64_t b = (n + 255) / 256;
  const int64_t cap = (int64_t)num_sms * 32;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

extern "C" int occamy_conv_bias_act_noalloc(const float *x, const int64_t dimX[4], const float *w,
                                            const int64_t dimW[4], const float *bias,
                                            const int64_t pads[2], const int64_t strides[2],
                                            int64_t activMode, float *y, cudaStream_t stream) {
  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess || dev < 0 || dev >= OCCAMY_NOALLOC_MAX_DEVICES) {
    fprintf(stderr, "[occamy_b200] noalloc conv: no usable current device (%s)\n",
            cudaGetErrorString(ce));
    return -1;
  }
  DeviceSetup &su = g_setup[dev];
  std::call_once(su.once, setup_device, std::ref(su), dev);
  if (!su.ready) return -1;

  // every extent is checked as a 64-bit value before it is narrowed
  for (int i = 0; i < 4; ++i)
    if (dimX[i] <= 0 || dimX[i] > INT_MAX || dimW[i] <= 0 || dimW[i] > INT_MAX) {
      fprintf(stderr, "[occamy_b200] noalloc conv: extent out of range\n");
      return -3;
    }
  for (int i = 0; i < 2; ++i)
    if (pads[i] < 0 || pads[i] > 1024 || strides[i] < 1 || strides[i] > 1024) {
      fprintf(stderr, "[occamy_b200] noalloc conv: pad / stride out of range\n");
      return -3;
    }
  const int N = (int)dimX[0], C = (int)dimX[1], H = (int)dimX[2], W = (int)dimX[3];
  const int K = (int)dimW[0], R = (int)dimW[2], S = (int)dimW[3];
  const int ph = (int)pads[0], pw = (int)pads[1], sh = (int)strides[0], sw = (int)strides[1];
  if (dimW[1] != C) {
    fprintf(stderr, "[occamy_b200] noalloc conv: inconsistent shape\n");
    return -3;
  }
  if ((int64_t)H + 2 * ph < R || (int64_t)W + 2 * pw < S) {   // the filter does not fit once
    fprintf(stderr, "[occamy_b200] noalloc conv: empty output\n");
    return -3;
  }
  const int P = (H + 2 * ph - R) / sh + 1, Q = (W + 2 * pw - S) / sw + 1;
  int act;
  float lo = 0.f, hi = 0.f;
  if (activMode == 1) act = occ::ACT_RELU;
  else if (activMode == 3) { act = occ::ACT_CLIP; hi = 6.f; }
  else if (activMode == 5) act = occ::ACT_IDENTITY;
  else {
    fprintf(stderr, "[occamy_b200] noalloc conv: activation mode %lld not supported (1, 3, 5)\n",
            (long long)activMode);
    return -3;
  }

  // carve the fixed array: [x as NHWC bf16][packed filter][y as NHWC bf16] ... [error word]
  const size_t x_bytes = align_up((size_t)N * C * H * W * 2, 1024);
  const size_t w_bytes = align_up((size_t)R * S * K * C * 2, 1024);
  const size_t y_bytes = align_up((size_t)N * K * P * Q * 2, 1024);
  const size_t need = x_bytes + w_bytes + y_bytes;
  if (need > OCCAMY_NOALLOC_ERR_OFFSET) {
    fprintf(stderr,
            "[occamy_b200] noalloc conv: needs %zu bytes of scratch, the fixed array holds %u "
            "(use DNNConvBiasActivFunc, which allocates, for problems of this size)\n",
            need, (unsigned)OCCAMY_NOALLOC_ERR_OFFSET);
    return -2;
  }
  bf16 *xs = reinterpret_cast<bf16 *>(su.scratch);
  bf16 *ws = reinterpret_cast<bf16 *>(su.scratch + x_bytes);
  bf16 *ys = reinterpret_cast<bf16 *>(su.scratch + x_bytes + w_bytes);
  int *err_word = reinterpret_cast<int *>(su.scratch + OCCAMY_NOALLOC_ERR_OFFSET);

  occ::TcConvArgs a;
  memset(&a, 0, sizeof(a));
  a.x = xs; a.w = ws; a.bias = bias; a.y = ys;
  a.N = N; a.H = H; a.W = W; a.Cf = C; a.K = K; a.P = P; a.Q = Q; a.R = R; a.S = S;
  a.pad_h = ph; a.pad_w = pw; a.stride_h = sh; a.stride_w = sw;
  a.act = act; a.lo = lo; a.hi = hi;
  if (C % 16 != 0 || K % 8 != 0 || !occ::tc_conv_supported(a)) {
    fprintf(stderr, "[occamy_b200] noalloc conv: shape outside the tensor-core kernel's range "
                    "(needs C %% 16 == 0, K %% 8 == 0, stride <= 2, at most 32 taps)\n");
    return -3;
  }

  // The array keeps whatever the previous call left.  The working copies are fully
  // overwritten before they are read; the error word is zero from load time on and is
  // deliberately NOT cleared here, so that a report of an earlier call is not lost.
  const int64_t xn = (int64_t)N * C * H * W, wn = (int64_t)R * S * K * C,
                yn = (int64_t)N * K * P * Q;
  na_nchw_to_nhwc<<<blocks_for(xn, su.num_sms), 256, 0, stream>>>(x, xs, C, H * W, xn);
  na_pack_krsc<<<blocks_for(wn, su.num_sms), 256, 0, stream>>>(w, ws, K, C, R * S, wn);
  if (!occ::launch_tc_conv_stateless(a, err_word, su.num_sms, stream)) {
    fprintf(stderr, "[occamy_b200] noalloc conv: kernel launch failed\n");
    return -4;
  }
  na_nhwc_to_nchw<<<blocks_for(yn, su.num_sms), 256, 0, stream>>>(ys, y, K, P * Q, yn);
  ce = cudaGetLastError();
  return ce == cudaSuccess ? 0 : (int)ce;
}

// Reads (and with `clear` resets) the error word of the current device's array: 0, or the
// code 1001..1006 of a kernel whose bounded wait ran out in some earlier call.  A plain
// blocking copy from the cached address: allocates nothing.  Synchronise the stream the calls
// went to first; a device on which the entry point was never called reports 0.
extern "C" int occamy_noalloc_last_error(int clear) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= OCCAMY_NOALLOC_MAX_DEVICES) return 0;
  DeviceSetup &su = g_setup[dev];
  if (!su.ready) return 0;
  int word = 0;
  if (cudaMemcpy(&word, su.scratch + OCCAMY_NOALLOC_ERR_OFFSET, sizeof(int),
                 cudaMemcpyDeviceToHost) != cudaSuccess)
    return -1;
  if (word && clear) cudaMemset(su.scratch + OCCAMY_NOALLOC_ERR_OFFSET, 0, sizeof(int));
  return word;
}

// Bytes of the fixed array that the working copies of one call may use.
extern "C" int64_t occamy_noalloc_capacity(void) { return (int64_t)OCCAMY_NOALLOC_ERR_OFFSET; }

namespace occ {
int noalloc_poll_error(bool clear) { return occamy_noalloc_last_error(clear ? 1 : 0); }
}  // namespace occ
