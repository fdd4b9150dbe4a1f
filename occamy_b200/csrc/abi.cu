// The C-ABI entry points on the CNN hot path (declared in include/occamy_dnn_api.h) and
// the dispatch between the fp32 NCHW kernels and the bf16 NHWC / tensor-core kernels.
#include <cstring>
#include <vector>

#include "kernels.h"
#include "runtime.h"
#include "trace.h"

#define OCCAMY_NO_VENDOR_TYPES
typedef cudaError_t occamy_cuda_error_t;
struct cudnnContext;
typedef struct cudnnContext *cudnnHandle_t;
#include "../../include/occamy_dnn_api.h"

using namespace occ;

namespace {

struct PoolRec {
  void *base;
  size_t bytes;
};
std::vector<PoolRec> g_pools;
// Pool blocks of finished inferences, kept so that the next wrapDNNMemPoolInit of the same
// size costs no cudaMalloc / cudaFree (a compiled model creates and frees its pool on every
// call).  Up to OCCAMY_POOL_BLOCKS (default 2, 0 = off) blocks of one size are kept and
// handed out in turn: consecutive inferences then live in different blocks, and the input
// upload of the next one can run on the copy stream while the kernels of the current one
// are still executing.
struct CachedPool {
  void *base;
  size_t bytes;
  cudaEvent_t done;   // recorded on the launch stream when the block's last user finished
};
std::vector<CachedPool> g_pool_cache;   // oldest first
cudaEvent_t g_block_ready = nullptr;    // `done` of the block the current inference lives in
void *g_cur_pool = nullptr;
size_t g_cur_pool_bytes = 0;
cudaStream_t g_copy_stream = nullptr;
int64_t g_launches_at_pool_init = 0;   // kernel + copy count when the current pool was set up

int pool_cache_blocks() {
  static int v = -1;
  if (v < 0) {
    const char *e = getenv("OCCAMY_POOL_BLOCKS");
    if (!e) e = getenv("OCCAMY_POOL_CACHE");
    v = e ? atoi(e) : 2;
    if (v < 0) v = 0;
    if (v > 4) v = 4;
  }
  return v;
}

void free_cached_pool(CachedPool &c) {
  OCC_CUDA(cudaEventSynchronize(c.done));
  OCC_CUDA(cudaFree(c.base));
  OCC_CUDA(cudaEventDestroy(c.done));
}

void die(const char *what, cudaError_t e, size_t size) {
  // Same convention as the reference's memory wrappers (cuda/wrapDNNMalloc.cpp:11-16).
  printf("[%s] GPU error: (size: %zu) %s\n", what, size, cudaGetErrorString(e));
  exit(-1);
}

enum PackLayout { PACK_KRSC = 1, PACK_DW = 2, PACK_FOLD = 3, PACK_RAW = 4, PACK_STEM = 5, PACK_SPLIT = 6 };
// fp32 mode: dense convolutions and GEMMs on the tensor cores with split operands (see
// launch_split3_nchw); off with OCCAMY_FP32_TC=0 or occamy_set_fp32_tensor_cores(0), which
// leaves the CUDA-core kernels.
int g_fp32_tc = -1;
bool fp32_tc_enabled() {
  if (g_fp32_tc < 0) {
    const char *e = getenv("OCCAMY_FP32_TC");
    g_fp32_tc = (e && !strcmp(e, "0")) ? 0 : 1;
  }
  return g_fp32_tc == 1;
}

// Device pointer of the packed form of the filter at `w`; resident across calls when the
// filter was uploaded from host memory (a compiled model's constant), otherwise packed
// into scratch.  `packed_bytes` is the size of the packed form.
// Set by packed_weights: the returned copy was already on the device before this call (no
// kernel or copy was enqueued to produce it).
bool g_pack_was_resident = false;

void *packed_weights(const float *w, int layout, size_t packed_bytes, int K, int C, int R, int S,
                     int Sp, int Cp) {
  Runtime &r = rt();
  g_pack_was_resident = false;
  uintptr_t base;
  TensorRec *rec = reg_find(w, &base);
  const bool cacheable = r.cache_weights && rec && base == (uintptr_t)w && rec->host_src;
  // fp32 layouts are shared by the two 16-bit modes, 16-bit ones are packed per element type
  const bool f16 = mode_f16() && layout != PACK_DW && layout != PACK_RAW && layout != PACK_SPLIT;
  WeightKey key{nullptr, 0, layout * 4096 + Sp * 64 + Cp + (f16 ? (1 << 20) : 0)};
  if (cacheable) {
    key.src = rec->host_src;
    key.bytes = rec->host_bytes;
    auto it = r.wcache.find(key);
    if (it != r.wcache.end() && it->second.hash == rec->host_hash && it->second.bytes == packed_bytes) {
      g_pack_was_resident = true;
      return it->second.dev;
    }
  }
  ensure_f32(w);
  void *dst = nullptr;
  if (cacheable) {
    PackedWeight &pw = r.wcache[key];
    if (pw.dev && pw.bytes != packed_bytes) {
      OCC_CUDA(cudaStreamSynchronize(r.stream));
      OCC_CUDA(cudaFree(pw.dev));
      pw.dev = nullptr;
    }
    if (!pw.dev) OCC_CUDA(cudaMalloc(&pw.dev, packed_bytes));
    pw.bytes = packed_bytes;
    pw.hash = rec->host_hash;
    pw.layout = layout;
    dst = pw.dev;
    r.resident[rec->host_src] = std::make_pair(rec->host_bytes, rec->host_hash);
  } else {
    dst = scratch_get(layout == PACK_STEM ? 5 : 1, packed_bytes);
  }
  if (!dst) return nullptr;
  if (layout == PACK_KRSC) launch_pack_krsc_bf16(w, (bf16 *)dst, K, C, R, S, Cp, f16, r.stream);
  else if (layout == PACK_DW) launch_pack_dw_f32(w, (float *)dst, C, R, S, r.stream);
  else if (layout == PACK_RAW)
    OCC_CUDA(cudaMemcpyAsync(dst, w, packed_bytes, cudaMemcpyDeviceToDevice, r.stream));
  else if (layout == PACK_STEM) launch_pack_stem_bf16(w, (bf16 *)dst, C, R, S, Cp, Sp * Cp, r.stream);
  else if (layout == PACK_SPLIT) launch_pack_krsc_split(w, (bf16 *)dst, K, C, R, S, Cp, r.stream);
  else launch_pack_fold_bf16(w, (bf16 *)dst, K, C, R, S, Sp, Cp, f16, r.stream);
  return dst;
}

// Small fp32 constants (biases): the resident copy when there is one, else the tensor itself.
const float *resident_f32(const float *p, size_t bytes) {
  uintptr_t base;
  TensorRec *rec = reg_find(p, &base);
  if (rt().cache_weights && rec && base == (uintptr_t)p && rec->host_src && rec->host_bytes == bytes) {
    const float *d = (const float *)packed_weights(p, PACK_RAW, bytes, 0, 0, 0, 0, 0, 0);
    if (d) return d;
  }
  g_pack_was_resident = false;
  ensure_f32(p);
  return p;
}

// ---- a convolution resolved down to launch arguments ------------------------------
// `prepare_*` does everything that depends on the inputs' current state (layout
// conversion into scratch, packed-weight lookup, bias lookup); what is left is a launch
// that only needs to be told where to write, which residual to add and how to clamp.
struct ConvJob {
  bool active = false;
  bool depthwise = false;
  ConvGeom g;
  TcConvArgs a;               // dense: tensor-core arguments (x, w, bias resolved)
  const bf16 *dw_x = nullptr; // depthwise
  const float *dw_w = nullptr;
  const float *bias = nullptr;
  float *out = nullptr;       // tensor the result goes to
  bool bias_set = false, res_set = false, act_set = false;
  int absorbed = 0;           // later calls folded into this one so far
  // device ranges still to be read: [0] input, [1] residual operand, [2] a bias that is read
  // from the caller's tensor (no resident copy exists)
  uintptr_t dep_lo[3] = {0, 0, 0}, dep_hi[3] = {0, 0, 0};
  // folded (few-channel) form: what the fused convolution + pool kernel needs besides `a`
  const bf16 *w_stem = nullptr;   // filter in that kernel's layout, packed while the filter is live
};

ConvJob g_pending;  // convolution held back while later calls are folded into it

// A bias without a resident copy is read from the caller's tensor when the (possibly held-back)
// kernel finally runs: until then that tensor must neither be freed nor overwritten.
void job_track_bias(ConvJob &job, const float *used, const float *callers, int channels) {
  job.dep_lo[2] = job.dep_hi[2] = 0;
  if (used && used == callers) {
    job.dep_lo[2] = (uintptr_t)callers;
    job.dep_hi[2] = (uintptr_t)callers + (size_t)channels * 4;
  }
}

bool prepare_dense(const float *x, const float *w, const float *bias, const ConvGeom &g,
                   ConvJob &job) {
  Runtime &r = rt();
  if (g.groups != 1 || g.K % 8 != 0) return false;
  if (g.act != ACT_IDENTITY && g.act != ACT_RELU && g.act != ACT_CLIP) return false;
  TcConvArgs &a = job.a;
  memset(&a, 0, sizeof(a));
  a.N = g.N; a.K = g.K; a.P = g.P; a.Q = g.Q;
  a.act = g.act; a.lo = g.lo; a.hi = g.hi;
  a.f16 = mode_f16() ? 1 : 0;
  const bool folded = g.C < 16;
  int Sp = 0, Cp = 0, Wp = 0;
  if (folded) {
    // channels padded so that one output column's step along the row is a multiple of 16 bytes
    Cp = g.C <= 4 ? (g.stride_w % 2 == 0 ? 4 : 8) : (g.C <= 8 ? 8 : 16);
    const int unit = 16 / Cp;
    Sp = (g.S + unit - 1) / unit * unit;
    Wp = g.pad_w + g.W;
    if (Wp < (g.Q - 1) * g.stride_w + Sp) Wp = (g.Q - 1) * g.stride_w + Sp;
    Wp = (Wp + 7) / 8 * 8;
    a.H = g.H; a.W = g.Q; a.Cf = Sp * Cp;
    a.R = g.R; a.S = 1;
    a.pad_h = g.pad_h; a.pad_w = 0; a.stride_h = g.stride_h; a.stride_w = 1;
    a.w_step = g.stride_w * Cp;
    a.row_elems = Wp * Cp;
  } else {
    if (g.C % 8 != 0) return false;
    // Pixels are padded to a multiple of 32 bytes with zero channels: rows at a 48-byte pitch
    // (24 channels) load at little more than half the speed of rows at 64 (measured:
    // 24->144 at 56x56, 0.044 ms padded, 0.072 ms not).
    Cp = (g.C + 15) / 16 * 16;
    a.H = g.H; a.W = g.W; a.Cf = Cp;
    a.R = g.R; a.S = g.S;
    a.pad_h = g.pad_h; a.pad_w = g.pad_w; a.stride_h = g.stride_h; a.stride_w = g.stride_w;
  }
  a.x = (const bf16 *)16;  // placeholders so the support check sees aligned pointers
  a.w = (const bf16 *)16;
  a.y = (bf16 *)16;
  if (!tc_conv_supported(a)) return false;

  job.dep_lo[0] = job.dep_hi[0] = 0;
  if (folded) {
    ensure_f32(x);
    bf16 *xf = (bf16 *)scratch_get(0, (size_t)g.N * g.H * Wp * Cp * 2);
    if (!xf) return false;
    launch_pad_input_bf16(x, xf, g.N, g.C, g.H, g.W, Wp, Cp, g.pad_w, mode_f16(), r.stream);
    a.x = xf;
    a.w = (const bf16 *)packed_weights(w, PACK_FOLD, (size_t)g.R * g.K * a.Cf * 2, g.K, g.C, g.R,
                                       g.S, Sp, Cp);
  } else {
    const bf16 *xb = nullptr;
    if (is_act16(x, g.N, g.C, g.H, g.W)) {
      xb = (const bf16 *)x;
      if (Cp == g.C) {
        job.dep_lo[0] = (uintptr_t)x;
        job.dep_hi[0] = (uintptr_t)x + (size_t)g.N * g.C * g.H * g.W * 2;
      }
    } else {
      ensure_f32(x);
      bf16 *xc = (bf16 *)scratch_get(0, (size_t)g.N * g.C * g.H * g.W * 2);
      if (!xc) return false;
      launch_nchw_f32_to_nhwc_bf16(x, xc, g.N, g.C, g.H, g.W, mode_f16(), r.stream);
      xb = xc;
    }
    if (Cp != g.C) {   // the kernel reads the padded copy, made now: no dependence on x later
      bf16 *xp = (bf16 *)scratch_get(6, (size_t)g.N * Cp * g.H * g.W * 2);
      if (!xp) return false;
      launch_pad_channels_bf16(xb, xp, (int64_t)g.N * g.H * g.W, g.C, Cp, r.stream);
      xb = xp;
    }
    a.x = xb;
    a.w = (const bf16 *)packed_weights(w, PACK_KRSC, (size_t)g.R * g.S * g.K * Cp * 2, g.K, g.C,
                                       g.R, g.S, 0, Cp);
  }
  if (!a.w) return false;
  bool ready = g_pack_was_resident;
  a.bias = bias ? resident_f32(bias, (size_t)g.K * 4) : nullptr;
  if (bias) ready = ready && g_pack_was_resident;
  job_track_bias(job, a.bias, bias, g.K);
  // filter and bias were on the device before this call: the kernel may fetch them while the
  // kernel before it is still running
  a.consts_ready = ready ? 1 : 0;
  job.depthwise = false;
  job.g = g;
  job.bias_set = bias != nullptr;
  job.act_set = g.act != ACT_IDENTITY;
  job.res_set = false;
  job.w_stem = nullptr;
  return true;
}

bool prepare_depthwise(const float *x, const float *w, const float *bias, const ConvGeom &g,
                       ConvJob &job) {
  Runtime &r = rt();
  if (g.C % 8 != 0) return false;
  job.dep_lo[0] = job.dep_hi[0] = 0;
  if (is_act16(x, g.N, g.C, g.H, g.W)) {
    job.dw_x = (const bf16 *)x;
    job.dep_lo[0] = (uintptr_t)x;
    job.dep_hi[0] = (uintptr_t)x + (size_t)g.N * g.C * g.H * g.W * 2;
  } else {
    ensure_f32(x);
    bf16 *xc = (bf16 *)scratch_get(0, (size_t)g.N * g.C * g.H * g.W * 2);
    if (!xc) return false;
    launch_nchw_f32_to_nhwc_bf16(x, xc, g.N, g.C, g.H, g.W, mode_f16(), r.stream);
    job.dw_x = xc;
  }
  job.dw_w = (const float *)packed_weights(w, PACK_DW, (size_t)g.R * g.S * g.C * 4, g.K, g.C, g.R,
                                          g.S, 0, 0);
  if (!job.dw_w) return false;
  job.bias = bias ? resident_f32(bias, (size_t)g.C * 4) : nullptr;
  job_track_bias(job, job.bias, bias, g.C);
  job.depthwise = true;
  job.g = g;
  job.bias_set = bias != nullptr;
  job.act_set = g.act != ACT_IDENTITY;
  job.res_set = false;
  return true;
}

bool ranges_overlap(uintptr_t alo, uintptr_t ahi, uintptr_t blo, uintptr_t bhi) {
  return ahi > alo && bhi > blo && alo < bhi && blo < ahi;
}

void launch_job(ConvJob &job) {
  Runtime &r = rt();
  const ConvGeom &g = job.g;
  // A convolution that was held back may find its output placed over memory it still has
  // to read (the planner reuses a tensor's bytes as soon as the recorded program no longer
  // needs them).  The input then moves to scratch first; a residual operand may stay only
  // if the output covers it exactly (each tile reads its residual before it is stored).
  const uintptr_t olo = (uintptr_t)job.out;
  const uintptr_t ohi = olo + (size_t)g.N * g.K * g.P * g.Q * 2;
  if (ranges_overlap(olo, ohi, job.dep_lo[0], job.dep_hi[0])) {
    const size_t bytes = job.dep_hi[0] - job.dep_lo[0];
    void *tmp = scratch_get(4, bytes);
    OCC_CUDA(cudaMemcpyAsync(tmp, (const void *)job.dep_lo[0], bytes, cudaMemcpyDeviceToDevice,
                             r.stream));
    if (job.depthwise) job.dw_x = (const bf16 *)tmp;
    else job.a.x = (const bf16 *)tmp;
    count(CNT_LAUNCHES);
  }
  if (ranges_overlap(olo, ohi, job.dep_lo[1], job.dep_hi[1]) &&
      !(olo == job.dep_lo[1] && ohi == job.dep_hi[1])) {
    const size_t bytes = job.dep_hi[1] - job.dep_lo[1];
    void *tmp = scratch_get(5, bytes);
    OCC_CUDA(cudaMemcpyAsync(tmp, (const void *)job.dep_lo[1], bytes, cudaMemcpyDeviceToDevice,
                             r.stream));
    job.a.residual = (const bf16 *)tmp;
    count(CNT_LAUNCHES);
  }
  if (ranges_overlap(olo, ohi, job.dep_lo[2], job.dep_hi[2])) {
    const size_t bytes = job.dep_hi[2] - job.dep_lo[2];
    void *tmp = scratch_get(7, bytes);
    OCC_CUDA(cudaMemcpyAsync(tmp, (const void *)job.dep_lo[2], bytes, cudaMemcpyDeviceToDevice,
                             r.stream));
    if (job.depthwise) job.bias = (const float *)tmp;
    else job.a.bias = (const float *)tmp;
    count(CNT_LAUNCHES);
  }
  if (job.depthwise) {
    launch_depthwise_bf16(job.dw_x, job.dw_w, job.bias, (bf16 *)job.out, g, mode_f16(), r.stream);
  } else {
    job.a.y = (bf16 *)job.out;
    job.a.act = g.act; job.a.lo = g.lo; job.a.hi = g.hi;
    launch_tc_conv(job.a, r.stream);
  }
  mark_act16(job.out, g.N, g.K, g.P, g.Q);
}

// Executes the held-back convolution as far as it has been built up.
void flush_pending() {
  if (!g_pending.active) return;
  g_pending.active = false;
  if (g_pending.absorbed) trace_count_chain();
  launch_job(g_pending);
}

// [p, p+bytes) is about to be overwritten or freed (`writes`), or merely handed out again:
// in the first case whatever still has to read it must run first.  Handing a range out
// writes nothing (its zero fill is lazy), so a held-back convolution may keep reading its
// inputs from it; launch_job() deals with the case that its own output lands there.
void pending_guard_range(const void *p, size_t bytes, bool writes) {
  if (!g_pending.active) return;
  const uintptr_t lo = (uintptr_t)p, hi = lo + bytes;
  if (writes)
    for (int k = 0; k < 3; ++k)
      if (ranges_overlap(lo, hi, g_pending.dep_lo[k], g_pending.dep_hi[k])) {
        if (rt().log) fprintf(stderr, "[occamy] held-back conv runs early: input %d overwritten\n", k);
        flush_pending();
        return;
      }
  // the tensor it is going to write must also still belong to it
  const uintptr_t olo = (uintptr_t)g_pending.out;
  const uintptr_t ohi = olo + (size_t)g_pending.g.N * g_pending.g.K * g_pending.g.P * g_pending.g.Q * 2;
  if (ranges_overlap(lo, hi, olo, ohi)) {
    if (rt().log) fprintf(stderr, "[occamy] held-back conv runs early: output re-handed out\n");
    flush_pending();
  }
}

// Common tail of every traced entry point: record the call, end the speculation when the
// recorded sequence is left, run the held-back convolution unless this call continues it.
void before_write_hook(const void *p, size_t bytes) { pending_guard_range(p, bytes, true); }

Role step(Entry &e, bool passive) {
  rt().before_write = before_write_hook;
  bool deviated = false;
  const Role role = trace_step(e, &deviated);
  if (deviated) {
    flush_pending();
    // Tensors that fusion skipped earlier in this inference stay unwritten.  The recorded
    // program had no reader for them; should this (different) program read one, that read
    // reports error 990.  A shared prefix alone - two models with the same first layers - is
    // not an error.
    if (trace_has_elided() && rt().log)
      fprintf(stderr, "[occamy] call sequence left the recorded one after tensors were skipped\n");
  }
  if (!passive && role != R_ABSORB) {
    if (g_pending.active && rt().log)
      fprintf(stderr, "[occamy] held-back conv closed by call sym %d (absorbed %d)\n", e.sym,
              g_pending.absorbed);
    flush_pending();
  }
  return role;
}

void elide(void *p) {
  uintptr_t base;
  TensorRec *rec = reg_find(p, &base);
  if (rec && base == (uintptr_t)p) rec->fmt = FMT_ELIDED;
  trace_note_elided();
}

// fp32 mode on the tensor cores: x and the filter are carried as three bf16 parts each and the
// six part products that matter are accumulated in fp32 (TMEM); the result is written as the
// ABI's fp32 NCHW tensor by the kernel's epilogue.  False when the shape is outside what the
// kernel takes (the CUDA-core kernel runs then).
bool conv_f32_on_tensor_cores(const float *x, const float *w, const float *bias, const ConvGeom &g,
                              float *y) {
  Runtime &r = rt();
  if (g.groups != 1 || g.R * g.S * 6 > 64) return false;
  if (g.act != ACT_IDENTITY && g.act != ACT_RELU && g.act != ACT_CLIP) return false;
  const int Cp = (g.C + 15) / 16 * 16;
  TcConvArgs a;
  memset(&a, 0, sizeof(a));
  a.N = g.N; a.H = g.H; a.W = g.W; a.Cf = Cp; a.K = g.K; a.P = g.P; a.Q = g.Q; a.R = g.R; a.S = g.S;
  a.pad_h = g.pad_h; a.pad_w = g.pad_w; a.stride_h = g.stride_h; a.stride_w = g.stride_w;
  a.act = g.act; a.lo = g.lo; a.hi = g.hi;
  a.split = 1;
  a.out_f32 = y;
  a.out_nchw = 1;
  a.ldo = g.K;
  a.x = (const bf16 *)16;
  a.w = (const bf16 *)16;
  if (!tc_conv_supported(a)) return false;
  // Tiny problems stay on the CUDA-core kernel: three extra passes cost more than they save.
  if ((double)g.N * g.P * g.Q * g.K * g.C * g.R * g.S < 1e6) return false;
  ensure_f32(x);
  bf16 *xs = (bf16 *)scratch_get(0, (size_t)3 * g.N * g.H * g.W * Cp * 2);
  if (!xs) return false;
  launch_split3_nchw(x, xs, g.N, g.C, Cp, g.H, g.W, r.stream);
  const bf16 *ws = (const bf16 *)packed_weights(w, PACK_SPLIT, (size_t)6 * g.R * g.S * g.K * Cp * 2, g.K,
                                                 g.C, g.R, g.S, 0, Cp);
  if (!ws) return false;
  a.x = xs;
  a.w = ws;
  a.bias = bias ? resident_f32(bias, (size_t)g.K * 4) : nullptr;
  a.consts_ready = 0;
  launch_tc_conv(a, r.stream);
  mark_f32(y);
  return true;
}

float *conv_common(int sym, float *x, const int64_t *dX, float *w, const int64_t *dW, float *bias,
                   int64_t groups, const int64_t *pads, const int64_t *strides, int act, float lo,
                   float hi, int64_t act_mode, float *y) {
  Runtime &r = rt();
  ConvGeom g;
  g.N = (int)dX[0]; g.C = (int)dX[1]; g.H = (int)dX[2]; g.W = (int)dX[3];
  g.K = (int)dW[0]; g.R = (int)dW[2]; g.S = (int)dW[3];
  g.groups = (int)(groups < 1 ? 1 : groups);
  g.pad_h = (int)pads[0]; g.pad_w = (int)pads[1];
  g.stride_h = (int)strides[0]; g.stride_w = (int)strides[1];
  g.act = act; g.lo = lo; g.hi = hi;
  const bool shape_ok = !(g.stride_h < 1 || g.stride_w < 1 || g.C % g.groups || g.K % g.groups ||
                          dW[1] * g.groups != g.C);
  g.P = shape_ok ? (g.H + 2 * g.pad_h - g.R) / g.stride_h + 1 : 0;
  g.Q = shape_ok ? (g.W + 2 * g.pad_w - g.S) / g.stride_w + 1 : 0;
  const bool depthwise = g.groups > 1 && g.groups == g.C && g.K == g.C;

  Entry e = trace_entry(sym);
  te_ptr(e, x); te_ptr(e, w); te_ptr(e, bias); te_ptr(e, y);
  te_dims(e, dX, 4); te_dims(e, dW, 4); te_dims(e, pads, 2); te_dims(e, strides, 2);
  te_i(e, groups); te_i(e, act_mode);
  e.in[0] = (uintptr_t)x; e.in[1] = (uintptr_t)w; e.in[2] = (uintptr_t)bias;
  e.in_bytes[0] = numel4(dX) * 4; e.in_bytes[1] = numel4(dW) * 4; e.in_bytes[2] = dW[0] * 4;
  e.out = (uintptr_t)y;
  e.dims[0] = g.N; e.dims[1] = g.K; e.dims[2] = g.P; e.dims[3] = g.Q;
  e.out_bytes = (int64_t)g.N * g.K * g.P * g.Q * 4;
  e.kind = (int)act_mode;
  e.depthwise = depthwise;
  e.fusable = shape_ok && r.mode != MATH_FP32 && g.P > 0 && g.Q > 0 && g.N > 0 &&
              (depthwise ? g.C % 8 == 0
                         : (g.groups == 1 && g.K % 8 == 0 && (g.C < 16 || g.C % 8 == 0)));
  // the fused convolution + max-pool kernel takes 64-channel stems whose column step is 16 bytes
  e.poolable = e.fusable && r.mode == MATH_BF16 && !depthwise && g.C <= 4 && g.K == 64 && g.stride_w == 2 && g.Q <= 128 &&
               g.S <= 16 && g.R <= 11;
  const Role role = step(e, false);

  if (!shape_ok) {
    set_error(997, "convolution: inconsistent shape");
    return y;
  }
  if (g.P <= 0 || g.Q <= 0 || g.N == 0) return y;
  if (r.log)
    fprintf(stderr, "[occamy] conv x[%d,%d,%d,%d] w[%d,%d,%d,%d] g%d s%d p%d act%d role%d\n", g.N,
            g.C, g.H, g.W, g.K, (int)dW[1], g.R, g.S, g.groups, g.stride_h, g.pad_h, act,
            (int)role);
  if (r.mode != MATH_FP32) {
    ConvJob job;
    const bool ok = depthwise ? prepare_depthwise(x, w, bias, g, job)
                              : (g.groups == 1 && prepare_dense(x, w, bias, g, job));
    if (ok) {
      job.out = y;
      if (role == R_DEFER) {   // later calls of the recorded sequence fold into this one
        if (e.poolable && !depthwise && job.a.w_step) {
          // the pool that may join later runs after the filter tensor has been given back
          const int cp = job.a.w_step / g.stride_w;
          job.w_stem = (const bf16 *)packed_weights(w, PACK_STEM, stem_pool_weight_bytes(g.R, job.a.Cf),
                                                    g.K, g.C, g.R, g.S, job.a.Cf / cp, cp);
        }
        g_pending = job;
        g_pending.active = true;
        return y;
      }
      launch_job(job);
      return y;
    }
  }
  if (r.mode == MATH_FP32 && fp32_tc_enabled() && conv_f32_on_tensor_cores(x, w, bias, g, y)) return y;
  ensure_f32(x);
  ensure_f32(w);
  if (bias) ensure_f32(bias);
  if (depthwise) launch_depthwise_f32(x, w, bias, y, g, r.stream);
  else launch_conv_f32(x, w, bias, y, g, r.stream);
  mark_f32(y);
  return y;
}

// The held-back convolution takes over a following element-wise call.  `out` is where that
// call would have written; the convolution's own output is skipped unless it is the same.
void pending_retarget(float *out) {
  g_pending.absorbed++;
  if (out != g_pending.out) {
    elide(g_pending.out);
    g_pending.out = out;
  }
}

int64_t prod(const int64_t *d, int64_t rank) {
  int64_t n = 1;
  for (int64_t i = 0; i < rank; ++i) n *= d[i];
  return n;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------- memory pool
cudaError_t wrapDNNMalloc(void **devPtr, size_t size) {
  rt();
  cudaError_t err = cudaMalloc(devPtr, size ? size : 1);
  if (err != cudaSuccess) die("Malloc", err, size);
  Entry e = trace_entry(S_MALLOC);
  te_i(e, (int64_t)size);
  e.out = (uintptr_t)*devPtr;
  e.out_bytes = (int64_t)size;
  step(e, true);
  pending_guard_range(*devPtr, size, false);
  reg_new(*devPtr, size, FMT_ZERO);  // zero fill is issued only if somebody reads it unwritten
  return cudaSuccess;
}

cudaError_t wrapDNNMemPoolInit(void **devPtr, size_t size) {
  Runtime &r = rt();
  *devPtr = nullptr;
  cudaEvent_t ready = nullptr;
  int same = 0;
  for (const CachedPool &c : g_pool_cache) same += c.bytes == size;
  if (same >= pool_cache_blocks() && same > 0) {
    for (size_t i = 0; i < g_pool_cache.size(); ++i)   // the oldest block of this size
      if (g_pool_cache[i].bytes == size) {
        *devPtr = g_pool_cache[i].base;
        ready = g_pool_cache[i].done;
        g_pool_cache.erase(g_pool_cache.begin() + i);
        break;
      }
  } else {
    // blocks of other sizes make room first
    for (size_t i = 0; i < g_pool_cache.size();)
      if (g_pool_cache[i].bytes != size) {
        free_cached_pool(g_pool_cache[i]);
        g_pool_cache.erase(g_pool_cache.begin() + i);
      } else {
        ++i;
      }
    cudaError_t err = cudaMalloc(devPtr, size ? size : 1);
    if (err != cudaSuccess && !g_pool_cache.empty()) {   // no room for a second block
      cudaGetLastError();
      *devPtr = g_pool_cache[0].base;
      ready = g_pool_cache[0].done;
      g_pool_cache.erase(g_pool_cache.begin());
    } else if (err != cudaSuccess) {
      die("MemPoolInit", err, size);
    }
  }
  if (g_block_ready) OCC_CUDA(cudaEventDestroy(g_block_ready));
  g_block_ready = ready;
  g_cur_pool = *devPtr;
  g_cur_pool_bytes = size;
  g_launches_at_pool_init = r.counters[CNT_LAUNCHES] + r.main_copies;
  g_pools.push_back(PoolRec{*devPtr, size});
  if ((int64_t)size > r.counters[CNT_POOL_HWM]) r.counters[CNT_POOL_HWM] = (int64_t)size;
  trace_set_pool(*devPtr, size);
  Entry e = trace_entry(S_POOLINIT);
  te_i(e, (int64_t)size);
  step(e, false);
  return cudaSuccess;
}

cudaError_t wrapDNNMemOffset(void **devPtr, void *basePtr, size_t offset, size_t mallocSize) {
  *devPtr = (char *)basePtr + offset;
  Entry e = trace_entry(S_MEMOFFSET);
  te_ptr(e, *devPtr);
  te_i(e, (int64_t)mallocSize);
  e.out = (uintptr_t)*devPtr;
  e.out_bytes = (int64_t)mallocSize;
  step(e, true);
  pending_guard_range(*devPtr, mallocSize, false);
  reg_new(*devPtr, mallocSize, FMT_ZERO);
  return cudaSuccess;
}

cudaError_t wrapDNNMemcpy(void *dst, const void *src, size_t count_, int kind,
                          cudaStream_t /*stream*/) {
  Runtime &r = rt();
  if (count_ == 0) return cudaSuccess;
  cudaError_t err = cudaSuccess;
  if (kind == 1 || kind == 3) {
    Entry e = trace_entry(kind == 1 ? S_H2D : S_D2D);
    te_ptr(e, dst);
    te_i(e, (int64_t)count_);
    if (kind == 3) {
      te_ptr(e, src);
      e.in[0] = (uintptr_t)src;
      e.in_bytes[0] = (int64_t)count_;
    }
    e.out = (uintptr_t)dst;
    e.out_bytes = (int64_t)count_;
    step(e, kind == 1);
    if (kind == 3) {
      pending_guard_range(dst, count_, true);
      ensure_f32(src);
    }
    uintptr_t base;
    TensorRec *rec = reg_find(dst, &base);
    const bool whole = rec && base == (uintptr_t)dst && count_ + 32 > rec->bytes;
    if (rec && !whole) ensure_f32(dst);
    if (kind == 1 && whole) {
      rec->host_src = src;
      rec->host_bytes = count_;
      rec->host_hash = host_hash(src, count_);
      // A constant whose packed form is already resident need not cross PCIe again; the
      // copy is made later only if something other than a convolution / GEMM reads it.
      if (r.cache_weights) {
        auto it = r.resident.find(src);
        if (it != r.resident.end() && it->second.first == count_ &&
            it->second.second == rec->host_hash) {
          rec->fmt = FMT_PENDING;   // nothing is written now
          count(CNT_H2D_SKIPPED, (int64_t)count_);
          return cudaSuccess;
        }
      }
    }
    if (kind == 1) pending_guard_range(dst, count_, true);
    const bool in_pool = g_cur_pool && (uintptr_t)dst >= (uintptr_t)g_cur_pool &&
                         (uintptr_t)dst + count_ <= (uintptr_t)g_cur_pool + g_cur_pool_bytes;
    if (kind == 1 && whole && in_pool && count_ >= (1u << 20) && pool_cache_blocks() >= 2) {
      // Large upload into a fresh tensor of this inference's pool block: nothing enqueued
      // for this inference touches these bytes yet, and the block's previous user is done
      // once `g_block_ready` has fired, so the copy need not queue behind the kernels of
      // the previous inference.  Later work on the launch stream waits for it.
      if (!g_copy_stream) OCC_CUDA(cudaStreamCreateWithFlags(&g_copy_stream, cudaStreamNonBlocking));
      if (g_block_ready) OCC_CUDA(cudaStreamWaitEvent(g_copy_stream, g_block_ready, 0));
      if (r.counters[CNT_LAUNCHES] + r.main_copies != g_launches_at_pool_init) {
        // work of this inference is already queued and may still read bytes that the pool
        // plan has recycled for this tensor: the copy goes behind it
        cudaEvent_t before;
        OCC_CUDA(cudaEventCreateWithFlags(&before, cudaEventDisableTiming));
        OCC_CUDA(cudaEventRecord(before, r.stream));
        OCC_CUDA(cudaStreamWaitEvent(g_copy_stream, before, 0));
        OCC_CUDA(cudaEventDestroy(before));
      }
      err = cudaMemcpyAsync(dst, src, count_, cudaMemcpyHostToDevice, g_copy_stream);
      cudaEvent_t ev;
      OCC_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
      OCC_CUDA(cudaEventRecord(ev, g_copy_stream));
      OCC_CUDA(cudaStreamWaitEvent(r.stream, ev, 0));
      OCC_CUDA(cudaEventDestroy(ev));
    } else {
      err = cudaMemcpyAsync(dst, src, count_,
                            kind == 1 ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice,
                            r.stream);
      r.main_copies++;
    }
    if (kind == 1) count(CNT_H2D_BYTES, (int64_t)count_);
    if (rec && whole) {
      rec->fmt = FMT_F32;
      if (kind == 3) rec->host_src = nullptr;
    }
  } else if (kind == 2) {
    Entry e = trace_entry(S_D2H);
    te_ptr(e, src);
    te_i(e, (int64_t)count_);
    e.in[0] = (uintptr_t)src;
    e.in_bytes[0] = (int64_t)count_;
    step(e, false);
    uintptr_t base;
    TensorRec *rec = reg_find(src, &base);
    const void *from = src;
    if (rec && fmt_is_16(rec->fmt) && base == (uintptr_t)src) {
      // convert into scratch instead of in place: the tensor keeps its fast format
      const size_t elems = (size_t)(rec->n * rec->c * rec->h * rec->w);
      float *tmp = (float *)scratch_get(2, elems * 4);
      launch_nhwc_bf16_to_nchw_f32((const bf16 *)src, tmp, (int)rec->n, (int)rec->c, (int)rec->h,
                                   (int)rec->w, rec->fmt == FMT_F16_NHWC, r.stream);
      count(CNT_MATERIALIZE);
      from = tmp;
    } else {
      ensure_f32(src);
    }
    err = cudaMemcpyAsync(dst, from, count_, cudaMemcpyDeviceToHost, r.stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(r.stream);
    // surface a kernel-side watchdog report, if any
    if (r.dev_err && r.host_err) {
      cudaMemcpy(r.host_err, r.dev_err, sizeof(int), cudaMemcpyDeviceToHost);
      if (*r.host_err) {
        set_error(*r.host_err, "kernel watchdog");
        cudaMemset(r.dev_err, 0, sizeof(int));
      }
    }
  } else {
    Entry e = trace_entry(S_OPAQUE);
    step(e, false);
    err = cudaMemcpyAsync(dst, src, count_, (cudaMemcpyKind)kind, r.stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(r.stream);
  }
  if (err != cudaSuccess) {
    printf("[Memcpy] GPU error: %s\n", cudaGetErrorString(err));
    exit(-1);
  }
  return cudaSuccess;
}

cudaError_t wrapDNNDealloc(void *devPtr) {
  Runtime &r = rt();
  if (!devPtr) return cudaSuccess;
  size_t bytes = 0;
  bool was_pool = false;
  for (size_t i = 0; i < g_pools.size(); ++i)
    if (g_pools[i].base == devPtr) {
      bytes = g_pools[i].bytes;
      was_pool = true;
      g_pools.erase(g_pools.begin() + i);
      break;
    }
  if (was_pool) {
    Entry e = trace_entry(S_POOLFREE);
    step(e, false);   // runs whatever is still held back
    trace_set_pool(nullptr, 0);
    if (devPtr == g_cur_pool) {
      g_cur_pool = nullptr;
      g_cur_pool_bytes = 0;
    }
    if (pool_cache_blocks() > 0) {
      // Work still in flight on the launch stream is ordered before anything a later
      // inference enqueues there, so the block can be handed out again without waiting;
      // the event lets the copy stream know when its bytes are really free.
      if (bytes) reg_drop_range(devPtr, bytes);
      CachedPool c{devPtr, bytes, nullptr};
      OCC_CUDA(cudaEventCreateWithFlags(&c.done, cudaEventDisableTiming));
      OCC_CUDA(cudaEventRecord(c.done, r.stream));
      g_pool_cache.push_back(c);
      while ((int)g_pool_cache.size() > pool_cache_blocks()) {
        free_cached_pool(g_pool_cache[0]);
        g_pool_cache.erase(g_pool_cache.begin());
      }
      return cudaSuccess;
    }
  } else {
    uintptr_t base;
    TensorRec *rec = reg_find(devPtr, &base);
    if (rec && base == (uintptr_t)devPtr) bytes = rec->bytes;
    Entry e = trace_entry(S_DEALLOC);
    te_ptr(e, devPtr);
    e.out = (uintptr_t)devPtr;
    e.out_bytes = (int64_t)bytes;
    step(e, true);
    pending_guard_range(devPtr, bytes ? bytes : 1, true);
  }
  OCC_CUDA(cudaStreamSynchronize(r.stream));
  if (bytes) reg_drop_range(devPtr, bytes);
  cudaError_t err = cudaFree(devPtr);
  if (err != cudaSuccess) {
    printf("[Dealloc] GPU error: %s\n", cudaGetErrorString(err));
    exit(-1);
  }
  return cudaSuccess;
}

// ---------------------------------------------------------------- handle
// The compiled function creates the handle on entry and destroys it before it returns:
// these two calls delimit one inference for the call trace.
int cudnnCreate(cudnnContext **handle) {
  rt();
  *handle = reinterpret_cast<cudnnContext *>(malloc(16));
  flush_pending();
  trace_begin();
  return *handle ? 0 : 2;
}
int cudnnDestroy(cudnnContext *handle) {
  flush_pending();
  trace_end();
  free(handle);
  return 0;
}

// ---------------------------------------------------------------- convolution
float *DNNConvFunc(cudnnContext *, float *x, int64_t dimX[4], float *w, int64_t dimW[4],
                   float * /*workspace*/, int64_t /*workspaceSize*/, int64_t /*algo*/,
                   int64_t groups, int64_t pads[2], int64_t strides[2], float *y) {
  return conv_common(S_CONV, x, dimX, w, dimW, nullptr, groups, pads, strides, ACT_IDENTITY, 0.f,
                     0.f, 5, y);
}

float *DNNConvBiasActivFunc(cudnnContext *, float *x, int64_t dimX[4], float *w, int64_t dimW[4],
                            float *bias, int64_t dimB[4], float * /*workspace*/,
                            int64_t /*workspaceSize*/, int64_t /*algo*/, int64_t pads[2],
                            int64_t strides[2], int64_t activMode, float *y) {
  (void)dimB;
  int act = ACT_IDENTITY;
  float lo = 0.f, hi = 0.f;
  if (activMode == 1) act = ACT_RELU;
  else if (activMode == 3) { act = ACT_CLIP; lo = 0.f; hi = 6.f; }
  else if (activMode == 0) act = ACT_SIGMOID;
  else if (activMode == 2) act = ACT_TANH;
  return conv_common(S_CONV_BIAS_ACT, x, dimX, w, dimW, bias, 1, pads, strides, act, lo, hi,
                     activMode, y);
}

// ---------------------------------------------------------------- element-wise
float *DNNActiveFunc(cudnnContext *, float *x, int64_t dimX[4], int32_t mode, float *y) {
  Runtime &r = rt();
  const int64_t n = numel4(dimX);
  const int act = mode == 0 ? ACT_SIGMOID : (mode == 1 ? ACT_RELU : (mode == 2 ? ACT_TANH : ACT_IDENTITY));
  Entry e = trace_entry(S_ACTIVE);
  te_ptr(e, x); te_ptr(e, y); te_dims(e, dimX, 4); te_i(e, mode);
  e.in[0] = (uintptr_t)x; e.in_bytes[0] = n * 4; e.out = (uintptr_t)y; e.out_bytes = n * 4;
  for (int i = 0; i < 4; ++i) e.dims[i] = dimX[i];
  e.kind = mode == 1 ? CK_RELU : CK_NONE;
  const Role role = step(e, false);
  if (role == R_ABSORB && g_pending.active) {
    const ConvGeom &g = g_pending.g;
    if (mode == 1 && x == g_pending.out && !g_pending.act_set && dimX[0] == g.N &&
        dimX[1] == g.K && dimX[2] == g.P && dimX[3] == g.Q) {
      pending_retarget(y);
      g_pending.g.act = ACT_RELU;
      g_pending.act_set = true;
      flush_pending();   // an activation closes the chain
      return y;
    }
    flush_pending();
  }
  if (is_act16(x, dimX[0], dimX[1], dimX[2], dimX[3])) {
    launch_add_act_bf16((const bf16 *)x, nullptr, nullptr, (int)dimX[1], (bf16 *)y, n, act, 0.f,
                        0.f, mode_f16(), r.stream);
    mark_act16(y, dimX[0], dimX[1], dimX[2], dimX[3]);
    return y;
  }
  ensure_f32(x);
  launch_act_f32(x, y, n, act, 0.f, 0.f, r.stream);
  mark_f32(y);
  return y;
}

float *CUDAClipFunc(float *x, float *y, int64_t *dimOut, float lo, float hi, int64_t rank) {
  Runtime &r = rt();
  const int64_t n = prod(dimOut, rank);
  Entry e = trace_entry(S_CLIP);
  te_ptr(e, x); te_ptr(e, y); te_dims(e, dimOut, (int)rank); te_f(e, lo); te_f(e, hi);
  e.in[0] = (uintptr_t)x; e.in_bytes[0] = n * 4; e.out = (uintptr_t)y; e.out_bytes = n * 4;
  for (int i = 0; i < 4 && i < rank; ++i) e.dims[i] = dimOut[i];
  e.kind = rank == 4 ? CK_CLIP : CK_NONE;
  const Role role = step(e, false);
  if (role == R_ABSORB && g_pending.active) {
    const ConvGeom &g = g_pending.g;
    if (rank == 4 && x == g_pending.out && !g_pending.act_set && dimOut[0] == g.N &&
        dimOut[1] == g.K && dimOut[2] == g.P && dimOut[3] == g.Q) {
      pending_retarget(y);
      g_pending.g.act = ACT_CLIP;
      g_pending.g.lo = lo;
      g_pending.g.hi = hi;
      g_pending.act_set = true;
      flush_pending();
      return y;
    }
    flush_pending();
  }
  if (rank == 4 && is_act16(x, dimOut[0], dimOut[1], dimOut[2], dimOut[3])) {
    launch_add_act_bf16((const bf16 *)x, nullptr, nullptr, (int)dimOut[1], (bf16 *)y, n, ACT_CLIP,
                        lo, hi, mode_f16(), r.stream);
    mark_act16(y, dimOut[0], dimOut[1], dimOut[2], dimOut[3]);
    return y;
  }
  ensure_f32(x);
  launch_act_f32(x, y, n, ACT_CLIP, lo, hi, r.stream);
  mark_f32(y);
  return y;
}

float *DNNTensorOpFunc(cudnnContext *, int64_t opMode, float *A, int64_t *dimA, int32_t rankA,
                       float *B, int64_t *dimB, int32_t rankB, float *out, int64_t *dimOut,
                       int32_t rankOut, float bias) {
  Runtime &r = rt();
  (void)dimOut;
  (void)rankOut;
  const bool rank_ok = rankA <= 8 && rankB <= rankA && rankA >= 1;
  // B's shape padded with leading 1s to A's rank
  int64_t dB[8] = {1, 1, 1, 1, 1, 1, 1, 1};
  if (rank_ok)
    for (int i = 0; i < rankA; ++i) dB[i] = i < rankA - rankB ? 1 : dimB[i - (rankA - rankB)];
  bool same = rank_ok && rankA == 4;
  for (int i = 0; same && i < 4; ++i) same = dB[i] == dimA[i];
  const bool bias_shape = rank_ok && rankA == 4 && dB[0] == 1 && dB[1] == dimA[1] && dB[2] == 1 &&
                          dB[3] == 1 && !same;

  Entry e = trace_entry(S_TENSOR_OP);
  te_ptr(e, A); te_ptr(e, B); te_ptr(e, out);
  te_i(e, opMode); te_f(e, bias);
  if (rank_ok) { te_dims(e, dimA, rankA); te_dims(e, dB, rankA); }
  e.in[0] = (uintptr_t)A; e.in[1] = opMode == 4 ? 0 : (uintptr_t)B; e.out = (uintptr_t)out;
  e.out_bytes = rank_ok ? prod(dimA, rankA) * 4 : 0;
  e.in_bytes[0] = e.out_bytes;
  e.in_bytes[1] = rank_ok ? prod(dB, rankA) * 4 : 0;
  for (int i = 0; i < 4 && i < rankA; ++i) e.dims[i] = dimA[i];
  if (opMode == 0 && bias == 1.0f) e.kind = bias_shape ? CK_BIAS_ADD : (same ? CK_SAME_ADD : CK_NONE);
  const Role role = step(e, false);

  if (!rank_ok) {
    set_error(996, "tensor op: unsupported rank");
    return out;
  }
  if (role == R_ABSORB && g_pending.active) {
    const ConvGeom &g = g_pending.g;
    const bool dims_ok = dimA[0] == g.N && dimA[1] == g.K && dimA[2] == g.P && dimA[3] == g.Q;
    if (e.kind == CK_BIAS_ADD && dims_ok && A == g_pending.out && !g_pending.bias_set &&
        !g_pending.res_set && !g_pending.act_set) {
      const float *bd = resident_f32(B, (size_t)g.K * 4);
      if (g_pending.depthwise) g_pending.bias = bd;
      else g_pending.a.bias = bd;
      job_track_bias(g_pending, bd, B, g.K);
      if (!g_pack_was_resident) g_pending.a.consts_ready = 0;
      g_pending.bias_set = true;
      pending_retarget(out);
      return out;
    }
    if (e.kind == CK_SAME_ADD && dims_ok && !g_pending.depthwise && !g_pending.res_set &&
        !g_pending.act_set && ((A == g_pending.out) != (B == g_pending.out))) {
      const float *other = A == g_pending.out ? B : A;
      if (is_act16(other, g.N, g.K, g.P, g.Q)) {
        g_pending.a.residual = (const bf16 *)other;
        g_pending.res_set = true;
        g_pending.dep_lo[1] = (uintptr_t)other;
        g_pending.dep_hi[1] = (uintptr_t)other + (size_t)g.N * g.K * g.P * g.Q * 2;
        pending_retarget(out);
        return out;
      }
    }
    flush_pending();
  }
  if (opMode == 0 && rankA == 4 && bias == 1.0f &&
      is_act16(A, dimA[0], dimA[1], dimA[2], dimA[3])) {
    const int64_t n = numel4(dimA);
    if (same && is_act16(B, dimA[0], dimA[1], dimA[2], dimA[3])) {
      launch_add_act_bf16((const bf16 *)A, (const bf16 *)B, nullptr, (int)dimA[1], (bf16 *)out, n,
                          ACT_IDENTITY, 0.f, 0.f, mode_f16(), r.stream);
      mark_act16(out, dimA[0], dimA[1], dimA[2], dimA[3]);
      return out;
    }
    if (bias_shape) {
      // a bias vector uploaded from host memory is kept resident like the filters are
      const float *bd = resident_f32(B, (size_t)dimA[1] * 4);
      launch_add_act_bf16((const bf16 *)A, nullptr, bd, (int)dimA[1], (bf16 *)out, n, ACT_IDENTITY,
                          0.f, 0.f, mode_f16(), r.stream);
      mark_act16(out, dimA[0], dimA[1], dimA[2], dimA[3]);
      return out;
    }
  }
  ensure_f32(A);
  if (opMode != 4) ensure_f32(B);
  if (opMode != 0 && opMode != 1 && opMode != 4) {
    set_error(996, "tensor op: unsupported mode");
    return out;
  }
  launch_tensor_op_f32((int)opMode, A, B, out, rankA, dimA, dB, bias, r.stream);
  mark_f32(out);
  return out;
}

// ---------------------------------------------------------------- pooling / reduction
static float *pool_common(int sym, float *x, int64_t *dI, float *y, int64_t *dO, int64_t *kernel,
                          int64_t *padding, int64_t *stride, bool avg) {
  Runtime &r = rt();
  const int N = (int)dI[0], C = (int)dI[1], H = (int)dI[2], W = (int)dI[3];
  const int P = (int)dO[2], Q = (int)dO[3];
  const int ph = (int)padding[0], pw = (int)padding[2];
  Entry e = trace_entry(sym);
  te_ptr(e, x); te_ptr(e, y); te_dims(e, dI, 4); te_dims(e, dO, 4); te_dims(e, kernel, 2);
  te_dims(e, padding, 4); te_dims(e, stride, 2);
  e.in[0] = (uintptr_t)x; e.in_bytes[0] = numel4(dI) * 4; e.out = (uintptr_t)y;
  e.out_bytes = numel4(dO) * 4;
  if (!avg && kernel[0] == 3 && kernel[1] == 3 && stride[0] == 2 && stride[1] == 2 && ph == 1 &&
      pw == 1 && padding[1] == 1 && padding[3] == 1)
    e.kind = CK_POOL_3S2;
  const Role role = step(e, false);
  if (role == R_ABSORB && g_pending.active) {
    // the held-back stem convolution and this pool run as one kernel
    ConvJob &j = g_pending;
    const ConvGeom &g = j.g;
    bool done = false;
    if (!j.depthwise && j.w_stem && !j.res_set && x == j.out && N == g.N && C == g.K && H == g.P &&
        W == g.Q && e.kind == CK_POOL_3S2) {
      StemPoolArgs sa;
      memset(&sa, 0, sizeof(sa));
      sa.x = j.a.x;
      sa.bias = j.a.bias;
      sa.y = (bf16 *)y;
      sa.N = g.N; sa.H = g.H; sa.row_bytes = j.a.row_elems * 2; sa.w_step_bytes = j.a.w_step * 2;
      sa.P = g.P; sa.Q = g.Q; sa.K = g.K; sa.R = g.R; sa.Cf = j.a.Cf;
      sa.pad_h = g.pad_h; sa.stride_h = g.stride_h;
      sa.PP = P; sa.QP = Q;
      sa.lo = j.a.act == ACT_RELU ? 0.0f : (j.a.act == ACT_CLIP ? j.a.lo : -INFINITY);
      sa.hi = j.a.act == ACT_CLIP ? j.a.hi : INFINITY;
      sa.w = j.w_stem;
      if (stem_pool_supported(sa)) {
        if (launch_stem_pool(sa, r.dev_err, r.num_sms, r.stream)) {
          j.active = false;
          j.absorbed++;
          elide(j.out);
          trace_count_chain();
          mark_act16(y, N, C, P, Q);
          done = true;
        }
      }
    }
    if (done) return y;
    flush_pending();
  }
  if (r.mode != MATH_FP32 && C % 8 == 0 && is_act16(x, N, C, H, W)) {
    launch_pool_bf16((const bf16 *)x, (bf16 *)y, N, C, H, W, P, Q, (int)kernel[0], (int)kernel[1],
                     ph, pw, (int)stride[0], (int)stride[1], avg, mode_f16(), r.stream);
    mark_act16(y, N, C, P, Q);
    return y;
  }
  ensure_f32(x);
  launch_pool_f32(x, y, N, C, H, W, P, Q, (int)kernel[0], (int)kernel[1], ph, pw, (int)stride[0],
                  (int)stride[1], avg, r.stream);
  mark_f32(y);
  return y;
}

float *DNNMaxPoolFunc(cudnnContext *, float *x, int64_t dimIn[4], float *y, int64_t dimOut[4],
                      int64_t kernel[2], int64_t padding[4], int64_t stride[2]) {
  return pool_common(S_MAXPOOL, x, dimIn, y, dimOut, kernel, padding, stride, false);
}

float *DNNAveragePoolFunc(cudnnContext *, float *x, int64_t dimIn[4], float *y, int64_t dimOut[4],
                          int64_t kernel[2], int64_t padding[4], int64_t stride[2]) {
  return pool_common(S_AVGPOOL, x, dimIn, y, dimOut, kernel, padding, stride, true);
}

float *DNNReduceFunc(cudnnContext *, int32_t rank, float *x, int64_t *dimIn, float *y,
                     int64_t *dimOut, int32_t mode) {
  Runtime &r = rt();
  Entry e = trace_entry(S_REDUCE);
  te_ptr(e, x); te_ptr(e, y); te_i(e, mode);
  if (rank <= 8 && rank > 0) { te_dims(e, dimIn, rank); te_dims(e, dimOut, rank); }
  e.in[0] = (uintptr_t)x; e.out = (uintptr_t)y;
  e.out_bytes = rank <= 8 && rank > 0 ? prod(dimOut, rank) * 4 : 0;
  e.in_bytes[0] = rank <= 8 && rank > 0 ? prod(dimIn, rank) * 4 : 0;
  step(e, false);
  if (mode != 5 || rank > 8) {
    set_error(995, "reduce: only mode 5 (mean) is implemented");
    return y;
  }
  if (rank == 4 && dimOut[2] == 1 && dimOut[3] == 1 && dimOut[0] == dimIn[0] &&
      dimOut[1] == dimIn[1] && dimIn[1] % 8 == 0 &&
      is_act16(x, dimIn[0], dimIn[1], dimIn[2], dimIn[3])) {
    launch_gap_bf16((const bf16 *)x, y, (int)dimIn[0], (int)(dimIn[2] * dimIn[3]), (int)dimIn[1],
                    mode_f16(), r.stream);
    mark_f32(y);
    return y;
  }
  ensure_f32(x);
  launch_reduce_mean_f32(x, y, rank, dimIn, dimOut, r.stream);
  mark_f32(y);
  return y;
}

// ---------------------------------------------------------------- classifier head
float *CUBLASMatmul2dFunc(int64_t /*rank*/, float *A, int64_t dimA[2], float *B, int64_t dimB[2],
                          float * /*C*/, int64_t * /*dimC*/, float *out, int64_t * /*dimOut*/,
                          float alpha, float beta, int64_t transA, int64_t transB) {
  Runtime &r = rt();
  const int M = (int)(transA ? dimA[1] : dimA[0]);
  const int K = (int)(transA ? dimA[0] : dimA[1]);
  const int N = (int)(transB ? dimB[0] : dimB[1]);
  Entry e = trace_entry(S_MATMUL);
  te_ptr(e, A); te_ptr(e, B); te_ptr(e, out); te_dims(e, dimA, 2); te_dims(e, dimB, 2);
  te_f(e, alpha); te_f(e, beta); te_i(e, transA); te_i(e, transB);
  e.in[0] = (uintptr_t)A; e.in[1] = (uintptr_t)B; e.in[2] = beta != 0.0f ? (uintptr_t)out : 0;
  e.out = (uintptr_t)out; e.out_bytes = (int64_t)M * N * 4;
  e.in_bytes[0] = dimA[0] * dimA[1] * 4; e.in_bytes[1] = dimB[0] * dimB[1] * 4;
  e.in_bytes[2] = e.out_bytes;
  step(e, false);
  if (r.log) fprintf(stderr, "[occamy] matmul2d M%d N%d K%d tA%d tB%d\n", M, N, K, (int)transA, (int)transB);
  const bool out_zero = is_zero(out);
  if (r.mode != MATH_FP32 && !transA && transB && alpha == 1.0f && (beta == 0.0f || out_zero) &&
      K % 16 == 0 && M > 0) {
    TcConvArgs a;
    memset(&a, 0, sizeof(a));
    a.N = 1; a.H = 1; a.W = M; a.Cf = K; a.K = N; a.P = 1; a.Q = M; a.R = 1; a.S = 1;
    a.stride_h = a.stride_w = 1;
    a.act = ACT_IDENTITY;
    a.out_f32 = out;
    a.ldo = N;
    a.f16 = mode_f16() ? 1 : 0;
    a.x = (const bf16 *)16;
    a.w = (const bf16 *)16;
    if (tc_conv_supported(a)) {
      ensure_f32(A);
      bf16 *ab = (bf16 *)scratch_get(0, (size_t)M * K * 2);
      const bf16 *wb = (const bf16 *)packed_weights(B, PACK_KRSC, (size_t)N * K * 2, N, K, 1, 1, 0, 0);
      if (ab && wb) {
        launch_f32_to_bf16(A, ab, (int64_t)M * K, mode_f16(), r.stream);
        a.x = ab;
        a.w = wb;
        launch_tc_conv(a, r.stream);
        mark_f32(out);
        return out;
      }
    }
  }
  if (r.mode == MATH_FP32 && fp32_tc_enabled() && !transA && transB && alpha == 1.0f &&
      (beta == 0.0f || out_zero) && M > 0 && (double)M * N * K >= 1e6) {
    // the same split-operand scheme as the convolutions, as a 1x1 convolution over M "pixels"
    const int Kp = (K + 15) / 16 * 16;
    TcConvArgs a;
    memset(&a, 0, sizeof(a));
    a.N = 1; a.H = 1; a.W = M; a.Cf = Kp; a.K = N; a.P = 1; a.Q = M; a.R = 1; a.S = 1;
    a.stride_h = a.stride_w = 1;
    a.act = ACT_IDENTITY;
    a.split = 1;
    a.out_f32 = out;
    a.ldo = N;
    a.x = (const bf16 *)16;
    a.w = (const bf16 *)16;
    if (tc_conv_supported(a)) {
      ensure_f32(A);
      bf16 *as = (bf16 *)scratch_get(0, (size_t)3 * M * Kp * 2);
      const bf16 *ws = (const bf16 *)packed_weights(B, PACK_SPLIT, (size_t)6 * N * Kp * 2, N, K, 1, 1, 0, Kp);
      if (as && ws) {
        launch_split3_rows(A, as, M, K, Kp, (int)dimA[1], r.stream);
        a.x = as;
        a.w = ws;
        launch_tc_conv(a, r.stream);
        mark_f32(out);
        return out;
      }
    }
  }
  ensure_f32(A);
  ensure_f32(B);
  if (beta != 0.0f) ensure_f32(out);
  launch_gemm_f32(A, B, out, M, N, K, (int)dimA[1], (int)dimB[1], alpha, out_zero ? 0.0f : beta,
                  transA != 0, transB != 0, r.stream);
  mark_f32(out);
  return out;
}

float *CUDASoftmaxFunc(float *x, int64_t *dimIn, float *y, int64_t * /*dimOut*/, int64_t axis,
                       int64_t rank) {
  Runtime &r = rt();
  if (axis < 0) axis += rank;
  int64_t outer = 1, inner = 1;
  for (int64_t i = 0; i < axis; ++i) outer *= dimIn[i];
  for (int64_t i = axis + 1; i < rank; ++i) inner *= dimIn[i];
  Entry e = trace_entry(S_SOFTMAX);
  te_ptr(e, x); te_ptr(e, y); te_dims(e, dimIn, (int)rank); te_i(e, axis);
  e.in[0] = (uintptr_t)x; e.out = (uintptr_t)y; e.out_bytes = prod(dimIn, rank) * 4;
  e.in_bytes[0] = e.out_bytes;
  step(e, false);
  ensure_f32(x);
  launch_softmax_f32(x, y, outer, dimIn[axis], inner, r.stream);
  mark_f32(y);
  return y;
}

static float *copy_common(int sym, float *x, int64_t *dimIn, int64_t rank, float *y) {
  Runtime &r = rt();
  const int64_t n = prod(dimIn, rank);
  Entry e = trace_entry(sym);
  te_ptr(e, x); te_ptr(e, y); te_dims(e, dimIn, (int)rank);
  e.in[0] = (uintptr_t)x; e.in_bytes[0] = n * 4; e.out = (uintptr_t)y; e.out_bytes = n * 4;
  step(e, false);
  ensure_f32(x);
  OCC_CUDA(cudaMemcpyAsync(y, x, (size_t)n * 4, cudaMemcpyDeviceToDevice, r.stream));
  mark_f32(y);
  return y;
}

float *CUDAFlattenFunc(float *x, int64_t *dimIn, float *y, int64_t * /*dimOut*/, int32_t /*axis*/,
                       int64_t rank) {
  return copy_common(S_FLATTEN, x, dimIn, rank, y);
}

float *CUDAReshapeFunc(float *x, int64_t *dimIn, int64_t rank, float *y) {
  return copy_common(S_RESHAPE, x, dimIn, rank, y);
}

// Called by the entry points outside this file: they take part in no chain and their
// reads are not tracked, so they end the speculation for this inference.
void occamy_internal_opaque_call(void) {
  Entry e = trace_entry(S_OPAQUE);
  step(e, false);
}

// ---------------------------------------------------------------- controls
void occamy_set_math_mode(int mode) {
  flush_pending();   // what is held back was prepared for the mode it arrived in
  rt().mode = mode == 0 ? MATH_FP32 : (mode == 2 ? MATH_F16 : MATH_BF16);
}
int occamy_get_math_mode(void) { return (int)rt().mode; }

int occamy_last_error(int clear) {
  Runtime &r = rt();
  if (r.last_error == 0) {   // a watchdog report of the allocation-free entry point, if any
    const int na = noalloc_poll_error(clear != 0);
    if (na > 0) set_error(na, "kernel watchdog (occamy_conv_bias_act_noalloc)");
  }
  const int e = r.last_error;
  if (clear) r.last_error = 0;
  return e;
}

int occamy_synchronize(void) {
  Runtime &r = rt();
  flush_pending();
  cudaError_t e = cudaStreamSynchronize(r.stream);
  if (e != cudaSuccess) set_error((int)e, "synchronize");
  if (r.dev_err && r.host_err) {
    cudaMemcpy(r.host_err, r.dev_err, sizeof(int), cudaMemcpyDeviceToHost);
    if (*r.host_err) {
      set_error(*r.host_err, "kernel watchdog");
      cudaMemset(r.dev_err, 0, sizeof(int));
    }
  }
  const int na = noalloc_poll_error(true);
  if (na > 0) set_error(na, "kernel watchdog (occamy_conv_bias_act_noalloc)");
  return (int)e;
}

cudaStream_t occamy_stream(void) { return rt().stream; }

void occamy_selftest_bounded_wait(void) {
  flush_pending();
  launch_selftest_bounded_wait(rt().stream);
}

void occamy_get_counters(int64_t out[8]) {
  Runtime &r = rt();
  for (int i = 0; i < 8; ++i) out[i] = r.counters[i];
}

int64_t occamy_fused_chains(void) { return trace_fused_chains(); }
void occamy_clear_weight_cache(void);

void occamy_profile_begin(void) {
  Runtime &r = rt();
  r.prof_count = 0;
  r.profiling = true;
}

int occamy_profile_end(float *ms, int cap) {
  Runtime &r = rt();
  flush_pending();
  r.profiling = false;
  OCC_CUDA(cudaStreamSynchronize(r.stream));
  const int n = r.prof_count;
  for (int i = 0; i < n && i < cap; ++i) {
    float t = 0.f;
    OCC_CUDA(cudaEventElapsedTime(&t, r.prof_events[2 * i], r.prof_events[2 * i + 1]));
    ms[i] = t;
  }
  r.prof_count = 0;
  return n;
}

void occamy_set_cross_call_fusion(int on) {
  flush_pending();
  trace_set_enabled(on != 0);
}

void occamy_set_fp32_tensor_cores(int on) { g_fp32_tc = on ? 1 : 0; }

void occamy_set_weight_cache(int on) {
  if (!on) occamy_clear_weight_cache();
  rt().cache_weights = on != 0;
}

void occamy_clear_weight_cache(void) {
  Runtime &r = rt();
  flush_pending();
  OCC_CUDA(cudaStreamSynchronize(r.stream));
  for (auto &kv : r.wcache)
    if (kv.second.dev) cudaFree(kv.second.dev);
  r.wcache.clear();
  r.resident.clear();
}

}  // extern "C"
