// Process-wide state of the operator runtime: the launch stream, the registry that
// records in which format each caller-owned tensor currently sits, scratch space,
// the resident packed-weight cache and the error / counter words.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <unordered_map>
#include <vector>

namespace occ {

// Arithmetic of the convolution / GEMM kernels and storage of the activations between them:
// fp32 NCHW throughout; or tensor cores on 16-bit NHWC activations, bf16 (8 mantissa bits, fp32's
// range) or fp16 (11 mantissa bits, values up to 65504).
enum MathMode { MATH_FP32 = 0, MATH_BF16 = 1, MATH_F16 = 2 };

// Format of the bytes behind a caller-owned device pointer.
enum Fmt {
  FMT_F32 = 0,        // what the ABI says: dense fp32, NCHW
  FMT_ZERO = 1,       // freshly handed out; reads as zero, memset not yet issued
  FMT_BF16_NHWC = 2,  // produced by a tensor-core-mode kernel: bf16, NHWC, dims below
  FMT_PENDING = 3,    // host->device upload deferred (constant already packed on device)
  FMT_ELIDED = 4,     // never written: a cross-call fusion skipped it (reading it is an error)
  FMT_F16_NHWC = 5    // like FMT_BF16_NHWC with fp16 elements (MATH_F16)
};
inline bool fmt_is_16(Fmt f) { return f == FMT_BF16_NHWC || f == FMT_F16_NHWC; }

struct TensorRec {
  size_t bytes = 0;  // extent of the allocation handed to the caller
  Fmt fmt = FMT_F32;
  int64_t n = 0, c = 0, h = 0, w = 0;  // logical NCHW dims of a 16-bit NHWC tensor
  const void *host_src = nullptr;      // source of the last host->device upload, if any
  size_t host_bytes = 0;
  uint64_t host_hash = 0;
};

struct PackedWeight {
  void *dev = nullptr;
  size_t bytes = 0;
  uint64_t hash = 0;
  int layout = 0;  // packing variant, see pack_weights()
};

struct WeightKey {
  const void *src;
  size_t bytes;
  int layout;
  bool operator==(const WeightKey &o) const {
    return src == o.src && bytes == o.bytes && layout == o.layout;
  }
};
struct WeightKeyHash {
  size_t operator()(const WeightKey &k) const {
    return std::hash<const void *>()(k.src) ^ (k.bytes * 1000003u) ^ (size_t)k.layout * 7919u;
  }
};

enum Counter {
  CNT_LAUNCHES = 0,
  CNT_H2D_BYTES = 1,
  CNT_H2D_SKIPPED = 2,
  CNT_POOL_HWM = 3,
  CNT_TC_LAUNCHES = 4,
  CNT_MATERIALIZE = 5,
  CNT_TMAP_ENCODES = 6,
  CNT_SIMT_LAUNCHES = 7
};

struct Runtime {
  cudaStream_t stream = nullptr;
  int device = -1;
  int num_sms = 148;
  MathMode mode = MATH_BF16;
  int last_error = 0;
  int64_t counters[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int64_t main_copies = 0;  // copies / memsets enqueued on the launch stream (not kernels)
  std::map<uintptr_t, TensorRec> recs;  // keyed by device base pointer
  std::unordered_map<WeightKey, PackedWeight, WeightKeyHash> wcache;
  // host sources whose packed form is resident: source -> (bytes, fingerprint)
  std::unordered_map<const void *, std::pair<size_t, uint64_t>> resident;
  void *scratch[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  size_t scratch_bytes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int *dev_err = nullptr;   // device word the kernels' bounded waits report into
  int *host_err = nullptr;  // pinned mirror
  bool log = false;
  bool cache_weights = true;
  // called before the runtime itself writes into a caller-owned range (lazy zero fill,
  // deferred upload, layout conversion), so that a held-back kernel can read it first
  void (*before_write)(const void *p, size_t bytes) = nullptr;
  // optional CUDA-event pair around every tensor-core launch (occamy_profile_begin/end)
  bool profiling = false;
  int prof_count = 0;
  std::vector<cudaEvent_t> prof_events;
};

Runtime &rt();  // lazily initialised on the current device

void set_error(int code, const char *where);
#define OCC_CUDA(call)                                        \
  do {                                                        \
    cudaError_t e_ = (call);                                  \
    if (e_ != cudaSuccess) ::occ::set_error((int)e_, #call);  \
  } while (0)

// ---- registry --------------------------------------------------------------
// Record that [p, p+bytes) now is a fresh tensor; drops records it overlaps.
void reg_new(void *p, size_t bytes, Fmt fmt);
void reg_drop_range(void *p, size_t bytes);
// Record that contains p, or nullptr.  *base receives its base pointer.
TensorRec *reg_find(const void *p, uintptr_t *base = nullptr);
// Make the bytes behind p plain fp32 NCHW (memset, upload or layout conversion as needed).
void ensure_f32(const void *p);
// True when p is the base of a 16-bit NHWC tensor with exactly these logical dims, stored in
// the element type of the CURRENT mode (a tensor left behind in the other 16-bit type is
// converted back to fp32 by its next reader, like any other foreign format).
bool is_act16(const void *p, int64_t n, int64_t c, int64_t h, int64_t w);
// Mark p as fully overwritten by an fp32 kernel / by a 16-bit NHWC kernel of the current mode.
void mark_f32(void *p);
void mark_act16(void *p, int64_t n, int64_t c, int64_t h, int64_t w);
// The current mode stores fp16 (else bf16) in its 16-bit tensors.
bool mode_f16();
// A tensor that reads as zero and has not been written since it was handed out.
bool is_zero(const void *p);

void *scratch_get(int slot, size_t bytes);
// Error word of the allocation-free entry point on the current device (0 when it was never
// used there); see no_alloc.cu.
int noalloc_poll_error(bool clear);
uint64_t host_hash(const void *src, size_t bytes);

inline void count(Counter c, int64_t v = 1) { rt().counters[c] += v; }
inline int64_t numel4(const int64_t *d) { return d[0] * d[1] * d[2] * d[3]; }

}  // namespace occ
