// Runtime state: lazy initialisation, the tensor-format registry, scratch space.
#include "runtime.h"

#include <cstring>

#include "kernels.h"

namespace occ {

static Runtime *g_rt = nullptr;

void set_error(int code, const char *where) {
  Runtime *r = g_rt;
  if (r && r->last_error == 0) r->last_error = code;
  fprintf(stderr, "[occamy_b200] error %d at %s%s%s\n", code, where,
          code > 0 && code < 1000 ? ": " : "",
          code > 0 && code < 1000 ? cudaGetErrorString((cudaError_t)code) : "");
}

Runtime &rt() {
  if (g_rt) return *g_rt;
  Runtime *r = new Runtime();
  g_rt = r;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    // No usable GPU: this library has no CPU path.  Say so and stop.
    fprintf(stderr, "[occamy_b200] fatal: no CUDA device (%s); the runtime has no CPU fallback\n",
            cudaGetErrorString(e));
    exit(-1);
  }
  r->device = dev;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) == cudaSuccess) {
    r->num_sms = prop.multiProcessorCount;
    if (prop.major != 10) {
      fprintf(stderr,
              "[occamy_b200] fatal: device %d is sm_%d%d; this build contains sm_100a code only\n",
              dev, prop.major, prop.minor);
      exit(-1);
    }
  }
  OCC_CUDA(cudaStreamCreateWithFlags(&r->stream, cudaStreamNonBlocking));
  OCC_CUDA(cudaMalloc(&r->dev_err, sizeof(int)));
  OCC_CUDA(cudaMemset(r->dev_err, 0, sizeof(int)));
  OCC_CUDA(cudaMallocHost(&r->host_err, sizeof(int)));
  if (r->host_err) *r->host_err = 0;
  const char *m = getenv("OCCAMY_MATH");
  if (m && (!strcmp(m, "fp32") || !strcmp(m, "0"))) r->mode = MATH_FP32;
  if (m && (!strcmp(m, "bf16") || !strcmp(m, "1"))) r->mode = MATH_BF16;
  if (m && (!strcmp(m, "fp16") || !strcmp(m, "f16") || !strcmp(m, "2"))) r->mode = MATH_F16;
  const char *l = getenv("OCCAMY_LOG");
  r->log = l && *l && strcmp(l, "0");
  const char *c = getenv("OCCAMY_CACHE_WEIGHTS");
  if (c && !strcmp(c, "0")) r->cache_weights = false;
  return *r;
}

// ---------------------------------------------------------------- registry
void reg_drop_range(void *p, size_t bytes) {
  Runtime &r = rt();
  const uintptr_t lo = (uintptr_t)p, hi = lo + bytes;
  auto it = r.recs.lower_bound(lo);
  if (it != r.recs.begin()) {
    auto prev = std::prev(it);
    if (prev->first + prev->second.bytes > lo) it = prev;
  }
  // Handing out [lo, hi) again ends the life of every tensor it touches (the reference
  // zero-fills the range at this point), so their records go, partly covered ones too.
  while (it != r.recs.end() && it->first < hi) it = r.recs.erase(it);
}

void reg_new(void *p, size_t bytes, Fmt fmt) {
  if (!p || bytes == 0) return;
  reg_drop_range(p, bytes);
  TensorRec rec;
  rec.bytes = bytes;
  rec.fmt = fmt;
  rt().recs[(uintptr_t)p] = rec;
}

TensorRec *reg_find(const void *p, uintptr_t *base) {
  Runtime &r = rt();
  const uintptr_t a = (uintptr_t)p;
  auto it = r.recs.upper_bound(a);
  if (it == r.recs.begin()) return nullptr;
  --it;
  if (a >= it->first + it->second.bytes) return nullptr;
  if (base) *base = it->first;
  return &it->second;
}

bool mode_f16() { return rt().mode == MATH_F16; }

bool is_act16(const void *p, int64_t n, int64_t c, int64_t h, int64_t w) {
  uintptr_t base;
  TensorRec *rec = reg_find(p, &base);
  const Fmt want = mode_f16() ? FMT_F16_NHWC : FMT_BF16_NHWC;
  return rec && base == (uintptr_t)p && rec->fmt == want && rec->n == n && rec->c == c &&
         rec->h == h && rec->w == w;
}

bool is_zero(const void *p) {
  uintptr_t base;
  TensorRec *rec = reg_find(p, &base);
  return rec && rec->fmt == FMT_ZERO;
}

void mark_f32(void *p) {
  uintptr_t base;
  TensorRec *rec = reg_find(p, &base);
  if (!rec) return;
  if (base != (uintptr_t)p && rec->fmt != FMT_F32) {
    ensure_f32((const void *)base);  // partial overwrite of a specially formatted tensor
    return;
  }
  rec->fmt = FMT_F32;
  rec->host_src = nullptr;
}

void mark_act16(void *p, int64_t n, int64_t c, int64_t h, int64_t w) {
  uintptr_t base;
  TensorRec *rec = reg_find(p, &base);
  const Fmt fmt = mode_f16() ? FMT_F16_NHWC : FMT_BF16_NHWC;
  if (!rec || base != (uintptr_t)p) {
    // Unknown or interior pointer: record it as its own tensor of the fp32 extent.
    reg_new(p, (size_t)(n * c * h * w) * 4, fmt);
    rec = reg_find(p, &base);
  }
  rec->fmt = fmt;
  rec->n = n;
  rec->c = c;
  rec->h = h;
  rec->w = w;
  rec->host_src = nullptr;
}

void ensure_f32(const void *p) {
  uintptr_t base;
  TensorRec *rec = reg_find(p, &base);
  if (!rec || rec->fmt == FMT_F32) return;
  Runtime &r = rt();
  if (rec->fmt != FMT_ELIDED && r.before_write) {
    const Fmt keep = rec->fmt;
    r.before_write((const void *)base, rec->bytes);
    rec = reg_find(p, &base);          // the hook may have launched work that re-tags tensors
    if (!rec || rec->fmt != keep) return ensure_f32(p);
  }
  if (rec->fmt == FMT_ELIDED) {
    set_error(990, "read of a tensor that cross-call fusion skipped (set OCCAMY_FUSE_ACROSS_CALLS=0)");
  } else if (rec->fmt == FMT_ZERO) {
    OCC_CUDA(cudaMemsetAsync((void *)base, 0, rec->bytes, r.stream));
    r.main_copies++;
  } else if (rec->fmt == FMT_PENDING) {
    OCC_CUDA(cudaMemcpyAsync((void *)base, rec->host_src, rec->host_bytes, cudaMemcpyHostToDevice,
                             r.stream));
    r.main_copies++;
    count(CNT_H2D_BYTES, (int64_t)rec->host_bytes);
  } else if (fmt_is_16(rec->fmt)) {
    const size_t elems = (size_t)(rec->n * rec->c * rec->h * rec->w);
    void *tmp = scratch_get(3, elems * 2);
    OCC_CUDA(cudaMemcpyAsync(tmp, (void *)base, elems * 2, cudaMemcpyDeviceToDevice, r.stream));
    launch_nhwc_bf16_to_nchw_f32((const bf16 *)tmp, (float *)base, (int)rec->n, (int)rec->c,
                                 (int)rec->h, (int)rec->w, rec->fmt == FMT_F16_NHWC, r.stream);
    count(CNT_MATERIALIZE);
  }
  rec->fmt = FMT_F32;
}

void *scratch_get(int slot, size_t bytes) {
  Runtime &r = rt();
  if (r.scratch_bytes[slot] >= bytes) return r.scratch[slot];
  // Growing: work already enqueued may still use the old block.
  if (r.scratch[slot]) {
    OCC_CUDA(cudaStreamSynchronize(r.stream));
    OCC_CUDA(cudaFree(r.scratch[slot]));
  }
  size_t want = bytes + bytes / 8;
  want = (want + 0xFFFFF) & ~(size_t)0xFFFFF;
  void *p = nullptr;
  OCC_CUDA(cudaMalloc(&p, want));
  r.scratch[slot] = p;
  r.scratch_bytes[slot] = p ? want : 0;
  return p;
}

uint64_t host_hash(const void *src, size_t bytes) {
  // Fingerprint used to notice that a host buffer taken for a constant has changed: a
  // multiplicative hash over the length, the first and last 512 bytes, and 64-byte blocks
  // spread evenly over the whole buffer (up to 256 of them), so that a change in the interior
  // is seen too.  A few tens of kilobytes are read whatever the size of the constant.  Eight
  // bytes per step in four independent lanes: this runs for every constant of every inference
  // (a byte-serial hash cost 20 us per constant, 2 ms per ResNet-50 inference, and made small
  // batches host-bound).
  const unsigned char *b = (const unsigned char *)src;
  uint64_t lane[4] = {1469598103934665603ull ^ bytes, 0x9e3779b97f4a7c15ull, 0xc2b2ae3d27d4eb4full,
                      0x165667b19e3779f9ull};
  auto mix = [&](size_t lo, size_t hi) {
    size_t i = lo;
    for (; i + 32 <= hi; i += 32) {
      uint64_t w[4];
      memcpy(w, b + i, 32);
      for (int j = 0; j < 4; ++j) lane[j] = (lane[j] ^ w[j]) * 1099511628211ull;
    }
    for (int j = 0; i < hi; ++i, j = (j + 1) & 3) lane[j] = (lane[j] ^ b[i]) * 1099511628211ull;
  };
  const size_t head = bytes < 512 ? bytes : 512;
  mix(0, head);
  if (bytes > 512) mix(bytes - 512 > head ? bytes - 512 : head, bytes);
  if (bytes > 1024) {
    const size_t inner = bytes - 1024;
    size_t blocks = inner / 64 < 256 ? inner / 64 : 256;
#ifdef OCCAMY_TUNING
    static const int forced = getenv("OCCAMY_HASH_BLOCKS") ? atoi(getenv("OCCAMY_HASH_BLOCKS")) : -1;
    if (forced >= 0 && (size_t)forced < blocks) blocks = (size_t)forced;
#endif
    for (size_t k = 0; k < blocks; ++k) {
      // block k starts at an even share of the interior, rounded down to 8 bytes
      const size_t at = 512 + ((inner - 64) * k / (blocks > 1 ? blocks - 1 : 1) & ~(size_t)7);
      mix(at, at + 64);
    }
  }
  uint64_t h = lane[0];
  for (int j = 1; j < 4; ++j) {
    h ^= lane[j] + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    h *= 1099511628211ull;
  }
  return h ^ (h >> 29);
}

}  // namespace occ
