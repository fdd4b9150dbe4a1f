// Implicit-GEMM convolution / GEMM on the sm_100a tensor cores.
//
//   D[m, k] = act( sum_{tap, c} A_tap[m, c] * Wp[tap, k, c] + bias[k] (+ residual[m, k]) )
//
// m runs over output pixels (n, p, q), k over output channels, c over input channels.
// A is never materialised: for every filter tap the producer issues one tiled TMA load of
// a [tn x th x tw] pixel box x BK channels straight out of the NHWC bf16 activation
// tensor, shifted by the tap's (dh, dw); out-of-image pixels are zero-filled by TMA,
// which implements the padding.  Strided convolutions read through per-phase tensor
// maps whose strides are the convolution stride (h = stride*(p + a) + b for tap offset
// stride*a + b), so the same shifted-box scheme applies.
//
// The kernels run one persistent CTA per SM with warp-specialised roles (TMA producer, MMA
// issuer, epilogue warps, slab store); the pixel-M kernel template lives in conv_tc_dev.cuh,
// the pixel-N variant and the host-side planning (tile shapes, tensor maps, shared-memory
// budget) in this file.  Every wait on an mbarrier is bounded; when a bound is hit the
// kernel records a code in the error word, drains and returns.
#include <cmath>
#include <cstring>
#include <unordered_map>
#include <vector>

#include "conv_tc_dev.cuh"
#include "kernels.h"
#include "runtime.h"

namespace occ {

// ------------------------------------------------------------------ pixel-N variant
// One tcgen05.mma takes the same ~155 cycles whatever its N, so a layer with few output
// channels wastes most of the tensor pipe when the channels are the N dimension.  This
// variant swaps the operands: the filter tile (128 output channels x BK) is the M side, up
// to 256 pixels are the N side, D^T[channel, pixel] lands in TMEM with one channel per lane.
// The epilogue thread of a lane owns that channel (bias is a scalar), walks the pixels and
// transposes through the staged NHWC slabs with 2-byte stores (a warp writes 64 contiguous
// bytes of one pixel), which TMA then stores as before.  Used for K <= 128.
__global__ void __launch_bounds__(TC_THREADS, 1) tc_conv_pn_kernel(const __grid_constant__ TcParams p) {
  constexpr int SLAB_BYTES = 256 * 128;   // 256 pixel rows x 64 channels of bf16
  constexpr uint32_t TMEM_COLS = 512;     // two accumulators of 256 pixel columns

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const int bk = p.bk, stages = p.stages;
  const uint32_t w_bytes = 128u * bk * 2u, x_bytes = 256u * bk * 2u;
  const uint32_t sW = base;
  const uint32_t sX = sW + stages * w_bytes;
  const uint32_t sD = sX + stages * x_bytes;            // 2 slabs: channels 0-63, 64-127
  const uint32_t sMisc = sD + 2 * SLAB_BYTES;
  uint8_t *misc_ptr = base_ptr + (sMisc - base);
  uint64_t *bars = reinterpret_cast<uint64_t *>(misc_ptr);
  const uint32_t bar0 = sMisc;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (stages + s); };
  auto tfull_bar = [&](int s) { return bar0 + 8u * (2 * stages + s); };
  auto tempty_bar = [&](int s) { return bar0 + 8u * (2 * stages + 2 + s); };
  const uint32_t rfull_bar = bar0 + 8u * (2 * stages + 4);
  volatile uint32_t *tmem_holder = reinterpret_cast<volatile uint32_t *>(bars + 2 * stages + 5);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * stages + 6);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), TC_EPI_THREADS / 32);   // one arrival per epilogue warp
    }
    mbar_init(rfull_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32((const void *)tmem_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_launch_dependents();   // the next kernel's prologue may overlap this one
  pdl_wait();                // nothing above touched global memory

  const int rows_valid = p.tw * p.th * p.tn;   // pixels per tile (<= 256)
  const int ksteps = p.num_taps * p.cblocks;
  int err_code = 0;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx_bytes = (uint32_t)rows_valid * bk * 2u + w_bytes;
      for (int tile = blockIdx.x; tile < p.total_tiles && !err_code; tile += gridDim.x) {
        const int kt = tile % p.tiles_k;
        int sp = tile / p.tiles_k;
        const int q0 = (sp % p.tiles_w) * p.tw;
        sp /= p.tiles_w;
        const int p0 = (sp % p.tiles_h) * p.th;
        const int n0 = (sp / p.tiles_h) * p.tn;
        const int k0 = kt * 128;
        for (int t = 0; t < p.num_taps && !err_code; ++t) {
          const TcTap tap = p.taps[t];
          for (int cb = 0; cb < p.cblocks; ++cb) {
            if (!mbar_wait_hot(empty_bar(stage), phase ^ 1u, abort_flag)) {
              err_code = 1;
              break;
            }
            mbar_expect_tx(full_bar(stage), tx_bytes);
            tma_load_4d(sX + stage * x_bytes, &p.tmA[tap.map], full_bar(stage), cb * bk,
                        q0 + tap.dw, p0 + tap.dh, n0);
            tma_load_3d(sW + stage * w_bytes, &p.tmB, full_bar(stage), cb * bk, k0, t);
            if (++stage == stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                             ((uint32_t)(p.n_mma >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      // Straight-line k-step body, one copy of the tile loop per MMAs-per-k-step, descriptors
      // as 32-bit halves: this thread's instructions between two k-steps are time the tensor
      // pipe runs dry (see tc_conv_kernel).
      const uint64_t w0 = make_smem_desc(sW, bk), x0 = make_smem_desc(sX, bk);
      const uint32_t w_hi = (uint32_t)(w0 >> 32), x_hi = (uint32_t)(x0 >> 32);
      const uint32_t w_lo0 = (uint32_t)w0, x_lo0 = (uint32_t)x0;
      const uint32_t w_step = (uint32_t)w_bytes >> 4, x_step = (uint32_t)x_bytes >> 4;
      auto run_tiles = [&](auto nk_c) {
        constexpr int NK = decltype(nk_c)::value;
        uint32_t w_lo = w_lo0, x_lo = x_lo0;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
          if (!mbar_wait_hot(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
            err_code = 2;
            return;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * 256);
          for (int ks = 0; ks < ksteps; ++ks) {
            if (!mbar_wait_hot(full_bar(stage), phase, abort_flag)) {
              err_code = 3;
              return;
            }
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < NK; ++kk)
              mma_lohi(d_tmem, w_lo + 2u * kk, w_hi, x_lo + 2u * kk, x_hi, idesc,
                       kk ? 1u : (uint32_t)(ks != 0));
            tc_commit(empty_bar(stage));
            w_lo += w_step;
            x_lo += x_step;
            if (++stage == stages) {
              stage = 0;
              phase ^= 1u;
              w_lo = w_lo0;
              x_lo = x_lo0;
            }
          }
          tc_commit(tfull_bar(acc));
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }
      };
      if (bk == 64) run_tiles(std::integral_constant<int, 4>{});
      else if (bk == 32) run_tiles(std::integral_constant<int, 2>{});
      else run_tiles(std::integral_constant<int, 1>{});
    }
  } else {
    const float act_lo = p.lo, act_hi = p.hi;
    const int quad = warp & 3;                 // TMEM lane quadrant = 32 output channels
    const int half = (warp - 2) >> 2;          // which 128 of the 256 pixel columns
    const int c_local = quad * 32 + lane;      // this thread's channel within the 128-tile
    const int slab = c_local >> 6, cin = c_local & 63;
    const bool leader = threadIdx.x == 64;
    int acc = 0;
    uint32_t acc_phase = 0, r_phase = 0;
    // With at most 64 output channels only one slab is used per tile, so the two slab
    // buffers alternate and a tile's store need not have drained before the next one writes.
    const bool one_slab = p.K <= 64;
    uint32_t flip = 0;
    for (int tile = blockIdx.x; tile < p.total_tiles && !err_code; tile += gridDim.x) {
      const int kt = tile % p.tiles_k;
      int sp = tile / p.tiles_k;
      const int q0 = (sp % p.tiles_w) * p.tw;
      sp /= p.tiles_w;
      const int p0 = (sp % p.tiles_h) * p.th;
      const int n0 = (sp / p.tiles_h) * p.tn;
      const int k0 = kt * 128;
      const int nslab = min(2, (p.K - k0 + 63) / 64);
      const int ch = k0 + c_local;
      const float bias = (p.bias && ch < p.K) ? p.bias[ch] : 0.0f;
      const uint32_t sDt = sD + (one_slab ? flip * SLAB_BYTES : 0u);
      if (leader) {
        // the stores that last read the slab(s) about to be written have drained
        if (one_slab) tma_store_wait_read<1>();
        else tma_store_wait_read<0>();
        if (p.has_res) {
          mbar_expect_tx(rfull_bar, (uint32_t)(nslab * rows_valid) * 128u);
          for (int sl = 0; sl < nslab; ++sl)
            tma_load_4d(sDt + sl * SLAB_BYTES, &p.tmR, rfull_bar, k0 + sl * 64, q0, p0, n0);
        }
      }
      epi_bar();
      if (!mbar_wait_hot(tfull_bar(acc), acc_phase, abort_flag)) {
        err_code = 4;
        break;
      }
      tc_fence_after();
      if (p.has_res) {
        if (!mbar_wait_hot(rfull_bar, r_phase, abort_flag)) {
          err_code = 5;
          break;
        }
        r_phase ^= 1u;
      }
      const bool active = slab < nslab;        // warp-uniform (a warp covers 32 channels)
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) +
                              (uint32_t)(acc * 256 + half * 128);
      uint8_t *dslab = base_ptr + (sDt + slab * SLAB_BYTES - base);
      const int col_end = min(128, p.n_mma - half * 128);   // columns of this half in use
      if (active && col_end > 0) {
        uint32_t rr[2][32];
        tc_ld32(t_addr, rr[0]);
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          if (c4 * 32 >= col_end) break;
          tc_ld_wait();
          if ((c4 + 1) * 32 < col_end) tc_ld32(t_addr + (uint32_t)((c4 + 1) * 32), rr[(c4 + 1) & 1]);
          const uint32_t *r = rr[c4 & 1];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int pix = half * 128 + c4 * 32 + j;
            __nv_bfloat16 *cell = reinterpret_cast<__nv_bfloat16 *>(
                dslab + slab_off(pix, cin >> 3, 128) + (cin & 7) * 2);
            float v = __uint_as_float(r[j]) + bias;
            if (p.has_res) v += __bfloat162float(*cell);
            *cell = __float2bfloat16_rn(tc_act(v, act_lo, act_hi));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      fence_async_smem();
      epi_bar();
      if (leader) {
        for (int sl = 0; sl < nslab; ++sl)
          tma_store_4d(&p.tmD, sDt + sl * SLAB_BYTES, k0 + sl * 64, q0, p0, n0);
        tma_store_commit();
      }
      flip ^= 1u;
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (leader) tma_store_wait_read<0>();
  }

  if (err_code) {
    atomicExch(p.err, 1000 + err_code);
    *abort_flag = 1;
    for (int i = 0; i < 50; ++i) __nanosleep(20000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ------------------------------------------------------------------ watchdog self-test
// One thread waits, with the very wait every role of the kernels above uses, on an mbarrier
// that nobody will ever arrive at.  The wait has to give up at its bound (about two seconds),
// the kernel then reports code 1099 the way the convolution kernels report theirs and returns:
// shows on a live GPU that a stuck pipeline ends in an error code, not in a hang.
__global__ void tc_selftest_wait_kernel(int *err) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait_slow(smem_u32(&bar), 0, &abort_flag)) atomicExch(err, 1099);
  }
}

void launch_selftest_bounded_wait(cudaStream_t s) {
  tc_selftest_wait_kernel<<<1, 32, 0, s>>>(rt().dev_err);
  count(CNT_LAUNCHES);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
    if (e != cudaSuccess || !sym) {
      set_error(e ? (int)e : 999, "cuTensorMapEncodeTiled entry point");
      return nullptr;
    }
    fn = (EncodeTiledFn)sym;
  }
  return fn;
}

static CUtensorMapSwizzle swizzle_for(int row_bytes) {
  return row_bytes >= 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

// bf16 tensor map of rank `rank` (<= 4): dims/box innermost first, strides in bytes for
// dims 1..rank-1.  `counted` is false only while a plan is built for the allocation-free
// entry point, which must not touch the lazily initialised runtime state.
static bool make_map(CUtensorMap *m, const void *ptr, int rank, const uint64_t *dims,
                     const uint64_t *strides, const uint32_t *box, int row_bytes, bool counted) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gd[4], gs[3];
  cuuint32_t bx[4], es[4];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides[i];
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void *>(ptr),
                  gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(row_bytes),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (counted) count(CNT_TMAP_ENCODES);
  if (r != CUDA_SUCCESS) {
    set_error(2000 + (int)r, "cuTensorMapEncodeTiled");
    return false;
  }
  return true;
}

// Pixel box (tw x th x tn <= limit) that covers a Q x P x N output grid with the fewest tiles.
static void choose_box(int Q, int P, int N, int limit, int *tw, int *th, int *tn) {
  long best = -1;
  int bw = 1, bh = 1, bn = 1;
  for (int w = 1; w <= (Q < limit ? Q : limit); ++w) {
    const long cw = (Q + w - 1) / w;
    for (int h = 1; h <= P && h <= 256 && w * h <= limit; ++h) {
      const long ch = (P + h - 1) / h;
      int n = limit / (w * h);
      if (n > N) n = N;
      // any n in [1, n] is legal; fewer tiles with the largest, but try divisors too
      for (int nn = n; nn >= 1; nn = (nn > 8 ? nn / 2 : nn - 1)) {
        const long tiles = cw * ch * ((N + nn - 1) / nn);
        if (best < 0 || tiles < best || (tiles == best && w > bw)) {
          best = tiles;
          bw = w;
          bh = h;
          bn = nn;
        }
      }
    }
  }
  *tw = bw;
  *th = bh;
  *tn = bn;
}

// Channels per k-step.  The exact choice is the largest of 64 / 32 / 16 that divides the channel
// count.  The last k-block may also reach past the last channel (TMA fills what is out of
// bounds with zeros), and a k-step has a fixed cost in every single-threaded role, so fewer,
// fuller k-steps are taken when they at least halve the count (144 channels: three k-steps of
// 64 instead of nine of 16; measured 0.058 -> 0.050 ms on 144->24 at 56x56, while 96 channels
// as two k-steps of 64 instead of three of 32 were 13 % slower).
static int pick_bk(int Cf) {
  if (Cf <= 0 || Cf % 8 != 0) return 0;
  const int exact = Cf % 64 == 0 ? 64 : (Cf % 32 == 0 ? 32 : (Cf % 16 == 0 ? 16 : 0));
  const int wide = Cf <= 16 ? 16 : (Cf <= 32 ? 32 : 64);
  if (exact == 0) return wide;
  return Cf / exact >= 2 * ((Cf + wide - 1) / wide) ? wide : exact;
}
// Output-channel tile.  Wide tiles re-read the activations less and keep the tensor pipe
// busier per instruction, but when a layer has few pixels they leave SMs idle; pick the
// width with the lowest modelled time: waves x (k-steps x cost per k-step + epilogue slabs).
static int pick_bn(int K, long sp_tiles, int ksteps, int num_sms, int widest_allowed = 256) {
#ifdef OCCAMY_TUNING   // sweep builds only: force the tile width from the environment
  if (const char *f = getenv("OCCAMY_TC_BN")) {
    const int v = atoi(f);
    if (v == 32 || v == 64 || v == 128 || v == 256) return v;
  }
#endif
  const int cand[4] = {256, 128, 64, 32};
  const double kcost[4] = {900.0, 780.0, 715.0, 700.0};  // cycles per 64-deep k-step
  int widest = 32;
  while (widest < K && widest < widest_allowed) widest *= 2;
  int best = widest;
  double best_cost = -1.0;
  for (int i = 0; i < 4; ++i) {
    const int bn = cand[i];
    if (bn > widest) continue;
    const long tiles = sp_tiles * ((K + bn - 1) / bn);
    const long waves = (tiles + num_sms - 1) / num_sms;
    const int slabs = bn >= 64 ? bn / 64 : 1;
    const double cost = (double)waves * (ksteps * kcost[i] + slabs * 700.0);
    if (best_cost < 0 || cost < best_cost * 0.97) {   // ties go to the wider tile
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

bool tc_conv_supported(const TcConvArgs &a) {
  if (pick_bk(a.Cf) == 0) return false;
  if (a.act != ACT_IDENTITY && a.act != ACT_RELU && a.act != ACT_CLIP) return false;
  if (a.stride_h < 1 || a.stride_w < 1 || a.stride_h > 2 || a.stride_w > 2) return false;
  if (a.w_step && ((a.w_step * 2) % 16 || (a.row_elems * 2) % 16 || a.S != 1)) return false;
  if (a.R * a.S * (a.split ? 6 : 1) > TC_MAX_TAPS) return false;
  if (!a.out_f32 && a.K % 8 != 0) return false;
  if (a.split && (!a.out_f32 || a.w_step || a.f16)) return false;
  if (a.out_f32 && a.residual) return false;
  // the row-major fp32 output is indexed by the flattened pixel number (plain GEMM view only)
  if (a.out_f32 && !a.out_nchw && !(a.R == 1 && a.S == 1 && a.stride_h == 1 && a.stride_w == 1 &&
                                    a.pad_h == 0 && a.pad_w == 0))
    return false;
  if ((uintptr_t)a.x % 16 || (uintptr_t)a.w % 16) return false;
  if (a.y && (uintptr_t)a.y % 16) return false;
  if ((int64_t)a.N * a.P * a.Q >= (1ll << 31)) return false;
  if (a.K > 4096) return false;   // the bias vector has to fit in shared memory
  return true;
}

struct ArgsKey {
  TcConvArgs a;
  bool operator==(const ArgsKey &o) const { return memcmp(&a, &o.a, sizeof(a)) == 0; }
};
struct ArgsKeyHash {
  size_t operator()(const ArgsKey &k) const {
    const unsigned char *b = (const unsigned char *)&k.a;
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(k.a); ++i) h = (h ^ b[i]) * 1099511628211ull;
    return (size_t)h;
  }
};
struct Plan {
  TcParams p;
  int mode;  // TC_MODE_* of the pixel-M kernel
  int bn;
  int dc;    // channels per output slab
  bool pn;   // pixel-N variant
  bool pair; // CTA-pair form: the grid is launched as clusters of two
  bool duo;  // two independent CTAs per SM (one epilogue warp per TMEM quadrant)
  size_t smem;
  bool ok;
};

static TcFastDiv make_fastdiv(int d) {
  TcFastDiv f{0u, 0u};
  if (d <= 1) return f;
  int s = 0;
  while ((1ll << s) < d) ++s;                    // s = ceil(log2 d)
  f.mul = (uint32_t)((((uint64_t)1 << (31 + s)) + d - 1) / d);
  f.shift = (uint32_t)(s - 1);
  return f;
}

static int floordiv(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }

#ifdef OCCAMY_TC_TIMERS
// analysis builds only: the device words the kernels' role timers add to
static long long *tc_timer_words() {
  static long long *w = nullptr;
  if (!w) {
    cudaMalloc(&w, 20 * sizeof(long long));
    cudaMemset(w, 0, 20 * sizeof(long long));
  }
  return w;
}
extern "C" void occamy_tc_timers(long long *out, int clear) {
  cudaDeviceSynchronize();
  cudaMemcpy(out, tc_timer_words(), 20 * sizeof(long long), cudaMemcpyDeviceToHost);
  if (clear) cudaMemset(tc_timer_words(), 0, 20 * sizeof(long long));
}
#endif

static Plan build_plan(const TcConvArgs &a, int *err_word, int num_sms, bool counted,
                       bool allow_halo = true) {
  Plan pl;
  memset(&pl, 0, sizeof(pl));
  TcParams &p = pl.p;
  const int bk = pick_bk(a.Cf);
  p.bk = bk;
  p.cblocks = (a.Cf + bk - 1) / bk;
  p.K = a.K;
  p.bias = a.bias;
  p.has_res = a.residual ? 1 : 0;
  p.act = a.act;
  p.lo = a.act == ACT_RELU ? 0.0f : (a.act == ACT_CLIP ? a.lo : -INFINITY);
  p.hi = a.act == ACT_CLIP ? a.hi : INFINITY;
  p.out_f32 = a.out_f32;
  p.ldo = a.ldo;
  p.out_hw = a.out_f32 && a.out_nchw ? a.P * a.Q : 0;
  // fp32 operands as three bf16 parts: six (activation part, filter part) products per tap
  const int parts = a.split ? 3 : 1, combos = a.split ? 6 : 1;
  static const int a_part[6] = {0, 0, 0, 1, 1, 2};
  const int64_t plane = (int64_t)a.N * a.H * a.W * a.Cf;   // elements of one activation part
  p.err = err_word;
#ifdef OCCAMY_TC_TIMERS
  p.timers = tc_timer_words();
#endif
  p.consts_ready = a.consts_ready;
  const bool flat = a.R == 1 && a.S == 1 && a.stride_h == 1 && a.stride_w == 1 && a.pad_h == 0 &&
                    a.pad_w == 0 && a.w_step == 0;
  // output grid the tiles are cut from
  int Qg = a.Q, Pg = a.P, Ng = a.N;
  if (flat) {
    Qg = a.N * a.P * a.Q;
    Pg = 1;
    Ng = 1;
  }
  p.m_total = Qg;
  p.gq = Qg;
  p.gp = Pg;
  p.gn = Ng;
#ifdef OCCAMY_TUNING
  static const bool pn_allowed = !(getenv("OCCAMY_TC_PIXEL_N") && !strcmp(getenv("OCCAMY_TC_PIXEL_N"), "0"));
  static const bool halo_allowed = !(getenv("OCCAMY_TC_HALO") && !strcmp(getenv("OCCAMY_TC_HALO"), "0"));
#else
  constexpr bool pn_allowed = true, halo_allowed = true;
#endif
  // worth it only where the tensor pipe is the limit: the transposing epilogue is slower
  // than the plain one, which hurts the HBM-bound 1x1 layers
  // 3x3 / stride 1 / pad 1 with 64 -> 64 channels and rows of at most 126 pixels: the input
  // block of a tile is loaded once and the taps are windows of it (TC_MODE_HALO)
  const bool halo = allow_halo && halo_allowed && !a.f16 && !a.split && !a.out_f32 && a.R == 3 && a.S == 3 &&
                    a.stride_h == 1 && a.stride_w == 1 && a.pad_h == 1 && a.pad_w == 1 &&
                    a.Cf == 64 && a.K == 64 && a.W + 2 <= 128 && a.w_step == 0 && a.Q == a.W &&
                    a.P == a.H;
  const bool pn = !halo && pn_allowed && !a.f16 && !a.out_f32 && a.K <= 128 && a.R * a.S > 1 &&
                  a.R * a.S * a.Cf >= 9 * 64;
  pl.pn = pn;
  if (halo) {
    p.tw = a.W + 2;                      // two junk columns that the store clips
    p.th = 128 / p.tw < a.P ? 128 / p.tw : a.P;
    p.tn = 1;
    p.halo = 1;
    p.halo_wp = p.tw;
    p.halo_a_bytes = ((p.th + 2) * p.tw * 128 + 1023) / 1024 * 1024;
  } else {
    choose_box(Qg, Pg, Ng, pn ? 256 : 128, &p.tw, &p.th, &p.tn);
  }
  p.n_mma = (p.tw * p.th * p.tn + 15) / 16 * 16;
  p.tiles_w = halo ? 1 : (Qg + p.tw - 1) / p.tw;
  p.tiles_h = (Pg + p.th - 1) / p.th;
  p.tiles_n = (Ng + p.tn - 1) / p.tn;
  const int nsm = num_sms > 0 ? num_sms : 148;
  const int bn = pn ? 128
                    : halo ? 64
                    : pick_bn(a.K, (long)p.tiles_w * p.tiles_h * p.tiles_n,
                              (a.R * a.S * combos * a.Cf + 63) / 64, nsm, a.split ? 128 : 256);
  pl.bn = bn;
  p.tiles_k = (a.K + bn - 1) / bn;
  p.sp_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
  // CTA pairs (see TC_MODE_PAIR) for the 256-channel tiles of 1x1 layers with a long reduction
  const int ksteps64p = (a.R * a.S * a.Cf + 63) / 64;
#ifdef OCCAMY_TUNING
  static const bool pair_allowed = !(getenv("OCCAMY_TC_PAIR") && !strcmp(getenv("OCCAMY_TC_PAIR"), "0"));
#else
  constexpr bool pair_allowed = true;
#endif
  // Measured on ResNet-50 at batch 256: 5-8 % faster on the 1x1 layers with 1024 and 2048
  // input channels, 3-4 % on the 3x3 layers with 256 and 512 channels, 25 % slower on
  // reductions of four steps: taken for reductions of 16 k-steps and more.
  bool pair = pair_allowed && !pn && !halo && !a.out_f32 && bn == 256 && ksteps64p >= 16 &&
              p.sp_tiles >= 2 && nsm >= 2;
#ifdef OCCAMY_TUNING
  if (getenv("OCCAMY_TC_PAIR") && !strcmp(getenv("OCCAMY_TC_PAIR"), "2"))   // every 256-channel tile
    pair = !pn && !halo && !a.out_f32 && !a.split && bn == 256 && p.sp_tiles >= 2 && nsm >= 2;
#endif
  pl.pair = pair;
  p.total_tiles = (pair ? (p.sp_tiles + 1) / 2 : p.sp_tiles) * p.tiles_k;
  p.div_k = make_fastdiv(p.tiles_k);
  p.div_w = make_fastdiv(p.tiles_w);
  p.div_h = make_fastdiv(p.tiles_h);

  const uint32_t boxA[4] = {(uint32_t)bk, (uint32_t)p.tw, (uint32_t)p.th, (uint32_t)p.tn};
  bool ok = true;
  if (halo) {
    const uint64_t dims[4] = {(uint64_t)a.Cf, (uint64_t)a.W, (uint64_t)a.H, (uint64_t)a.N};
    const uint64_t st[3] = {(uint64_t)a.Cf * 2, (uint64_t)a.W * a.Cf * 2, (uint64_t)a.H * a.W * a.Cf * 2};
    const uint32_t box[4] = {64u, (uint32_t)p.tw, (uint32_t)(p.th + 2), 1u};
    ok &= make_map(&p.tmA[0], a.x, 4, dims, st, box, 128, counted);
    p.num_taps = 9;
  } else if (flat) {
    const uint64_t dims[4] = {(uint64_t)a.Cf, (uint64_t)Qg, 1, 1};
    const uint64_t st[3] = {(uint64_t)a.Cf * 2, (uint64_t)Qg * a.Cf * 2, (uint64_t)Qg * a.Cf * 2};
    for (int part = 0; part < parts; ++part)
      ok &= make_map(&p.tmA[part], a.x + part * plane, 4, dims, st, boxA, bk * 2, counted);
    p.num_taps = combos;
    for (int j = 0; j < combos; ++j) p.taps[j] = TcTap{a.split ? a_part[j] : 0, 0, 0};
  } else {
    // one tensor map per (row phase, column phase) of the stride
    const int sh = a.stride_h, sw = a.stride_w;
    int map_of[2][2] = {{-1, -1}, {-1, -1}};
    int nmaps = 0;
    p.num_taps = 0;
    for (int r = 0; r < a.R; ++r)
      for (int s2 = 0; s2 < a.S; ++s2) {
        const int eh = r - a.pad_h, ew = s2 - a.pad_w;
        const int ah = floordiv(eh, sh), bh = eh - ah * sh;
        const int aw = floordiv(ew, sw), bw = ew - aw * sw;
        if (map_of[bh][bw] < 0) {
          const int Hm = (a.H - bh + sh - 1) / sh, Wm = (a.W - bw + sw - 1) / sw;
          // elements from one pixel to the next and from one row to the next (the folded
          // form's pixels are overlapping windows of a padded row)
          const int64_t px = a.w_step ? a.w_step : a.Cf;
          const int64_t rowe = a.row_elems ? a.row_elems : (int64_t)a.W * a.Cf;
          const bf16 *ptr = a.x + bh * rowe + bw * px;
          const uint64_t dims[4] = {(uint64_t)a.Cf, (uint64_t)(Wm > 0 ? Wm : 1),
                                    (uint64_t)(Hm > 0 ? Hm : 1), (uint64_t)a.N};
          const uint64_t st[3] = {(uint64_t)(sw * px * 2), (uint64_t)(sh * rowe * 2),
                                  (uint64_t)(a.H * rowe * 2)};
          // the maps of one stride phase, one per operand part, sit next to one another
          for (int part = 0; part < parts; ++part)
            ok &= make_map(&p.tmA[nmaps * parts + part], ptr + part * plane, 4, dims, st, boxA,
                           bk * 2, counted);
          map_of[bh][bw] = nmaps++;
        }
        for (int j = 0; j < combos; ++j)
          p.taps[p.num_taps++] = TcTap{map_of[bh][bw] * parts + (a.split ? a_part[j] : 0), aw, ah};
      }
  }
  {
    const uint64_t dims[3] = {(uint64_t)a.Cf, (uint64_t)a.K, (uint64_t)(a.R * a.S * combos)};
    const uint64_t st[2] = {(uint64_t)a.Cf * 2, (uint64_t)a.K * a.Cf * 2};
    const uint32_t box[3] = {(uint32_t)bk, (uint32_t)(pair ? bn / 2 : bn), 1};
    ok &= make_map(&p.tmB, a.w, 3, dims, st, box, bk * 2, counted);
  }
  // For 256-wide tiles with a long reduction, 32-channel slabs free enough shared memory
  // for a fourth ring stage, which those layers need more than a cheap epilogue.
  const int ksteps64 = (a.R * a.S * combos * a.Cf + 63) / 64;
  int dc = pn ? 64 : (bn < 64 ? bn : (bn == 256 && bk == 64 && ksteps64 >= 16 ? 32 : 64));
  if (a.out_f32 && bn >= 64) dc = 64;   // the fp32-output flavour is compiled for 64-channel slabs
#ifdef OCCAMY_TUNING
  if (const char *f = getenv("OCCAMY_TC_DC"))   // slab width of the 256-wide tiles
    if (!pn && bn == 256 && (atoi(f) == 32 || atoi(f) == 64)) dc = atoi(f);
#endif
  pl.dc = dc;
  pl.mode = a.out_f32 ? (TC_MODE_F32 | TC_MODE_CLAMP)
                      : ((a.residual ? TC_MODE_RES : 0) | (a.act == ACT_RELU ? 0 : TC_MODE_CLAMP) |
                         (halo ? TC_MODE_HALO : 0));
  if (a.f16) pl.mode |= TC_MODE_F16;
  if (pair) pl.mode |= TC_MODE_PAIR;
  if (a.split) pl.mode |= TC_MODE_SPLIT;
  if (!a.out_f32) {
    const uint64_t dims[4] = {(uint64_t)a.K, (uint64_t)Qg, (uint64_t)Pg, (uint64_t)Ng};
    const uint64_t st[3] = {(uint64_t)a.K * 2, (uint64_t)Qg * a.K * 2, (uint64_t)Pg * Qg * a.K * 2};
    const uint32_t box[4] = {(uint32_t)dc, (uint32_t)p.tw, (uint32_t)p.th, (uint32_t)p.tn};
    ok &= make_map(&p.tmD, a.y, 4, dims, st, box, dc * 2, counted);
    if (a.residual) ok &= make_map(&p.tmR, a.residual, 4, dims, st, box, dc * 2, counted);
  }
  // One channel tile: every tile multiplies by the same weights.  If they are tiny they are
  // fetched once per CTA into an area of their own instead of once per tile into the ring: all
  // CTAs asking L2 for the same 16 to 32 lines of weights for every tile is what bounded the
  // few-channel layers (1.5x on 32->16 and 16->96 channels at 112x112).  Measured: no gain at
  // 6 to 9 KB of weights, slower at 8 KB (64->64) and 32 KB (64->256 with residual).
  const int ksteps_tile = p.num_taps * p.cblocks;
  const size_t b_tile_bytes = (size_t)(pair ? bn / 2 : bn) * bk * 2;
  // (With two CTAs per SM the single loading thread of a CTA is what the others wait for, and
  // weights of up to 16 KB pay as well: 144->24 at 56x56 has nine k-steps of 1 KB each.)
  const bool duo_wanted = !pn && !halo && !pair && !a.split && !a.out_f32 && dc == 32 && bn == 32 && nsm >= 2;
  bool bres = !pn && !halo && !pair && p.tiles_k == 1 &&
              ksteps_tile * b_tile_bytes <= (size_t)(duo_wanted ? 16 : 4) * 1024;
#ifdef OCCAMY_TUNING
  if (const char *f = getenv("OCCAMY_TC_BRES")) bres = bres && atoi(f) != 0;
#endif
  p.b_resident = bres ? 1 : 0;
  // shared memory: ring + output slabs + bias + barriers + alignment
  const size_t stage_bytes = pn     ? (size_t)(128 + 256) * bk * 2
                             : halo ? (size_t)p.halo_a_bytes
                                    : 128 * bk * 2 + (bres ? 0 : b_tile_bytes);
  p.bias_floats = (a.K + bn - 1) / bn * bn;
  const size_t slab_bytes = (size_t)128 * dc * 2;
  const size_t fixed0 = pn ? 1024 + 2 * 256 * 128 + 8 * 80
                           : (size_t)p.bias_floats * 4 + 8 * 80 +
                                 (halo ? (size_t)9 * bn * bk * 2 : 0) +   // halo: resident weights
                                 (bres ? ksteps_tile * b_tile_bytes : 0);
  // Two CTAs per SM for the 32-channel tiles.  Such a tile is a few hundred cycles of memory
  // traffic, but each of the single-threaded roles (loads, MMA issue, slab stores) spends about
  // a thousand cycles of dependent instructions and barrier round trips on it; two resident
  // CTAs overlap those (measured 1.2x to 1.6x on the layers with up to 32 output channels; no
  // gain for 64-channel tiles).  They share the SM's shared memory, registers (one epilogue warp per TMEM
  // quadrant, 256 threads) and TMEM (at most 256 columns each).
  bool duo = duo_wanted;
#ifdef OCCAMY_TUNING
  if (const char *f = getenv("OCCAMY_TC_DUO"))
    duo = atoi(f) != 0 && !pn && !halo && !pair && !a.split && !a.out_f32 && dc == 32 && bn == 32;
#endif
  int dbuf = 0, pend = 0, stages = 0;
  for (;; duo = false) {
    const size_t limit = duo ? TC_SMEM_DUO : (size_t)TC_SMEM_LIMIT;
    dbuf = pn ? 0 : (3 + TC_NSTORE - 1) / TC_NSTORE * TC_NSTORE;
    if (a.out_f32) dbuf = TC_NSTORE;      // written straight from registers: no slabs are staged
    if (!pn && a.residual && !duo) {
      // The residual slab of an output slab is fetched into its buffer ahead of time, and a
      // slab is consumed faster than the fetch takes: whatever shared memory three ring stages
      // leave goes to slab buffers.
      int min_stages = 3;
#ifdef OCCAMY_TUNING
      if (const char *f = getenv("OCCAMY_TC_RES_STAGES")) min_stages = atoi(f) > 1 ? atoi(f) : min_stages;
#endif
      dbuf = (int)((limit - fixed0 - min_stages * stage_bytes) / slab_bytes);
      if (dbuf > 8) dbuf = 8;
      if (dbuf < 3) dbuf = 3;
      dbuf = dbuf / TC_NSTORE * TC_NSTORE;
      if (dbuf < TC_NSTORE * 2) dbuf = TC_NSTORE * 2;
    }
    // Stores in flight.  A store thread may run ahead of `pend` unfinished stores; each needs a
    // buffer of its own on top of the ones that are filling.  Sized for about 48 KB of stores
    // in flight per SM, as long as four ring stages remain: the layers with long reductions
    // need those more.
    pend = 0;
    if (!pn && !a.out_f32) {
      const size_t aim = duo ? 24 * 1024 : 48 * 1024;
      pend = (int)((aim + TC_NSTORE * slab_bytes - 1) / (TC_NSTORE * slab_bytes)) - 1;
      if (pend > 3) pend = 3;
#ifdef OCCAMY_TUNING
      if (const char *f = getenv("OCCAMY_TC_STORE_PEND")) pend = atoi(f) < 0 ? 0 : (atoi(f) > 3 ? 3 : atoi(f));
#endif
      for (; pend > 0; --pend) {
        const int need = TC_NSTORE * (pend + 2);   // pend + 1 in a store, one filling, per thread
        if (dbuf >= need) break;
        if (fixed0 + need * slab_bytes + (duo ? 3 : 4) * stage_bytes <= limit) {
          dbuf = need;
          break;
        }
      }
    }
    const size_t fixed = fixed0 + dbuf * slab_bytes;
    stages = fixed < limit ? (int)((limit - fixed) / stage_bytes) : 0;
    if (stages > 8) stages = 8;
    pl.smem = fixed + stages * stage_bytes;
    if (!duo || stages >= 3) break;
  }
  if (stages < 2) ok = false;
  pl.duo = duo;
  p.stages = stages;
  p.dbuf = dbuf;
  p.store_pend = pend;
  // one CTA per SM (TMEM is per SM), or two for the duo form (its registers allow no third)
  if (!duo && pl.smem < 120 * 1024) pl.smem = 120 * 1024;
#ifdef OCCAMY_TUNING
  if (getenv("OCCAMY_TC_PLAN_LOG"))
    fprintf(stderr, "[tcplan] K %d Cf %d RS %d px %dx%dx%d box %dx%dx%d bn %d dc %d pn %d bk %d stages %d dbuf %d pend %d duo %d tiles %d smem %zu\n",
            a.K, a.Cf, a.R * a.S, Qg, Pg, Ng, p.tw, p.th, p.tn, bn, dc, (int)pn, bk, stages, dbuf, pend, (int)duo,
            p.total_tiles, pl.smem);
#endif
  if (halo && !ok) return build_plan(a, err_word, num_sms, counted, false);   // e.g. the block map was refused
  pl.ok = ok;
  return pl;
}

static void launch_plan_pn(const Plan &pl, int num_sms, cudaStream_t s) {
  static unsigned char attr_done[TC_MAX_DEVICES] = {};
  if (tc_first_use_on_device(attr_done))
    cudaFuncSetAttribute(tc_conv_pn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         TC_SMEM_LIMIT);
  int grid = pl.p.total_tiles < num_sms ? pl.p.total_tiles : num_sms;
  tc_launch_pdl(tc_conv_pn_kernel, grid, TC_THREADS, pl.smem, s, pl.p);
}

static void launch_any(const Plan &pl, int num_sms, cudaStream_t s) {
  if (pl.pn) {
    launch_plan_pn(pl, num_sms, s);
    return;
  }
  int grid = pl.p.total_tiles < num_sms ? pl.p.total_tiles : num_sms;
  if (pl.pair) {   // two CTAs per tile index, an even number of CTAs
    grid = 2 * pl.p.total_tiles < num_sms ? 2 * pl.p.total_tiles : num_sms / 2 * 2;
  }
  bool ok;
  if (pl.duo) {
    grid = pl.p.total_tiles < 2 * num_sms ? pl.p.total_tiles : 2 * num_sms;
    ok = pl.bn == 32   ? tc_launch_32_32_duo(pl.p, pl.mode, grid, pl.smem, s)
         : pl.bn == 64 ? tc_launch_64_64_duo(pl.p, pl.mode, grid, pl.smem, s)
                       : tc_launch_128_64_duo(pl.p, pl.mode, grid, pl.smem, s);
    if (!ok) set_error(997, "tensor-core conv: no two-per-SM kernel for this epilogue");
    return;
  }
  switch (pl.bn) {
    case 32: ok = tc_launch_32_32(pl.p, pl.mode, grid, pl.smem, s); break;
    case 64: ok = tc_launch_64_64(pl.p, pl.mode, grid, pl.smem, s); break;
    case 128: ok = tc_launch_128_64(pl.p, pl.mode, grid, pl.smem, s); break;
    default:
      ok = pl.dc == 32 ? tc_launch_256_32(pl.p, pl.mode, grid, pl.smem, s)
                       : tc_launch_256_64(pl.p, pl.mode, grid, pl.smem, s);
      break;
  }
  if (!ok) set_error(997, "tensor-core conv: no kernel for this tile shape and epilogue");
}

void launch_tc_conv(const TcConvArgs &a, cudaStream_t s) {
  static std::unordered_map<ArgsKey, Plan, ArgsKeyHash> plans;
  ArgsKey key;
  memset(&key, 0, sizeof(key));
  key.a = a;
  auto it = plans.find(key);
  if (it == plans.end()) {
    if (plans.size() > 4096) plans.clear();
    it = plans.emplace(key, build_plan(a, rt().dev_err, rt().num_sms, true)).first;
  }
  const Plan &pl = it->second;
  if (!pl.ok) {
    set_error(998, "tensor-core conv plan");
    return;
  }
  if (pl.p.total_tiles == 0) return;
  Runtime &r = rt();
  int prof_slot = -1;
  if (r.profiling) {
    prof_slot = r.prof_count++;
    while ((int)r.prof_events.size() < 2 * (prof_slot + 1)) {
      cudaEvent_t e;
      OCC_CUDA(cudaEventCreate(&e));
      r.prof_events.push_back(e);
    }
    OCC_CUDA(cudaEventRecord(r.prof_events[2 * prof_slot], s));
  }
  launch_any(pl, r.num_sms, s);
  if (prof_slot >= 0) OCC_CUDA(cudaEventRecord(r.prof_events[2 * prof_slot + 1], s));
  OCC_CUDA(cudaGetLastError());
  count(CNT_LAUNCHES);
  count(CNT_TC_LAUNCHES);
}

// Launch without touching the runtime's state or any cache: the plan (tensor maps) is
// rebuilt on every call, the kernel's error word and the SM count come from the caller.
// Used by the entry point that must not allocate.
bool launch_tc_conv_stateless(const TcConvArgs &a, int *err_word, int num_sms, cudaStream_t s) {
  const Plan pl = build_plan(a, err_word, num_sms, false);
  if (!pl.ok) return false;
  if (pl.p.total_tiles == 0) return true;
  launch_any(pl, num_sms, s);
  return cudaGetLastError() == cudaSuccess;
}

}  // namespace occ
