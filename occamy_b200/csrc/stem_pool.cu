// Few-channel convolution (an RGB stem) fused with the 3x3 / stride 2 / pad 1 max pool that
// follows it: conv + bias + clamp + pool in one pass, the full-resolution convolution
// output never leaves the SM.
//
// Input: the padded channels-last image rows the folded convolution uses,
// x[n][h][wp][Cp] bf16 with 16 bytes per output-column step, so the A vector of output
// column q (Cf = Sp*Cp values starting at pixel q*stride) is a window at byte 16*q of the
// row and neighbouring windows overlap.  A row is copied to shared memory ONCE (bulk copy)
// and the tensor core reads the overlapping windows in place: the operand descriptor is the
// un-swizzled K-major form with 16 bytes from one 8-element K chunk to the next and 128
// bytes from one group of 8 rows to the next, which is exactly "row m starts at byte 16*m".
// One MMA row block is one convolution output row (Q <= 128 columns).
//
// One persistent CTA per SM works through units of (image, band of pooled rows):
//   warp 0      producer (one lane): bulk-copies the weights once, then input rows into a ring
//   2 warps     MMA issuers (one lane each, alternate convolution rows): per row R taps x
//               Cf/16 tcgen05.mma (128 x 64 x 16) into one of four TMEM accumulators;
//               release input rows
//   8 warps     epilogue: accumulator -> + bias -> clamp -> bf16 -> convolution-row ring in
//               shared memory (swizzled so that a warp's 128-byte rows spread over banks)
//   8 warps     pool: max over the 3x3 windows of three ring rows -> global memory
// Every wait is bounded; a wait that runs out records a code and the kernel drains.
#include "conv_tc_dev.cuh"
#include "kernels.h"
#include "runtime.h"

namespace occ {

namespace {

constexpr int ST_EPI_WARPS = 8;    // two per TMEM lane quadrant, 32 channels each
constexpr int ST_POOL_WARPS = 8;
constexpr int ST_ISSUER_B = 2 + ST_EPI_WARPS + ST_POOL_WARPS;   // warp of the second MMA issuer
constexpr int ST_THREADS = 32 * (ST_ISSUER_B + 1);
constexpr int ST_NIN = 8;     // input ring slots (a slot holds stride_h rows)
constexpr int ST_NCR = 6;     // convolution-row ring slots
constexpr int ST_NACC = 4;    // TMEM accumulators (64 columns each)
constexpr int ST_K = 64;      // output channels

struct StemParams {
  const bf16 *x;       // [N][H][row_bytes / 2]
  const bf16 *w;       // packed [R][Cf / 8][64][8]
  const float *bias;   // [64] or null
  bf16 *y;             // [N][PP][QP][64]
  int N, H, row_bytes;
  int row_slot, slot_bytes;   // bytes reserved per input row / per group of stride_h rows
  int G;                      // groups one convolution row reads
  int P, Q;            // convolution output
  int R, Cf, pad_h, stride_h;
  int PP, QP;          // pooled output
  int bands, band_rows, units;
  int cr_bytes;        // bytes of one convolution-row ring slot
  float lo, hi;
  int *err;
};

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// Un-swizzled K-major operand: `lbo` bytes between 8-element K chunks, `sbo` bytes between
// groups of 8 rows.
__device__ __forceinline__ uint64_t desc_plain(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) |
         ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}

// The same, issued only when `valid` is non-zero (a predicated instruction, not a branch:
// a taken branch costs the single issuing thread more than the MMA it would skip).
__device__ __forceinline__ void mma_lohi_if(uint32_t valid, uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                            uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\n.reg .b64 da, db;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "setp.ne.b32 q, %7, 0;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(valid)
      : "memory");
}

// All MMAs of one convolution row, straight-line: R taps x KK K-steps, taps outside
// [r_lo, r_hi] predicated off.  Tap r reads row r % SH of the group in ring slot
// s0 + r / SH.
template <int R, int KK, int SH>
__device__ __forceinline__ void issue_row(uint32_t d_tmem, int r_lo, int r_hi, uint32_t s0,
                                          uint32_t a_lo0, uint32_t a_hi, uint32_t slot_desc,
                                          uint32_t row_desc, uint32_t b_lo0, uint32_t b_hi,
                                          uint32_t tap_desc, uint32_t kstep_desc, uint32_t idesc) {
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t valid = (r >= r_lo && r <= r_hi) ? 1u : 0u;
    const uint32_t s = (s0 + (uint32_t)(r / SH)) % ST_NIN;
    const uint32_t a_lo = a_lo0 + s * slot_desc + (uint32_t)(r % SH) * row_desc;
    const uint32_t b_lo = b_lo0 + (uint32_t)r * tap_desc;
#pragma unroll
    for (int kk = 0; kk < KK; ++kk)
      mma_lohi_if(valid, d_tmem, a_lo + 2 * kk, a_hi, b_lo + kk * kstep_desc, b_hi, idesc,
                  (r != r_lo || kk != 0) ? 1u : 0u);
  }
}

// byte offset of 16-byte chunk `c` (0..7) of pixel `px` in a convolution-row ring slot
__device__ __forceinline__ uint32_t cr_off(int px, int c) {
  return (uint32_t)(px * 128 + ((c ^ (px & 7)) << 4));
}

__global__ void __launch_bounds__(ST_THREADS, 1) stem_pool_kernel(const StemParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t w_bytes = (uint32_t)p.R * p.Cf * ST_K * 2;
  const uint32_t sW = base;
  const uint32_t sIn = sW + ((w_bytes + 1023u) & ~1023u);
  const uint32_t sCr = sIn + ST_NIN * p.slot_bytes;
  const uint32_t sMisc = sCr + ST_NCR * p.cr_bytes;
  uint8_t *misc_ptr = base_ptr + (sMisc - base);
  float *bias_s = reinterpret_cast<float *>(misc_ptr);                 // 64 floats
  uint64_t *bars = reinterpret_cast<uint64_t *>(misc_ptr + 256);
  const uint32_t bar0 = sMisc + 256;
  const uint32_t w_full = bar0;
  auto in_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto in_empty = [&](int s) { return bar0 + 8u * (1 + ST_NIN + s); };
  auto tfull = [&](int s) { return bar0 + 8u * (1 + 2 * ST_NIN + s); };
  auto tempty = [&](int s) { return bar0 + 8u * (1 + 2 * ST_NIN + ST_NACC + s); };
  auto cr_full = [&](int s) { return bar0 + 8u * (1 + 2 * ST_NIN + 2 * ST_NACC + s); };
  auto cr_empty = [&](int s) { return bar0 + 8u * (1 + 2 * ST_NIN + 2 * ST_NACC + ST_NCR + s); };
  constexpr int NBARS = 1 + 2 * ST_NIN + 2 * ST_NACC + 2 * ST_NCR;
  volatile uint32_t *tmem_holder = reinterpret_cast<volatile uint32_t *>(bars + NBARS);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + NBARS + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = ST_NACC * ST_K;

  if (threadIdx.x == 0) {
    mbar_init(w_full, 1);
    for (int s = 0; s < ST_NIN; ++s) {
      mbar_init(in_full(s), 1);
      mbar_init(in_empty(s), 2);   // both MMA issuers hand a group back
    }
    for (int s = 0; s < ST_NACC; ++s) {
      mbar_init(tfull(s), 1);
      mbar_init(tempty(s), ST_EPI_WARPS);
    }
    for (int s = 0; s < ST_NCR; ++s) {
      mbar_init(cr_full(s), ST_EPI_WARPS);
      mbar_init(cr_empty(s), ST_POOL_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // the tail of every input slot (past the row) is read by the MMA rows beyond Q: keep it finite
  for (uint32_t i = threadIdx.x * 16u; i < (uint32_t)ST_NIN * p.slot_bytes; i += ST_THREADS * 16u)
    *reinterpret_cast<uint4 *>(base_ptr + (sIn - base) + i) = make_uint4(0, 0, 0, 0);
  if (threadIdx.x < ST_K) bias_s[threadIdx.x] = p.bias ? p.bias[threadIdx.x] : 0.0f;
  fence_async_smem();
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
  int err_code = 0;
  pdl_launch_dependents();   // the next kernel's prologue may overlap this one
  pdl_wait();

  // pooled rows [i0, i1) and convolution rows [h_lo, h_hi] of a unit
  auto unit_rows = [&](int unit, int &n, int &i0, int &i1, int &h_lo, int &h_hi) {
    n = unit / p.bands;
    const int b = unit - n * p.bands;
    i0 = b * p.band_rows;
    i1 = min(i0 + p.band_rows, p.PP);
    h_lo = max(2 * i0 - 1, 0);
    h_hi = min(2 * (i1 - 1) + 1, p.P - 1);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    // Input rows travel in groups of stride_h rows, one ring slot and one barrier per
    // group: group g holds rows g*stride_h - pad_h ... + stride_h - 1, convolution row h
    // reads groups h ... h + G - 1 and is the last reader of group h.
    if (lane == 0) {
      mbar_expect_tx(w_full, w_bytes);
      bulk_g2s(sW, p.w, w_bytes, w_full);
      uint32_t gq = 0;   // groups loaded so far
      for (int unit = blockIdx.x; unit < p.units && !err_code; unit += gridDim.x) {
        int n, i0, i1, h_lo, h_hi;
        unit_rows(unit, n, i0, i1, h_lo, h_hi);
        const uint8_t *img = reinterpret_cast<const uint8_t *>(p.x) +
                             (size_t)n * p.H * p.row_bytes;
        for (int g = h_lo; g <= h_hi + p.G - 1; ++g, ++gq) {
          const uint32_t s = gq % ST_NIN, ph = (gq / ST_NIN) & 1u;
          if (!mbar_wait_sleepy(in_empty(s), ph ^ 1u, abort_flag)) {
            err_code = 1;
            break;
          }
          const int j0 = g * p.stride_h - p.pad_h;
          int valid = 0;
          for (int k = 0; k < p.stride_h; ++k) valid += (j0 + k >= 0 && j0 + k < p.H);
          mbar_expect_tx(in_full(s), (uint32_t)(valid * p.row_bytes));   // 0 bytes: a plain arrival
          for (int k = 0; k < p.stride_h; ++k)
            if (j0 + k >= 0 && j0 + k < p.H)
              bulk_g2s(sIn + s * p.slot_bytes + k * p.row_slot, img + (size_t)(j0 + k) * p.row_bytes,
                       (uint32_t)p.row_bytes, in_full(s));
        }
      }
    }
  } else if (warp == 1 || warp == ST_ISSUER_B) {
    // ------------------------------------------------------------ MMA issuers
    // Two threads (in two warps) take alternate convolution rows: the MMAs are short (64
    // columns) and one thread cannot issue them as fast as the tensor core retires them.
    // Both read every input group, so a group goes back to the producer when both have
    // committed it (each does so once it will not read the group again).
    if (lane == 0) {
      const int me = warp == 1 ? 0 : 1;
      constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) |
                                 ((uint32_t)(ST_K >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      if (!mbar_wait_hot(w_full, 0, abort_flag)) err_code = 2;
      uint32_t gbase = 0;   // ring index of the unit's first group
      uint32_t cbase = 0;   // convolution rows before this unit
      const int kk_n = p.Cf / 16;
      const uint64_t adesc0 = desc_plain(sIn, 16, 128);
      const uint64_t bdesc0 = desc_plain(sW, ST_K * 16, 128);
      const uint32_t a_lo0 = (uint32_t)adesc0, a_hi = (uint32_t)(adesc0 >> 32);
      const uint32_t b_lo0 = (uint32_t)bdesc0, b_hi = (uint32_t)(bdesc0 >> 32);
      const uint32_t slot_desc = (uint32_t)p.slot_bytes >> 4;        // descriptor steps
      const uint32_t row_desc = (uint32_t)p.row_slot >> 4;
      const uint32_t tap_desc = ((uint32_t)p.Cf * ST_K * 2) >> 4;
      const uint32_t kstep_desc = (2 * ST_K * 16) >> 4;
      for (int unit = blockIdx.x; unit < p.units && !err_code; unit += gridDim.x) {
        int n, i0, i1, h_lo, h_hi;
        unit_rows(unit, n, i0, i1, h_lo, h_hi);
        const int rows = h_hi - h_lo + 1;
        const int groups = rows + p.G - 1;        // groups the producer loads for this unit
        int waited = 0, released = 0;             // groups (unit-relative) waited for / committed
        // rows of the unit whose running number (over all units) has my parity
        for (int k = (int)((cbase + (uint32_t)me) & 1u); k < rows && !err_code; k += 2) {
          const uint32_t c = cbase + (uint32_t)k;
          const uint32_t a = c % ST_NACC, aph = (c / ST_NACC) & 1u;
          if (!mbar_wait_hot(tempty(a), aph ^ 1u, abort_flag)) {
            err_code = 3;
            break;
          }
          for (; waited < k + p.G; ++waited) {     // row k reads groups k ... k + G - 1
            const uint32_t gq = gbase + (uint32_t)waited;
            if (!mbar_wait_hot(in_full(gq % ST_NIN), (gq / ST_NIN) & 1u, abort_flag)) err_code = 4;
          }
          if (err_code) break;
          tc_fence_after();
          // taps whose input row lies inside the image (a row of padding contributes nothing)
          const int h = h_lo + k;
          const int jb = h * p.stride_h - p.pad_h;
          const int r_lo = max(0, -jb), r_hi = min(p.R - 1, p.H - 1 - jb);
          const uint32_t d_tmem = tmem_base + a * ST_K;
          const uint32_t s0 = (gbase + (uint32_t)k) % ST_NIN;
          // The issue code is straight-line: every taken branch costs the issuing thread more
          // than an MMA.
          if (p.R == 7 && kk_n == 2 && p.stride_h == 2) {
            issue_row<7, 2, 2>(d_tmem, r_lo, r_hi, s0, a_lo0, a_hi, slot_desc, row_desc, b_lo0, b_hi,
                               tap_desc, kstep_desc, IDESC);
          } else {
            uint32_t accumulate = 0;
            for (int r = r_lo; r <= r_hi; ++r) {
              const uint32_t s = (s0 + (uint32_t)(r / p.stride_h)) % ST_NIN;
              const uint32_t a_lo = a_lo0 + s * slot_desc + (uint32_t)(r % p.stride_h) * row_desc;
              const uint32_t b_lo = b_lo0 + (uint32_t)r * tap_desc;
              // 16 K values further on: 32 bytes along the row for A, two K chunks for B
              for (int kk = 0; kk < kk_n; ++kk) {
                mma_lohi(d_tmem, a_lo + 2 * kk, a_hi, b_lo + kk * kstep_desc, b_hi, IDESC, accumulate);
                accumulate = 1;
              }
            }
          }
          tc_commit(tfull(a));
          // my next row is k + 2: groups below it are of no more use to me
          for (; released < k + 2 && released < groups; ++released)
            tc_commit(in_empty((gbase + (uint32_t)released) % ST_NIN));
        }
        // whatever of the unit I have not committed yet (also when none of its rows was mine)
        for (; released < groups; ++released)
          tc_commit(in_empty((gbase + (uint32_t)released) % ST_NIN));
        gbase += (uint32_t)groups;
        cbase += (uint32_t)rows;
      }
    }
  } else if (warp < 2 + ST_EPI_WARPS) {
    // ------------------------------------------------------------ epilogue
    const int quad = warp & 3;               // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;        // channels [32 * half, 32 * half + 32)
    const int px = quad * 32 + lane;         // convolution output column
    const float lo = p.lo, hi = p.hi;
    const bool relu_only = lo == 0.0f && hi == INFINITY;
    uint32_t off[4];                         // this thread's four 16-byte pieces of a ring row
#pragma unroll
    for (int k = 0; k < 4; ++k) off[k] = cr_off(px, half * 4 + k);
    uint32_t c = 0;
    for (int unit = blockIdx.x; unit < p.units && !err_code; unit += gridDim.x) {
      int n, i0, i1, h_lo, h_hi;
      unit_rows(unit, n, i0, i1, h_lo, h_hi);
      for (int h = h_lo; h <= h_hi; ++h, ++c) {
        const uint32_t a = c % ST_NACC, aph = (c / ST_NACC) & 1u;
        const uint32_t cs = c % ST_NCR, cph = (c / ST_NCR) & 1u;
        if (!mbar_wait_sleepy(tfull(a), aph, abort_flag)) {
          err_code = 5;
          break;
        }
        tc_fence_after();
        uint32_t r[32];
        tc_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + a * ST_K + half * 32, r);
        tc_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty(a));
        uint32_t pk[16];
        const float4 *b4 = reinterpret_cast<const float4 *>(bias_s + half * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 b = b4[j];
          const uint64_t v0 = f2_add(f2_pack(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1])),
                                     f2_pack(b.x, b.y));
          const uint64_t v1 =
              f2_add(f2_pack(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])),
                     f2_pack(b.z, b.w));
          if (relu_only) {
            pk[2 * j] = f2_to_bf16x2_relu(v0);
            pk[2 * j + 1] = f2_to_bf16x2_relu(v1);
          } else {
            float x0, x1, x2, x3;
            f2_unpack(v0, x0, x1);
            f2_unpack(v1, x2, x3);
            pk[2 * j] = f2_to_bf16x2(f2_pack(tc_act(x0, lo, hi), tc_act(x1, lo, hi)));
            pk[2 * j + 1] = f2_to_bf16x2(f2_pack(tc_act(x2, lo, hi), tc_act(x3, lo, hi)));
          }
        }
        if (!mbar_wait_sleepy(cr_empty(cs), cph ^ 1u, abort_flag)) {
          err_code = 6;
          break;
        }
        if (px < p.Q) {
          uint8_t *row = base_ptr + (sCr - base) + cs * p.cr_bytes;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            *reinterpret_cast<uint4 *>(row + off[k]) =
                make_uint4(pk[4 * k], pk[4 * k + 1], pk[4 * k + 2], pk[4 * k + 3]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(cr_full(cs));
      }
    }
  } else if (warp < ST_ISSUER_B) {
    // ------------------------------------------------------------ pool
    const int pt = threadIdx.x - 32 * (2 + ST_EPI_WARPS);
    constexpr int PT = 32 * ST_POOL_WARPS;
    uint32_t cbase = 0;                    // ring index of the unit's first convolution row
    const int items = p.QP * 8;            // (pooled column, 16-byte channel chunk)
    for (int unit = blockIdx.x; unit < p.units && !err_code; unit += gridDim.x) {
      int n, i0, i1, h_lo, h_hi;
      unit_rows(unit, n, i0, i1, h_lo, h_hi);
      int rel = h_lo;   // next convolution row to hand back to the epilogue
      for (int i = i0; i < i1 && !err_code; ++i) {
        // Window rows / columns outside the image are replaced by the nearest inside one:
        // a duplicate does not change a maximum, and the code stays free of branches.
        const uint8_t *rows[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          const int hh = min(max(2 * i - 1 + k, 0), p.P - 1);
          const uint32_t cc = cbase + (uint32_t)(hh - h_lo);
          if (!mbar_wait_sleepy(cr_full(cc % ST_NCR), (cc / ST_NCR) & 1u, abort_flag)) err_code = 7;
          rows[k] = base_ptr + (sCr - base) + (cc % ST_NCR) * p.cr_bytes;
        }
        if (err_code) break;
        bf16 *yrow = p.y + ((size_t)n * p.PP + i) * p.QP * ST_K;
        for (int it = pt; it < items; it += PT) {
          const int jq = it >> 3, ch = it & 7;
          uint32_t o3[3];
#pragma unroll
          for (int k = 0; k < 3; ++k) o3[k] = cr_off(min(max(2 * jq - 1 + k, 0), p.Q - 1), ch);
          uint4 v[9];
#pragma unroll
          for (int a = 0; a < 3; ++a)
#pragma unroll
            for (int k = 0; k < 3; ++k) v[a * 3 + k] = *reinterpret_cast<const uint4 *>(rows[a] + o3[k]);
          uint4 o;
          uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 m = *reinterpret_cast<const __nv_bfloat162 *>(
                reinterpret_cast<const uint32_t *>(&v[0]) + e);
#pragma unroll
            for (int t = 1; t < 9; ++t)
              m = __hmax2_nan(m, *reinterpret_cast<const __nv_bfloat162 *>(
                                     reinterpret_cast<const uint32_t *>(&v[t]) + e));
            ow[e] = *reinterpret_cast<uint32_t *>(&m);
          }
          *reinterpret_cast<uint4 *>(yrow + (size_t)jq * ST_K + ch * 8) = o;
        }
        // convolution rows the next pooled row does not read go back to the epilogue
        const int keep = i + 1 == i1 ? h_hi + 1 : 2 * (i + 1) - 1;
        __syncwarp();
        for (; rel < keep && rel <= h_hi; ++rel)
          if (lane == 0) mbar_arrive(cr_empty((cbase + (uint32_t)(rel - h_lo)) % ST_NCR));
      }
      cbase += (uint32_t)(h_hi - h_lo + 1);
    }
  }

  if (err_code) {
    atomicExch(p.err, 1100 + err_code);
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

// fp32 KCRS (C <= Cp) -> bf16 [R][Cf/8][64][8]: tap row r, K chunk j, output channel n, and
// within the chunk k = 8j + e = s*Cp + c.
__global__ void pack_stem_kernel(const float *__restrict__ w, bf16 *__restrict__ out, int C, int R,
                                 int S, int Cp, int Cf, int total) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int e = i & 7;
    const int n = (i >> 3) % ST_K;
    const int j = (i / (8 * ST_K)) % (Cf / 8);
    const int r = i / (8 * ST_K * (Cf / 8));
    const int k = j * 8 + e;
    const int s2 = k / Cp, c = k % Cp;
    float v = 0.0f;
    if (s2 < S && c < C) v = w[(((int64_t)n * C + c) * R + r) * S + s2];
    out[i] = __float2bfloat16_rn(v);
  }
}

}  // namespace

bool stem_pool_supported(const StemPoolArgs &a) {
  if (a.K != ST_K || a.Cf % 16 || a.Cf > 64 || a.R < 1 || a.R > 11) return false;
  if (a.w_step_bytes != 16 || a.row_bytes % 16 || a.row_bytes > 8192) return false;
  if (a.Q < 1 || a.Q > 128 || a.P < 1 || a.stride_h < 1 || a.stride_h > 4) return false;
  if ((a.R - 1) / a.stride_h + 1 > ST_NIN - 2) return false;   // groups a row holds at once
  if (a.PP != (a.P + 2 - 3) / 2 + 1 || a.QP != (a.Q + 2 - 3) / 2 + 1) return false;
  if ((uintptr_t)a.x % 16 || (uintptr_t)a.w % 16 || (uintptr_t)a.y % 16) return false;
  // the last window the tensor core reads for a real column must lie inside the row
  if (16 * (a.Q - 1) + a.Cf * 2 > a.row_bytes) return false;
  return true;
}

size_t stem_pool_weight_bytes(int R, int Cf) { return (size_t)R * Cf * ST_K * 2; }

void launch_pack_stem_bf16(const float *w, bf16 *out, int C, int R, int S, int Cp, int Cf,
                           cudaStream_t s) {
  const int total = R * Cf * ST_K;
  pack_stem_kernel<<<(total + 255) / 256, 256, 0, s>>>(w, out, C, R, S, Cp, Cf, total);
  count(CNT_LAUNCHES);
}

bool launch_stem_pool(const StemPoolArgs &a, int *err_word, int num_sms, cudaStream_t s) {
  if (!stem_pool_supported(a)) return false;
  StemParams p;
  memset(&p, 0, sizeof(p));
  p.x = a.x; p.w = a.w; p.bias = a.bias; p.y = a.y;
  p.N = a.N; p.H = a.H; p.row_bytes = a.row_bytes;
  const int reach = 16 * 127 + a.Cf * 2;   // last byte + 1 the 128 MMA rows touch
  p.row_slot = ((a.row_bytes > reach ? a.row_bytes : reach) + 127) / 128 * 128;
  p.slot_bytes = p.row_slot * a.stride_h;
  p.G = (a.R - 1) / a.stride_h + 1;
  p.P = a.P; p.Q = a.Q; p.R = a.R; p.Cf = a.Cf; p.pad_h = a.pad_h; p.stride_h = a.stride_h;
  p.PP = a.PP; p.QP = a.QP;
  p.lo = a.lo; p.hi = a.hi;
  p.err = err_word;
  // bands: enough units to balance the SMs, each band re-computes one convolution row
  int bands = 1;
  while ((int64_t)a.N * bands < 6ll * num_sms && a.PP / (bands * 2) >= 4) bands *= 2;
  p.bands = bands;
  p.band_rows = (a.PP + bands - 1) / bands;
  p.bands = (a.PP + p.band_rows - 1) / p.band_rows;
  p.units = a.N * p.bands;
  p.cr_bytes = (a.Q * 128 + 1023) / 1024 * 1024;
  const size_t w_bytes = (stem_pool_weight_bytes(a.R, a.Cf) + 1023) / 1024 * 1024;
  const size_t smem = 1024 + w_bytes + (size_t)ST_NIN * p.slot_bytes + (size_t)ST_NCR * p.cr_bytes +
                      256 + 8 * 64;
  if (smem > (size_t)TC_SMEM_LIMIT || p.units == 0) return false;
  static unsigned char attr_done[TC_MAX_DEVICES] = {};
  if (tc_first_use_on_device(attr_done))
    cudaFuncSetAttribute(stem_pool_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         TC_SMEM_LIMIT);
  const int grid = p.units < num_sms ? p.units : num_sms;
  Runtime &r = rt();
  int prof_slot = -1;
  if (r.profiling) {   // timed like the other tensor-core launches
    prof_slot = r.prof_count++;
    while ((int)r.prof_events.size() < 2 * (prof_slot + 1)) {
      cudaEvent_t e;
      OCC_CUDA(cudaEventCreate(&e));
      r.prof_events.push_back(e);
    }
    OCC_CUDA(cudaEventRecord(r.prof_events[2 * prof_slot], s));
  }
  // at least half of the shared memory, so that one CTA (one TMEM allocation) runs per SM
  tc_launch_pdl(stem_pool_kernel, grid, ST_THREADS, smem < 120 * 1024 ? 120 * 1024 : smem, s, p);
  if (prof_slot >= 0) OCC_CUDA(cudaEventRecord(r.prof_events[2 * prof_slot + 1], s));
  count(CNT_LAUNCHES);
  count(CNT_TC_LAUNCHES);
  return cudaGetLastError() == cudaSuccess;
}

}  // namespace occ
