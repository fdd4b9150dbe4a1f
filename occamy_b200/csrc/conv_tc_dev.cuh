// Device side of the tcgen05 implicit-GEMM convolution: parameter block, PTX wrappers and
// the pixel-M kernel template.  Included by the translation units that instantiate the
// kernel (one per tile shape, so that they compile in parallel) and by the host planner.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <type_traits>

namespace occ {

constexpr int TC_THREADS = 320;      // pixel-N kernel: 1 producer warp + 1 MMA warp + 8 epilogue warps
constexpr int TC_EW = 2;             // tc_conv_kernel: epilogue warps per TMEM lane quadrant
constexpr int TC_NSTORE = 2;         // tc_conv_kernel: slab-store threads (slab buffers: a multiple)
constexpr int TC_EPI_THREADS = 256;
constexpr int TC_DBUF = 3;           // output slab buffers in shared memory
constexpr int TC_MAX_TAPS = 64;
constexpr int TC_MAX_AMAPS = 12;      // A tensor maps: 4 stride phases x 3 operand parts
constexpr int TC_SMEM_LIMIT = 232448;  // 227 KB
constexpr size_t TC_SMEM_DUO = 113 * 1024;  // per CTA when two share an SM (1 KB each is reserved)

// Division of a tile index (< 2^31) by a positive constant: q = umulhi(x, mul) >> shift,
// with mul == 0 standing for a divisor of one.
struct TcFastDiv {
  uint32_t mul, shift;
};

struct TcTap {
  int map, dw, dh;
};

struct alignas(64) TcParams {
  CUtensorMap tmA[TC_MAX_AMAPS];
  CUtensorMap tmB;
  CUtensorMap tmD;
  CUtensorMap tmR;
  TcTap taps[TC_MAX_TAPS];
  int num_taps, cblocks, bk, stages;
  int tiles_w, tiles_h, tiles_n, tiles_k, total_tiles;
  TcFastDiv div_k, div_w, div_h;   // divisions by tiles_k / tiles_w / tiles_h
  int tw, th, tn, K;
  const float *bias;
  int has_res, act;
  int gq, gp, gn;        // extents of the output grid the tiles are cut from
  float lo, hi;
  float *out_f32;
  int ldo;
  int out_hw;            // fp32 output: 0 = row-major [pixel][ldo]; else P * Q of an NCHW tensor
                         // [N][K][P][Q] that the epilogue writes directly (one channel per store
                         // instruction, consecutive lanes on consecutive pixels)
  int m_total;
  int consts_ready;      // filter and bias were resident before the launch: they may be
                         // fetched before the previous kernel in the stream has finished
  int halo;              // 3x3 halo form: the A block of a tile is loaded once, the taps are
                         // windows of it (see TC_MODE_HALO); then:
  int halo_wp;           //   pixels per block row (output width + 2)
  int halo_a_bytes;      //   bytes of one staged block, a multiple of 1024
  int bias_floats;       // K rounded up to whole channel tiles: bias entries kept in shared memory
  int dbuf;              // output slab buffers in shared memory (an even number, 4..12)
  int store_pend;        // stores a store thread may leave in flight behind its newest (0..3)
  int b_resident;        // one channel tile: the weight tiles of all k-steps are fetched once per CTA
#ifdef OCCAMY_TC_TIMERS
  long long *timers;     // 5 roles x 4 counters, or null
#endif
  int n_mma;             // pixel-N variant: N of the MMA (pixels per tile rounded up to 16)
  int sp_tiles;          // pixel tiles (tiles_w * tiles_h * tiles_n); with TC_MODE_PAIR the tile
                         // index counts PAIRS of them and total_tiles = ceil(sp_tiles / 2) * tiles_k
  int *err;
};

// Epilogue flavours the pixel-M kernel is compiled for (template parameter MODE).
// Per-role wait timers of CTA 0, for analysis builds only (-DOCCAMY_TC_TIMERS): four counters per
// role -- cycles in up to three kinds of wait and the role's total.
#ifdef OCCAMY_TC_TIMERS
#define TCT_DECL                      \
  long long tct_[4] = {0, 0, 0, 0};   \
  const long long tct_start_ = clock64();
#define TCT_WAIT(i, expr)                \
  ([&]() {                               \
    const long long t_ = clock64();      \
    const bool r_ = (expr);              \
    tct_[i] += clock64() - t_;           \
    return r_;                           \
  }())
#define TCT_FLUSH(slot)                                                  \
  if (blockIdx.x == 0 && p.timers) {                                     \
    for (int i_ = 0; i_ < 3; ++i_) p.timers[(slot) * 4 + i_] += tct_[i_]; \
    p.timers[(slot) * 4 + 3] += clock64() - tct_start_;                  \
  }
#else
#define TCT_DECL
#define TCT_WAIT(i, expr) (expr)
#define TCT_FLUSH(slot)
#endif
constexpr int TC_MODE_RES = 1;     // adds a residual tensor
constexpr int TC_MODE_CLAMP = 2;   // general clamp to [lo, hi]; otherwise ReLU
constexpr int TC_MODE_F32 = 4;     // fp32 row-major output straight to global memory (GEMM head)
// 3x3 / stride 1 / pad 1 with 64 input channels and resident weights: the producer loads a
// tile's input block (its rows plus one row above and below, whole image width plus one zero
// column on either side) ONCE and the nine taps are windows of that block, shifted by whole
// pixels - a swizzled operand may start at any multiple of 128 bytes inside a 1024-aligned
// buffer.  The tile is th full rows of width W + 2; its two extra columns are junk that the
// TMA store clips.
constexpr int TC_MODE_HALO = 8;
// Operands and output are fp16 instead of bf16 (same MMA kind, same rate, other format bits
// in the instruction descriptor and other conversion instructions in the epilogue).
constexpr int TC_MODE_F16 = 16;
// Two CTAs on neighbouring SMs (a cluster of two) work as one 256-pixel x BN tile: each loads
// its own 128 pixels of A and HALF of the B tile, the first CTA of the pair issues
// tcgen05.mma.cta_group::2 instructions that read both halves, and each CTA's TMEM receives
// the accumulator rows of its own pixels.  Shared memory takes in two thirds of the bytes per
// flop of the single-CTA form, which is what bounds the long-reduction layers.  No multicast
// load is involved: every TMA load has one destination.
constexpr int TC_MODE_PAIR = 32;
// fp32 operands carried as bf16 parts (six taps per filter tap, see the planner): the hi * hi
// products go into one accumulator and the five correction products into a second one, which
// the epilogue adds.  The tensor core truncates when it adds into an fp32 accumulator, a bias
// toward zero that grows with the number of additions at full magnitude; kept apart, the small
// terms cost the main sum no additions (and their own truncation is 2^-8 smaller).
constexpr int TC_MODE_SPLIT = 64;

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t cnt) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(cnt));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t a, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t a) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t a, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(a), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~2 s of polling or as soon as another role has given up.
// The polling loop is kept out of line: every role has several waits, and the kernel's code
// has to stay small enough for the instruction cache.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t a, uint32_t parity, volatile int *abort_flag) {
  const long long t0 = clock64();
  int it = 0;
  while (!mbar_try(a, parity)) {
    if ((++it & 15) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > 4000000000LL) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ bool mbar_wait(uint32_t a, uint32_t parity, volatile int *abort_flag) {
  if (mbar_try(a, parity)) return true;
  return mbar_wait_slow(a, parity, abort_flag);
}
// The same wait for roles with slack: sleeps between polls, so that many waiting warps do
// not take issue slots away from a single thread that is issuing short MMAs.
static __device__ __noinline__ bool mbar_wait_sleepy(uint32_t a, uint32_t parity,
                                                     volatile int *abort_flag) {
  if (mbar_try(a, parity)) return true;
  const long long t0 = clock64();
  int it = 0;
  while (!mbar_try(a, parity)) {
    __nanosleep(128);
    if ((++it & 15) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > 4000000000LL) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}
// The same wait, polling loop inline: for the producer and MMA roles, whose loops are tiny
// and where the return from a call would sit on the critical path of every k-step.
__device__ __forceinline__ bool mbar_wait_hot(uint32_t a, uint32_t parity,
                                              volatile int *abort_flag) {
  if (mbar_try(a, parity)) return true;
  const long long t0 = clock64();
  int it = 0;
  while (!mbar_try(a, parity)) {
    if ((++it & 15) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > 4000000000LL) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *m, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(m), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *m, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(m), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *m, uint32_t src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(m),
      "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// ---- CTA-pair forms (TC_MODE_PAIR).  `bar` is a shared::cluster address, normally of a
// barrier in the pair's first CTA; the data always lands in the issuing CTA's own memory.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap *m, uint32_t bar,
                                                 int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(m), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *m, uint32_t bar,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(m), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Completion of the pair's MMAs so far, signalled on the barrier at this offset in both CTAs.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void mma_lohi_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                              uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n.reg .b64 da, db;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap *m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may
// start while the kernel before it in the stream is still running.  `pdl_wait` returns once
// that kernel has completed and its writes are visible: nothing before it may touch memory
// other kernels write or read.  `pdl_launch_dependents` lets the kernel after this one be
// scheduled as soon as SMs free up, so that its prologue overlaps this kernel's tail.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Two fp32 values in one 64-bit register (packed fp32 arithmetic of sm_100).
__device__ __forceinline__ uint64_t f2_pack(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float &a, float &b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// (a, b) -> two 16-bit values (bf16, or fp16 when F16) with a in the low half; the second form
// clamps negatives to zero.
template <bool F16 = false>
__device__ __forceinline__ uint32_t f2_to_bf16x2(uint64_t v) {
  float a, b;
  f2_unpack(v, a, b);
  uint32_t r;
  if constexpr (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
template <bool F16 = false>
__device__ __forceinline__ uint32_t f2_to_bf16x2_relu(uint64_t v) {
  float a, b;
  f2_unpack(v, a, b);
  uint32_t r;
  if constexpr (F16) asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  else asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
// two 16-bit values in one word -> packed fp32 pair (low half first)
template <bool F16>
__device__ __forceinline__ uint64_t pair16_to_f2(uint32_t w) {
  if constexpr (F16) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&w));
    return f2_pack(t.x, t.y);
  } else {   // a bf16 is the top half of the fp32 of its value
    return f2_pack(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  }
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// One MMA; the descriptors arrive as 32-bit halves (address field in the low word).
__device__ __forceinline__ void mma_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                         uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n.reg .b64 da, db;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7])
      : "r"(taddr)
      : "memory");
}
template <int W>
__device__ __forceinline__ void tc_ld(uint32_t taddr, uint32_t *r) {
  if constexpr (W == 32) tc_ld32(taddr, r);
  else if constexpr (W == 16) tc_ld16(taddr, r);
  else tc_ld8(taddr, r);
}
__device__ __forceinline__ void tc_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
template <int THREADS>
__device__ __forceinline__ void epi_bar_n() {
  asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
}

// Shared-memory matrix descriptor for a K-major bf16 tile whose rows are `bk` elements
// (32 / 64 / 128 bytes, swizzled with the matching 32B / 64B / 128B pattern): 8-row groups
// are 8*bk*2 bytes apart; descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, int bk) {
  const uint32_t sbo = (uint32_t)(8 * bk * 2);
  const uint64_t layout = bk == 64 ? 2ull : (bk == 32 ? 4ull : 6ull);
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(sbo >> 4) << 32) |
         (1ull << 46) | (layout << 61);
}

// The fused activations (identity, ReLU, clipped ReLU) are all a clamp to [lo, hi]; keeping
// the epilogue to that one form keeps its unrolled body small.
__device__ __forceinline__ float tc_act(float v, float lo, float hi) {
  return fminf(fmaxf(v, lo), hi);
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a staged slab whose rows are
// `row_bytes` (64 or 128) long, with the TMA swizzle of that width applied.
__device__ __forceinline__ uint32_t slab_off(int row, int chunk, int row_bytes) {
  const uint32_t off = (uint32_t)(row * row_bytes + chunk * 16);
  const uint32_t mask = (uint32_t)(row_bytes / 16 - 1);
  return off ^ (((off >> 7) & mask) << 4);
}

// ------------------------------------------------------------------ tile walk
__device__ __forceinline__ uint32_t tc_fdiv(uint32_t x, TcFastDiv d) {
  return d.mul ? (__umulhi(x, d.mul) >> d.shift) : x;
}
struct TcTile {
  int k0, q0, p0, n0;   // first output channel / column / row / image of the tile
};
// Tiles are numbered channel-tile fastest, then column, row and image tiles.
// In a CTA pair `rank` selects the pixel tile of the pair; the second CTA of an odd last pair
// gets the first one's tile again (`ghost`): it computes it and stores nothing.
template <int BN, bool PAIR = false>
__device__ __forceinline__ TcTile tc_decode(const TcParams &p, int tile, uint32_t rank = 0,
                                            bool *ghost = nullptr) {
  uint32_t sp = tc_fdiv((uint32_t)tile, p.div_k);
  const uint32_t kt = (uint32_t)tile - sp * (uint32_t)p.tiles_k;
  if constexpr (PAIR) {
    sp = 2u * sp + rank;
    const bool g = sp >= (uint32_t)p.sp_tiles;
    if (g) sp -= 1u;
    if (ghost) *ghost = g;
  }
  const uint32_t s2 = tc_fdiv(sp, p.div_w);
  const uint32_t wq = sp - s2 * (uint32_t)p.tiles_w;
  const uint32_t nn = tc_fdiv(s2, p.div_h);
  const uint32_t hp = s2 - nn * (uint32_t)p.tiles_h;
  TcTile t;
  t.k0 = (int)kt * BN;
  t.q0 = (int)wq * p.tw;
  t.p0 = (int)hp * p.th;
  t.n0 = (int)nn * p.tn;
  return t;
}

// ------------------------------------------------------------------ the kernel
// Pixels are the M side of the MMA (128 per tile), output channels the N side (BN per tile).
//   DC   channels per staged output slab (64; 32 trades slab size for ring depth)
//   EW   epilogue warps per TMEM lane quadrant; they split a slab's channels between them
//   MODE epilogue flavour (TC_MODE_* bits); one flavour per instantiation keeps the code of
//        a launch small, which matters: the roles run different code at the same time and
//        instruction-cache misses stall all of them
//
// One persistent CTA per SM:
//   warp 0            TMA producer (one lane): fills a ring of {A, B} stages
//   warp 1            MMA issuer (one lane): tcgen05.mma 128 x BN x 16, fp32 accumulators in
//                     TMEM, two accumulator buffers
//   warps 2..2+4*EW   epilogue: tcgen05.ld the finished accumulator, add bias / residual,
//                     activation, convert to bf16, write 128-pixel slabs of DC channels into
//                     swizzled shared memory
//   TC_NSTORE warps   slab store (one lane each): hand slab buffers to the epilogue (empty,
//                     or pre-loaded with the residual slab) and TMA-store written slabs
//   last warp         second MMA issuer of the halo form (idle otherwise)
// Every wait on an mbarrier is bounded; when a bound is hit the kernel records a code in the
// error word, drains and returns.
// Threads of a CTA: producer and MMA warps, 4 * EW epilogue warps, the slab-store warps and (for
// the halo form, which exists with EW == 2 only) the warp of the second MMA issuer.
constexpr int tc_block_threads(int ew) { return 64 + 128 * ew + 32 * TC_NSTORE + (ew == 1 ? 0 : 32); }

template <int BN, int DC, int EW, int MODE>
__global__ void __launch_bounds__(tc_block_threads(EW), EW == 1 ? 2 : 1)
    tc_conv_kernel(const __grid_constant__ TcParams p) {
  constexpr bool RES = (MODE & TC_MODE_RES) != 0;
  constexpr bool CLAMP = (MODE & TC_MODE_CLAMP) != 0;
  constexpr bool F32 = (MODE & TC_MODE_F32) != 0;
  constexpr bool HALO = (MODE & TC_MODE_HALO) != 0;
  constexpr bool F16 = (MODE & TC_MODE_F16) != 0;
  constexpr bool PAIR = (MODE & TC_MODE_PAIR) != 0;
  constexpr bool SPLIT = (MODE & TC_MODE_SPLIT) != 0;
  static_assert(!(PAIR && (HALO || F32)), "the CTA-pair form exists for the plain epilogues only");
  static_assert(!SPLIT || (F32 && !HALO && BN <= 128), "split operands: fp32 output, four accumulators");
  constexpr int ACC_COLS = SPLIT ? 2 * BN : BN;   // TMEM columns of one tile's accumulator(s)
  constexpr int EPI_THREADS = 128 * EW;
  constexpr int STORE_WARP = 2 + 4 * EW;
  constexpr int CW = DC / EW;                  // channels one epilogue thread handles per slab
  constexpr int NSLAB = BN / DC;
  constexpr int SLAB_BYTES = 128 * DC * 2;
  // fp32 accumulator; A and B formats: 1 = bf16, 0 = fp16; N / 8 and M / 16
  constexpr uint32_t IDESC = (1u << 4) | (F16 ? 0u : ((1u << 7) | (1u << 10))) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((PAIR ? 256 : 128) >> 4) << 24);
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;
  constexpr int BROWS = PAIR ? BN / 2 : BN;    // rows of the B tile this CTA loads

  // The swizzled operand tiles need 1024-byte alignment.  The kernel has no static shared
  // memory, so its dynamic block starts on such a boundary and the host budgets no slack for
  // rounding up; should that ever not hold, the launch reports it instead of running past
  // the end of its allocation.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if ((smem_u32(smem_raw) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicExch(p.err, 1007);
    return;
  }
  const uint32_t base = smem_u32(smem_raw);
  uint8_t *base_ptr = smem_raw;
  const int bk = p.bk, stages = p.stages, dbuf = p.dbuf;
  // halo form: the ring carries input blocks only, the weights of all taps sit behind it
  const uint32_t a_bytes = HALO ? (uint32_t)p.halo_a_bytes : 128u * bk * 2u;
  const uint32_t b_bytes = (uint32_t)BROWS * bk * 2u;
  const uint32_t sA = base;
  const uint32_t sB = sA + stages * a_bytes;
  // weight tiles: one per ring stage, or (halo form, resident form) one per k-step of a tile
  const bool bres = !HALO && !PAIR && p.b_resident != 0;
  // Activations and weights of a k-step are requested by two threads of different warps (the
  // weight loader is the warp that issues MMAs in the halo form, idle otherwise): a lone loading
  // thread was busy 78 % of the time on the 3x3 layers (barrier poll, arming arrival and two
  // TMA requests per k-step).  Measured 3 % on those layers, nothing elsewhere.
  constexpr bool SPLIT_LOAD = !HALO && !PAIR && EW == 2;
  const bool two_loaders = SPLIT_LOAD && !bres;
  constexpr int WLOAD_WARP = 2 + 4 * EW + TC_NSTORE;
  const uint32_t b_slots = HALO ? (uint32_t)p.num_taps
                                : (bres ? (uint32_t)(p.num_taps * p.cblocks) : (uint32_t)stages);
  const uint32_t sD = sB + b_slots * b_bytes;   // dbuf output slabs
  const uint32_t sMisc = sD + dbuf * SLAB_BYTES;
  uint8_t *misc_ptr = base_ptr + (sMisc - base);
  float *bias_s = reinterpret_cast<float *>(misc_ptr);          // bias of every output channel
  uint64_t *bars = reinterpret_cast<uint64_t *>(misc_ptr + p.bias_floats * 4);
  const uint32_t bar0 = sMisc + p.bias_floats * 4;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (stages + s); };
  auto tfull_bar = [&](int s) { return bar0 + 8u * (2 * stages + s); };
  auto tempty_bar = [&](int s) { return bar0 + 8u * (2 * stages + 2 + s); };
  auto rfull_bar = [&](int s) { return bar0 + 8u * (2 * stages + 4 + s); };
  auto dfull_bar = [&](int s) { return bar0 + 8u * (2 * stages + 4 + dbuf + s); };
  const uint32_t wfull_bar = bar0 + 8u * (2 * stages + 4 + 2 * dbuf);   // halo form: weights landed
  volatile uint32_t *tmem_holder =
      reinterpret_cast<volatile uint32_t *>(bars + 2 * stages + 5 + 2 * dbuf);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * stages + 6 + 2 * dbuf);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;     // 0: the CTA that issues the MMAs
  const int tile0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tstep = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    // descriptor fetches are off the critical path of the first loads / stores
    tma_prefetch_map(&p.tmA[0]);
    tma_prefetch_map(&p.tmB);
    if (!F32) tma_prefetch_map(&p.tmD);
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), two_loaders ? 2 : 1);   // one arming arrival per loading thread
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      // one arrival per epilogue warp (of both CTAs of a pair): arrivals on one barrier are
      // serialised
      mbar_init(tempty_bar(s), (PAIR ? 2 : 1) * EPI_THREADS / 32);
    }
    for (int s = 0; s < dbuf; ++s) {
      mbar_init(rfull_bar(s), 1);
      mbar_init(dfull_bar(s), EPI_THREADS / 32);
    }
    mbar_init(wfull_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    if constexpr (PAIR) {   // the same warp of both CTAs allocates for the pair
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32((const void *)tmem_holder)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32((const void *)tmem_holder)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  // both CTAs' barriers exist before either signals the other's
  if constexpr (PAIR) cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int rows_valid = p.tw * p.th * p.tn;
  const int ksteps = p.num_taps * p.cblocks;
  int err_code = 0;
  // Everything above touched only this CTA's shared memory and TMEM, so it may overlap the
  // previous kernel in the stream.  Resident weights may be fetched early as well: the
  // producer requests the weight tiles of its first k-steps (halo form: all of them) now.
  int pre_b = 0;   // leading k-steps of the first tile whose weight tile is already on its way
  // resident form: the weight tiles of every k-step, once, announced on the "weights landed" barrier
  auto load_resident_b = [&]() {
    mbar_expect_tx(wfull_bar, (uint32_t)ksteps * b_bytes);
    int i = 0;
    for (int t = 0; t < p.num_taps; ++t)
      for (int cb = 0; cb < p.cblocks; ++cb, ++i)
        tma_load_3d(sB + i * b_bytes, &p.tmB, wfull_bar, cb * bk, 0, t);
  };
  if (!PAIR && warp == (two_loaders ? WLOAD_WARP : 0) && lane == 0 && p.consts_ready &&
      (int)blockIdx.x < p.total_tiles) {
    if constexpr (HALO) {
      mbar_expect_tx(wfull_bar, (uint32_t)p.num_taps * b_bytes);
      for (int t = 0; t < p.num_taps; ++t)
        tma_load_3d(sB + t * b_bytes, &p.tmB, wfull_bar, 0, 0, t);
    } else if (bres) {
      load_resident_b();
    } else {
      const TcTile tl = tc_decode<BN>(p, blockIdx.x);
      pre_b = min(stages, ksteps);
      int t = 0, cb = 0;
      for (int s = 0; s < pre_b; ++s) {
        // a lone loader arms the barrier for both operands here; of two, each arms its own
        mbar_expect_tx(full_bar(s), two_loaders ? b_bytes : (uint32_t)rows_valid * bk * 2u + b_bytes);
        tma_load_3d(sB + s * b_bytes, &p.tmB, full_bar(s), cb * bk, tl.k0, t);
        if (++cb == p.cblocks) {
          cb = 0;
          ++t;
        }
      }
    }
  }
  pdl_launch_dependents();
  pdl_wait();   // from here on memory that other kernels write is read and written

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      if constexpr (HALO) {
        // weights of all taps once (unless they were requested early), then one input block
        // per tile
        if (!p.consts_ready) {
          mbar_expect_tx(wfull_bar, (uint32_t)p.num_taps * b_bytes);
          for (int t = 0; t < p.num_taps; ++t)
            tma_load_3d(sB + t * b_bytes, &p.tmB, wfull_bar, 0, 0, t);
        }
        const uint32_t blk_bytes = (uint32_t)((p.th + 2) * p.halo_wp) * 128u;
        for (int tile = blockIdx.x; tile < p.total_tiles && !err_code; tile += gridDim.x) {
          const TcTile tl = tc_decode<BN>(p, tile);
          if (!mbar_wait_hot(empty_bar(stage), phase ^ 1u, abort_flag)) {
            err_code = 1;
            break;
          }
          mbar_expect_tx(full_bar(stage), blk_bytes);
          // column -1 and row p0 - 1 onwards; what lies outside the image arrives as zeros
          tma_load_4d(sA + stage * a_bytes, &p.tmA[0], full_bar(stage), 0, -1, tl.p0 - 1, tl.n0);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      } else {
      const uint32_t tx_bytes = (uint32_t)rows_valid * bk * 2u + (bres ? 0u : b_bytes);
      if (bres && !p.consts_ready) load_resident_b();
      TCT_DECL
      for (int tile = tile0; tile < p.total_tiles && !err_code; tile += tstep) {
        const TcTile tl = tc_decode<BN, PAIR>(p, tile, rank);
        for (int t = 0; t < p.num_taps && !err_code; ++t) {
          const TcTap tap = p.taps[t];
          for (int cb = 0; cb < p.cblocks; ++cb) {
            if (!TCT_WAIT(0, mbar_wait_hot(empty_bar(stage), phase ^ 1u, abort_flag))) {
              err_code = 1;
              break;
            }
            if constexpr (PAIR) {
              // Both CTAs' bytes are counted on the first CTA's barrier, which that CTA arms
              // for the two of them; each CTA fetches its own pixels and its half of B.
              const uint32_t fb = cluster_map(full_bar(stage), 0);
              if (rank == 0) mbar_expect_tx(full_bar(stage), 2u * tx_bytes);
              tma_load_3d_pair(sB + stage * b_bytes, &p.tmB, fb, cb * bk,
                               tl.k0 + (int)rank * BROWS, t);
              tma_load_4d_pair(sA + stage * a_bytes, &p.tmA[tap.map], fb, cb * bk, tl.q0 + tap.dw,
                               tl.p0 + tap.dh, tl.n0);
              if (++stage == stages) {
                stage = 0;
                phase ^= 1u;
              }
              continue;
            }
            if (two_loaders) {
              mbar_expect_tx(full_bar(stage), tx_bytes - b_bytes);   // the weight loader arms its own
            } else if (pre_b > 0) {
              --pre_b;   // this stage's barrier is armed and its weight tile on its way
            } else if (bres) {
              mbar_expect_tx(full_bar(stage), tx_bytes);   // the weights are resident
            } else {
              mbar_expect_tx(full_bar(stage), tx_bytes);
              tma_load_3d(sB + stage * b_bytes, &p.tmB, full_bar(stage), cb * bk, tl.k0, t);
            }
            tma_load_4d(sA + stage * a_bytes, &p.tmA[tap.map], full_bar(stage), cb * bk,
                        tl.q0 + tap.dw, tl.p0 + tap.dh, tl.n0);
            if (++stage == stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      TCT_FLUSH(0)
      }
    }
  } else if (warp == 1 || (HALO && warp == STORE_WARP + TC_NSTORE)) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && rank == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      if constexpr (HALO) {
        // 3x3 taps as shifted windows of the staged block: (dh * wp + dw) pixels of 128 bytes
        // further on.  Straight-line issue code: the MMAs are short when BN is small, and a
        // taken branch costs the issuing thread more than one of them.
        const uint64_t d0 = make_smem_desc(sA, 64);
        const uint32_t a_hi = (uint32_t)(d0 >> 32), b_hi = a_hi;
        const uint32_t a_lo0 = (uint32_t)d0;
        const uint32_t b_lo0 = (uint32_t)make_smem_desc(sB, 64);
        const uint32_t stage_desc = a_bytes >> 4, tap_desc = b_bytes >> 4;
        const uint32_t wp8 = (uint32_t)p.halo_wp * 8u;   // one block row in descriptor units
        if (!mbar_wait_hot(wfull_bar, 0, abort_flag)) err_code = 3;
        // Two issuing threads take alternate tiles (and with them alternate accumulators):
        // 36 MMAs of 48 cycles per tile are more than one thread issues in that time.
        const int me = warp == 1 ? 0 : 1;
        int it = 0;   // tiles of this CTA so far
        for (int tile = blockIdx.x; tile < p.total_tiles && !err_code; tile += gridDim.x, ++it) {
          if (++stage == stages) {   // ring stage and accumulator advance with every tile
            stage = 0;
            phase ^= 1u;
          }
          const int my_stage = stage == 0 ? stages - 1 : stage - 1;
          const uint32_t my_phase = stage == 0 ? phase ^ 1u : phase;
          const int my_acc = it & 1;
          const uint32_t my_acc_phase = (uint32_t)(it >> 1) & 1u;
          if ((it & 1) != me) continue;
          if (!mbar_wait_hot(tempty_bar(my_acc), my_acc_phase ^ 1u, abort_flag)) {
            err_code = 2;
            break;
          }
          if (!mbar_wait_hot(full_bar(my_stage), my_phase, abort_flag)) {
            err_code = 3;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(my_acc * BN);
          const uint32_t a_lo = a_lo0 + (uint32_t)my_stage * stage_desc;
#pragma unroll
          for (int t = 0; t < 9; ++t) {
            const uint32_t at = a_lo + (uint32_t)(t / 3) * wp8 + (uint32_t)(t % 3) * 8u;
            const uint32_t bt = b_lo0 + (uint32_t)t * tap_desc;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              mma_lohi(d_tmem, at + 2 * kk, a_hi, bt + 2 * kk, b_hi, IDESC, (t | kk) ? 1u : 0u);
          }
          tc_commit(empty_bar(my_stage));
          tc_commit(tfull_bar(my_acc));
        }
      } else {
      TCT_DECL
      if (bres && !mbar_wait_hot(wfull_bar, 0, abort_flag)) err_code = 3;
      {
        // This thread's instruction stream is the kernel's critical path on the tensor-bound
        // layers: the tensor pipe takes MMAs in order and holds very few that have not started,
        // so every instruction between the last MMA of one k-step and the first of the next is
        // time the pipe runs dry (an extra loop and a flag per k-step measured 17 % on the 3x3
        // layers).  Hence: one copy of the tile loop per number of MMAs in a k-step, the
        // k-step body straight-line, descriptors as 32-bit halves that advance by adding, the
        // accumulate flag a predicate.
        const uint64_t a0 = make_smem_desc(sA, bk), b0 = make_smem_desc(sB, bk);
        const uint32_t a_hi = (uint32_t)(a0 >> 32), b_hi = (uint32_t)(b0 >> 32);
        const uint32_t a_lo0 = (uint32_t)a0, b_lo0 = (uint32_t)b0;
        const uint32_t a_step = a_bytes >> 4, b_step = b_bytes >> 4;   // one stage, in descriptor units
        auto run_tiles = [&](auto nk_c) {
          constexpr int NK = decltype(nk_c)::value;   // MMAs per k-step: bk / 16
          uint32_t a_lo = a_lo0, b_lo = b_lo0;
          for (int tile = tile0; tile < p.total_tiles; tile += tstep) {
            if (!TCT_WAIT(0, mbar_wait_hot(tempty_bar(acc), acc_phase ^ 1u, abort_flag))) {
              err_code = 2;
              return;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(acc * ACC_COLS);
            // split operands: tap 0 of every group of six is hi * hi and goes to the main
            // accumulator, the other five (corrections) to the second one
            uint32_t seen_main = 0, seen_corr = 0;
            int cb_in_tap = 0, combo = 0;
            for (int ks = 0; ks < ksteps; ++ks) {
              if (!TCT_WAIT(1, mbar_wait_hot(full_bar(stage), phase, abort_flag))) {
                err_code = 3;
                return;
              }
              tc_fence_after();
              const uint32_t bl = bres ? b_lo0 + (uint32_t)ks * b_step : b_lo;
              if constexpr (SPLIT) {
                const bool corr = combo != 0;
                const uint32_t d = corr ? d_tmem + (uint32_t)BN : d_tmem;
                const uint32_t first = corr ? seen_corr : seen_main;
#pragma unroll
                for (int kk = 0; kk < NK; ++kk)
                  mma_lohi(d, a_lo + 2u * kk, a_hi, bl + 2u * kk, b_hi, IDESC, kk ? 1u : first);
                if (corr) seen_corr = 1u;
                else seen_main = 1u;
                if (++cb_in_tap == p.cblocks) {
                  cb_in_tap = 0;
                  if (++combo == 6) combo = 0;
                }
              } else {
#pragma unroll
                for (int kk = 0; kk < NK; ++kk) {
                  const uint32_t accumulate = kk ? 1u : (uint32_t)(ks != 0);
                  if constexpr (PAIR)   // the same offsets in the other CTA hold its pixels and B half
                    mma_lohi_pair(d_tmem, a_lo + 2u * kk, a_hi, bl + 2u * kk, b_hi, IDESC, accumulate);
                  else
                    mma_lohi(d_tmem, a_lo + 2u * kk, a_hi, bl + 2u * kk, b_hi, IDESC, accumulate);
                }
              }
              if constexpr (PAIR) tc_commit_pair(empty_bar(stage));   // frees the stage in both CTAs
              else tc_commit(empty_bar(stage));
              a_lo += a_step;
              b_lo += b_step;
              if (++stage == stages) {
                stage = 0;
                phase ^= 1u;
                a_lo = a_lo0;
                b_lo = b_lo0;
              }
            }
            if constexpr (PAIR) tc_commit_pair(tfull_bar(acc));
            else tc_commit(tfull_bar(acc));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
          }
        };
        if (!err_code) {
          if (bk == 64) run_tiles(std::integral_constant<int, 4>{});
          else if (bk == 32) run_tiles(std::integral_constant<int, 2>{});
          else run_tiles(std::integral_constant<int, 1>{});
        }
      }
      TCT_FLUSH(1)
      }
    }
  } else if (warp >= STORE_WARP && warp < STORE_WARP + TC_NSTORE) {
    // ------------------------------------------------------------ slab store
    // TC_NSTORE threads (one per warp) own the output slab buffers, slab d belonging to
    // thread d % TC_NSTORE: the owner hands the buffer to the epilogue warps ("ready": free,
    // or holding the residual slab the epilogue adds in place) and sends the written slab to
    // global memory.  The epilogue warps never wait for one another.  More than one thread,
    // because a single thread's issue rate (TMA store + residual load + bookkeeping per slab)
    // limits the layers whose tiles are short.
    if constexpr (!F32) {
      if (lane == 0) {
        const uint32_t me = (uint32_t)(warp - STORE_WARP);
        auto nslab_of = [&](const TcTile &t) { return min(NSLAB, (p.K - t.k0 + DC - 1) / DC); };
        // cursor over the slabs this thread makes ready: (tile, slab) of slab number r_next
        uint32_t r_next = me;
        int r_tile = tile0, r_sl = 0;
        TcTile rt_ = tc_decode<BN, PAIR>(p, r_tile, rank);
        int r_ns = nslab_of(rt_);
        auto r_advance = [&]() {          // one slab further
          if (++r_sl == r_ns) {
            r_sl = 0;
            r_tile += tstep;
            if (r_tile < p.total_tiles) {
              rt_ = tc_decode<BN, PAIR>(p, r_tile, rank);
              r_ns = nslab_of(rt_);
            }
          }
        };
        // Without a residual a hand-out needs no coordinates, and when every tile has the same
        // number of slabs the count of this CTA's slabs says where to stop: no cursor at all.
        // (This thread's instructions per slab are what the few-channel layers with wide
        // outputs wait for; divisions by the runtime buffer count are replaced by counters
        // that step by TC_NSTORE for the same reason.)
        const bool uniform = !RES && (p.tiles_k == 1 || p.K % BN == 0);
        uint32_t left = 0;   // uniform form: hand-outs this thread still owes
        if (uniform && tile0 < p.total_tiles) {
          const uint32_t my_tiles = (uint32_t)((p.total_tiles - tile0 + tstep - 1) / tstep);
          const uint32_t per_tile = (uint32_t)min(NSLAB, (p.tiles_k == 1 ? p.K + DC - 1 : BN) / DC);
          const uint32_t total = my_tiles * per_tile;
          left = total > me ? (total - me + TC_NSTORE - 1) / TC_NSTORE : 0u;
        }
        if (!uniform)
          for (uint32_t i = 0; i < me && r_tile < p.total_tiles; ++i) r_advance();
        uint32_t rb = me;   // buffer of my next hand-out: steps by TC_NSTORE around the ring
        auto ready_one = [&]() {          // hand out slab r_next, move to my next one
          if (uniform) {
            if (left == 0) return;
            --left;
            mbar_arrive(rfull_bar(rb));
            rb += TC_NSTORE;
            if (rb >= (uint32_t)dbuf) rb -= (uint32_t)dbuf;
            return;
          }
          if (r_tile >= p.total_tiles) return;
          if constexpr (RES) {
            mbar_expect_tx(rfull_bar(rb), (uint32_t)rows_valid * DC * 2u);
            tma_load_4d(sD + rb * SLAB_BYTES, &p.tmR, rfull_bar(rb), rt_.k0 + r_sl * DC, rt_.q0,
                        rt_.p0, rt_.n0);
          } else {
            mbar_arrive(rfull_bar(rb));
          }
          r_next += TC_NSTORE;
          rb += TC_NSTORE;
          if (rb >= (uint32_t)dbuf) rb -= (uint32_t)dbuf;
          for (int i = 0; i < TC_NSTORE && r_tile < p.total_tiles; ++i) r_advance();
        };
        for (int i = 0; i < dbuf / TC_NSTORE; ++i) ready_one();     // every buffer starts out free
        uint32_t d = 0;   // running slab number
        uint32_t mine = 0;   // stores this thread has issued
        uint32_t b = me, ph = 0;   // buffer and barrier phase of my next slab
        TCT_DECL
        for (int tile = tile0; tile < p.total_tiles && !err_code; tile += tstep) {
          bool ghost = false;
          const TcTile tl = tc_decode<BN, PAIR>(p, tile, rank, &ghost);
          const int nslab = nslab_of(tl);
          for (int sl = 0; sl < nslab; ++sl, ++d) {
            if (d % TC_NSTORE != me) continue;
            if (!TCT_WAIT(0, mbar_wait(dfull_bar(b), ph, abort_flag))) {
              err_code = 6;
              break;
            }
            if (!ghost)   // the duplicate tile of an odd last pair is computed, not stored
              tma_store_4d(&p.tmD, sD + b * SLAB_BYTES, tl.k0 + sl * DC, tl.q0, tl.p0, tl.n0);
            tma_store_commit();
            // Up to store_pend of my earlier stores may still be reading their buffers; the
            // one before those is done, and its buffer goes to the slab dbuf further on.
            // Every buffer that is not in a store is then filling (residual fetch, epilogue),
            // which is also what hides the residual's memory latency.  (Waiting for each
            // store before the next is issued costs this thread up to a quarter of its time
            // on layers with narrow slabs; several in flight measured 6 % on 16->96 channels
            // and nothing on the wide layers.)
#ifdef OCCAMY_TC_TIMERS
            const long long tw_ = clock64();
#endif
            switch (p.store_pend) {
              case 0: tma_store_wait_read<0>(); break;
              case 1: tma_store_wait_read<1>(); break;
              case 2: tma_store_wait_read<2>(); break;
              default: tma_store_wait_read<3>(); break;
            }
#ifdef OCCAMY_TC_TIMERS
            tct_[1] += clock64() - tw_;
#endif
            if (mine++ >= (uint32_t)p.store_pend) ready_one();
            b += TC_NSTORE;
            if (b >= (uint32_t)dbuf) {
              b -= (uint32_t)dbuf;
              ph ^= 1u;
            }
          }
        }
        tma_store_wait_read<0>();
        if (me == 0) { TCT_FLUSH(4) }
      }
    }
  } else if (SPLIT_LOAD && warp == WLOAD_WARP) {
    // ------------------------------------------------------------ weight loader (see two_loaders)
    if (lane == 0 && two_loaders) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = tile0; tile < p.total_tiles && !err_code; tile += tstep) {
        const TcTile tl = tc_decode<BN, PAIR>(p, tile, rank);
        for (int t = 0; t < p.num_taps && !err_code; ++t) {
          for (int cb = 0; cb < p.cblocks; ++cb) {
            if (pre_b > 0) {
              --pre_b;   // requested before the wait for the previous kernel
            } else {
              if (!mbar_wait_hot(empty_bar(stage), phase ^ 1u, abort_flag)) {
                err_code = 1;
                break;
              }
              mbar_expect_tx(full_bar(stage), b_bytes);
              tma_load_3d(sB + stage * b_bytes, &p.tmB, full_bar(stage), cb * bk, tl.k0, t);
            }
            if (++stage == stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp < STORE_WARP) {
    // ------------------------------------------------------------ epilogue (4 * EW warps)
    const int quad = warp & 3;               // TMEM lane quadrant this warp may read
    const int part = (warp - 2) >> 2;        // which part of a slab's channels
    const int row = quad * 32 + lane;        // accumulator row == pixel index in the tile
    const int et = threadIdx.x - 64;         // 0..EPI_THREADS-1
    // swizzled offsets of this thread's 16-byte pieces inside a slab buffer
    uint32_t soff[CW / 8];
#pragma unroll
    for (int c4 = 0; c4 < CW / 8; ++c4) soff[c4] = slab_off(row, part * (CW / 8) + c4, DC * 2);
    // The whole bias vector goes to shared memory once: a global load per tile would put
    // the memory latency on every tile's critical path.
    for (int i = et; i < p.bias_floats; i += EPI_THREADS)
      bias_s[i] = (p.bias && i < p.K) ? p.bias[i] : 0.0f;
    epi_bar_n<EPI_THREADS>();
    const float act_lo = p.lo, act_hi = p.hi;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t buf = 0, buf_phase = 0;         // slab buffer the next slab goes through

    TCT_DECL
    for (int tile = tile0; tile < p.total_tiles && !err_code; tile += tstep) {
      const TcTile tl = tc_decode<BN, PAIR>(p, tile, rank);
      const int nslab = min(NSLAB, (p.K - tl.k0 + DC - 1) / DC);
      const float *bias_t = bias_s + tl.k0 + part * CW;
      bool f32_ok = false;        // fp32 NCHW output: does this thread's row hold a real pixel,
      int64_t f32_base = 0;       // and where does its channel 0 go
      if constexpr (F32) {
        if (p.out_hw) {
          const int twi = row % p.tw, r2 = row / p.tw;
          const int thi = r2 % p.th, tni = r2 / p.th;
          const int q = tl.q0 + twi, pp = tl.p0 + thi, n = tl.n0 + tni;
          f32_ok = row < rows_valid && q < p.gq && pp < p.gp && n < p.gn;
          const int64_t lin = ((int64_t)n * p.gp + pp) * p.gq + q;   // pixel number in the grid
          const int64_t img = lin / p.out_hw;
          f32_base = img * (int64_t)p.K * p.out_hw + (lin - img * p.out_hw);
        }
      }
      if (!TCT_WAIT(0, mbar_wait(tfull_bar(acc), acc_phase, abort_flag))) {
        err_code = 4;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) +
                             (uint32_t)(acc * ACC_COLS + part * CW);
      // every TMEM read of this tile has landed: the MMA warp may overwrite the buffer
      auto release_acc = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(cluster_map(tempty_bar(acc), 0));
          else mbar_arrive(tempty_bar(acc));
        }
      };
      // one slab: r holds this thread's CW accumulator columns of slab sl
      auto slab = [&](const uint32_t *r, int sl) -> bool {
        uint64_t v2[CW / 2];   // two channels per 64-bit register: packed fp32 adds
        {
          const float4 *b4 = reinterpret_cast<const float4 *>(bias_t + sl * DC);
#pragma unroll
          for (int j = 0; j < CW / 4; ++j) {
            const float4 b = b4[j];
            v2[2 * j] = f2_add(f2_pack(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1])),
                               f2_pack(b.x, b.y));
            v2[2 * j + 1] =
                f2_add(f2_pack(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])),
                       f2_pack(b.z, b.w));
          }
        }
        if constexpr (F32) {
          const int c0 = tl.k0 + sl * DC + part * CW;
          if (p.out_hw) {
            // NCHW: this thread's pixel is (n, pq); channel c lies c * P*Q floats further on
            if (f32_ok) {
              float *o = p.out_f32 + f32_base + (int64_t)c0 * p.out_hw;
#pragma unroll
              for (int j = 0; j < CW / 2; ++j) {
                float a, b;
                f2_unpack(v2[j], a, b);
                if (c0 + 2 * j < p.K) o[(int64_t)(2 * j) * p.out_hw] = tc_act(a, act_lo, act_hi);
                if (c0 + 2 * j + 1 < p.K)
                  o[(int64_t)(2 * j + 1) * p.out_hw] = tc_act(b, act_lo, act_hi);
              }
            }
            return true;
          }
          const int m = tl.q0 + row;
          if (row < rows_valid && m < p.m_total) {
            float *o = p.out_f32 + (int64_t)m * p.ldo + c0;
#pragma unroll
            for (int j = 0; j < CW / 2; ++j) {
              float a, b;
              f2_unpack(v2[j], a, b);
              if (c0 + 2 * j < p.K) o[2 * j] = tc_act(a, act_lo, act_hi);
              if (c0 + 2 * j + 1 < p.K) o[2 * j + 1] = tc_act(b, act_lo, act_hi);
            }
          }
          return true;
        } else {
          // the buffer is free, or (residual) holds the slab to add
          if (!TCT_WAIT(1, mbar_wait(rfull_bar(buf), buf_phase, abort_flag))) return false;
          uint8_t *dptr = base_ptr + (sD - base) + buf * SLAB_BYTES;
          if constexpr (RES) {
#pragma unroll
            for (int c4 = 0; c4 < CW / 8; ++c4) {
              const uint4 rv = *reinterpret_cast<const uint4 *>(dptr + soff[c4]);
              const uint32_t w4[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e)
                v2[c4 * 4 + e] = f2_add(v2[c4 * 4 + e], pair16_to_f2<F16>(w4[e]));
            }
          }
          uint32_t pk[CW / 2];
#pragma unroll
          for (int j = 0; j < CW / 2; ++j) {
            if constexpr (CLAMP) {
              float a, b;
              f2_unpack(v2[j], a, b);
              pk[j] = f2_to_bf16x2<F16>(f2_pack(tc_act(a, act_lo, act_hi), tc_act(b, act_lo, act_hi)));
            } else {
              pk[j] = f2_to_bf16x2_relu<F16>(v2[j]);   // ReLU rides on the conversion
            }
          }
#pragma unroll
          for (int c4 = 0; c4 < CW / 8; ++c4)
            *reinterpret_cast<uint4 *>(dptr + soff[c4]) =
                make_uint4(pk[c4 * 4], pk[c4 * 4 + 1], pk[c4 * 4 + 2], pk[c4 * 4 + 3]);
          // this warp's part of the slab is written: tell the store thread
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(dfull_bar(buf));
          if (++buf == (uint32_t)dbuf) {
            buf = 0;
            buf_phase ^= 1u;
          }
          return true;
        }
      };
      // Slabs in pairs, so that the registers of one slab are loaded while the other is
      // worked on and the loop body (two slabs) stays small.
      uint32_t ra[CW], rb[CW];
      bool ok = true;
      if constexpr (SPLIT) {
        // main and correction accumulators of a slab are read together and added here
#pragma unroll 1
        for (int sl = 0; sl < nslab && ok; ++sl) {
          tc_ld<CW>(t_row + (uint32_t)(sl * DC), ra);
          tc_ld<CW>(t_row + (uint32_t)(BN + sl * DC), rb);
          tc_ld_wait();
          if (sl + 1 == nslab) release_acc();
#pragma unroll
          for (int j = 0; j < CW; ++j)
            ra[j] = __float_as_uint(__uint_as_float(ra[j]) + __uint_as_float(rb[j]));
          ok = slab(ra, sl);
        }
      } else {
      tc_ld<CW>(t_row, ra);
#pragma unroll 1
      for (int sl = 0; sl < nslab && ok; sl += 2) {
        tc_ld_wait();
        if (sl + 1 < nslab) tc_ld<CW>(t_row + (uint32_t)((sl + 1) * DC), rb);
        else release_acc();
        ok = slab(ra, sl);
        if (sl + 1 < nslab && ok) {
          tc_ld_wait();
          if (sl + 2 < nslab) tc_ld<CW>(t_row + (uint32_t)((sl + 2) * DC), ra);
          else release_acc();
          ok = slab(rb, sl + 1);
        }
      }
      }
      if (!ok) {
        err_code = 5;
        break;
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0 && quad == 0) { TCT_FLUSH(2 + part) }
  }

  if (err_code) {
    atomicExch(p.err, 1000 + err_code);
    *abort_flag = 1;
    // let copies that are still in flight land before shared memory is given back
    for (int i = 0; i < 50; ++i) __nanosleep(20000);
  }
  tc_fence_before();
  __syncthreads();
  // neither CTA of a pair leaves (or frees TMEM) while the other may still signal its barriers
  // or have MMAs reading its shared memory
  if constexpr (PAIR) cluster_sync_all();
  if (warp == 2) {
    if constexpr (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(TMEM_COLS)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(TMEM_COLS)
                   : "memory");
  }
}

// Launchers of the instantiations, one translation unit per tile shape.  `mode` is a
// combination of TC_MODE_* the shape is compiled for; false when it is not.
bool tc_launch_256_64(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s);
bool tc_launch_256_32(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s);
bool tc_launch_128_64(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s);
bool tc_launch_64_64(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s);
bool tc_launch_32_32(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s);
bool tc_launch_32_32_duo(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s);
bool tc_launch_64_64_duo(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s);
bool tc_launch_128_64_duo(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s);

// Launch with programmatic stream serialisation (see pdl_wait); `cluster` > 1 launches the
// grid as thread-block clusters of that many CTAs.
template <typename Kernel, typename Params>
inline void tc_launch_pdl(Kernel kernel, int grid, int threads, size_t smem, cudaStream_t s,
                          const Params &p, int cluster = 1) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cluster > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  cudaLaunchKernelEx(&cfg, kernel, p);
}

// A function attribute (the dynamic shared memory limit) belongs to the current device.  Each
// launcher keeps one flag array and asks this helper whether the attribute still has to be set
// on the device the launch goes to.
constexpr int TC_MAX_DEVICES = 64;
inline bool tc_first_use_on_device(unsigned char (&done)[TC_MAX_DEVICES]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= TC_MAX_DEVICES) return true;
  if (done[dev]) return false;
  done[dev] = 1;
  return true;
}

// Body shared by the launchers: picks the instantiation for `mode`, raises its dynamic
// shared memory limit once per device, launches.
template <int BN, int DC, int MODE, int EW = TC_EW>
inline void tc_launch_one(const TcParams &p, int grid, size_t smem, cudaStream_t s) {
  static unsigned char attr_done[TC_MAX_DEVICES] = {};
  if (tc_first_use_on_device(attr_done)) {
    cudaFuncSetAttribute(tc_conv_kernel<BN, DC, EW, MODE>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_LIMIT);
    // all of the SM's configurable memory as shared memory: the kernel reads nothing through
    // L1, and two CTAs of the 113 KB form fit an SM only then
    cudaFuncSetAttribute(tc_conv_kernel<BN, DC, EW, MODE>,
                         cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  }
  // (A launch of the two-per-SM form whose CTAs were not all resident at once would still be
  // safe behind a dependent launch: dependents start only after every CTA of this grid has
  // executed launch_dependents, which comes after its TMEM allocation.)
  tc_launch_pdl(tc_conv_kernel<BN, DC, EW, MODE>, grid, tc_block_threads(EW), smem,
                s, p, (MODE & TC_MODE_PAIR) ? 2 : 1);
}
// The 16-bit flavours of a tile shape with one epilogue warp per TMEM quadrant: a CTA of
// 256 threads, two of which fit an SM.
template <int BN, int DC>
inline bool tc_launch_mode_duo(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s) {
  constexpr int H = TC_MODE_F16, R = TC_MODE_RES, C = TC_MODE_CLAMP;
  switch (mode) {
    case 0: tc_launch_one<BN, DC, 0, 1>(p, grid, smem, s); return true;
    case R: tc_launch_one<BN, DC, R, 1>(p, grid, smem, s); return true;
    case C: tc_launch_one<BN, DC, C, 1>(p, grid, smem, s); return true;
    case R | C: tc_launch_one<BN, DC, R | C, 1>(p, grid, smem, s); return true;
    case H: tc_launch_one<BN, DC, H, 1>(p, grid, smem, s); return true;
    case H | R: tc_launch_one<BN, DC, H | R, 1>(p, grid, smem, s); return true;
    case H | C: tc_launch_one<BN, DC, H | C, 1>(p, grid, smem, s); return true;
    case H | R | C: tc_launch_one<BN, DC, H | R | C, 1>(p, grid, smem, s); return true;
    default: return false;
  }
}
template <int BN, int DC, bool WITH_F32, bool WITH_HALO = false>
inline bool tc_launch_mode(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s) {
  if constexpr (BN == 256) {   // the CTA-pair flavours (bf16 and fp16, plain epilogues)
    constexpr int P2 = TC_MODE_PAIR, H2 = TC_MODE_F16;
    switch (mode) {
      case P2: tc_launch_one<BN, DC, P2>(p, grid, smem, s); return true;
      case P2 | TC_MODE_RES: tc_launch_one<BN, DC, P2 | TC_MODE_RES>(p, grid, smem, s); return true;
      case P2 | TC_MODE_CLAMP: tc_launch_one<BN, DC, P2 | TC_MODE_CLAMP>(p, grid, smem, s); return true;
      case P2 | TC_MODE_RES | TC_MODE_CLAMP:
        tc_launch_one<BN, DC, P2 | TC_MODE_RES | TC_MODE_CLAMP>(p, grid, smem, s);
        return true;
      case P2 | H2: tc_launch_one<BN, DC, P2 | H2>(p, grid, smem, s); return true;
      case P2 | H2 | TC_MODE_RES: tc_launch_one<BN, DC, P2 | H2 | TC_MODE_RES>(p, grid, smem, s); return true;
      case P2 | H2 | TC_MODE_CLAMP: tc_launch_one<BN, DC, P2 | H2 | TC_MODE_CLAMP>(p, grid, smem, s); return true;
      case P2 | H2 | TC_MODE_RES | TC_MODE_CLAMP:
        tc_launch_one<BN, DC, P2 | H2 | TC_MODE_RES | TC_MODE_CLAMP>(p, grid, smem, s);
        return true;
      default: break;
    }
  }
  if constexpr (WITH_F32 && BN <= 128) {
    if (mode == (TC_MODE_SPLIT | TC_MODE_F32 | TC_MODE_CLAMP)) {
      tc_launch_one<BN, DC, TC_MODE_SPLIT | TC_MODE_F32 | TC_MODE_CLAMP>(p, grid, smem, s);
      return true;
    }
  }
  constexpr int H = TC_MODE_F16;
  switch (mode) {   // the fp16 flavours first (no halo form among them)
    case H: tc_launch_one<BN, DC, H>(p, grid, smem, s); return true;
    case H | TC_MODE_RES: tc_launch_one<BN, DC, H | TC_MODE_RES>(p, grid, smem, s); return true;
    case H | TC_MODE_CLAMP: tc_launch_one<BN, DC, H | TC_MODE_CLAMP>(p, grid, smem, s); return true;
    case H | TC_MODE_RES | TC_MODE_CLAMP:
      tc_launch_one<BN, DC, H | TC_MODE_RES | TC_MODE_CLAMP>(p, grid, smem, s);
      return true;
    case H | TC_MODE_F32 | TC_MODE_CLAMP:
      if constexpr (WITH_F32) {
        tc_launch_one<BN, DC, H | TC_MODE_F32 | TC_MODE_CLAMP>(p, grid, smem, s);
        return true;
      }
      return false;
    default: break;
  }
  switch (mode) {
    case 0: tc_launch_one<BN, DC, 0>(p, grid, smem, s); return true;
    case TC_MODE_RES: tc_launch_one<BN, DC, TC_MODE_RES>(p, grid, smem, s); return true;
    case TC_MODE_CLAMP: tc_launch_one<BN, DC, TC_MODE_CLAMP>(p, grid, smem, s); return true;
    case TC_MODE_RES | TC_MODE_CLAMP:
      tc_launch_one<BN, DC, TC_MODE_RES | TC_MODE_CLAMP>(p, grid, smem, s);
      return true;
    case TC_MODE_F32 | TC_MODE_CLAMP:
      if constexpr (WITH_F32) {
        tc_launch_one<BN, DC, TC_MODE_F32 | TC_MODE_CLAMP>(p, grid, smem, s);
        return true;
      }
      return false;
    default: break;
  }
  if constexpr (WITH_HALO) {
    switch (mode) {
      case TC_MODE_HALO: tc_launch_one<BN, DC, TC_MODE_HALO>(p, grid, smem, s); return true;
      case TC_MODE_HALO | TC_MODE_RES:
        tc_launch_one<BN, DC, TC_MODE_HALO | TC_MODE_RES>(p, grid, smem, s);
        return true;
      case TC_MODE_HALO | TC_MODE_CLAMP:
        tc_launch_one<BN, DC, TC_MODE_HALO | TC_MODE_CLAMP>(p, grid, smem, s);
        return true;
      case TC_MODE_HALO | TC_MODE_RES | TC_MODE_CLAMP:
        tc_launch_one<BN, DC, TC_MODE_HALO | TC_MODE_RES | TC_MODE_CLAMP>(p, grid, smem, s);
        return true;
      default: break;
    }
  }
  return false;
}

}  // namespace occ
