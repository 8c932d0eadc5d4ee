// Shared device-side building blocks of the sm_100a decode path: PTX wrappers (mbarrier, 1-D bulk copies,
// coherent loads), bounded waits that report instead of hanging, the tiled streaming weight layout and the int4 tile x
// vector product (fp16 mma.sync) that every GEMV phase uses.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fb {

// ------------------------------------------------------------------------------------------------ constants
#ifndef FB_ACC2
#define FB_ACC2 0     // 1: two accumulator sets in the unrolled tile product; measured no faster
#endif
#ifndef FB_CW
#define FB_CW 14      // 14 consumers + 1 producer = 15 warps -> at most 4 per scheduler -> 128 registers per thread
#endif
constexpr int kConsumerWarps = FB_CW;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;    // + one producer warp (lane 0 issues the bulk copies)
constexpr int kStages = 8;                         // ring depth: 8 x 22.5 KB = 180 KB of weights in flight per SM
constexpr int kStageBytes = 23040;                 // a stage holds whole tiles (4 tiles of K = 2560, 1 of K = 8192 ...)
constexpr int kScratchBytes = 40960;               // activations of the phase (<= 14336 fp16), then attention scratch
constexpr int kTailBytes = 6144;                   // mbarriers, flags, reductions, slice partials, owned rows, group factors
constexpr int kSmemBytes = kStages * kStageBytes + kScratchBytes + kTailBytes;
constexpr int kMaxOwnRows = 64;                    // rows of the residual stream one CTA may own
constexpr int kMaxGroups = 112;                    // K <= 14336

// named barriers (0 is __syncthreads)
constexpr int kBarConsumers = 1;                   // all consumer threads

// device status words (global memory, owned by the context)
struct DevStatus {
  int code;        // 0 ok, else FB_ERR_TIMEOUT
  int where;       // phase id of the wait that gave up
  int layer, block, expected, seen;
  int abort;       // set with the first failure; every other wait polls it and leaves
  int pad;
};

enum Where { W_FULL = 2, W_EMPTY = 3, W_FLAG = 5, W_LANDED = 6 };

// ------------------------------------------------------------------------------------------------ small helpers
__device__ __forceinline__ float bf2f(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
__device__ __forceinline__ float bflo(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float bfhi(uint32_t p) { return __uint_as_float(p & 0xffff0000u); }
__device__ __forceinline__ uint16_t f2bf(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
__device__ __forceinline__ float rbf(float f) { return bf2f(f2bf(f)); }   // round an fp32 value to bf16 precision

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// loads that must see data written by other SMs during this launch: L2 is the point of coherence
__device__ __forceinline__ uint32_t ld_cg_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint16_t ld_cg_u16(const void* p) {
  uint16_t v;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_volatile_s32(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ------------------------------------------------------------------------------------------------ mbarrier + bulk copy
__device__ __forceinline__ void mbar_init(uint64_t* b, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
  return ok != 0;
}
// global -> this CTA's shared memory, size and both addresses multiples of 16; completion counted on `bar`
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// ------------------------------------------------------------------------------------------------ bounded waits
// Every wait in this library has an iteration limit. When it runs out the waiter records where it gave up and
// raises the abort word; every other waiter polls that word and leaves too, so the launch always ends.
struct WaitCtl {
  DevStatus* st;        // global
  volatile int* s_abort;  // shared: this CTA saw a failure
  unsigned limit;       // spin limit per wait
};

__device__ __forceinline__ void report_fail(const WaitCtl& c, int where, int layer, int expected, int seen) {
  if (atomicCAS(&c.st->code, 0, 5 /*FB_ERR_TIMEOUT*/) == 0) {
    c.st->where = where; c.st->layer = layer; c.st->block = (int)blockIdx.x; c.st->expected = expected; c.st->seen = seen;
  }
  atomicExch(&c.st->abort, 1);
  *c.s_abort = 1;
  __threadfence();
}

__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, const WaitCtl& c, int where, int layer) {
  if (mbar_try(b, parity)) return true;
  for (unsigned i = 0; i < c.limit; i++) {
    if (mbar_try(b, parity)) return true;
    if ((i & 63) == 63) {
      if (*c.s_abort) return false;
      if ((i & 1023) == 1023) {
        if (ld_volatile_s32(&c.st->abort)) { *c.s_abort = 1; return false; }
        __nanosleep(64);
      }
    }
  }
  report_fail(c, where, layer, (int)parity, -1);
  return false;
}

// ------------------------------------------------------------------------------------------------ streaming layout
// Weights are stored as TILES of RT consecutive stream rows x all K columns, laid out for the tensor pipe: a tile is
// a sequence of "steps", 128 bytes each = one 32-bit word per lane of a warp, and a step is exactly the A operand of one
// mma.m16n8k16. Batch-1 decode has no second matrix dimension to fill the 16 MMA rows with, so the 16 rows of a step
// are RT weight rows x NJ = 16/RT column ranges of K/NJ columns each: MMA row i = (tile row i % RT, range i / RT), and
// column n of the B operand carries the activations of range n. Output C[i][i / RT] is then the partial dot product
// of tile row i % RT over range i / RT; the other columns are ignored.
//
// Inside a word the eight nibbles are placed so that no arithmetic is needed to turn them into fp16 operands:
//   w & 0x000F000F        -> (nib0, nib4) as fp16 SUBNORMALS nib * 2^-24   = A[g  ][2t], A[g  ][2t+1]
//   w & 0x00F000F0        -> (nib1, nib5) as 16 * nib * 2^-24              = A[g+8][2t], A[g+8][2t+1]
//   (w >> 8) & the same   -> (nib2, nib6), (nib3, nib7)                    = A[g][2t+8..], A[g+8][2t+8..]
// for lane (g = lane / 4, t = lane % 4). The tensor pipe multiplies subnormals exactly, so C = 2^-24 * sum nib * x for
// the first eight MMA rows and 16 times that for the last eight; the per-group flush folds 2^24 (or 2^20), the group's
// bf16 scale and the activations' power-of-two factor into one fp32 multiply, and removes the nibble offset with
// -8 * scale * sum(x) (and adds zero * sum(x) for the asymmetric layout). Products and the subtraction are exact in
// fp32 terms: the arithmetic is the reference's sum (nib - 8) * s * x with a different summation order.
//
// Steps are stored four to a block: block bq holds, for every lane, the words of steps 4bq..4bq+3 as one 16-byte
// vector. Range j walks its columns with its steps rotated inside each block (local step (s & ~3) | ((s + j) & 3)),
// which spreads the ranges' activation loads over different shared-memory banks. After the nibble area come the
// tile's scales as bf16 [K/128][RT], then (asymmetric layout) the zeros in the same shape.
__host__ __device__ constexpr int tile_rt(int k) {
  const int g = k / 128;
  if (g % 4 == 0 && 4 * (k / 2 + g * 4) <= 23040) return 4;
  if (g % 8 == 0) return 2;
  if (g % 2 == 0) return 8;
  return 16;
}
__host__ __device__ constexpr int tile_bytes(int k, int has_zeros) {
  return tile_rt(k) * (k / 2 + (k / 128) * 2 * (has_zeros ? 2 : 1));
}
// bytes per stream row (a tile is RT of these; only whole tiles are addressable)
__host__ __device__ constexpr int rec_bytes_of(int k, int has_zeros) { return tile_bytes(k, has_zeros) / tile_rt(k); }
__host__ __device__ constexpr int pad_rows(int rows, int k) { return (rows + tile_rt(k) - 1) / tile_rt(k) * tile_rt(k); }
__host__ __device__ __forceinline__ int local_step(int s, int j) { return (s & ~3) | ((s + j) & 3); }

// stream row j of a matrix holds source row perm(j)
//   order 0: identity
//   order 1: rows [0, order_rows) are heads of `arg` rows; inside a head stream rows (2p, 2p+1) hold dims (p, p+arg/2),
//            so one thread gets both halves of a RoPE pair; rows beyond order_rows (V) keep their order
//   order 2: stream rows (2i, 2i+1) hold (gate_i, up_i) = source rows (i, i+arg)
__host__ __device__ __forceinline__ int perm_row(int j, int order, int arg, int order_rows) {
  if (order == 1) {
    if (j >= order_rows) return j;
    const int head = j / arg, w = j % arg;
    return head * arg + (w >> 1) + (w & 1) * (arg >> 1);
  }
  if (order == 2) return (j >> 1) + (j & 1) * arg;
  return j;
}

// Compile-time schedule of one matrix shape. KS > 1 cuts a tile's blocks into KS slices that different warps take
// (phases that give a CTA only a handful of tiles); TPS tiles travel in one bulk copy / ring stage.
template <int K_, int KS_ = 1, int TPS_ = 0>
struct TCfg {
  static constexpr int K = K_, KS = KS_, RT = tile_rt(K_);
  static constexpr int NJ = 16 / RT, G = K / 128, RG = G / NJ, BQ = RG * 2;     // rounds (8 steps) per range; 4-step blocks
  static constexpr int NB = BQ / KS;                                             // blocks per slice
  static constexpr int NIB = RT * K / 2;
  static constexpr int tile(bool hz) { return tile_bytes(K_, hz); }
  static constexpr int TPS_FIT = kStageBytes / tile_bytes(K_, 1);
  static constexpr int TPS = TPS_ > 0 ? TPS_ : (KS_ > 1 ? (TPS_FIT > 2 ? 2 : TPS_FIT) : (TPS_FIT > 8 ? 8 : TPS_FIT));
  static constexpr int TILE_ROWS = TPS * RT;                                      // rows per ring stage
  static_assert(K % 128 == 0 && G % NJ == 0 && BQ % KS == 0, "columns must split into whole groups per range and slice");
  static_assert(TPS >= 1 && TPS * tile_bytes(K_, 1) <= kStageBytes, "a stage holds whole tiles");
  static_assert(KS == 1 || (RT <= 4 && TPS <= 2 && KS <= 4), "slice partials: 4 rows x 4 slices x 2 tiles per stage");
  static_assert(tile_bytes(K_, 0) % 16 == 0 && tile_bytes(K_, 1) % 16 == 0, "bulk copies move multiples of 16 bytes");
};

// activations of the current phase in shared memory: fp16 in B-operand order (inside every 16 columns the halves are
// [2t, 2t+1, 2t+8, 2t+9] for t = 0..3) and, per group of 128 columns, {2^24 / m, 2^20 / m, -8 * sum x, sum x} where m is
// the power of two the group was multiplied by before the conversion to fp16
struct XStage {
  const __half* xh;
  const float4* xf;
};

// Convert 4 consecutive bf16 activations (elements 4*lane .. 4*lane+3 of one group of 128, one group per warp) and
// store them; lane 0 also writes the group's factors. The whole warp must call this together.
__device__ __forceinline__ void stage_group_fp16(uint32_t p01, uint32_t p23, __half* xh_group, float4* xf_group, int lane) {
  const uint32_t e0 = (p01 >> 7) & 255, e1 = (p01 >> 23) & 255, e2 = (p23 >> 7) & 255, e3 = (p23 >> 23) & 255;
  const uint32_t em = __reduce_max_sync(0xffffffffu, max(max(e0, e1), max(e2, e3)));
  uint32_t mf = 268u - em;                    // exponent field of m: the group's largest magnitude lands in [2^14, 2^15)
  mf = mf > 253u ? 253u : (mf < 24u ? 24u : mf);
  const float mult = __uint_as_float(mf << 23), inv = __uint_as_float((254u - mf) << 23);
  const float f0 = bflo(p01), f1 = bfhi(p01), f2 = bflo(p23), f3 = bfhi(p23);
  const __half2 h01 = __floats2half2_rn(f0 * mult, f1 * mult), h23 = __floats2half2_rn(f2 * mult, f3 * mult);
  float sx = (f0 + f1) + (f2 + f3);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sx += __shfl_xor_sync(0xffffffffu, sx, o);
  // element c = 4 * (lane % 4) + e of its 16-block: the pair (c, c+1) goes to half2 slot 2 * ((c % 8) / 2) + c / 8
  const int c = (lane & 3) * 4;
  __half2* dst = reinterpret_cast<__half2*>(xh_group + (lane >> 2) * 16);
  __syncwarp();                               // in-place use: every lane has read its source words
  dst[((c % 8) / 2) * 2 + (c / 8)] = h01;
  dst[(((c + 2) % 8) / 2) * 2 + ((c + 2) / 8)] = h23;
  if (lane == 0) *xf_group = make_float4(inv * 16777216.f, inv * 1048576.f, -8.f * sx, sx);
}

// ------------------------------------------------------------------------------------------------ tile x vector
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ float lds_bf16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return __uint_as_float(((uint32_t)v) << 16);
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_first(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// Programmatic dependent launch: every kernel of the verify chain is launched with the stream-serialisation attribute.
// pdl_trigger() lets the next kernel's CTAs start (and prefetch what does not depend on this kernel) once every CTA of
// this kernel has called it; pdl_wait() returns when the previous kernel has completed and its writes are visible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// launch with programmatic stream serialisation: the kernel may start while its predecessor drains (see pdl_wait)
template <class... KArgs, class... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// bf16 tensor-core helpers shared by the verify attention and the long-cache decode attention
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16_first(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) { return (uint32_t)f2bf(lo) | ((uint32_t)f2bf(hi) << 16); }

// Fully unrolled form of the tile product (same contract as tile_dot_rolled below): every block's flags and offsets
// are compile-time constants. Fastest per tile (5.3 TB/s on the stand-alone GEMV against 4.7 for the rolled form), but
// ~10 KB of straight-line code per call site.
template <class C, bool HZ>
__device__ __forceinline__ void tile_dot_unrolled(const uint8_t* tile, int slice, const XStage& x, int lane, float& out_lo,
                                         float& out_hi) {
  constexpr int RT = C::RT, NB = C::NB;
  const int g = lane >> 2, t = lane & 3;
  const int jl = g / RT, jh = (g + 8) / RT, jb = g % C::NJ;
  const int rl = g % RT, rh = (g + 8) % RT;
  const int b0 = C::KS == 1 ? 0 : slice * NB;
  const uint32_t tb = smem_u32(tile);
  const uint32_t wa = tb + (uint32_t)(b0 * 32 + lane) * 16;
  const uint32_t xbase = smem_u32(x.xh) + (uint32_t)(jb * (C::K / C::NJ) + 4 * t) * 2 + (uint32_t)b0 * 128;
  uint32_t xa[4];
#pragma unroll
  for (int i = 0; i < 4; i++) xa[i] = xbase + 32 * ((i + jb) & 3);
  const uint32_t ml = tb + C::NIB + (uint32_t)(jl * C::RG * RT + rl) * 2;
  const uint32_t mh = tb + C::NIB + (uint32_t)(jh * C::RG * RT + rh) * 2;
  const uint32_t fl = smem_u32(x.xf) + (uint32_t)(jl * C::RG) * 16, fh = smem_u32(x.xf) + (uint32_t)(jh * C::RG) * 16;
  float ct[4] = {0.f, 0.f, 0.f, 0.f}, cg[4], ch[4];
  float zl = 0.f, zh = 0.f;
  uint4 w4 = lds128(wa);
  uint2 xb[4];
#pragma unroll
  for (int i = 0; i < 4; i++) xb[i] = lds64(xa[i]);
  const bool odd0 = (NB % 2 == 0) ? false : (b0 & 1);           // the slice starts in the middle of a round
#ifdef FB_DOT_UNROLL2
#pragma unroll 2
#else
#pragma unroll
#endif
  for (int bi = 0; bi < NB; bi++) {
    uint4 wn;
    uint2 xn[4];
    if (bi + 1 < NB) {                                           // next block's operands are in flight during this one
      wn = lds128(wa + (bi + 1) * 512);
#pragma unroll
      for (int i = 0; i < 4; i++) xn[i] = lds64(xa[i] + (bi + 1) * 128);
    }
    const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
    const bool first = (bi == 0) || (((bi & 1) != 0) == odd0);   // block b0 + bi opens a round
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t w2 = ws[i] >> 8;
      const uint32_t a[4] = {ws[i] & 0x000F000Fu, ws[i] & 0x00F000F0u, w2 & 0x000F000Fu, w2 & 0x00F000F0u};
      if (FB_ACC2 && (i & 1)) {
        if (first && i == 1) mma_f16_first(ch, a, xb[i].x, xb[i].y);
        else mma_f16(ch, a, xb[i].x, xb[i].y);
      } else {
        if (first && i == 0) mma_f16_first(cg, a, xb[i].x, xb[i].y);
        else mma_f16(cg, a, xb[i].x, xb[i].y);
      }
    }
    const bool closes = (((bi & 1) != 0) != odd0);               // block b0 + bi closes a round
    if (closes || bi == NB - 1) {
      const uint32_t ro = (NB % 2 == 0) ? (uint32_t)(b0 >> 1) + (bi >> 1) : (uint32_t)((b0 + bi) >> 1);
      const float4 Fl = lds128f(fl + ro * 16), Fh = lds128f(fh + ro * 16);
      const float sl = lds_bf16(ml + ro * RT * 2), sh = lds_bf16(mh + ro * RT * 2);
      const float sl2 = sl * Fl.x, sh2 = sh * Fh.y;
      if (FB_ACC2) { cg[0] += ch[0]; cg[1] += ch[1]; cg[2] += ch[2]; cg[3] += ch[3]; }
      ct[0] = fmaf(sl2, cg[0], ct[0]); ct[1] = fmaf(sl2, cg[1], ct[1]);
      ct[2] = fmaf(sh2, cg[2], ct[2]); ct[3] = fmaf(sh2, cg[3], ct[3]);
      if (closes) {                                              // once per (row, group): offset and zero point
        zl = fmaf(sl, Fl.z, zl);
        zh = fmaf(sh, Fh.z, zh);
        if (HZ) {
          zl = fmaf(lds_bf16(ml + C::G * RT * 2 + ro * RT * 2), Fl.w, zl);
          zh = fmaf(lds_bf16(mh + C::G * RT * 2 + ro * RT * 2), Fh.w, zh);
        }
      }
    }
    if (bi + 1 < NB) {
      w4 = wn;
#pragma unroll
      for (int i = 0; i < 4; i++) xb[i] = xn[i];
    }
  }
  // valid outputs: MMA row g -> column jl, MMA row g + 8 -> column jh
  const float vl = (jl == 2 * t) ? ct[0] + zl : ((jl == 2 * t + 1) ? ct[1] + zl : 0.f);
  const float vh = (jh == 2 * t) ? ct[2] + zh : ((jh == 2 * t + 1) ? ct[3] + zh : 0.f);
  if (RT <= 8) {
    float v = vl + vh;
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
#pragma unroll
    for (int o = 4 * RT; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    out_lo = v;
    out_hi = 0.f;
  } else {
    out_lo = vl;
    out_hi = vh;
  }
}

// One slice (NB blocks) of one tile against the staged activations. RT <= 8: on return every lane with lane / 4 % RT == r
// holds the slice's total of tile row r in out_lo. RT == 16: lane 4g holds row g in out_lo and row g + 8 in out_hi.
// The block loop is ROLLED over rounds (two rounds = four blocks of four MMA steps and two group flushes per iteration): the
// product of a tile is ~4 KB of code that every block of every tile reuses, instead of NB fully unrolled blocks (~10 KB per call
// site, executed once per tile) streaming through the instruction cache.
template <class C, bool HZ>
__device__ __forceinline__ void tile_dot_rolled(const uint8_t* tile, int slice, const XStage& x, int lane, float& out_lo,
                                         float& out_hi) {
  constexpr int RT = C::RT, NB = C::NB;
  const int g = lane >> 2, t = lane & 3;
  const int jl = g / RT, jh = (g + 8) / RT, jb = g % C::NJ;
  const int rl = g % RT, rh = (g + 8) % RT;
  const int b0 = C::KS == 1 ? 0 : slice * NB;
  const uint32_t tb = smem_u32(tile);
  uint32_t wa = tb + (uint32_t)(b0 * 32 + lane) * 16;
  const uint32_t xbase = smem_u32(x.xh) + (uint32_t)(jb * (C::K / C::NJ) + 4 * t) * 2 + (uint32_t)b0 * 128;
  uint32_t xa[4];
#pragma unroll
  for (int i = 0; i < 4; i++) xa[i] = xbase + 32 * ((i + jb) & 3);
  uint32_t ml = tb + C::NIB + (uint32_t)(jl * C::RG * RT + rl) * 2;
  uint32_t mh = tb + C::NIB + (uint32_t)(jh * C::RG * RT + rh) * 2;
  uint32_t fl = smem_u32(x.xf) + (uint32_t)(jl * C::RG) * 16, fh = smem_u32(x.xf) + (uint32_t)(jh * C::RG) * 16;
  float ct[4] = {0.f, 0.f, 0.f, 0.f}, cg[4];
  float zl = 0.f, zh = 0.f;
  const bool odd0 = (NB % 2 == 0) ? false : (b0 & 1);           // the slice starts in the middle of a round
  {                                                              // first round of the slice
    const uint32_t ro0 = (uint32_t)(b0 >> 1);
    ml += ro0 * RT * 2; mh += ro0 * RT * 2; fl += ro0 * 16; fh += ro0 * 16;
  }
  uint4 w4 = lds128(wa);
  uint2 xb[4];
#pragma unroll
  for (int i = 0; i < 4; i++) xb[i] = lds64(xa[i]);
  // one block: four MMA steps; the next block's operands are requested before this block's MMAs
  auto block = [&](bool first, bool more) {
    uint4 wn = w4;
    uint2 xn[4];
#pragma unroll
    for (int i = 0; i < 4; i++) xn[i] = xb[i];
    if (more) {
      wn = lds128(wa + 512);
#pragma unroll
      for (int i = 0; i < 4; i++) xn[i] = lds64(xa[i] + 128);
    }
    const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t w2 = ws[i] >> 8;
      const uint32_t a[4] = {ws[i] & 0x000F000Fu, ws[i] & 0x00F000F0u, w2 & 0x000F000Fu, w2 & 0x00F000F0u};
      if (first && i == 0) mma_f16_first(cg, a, xb[i].x, xb[i].y);
      else mma_f16(cg, a, xb[i].x, xb[i].y);
    }
    wa += 512;
#pragma unroll
    for (int i = 0; i < 4; i++) xa[i] += 128;
    w4 = wn;
#pragma unroll
    for (int i = 0; i < 4; i++) xb[i] = xn[i];
  };
  // the group's flush; `whole`: this slice closes the round (offset and zero point once per (row, group))
  auto flush = [&](bool whole) {
    const float4 Fl = lds128f(fl), Fh = lds128f(fh);
    const float sl = lds_bf16(ml), sh = lds_bf16(mh);
    const float sl2 = sl * Fl.x, sh2 = sh * Fh.y;
    ct[0] = fmaf(sl2, cg[0], ct[0]); ct[1] = fmaf(sl2, cg[1], ct[1]);
    ct[2] = fmaf(sh2, cg[2], ct[2]); ct[3] = fmaf(sh2, cg[3], ct[3]);
    if (whole) {
      zl = fmaf(sl, Fl.z, zl);
      zh = fmaf(sh, Fh.z, zh);
      if (HZ) {
        zl = fmaf(lds_bf16(ml + C::G * RT * 2), Fl.w, zl);
        zh = fmaf(lds_bf16(mh + C::G * RT * 2), Fh.w, zh);
      }
    }
    ml += RT * 2; mh += RT * 2; fl += 16; fh += 16;
  };
  int left = NB;                                                 // blocks still to do
  if (odd0) {                                                    // second half of a round another slice opened
    block(true, left > 1);
    flush(true);
    left--;
  }
#pragma unroll 1
  for (; left >= 4; left -= 4) {                                 // two rounds per iteration (+1.8 % tokens/s over one)
    block(true, true);
    block(false, true);
    flush(true);
    block(true, true);
    block(false, left > 4);
    flush(true);
  }
#pragma unroll 1
  for (; left >= 2; left -= 2) {
    block(true, true);
    block(false, left > 2);
    flush(true);
  }
  if (left) {                                                    // first half of a round the next slice closes
    block(true, false);
    flush(false);
  }
  // valid outputs: MMA row g -> column jl, MMA row g + 8 -> column jh
  const float vl = (jl == 2 * t) ? ct[0] + zl : ((jl == 2 * t + 1) ? ct[1] + zl : 0.f);
  const float vh = (jh == 2 * t) ? ct[2] + zh : ((jh == 2 * t + 1) ? ct[3] + zh : 0.f);
  if (RT <= 8) {
    float v = vl + vh;
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
#pragma unroll
    for (int o = 4 * RT; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    out_lo = v;
    out_hi = 0.f;
  } else {
    out_lo = vl;
    out_hi = vh;
  }
}

// ROLL selects the form. The decode megakernel runs the rolled one in every phase: its per-layer code does not fit the
// instruction cache, and with ~10 KB of straight-line code per phase less to fetch the whole layer got faster (QKV
// 2.14 -> 1.81 µs, O 2.21 -> 1.85 µs, attention 4.4 -> 4.0 µs, gate/up 4.42 -> 4.77 µs; 862 -> 897 tok/s; rolling only the
// small phases gave nothing back: 868 tok/s). The stand-alone GEMV, a small kernel, keeps the unrolled form.
template <class C, bool HZ, bool ROLL = false>
__device__ __forceinline__ void tile_dot(const uint8_t* tile, int slice, const XStage& x, int lane, float& out_lo,
                                         float& out_hi) {
  if constexpr (ROLL) tile_dot_rolled<C, HZ>(tile, slice, x, lane, out_lo, out_hi);
  else tile_dot_unrolled<C, HZ>(tile, slice, x, lane, out_lo, out_hi);
}

}  // namespace fb
