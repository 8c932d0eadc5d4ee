// Shared device-side building blocks of the sm_100a decode path: PTX wrappers (mbarrier, 1-D bulk copies,
// coherent loads), bounded waits that report instead of hanging, the streaming weight layout and the int4 row
// dot product that every GEMV phase uses.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fb {

// ------------------------------------------------------------------------------------------------ constants
#ifndef FB_CW
#define FB_CW 14      // 14 consumers + 1 producer = 15 warps -> at most 4 per scheduler -> 128 registers per thread; 14 also
#endif                // divides the 28 four-row blocks a CTA gets of the gate/up matrix (3B-class) into exactly 2 rounds
#ifndef FB_DOT
#define FB_DOT 0      // 0: bf16 pairs + fma.rn.f32.bf16 (activations packed bf16 in registers)
#endif                // 1: prmt -> fp32 weights + fma.rn.f32 (activations fp32 in registers)
constexpr int kConsumerWarps = FB_CW;              // groups of 4 warps; group g consumes weight tiles t with t % kGroups == g
constexpr int kWarpsPerGroup = 4;
constexpr int kGroups = kConsumerWarps / kWarpsPerGroup;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;    // + one producer warp (lane 0 issues the bulk copies)
constexpr int kStages = 8;                         // ring depth: 8 x 22 KB = 176 KB of weights in flight per SM
constexpr int kStageBytes = 23040;              // largest tile: 3 rows of K=14336 with zeros = 22848 B
constexpr int kScratchBytes = 40960;               // x staging (<= 14336 bf16) + per-phase results; attention merge area
constexpr int kXBytes = 28672;
constexpr int kResFloats = (kScratchBytes - kXBytes) / 4;   // 3072 row results per CTA per phase
constexpr int kTailBytes = 4096;                   // mbarriers, flags, reduction scratch, slice partials, owned residual rows
constexpr int kSmemBytes = kStages * kStageBytes + kScratchBytes + kTailBytes;
constexpr int kMaxOwnRows = 64;                    // rows of the residual stream one CTA may own

// named barriers (0 is __syncthreads)
constexpr int kBarConsumers = 1;                   // all 512 consumer threads
constexpr int kBarGroup0 = 2;                      // 2..5: one per consumer group (128 threads)

// device status words (global memory, owned by the context)
struct DevStatus {
  int code;        // 0 ok, else FB_ERR_TIMEOUT
  int where;       // phase id of the wait that gave up
  int layer, block, expected, seen;
  int abort;       // set with the first failure; every other wait polls it and leaves
  int pad;
};

enum Where { W_GRIDBAR = 1, W_FULL = 2, W_EMPTY = 3, W_DRAIN = 4, W_FLAG = 5 };

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
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
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
__device__ __forceinline__ float ld_cg_f32(const void* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const unsigned* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
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
// One record per weight row: K/2 bytes of nibble words in the caller's word order, then K/128 bf16 scales,
// then (asymmetric layout only) K/128 bf16 zeros, padded to 16 bytes. Records are contiguous, so any run of rows is
// one aligned byte range that a single 1-D bulk copy can bring in together with its scales.
__host__ __device__ __forceinline__ int rec_bytes_of(int k, int has_zeros) {
  const int meta = (k / 128) * 2 * (has_zeros ? 2 : 1);
  return k / 2 + ((meta + 15) & ~15);
}
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

// Per-K compile-time schedule. A consumer group (4 warps) owns one tile at a time; inside it warp wg takes the
// K-slice wg % KS of the row blocks wg / KS, wg / KS + 4/KS, ... (RB rows per block). A lane owns units
// u = lane + 32*i (i < NI) of U consecutive words inside its slice and keeps the matching activations in registers
// for the whole phase.
template <int K_, int KS_, int U_, int NI_, int RB_, int TILE_ROWS_>
struct KCfg {
  static constexpr int K = K_, KS = KS_, U = U_, NI = NI_, RB = RB_, TILE_ROWS = TILE_ROWS_;
  static constexpr int SLICE_WORDS = K / 8 / KS;
  static constexpr int UNITS = SLICE_WORDS / U;           // units per slice
  static constexpr bool PRED = (UNITS != 32 * NI);         // last i is partially filled
  static constexpr int NSUB = kWarpsPerGroup / KS;         // row sub-groups per consumer group
  static_assert(K % 128 == 0 && SLICE_WORDS % U == 0 && UNITS <= 32 * NI && UNITS > 32 * (NI - 1), "bad KCfg");
  static_assert(kWarpsPerGroup % KS == 0, "KS must divide the group");
  static_assert((SLICE_WORDS * 8) % 128 == 0 || KS == 1, "slices must hold whole groups");
  static_assert((U * 8) <= 128 && 128 % (U * 8) == 0, "a unit stays inside one group");
};
using K512 = KCfg<512, 1, 2, 1, 4, 64>;
using K1408 = KCfg<1408, 1, 2, 3, 4, 28>;
using K2560 = KCfg<2560, 1, 2, 5, 4, 16>;
using K4096 = KCfg<4096, 2, 4, 2, 4, 8>;
using K8192 = KCfg<8192, 4, 4, 2, 4, 4>;
using K14336 = KCfg<14336, 4, 4, 4, 2, 2>;   // even blocks: epilogues pair rows (2i, 2i+1)
// Same K, finer work units for phases that give a CTA only ~20 rows (QKV, O, down): blocks of 2 rows and small
// tiles keep all consumer warps busy and shorten the tail that the next phase has to wait for.
using K512S = KCfg<512, 1, 2, 1, 2, 16>;
using K1408S = KCfg<1408, 1, 2, 3, 2, 8>;
using K2560S = KCfg<2560, 1, 2, 5, 2, 8>;
using K4096S = KCfg<4096, 2, 4, 2, 2, 4>;
using K8192S = KCfg<8192, 4, 4, 2, 2, 2>;
// K values that only appear under tensor parallelism (a rank's slice of the attention output or of the FFN)
using K640 = KCfg<640, 1, 2, 2, 2, 16>;
using K1024 = KCfg<1024, 1, 4, 1, 2, 16>;
using K1280 = KCfg<1280, 1, 2, 3, 2, 8>;
using K1792 = KCfg<1792, 1, 4, 2, 2, 8>;
using K2048 = KCfg<2048, 1, 4, 2, 2, 8>;
using K3584 = KCfg<3584, 2, 4, 2, 2, 4>;
using K7168 = KCfg<7168, 4, 4, 2, 2, 2>;
template <class KC> struct SmallOf { using type = KC; };
template <> struct SmallOf<K512> { using type = K512S; };
template <> struct SmallOf<K1408> { using type = K1408S; };
template <> struct SmallOf<K2560> { using type = K2560S; };
template <> struct SmallOf<K4096> { using type = K4096S; };
template <> struct SmallOf<K8192> { using type = K8192S; };

// activations of one lane for its units + the fp32 sum of every unit (for the offset trick below)
template <class KC>
struct XRegs {
#if FB_DOT == 0
  uint32_t p[KC::NI][KC::U * 4];     // packed bf16 pairs
#else
  float p[KC::NI][KC::U * 8];        // fp32
#endif
  float sum[KC::NI];
};

// Load a lane's slice from the staged activations x_s (bf16[K] in shared memory).
template <class KC>
__device__ __forceinline__ void load_x_slice(const uint16_t* x_s, int slice, int lane, XRegs<KC>& x) {
#pragma unroll
  for (int i = 0; i < KC::NI; i++) {
    const int unit = lane + 32 * i;
    const bool ok = !KC::PRED || unit < KC::UNITS;
    const uint4* src = reinterpret_cast<const uint4*>(x_s + (size_t)(slice * KC::SLICE_WORDS + unit * KC::U) * 8);
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < KC::U; w++) {
      uint4 v = ok ? src[w] : make_uint4(0, 0, 0, 0);
#if FB_DOT == 0
      x.p[i][4 * w + 0] = v.x; x.p[i][4 * w + 1] = v.y; x.p[i][4 * w + 2] = v.z; x.p[i][4 * w + 3] = v.w;
#else
      x.p[i][8 * w + 0] = bflo(v.x); x.p[i][8 * w + 1] = bfhi(v.x); x.p[i][8 * w + 2] = bflo(v.y); x.p[i][8 * w + 3] = bfhi(v.y);
      x.p[i][8 * w + 4] = bflo(v.z); x.p[i][8 * w + 5] = bfhi(v.z); x.p[i][8 * w + 6] = bflo(v.w); x.p[i][8 * w + 7] = bfhi(v.w);
#endif
      s += bflo(v.x); s += bfhi(v.x); s += bflo(v.y); s += bfhi(v.y);
      s += bflo(v.z); s += bfhi(v.z); s += bflo(v.w); s += bfhi(v.w);
    }
    x.sum[i] = s;
  }
}

#if FB_DOT == 0
// One packed word (8 nibbles) against 8 activations: acc += sum_k (1 + nib_k/16) * x_k, exact products, fp32 adds.
// ((w >> (4j-3)) & 0x00780078) | 0x3F803F80 is the bf16 pair (1 + nib_j/16, 1 + nib_{j+4}/16): the nibble sits in the
// top four mantissa bits. fma.rn.f32.bf16 multiplies two bf16 scalars into an fp32 accumulator in one instruction.
// The caller removes the offset: sum_k (nib_k - 8) x_k = 16 * (acc - 1.5 * sum_k x_k). (Putting the nibble in the LOW
// mantissa bits saves one shift but makes the offset 136 instead of 1.5, and the cancellation then costs ~7 bits of
// the fp32 sum: enough to flip bf16 roundings downstream.)
constexpr float kDotOffset = 1.5f;
constexpr float kDotScale = 16.f;
__device__ __forceinline__ void dot_word(uint32_t w, const uint32_t* x, float& a0, float& a1) {
  const uint32_t M = 0x00780078u, C = 0x3F803F80u;
  const uint32_t t0 = ((w << 3) & M) | C, t1 = ((w >> 1) & M) | C, t2 = ((w >> 5) & M) | C, t3 = ((w >> 9) & M) | C;
  asm("{ .reg .b16 tl, th, xl, xh, yl, yh;\n"
      "mov.b32 {tl,th}, %2; mov.b32 {xl,xh}, %6; mov.b32 {yl,yh}, %8;\n"
      "fma.rn.f32.bf16 %0, tl, xl, %0; fma.rn.f32.bf16 %1, th, yl, %1;\n"
      "mov.b32 {tl,th}, %3;\n"
      "fma.rn.f32.bf16 %0, tl, xh, %0; fma.rn.f32.bf16 %1, th, yh, %1;\n"
      "mov.b32 {tl,th}, %4; mov.b32 {xl,xh}, %7; mov.b32 {yl,yh}, %9;\n"
      "fma.rn.f32.bf16 %0, tl, xl, %0; fma.rn.f32.bf16 %1, th, yl, %1;\n"
      "mov.b32 {tl,th}, %5;\n"
      "fma.rn.f32.bf16 %0, tl, xh, %0; fma.rn.f32.bf16 %1, th, yh, %1; }\n"
      : "+f"(a0), "+f"(a1)
      : "r"(t0), "r"(t1), "r"(t2), "r"(t3), "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]));
}
constexpr int kXPerWord = 4;
#else
// One packed word against 8 fp32 activations. Byte b of ((w << 3) & 0x78787878) | 0x80808080 is 0x80 | nib_{2b} << 3;
// one PRMT drops it under 0x3F into bits 16..23 of a float: 0x3F800000 | nib << 19 = 1 + nib/16 exactly. So
// acc += sum_k (1 + nib_k/16) x_k and the caller uses sum_k (nib_k - 8) x_k = 16 * (acc - 1.5 * sum_k x_k).
constexpr float kDotOffset = 1.5f;
constexpr float kDotScale = 16.f;
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ void dot_word(uint32_t w, const float* x, float& a0, float& a1) {
  const uint32_t e = ((w << 3) & 0x78787878u) | 0x80808080u, o = ((w >> 1) & 0x78787878u) | 0x80808080u;
#pragma unroll
  for (int b = 0; b < 4; b++) {
    const float fe = __uint_as_float(prmt(e, 0x3F000000u, 0x7044u | (b << 8)));
    const float fo = __uint_as_float(prmt(o, 0x3F000000u, 0x7044u | (b << 8)));
    a0 = fmaf(fe, x[2 * b], a0);
    a1 = fmaf(fo, x[2 * b + 1], a1);
  }
}
constexpr int kXPerWord = 8;
#endif

// RB rows of one tile against the lane's activations: acc[r] += sum over the lane's units of s*(dot) [+ z*sum x].
// `rows` are byte offsets of the RB records inside the tile (clamped by the caller for ragged tails).
template <class KC, bool HZ, class XR>
__device__ __forceinline__ void rowblock_dot(const uint8_t* tile, const int (&rows)[KC::RB], int slice, int lane,
                                             const XR& x, float (&acc)[KC::RB]) {
  constexpr int K = KC::K;
#pragma unroll
  for (int i = 0; i < KC::NI; i++) {
    const int unit = lane + 32 * i;
    const bool ok = !KC::PRED || unit < KC::UNITS;
    const int word = slice * KC::SLICE_WORDS + (ok ? unit : 0) * KC::U;
    const int g = word >> 4;
    const float off = kDotOffset * x.sum[i];
#pragma unroll
    for (int r = 0; r < KC::RB; r++) {
      const uint8_t* rec = tile + rows[r];
      float p0 = 0.f, p1 = 0.f;
      if (KC::U == 2) {
        const uint2 w = *reinterpret_cast<const uint2*>(rec + 4 * word);
        dot_word(w.x, &x.p[i][0], p0, p1);
        dot_word(w.y, &x.p[i][kXPerWord], p0, p1);
      } else {
        const uint4 w = *reinterpret_cast<const uint4*>(rec + 4 * word);
        dot_word(w.x, &x.p[i][0], p0, p1);
        dot_word(w.y, &x.p[i][kXPerWord], p0, p1);
        dot_word(w.z, &x.p[i][2 * kXPerWord], p0, p1);
        dot_word(w.w, &x.p[i][3 * kXPerWord], p0, p1);
      }
      const float s = bf2f(*reinterpret_cast<const uint16_t*>(rec + K / 2 + 2 * g)) * kDotScale;
      const float t = (p0 + p1) - off;
      acc[r] = fmaf(s, t, acc[r]);
      if (HZ) {
        const float z = bf2f(*reinterpret_cast<const uint16_t*>(rec + K / 2 + K / 64 + 2 * g));
        acc[r] = fmaf(z, x.sum[i], acc[r]);
      }
    }
  }
}

// Sum acc[r] over the 32 lanes for RB <= 4 rows with a transposed butterfly (6 shuffles for 4 rows instead of 20).
// On return lane (r << 3) holds the total of row r in `out`.
template <int RB>
__device__ __forceinline__ float reduce_rows(float (&acc)[RB], int lane) {
  float a[4];
#pragma unroll
  for (int r = 0; r < 4; r++) a[r] = r < RB ? acc[r] : 0.f;
  const bool hi16 = lane & 16, hi8 = lane & 8;
  const float s0 = hi16 ? a[0] : a[2], s1 = hi16 ? a[1] : a[3];
  const float k0 = hi16 ? a[2] : a[0], k1 = hi16 ? a[3] : a[1];
  const float b0 = k0 + __shfl_xor_sync(0xffffffffu, s0, 16);
  const float b1 = k1 + __shfl_xor_sync(0xffffffffu, s1, 16);
  float c = (hi8 ? b1 : b0) + __shfl_xor_sync(0xffffffffu, hi8 ? b0 : b1, 8);
  c += __shfl_xor_sync(0xffffffffu, c, 4);
  c += __shfl_xor_sync(0xffffffffu, c, 2);
  c += __shfl_xor_sync(0xffffffffu, c, 1);
  return c;   // row index = (lane >> 3): bit4 -> +2, bit3 -> +1
}

}  // namespace fb
