// int4 x bf16 GEMM of the M-token verify path on the 5th-generation tensor cores (tcgen05): every weight row is read
// once and multiplied with all MT <= 64 candidate tokens.
//
// D[128 weight rows][MT tokens] (fp32, in TENSOR MEMORY) = A[128][64] * B[MT][64]^T per 64-column chunk, issued by one
// thread as four tcgen05.mma (K = 16 each). A is the chunk's weights dequantised to bf16 (nib - 8) / 64 — exact — and
// written by 128 threads into shared memory in the K-major 128-byte-swizzle layout the MMA reads; B is the tokens'
// activations, copied into the same layout by cp.async. A group of 128 columns (two chunks) shares one bf16 scale per
// row, so every group accumulates into its own TMEM accumulator (two, used alternately); four epilogue warps read a
// finished group with tcgen05.ld and fold it into per-thread fp32 sums with the row's scale: the arithmetic is the
// reference's sum (nib - 8) * s * x with fp32 accumulation (reference: kernels/verify_mega.cu:18-75), only the order of
// summation differs. The asymmetric layout's zero points ride the same chunks as a second MMA with A = z (exact in bf16)
// into a third accumulator.
//
// Weight layout ("TC layout", a second library-owned copy made by tc_repack): per block of 128 rows, K / 64 chunks of
// 4 KB [8 words][128 rows] — word (w, r) holds columns 8w .. 8w+7 of row r with the nibbles ordered so that the four
// mask-and-fma conversions yield ADJACENT column pairs — then the block's scales [K / 128][128 rows] (and zeros).
// One 1-D bulk copy brings a chunk; the dequantising thread of row r reads its eight words without bank conflicts and
// writes eight 16-byte pieces.
//
// Work item = (row block, K split); CTAs take items round-robin. K splits (whole groups) give the small matrices enough
// items to occupy the GPU; their fp32 partials meet in global memory and the split that arrives last adds them in split
// order (deterministic) and runs the epilogue. Every wait is bounded.
#pragma once
#include "fb_common.cuh"
#include "fb_verify.cuh"

namespace fb {

constexpr int kTcRaw = 8;         // raw int4 chunks in flight (4 KB each)
constexpr int kTcStages = 4;      // dequantised A / activation B stages
constexpr int kTcThreads = 14 * 32;
constexpr int kTcRowBlock = 128;

__host__ __device__ constexpr size_t tc_block_bytes(int k, int has_zeros) {
  return (size_t)(k / 64) * 4096 + (size_t)(k / 128) * 256 * (has_zeros ? 2 : 1);
}
__host__ __device__ constexpr size_t tc_matrix_bytes(int rows, int k, int has_zeros) {
  return (size_t)((rows + kTcRowBlock - 1) / kTcRowBlock) * tc_block_bytes(k, has_zeros);
}

// caller layout (word c of a row = columns 8c .. 8c+7, column 8c+m in bits [4m, 4m+4)) -> TC layout.
// grid (row blocks, layers), 256 threads.
__global__ void tc_repack(const uint32_t* q, const uint16_t* sc, const uint16_t* zr, int rows, int K, int order, int order_arg,
                          int order_rows, uint8_t* out) {
  const bool hz = zr != nullptr;
  const int rb = blockIdx.x, nrb = gridDim.x, G = K / 128, nw = K / 8;
  uint8_t* blk = out + ((size_t)blockIdx.y * nrb + rb) * tc_block_bytes(K, hz);
  __shared__ int src_row[128];
  if (threadIdx.x < 128) {
    const int j = rb * 128 + threadIdx.x;
    src_row[threadIdx.x] = j < rows ? (int)blockIdx.y * rows + perm_row(j, order, order_arg, order_rows) : -1;
  }
  __syncthreads();
  uint32_t* words = reinterpret_cast<uint32_t*>(blk);
  for (int i = threadIdx.x; i < nw * 128; i += blockDim.x) {
    const int r = i & 127, wq = (i >> 7) & 7, kc = i >> 10;
    uint32_t d = 0x88888888u;                                  // padding rows: value 0
    if (src_row[r] >= 0) {
      const uint32_t s = __ldg(q + (size_t)src_row[r] * nw + kc * 8 + wq);
      // column offset e goes to nibble slot [0, 4, 1, 5, 2, 6, 3, 7][e]: (w & 0x000F000F) is then columns (0, 1),
      // (w & 0x00F000F0) columns (2, 3), and the same two masks on w >> 8 columns (4, 5) and (6, 7)
      d = (s & 0xFu) | ((s >> 4 & 0xFu) << 16) | ((s >> 8 & 0xFu) << 4) | ((s >> 12 & 0xFu) << 20) | ((s >> 16 & 0xFu) << 8) |
          ((s >> 20 & 0xFu) << 24) | ((s >> 24 & 0xFu) << 12) | ((s >> 28 & 0xFu) << 28);
    }
    words[i] = d;
  }
  uint16_t* meta = reinterpret_cast<uint16_t*>(blk + (size_t)(K / 64) * 4096);
  for (int i = threadIdx.x; i < G * 128; i += blockDim.x) {
    const int r = i & 127, g = i >> 7, row = src_row[r];
    meta[i] = row >= 0 ? sc[(size_t)row * G + g] : 0;
    if (hz) meta[G * 128 + i] = row >= 0 ? zr[(size_t)row * G + g] : 0;
  }
}

// cos / sin of every (token, rotation pair): the QKV epilogue reads them instead of evaluating sincosf per output
__global__ void v_rope_table(const int32_t* depth, const float* invf, int pos, int half, float2* out) {
  const int m = blockIdx.x;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf((float)(pos + depth[m]) * invf[i], &sn, &cs);
    out[(size_t)m * half + i] = make_float2(cs, sn);
  }
}

struct VtcParams {
  const uint8_t* w;          // TC layout of this matrix
  const uint16_t* x;         // activations bf16 [M][K], natural order
  int rows, K, M, has_zeros, nsplit;
  float* part;               // split-K partials [items][MT][128]
  unsigned* counters;        // [row blocks], zero between launches (the last split resets its counter)
  DevStatus* status;
  unsigned spin_limit;
  // epilogue operands
  uint16_t* h;               // RESID: bf16 [M][out_ld] in/out
  uint16_t* q;               // QKV: bf16 [M][n_head * HD]
  uint16_t *kc, *vc;         // QKV: layer base of the caches [max_seq][nkv][HD]
  uint16_t* act;             // SWIGLU: bf16 [M][out_ld]
  float* logits;             // LOGITS: f32 [M][out_ld]
  const float2* rope;        // QKV: [M][HD / 2] (cos, sin)
  int n_head, nkv, pos, out_ld, head_dim;
  float resid, logits_scaling;
};

__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// nibble pairs in bits (0..3, 16..19) / (4..7, 20..23) -> bf16 pair ((nib - 8) / 64, ...): the masked bits are the bf16
// subnormals nib * 2^-133 (16 nib * 2^-133); one bf16x2 fma with 2^127 (2^123) and -1/8
__device__ __forceinline__ uint32_t tc_cvt_lo(uint32_t w) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(w & 0x000F000Fu), "r"(0x7F007F00u), "r"(0xBE00BE00u));
  return d;
}
__device__ __forceinline__ uint32_t tc_cvt_hi(uint32_t w) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(w & 0x00F000F0u), "r"(0x7D007D00u), "r"(0xBE00BE00u));
  return d;
}
// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr));
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// shared-memory plan (bytes): raw ring, A stages (+ zero-point A stages), B stages, scales (2 items), barriers
constexpr int kTcMaxGroups = 32;  // groups of one work item (the host raises the K split until this holds)
template <int MT>
struct VtcSmem {
  static constexpr int RAW = 0;
  static constexpr int A = RAW + kTcRaw * 4096;
  static constexpr int AZ = A + kTcStages * 16384;                 // asymmetric layout only: A = z per row, per group parity
  static constexpr int B = AZ + 2 * 16384;
  static constexpr int SC = B + kTcStages * MT * 128;
  static constexpr int SC_BYTES = kTcMaxGroups * 256 * 2;          // scales, then zeros
  static constexpr int BAR = SC + 2 * SC_BYTES;
  static constexpr int TOTAL = BAR + 512 + 1024;                   // + slack to align the base to 1024 bytes
};

// work items of this CTA in order; every role walks the same sequence
struct TcWalk {
  int item, nitems, nsplit, gtot, step;
  int rb, sp, g0, g1;
  __device__ __forceinline__ TcWalk(int rows, int K, int ns) {
    nsplit = ns; gtot = K / 128;
    nitems = ((rows + kTcRowBlock - 1) / kTcRowBlock) * ns;
    item = (int)blockIdx.x; step = (int)gridDim.x;
    set();
  }
  __device__ __forceinline__ bool valid() const { return item < nitems; }
  __device__ __forceinline__ void set() {
    rb = item / nsplit; sp = item % nsplit;
    g0 = (int)((long long)gtot * sp / nsplit); g1 = (int)((long long)gtot * (sp + 1) / nsplit);
  }
  __device__ __forceinline__ void next() { item += step; set(); }
};

template <int MT, int EPI>
__global__ void __launch_bounds__(kTcThreads, 1) v_gemm_tc(const VtcParams P) {
  using S = VtcSmem<MT>;
  extern __shared__ __align__(1024) uint8_t tsm_raw[];
  // the swizzle pattern is a function of the absolute shared-memory address: tiles must start on 1024-byte boundaries
  uint8_t* tsm = tsm_raw + ((1024u - (smem_u32(tsm_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tsm + S::BAR);
  uint64_t *raw_full = bars, *raw_empty = bars + kTcRaw, *ab_full = bars + 2 * kTcRaw, *ab_empty = ab_full + kTcStages,
           *acc_full = ab_empty + kTcStages, *acc_empty = acc_full + 2, *sc_full = acc_empty + 2, *sc_empty = sc_full + 2;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(sc_empty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool hz = P.has_zeros != 0;
  const int K = P.K, G = K / 128;
  const size_t blk_bytes = tc_block_bytes(K, hz);
  if (tid == 0) {
    for (int i = 0; i < kTcRaw; i++) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], 4); }
    for (int i = 0; i < kTcStages; i++) { mbar_init(&ab_full[i], 8); mbar_init(&ab_empty[i], 1); }
    for (int i = 0; i < 2; i++) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); mbar_init(&sc_full[i], 1); mbar_init(&sc_empty[i], 4); }
    *s_abort = 0;
    mbar_fence_init();
  }
  constexpr int TCOLS = 256;                                  // two group accumulators + the zero-point accumulator
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(TCOLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  WaitCtl wc{P.status, s_abort, P.spin_limit};
  pdl_trigger();

  if (warp == 0) {
    // ---------------- producer: raw int4 chunks and the item's scales (weights do not depend on the previous kernel)
    if (lane == 0) {
      uint32_t it = 0, ii = 0;
      for (TcWalk w(P.rows, K, P.nsplit); w.valid(); w.next(), ii++) {
        const uint8_t* blk = P.w + (size_t)w.rb * blk_bytes;
        const int b = ii & 1, ng = w.g1 - w.g0;
        if (!mbar_wait(&sc_empty[b], ((ii >> 1) & 1) ^ 1, wc, W_EMPTY, 1)) break;
        mbar_expect_tx(&sc_full[b], (uint32_t)ng * 256 * (hz ? 2 : 1));
        bulk_g2s(tsm + S::SC + b * S::SC_BYTES, blk + (size_t)(K / 64) * 4096 + (size_t)w.g0 * 256, ng * 256, &sc_full[b]);
        if (hz)
          bulk_g2s(tsm + S::SC + b * S::SC_BYTES + kTcMaxGroups * 256, blk + (size_t)(K / 64) * 4096 + (size_t)(G + w.g0) * 256, ng * 256,
                   &sc_full[b]);
        bool ok = true;
        for (int c = 2 * w.g0; c < 2 * w.g1 && ok; c++, it++) {
          const int s = it % kTcRaw;
          ok = mbar_wait(&raw_empty[s], ((it / kTcRaw) & 1) ^ 1, wc, W_EMPTY, 2);
          if (!ok) break;
          mbar_expect_tx(&raw_full[s], 4096);
          bulk_g2s(tsm + S::RAW + s * 4096, blk + (size_t)c * 4096, 4096, &raw_full[s]);
        }
        if (!ok) break;
      }
      // every copy issued must have landed before the CTA may exit: the consumers wait for all of them in a clean run;
      // after a failure, wait here (bounded)
      if (*s_abort) {
        for (int k = 0; k < kTcRaw && k < (int)it; k++) {
          const uint32_t j = it - 1 - k;
          for (unsigned i = 0; i < wc.limit; i++) {
            if (mbar_try(&raw_full[j % kTcRaw], (j / kTcRaw) & 1)) break;
            if ((i & 1023) == 1023) __nanosleep(64);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue: one thread
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MT >> 3) << 17) | ((128u >> 4) << 24);
      uint32_t it = 0, gi = 0;
      bool ok = true;
      for (TcWalk w(P.rows, K, P.nsplit); w.valid() && ok; w.next()) {
        for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
          const int a = gi & 1;
          ok = mbar_wait(&acc_empty[a], ((gi >> 1) & 1) ^ 1, wc, W_EMPTY, 3);
          for (int half = 0; half < 2 && ok; half++, it++) {
            const int s = it % kTcStages;
            ok = mbar_wait(&ab_full[s], (it / kTcStages) & 1, wc, W_FULL, 4);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem_u32(tsm + S::A + s * 16384), sb = smem_u32(tsm + S::B + s * MT * 128);
            const uint32_t sz = smem_u32(tsm + S::AZ + (gi & 1) * 16384);
#pragma unroll
            for (int k = 0; k < 4; k++) {
              tc_mma(tmem + a * MT, tc_desc(sa + k * 32), tc_desc(sb + k * 32), idesc, (half | k) ? 1u : 0u);
              if (hz) tc_mma(tmem + 2 * MT, tc_desc(sz + k * 32), tc_desc(sb + k * 32), idesc, (g > w.g0 || half || k) ? 1u : 0u);
            }
            tc_commit(&ab_empty[s]);
          }
          if (ok) tc_commit(&acc_full[a]);
        }
      }
    }
  } else if (warp < 6) {
    // ---------------- dequantise: thread = row of the block; 8 words -> 8 swizzled 16-byte pieces per chunk
    const int row = (warp - 2) * 32 + lane;
    const uint32_t rsw = (uint32_t)(row >> 3) * 1024 + (uint32_t)(row & 7) * 128, rx = (uint32_t)(row & 7);
    uint32_t it = 0, gi = 0, ii = 0;
    bool ok = true;
    for (TcWalk w(P.rows, K, P.nsplit); w.valid() && ok; w.next(), ii++) {
      for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
        for (int half = 0; half < 2 && ok; half++, it++) {
          const int sr = it % kTcRaw, s = it % kTcStages;
          ok = mbar_wait(&raw_full[sr], (it / kTcRaw) & 1, wc, W_FULL, 5) &&
               mbar_wait(&ab_empty[s], ((it / kTcStages) & 1) ^ 1, wc, W_EMPTY, 6);
          if (!ok) break;
          const uint32_t raw = smem_u32(tsm + S::RAW + sr * 4096) + (uint32_t)row * 4, dst = smem_u32(tsm + S::A + s * 16384) + rsw;
          uint32_t wv[8];
#pragma unroll
          for (int q8 = 0; q8 < 8; q8++) wv[q8] = lds32(raw + q8 * 512);
#pragma unroll
          for (int q8 = 0; q8 < 8; q8++)
            sts128(dst + (((uint32_t)q8 ^ rx) << 4), tc_cvt_lo(wv[q8]), tc_cvt_hi(wv[q8]), tc_cvt_lo(wv[q8] >> 8), tc_cvt_hi(wv[q8] >> 8));
          if (hz && half == 0) {
            // the group's zero point of this row, replicated over a 64-column tile: A_z = z. The tile is shared by the
            // group's two chunks and reused every second group: its last readers are the MMAs of chunks it-4 and it-3,
            // so the stage of chunk it+1 (= it-3's) must be free too; then the scales must have landed
            ok = mbar_wait(&ab_empty[(it + 1) % kTcStages], (((it + 1) / kTcStages) & 1) ^ 1, wc, W_EMPTY, 6) &&
                 mbar_wait(&sc_full[ii & 1], (ii >> 1) & 1, wc, W_FULL, 7);
            if (!ok) break;
            const uint16_t z = reinterpret_cast<const uint16_t*>(tsm + S::SC + (ii & 1) * S::SC_BYTES + kTcMaxGroups * 256)[(g - w.g0) * 128 + row];
            const uint32_t zz = (uint32_t)z | ((uint32_t)z << 16), dz = smem_u32(tsm + S::AZ + (gi & 1) * 16384) + rsw;
#pragma unroll
            for (int q8 = 0; q8 < 8; q8++) sts128(dz + ((uint32_t)q8 << 4), zz, zz, zz, zz);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) { mbar_arrive(&raw_empty[sr]); mbar_arrive(&ab_full[s]); }
        }
      }
    }
  } else if (warp < 10) {
    // ---------------- activations: cp.async pieces into the swizzled B stages, three chunks ahead
    pdl_wait();                                                  // the activations are the previous kernel's output
    const int lt = (warp - 6) * 32 + lane;
    constexpr int PIECES = MT * 8, PPT = (PIECES + 127) / 128, AHEAD = kTcStages - 1;
    auto issue = [&](int chunk, int s) {
      uint8_t* dst = tsm + S::B + s * MT * 128;
#pragma unroll
      for (int k = 0; k < PPT; k++) {
        const int i = lt + k * 128;
        if (i < PIECES) {
          const int m = i >> 3, c = i & 7;
          uint8_t* d = dst + (m >> 3) * 1024 + (m & 7) * 128 + ((c ^ (m & 7)) << 4);
          if (m < P.M) cp_async16(d, P.x + (size_t)m * K + chunk * 64 + c * 8);
          else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
      }
    };
    // the chunk sequence of this CTA, walked twice: once for issuing (ahead), once for completing
    TcWalk wi(P.rows, K, P.nsplit);
    int ci = wi.valid() ? 2 * wi.g0 : 0;
    uint32_t iti = 0;
    bool ok = true;
    auto issue_next = [&]() {
      if (wi.valid() && ok) {
        const int s = iti % kTcStages;
        ok = mbar_wait(&ab_empty[s], ((iti / kTcStages) & 1) ^ 1, wc, W_EMPTY, 8);
        if (ok) issue(ci, s);
        iti++;
        if (++ci >= 2 * wi.g1) { wi.next(); ci = wi.valid() ? 2 * wi.g0 : 0; }
      }
      cp_async_commit();
    };
    for (int j = 0; j < AHEAD; j++) issue_next();
    uint32_t it = 0;
    for (TcWalk w(P.rows, K, P.nsplit); w.valid() && ok; w.next()) {
      for (int c = 2 * w.g0; c < 2 * w.g1 && ok; c++, it++) {
        cp_async_wait<AHEAD - 1>();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ab_full[it % kTcStages]);
        issue_next();
      }
    }
    cp_async_wait<0>();
  } else {
    // ---------------- epilogue: thread = row of the block (TMEM lane), MT fp32 sums in registers
    const int quad = warp & 3, row = quad * 32 + lane;
    const uint32_t tlane = tmem + ((uint32_t)(quad * 32) << 16);
    uint32_t gi = 0, ii = 0;
    bool ok = true;
    pdl_wait();
    for (TcWalk w(P.rows, K, P.nsplit); w.valid() && ok; w.next(), ii++) {
      float y[MT];
#pragma unroll
      for (int t = 0; t < MT; t++) y[t] = 0.f;
      const int b = ii & 1;
      ok = mbar_wait(&sc_full[b], (ii >> 1) & 1, wc, W_FULL, 9);
      const uint16_t* scs = reinterpret_cast<const uint16_t*>(tsm + S::SC + b * S::SC_BYTES);
      for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
        const int a = gi & 1;
        ok = mbar_wait(&acc_full[a], (gi >> 1) & 1, wc, W_FULL, 10);
        if (!ok) break;
        tc_fence_after();
        const float s64 = bf2f(scs[(g - w.g0) * 128 + row]) * 64.0f;
#pragma unroll
        for (int c8 = 0; c8 < MT / 8; c8++) {
          uint32_t v[8];
          tc_ld8(tlane + a * MT + c8 * 8, v);
          tc_ld_wait();
#pragma unroll
          for (int e = 0; e < 8; e++) y[c8 * 8 + e] = fmaf(s64, __uint_as_float(v[e]), y[c8 * 8 + e]);
        }
        if (hz && g == w.g1 - 1) {                               // the item's zero-point sums: sum_g z_g * sum_k x_k
#pragma unroll
          for (int c8 = 0; c8 < MT / 8; c8++) {
            uint32_t v[8];
            tc_ld8(tlane + 2 * MT + c8 * 8, v);
            tc_ld_wait();
#pragma unroll
            for (int e = 0; e < 8; e++) y[c8 * 8 + e] += __uint_as_float(v[e]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[a]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sc_empty[b]);
      if (!ok) break;
      // ---- K splits meet in global memory; the split that arrives last adds them in split order ----
      if (P.nsplit > 1) {
        // each epilogue warp settles its own 32 rows: no block-wide barrier on a path that a failed wait may leave
        float* mine = P.part + (size_t)w.item * MT * 128;
#pragma unroll
        for (int t = 0; t < MT; t++) mine[t * 128 + row] = y[t];
        __threadfence();
        __syncwarp();
        unsigned old = 0;
        if (lane == 0) {
          old = atomicAdd(P.counters + w.rb * 4 + quad, 1u);
          if (old == (unsigned)P.nsplit - 1u) P.counters[w.rb * 4 + quad] = 0u;
        }
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old != (unsigned)P.nsplit - 1u) continue;
        __threadfence();
#pragma unroll
        for (int t = 0; t < MT; t++) y[t] = 0.f;
        for (int sp = 0; sp < P.nsplit; sp++) {
          const float* src = P.part + (size_t)(w.rb * P.nsplit + sp) * MT * 128;
#pragma unroll
          for (int t = 0; t < MT; t++) y[t] += __ldcg(src + t * 128 + row);
        }
      }
      // ---- epilogue proper: stream row `srow` of the matrix, token t -> y[t] ----
      const int srow = w.rb * 128 + row;
      if (EPI == EPI_RESID) {
#pragma unroll
        for (int t = 0; t < MT; t++)
          if (srow < P.rows && t < P.M) {
            uint16_t* hp = P.h + (size_t)t * P.out_ld + srow;
            *hp = f2bf(bf2f(*hp) + y[t] * P.resid);
          }
      } else if (EPI == EPI_LOGITS) {
#pragma unroll
        for (int t = 0; t < MT; t++)
          if (srow < P.rows && t < P.M) P.logits[(size_t)t * P.out_ld + srow] = y[t] / P.logits_scaling;
      } else if (EPI == EPI_SWIGLU) {
        // stream rows (2i, 2i+1) = (gate_i, up_i): neighbouring lanes
#pragma unroll
        for (int t = 0; t < MT; t++) {
          const float u = __shfl_xor_sync(0xffffffffu, y[t], 1);
          if (!(lane & 1) && srow < P.rows && t < P.M) {
            const float gg = rbf(y[t]), uu = rbf(u);
            P.act[(size_t)t * P.out_ld + (srow >> 1)] = f2bf((gg / (1.0f + __expf(-gg))) * uu);
          }
        }
      } else {
        // QKV: stream rows (2p, 2p+1) of a q / k head are dims (p, p + HD/2); v rows keep their order
        const int HD = P.head_dim, HP = HD >> 1, QD = P.n_head * HD;
        const int head = srow / HD, within = srow % HD;
#pragma unroll
        for (int t = 0; t < MT; t++) {
          const float o = __shfl_xor_sync(0xffffffffu, y[t], 1);
          if (!(lane & 1) && srow < P.rows && t < P.M) {
            if (head < P.n_head + P.nkv) {
              const int i = within >> 1;
              const float x0 = rbf(y[t]), x1 = rbf(o);
              const float2 cs = __ldg(P.rope + (size_t)t * HP + i);
              const uint16_t y0 = f2bf(x0 * cs.x - x1 * cs.y), y1 = f2bf(x1 * cs.x + x0 * cs.y);
              if (head < P.n_head) {
                P.q[(size_t)t * QD + head * HD + i] = y0;
                P.q[(size_t)t * QD + head * HD + i + HP] = y1;
              } else {
                uint16_t* kr = P.kc + ((size_t)(P.pos + t) * P.nkv + (head - P.n_head)) * HD;
                kr[i] = y0;
                kr[i + HP] = y1;
              }
            } else {
              uint16_t* vr = P.vc + ((size_t)(P.pos + t) * P.nkv + (head - P.n_head - P.nkv)) * HD;
              *reinterpret_cast<uint32_t*>(vr + within) = (uint32_t)f2bf(y[t]) | ((uint32_t)f2bf(o) << 16);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TCOLS));
}

}  // namespace fb
