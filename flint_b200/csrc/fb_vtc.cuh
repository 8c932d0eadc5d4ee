// int4 x bf16 GEMM of the M-token verify path on the 5th-generation tensor cores (tcgen05): every weight row is read
// once and multiplied with all MT <= 64 candidate tokens.
//
// D[128 weight rows][MT tokens] (fp32, in TENSOR MEMORY) = A[128][128] * B[MT][128]^T per group of 128 columns, issued by
// one thread as eight tcgen05.mma (K = 16 each). A is the chunk's weights dequantised to bf16 (nib - 8) / 64 — exact — by 128
// threads, thread = weight row = TMEM lane, and stored with tcgen05.st straight into tensor memory (a ring of four
// 64-column stages): routing A through shared memory would cost 8 bytes of shared-memory traffic per int4 byte and cap
// the kernel well below the HBM rate. B is the tokens' activations, copied by cp.async into shared memory in the K-major
// 128-byte-swizzle layout the MMA reads. A group of 128 columns shares one bf16 scale per
// row, so every group accumulates into its own TMEM accumulator (a ring of them); four epilogue warps read a
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

constexpr int kTcStages = 4;      // operand stages: A (dequantised group, 64 TMEM columns) and B (activations, shared memory)
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
// 32 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
      "%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
        "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// shared-memory plan (bytes): raw ring, A stages (+ zero-point A stages), B stages, scales (2 items), barriers
constexpr int kTcMaxGroups = 32;  // groups of one work item (the host raises the K split until this holds)
// shared-memory plan (bytes). The raw ring is what keeps HBM busy: 12..14 groups of 8 KB in flight per SM; a stage of
// activations is the group's two 64-column tiles.
template <int MT, bool HZ>
struct VtcSmem {
  static constexpr int NRAW = HZ ? 12 : 14;                        // raw int4 groups in flight (8 KB each)
  static constexpr int BSTAGE = MT * 256;                          // two [MT rows x 128 bytes] swizzled tiles
  static constexpr int RAW = 0;
  static constexpr int B = RAW + NRAW * 8192;
  static constexpr int SC = B + kTcStages * BSTAGE;
  static constexpr int SC_BYTES = kTcMaxGroups * 256 * (HZ ? 2 : 1);   // scales, then zeros
  static constexpr int EPI = SC + 2 * SC_BYTES;                    // the item's sums, fp32 [MT][128 rows]
  static constexpr int BAR = EPI + MT * 512;
  static constexpr int TOTAL = BAR + 2048 + 1024;                  // barriers, 1/rms per phase and token + slack to align the base
  static_assert(TOTAL <= 227 * 1024, "verify GEMM shared memory");
  // tensor memory columns: group accumulators, zero-point accumulator, A stages (64 columns = 128 bf16 per row), A_z
  // (8 columns = one k16 step of the row's zero point, the same for every step of the group)
  static constexpr int NACC = HZ ? 2 : 4;
  static constexpr int T_ACCZ = NACC * MT, T_A = T_ACCZ + (HZ ? MT : 0), T_AZ = T_A + kTcStages * 64;
  static_assert(T_AZ + (HZ ? kTcStages * 8 : 0) <= 512, "tensor memory columns");
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

__device__ __forceinline__ void tc_st8(uint32_t taddr, uint32_t z) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr), "r"(z) : "memory");
}

template <int MT, int EPI, bool HZ>
__global__ void __launch_bounds__(kTcThreads, 1) v_gemm_tc(const VtcParams P) {
  using S = VtcSmem<MT, HZ>;
  constexpr int NRAW = S::NRAW, NS = kTcStages, NACC = S::NACC;
  extern __shared__ __align__(1024) uint8_t tsm_raw[];
  // the swizzle pattern is a function of the absolute shared-memory address: tiles must start on 1024-byte boundaries
  uint8_t* tsm = tsm_raw + ((1024u - (smem_u32(tsm_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tsm + S::BAR);
  uint64_t *raw_full = bars, *raw_empty = bars + NRAW, *a_full = bars + 2 * NRAW, *b_full = a_full + NS, *s_empty = b_full + NS,
           *acc_full = s_empty + NS, *acc_empty = acc_full + NACC, *sc_full = acc_empty + NACC, *sc_empty = sc_full + 2;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(sc_empty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr bool hz = HZ;
  const int K = P.K, G = K / 128;
  const size_t blk_bytes = tc_block_bytes(K, hz);
  if (tid == 0) {
    for (int i = 0; i < NRAW; i++) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], 4); }
    for (int i = 0; i < NS; i++) { mbar_init(&a_full[i], 4); mbar_init(&b_full[i], 4); mbar_init(&s_empty[i], 1); }
    for (int i = 0; i < NACC; i++) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    for (int i = 0; i < 2; i++) { mbar_init(&sc_full[i], 1); mbar_init(&sc_empty[i], 4); }
    *s_abort = 0;
    mbar_fence_init();
  }
  constexpr int TCOLS = 512;
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
    // ---------------- producer: raw int4 groups and the item's scales (weights do not depend on the previous kernel)
    if (lane == 0) {
      uint32_t gi = 0, ii = 0;
      for (TcWalk w(P.rows, K, P.nsplit); w.valid(); w.next(), ii++) {
        const uint8_t* blk = P.w + (size_t)w.rb * blk_bytes;
        const int b = ii & 1, ng = w.g1 - w.g0;
        if (!mbar_wait(&sc_empty[b], ((ii >> 1) & 1) ^ 1, wc, W_EMPTY, 1)) break;
        mbar_expect_tx(&sc_full[b], (uint32_t)ng * 256 * (hz ? 2 : 1));
        bulk_g2s(tsm + S::SC + b * S::SC_BYTES, blk + (size_t)(K / 64) * 4096 + (size_t)w.g0 * 256, ng * 256, &sc_full[b]);
        if (hz)
          bulk_g2s(tsm + S::SC + b * S::SC_BYTES + kTcMaxGroups * 256, blk + (size_t)(K / 64) * 4096 + (size_t)(G + w.g0) * 256,
                   ng * 256, &sc_full[b]);
        bool ok = true;
        for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
          const int s = gi % NRAW;
          ok = mbar_wait(&raw_empty[s], ((gi / NRAW) & 1) ^ 1, wc, W_EMPTY, 2);
          if (!ok) break;
          mbar_expect_tx(&raw_full[s], 8192);
          bulk_g2s(tsm + S::RAW + s * 8192, blk + (size_t)g * 8192, 8192, &raw_full[s]);
        }
        if (!ok) break;
      }
      // every copy issued must have landed before the CTA may exit: the consumers wait for all of them in a clean run;
      // after a failure, wait here (bounded)
      if (*s_abort) {
        for (int k = 0; k < NRAW && k < (int)gi; k++) {
          const uint32_t j = gi - 1 - k;
          for (unsigned i = 0; i < wc.limit; i++) {
            if (mbar_try(&raw_full[j % NRAW], (j / NRAW) & 1)) break;
            if ((i & 1023) == 1023) __nanosleep(64);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue: one thread, eight MMAs per group, two commits
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MT >> 3) << 17) | ((128u >> 4) << 24);
      uint32_t gi = 0;
      bool ok = true;
      for (TcWalk w(P.rows, K, P.nsplit); w.valid() && ok; w.next()) {
        for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
          const int a = gi % NACC, s = gi % NS;
          ok = mbar_wait(&acc_empty[a], ((gi / NACC) & 1) ^ 1, wc, W_EMPTY, 3) && mbar_wait(&a_full[s], (gi / NS) & 1, wc, W_FULL, 4) &&
               mbar_wait(&b_full[s], (gi / NS) & 1, wc, W_FULL, 4);
          if (!ok) break;
          tc_fence_after();
          const uint32_t ta = tmem + S::T_A + s * 64, tz = tmem + S::T_AZ + s * 8;
          const uint32_t sb = smem_u32(tsm + S::B + s * S::BSTAGE);
#pragma unroll
          for (int k = 0; k < 8; k++) {
            const uint64_t db = tc_desc(sb + (k >> 2) * (MT * 128) + (k & 3) * 32);
            tc_mma_ts(tmem + a * MT, ta + k * 8, db, idesc, k ? 1u : 0u);
            if (hz) tc_mma_ts(tmem + S::T_ACCZ, tz, db, idesc, (g > w.g0 || k) ? 1u : 0u);
          }
          tc_commit(&s_empty[s]);
          tc_commit(&acc_full[a]);
        }
      }
    }
  } else if (warp < 6) {
    // ---------------- dequantise: thread = row of the block = TMEM lane; 16 words -> 64 packed bf16 pairs per group
    const int quad = warp & 3, row = quad * 32 + lane;
    const uint32_t tl = tmem + ((uint32_t)(quad * 32) << 16);
    uint32_t gi = 0, ii = 0;
    bool ok = true;
    for (TcWalk w(P.rows, K, P.nsplit); w.valid() && ok; w.next(), ii++) {
      if (hz) ok = mbar_wait(&sc_full[ii & 1], (ii >> 1) & 1, wc, W_FULL, 7);
      for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
        const int sr = gi % NRAW, s = gi % NS;
        ok = mbar_wait(&raw_full[sr], (gi / NRAW) & 1, wc, W_FULL, 5) && mbar_wait(&s_empty[s], ((gi / NS) & 1) ^ 1, wc, W_EMPTY, 6);
        if (!ok) break;
        tc_fence_after();
        const uint32_t raw = smem_u32(tsm + S::RAW + sr * 8192) + (uint32_t)row * 4;
#pragma unroll
        for (int c = 0; c < 2; c++) {
          uint32_t v[32];
#pragma unroll
          for (int q8 = 0; q8 < 8; q8++) {
            const uint32_t wv = lds32(raw + c * 4096 + q8 * 512);
            v[4 * q8] = tc_cvt_lo(wv); v[4 * q8 + 1] = tc_cvt_hi(wv); v[4 * q8 + 2] = tc_cvt_lo(wv >> 8); v[4 * q8 + 3] = tc_cvt_hi(wv >> 8);
          }
          tc_st32(tl + S::T_A + s * 64 + c * 32, v);
        }
        if (hz) {
          // the group's zero point of this row as one k16 step: A_z = z for every column
          const uint16_t z = reinterpret_cast<const uint16_t*>(tsm + S::SC + (ii & 1) * S::SC_BYTES + kTcMaxGroups * 256)[(g - w.g0) * 128 + row];
          tc_st8(tl + S::T_AZ + s * 8, (uint32_t)z | ((uint32_t)z << 16));
        }
        tc_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) { mbar_arrive(&raw_empty[sr]); mbar_arrive(&a_full[s]); }
      }
    }
  } else if (warp < 10) {
    // ---------------- activations: cp.async pieces into the swizzled B stages, three groups ahead
    pdl_wait();                                                  // the activations are the previous kernel's output
    const int lt = (warp - 6) * 32 + lane;
    constexpr int PIECES = MT * 16, PPT = (PIECES + 127) / 128, AHEAD = NS - 1;
    auto issue = [&](int g, int s) {
      uint8_t* dst = tsm + S::B + s * S::BSTAGE;
#pragma unroll
      for (int k = 0; k < PPT; k++) {
        const int i = lt + k * 128;
        if (i < PIECES) {
          const int c = i & 7, m = (i >> 3) % MT, tile = i / (8 * MT);
          uint8_t* d = dst + tile * (MT * 128) + (m >> 3) * 1024 + (m & 7) * 128 + ((c ^ (m & 7)) << 4);
          if (m < P.M) cp_async16(d, P.x + (size_t)m * K + g * 128 + tile * 64 + c * 8);
          else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
      }
    };
    // the group sequence of this CTA, walked twice: once for issuing (ahead), once for completing
    TcWalk wi(P.rows, K, P.nsplit);
    int gn = wi.valid() ? wi.g0 : 0;
    uint32_t gii = 0;
    bool ok = true;
    auto issue_next = [&]() {
      if (wi.valid() && ok) {
        const int s = gii % NS;
        ok = mbar_wait(&s_empty[s], ((gii / NS) & 1) ^ 1, wc, W_EMPTY, 8);
        if (ok) issue(gn, s);
        gii++;
        if (++gn >= wi.g1) { wi.next(); gn = wi.valid() ? wi.g0 : 0; }
      }
      cp_async_commit();
    };
    for (int j = 0; j < AHEAD; j++) issue_next();
    uint32_t gi = 0;
    for (TcWalk w(P.rows, K, P.nsplit); w.valid() && ok; w.next()) {
      for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
        cp_async_wait<AHEAD - 1>();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&b_full[gi % NS]);
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
        const int a = gi % NACC;
        ok = mbar_wait(&acc_full[a], (gi / NACC) & 1, wc, W_FULL, 10);
        if (!ok) break;
        tc_fence_after();
        const float s64 = bf2f(scs[(g - w.g0) * 128 + row]) * 64.0f;
        constexpr int HALF = MT >= 32 ? 32 : MT;                // columns per batch of loads: one wait per batch
#pragma unroll
        for (int h0 = 0; h0 < MT; h0 += HALF) {
          uint32_t v[HALF / 8][8];
#pragma unroll
          for (int c8 = 0; c8 < HALF / 8; c8++) tc_ld8(tlane + a * MT + h0 + c8 * 8, v[c8]);
          tc_ld_wait();
#pragma unroll
          for (int c8 = 0; c8 < HALF / 8; c8++)
#pragma unroll
            for (int e = 0; e < 8; e++) y[h0 + c8 * 8 + e] = fmaf(s64, __uint_as_float(v[c8][e]), y[h0 + c8 * 8 + e]);
        }
        if (hz && g == w.g1 - 1) {                               // the item's zero-point sums: sum_g z_g * sum_k x_k
#pragma unroll
          for (int c8 = 0; c8 < MT / 8; c8++) {
            uint32_t v[8];
            tc_ld8(tlane + S::T_ACCZ + c8 * 8, v);
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
      // ---- epilogue proper. The sums go through shared memory ([token][row], a warp touches only its own 32 rows) so
      // that the per-token work is a compact loop (unrolled over 64 tokens it is tens of KB of straight-line code that
      // runs once per item: one instruction-cache miss after the other). Tokens go in batches of 8 whose global loads
      // are all issued before the first dependent store.
      float* ys = reinterpret_cast<float*>(tsm + S::EPI);
      __syncwarp();
#pragma unroll
      for (int t = 0; t < MT; t++) ys[t * 128 + row] = y[t];
      __syncwarp();
      const int srow = w.rb * 128 + row;
      if (EPI == EPI_RESID) {
        if (srow < P.rows)
          for (int t0 = 0; t0 < P.M; t0 += 8) {
            uint16_t hv[8];
#pragma unroll
            for (int e = 0; e < 8; e++) hv[e] = t0 + e < P.M ? P.h[(size_t)(t0 + e) * P.out_ld + srow] : (uint16_t)0;
#pragma unroll
            for (int e = 0; e < 8; e++)
              if (t0 + e < P.M) P.h[(size_t)(t0 + e) * P.out_ld + srow] = f2bf(bf2f(hv[e]) + ys[(t0 + e) * 128 + row] * P.resid);
          }
      } else if (EPI == EPI_LOGITS) {
        if (srow < P.rows)
#pragma unroll 4
          for (int t = 0; t < P.M; t++) P.logits[(size_t)t * P.out_ld + srow] = ys[t * 128 + row] / P.logits_scaling;
      } else if (EPI == EPI_SWIGLU) {
        // stream rows (2i, 2i+1) = (gate_i, up_i): the even row's thread writes act_i
        if (!(lane & 1) && srow < P.rows)
#pragma unroll 4
          for (int t = 0; t < P.M; t++) {
            const float gg = rbf(ys[t * 128 + row]), uu = rbf(ys[t * 128 + row + 1]);
            P.act[(size_t)t * P.out_ld + (srow >> 1)] = f2bf((gg / (1.0f + __expf(-gg))) * uu);
          }
      } else {
        // QKV: stream rows (2p, 2p+1) of a q / k head are dims (p, p + HD/2); v rows keep their order
        const int HD = P.head_dim, HP = HD >> 1, QD = P.n_head * HD;
        const int head = srow / HD, within = srow % HD, i = within >> 1;
        if (!(lane & 1) && srow < P.rows) {
          if (head < P.n_head + P.nkv) {
            for (int t0 = 0; t0 < P.M; t0 += 8) {
              float2 cs[8];
#pragma unroll
              for (int e = 0; e < 8; e++) cs[e] = t0 + e < P.M ? __ldg(P.rope + (size_t)(t0 + e) * HP + i) : make_float2(1.f, 0.f);
#pragma unroll
              for (int e = 0; e < 8; e++) {
                const int t = t0 + e;
                if (t < P.M) {
                  const float x0 = rbf(ys[t * 128 + row]), x1 = rbf(ys[t * 128 + row + 1]);
                  const uint16_t y0 = f2bf(x0 * cs[e].x - x1 * cs[e].y), y1 = f2bf(x1 * cs[e].x + x0 * cs[e].y);
                  if (head < P.n_head) {
                    P.q[(size_t)t * QD + head * HD + i] = y0;
                    P.q[(size_t)t * QD + head * HD + i + HP] = y1;
                  } else {
                    uint16_t* kr = P.kc + ((size_t)(P.pos + t) * P.nkv + (head - P.n_head)) * HD;
                    kr[i] = y0;
                    kr[i + HP] = y1;
                  }
                }
              }
            }
          } else {
#pragma unroll 4
            for (int t = 0; t < P.M; t++) {
              uint16_t* vr = P.vc + ((size_t)(P.pos + t) * P.nkv + (head - P.n_head - P.nkv)) * HD;
              *reinterpret_cast<uint32_t*>(vr + within) = (uint32_t)f2bf(ys[t * 128 + row]) | ((uint32_t)f2bf(ys[t * 128 + row + 1]) << 16);
            }
          }
        }
      }
      __syncwarp();                                              // the staging rows are rewritten by the next item
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TCOLS));
}


// ------------------------------------------------------------------------------------------------ GEMM chain
// Up to four of the GEMMs above in ONE launch (O projection -> gate/up -> down -> next layer's QKV, or the LM head at
// the end): the warp roles and their rings simply keep running from one GEMM ("phase") into the next, so the weights of
// the next phase are already streaming — and partly dequantised in tensor memory — while the current one drains, and the
// per-launch ramp of a short pipeline is paid once per four GEMMs. Only the activation loaders need the other CTAs: they
// wait (bounded) on a grid-wide arrival counter that every epilogue warp bumps when its last item of the previous phase is
// in global memory. RMSNorm does not get a phase of its own: the epilogue that updates the residual rows also leaves, per
// 32-row warp, the sums of squares of the rows it wrote; the next phase's loaders reduce them in a fixed order to 1/rms per
// token and normalise the activation tiles in place, in shared memory, after their cp.async has landed:
// bf16((float(h) * r) * float(w)), the rounding of the reference's rmsnorm (reference: kernels/verify_mega.cu:78-104).
struct VtcPhase {
  const uint8_t* w;          // TC layout
  const uint16_t* x;         // bf16 [M][K]: activations, or (norm_w set) the residual stream to be normalised on the fly
  const uint16_t* norm_w;    // bf16 [K] RMSNorm weights or nullptr
  const float* ssq_in;       // [n_ssq][64]: partial sums of squares per token, written by the previous residual phase
  float* ssq_out;            // RESID: [row blocks * 4][64] or nullptr
  uint16_t* xn_out;          // norm_w set: the items of row block 0 also write the normalised rows here (feature output) or nullptr
  uint16_t* h;               // RESID
  uint16_t* q;               // QKV
  uint16_t *kc, *vc;         // QKV
  uint16_t* act;             // SWIGLU
  float* logits;             // LOGITS
  int rows, K, nsplit, epi, n_ssq, out_ld;
};
struct VchainParams {
  VtcPhase ph[4];
  int nph, M;
  float* part;
  unsigned* counters;
  unsigned* gbar;            // [4] arrivals of the epilogue warps per phase, zero at launch
  DevStatus* status;
  unsigned spin_limit;
  const float2* rope;
  int n_head, nkv, pos, head_dim, dim;
  float resid, logits_scaling, eps;
  long long* dbg;            // optional: %globaltimer stamps of CTA 0, 16 per phase
};

template <int MT, bool HZ>
__global__ void __launch_bounds__(kTcThreads, 1) v_chain_tc(const VchainParams P) {
  using S = VtcSmem<MT, HZ>;
  constexpr int NRAW = S::NRAW, NS = kTcStages, NACC = S::NACC;
  extern __shared__ __align__(1024) uint8_t tsm_raw[];
  uint8_t* tsm = tsm_raw + ((1024u - (smem_u32(tsm_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tsm + S::BAR);
  uint64_t *raw_full = bars, *raw_empty = bars + NRAW, *a_full = bars + 2 * NRAW, *b_full = a_full + NS, *s_empty = b_full + NS,
           *acc_full = s_empty + NS, *acc_empty = acc_full + NACC, *sc_full = acc_empty + NACC, *sc_empty = sc_full + 2;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(sc_empty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  float* s_rinv = reinterpret_cast<float*>(tsm + S::BAR + 1024);    // [4 phases][64] 1/rms per token
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr bool hz = HZ;
  if (tid == 0) {
    for (int i = 0; i < NRAW; i++) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], 4); }
    for (int i = 0; i < NS; i++) { mbar_init(&a_full[i], 4); mbar_init(&b_full[i], 4); mbar_init(&s_empty[i], 1); }
    for (int i = 0; i < NACC; i++) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    for (int i = 0; i < 2; i++) { mbar_init(&sc_full[i], 1); mbar_init(&sc_empty[i], 4); }
    *s_abort = 0;
    mbar_fence_init();
  }
  constexpr int TCOLS = 512;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(TCOLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;
  WaitCtl wc{P.status, s_abort, P.spin_limit};
#define CH_STAMP(ph, i) do { if (P.dbg && blockIdx.x == 0 && lane == 0) P.dbg[(ph) * 16 + (i)] = (long long)globaltimer_ns(); } while (0)
  const unsigned arrivals = gridDim.x;                                // one arrival per CTA and phase
  volatile int* s_epi = reinterpret_cast<volatile int*>(tsm + S::BAR + 960);      // [0..4) epilogue warps done per phase, [4..8) phase released, [8..12) loader warps done with their slice of the norm sums
  if (tid < 12) s_epi[tid] = 0;
  __syncthreads();

  if (warp == 0) {
    // ---------------- producer: runs ahead through the phases, bounded only by the raw ring
    if (lane == 0) {
      uint32_t gi = 0, ii = 0;
      bool ok = true;
      for (int ph = 0; ph < P.nph && ok; ph++) {
        const VtcPhase& F = P.ph[ph];
        const int K = F.K, G = K / 128;
        const size_t blk_bytes = tc_block_bytes(K, hz);
        for (TcWalk w(F.rows, K, F.nsplit); w.valid() && ok; w.next(), ii++) {
          const uint8_t* blk = F.w + (size_t)w.rb * blk_bytes;
          const int b = ii & 1, ng = w.g1 - w.g0;
          ok = mbar_wait(&sc_empty[b], ((ii >> 1) & 1) ^ 1, wc, W_EMPTY, 1);
          if (!ok) break;
          mbar_expect_tx(&sc_full[b], (uint32_t)ng * 256 * (hz ? 2 : 1));
          bulk_g2s(tsm + S::SC + b * S::SC_BYTES, blk + (size_t)(K / 64) * 4096 + (size_t)w.g0 * 256, ng * 256, &sc_full[b]);
          if (hz)
            bulk_g2s(tsm + S::SC + b * S::SC_BYTES + kTcMaxGroups * 256, blk + (size_t)(K / 64) * 4096 + (size_t)(G + w.g0) * 256,
                     ng * 256, &sc_full[b]);
          for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
            const int s = gi % NRAW;
            ok = mbar_wait(&raw_empty[s], ((gi / NRAW) & 1) ^ 1, wc, W_EMPTY, 2);
            if (!ok) break;
            mbar_expect_tx(&raw_full[s], 8192);
            bulk_g2s(tsm + S::RAW + s * 8192, blk + (size_t)g * 8192, 8192, &raw_full[s]);
          }
        }
      }
      if (*s_abort) {                                            // after a failure: wait (bounded) for the copies in flight
        for (int k = 0; k < NRAW && k < (int)gi; k++) {
          const uint32_t j = gi - 1 - k;
          for (unsigned i = 0; i < wc.limit; i++) {
            if (mbar_try(&raw_full[j % NRAW], (j / NRAW) & 1)) break;
            if ((i & 1023) == 1023) __nanosleep(64);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MT >> 3) << 17) | ((128u >> 4) << 24);
      uint32_t gi = 0;
      bool ok = true;
      for (int ph = 0; ph < P.nph && ok; ph++) {
        const VtcPhase& F = P.ph[ph];
        for (TcWalk w(F.rows, F.K, F.nsplit); w.valid() && ok; w.next()) {
          for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
            const int a = gi % NACC, s = gi % NS;
            ok = mbar_wait(&acc_empty[a], ((gi / NACC) & 1) ^ 1, wc, W_EMPTY, 3) && mbar_wait(&a_full[s], (gi / NS) & 1, wc, W_FULL, 4) &&
                 mbar_wait(&b_full[s], (gi / NS) & 1, wc, W_FULL, 4);
            if (!ok) break;
            tc_fence_after();
            const uint32_t ta = tmem + S::T_A + s * 64, tz = tmem + S::T_AZ + s * 8;
            const uint32_t sb = smem_u32(tsm + S::B + s * S::BSTAGE);
#pragma unroll
            for (int k = 0; k < 8; k++) {
              const uint64_t db = tc_desc(sb + (k >> 2) * (MT * 128) + (k & 3) * 32);
              tc_mma_ts(tmem + a * MT, ta + k * 8, db, idesc, k ? 1u : 0u);
              if (hz) tc_mma_ts(tmem + S::T_ACCZ, tz, db, idesc, (g > w.g0 || k) ? 1u : 0u);
            }
            tc_commit(&s_empty[s]);
            tc_commit(&acc_full[a]);
          }
        }
      }
    }
  } else if (warp < 6) {
    // ---------------- dequantise into tensor memory
    const int quad = warp & 3, row = quad * 32 + lane;
    const uint32_t tl = tmem + ((uint32_t)(quad * 32) << 16);
    uint32_t gi = 0, ii = 0;
    bool ok = true;
    for (int ph = 0; ph < P.nph && ok; ph++) {
      const VtcPhase& F = P.ph[ph];
      for (TcWalk w(F.rows, F.K, F.nsplit); w.valid() && ok; w.next(), ii++) {
        if (hz) ok = mbar_wait(&sc_full[ii & 1], (ii >> 1) & 1, wc, W_FULL, 7);
        for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
          const int sr = gi % NRAW, s = gi % NS;
          ok = mbar_wait(&raw_full[sr], (gi / NRAW) & 1, wc, W_FULL, 5) && mbar_wait(&s_empty[s], ((gi / NS) & 1) ^ 1, wc, W_EMPTY, 6);
          if (!ok) break;
          tc_fence_after();
          const uint32_t raw = smem_u32(tsm + S::RAW + sr * 8192) + (uint32_t)row * 4;
#pragma unroll
          for (int c = 0; c < 2; c++) {
            uint32_t v[32];
#pragma unroll
            for (int q8 = 0; q8 < 8; q8++) {
              const uint32_t wv = lds32(raw + c * 4096 + q8 * 512);
              v[4 * q8] = tc_cvt_lo(wv); v[4 * q8 + 1] = tc_cvt_hi(wv); v[4 * q8 + 2] = tc_cvt_lo(wv >> 8); v[4 * q8 + 3] = tc_cvt_hi(wv >> 8);
            }
            tc_st32(tl + S::T_A + s * 64 + c * 32, v);
          }
          if (hz) {
            const uint16_t z = reinterpret_cast<const uint16_t*>(tsm + S::SC + (ii & 1) * S::SC_BYTES + kTcMaxGroups * 256)[(g - w.g0) * 128 + row];
            tc_st8(tl + S::T_AZ + s * 8, (uint32_t)z | ((uint32_t)z << 16));
          }
          tc_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) { mbar_arrive(&raw_empty[sr]); mbar_arrive(&a_full[s]); }
        }
      }
    }
  } else if (warp < 10) {
    // ---------------- activations, phase by phase. A phase's activations exist only once every epilogue warp of the grid
    // has finished the previous phase, so the cp.async pipeline (three groups ahead) restarts at every phase boundary:
    // wait for the grid-wide arrival counter (bounded), prepare 1/rms, prime, then stream.
    const int lt = (warp - 6) * 32 + lane;
    constexpr int PIECES = MT * 16, PPT = (PIECES + 127) / 128, AHEAD = NS - 1;
    bool ok = true;
    uint32_t gi = 0;                                             // groups of this CTA so far, all phases (stage = gi % NS)
    for (int ph = 0; ph < P.nph && ok; ph++) {
      const VtcPhase& F = P.ph[ph];
      if (ph > 0) {                                              // every CTA of the grid has finished phase ph-1
        // one lane of the CTA polls the global counter (with a pause: 148 pollers on one line must not starve the
        // arrivals), the other loader warps watch a shared-memory flag
        if (lane == 0) {
          bool seen = false;
          for (unsigned i = 0; i < wc.limit; i++) {
            if (warp == 6) {
              unsigned v;
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(P.gbar + (ph - 1)) : "memory");
              if (v >= arrivals) { s_epi[4 + ph] = 1; seen = true; break; }
              __nanosleep(200);
            } else if (s_epi[4 + ph]) { seen = true; break; }
            if ((i & 15) == 15 && (*wc.s_abort || ld_volatile_s32(&wc.st->abort))) { *wc.s_abort = 1; break; }
          }
          if (!seen && *wc.s_abort == 0) report_fail(wc, W_FLAG, ph, (int)arrivals, -5);
          __threadfence();
        }
        __syncwarp();
        if (*wc.s_abort) { ok = false; break; }
      }
      if (warp == 6) CH_STAMP(ph, 0);
      float* rinv = s_rinv + ph * 64;
      if (F.norm_w) {
        // 1/rms per token from the partial sums, in a fixed order. The partials are independent L2 loads: the 128 loader
        // threads split them (thread = token x slice of the partials, many loads in flight each), meet in shared memory
        // (the epilogue staging area is idle between phases) and every warp adds the slices in slice order.
        constexpr int NSL = 128 / MT;
        float* sl = reinterpret_cast<float*>(tsm + S::EPI);
        const int m0 = lt % MT, slice = lt / MT, per = (F.n_ssq + NSL - 1) / NSL;
        if (m0 < P.M) {
          const int i0 = slice * per, i1 = min(F.n_ssq, i0 + per);
          float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
          int i = i0;
          for (; i + 4 <= i1; i += 4) {
            const float v0 = __ldcg(F.ssq_in + (size_t)i * 64 + m0), v1 = __ldcg(F.ssq_in + (size_t)(i + 1) * 64 + m0),
                        v2 = __ldcg(F.ssq_in + (size_t)(i + 2) * 64 + m0), v3 = __ldcg(F.ssq_in + (size_t)(i + 3) * 64 + m0);
            a0 += v0; a1 += v1; a2 += v2; a3 += v3;
          }
          for (; i < i1; i++) a0 += __ldcg(F.ssq_in + (size_t)i * 64 + m0);
          sl[slice * 64 + m0] = (a0 + a1) + (a2 + a3);
        }
        __threadfence_block();
        __syncwarp();
        if (lane == 0) {
          atomicAdd(const_cast<int*>(s_epi + 8 + ph), 1);
          bool seen = false;
          for (unsigned i = 0; i < wc.limit; i++) {
            if (s_epi[8 + ph] >= 4) { seen = true; break; }
            if ((i & 63) == 63 && *wc.s_abort) break;
          }
          if (!seen && *wc.s_abort == 0) report_fail(wc, W_FLAG, ph, 4, -6);
        }
        __syncwarp();
        if (*wc.s_abort) { ok = false; break; }
        __threadfence_block();
        for (int m = lane; m < P.M; m += 32) {
          float ss = 0.f;
#pragma unroll
          for (int q = 0; q < NSL; q++) ss += sl[q * 64 + m];
          rinv[m] = 1.0f / sqrtf(ss / (float)P.dim + P.eps);
        }
        __syncwarp();
      }
      if (warp == 6) CH_STAMP(ph, 1);
      TcWalk wi(F.rows, F.K, F.nsplit);                          // issue-side cursor of this phase
      int gn = wi.valid() ? wi.g0 : 0;
      uint32_t gii = gi;
      auto issue_next = [&]() {
        if (ok && wi.valid()) {
          const int s = gii % NS;
          ok = mbar_wait(&s_empty[s], ((gii / NS) & 1) ^ 1, wc, W_EMPTY, 8);
          if (ok) {
            uint8_t* dst = tsm + S::B + s * S::BSTAGE;
#pragma unroll
            for (int k = 0; k < PPT; k++) {
              const int i = lt + k * 128;
              if (i < PIECES) {
                const int c = i & 7, m = (i >> 3) % MT, tile = i / (8 * MT);
                uint8_t* d = dst + tile * (MT * 128) + (m >> 3) * 1024 + (m & 7) * 128 + ((c ^ (m & 7)) << 4);
                if (m < P.M) cp_async16(d, F.x + (size_t)m * F.K + gn * 128 + tile * 64 + c * 8);
                else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
              }
            }
          }
          gii++;
          if (++gn >= wi.g1) { wi.next(); gn = wi.valid() ? wi.g0 : 0; }
        }
        cp_async_commit();
      };
      for (int j = 0; j < AHEAD; j++) issue_next();
      for (TcWalk w(F.rows, F.K, F.nsplit); w.valid() && ok; w.next()) {
        for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
          cp_async_wait<AHEAD - 1>();
          if (F.norm_w) {
            // normalise this thread's own pieces in place: bf16((float(h) * r) * float(w))
            uint8_t* dst = tsm + S::B + (gi % NS) * S::BSTAGE;
#pragma unroll
            for (int k = 0; k < PPT; k++) {
              const int i = lt + k * 128;
              if (i < PIECES) {
                const int c = i & 7, m = (i >> 3) % MT, tile = i / (8 * MT);
                if (m < P.M) {
                  uint4* d = reinterpret_cast<uint4*>(dst + tile * (MT * 128) + (m >> 3) * 1024 + (m & 7) * 128 + ((c ^ (m & 7)) << 4));
                  const int col = g * 128 + tile * 64 + c * 8;
                  const uint4 hv = *d, wv = __ldg(reinterpret_cast<const uint4*>(F.norm_w + col));
                  const float r = rinv[m];
                  const uint32_t hh[4] = {hv.x, hv.y, hv.z, hv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
                  uint32_t o[4];
#pragma unroll
                  for (int e = 0; e < 4; e++)
                    o[e] = (uint32_t)f2bf(bflo(hh[e]) * r * bflo(ww[e])) | ((uint32_t)f2bf(bfhi(hh[e]) * r * bfhi(ww[e])) << 16);
                  const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
                  *d = ov;
                  if (F.xn_out && w.rb == 0) *reinterpret_cast<uint4*>(F.xn_out + (size_t)m * F.K + col) = ov;
                }
              }
            }
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&b_full[gi % NS]);
          if (warp == 6 && g == w.g0) CH_STAMP(ph, 2);
          issue_next();
        }
      }
      cp_async_wait<0>();
      if (warp == 6) CH_STAMP(ph, 3);
    }
  } else {
    // ---------------- epilogue
    const int quad = warp & 3, row = quad * 32 + lane;
    const uint32_t tlane = tmem + ((uint32_t)(quad * 32) << 16);
    uint32_t gi = 0, ii = 0;
    bool ok = true;
    for (int ph = 0; ph < P.nph && ok; ph++) {
      const VtcPhase& F = P.ph[ph];
      for (TcWalk w(F.rows, F.K, F.nsplit); w.valid() && ok; w.next(), ii++) {
        float y[MT];
#pragma unroll
        for (int t = 0; t < MT; t++) y[t] = 0.f;
        const int b = ii & 1;
        ok = mbar_wait(&sc_full[b], (ii >> 1) & 1, wc, W_FULL, 9);
        const uint16_t* scs = reinterpret_cast<const uint16_t*>(tsm + S::SC + b * S::SC_BYTES);
        for (int g = w.g0; g < w.g1 && ok; g++, gi++) {
          const int a = gi % NACC;
          ok = mbar_wait(&acc_full[a], (gi / NACC) & 1, wc, W_FULL, 10);
          if (!ok) break;
          tc_fence_after();
          const float s64 = bf2f(scs[(g - w.g0) * 128 + row]) * 64.0f;
          constexpr int HALF = MT >= 32 ? 32 : MT;
#pragma unroll
          for (int h0 = 0; h0 < MT; h0 += HALF) {
            uint32_t v[HALF / 8][8];
#pragma unroll
            for (int c8 = 0; c8 < HALF / 8; c8++) tc_ld8(tlane + a * MT + h0 + c8 * 8, v[c8]);
            tc_ld_wait();
#pragma unroll
            for (int c8 = 0; c8 < HALF / 8; c8++)
#pragma unroll
              for (int e = 0; e < 8; e++) y[h0 + c8 * 8 + e] = fmaf(s64, __uint_as_float(v[c8][e]), y[h0 + c8 * 8 + e]);
          }
          if (hz && g == w.g1 - 1) {
#pragma unroll
            for (int c8 = 0; c8 < MT / 8; c8++) {
              uint32_t v[8];
              tc_ld8(tlane + S::T_ACCZ + c8 * 8, v);
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
        if (warp == 10) CH_STAMP(ph, 4);
        if (F.nsplit > 1) {
          float* mine = P.part + (size_t)w.item * MT * 128;
#pragma unroll
          for (int t = 0; t < MT; t++) mine[t * 128 + row] = y[t];
          __threadfence();
          __syncwarp();
          unsigned old = 0;
          if (lane == 0) {
            old = atomicAdd(P.counters + w.rb * 4 + quad, 1u);
            if (old == (unsigned)F.nsplit - 1u) P.counters[w.rb * 4 + quad] = 0u;
          }
          old = __shfl_sync(0xffffffffu, old, 0);
          if (old != (unsigned)F.nsplit - 1u) continue;
          __threadfence();
#pragma unroll
          for (int t = 0; t < MT; t++) y[t] = 0.f;
          for (int sp = 0; sp < F.nsplit; sp++) {
            const float* src = P.part + (size_t)(w.rb * F.nsplit + sp) * MT * 128;
#pragma unroll
            for (int t = 0; t < MT; t++) y[t] += __ldcg(src + t * 128 + row);
          }
        }
        if (warp == 10) CH_STAMP(ph, 5);
        float* ys = reinterpret_cast<float*>(tsm + S::EPI);
        __syncwarp();
#pragma unroll
        for (int t = 0; t < MT; t++) ys[t * 128 + row] = y[t];
        __syncwarp();
        const int srow = w.rb * 128 + row;
        const bool live = srow < F.rows;
        if (F.epi == EPI_RESID) {
          for (int t0 = 0; t0 < P.M; t0 += 8) {
            uint16_t hv[8];
#pragma unroll
            for (int e = 0; e < 8; e++) hv[e] = (live && t0 + e < P.M) ? F.h[(size_t)(t0 + e) * F.out_ld + srow] : (uint16_t)0;
#pragma unroll
            for (int e = 0; e < 8; e++) {
              const int t = t0 + e;                               // warp-uniform
              if (t < P.M) {
                const float hn = live ? rbf(bf2f(hv[e]) + ys[t * 128 + row] * P.resid) : 0.f;
                if (live) F.h[(size_t)t * F.out_ld + srow] = f2bf(hn);
                if (F.ssq_out) {                                  // the 32 rows' share of sum(h^2) of token t
                  float sq = hn * hn;
#pragma unroll
                  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                  if (lane == 0) F.ssq_out[(size_t)(w.rb * 4 + quad) * 64 + t] = sq;
                }
              }
            }
          }
        } else if (F.epi == EPI_LOGITS) {
          if (live)
#pragma unroll 4
            for (int t = 0; t < P.M; t++) F.logits[(size_t)t * F.out_ld + srow] = ys[t * 128 + row] / P.logits_scaling;
        } else if (F.epi == EPI_SWIGLU) {
          if (!(lane & 1) && live)
#pragma unroll 4
            for (int t = 0; t < P.M; t++) {
              const float gg = rbf(ys[t * 128 + row]), uu = rbf(ys[t * 128 + row + 1]);
              F.act[(size_t)t * F.out_ld + (srow >> 1)] = f2bf((gg / (1.0f + __expf(-gg))) * uu);
            }
        } else {
          const int HD = P.head_dim, HP = HD >> 1, QD = P.n_head * HD;
          const int head = srow / HD, within = srow % HD, i = within >> 1;
          if (!(lane & 1) && live) {
            if (head < P.n_head + P.nkv) {
              for (int t0 = 0; t0 < P.M; t0 += 8) {
                float2 cs[8];
#pragma unroll
                for (int e = 0; e < 8; e++) cs[e] = t0 + e < P.M ? __ldg(P.rope + (size_t)(t0 + e) * HP + i) : make_float2(1.f, 0.f);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                  const int t = t0 + e;
                  if (t < P.M) {
                    const float x0 = rbf(ys[t * 128 + row]), x1 = rbf(ys[t * 128 + row + 1]);
                    const uint16_t y0 = f2bf(x0 * cs[e].x - x1 * cs[e].y), y1 = f2bf(x1 * cs[e].x + x0 * cs[e].y);
                    if (head < P.n_head) {
                      F.q[(size_t)t * QD + head * HD + i] = y0;
                      F.q[(size_t)t * QD + head * HD + i + HP] = y1;
                    } else {
                      uint16_t* kr = F.kc + ((size_t)(P.pos + t) * P.nkv + (head - P.n_head)) * HD;
                      kr[i] = y0;
                      kr[i + HP] = y1;
                    }
                  }
                }
              }
            } else {
#pragma unroll 4
              for (int t = 0; t < P.M; t++) {
                uint16_t* vr = F.vc + ((size_t)(P.pos + t) * P.nkv + (head - P.n_head - P.nkv)) * HD;
                *reinterpret_cast<uint32_t*>(vr + within) = (uint32_t)f2bf(ys[t * 128 + row]) | ((uint32_t)f2bf(ys[t * 128 + row + 1]) << 16);
              }
            }
          }
        }
        __syncwarp();
      }
      if (warp == 10) CH_STAMP(ph, 6);
      // this warp's results of the phase are in global memory: tell the grid (the loaders of the next phase wait for it)
      __threadfence();
      __syncwarp();
      if (lane == 0 && ph + 1 < P.nph) {                         // the CTA's last epilogue warp arrives for the CTA
        if (atomicAdd(const_cast<int*>(s_epi + ph), 1) == 3) {
          __threadfence();
          atomicAdd(P.gbar + ph, 1u);
        }
      }
      if (warp == 10) CH_STAMP(ph, 7);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TCOLS));
}

}  // namespace fb
