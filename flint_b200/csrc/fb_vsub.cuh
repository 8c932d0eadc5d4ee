// Verify GEMM for small trees (up to 26 tokens): int4 weights enter the tensor pipe as fp16 SUBNORMALS, exactly as in
// the decode kernel, so no instruction is spent on dequantisation: a weight word is split by four masks into the A
// fragment of one mma.m16n8k16, the tokens are the B columns (8 per MMA), and scales, the nibble offset and the
// activations' power-of-two factors are applied once per group of 128 columns to the fp32 partial sums.
//
// Weights live in a third, library-owned copy ("R32 layout"): tiles of 32 stream rows (the decode kernel's row order:
// RoPE pairs and gate/up pairs adjacent), cut along K into units of `ug` groups. A unit is what one bulk copy brings
// and one warp multiplies: for every 4 MMA steps and each 16-row half a block [32 lanes][4 words] (one 128-bit load
// per lane), then the unit's scales bf16 [ug][32 rows].
//
// One CTA per SM, persistent. A producer lane streams the CTA's units into a ring whose stages are owned one-to-one
// by consumer warps: warp (slot, u) multiplies unit u of the tile in flight on `slot`, the `upi` warps of a slot meet
// through their (consumed) stage buffers, add their partial sums in unit order and share the epilogue. The tokens'
// activations (all of K, or this CTA's K slice when K is split over CTAs) are copied into shared memory and converted
// there to fp16 in B-operand order with one power-of-two factor per (token, group); the QKV and gate/up GEMMs apply the
// RMSNorm on the way, so no norm kernel runs between GEMMs. K slices of different CTAs meet in global memory;
// the CTA that arrives last adds the partials in slice order, so results do not depend on timing.
#pragma once
#include "fb_verify.cuh"

namespace fb {

constexpr int kVsWarps = 12;                  // consumer warps; warp 12 is the producer
constexpr int kVsThreads = (kVsWarps + 1) * 32;
constexpr int kVsSmem = 227 * 1024;
constexpr int kVsMaxTokens = 26;
constexpr int kVsCounters = 16384;            // arrival counters of K-split GEMMs: 8 per tile

__host__ __device__ constexpr int vs_unit_bytes(int ug) { return ug * 2112; }        // 32 rows x 128 ug nibbles + scales
__host__ __device__ constexpr size_t vs_matrix_bytes(int rows, int k) {
  return (size_t)((rows + 31) / 32) * (size_t)(k / 128) * 2112;
}

struct VsPlan {
  int ok, ug, upi, nkc, nslot, kcg;           // groups per unit, units per item, K slices, tiles in flight, groups per slice
  int xs, acts_off, f_off, bar_off;           // activation row stride (bytes) and shared-memory offsets
};

// Geometry of one launch. K is cut into as few CTA slices as let the activations of a slice (for the largest tree), their
// factors and a ring of at least two tiles share the SM's shared memory; the unit size follows from K alone, so the
// weight copy does not depend on the tree. Smaller trees get a deeper ring.
__host__ __device__ inline VsPlan vs_plan(int K, int M, int tiles) {
  VsPlan p = {};
  if (K % 128 != 0 || M < 1 || M > kVsMaxTokens) return p;
  const int G = K / 128;
  for (int nkc = 1; nkc <= 16; nkc++) {
    if (G % nkc) continue;
    const int kcg = G / nkc;
    int ug = 0;
    for (int c = 5; c >= 2; c--)
      if (kcg % c == 0) { ug = c; break; }
    if (!ug) continue;
    const int upi = kcg / ug;
    if (upi > 6) continue;
    if (nkc > 1 && tiles * 8 > kVsCounters) continue;
    const int xs = kcg * 256 + 32;
    if ((kVsSmem - (kVsMaxTokens * (xs + kcg * 16 + 16) + 1024)) / (upi * vs_unit_bytes(ug)) < 2) continue;
    int nslot = (kVsSmem - (M * (xs + kcg * 16 + 16) + 1024)) / (upi * vs_unit_bytes(ug));
    if (nslot > kVsWarps / upi) nslot = kVsWarps / upi;
    p.ok = 1; p.ug = ug; p.upi = upi; p.nkc = nkc; p.nslot = nslot; p.kcg = kcg; p.xs = xs;
    p.acts_off = nslot * upi * vs_unit_bytes(ug);
    p.f_off = p.acts_off + M * xs;
    p.bar_off = p.f_off + M * (kcg * 16 + 16);             // factor rows are padded by 16 bytes: conflict-free reads
    return p;
  }
  return p;
}

// caller layout (word c of a row = columns 8c .. 8c+7, column 8c+m in bits [4m, 4m+4)) -> R32 layout.
// grid (tiles of 32 rows, layers), 256 threads; `ug` = groups per unit of this matrix.
__global__ void vs_repack(const uint32_t* q, const uint16_t* sc, int rows, int K, int ug, int order, int order_arg,
                          int order_rows, uint8_t* out) {
  const int T = blockIdx.x, ntile = gridDim.x, G = K / 128, nu = G / ug, ub = vs_unit_bytes(ug);
  uint8_t* tile = out + ((size_t)blockIdx.y * ntile + T) * (size_t)nu * ub;
  __shared__ int src_row[32];
  if (threadIdx.x < 32) {
    const int j = T * 32 + threadIdx.x;
    src_row[threadIdx.x] = j < rows ? (int)blockIdx.y * rows + perm_row(j, order, order_arg, order_rows) : -1;
  }
  __syncthreads();
  auto nib = [&](int r, int col) -> uint32_t {
    const int row = src_row[r];
    if (row < 0) return 8u;
    return (__ldg(q + (size_t)row * (K / 8) + (col >> 3)) >> (4 * (col & 7))) & 15u;
  };
  const int words_per_unit = ug * 512;                       // ug groups x 8 steps x 2 halves x 32 lanes
  for (int wi = threadIdx.x; wi < nu * words_per_unit; wi += blockDim.x) {
    const int u = wi / words_per_unit, r = wi % words_per_unit;
    const int i = r & 3, lane = (r >> 2) & 31, hb = r >> 7, h = hb & 1, b = hb >> 1;
    const int g = lane >> 2, t = lane & 3;
    const int col0 = (u * ug * 8 + 4 * b + i) * 16, rl = 16 * h + g, rh = rl + 8;
    const uint32_t w = nib(rl, col0 + 2 * t) | nib(rh, col0 + 2 * t) << 4 | nib(rl, col0 + 2 * t + 8) << 8 |
                       nib(rh, col0 + 2 * t + 8) << 12 | nib(rl, col0 + 2 * t + 1) << 16 | nib(rh, col0 + 2 * t + 1) << 20 |
                       nib(rl, col0 + 2 * t + 9) << 24 | nib(rh, col0 + 2 * t + 9) << 28;
    reinterpret_cast<uint32_t*>(tile + (size_t)u * ub)[r] = w;
  }
  for (int i = threadIdx.x; i < G * 32; i += blockDim.x) {
    const int r = i & 31, grp = i >> 5, u = grp / ug, gl = grp % ug, row = src_row[r];
    reinterpret_cast<uint16_t*>(tile + (size_t)u * ub + ug * 2048)[gl * 32 + r] = row >= 0 ? sc[(size_t)row * G + grp] : 0;
  }
}

struct VsubParams {
  const uint8_t* w;          // R32 layout of this matrix (layer offset applied)
  const uint16_t* x;         // bf16 [>= M][K], B-operand order inside every 16 columns; with norm_w: the residual rows in
                             // natural order, normalised while they are staged (K not split over CTAs)
  const uint16_t* norm_w;    // RMSNorm weight bf16 [K] or NULL
  float eps;
  int rows, K, M;
  VsPlan plan;
  float* part;               // K-split partial sums
  int* counters;             // [tiles][8], zero between launches
  DevStatus* status;
  unsigned spin_limit;
  // epilogue operands (as in VGemmParams)
  uint16_t* h;
  uint16_t* q;
  uint16_t *kc, *vc;
  uint16_t* act_t;
  float* logits;
  const float2* rope;        // [M][head_dim / 2] (cos, sin)
  int n_head, nkv, pos, head_dim, out_ld;
  float resid, logits_scaling;
  long long* dbg;            // 8 %globaltimer stamps of CTA 0 (NULL = off)
};

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float4 ld_cg_f4(const float4* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t vmaxu2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Bring this CTA's K slice of every token into shared memory (asynchronous 16-byte copies; every CTA copies the same rows,
// so each starts at a different 128-byte line and they do not walk L2 in lockstep), then convert it in place to fp16 in
// B-operand order with one power of two m per (token, group of 128): x * m has its largest magnitude in [2^14, 2^15).
// xf = {2^24 / m, 2^20 / m, -8 * sum x, sum x} per (token, group). A lane converts one block of 16 columns (the unit of the
// B-order permutation), eight lanes a group, a warp four groups at a time. With a norm weight the rows are the residual
// stream in natural order and xn = bf16((float(h) * r) * float(w)) is formed on the way. Ends with a consumer barrier.
__device__ __forceinline__ void vs_stage_acts(const VsubParams& P, int kc, uint8_t* acts, float4* xf, float* rinv, int tid,
                                              int warp, int lane) {
  const VsPlan& pl = P.plan;
  const bool norm = P.norm_w != nullptr;
  const int ppr = pl.kcg * 16, npiece = P.M * ppr;          // 16-byte pieces per token row
  const int rot = (int)(((long long)blockIdx.x * (npiece / 8)) / gridDim.x) * 8;
  for (int i0 = tid; i0 < npiece; i0 += kVsWarps * 32) {
    const int i = i0 + rot < npiece ? i0 + rot : i0 + rot - npiece;
    const int m = i / ppr, c = i % ppr;
    cp_async16(acts + (size_t)m * pl.xs + c * 16, P.x + (size_t)m * P.K + (size_t)kc * pl.kcg * 128 + c * 8);
  }
  cp_async_commit();
  cp_async_wait<0>();
  named_bar_sync(7, kVsWarps * 32);
  if (norm) {                                               // 1 / rms of every token (K is not split: the row is whole)
    for (int m = warp; m < P.M; m += kVsWarps) {
      float ss = 0.f;
      for (int c = lane; c < ppr; c += 32) {
        const uint4 v = *reinterpret_cast<const uint4*>(acts + (size_t)m * pl.xs + c * 16);
        const uint32_t p[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; e++) { ss = fmaf(bflo(p[e]), bflo(p[e]), ss); ss = fmaf(bfhi(p[e]), bfhi(p[e]), ss); }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) rinv[m] = 1.0f / sqrtf(ss / (float)P.K + P.eps);
    }
    named_bar_sync(7, kVsWarps * 32);
  }
  const int qpr = (pl.kcg + 3) / 4, nquad = P.M * qpr;      // quads of groups per token row
  const int sg = lane >> 3, sl = lane & 7;
  for (int qi = warp; qi < nquad; qi += kVsWarps) {
    const int m = qi / qpr, grp = (qi % qpr) * 4 + sg;
    const bool valid = grp < pl.kcg;
    uint8_t* cell = acts + (size_t)m * pl.xs + (size_t)(valid ? grp : 0) * 256 + sl * 32;
    const uint4 v0 = *reinterpret_cast<const uint4*>(cell), v1 = *reinterpret_cast<const uint4*>(cell + 16);
    uint32_t p[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};       // pairs, in storage order
    if (norm) {
      const float r = rinv[m];
      const uint4* wp = reinterpret_cast<const uint4*>(P.norm_w + (size_t)(valid ? grp : 0) * 128 + sl * 16);
      const uint4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
      const uint32_t q[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      uint32_t n[8];
#pragma unroll
      for (int e = 0; e < 8; e++)
        n[e] = (uint32_t)f2bf(bflo(p[e]) * r * bflo(q[e])) | ((uint32_t)f2bf(bfhi(p[e]) * r * bfhi(q[e])) << 16);
      // natural pair k = columns (2k, 2k+1) of the block goes to B-order slot 2k (k < 4) or 2(k - 4) + 1
#pragma unroll
      for (int e = 0; e < 4; e++) { p[2 * e] = n[e]; p[2 * e + 1] = n[e + 4]; }
    }
    uint32_t em = 0;
    float sx = 0.f;
#pragma unroll
    for (int e = 0; e < 8; e++) {
      em = vmaxu2(em, p[e] & 0x7F807F80u);
      sx += bflo(p[e]) + bfhi(p[e]);
    }
    em = max(em & 0xFFFFu, em >> 16) >> 7;                  // largest exponent field of the lane's 16 values
    if (!valid) { em = 0; sx = 0.f; }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {                       // the group's eight lanes
      em = max(em, __shfl_xor_sync(0xffffffffu, em, o));
      sx += __shfl_xor_sync(0xffffffffu, sx, o);
    }
    if (valid) {
      uint32_t mf = 268u - em;
      mf = mf > 253u ? 253u : (mf < 24u ? 24u : mf);
      const float mult = __uint_as_float(mf << 23), inv = __uint_as_float((254u - mf) << 23);
      uint32_t hq[8];
#pragma unroll
      for (int e = 0; e < 8; e++) {
        const __half2 hh = __floats2half2_rn(bflo(p[e]) * mult, bfhi(p[e]) * mult);
        hq[e] = *reinterpret_cast<const uint32_t*>(&hh);
      }
      *reinterpret_cast<uint4*>(cell) = make_uint4(hq[0], hq[1], hq[2], hq[3]);
      *reinterpret_cast<uint4*>(cell + 16) = make_uint4(hq[4], hq[5], hq[6], hq[7]);
      if (sl == 0) xf[m * (pl.kcg + 1) + grp] = make_float4(inv * 16777216.f, inv * 1048576.f, -8.f * sx, sx);
    }
  }
  named_bar_sync(7, kVsWarps * 32);
}

// Epilogue of one C fragment: v = {row r0: tokens m0, m0+1; row r0+8: tokens m0, m0+1}, r0 = tile row of lane group g.
// The whole warp calls this together (row pairs are exchanged between neighbouring lane groups).
template <int EPI>
__device__ __forceinline__ void vs_epilogue(const VsubParams& P, int row_base, int j, float4 v, int lane) {
  const int g = lane >> 2, t = lane & 3;
  if (EPI == EPI_RESID || EPI == EPI_LOGITS) {
    const float val[4] = {v.x, v.y, v.z, v.w};
    uint16_t old[4] = {0, 0, 0, 0};
    if (EPI == EPI_RESID) {                               // all four reads are in flight before the first write
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int r = row_base + g + (e >> 1) * 8, m = j * 8 + 2 * t + (e & 1);
        if (r < P.rows && m < P.M) old[e] = ld_cg_u16(P.h + (size_t)m * P.out_ld + r);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int r = row_base + g + (e >> 1) * 8, m = j * 8 + 2 * t + (e & 1);
      if (r < P.rows && m < P.M) {
        if (EPI == EPI_RESID) P.h[(size_t)m * P.out_ld + r] = f2bf(bf2f(old[e]) + val[e] * P.resid);
        else P.logits[(size_t)m * P.out_ld + r] = val[e] / P.logits_scaling;
      }
    }
  } else {
    // stream rows (2p, 2p+1) sit in lane groups (g even, g odd): the even group takes token m0, the odd one m0 + 1
    const int e = g & 1, m = j * 8 + 2 * t + e;
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
      const float own0 = hi ? v.z : v.x, own1 = hi ? v.w : v.y;
      const float recv = __shfl_xor_sync(0xffffffffu, e ? own0 : own1, 4);
      const float a0 = e ? recv : own0, a1 = e ? own1 : recv;          // values of rows rs, rs + 1 for token m
      const int rs = row_base + (g & ~1) + hi * 8;
      if (rs < P.rows && m < P.M) {
        if (EPI == EPI_SWIGLU) {
          const float gg = rbf(a0), uu = rbf(a1);
          P.act_t[(size_t)m * P.out_ld + k16_pos(rs >> 1)] = f2bf((gg / (1.0f + __expf(-gg))) * uu);
        } else {   // EPI_QKV: rows (2p, 2p+1) of a head are dims (p, p + HD/2); V rows keep their order
          const int HD = P.head_dim, HP = HD >> 1, QD = P.n_head * HD;
          const int head = rs / HD, within = rs % HD;
          if (head < P.n_head + P.nkv) {
            const int i = within >> 1;
            const float x0 = rbf(a0), x1 = rbf(a1);
            const float2 cs = __ldg(P.rope + (size_t)m * HP + i);
            const uint16_t y0 = f2bf(x0 * cs.x - x1 * cs.y), y1 = f2bf(x1 * cs.x + x0 * cs.y);
            if (head < P.n_head) {
              P.q[(size_t)m * QD + head * HD + i] = y0;
              P.q[(size_t)m * QD + head * HD + i + HP] = y1;
            } else {
              uint16_t* kr = P.kc + ((size_t)(P.pos + m) * P.nkv + (head - P.n_head)) * HD;
              kr[i] = y0;
              kr[i + HP] = y1;
            }
          } else {
            uint16_t* vr = P.vc + ((size_t)(P.pos + m) * P.nkv + (head - P.n_head - P.nkv)) * HD;
            vr[within] = f2bf(a0);
            vr[within + 1] = f2bf(a1);
          }
        }
      }
    }
  }
}

#define VS_STAMP(i) do { if (P.dbg && blockIdx.x == 0 && tid == 0) P.dbg[i] = (long long)globaltimer_ns(); } while (0)
template <int NT, int EPI>
__global__ void __launch_bounds__(kVsThreads, 1) v_gemm_sub(const VsubParams P) {
  extern __shared__ __align__(128) uint8_t vsm[];
  const VsPlan& pl = P.plan;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int ub = vs_unit_bytes(pl.ug), nst = pl.nslot * pl.upi;
  uint8_t* acts = vsm + pl.acts_off;
  float4* xf = reinterpret_cast<float4*>(vsm + pl.f_off);
  uint64_t* full = reinterpret_cast<uint64_t*>(vsm + pl.bar_off);
  uint64_t* empty = full + 16;
  volatile int* s_abort = reinterpret_cast<volatile int*>(vsm + pl.bar_off + 256);
  volatile int* s_prog = reinterpret_cast<volatile int*>(vsm + pl.bar_off + 264);
  if (tid == 0) {
    for (int s = 0; s < nst; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    *s_abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_trigger();
  WaitCtl wc{P.status, s_abort, P.spin_limit};
  // this CTA's K slice and its share of the tiles
  const int ntile = (P.rows + 31) / 32, G = (int)gridDim.x, b = (int)blockIdx.x;
  const int kc = b % pl.nkc, gi = b / pl.nkc, ng = (G - kc + pl.nkc - 1) / pl.nkc;
  const int t0 = (int)(((long long)ntile * gi) / ng), t1 = (int)(((long long)ntile * (gi + 1)) / ng);
  const int nitems = t1 - t0;
  const int nu_total = (P.K / 128) / pl.ug;                  // units per tile in global memory

  if (warp == kVsWarps) {
    // ------------------------------------------------------------ producer: weights do not depend on the previous kernel
    if (lane == 0) {
      int i = 0, u = 0;
      bool ok = true;
      for (i = 0; i < nitems && ok; i++) {
        const int slot = i % pl.nslot, k = i / pl.nslot;
        for (u = 0; u < pl.upi; u++) {
          const int s = slot * pl.upi + u;
          if (!mbar_wait(&empty[s], (k & 1) ^ 1, wc, W_EMPTY, i)) { ok = false; break; }
          mbar_expect_tx(&full[s], (uint32_t)ub);
          bulk_g2s(vsm + (size_t)s * ub, P.w + ((size_t)(t0 + i) * nu_total + (size_t)kc * pl.upi + u) * ub, (uint32_t)ub, &full[s]);
        }
      }
      // what was issued: a failed launch waits for it below before the CTA exits
      s_prog[0] = ok ? nitems : i - 1;                        // items whose units were all issued (the loop's
      s_prog[1] = ok ? 0 : u;                                 // increment ran before `ok` was tested)
    }
  } else {
    // ------------------------------------------------------------ consumers
    VS_STAMP(0);
    pdl_wait();
    VS_STAMP(1);
    vs_stage_acts(P, kc, acts, xf, reinterpret_cast<float*>(vsm + pl.bar_off + 384), tid, warp, lane);
    VS_STAMP(2);
    if (warp < nst) {
      const int slot = warp / pl.upi, u = warp % pl.upi;
      uint8_t* stage = vsm + (size_t)warp * ub;
      const uint32_t sb = smem_u32(stage);
      const uint32_t wa = sb + (uint32_t)lane * 16;
      const uint32_t sca = sb + (uint32_t)pl.ug * 2048 + (uint32_t)g * 2;
      // B fragments: token rows of the n-tiles (rows beyond M repeat the last token; their results are never written)
      uint32_t xa[NT], fa[NT][2];
#pragma unroll
      for (int j = 0; j < NT; j++) {
        const int mb = min(j * 8 + g, P.M - 1);
        xa[j] = smem_u32(acts) + (uint32_t)mb * pl.xs + (uint32_t)(u * pl.ug * 128 + 4 * t) * 2;
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const int mc = min(j * 8 + 2 * t + e, P.M - 1);
          fa[j][e] = smem_u32(xf) + (uint32_t)(mc * (pl.kcg + 1) + u * pl.ug) * 16;
        }
      }
      bool alive = true;
      for (int i = slot, k = 0; i < nitems; i += pl.nslot, k++) {
        float ct[2][NT][4];
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
          for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) ct[h][j][e] = 0.f;
        if (alive && !mbar_wait(&full[warp], k & 1, wc, W_FULL, i)) alive = false;
        if (k == 0) VS_STAMP(3);
        if (alive) {
          // Loads run one step (activations) and one block of 4 steps (weights) ahead of the MMAs that use them.
          // (the look-ahead of the last step / block reads the row's pad bytes / the bytes after the nibbles: unused)
          uint4 wc0 = lds128(wa), wc1 = lds128(wa + 512);
          uint2 bcur[NT];
#pragma unroll
          for (int j = 0; j < NT; j++) bcur[j] = lds64(xa[j]);
          for (int grp = 0; grp < pl.ug; grp++) {
            float cg[2][NT][4];
#pragma unroll
            for (int bq = 0; bq < 2; bq++) {
              const uint32_t nb = (uint32_t)(grp * 2 + bq + 1) * 1024;
              const uint4 wn0 = lds128(wa + nb), wn1 = lds128(wa + nb + 512);
              const uint32_t ws0[4] = {wc0.x, wc0.y, wc0.z, wc0.w}, ws1[4] = {wc1.x, wc1.y, wc1.z, wc1.w};
#pragma unroll
              for (int s4 = 0; s4 < 4; s4++) {
                const uint32_t xo = (uint32_t)(grp * 8 + bq * 4 + s4 + 1) * 32;
                uint2 bnext[NT];
#pragma unroll
                for (int j = 0; j < NT; j++) bnext[j] = lds64(xa[j] + xo);
                const uint32_t p0 = ws0[s4] >> 8, p1 = ws1[s4] >> 8;
                const uint32_t a0[4] = {ws0[s4] & 0x000F000Fu, ws0[s4] & 0x00F000F0u, p0 & 0x000F000Fu, p0 & 0x00F000F0u};
                const uint32_t a1[4] = {ws1[s4] & 0x000F000Fu, ws1[s4] & 0x00F000F0u, p1 & 0x000F000Fu, p1 & 0x00F000F0u};
#pragma unroll
                for (int j = 0; j < NT; j++) {
                  if (bq == 0 && s4 == 0) {
                    mma_f16_first(cg[0][j], a0, bcur[j].x, bcur[j].y);
                    mma_f16_first(cg[1][j], a1, bcur[j].x, bcur[j].y);
                  } else {
                    mma_f16(cg[0][j], a0, bcur[j].x, bcur[j].y);
                    mma_f16(cg[1][j], a1, bcur[j].x, bcur[j].y);
                  }
                }
#pragma unroll
                for (int j = 0; j < NT; j++) bcur[j] = bnext[j];
              }
              wc0 = wn0; wc1 = wn1;
            }
            // flush the group: rows g / g+8 of each half; the upper eight MMA rows carry 16 x their nibbles
            float sl[2], sh[2];
#pragma unroll
            for (int h = 0; h < 2; h++) {
              sl[h] = lds_bf16(sca + (uint32_t)(grp * 32 + h * 16) * 2);
              sh[h] = lds_bf16(sca + (uint32_t)(grp * 32 + h * 16 + 8) * 2);
            }
#pragma unroll
            for (int j = 0; j < NT; j++) {
              const float4 F0 = lds128f(fa[j][0] + (uint32_t)grp * 16), F1 = lds128f(fa[j][1] + (uint32_t)grp * 16);
#pragma unroll
              for (int h = 0; h < 2; h++) {
                ct[h][j][0] = fmaf(sl[h] * F0.x, cg[h][j][0], fmaf(sl[h], F0.z, ct[h][j][0]));
                ct[h][j][1] = fmaf(sl[h] * F1.x, cg[h][j][1], fmaf(sl[h], F1.z, ct[h][j][1]));
                ct[h][j][2] = fmaf(sh[h] * F0.y, cg[h][j][2], fmaf(sh[h], F0.z, ct[h][j][2]));
                ct[h][j][3] = fmaf(sh[h] * F1.y, cg[h][j][3], fmaf(sh[h], F1.z, ct[h][j][3]));
              }
            }
          }
        }
        if (k == 0) VS_STAMP(4);
        // ---- the slot's warps add their partial sums in unit order and share the fragments of the epilogue ----
        if (pl.upi > 1) {
          __syncwarp();                                     // every lane has finished reading the stage
#pragma unroll
          for (int h = 0; h < 2; h++)
#pragma unroll
            for (int j = 0; j < NT; j++)
              *reinterpret_cast<float4*>(stage + ((h * NT + j) * 32 + lane) * 16) =
                  make_float4(ct[h][j][0], ct[h][j][1], ct[h][j][2], ct[h][j][3]);
          named_bar_sync(1 + slot, pl.upi * 32);
        }
        const int tile = t0 + i;
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
          for (int j = 0; j < NT; j++) {
            const int qf = h * NT + j;
            if (pl.upi > 1 && qf % pl.upi != u) continue;   // warp-uniform
            float4 v = make_float4(ct[h][j][0], ct[h][j][1], ct[h][j][2], ct[h][j][3]);
            if (pl.upi > 1) {
              v = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int uu = 0; uu < pl.upi; uu++) {
                const float4 p = lds128f(smem_u32(vsm) + (uint32_t)(slot * pl.upi + uu) * ub + (uint32_t)(qf * 32 + lane) * 16);
                v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
              }
            }
            bool run = alive;
            if (pl.nkc > 1 && alive) {
              float4* mine = reinterpret_cast<float4*>(P.part) + (((size_t)tile * pl.nkc + kc) * (2 * NT) + qf) * 32 + lane;
              *mine = v;
              __threadfence();
              __syncwarp();
              int last = 0;
              if (lane == 0) {
                const int old = atomicAdd(P.counters + tile * 8 + qf, 1);
                last = old == pl.nkc - 1;
                if (last) P.counters[tile * 8 + qf] = 0;
              }
              last = __shfl_sync(0xffffffffu, last, 0);
              run = last != 0;
              if (run) {
                __threadfence();
                v = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int c = 0; c < pl.nkc; c++) {
                  const float4 p = ld_cg_f4(reinterpret_cast<const float4*>(P.part) + (((size_t)tile * pl.nkc + c) * (2 * NT) + qf) * 32 + lane);
                  v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
                }
              }
            }
            if (run) vs_epilogue<EPI>(P, tile * 32 + h * 16, j, v, lane);
          }
        if (k == 0) VS_STAMP(5);
        if (pl.upi > 1) named_bar_sync(1 + slot, pl.upi * 32);      // the partials have been read: the stages may go back
        __syncwarp();
        if (lane == 0) {
          fence_proxy_async_smem();
          mbar_arrive(&empty[warp]);
        }
      }
    }
  }
  __syncthreads();
  VS_STAMP(6);
  if (tid == 0 && *s_abort) {
    // every bulk copy that was issued must land before the CTA may exit: stage (slot, v) has had one load per
    // fully issued item of its slot, plus the interrupted item's if v is below the unit it stopped at
    const int idone = s_prog[0], ustop = s_prog[1];
    for (int s = 0; s < nst; s++) {
      const int slot = s / pl.upi, v = s % pl.upi;
      int cnt = idone > slot ? (idone - slot + pl.nslot - 1) / pl.nslot : 0;
      if (idone % pl.nslot == slot && v < ustop) cnt++;
      if (cnt == 0) continue;
      for (unsigned sp = 0; sp < wc.limit; sp++) {
        if (mbar_try(&full[s], (cnt - 1) & 1)) break;
        if ((sp & 1023) == 1023) __nanosleep(64);
      }
    }
  }
}

}  // namespace fb
