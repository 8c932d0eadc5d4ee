// M-token tree verification (EAGLE): every weight row is read once and applied to all M candidate tokens.
//
// First version of this path: a short sequence of kernels per layer on one stream (RMSNorm, int4 x bf16 GEMM with a
// fused epilogue, tree-masked attention), graph-capturable, instead of one persistent kernel. The contraction runs
// on the tensor pipe through warp-level mma (m16n8k16, bf16 x bf16 -> fp32): weight rows are the M dimension of the
// MMA, tokens the N dimension. Weights are dequantised in registers straight into A fragments as the exact bf16
// value (nibble - 8) / 16; the group scale (times 16) is applied in fp32 to each 128-column partial sum, so the
// arithmetic is the reference's (nib - 8) * s * x with fp32 accumulation, only the summation order differs.
//
// Activations that feed a GEMM are stored "k16-transposed": inside every block of 16 columns, column 4a+b sits at
// position 4b+a. A lane's B fragment (columns t, t+4 and 8+t, 12+t of a k16 step) is then one 8-byte shared-memory
// load, and the bf16 pair (nibble t, nibble t+4) that one shift+LOP3 extracts from a packed word is its A fragment.
#pragma once
#include "fb_common.cuh"

namespace fb {

__host__ __device__ __forceinline__ int k16_pos(int col) {       // where column `col` lives in the transposed layout
  const int c = col & 15;
  return (col & ~15) + ((c & 3) << 2) + (c >> 2);
}

// ------------------------------------------------------------------------------------------------ small kernels
// h[m] = bf16(float(embed[token[m]]) * mult), or a copy of the caller's residual rows
__global__ void v_embed(const int32_t* tokens, const uint16_t* embed, const uint16_t* h_in, uint16_t* h, int D, int vocab,
                        float mult, int* status_code) {
  const int m = blockIdx.x;
  int tok = 0;
  if (!h_in) {
    tok = tokens[m];
    if ((unsigned)tok >= (unsigned)vocab) { tok = 0; if (threadIdx.x == 0) atomicCAS(status_code, 0, 6); }
  }
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    h[(size_t)m * D + i] = h_in ? h_in[(size_t)m * D + i] : f2bf(bf2f(embed[(size_t)tok * D + i]) * mult);
}

// xn[m] = bf16((float(h) * r) * float(w)) in the k16-transposed layout; optionally also in natural order (feature out)
__global__ void v_rmsnorm(const uint16_t* h, const uint16_t* w, uint16_t* xn_t, uint16_t* xn_nat, int D, float eps) {
  const int m = blockIdx.x;
  const uint16_t* hm = h + (size_t)m * D;
  __shared__ float red[32];
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) { const float v = bf2f(hm[i]); ss = fmaf(v, v, ss); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); i++) tot += red[i];
  const float r = 1.0f / sqrtf(tot / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const uint16_t v = f2bf(bf2f(hm[i]) * r * bf2f(w[i]));
    xn_t[(size_t)m * D + k16_pos(i)] = v;
    if (xn_nat) xn_nat[(size_t)m * D + i] = v;
  }
}

// ------------------------------------------------------------------------------------------------ attention
// One CTA per (token m, kv head): the R query heads of the group share each K/V load. Query m sees every cached
// position t < pos and, among the M new slots pos..pos+M-1, those with amask[m][t - pos] != 0.
template <int HD, int R>
__global__ void __launch_bounds__(512) v_attn(const uint16_t* q, const uint16_t* kc, const uint16_t* vc,
                                              const uint8_t* amask, uint16_t* ao_t, int n_head, int nkv, int pos, int M,
                                              float scale) {
  constexpr int LPR = HD / 8, SEG = LPR <= 8 ? 8 : 16, PPW = 32 / SEG, NW = 16, BATCH = 4;
  const int m = blockIdx.x, kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg = lane / SEG, sl = lane % SEG;
  const bool active = sl < LPR;
  const int d0 = sl * 8, QD = n_head * HD, T = pos + M;
  __shared__ float wacc[NW][R][HD];
  __shared__ float wm[NW][R], wd[NW][R];
  float qf[R][8];
#pragma unroll
  for (int r = 0; r < R; r++) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (active) v = *reinterpret_cast<const uint4*>(q + (size_t)m * QD + (size_t)(kvh * R + r) * HD + d0);
    qf[r][0] = bflo(v.x); qf[r][1] = bfhi(v.x); qf[r][2] = bflo(v.y); qf[r][3] = bfhi(v.y);
    qf[r][4] = bflo(v.z); qf[r][5] = bfhi(v.z); qf[r][6] = bflo(v.w); qf[r][7] = bfhi(v.w);
  }
  float mx[R], den[R], acc[R][8];
#pragma unroll
  for (int r = 0; r < R; r++) {
    mx[r] = -1e30f; den[r] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; e++) acc[r][e] = 0.f;
  }
  for (int tb0 = warp * PPW; tb0 < T; tb0 += BATCH * NW * PPW) {
    uint4 kk[BATCH], vv[BATCH];
    bool valid[BATCH];
#pragma unroll
    for (int j = 0; j < BATCH; j++) {                 // all loads of a batch are issued before any is used
      const int t = tb0 + j * NW * PPW + seg;
      valid[j] = t < T;
      if (valid[j] && t >= pos) valid[j] = amask[m * M + (t - pos)] != 0;
      kk[j] = vv[j] = make_uint4(0, 0, 0, 0);
      if (valid[j] && active) {
        const size_t off = ((size_t)t * nkv + kvh) * HD + d0;
        kk[j] = *reinterpret_cast<const uint4*>(kc + off);
        vv[j] = *reinterpret_cast<const uint4*>(vc + off);
      }
    }
#pragma unroll
    for (int j = 0; j < BATCH; j++) {
      if (tb0 + j * NW * PPW >= T) break;             // warp-uniform
      const float kf[8] = {bflo(kk[j].x), bfhi(kk[j].x), bflo(kk[j].y), bfhi(kk[j].y), bflo(kk[j].z), bfhi(kk[j].z), bflo(kk[j].w), bfhi(kk[j].w)};
      const float vf[8] = {bflo(vv[j].x), bfhi(vv[j].x), bflo(vv[j].y), bfhi(vv[j].y), bflo(vv[j].z), bfhi(vv[j].z), bflo(vv[j].w), bfhi(vv[j].w)};
#pragma unroll
      for (int r = 0; r < R; r++) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) s = fmaf(qf[r][e], kf[e], s);
#pragma unroll
        for (int o = SEG / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        s *= scale;
        if (valid[j]) {
          const float m2 = fmaxf(mx[r], s);
          const float corr = __expf(mx[r] - m2), w = __expf(s - m2);
          den[r] = den[r] * corr + w;
#pragma unroll
          for (int e = 0; e < 8; e++) acc[r][e] = acc[r][e] * corr + w * vf[e];
          mx[r] = m2;
        }
      }
    }
  }
#pragma unroll
  for (int off = SEG; off < 32; off <<= 1) {
#pragma unroll
    for (int r = 0; r < R; r++) {
      const float mo = __shfl_xor_sync(0xffffffffu, mx[r], off);
      const float dn = __shfl_xor_sync(0xffffffffu, den[r], off);
      const float gm = fmaxf(mx[r], mo);
      const float wa = __expf(mx[r] - gm), wb = __expf(mo - gm);
      den[r] = den[r] * wa + dn * wb;
#pragma unroll
      for (int e = 0; e < 8; e++) {
        const float ao_ = __shfl_xor_sync(0xffffffffu, acc[r][e], off);
        acc[r][e] = acc[r][e] * wa + ao_ * wb;
      }
      mx[r] = gm;
    }
  }
  if (seg == 0 && active) {
#pragma unroll
    for (int r = 0; r < R; r++) {
#pragma unroll
      for (int e = 0; e < 8; e++) wacc[warp][r][d0 + e] = acc[r][e];
      if (sl == 0) { wm[warp][r] = mx[r]; wd[warp][r] = den[r]; }
    }
  }
  __syncthreads();
  for (int o = threadIdx.x; o < R * HD; o += blockDim.x) {
    const int r = o / HD, d = o % HD;
    float gm = -1e30f;
#pragma unroll
    for (int w = 0; w < NW; w++) gm = fmaxf(gm, wm[w][r]);
    float Dn = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < NW; w++) {
      const float e = __expf(wm[w][r] - gm);
      Dn += wd[w][r] * e;
      A += wacc[w][r][d] * e;
    }
    ao_t[(size_t)m * QD + k16_pos((kvh * R + r) * HD + d)] = f2bf(A / Dn);
  }
}

// ------------------------------------------------------------------------------------------------ int4 x bf16 GEMM
enum { EPI_QKV = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_LOGITS = 3 };

struct VGemmParams {
  const uint8_t* w;        // streaming records of this matrix (layer offset applied)
  const uint16_t* x_t;     // bf16 [MT][K], k16-transposed, rows >= M are padding
  int rows, K, rec, M, has_zeros;
  // epilogue operands
  uint16_t* h;             // RESID: bf16 [M][D] in/out
  uint16_t* q;             // QKV: bf16 [M][QD]
  uint16_t *kc, *vc;       // QKV: layer base of the caches
  uint16_t* act_t;         // SWIGLU: bf16 [MT][FF] transposed
  float* logits;           // LOGITS: f32 [M][vocab]
  const int32_t* depth;
  const float* invf;
  int n_head, nkv, pos, out_ld;
  float resid, logits_scaling;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// bf16 pair ((nib_t - 8)/16, (nib_{t+4} - 8)/16) of a packed word: rotate the two nibbles to mantissa bits 3..6 of each
// half, OR in 1.0, subtract 1.5
__device__ __forceinline__ uint32_t a_pair(uint32_t w, int rot) {
  const uint32_t v = (__funnelshift_r(w, w, rot) & 0x00780078u) | 0x3F803F80u;
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(v), "r"(0x3FC03FC0u));
  return d;
}

// CTA: 32 weight rows (two m16 tiles) x all MT tokens; its 8 warps are 2 row tiles x 4 quarters of every K chunk (a
// quarter never straddles a 128-column group). Every CTA re-reads the activations, so taller tiles halve that traffic;
// wide chunks amortise the per-chunk barrier; the pipeline is as deep as shared memory allows, because the kernel is
// latency-bound unless tens of KB of weights per SM are in flight.
template <int MT>
struct VCfg {
  static constexpr int RT = 32;
  static constexpr int KCMAX = MT <= 32 ? 512 : 256;            // widest K chunk whose activations still fit a stage
  template <int KC>
  static constexpr int stages() {
    constexpr int stage = RT * (KC / 2 + 16) + MT * (KC * 2 + 32);
    constexpr int budget = MT <= 16 ? 104 * 1024 : 200 * 1024;    // 2 CTAs per SM for the common 16-token case
    return budget / stage < 2 ? 2 : (budget / stage > 8 ? 8 : budget / stage);
  }
};
template <int MT, int KC, int EPI, int HD>
__global__ void __launch_bounds__(256) v_gemm(const VGemmParams P) {
  constexpr int RT = VCfg<MT>::RT, NT = MT / 8, STAGES = VCfg<MT>::template stages<KC>();
  constexpr int MTILES = RT / 16, KPARTS = 8 / MTILES;
  constexpr int WSTRIDE = KC / 2 + 16;          // bytes per weight row in a stage (padding de-conflicts the A loads)
  constexpr int XSTRIDE = KC * 2 + 32;          // bytes per token row in a stage
  constexpr int STAGE_BYTES = RT * WSTRIDE + MT * XSTRIDE;
  constexpr int QCOLS = KC / KPARTS, KSTEPS = QCOLS / 16;
  static_assert(QCOLS % 16 == 0 && 128 % QCOLS == 0, "a warp's quarter of a chunk lies inside one group");
  extern __shared__ __align__(128) uint8_t vsm[];
  uint16_t* s_scale = reinterpret_cast<uint16_t*>(vsm + STAGES * STAGE_BYTES);     // [RT][groups (+zeros)]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int mt = warp / KPARTS, kq = warp % KPARTS;
  const int row0 = blockIdx.x * RT;
  const int groups = P.K / 128, nchunk = P.K / KC;
  const int meta = groups * (P.has_zeros ? 2 : 1);

  // scales (and zeros) of the 32 rows, once
  for (int i = tid; i < RT * meta; i += 256) {
    const int r = i / meta, j = i % meta;
    const int row = min(row0 + r, P.rows - 1);
    s_scale[i] = reinterpret_cast<const uint16_t*>(P.w + (size_t)row * P.rec + P.K / 2)[j];
  }
  auto issue = [&](int chunk, int stage) {
    uint8_t* sw = vsm + stage * STAGE_BYTES;
    uint8_t* sx = sw + RT * WSTRIDE;
    constexpr int WCH = KC / 2 / 16;            // 16-byte pieces per weight row
    for (int i = tid; i < RT * WCH; i += 256) {
      const int r = i / WCH, c = i % WCH;
      const int row = min(row0 + r, P.rows - 1);
      cp_async16(sw + r * WSTRIDE + c * 16, P.w + (size_t)row * P.rec + (size_t)chunk * (KC / 2) + c * 16);
    }
    constexpr int XCH = KC * 2 / 16;
    for (int i = tid; i < MT * XCH; i += 256) {
      const int m = i / XCH, c = i % XCH;
      cp_async16(sx + m * XSTRIDE + c * 16, P.x_t + (size_t)m * P.K + (size_t)chunk * KC + c * 8);
    }
  };
  float ct[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int e = 0; e < 4; e++) ct[j][e] = 0.f;
  float xsum[NT][2];                              // asymmetric layout: sum of x per token over the warp's columns
  for (int s = 0; s < STAGES - 1; s++) {
    if (s < nchunk) issue(s, s);
    cp_async_commit();
  }
  const int rot = (4 * t - 3) & 31;
  for (int c = 0; c < nchunk; c++) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (c + STAGES - 1 < nchunk) issue(c + STAGES - 1, (c + STAGES - 1) % STAGES);
    cp_async_commit();
    const uint8_t* sw = vsm + (c % STAGES) * STAGE_BYTES;
    const uint8_t* sx = sw + RT * WSTRIDE;
    float cg[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) cg[j][e] = 0.f;
    if (P.has_zeros) {
#pragma unroll
      for (int j = 0; j < NT; j++) xsum[j][0] = xsum[j][1] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++) {
      const int colb = kq * QCOLS + ks * 16;      // first column of this k16 step inside the chunk
      const uint2 w_lo = *reinterpret_cast<const uint2*>(sw + (mt * 16 + g) * WSTRIDE + colb / 2);
      const uint2 w_hi = *reinterpret_cast<const uint2*>(sw + (mt * 16 + g + 8) * WSTRIDE + colb / 2);
      uint32_t a[4];
      a[0] = a_pair(w_lo.x, rot); a[1] = a_pair(w_hi.x, rot); a[2] = a_pair(w_lo.y, rot); a[3] = a_pair(w_hi.y, rot);
#pragma unroll
      for (int j = 0; j < NT; j++) {
        const uint2 b = *reinterpret_cast<const uint2*>(sx + (j * 8 + g) * XSTRIDE + colb * 2 + t * 8);
        mma_bf16(cg[j], a, b.x, b.y);
      }
      if (P.has_zeros) {
        // token sums for the z * sum(x) term: C fragment column pair (2t, 2t+1) of n-tile j = tokens j*8+2t, +1
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const uint4* xr = reinterpret_cast<const uint4*>(sx + (j * 8 + 2 * t + e) * XSTRIDE + colb * 2);
            const uint4 v0 = xr[0], v1 = xr[1];
            xsum[j][e] += bflo(v0.x) + bfhi(v0.x) + bflo(v0.y) + bfhi(v0.y) + bflo(v0.z) + bfhi(v0.z) + bflo(v0.w) + bfhi(v0.w) +
                          bflo(v1.x) + bfhi(v1.x) + bflo(v1.y) + bfhi(v1.y) + bflo(v1.z) + bfhi(v1.z) + bflo(v1.w) + bfhi(v1.w);
          }
      }
    }
    const int grp = (c * KC + kq * QCOLS) >> 7;
    const float s_lo = bf2f(s_scale[(mt * 16 + g) * meta + grp]) * 16.f;
    const float s_hi = bf2f(s_scale[(mt * 16 + g + 8) * meta + grp]) * 16.f;
#pragma unroll
    for (int j = 0; j < NT; j++) {
      ct[j][0] = fmaf(s_lo, cg[j][0], ct[j][0]); ct[j][1] = fmaf(s_lo, cg[j][1], ct[j][1]);
      ct[j][2] = fmaf(s_hi, cg[j][2], ct[j][2]); ct[j][3] = fmaf(s_hi, cg[j][3], ct[j][3]);
    }
    if (P.has_zeros) {
      const float z_lo = bf2f(s_scale[(mt * 16 + g) * meta + groups + grp]);
      const float z_hi = bf2f(s_scale[(mt * 16 + g + 8) * meta + groups + grp]);
#pragma unroll
      for (int j = 0; j < NT; j++) {
        ct[j][0] = fmaf(z_lo, xsum[j][0], ct[j][0]); ct[j][1] = fmaf(z_lo, xsum[j][1], ct[j][1]);
        ct[j][2] = fmaf(z_hi, xsum[j][0], ct[j][2]); ct[j][3] = fmaf(z_hi, xsum[j][1], ct[j][3]);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  // ---- reduce the 4 K-quarters of each row tile through shared memory: y[r][m], r < 32, m < MT ----
  float* red = reinterpret_cast<float*>(vsm);                     // [KPARTS][RT rows][MT]
#pragma unroll
  for (int j = 0; j < NT; j++) {
    float* base = red + ((size_t)kq * RT + mt * 16) * MT + j * 8 + 2 * t;
    base[(size_t)g * MT] = ct[j][0]; base[(size_t)g * MT + 1] = ct[j][1];
    base[(size_t)(g + 8) * MT] = ct[j][2]; base[(size_t)(g + 8) * MT + 1] = ct[j][3];
  }
  __syncthreads();
  auto Y = [&](int r, int m) {
    float v = red[(size_t)r * MT + m];
#pragma unroll
    for (int k = 1; k < KPARTS; k++) v += red[((size_t)k * RT + r) * MT + m];
    return v;
  };
  if (EPI == EPI_RESID) {
    for (int o = tid; o < RT * MT; o += 256) {
      const int r = o % RT, m = o / RT, row = row0 + r;
      if (row < P.rows && m < P.M) {
        uint16_t* hp = P.h + (size_t)m * P.out_ld + row;
        *hp = f2bf(bf2f(*hp) + Y(r, m) * P.resid);
      }
    }
  } else if (EPI == EPI_LOGITS) {
    for (int o = tid; o < RT * MT; o += 256) {
      const int r = o % RT, m = o / RT, row = row0 + r;
      if (row < P.rows && m < P.M) P.logits[(size_t)m * P.out_ld + row] = Y(r, m) / P.logits_scaling;
    }
  } else if (EPI == EPI_SWIGLU) {
    for (int o = tid; o < (RT / 2) * MT; o += 256) {
      const int pr = o % (RT / 2), m = o / (RT / 2), row = row0 + 2 * pr;
      if (row < P.rows && m < P.M) {
        const float gg = rbf(Y(2 * pr, m)), uu = rbf(Y(2 * pr + 1, m));
        P.act_t[(size_t)m * P.out_ld + k16_pos(row >> 1)] = f2bf((gg / (1.0f + __expf(-gg))) * uu);
      }
    }
  } else {   // EPI_QKV: stream rows (2p, 2p+1) of a head are dims (p, p + HD/2); V rows keep their order
    constexpr int HP = HD / 2;
    const int QD = P.n_head * HD;
    for (int o = tid; o < (RT / 2) * MT; o += 256) {
      const int pr = o % (RT / 2), m = o / (RT / 2), rs = row0 + 2 * pr;
      if (rs < P.rows && m < P.M) {
        const float a0 = Y(2 * pr, m), a1 = Y(2 * pr + 1, m);
        const int head = rs / HD, within = rs % HD;
        if (head < P.n_head + P.nkv) {
          const int i = within >> 1;
          const float x0 = rbf(a0), x1 = rbf(a1);
          float sn, cs;
          sincosf((float)(P.pos + P.depth[m]) * P.invf[i], &sn, &cs);
          const uint16_t y0 = f2bf(x0 * cs - x1 * sn), y1 = f2bf(x1 * cs + x0 * sn);
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

// dynamic shared memory of a launch: the stages (reused by the reduction) + `meta` bf16 scales/zeros per row
template <int MT, int KC>
constexpr int v_gemm_smem(int meta) {
  constexpr int RT = VCfg<MT>::RT;
  constexpr int stages = VCfg<MT>::template stages<KC>() * (RT * (KC / 2 + 16) + MT * (KC * 2 + 32));
  constexpr int red = (8 / (RT / 16)) * RT * MT * 4;
  return (stages > red ? stages : red) + ((RT * meta * 2 + 127) & ~127);
}

}  // namespace fb
