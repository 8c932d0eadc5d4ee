// M-token tree verification (EAGLE): every weight row is read once and applied to all M candidate tokens.
//
// A short sequence of kernels per layer on one stream (RMSNorm, int4 x bf16 GEMM with a fused epilogue, tree-masked
// attention), graph-capturable. The GEMM reads the same tiled streaming layout as the decode kernel and runs on the
// tensor pipe through warp-level mma (m16n8k16, bf16 x bf16 -> fp32): 16 weight rows are the M dimension of the MMA,
// 8 tokens the N dimension. A tile word holds, for one lane slot, the nibbles of one weight row in two column ranges
// (low and high nibble of every byte); masking them leaves bf16 SUBNORMALS nib * 2^-133 (or 16 * nib * 2^-133), and one
// bf16x2 fma with 2^127 turns those into the exact values (nib - 8) / 64 (or / 4). The group scale (times 64 or 4) is
// applied in fp32 to each group's partial sum, so the arithmetic is the reference's (nib - 8) * s * x with fp32
// accumulation; only the summation order differs.
//
// Activations that feed a GEMM are stored in "B order": inside every block of 16 columns the sequence is
// [0 1 8 9 | 2 3 10 11 | 4 5 12 13 | 6 7 14 15], so a lane's B fragment of a k16 step (columns 2t, 2t+1, 2t+8, 2t+9) is
// one 8-byte shared-memory load.
#pragma once
#include "fb_common.cuh"

namespace fb {


__host__ __device__ __forceinline__ int k16_pos(int col) {       // where column `col` lives in B order
  const int c = col & 15;
  return (col & ~15) + (((c & 7) >> 1) << 2) + ((c >> 3) << 1) + (c & 1);
}

// ------------------------------------------------------------------------------------------------ small kernels
// h[m] = bf16(float(embed[token[m]]) * mult), or a copy of the caller's residual rows
__global__ void v_embed(const int32_t* tokens, const uint16_t* embed, const uint16_t* h_in, uint16_t* h, int D, int vocab,
                        float mult, int* status_code) {
  const int m = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  int tok = 0;
  if (!h_in) {
    tok = tokens[m];
    if ((unsigned)tok >= (unsigned)vocab) { tok = 0; if (threadIdx.x == 0) atomicCAS(status_code, 0, 6); }
  }
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    h[(size_t)m * D + i] = h_in ? h_in[(size_t)m * D + i] : f2bf(bf2f(embed[(size_t)tok * D + i]) * mult);
}

// xn[m] = bf16((float(h) * r) * float(w)) in B order; optionally also in natural order (feature out).
// One CTA per token; a thread keeps its 8-element pieces in registers between the two passes (D <= 8 * 256 * NV).
template <int NV>
__global__ void __launch_bounds__(256) v_rmsnorm(const uint16_t* h, const uint16_t* w, uint16_t* xn_t, uint16_t* xn_nat, int D,
                                                 float eps) {
  const int m = blockIdx.x, tid = threadIdx.x;
  const uint4* hm = reinterpret_cast<const uint4*>(h + (size_t)m * D);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  const int nvec = D / 8;
  __shared__ float red[8];
  uint4 hv[NV], ww[NV];
  float ss = 0.f;
  pdl_trigger();
#pragma unroll
  for (int k = 0; k < NV; k++) {       // the norm weights do not depend on the previous kernel
    const int i = tid + k * 256;
    ww[k] = make_uint4(0, 0, 0, 0);
    if (i < nvec) ww[k] = __ldg(wv + i);
  }
  pdl_wait();
#pragma unroll
  for (int k = 0; k < NV; k++) {
    const int i = tid + k * 256;
    hv[k] = make_uint4(0, 0, 0, 0);
    if (i < nvec) hv[k] = hm[i];
    const uint32_t p[4] = {hv[k].x, hv[k].y, hv[k].z, hv[k].w};
#pragma unroll
    for (int e = 0; e < 4; e++) { ss = fmaf(bflo(p[e]), bflo(p[e]), ss); ss = fmaf(bfhi(p[e]), bfhi(p[e]), ss); }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) tot += red[i];
  const float r = 1.0f / sqrtf(tot / (float)D + eps);
#pragma unroll
  for (int k = 0; k < NV; k++) {
    const int i = tid + k * 256;
    if (i < nvec) {
      const uint32_t p[4] = {hv[k].x, hv[k].y, hv[k].z, hv[k].w}, q[4] = {ww[k].x, ww[k].y, ww[k].z, ww[k].w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; e++)
        o[e] = (uint32_t)f2bf(bflo(p[e]) * r * bflo(q[e])) | ((uint32_t)f2bf(bfhi(p[e]) * r * bfhi(q[e])) << 16);
      // elements 8i .. 8i+7 are half (i & 1) of a 16-block: pair e goes to 32-bit slot 2e + half of the block
      if (xn_t) {
        uint32_t* dst = reinterpret_cast<uint32_t*>(xn_t + (size_t)m * D + (size_t)(i >> 1) * 16);
#pragma unroll
        for (int e = 0; e < 4; e++) dst[2 * e + (i & 1)] = o[e];
      }
      if (xn_nat) reinterpret_cast<uint4*>(xn_nat + (size_t)m * D)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ attention

// Tree-masked attention of all M candidate tokens on the tensor pipe. One CTA per (kv head, span of cached positions,
// group of 64 query rows): the M * R query rows that share the kv head (row = token * R + head in group; a warp owns 16
// of them, blockIdx.z selects the CTA's four 16-row tiles) are the M dimension of the MMAs, 64
// positions at a time the N dimension of Q K^T and the K dimension of P V. Query m sees every cached position
// t < pos and, among the M new slots pos..pos+M-1, those with amask[m][t - pos] != 0. Probabilities enter P V as a
// sum of two bf16 values (p = hi + lo), which keeps their fp32 precision to ~2^-17. Every span writes, per query row,
// an un-normalised partial (acc[HD], running max, denominator); v_attn_merge combines the spans.
template <int HD, int R>
__global__ void __launch_bounds__(128) v_attn_mma(const uint16_t* q, const uint16_t* kc, const uint16_t* vc,
                                                  const uint8_t* amask, float* part, int n_head, int nkv, int pos, int M,
                                                  float scale, int span) {
  constexpr int CH = 64, KSTEPS = HD / 16, NTD = HD / 8, STR = HD * 2 + 16, PW = HD + 2;
  static_assert(HD % 16 == 0 && NTD % 2 == 0, "head_dim must be a multiple of 16");
  __shared__ __align__(16) uint8_t k_s[CH * STR];
  __shared__ __align__(16) uint8_t v_s[CH * STR];
  const int kvh = blockIdx.x, sp = blockIdx.y, S = gridDim.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int T = pos + M, QD = n_head * HD, rows = M * R;
  pdl_trigger();
  pdl_wait();
  const int t_begin = sp * span, t_end = min(T, t_begin + span);
  const int ntile = (rows + 15) / 16;
  {
    const int mt = (int)blockIdx.z * 4 + warp;
    const bool live = mt < ntile;
    const int r_lo = min(mt * 16 + g, rows - 1), r_hi = min(mt * 16 + g + 8, rows - 1);
    const int m_lo = r_lo / R, m_hi = r_hi / R;
    const uint16_t* q_lo = q + (size_t)m_lo * QD + (size_t)(kvh * R + r_lo % R) * HD;
    const uint16_t* q_hi = q + (size_t)m_hi * QD + (size_t)(kvh * R + r_hi % R) * HD;
    uint32_t aq[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++) {
      aq[ks][0] = *reinterpret_cast<const uint32_t*>(q_lo + 16 * ks + 2 * t);
      aq[ks][1] = *reinterpret_cast<const uint32_t*>(q_hi + 16 * ks + 2 * t);
      aq[ks][2] = *reinterpret_cast<const uint32_t*>(q_lo + 16 * ks + 2 * t + 8);
      aq[ks][3] = *reinterpret_cast<const uint32_t*>(q_hi + 16 * ks + 2 * t + 8);
    }
    float o[NTD][4];
#pragma unroll
    for (int j = 0; j < NTD; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) o[j][e] = 0.f;
    float mrun[2] = {-1e30f, -1e30f}, lrun[2] = {0.f, 0.f};
    for (int c0 = t_begin; c0 < t_end; c0 += CH) {
      __syncthreads();                                  // the previous chunk's readers are done
      for (int i = tid; i < CH * (HD / 8); i += 128) {
        const int row = i / (HD / 8), pc = i % (HD / 8), tp = c0 + row;
        uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);   // rows past the end: zeros (0 * garbage could be NaN)
        if (tp < T) {
          const size_t off = ((size_t)tp * nkv + kvh) * HD + pc * 8;
          kv = *reinterpret_cast<const uint4*>(kc + off);
          vv = *reinterpret_cast<const uint4*>(vc + off);
        }
        *reinterpret_cast<uint4*>(k_s + row * STR + pc * 16) = kv;
        *reinterpret_cast<uint4*>(v_s + row * STR + pc * 16) = vv;
      }
      __syncthreads();
      if (!live) continue;
      float s[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; nt++) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
          const uint8_t* kr = k_s + (nt * 8 + g) * STR + (16 * ks + 2 * t) * 2;
          mma_bf16(s[nt], aq[ks], *reinterpret_cast<const uint32_t*>(kr), *reinterpret_cast<const uint32_t*>(kr + 16));
        }
      }
      // scale, mask, row maxima (rows g and g + 8; a row's 64 scores live in the 4 lanes of a quad)
      float mx[2] = {-INFINITY, -INFINITY};
      const bool tree = c0 + CH > pos;                   // the chunk reaches into the M new slots
#pragma unroll
      for (int nt = 0; nt < 8; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int tp = c0 + nt * 8 + 2 * t + (e & 1);
          bool ok = tp < T;
          if (tree && ok && tp >= pos) ok = amask[(e < 2 ? m_lo : m_hi) * M + (tp - pos)] != 0;
          const float v = ok ? s[nt][e] * scale : -INFINITY;
          s[nt][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      float corr[2];
#pragma unroll
      for (int h = 0; h < 2; h++) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float mn = fmaxf(mrun[h], mx[h]);           // finite: the running maximum starts at -1e30
        corr[h] = __expf(mrun[h] - mn);
        mrun[h] = mn;
        lrun[h] *= corr[h];
      }
#pragma unroll
      for (int j = 0; j < NTD; j++) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
#pragma unroll
      for (int nt = 0; nt < 8; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float pv = __expf(s[nt][e] - mrun[e >> 1]);
          s[nt][e] = pv;
          lrun[e >> 1] += pv;                             // this lane's columns; the quad is summed at the end
        }
      // O += P V, 16 positions per step
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
        uint32_t ah[4], al[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float p0 = s[2 * kk + (e >> 1)][(e & 1) * 2], p1 = s[2 * kk + (e >> 1)][(e & 1) * 2 + 1];
          const float h0 = rbf(p0), h1 = rbf(p1);
          ah[e] = pack_bf16(h0, h1);
          al[e] = pack_bf16(p0 - h0, p1 - h1);
        }
#pragma unroll
        for (int j = 0; j < NTD; j += 2) {
          uint32_t b[4];
          const int mat = lane >> 3;
          ldmatrix_x4_trans(b, v_s + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * STR + (j + (mat >> 1)) * 16);
          mma_bf16(o[j], ah, b[0], b[1]);
          mma_bf16(o[j], al, b[0], b[1]);
          mma_bf16(o[j + 1], ah, b[2], b[3]);
          mma_bf16(o[j + 1], al, b[2], b[3]);
        }
      }
    }
    if (live) {
#pragma unroll
      for (int h = 0; h < 2; h++) {
        lrun[h] += __shfl_xor_sync(0xffffffffu, lrun[h], 1);
        lrun[h] += __shfl_xor_sync(0xffffffffu, lrun[h], 2);
        const int row = mt * 16 + g + 8 * h;
        if (row < rows) {
          float* pr = part + ((size_t)(kvh * S + sp) * rows + row) * PW;
#pragma unroll
          for (int j = 0; j < NTD; j++)
            *reinterpret_cast<float2*>(pr + j * 8 + 2 * t) = make_float2(o[j][2 * h], o[j][2 * h + 1]);
          if (t == 0) { pr[HD] = mrun[h]; pr[HD + 1] = lrun[h]; }
        }
      }
    }
  }
}

// one CTA per (token, kv head): combine the spans' partials, write bf16 in B order or natural order (S <= 32 spans)
template <int HD, int R>
__global__ void __launch_bounds__(256) v_attn_merge(const float* part, uint16_t* ao_t, int n_head, int nkv, int M, int S,
                                                    int natural) {
  constexpr int PW = HD + 2, MAXS = 32;
  const int m = blockIdx.x, kvh = blockIdx.y, rows = M * R, QD = n_head * HD;
  pdl_trigger();
  pdl_wait();
  for (int o = threadIdx.x; o < R * HD; o += blockDim.x) {
    const int r = o / HD, d = o % HD, row = m * R + r;
    const float* p0 = part + ((size_t)kvh * S * rows + row) * PW;
    float pm[MAXS], pl[MAXS], pa[MAXS];            // all loads are issued before the first one is used
#pragma unroll
    for (int s2 = 0; s2 < MAXS; s2++) {
      const float* ps = p0 + (size_t)(s2 < S ? s2 : 0) * rows * PW;
      pm[s2] = s2 < S ? ps[HD] : -1e30f;
      pl[s2] = s2 < S ? ps[HD + 1] : 0.f;
      pa[s2] = s2 < S ? ps[d] : 0.f;
    }
    float gm = -1e30f;
#pragma unroll
    for (int s2 = 0; s2 < MAXS; s2++) gm = fmaxf(gm, pm[s2]);
    float A = 0.f, Dn = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < MAXS; s2++) {
      const float e = __expf(pm[s2] - gm);
      Dn = fmaf(pl[s2], e, Dn);
      A = fmaf(pa[s2], e, A);
    }
    const int col = (kvh * R + r) * HD + d;
    ao_t[(size_t)m * QD + (natural ? col : k16_pos(col))] = f2bf(A / Dn);
  }
}

// ------------------------------------------------------------------------------------------------ int4 x bf16 GEMM
enum { EPI_QKV = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_LOGITS = 3 };

struct VGemmParams {
  const uint8_t* w;        // tiles of this matrix (layer offset applied)
  const uint16_t* x_t;     // bf16 [MT][K] in B order, rows >= M are padding
  int rows, M, has_zeros;
  // epilogue operands
  uint16_t* h;             // RESID: bf16 [M][D] in/out
  uint16_t* q;             // QKV: bf16 [M][QD]
  uint16_t *kc, *vc;       // QKV: layer base of the caches
  uint16_t* act_t;         // SWIGLU: bf16 [MT][FF] in B order
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

// low nibbles of a word's two halves (bits 0..3, 16..19) -> bf16 pair ((nib - 8) / 64, ...): the masked bits are the
// subnormals nib * 2^-133; times 2^127 minus 1/8
__device__ __forceinline__ uint32_t cvt_lo(uint32_t w) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(w & 0x000F000Fu), "r"(0x7F007F00u), "r"(0xBE00BE00u));
  return d;
}
// nibbles in bits 4..7, 20..23 -> ((nib - 8) / 4, ...): 16 * nib * 2^-133 times 2^127 minus 2
__device__ __forceinline__ uint32_t cvt_hi(uint32_t w) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(w & 0x00F000F0u), "r"(0x7F007F00u), "r"(0xC000C000u));
  return d;
}

// Persistent CTAs: CTA b takes the 32-row blocks b, b + grid, ... of the matrix and runs one cp.async pipeline over all
// their chunks, so the weights of the next block are already in flight while the epilogue of the current one runs.
// The warps are 2 (or 4) blocks of 16 rows x 4..8 roles; a role is a pair of column ranges (the low- and high-nibble range of
// the same tile words) and a share of every chunk's steps. The activations of all MT tokens stay resident in shared
// memory for the whole kernel when they fit (XRES); otherwise their chunks travel through the pipeline with the weights.
template <int MT, int K, int ROWS_ = 32>
struct VG {
  using C = TCfg<K>;
  static constexpr int RT = C::RT, NJ = C::NJ, ROWS = ROWS_, TILES = ROWS / RT, NMB = ROWS / 16;
  static constexpr int NW = MT <= 16 ? 16 : 8;             // warps: few tokens leave little work per warp, so use more
  static constexpr int NROLE = NW / NMB, NTHR = NW * 32;        // warps = 16-row blocks x roles
  static constexpr int PG = NJ >= 2 ? NJ / 2 : 1;          // pairs of ranges
  static constexpr int SPLIT = NROLE / PG;                 // warps that share the steps of one (row block, pair)
  static constexpr int XRS = K * 2 + 32;                   // resident activations: bytes per token row
  static constexpr bool XRES = MT * XRS <= 168 * 1024;
  static constexpr int stage_bytes(int nbc) { return TILES * nbc * 512 + (XRES ? 0 : MT * (NJ * 64 * nbc * 2 + 32)); }
  static constexpr int NBC = (C::BQ % 2 == 0 && (stage_bytes(2) <= 28 * 1024 || SPLIT > 4)) ? 2 : 1;   // 4-step blocks per chunk
  static constexpr int SPW = 4 * NBC / SPLIT;              // steps per warp per chunk
  static constexpr int XSTRIDE = NJ * 64 * NBC * 2 + 32;   // streamed activations: bytes per token row in a stage
  static constexpr int WBYTES = TILES * NBC * 512;
  static constexpr int STAGE = stage_bytes(NBC);
  static constexpr int RED = NROLE * ROWS * MT * 4;        // the roles' partial sums meet in shared memory
  static constexpr int XBYTES = XRES ? MT * XRS : 0;
  static constexpr int MB1 = ROWS * C::G * 2 * 2;          // one block's scales and zeros
  static constexpr int BUDGET = 216 * 1024 - XBYTES - RED - 2 * MB1;
  static constexpr int STAGES = BUDGET / STAGE < 2 ? 2 : (BUDGET / STAGE > 8 ? 8 : BUDGET / STAGE);
  static constexpr int NCHUNK = C::BQ / NBC;
  static constexpr int MDEPTH = (STAGES - 1) / NCHUNK + 2;  // scale blocks in flight
  static constexpr int smem() { return STAGES * STAGE + XBYTES + RED + MDEPTH * MB1; }
  static_assert(SPW >= 1 && SPW * SPLIT == 4 * NBC && C::BQ % NBC == 0 && PG * SPLIT == NROLE, "verify GEMM geometry");
  static_assert(smem() <= 227 * 1024, "verify GEMM shared memory");
};

template <int MT, int K, int EPI, int HD, int ROWS_ = 32>
__global__ void __launch_bounds__(VG<MT, K, ROWS_>::NTHR) v_gemm(const VGemmParams P) {
  using V = VG<MT, K, ROWS_>;
  using C = TCfg<K>;
  constexpr int RT = V::RT, NT = MT / 8, STAGES = V::STAGES, NBC = V::NBC, SPW = V::SPW, ROWS = V::ROWS, NCHUNK = V::NCHUNK;
  constexpr int G = C::G;
  constexpr bool XRES = V::XRES;
  constexpr int NTHR = V::NTHR;
  extern __shared__ __align__(128) uint8_t vsm[];
  const bool hz = P.has_zeros != 0;
  const int mbytes = RT * G * 2 * (hz ? 2 : 1);        // a tile's scale (and zero) block: bf16 [G][RT] (, [G][RT])
  uint8_t* s_x = vsm + STAGES * V::STAGE;               // [MT][XRS] resident activations
  float* red = reinterpret_cast<float*>(s_x + V::XBYTES);   // [roles][ROWS][MT]
  uint8_t* s_meta = reinterpret_cast<uint8_t*>(red) + V::RED;   // [MDEPTH][TILES][mbytes]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int mb = warp % V::NMB, role = warp / V::NMB, pg = role % V::PG, kq = role / V::PG;
  const int ntiles = (P.rows + RT - 1) / RT, nrb = (P.rows + ROWS - 1) / ROWS;
  const int tile_b = C::NIB + mbytes;
  const int nmine = (int)blockIdx.x < nrb ? (nrb - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int nitems = nmine * NCHUNK;

  // every thread copies the same pieces of every chunk: (tile, block, 16-byte piece) -> fixed source and destination offsets
  constexpr int WPIECES = V::TILES * NBC * 32, WPT = (WPIECES + NTHR - 1) / NTHR;
  int wtile[WPT], wsrc[WPT], wdst[WPT];
#pragma unroll
  for (int k = 0; k < WPT; k++) {
    const int i = tid + k * NTHR;
    const int p16 = i & 31, b = (i >> 5) % NBC, tl = (i >> 5) / NBC;
    wtile[k] = i < WPIECES ? tl : -1;
    wsrc[k] = b * 512 + p16 * 16;
    wdst[k] = ((tl * NBC + b) * 32 + p16) * 16;
  }
  auto issue_w = [&](int n) {
    const int bi = n / NCHUNK, chunk = n % NCHUNK, tile0 = ((int)blockIdx.x + bi * (int)gridDim.x) * V::TILES;
    uint8_t* sw = vsm + (n % STAGES) * V::STAGE;
    const uint8_t* src = P.w + (size_t)chunk * (NBC * 512);
#pragma unroll
    for (int k = 0; k < WPT; k++)
      if (wtile[k] >= 0)
        cp_async16(sw + wdst[k], src + (size_t)min(tile0 + wtile[k], ntiles - 1) * tile_b + wsrc[k]);
    if (chunk == 0) {                                   // the block's scales travel with its first chunk
      uint8_t* sm = s_meta + (bi % V::MDEPTH) * V::MB1;
      for (int i = tid; i < V::TILES * (mbytes / 16); i += NTHR) {
        const int tl = i / (mbytes / 16), pc = i % (mbytes / 16);
        cp_async16(sm + tl * mbytes + pc * 16, P.w + (size_t)min(tile0 + tl, ntiles - 1) * tile_b + C::NIB + pc * 16);
      }
    }
  };
  auto issue_x = [&](int n) {                           // streamed activations only
    const int chunk = n % NCHUNK;
    uint8_t* sx = vsm + (n % STAGES) * V::STAGE + V::WBYTES;
    constexpr int PCS = 64 * NBC * 2 / 16;      // 16-byte pieces per (token, range)
    for (int i = tid; i < MT * V::NJ * PCS; i += NTHR) {
      const int c = i % PCS, j = (i / PCS) % V::NJ, m = i / (PCS * V::NJ);
      cp_async16(sx + m * V::XSTRIDE + j * (64 * NBC * 2) + c * 16,
                 P.x_t + (size_t)m * K + j * (K / V::NJ) + chunk * (64 * NBC) + c * 8);
    }
  };
  // weights and scales do not depend on the previous kernel: they are in flight before its results are awaited
  pdl_trigger();
  for (int s = 0; s < STAGES - 1; s++)
    if (s < nitems) issue_w(s);
  pdl_wait();
  if (XRES) {
    for (int i = tid; i < MT * (K / 8); i += NTHR) {
      const int m = i / (K / 8), c = i % (K / 8);
      cp_async16(s_x + m * V::XRS + c * 16, P.x_t + (size_t)m * K + c * 8);
    }
  }
  for (int s = 0; s < STAGES - 1; s++) {
    if (!XRES && s < nitems) issue_x(s);
    cp_async_commit();
  }
  // this lane's two weight rows of the 16-row block and their word slots
  const int row_lo = mb * 16 + g, row_hi = row_lo + 8;
  const int slot_lo = RT == 16 ? 4 * g + t : 4 * (row_lo % RT + RT * pg) + t;
  const int slot_hi = RT == 16 ? slot_lo : 4 * (row_hi % RT + RT * pg) + t;
  const int tl_lo = RT == 16 ? mb : row_lo / RT, tl_hi = RT == 16 ? mb : row_hi / RT;
  const int jA = pg, jB = pg + V::PG;                  // ranges of the low / high nibbles (RT == 16: one range)
  const int moff_lo = (row_lo / RT) * mbytes + (row_lo % RT) * 2, moff_hi = (row_hi / RT) * mbytes + (row_hi % RT) * 2;
  float ct[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int e = 0; e < 4; e++) ct[j][e] = 0.f;
  for (int n = 0; n < nitems; n++) {
    const int c = n % NCHUNK, bi = n / NCHUNK;
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (n + STAGES - 1 < nitems) {
      issue_w(n + STAGES - 1);
      if (!XRES) issue_x(n + STAGES - 1);
    }
    cp_async_commit();
    const uint8_t* sw = vsm + (n % STAGES) * V::STAGE;
    const uint8_t* sx = XRES ? s_x : sw + V::WBYTES;
    const uint8_t* sm = s_meta + (bi % V::MDEPTH) * V::MB1;
    const int sc0 = kq * SPW;                           // first chunk-local step of this warp
    uint32_t w1[SPW], w2[SPW];
#pragma unroll
    for (int k = 0; k < SPW; k++) {
      const int sc = sc0 + k, b = sc >> 2, i = sc & 3;
      w1[k] = *reinterpret_cast<const uint32_t*>(sw + ((tl_lo * NBC + b) * 32 + slot_lo) * 16 + i * 4);
      w2[k] = RT == 16 ? w1[k] : *reinterpret_cast<const uint32_t*>(sw + ((tl_hi * NBC + b) * 32 + slot_hi) * 16 + i * 4);
    }
    const int round = (c * NBC) >> 1;                   // the chunk lies inside one round (8 steps) of every range
#pragma unroll
    for (int pass = 0; pass < (RT == 16 ? 1 : 2); pass++) {
      const int jr = pass == 0 ? jA : jB;
      float cg[NT][4];                                  // the first step's MMA starts them from zero
      float xsum[NT][2];
      if (hz) {
#pragma unroll
        for (int j = 0; j < NT; j++) xsum[j][0] = xsum[j][1] = 0.f;
      }
      // first byte of this range's columns of the chunk inside a token row
      const int xoff = XRES ? (jr * (K / V::NJ) + c * (64 * NBC)) * 2 : jr * (64 * NBC * 2);
      constexpr int XS = XRES ? V::XRS : V::XSTRIDE;
#pragma unroll
      for (int k = 0; k < SPW; k++) {
        const int sc = sc0 + k;
        const int sl = (sc & ~3) | ((sc + jr) & 3);     // this range's local step inside the chunk
        uint32_t a[4];
        if (RT == 16) {
          a[0] = cvt_lo(w1[k]); a[1] = cvt_hi(w1[k]); a[2] = cvt_lo(w1[k] >> 8); a[3] = cvt_hi(w1[k] >> 8);
        } else if (pass == 0) {
          a[0] = cvt_lo(w1[k]); a[1] = cvt_lo(w2[k]); a[2] = cvt_lo(w1[k] >> 8); a[3] = cvt_lo(w2[k] >> 8);
        } else {
          a[0] = cvt_hi(w1[k]); a[1] = cvt_hi(w2[k]); a[2] = cvt_hi(w1[k] >> 8); a[3] = cvt_hi(w2[k] >> 8);
        }
        const uint8_t* xw = sx + xoff + sl * 32;
#pragma unroll
        for (int j = 0; j < NT; j++) {
          const uint2 b = *reinterpret_cast<const uint2*>(xw + (j * 8 + g) * XS + t * 8);
          if (k == 0) mma_bf16_first(cg[j], a, b.x, b.y);
          else mma_bf16(cg[j], a, b.x, b.y);
        }
        if (hz) {
          // token sums for the z * sum(x) term: C fragment column pair (2t, 2t+1) of n-tile j = tokens j*8+2t, +1
#pragma unroll
          for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
              const uint4* xr = reinterpret_cast<const uint4*>(xw + (j * 8 + 2 * t + e) * XS);
              const uint4 v0 = xr[0], v1 = xr[1];
              xsum[j][e] += bflo(v0.x) + bfhi(v0.x) + bflo(v0.y) + bfhi(v0.y) + bflo(v0.z) + bfhi(v0.z) + bflo(v0.w) + bfhi(v0.w) +
                            bflo(v1.x) + bfhi(v1.x) + bflo(v1.y) + bfhi(v1.y) + bflo(v1.z) + bfhi(v1.z) + bflo(v1.w) + bfhi(v1.w);
            }
        }
      }
      const int grp = jr * C::RG + round;
      // rows g / g+8 of the block; RT == 16 mixes low (x64) and high (x4) nibbles in one MMA
      const float f_lo = (RT == 16 || pass == 0) ? 64.f : 4.f, f_hi = (RT == 16) ? 4.f : f_lo;
      const uint16_t* m_lo = reinterpret_cast<const uint16_t*>(sm + moff_lo);
      const uint16_t* m_hi = reinterpret_cast<const uint16_t*>(sm + moff_hi);
      const float s_lo = bf2f(m_lo[grp * RT]) * f_lo, s_hi = bf2f(m_hi[grp * RT]) * f_hi;
#pragma unroll
      for (int j = 0; j < NT; j++) {
        ct[j][0] = fmaf(s_lo, cg[j][0], ct[j][0]); ct[j][1] = fmaf(s_lo, cg[j][1], ct[j][1]);
        ct[j][2] = fmaf(s_hi, cg[j][2], ct[j][2]); ct[j][3] = fmaf(s_hi, cg[j][3], ct[j][3]);
      }
      if (hz) {
        const float z_lo = bf2f(m_lo[(G + grp) * RT]), z_hi = bf2f(m_hi[(G + grp) * RT]);
#pragma unroll
        for (int j = 0; j < NT; j++) {
          ct[j][0] = fmaf(z_lo, xsum[j][0], ct[j][0]); ct[j][1] = fmaf(z_lo, xsum[j][1], ct[j][1]);
          ct[j][2] = fmaf(z_hi, xsum[j][0], ct[j][2]); ct[j][3] = fmaf(z_hi, xsum[j][1], ct[j][3]);
        }
      }
    }
    if (c != NCHUNK - 1) continue;
    // ---- the block is complete: its 4 roles meet in shared memory: y[r][m], r < 32, m < MT ----
    const int row0 = ((int)blockIdx.x + bi * (int)gridDim.x) * ROWS;
#pragma unroll
    for (int j = 0; j < NT; j++) {
      float* base = red + ((size_t)role * ROWS + mb * 16) * MT + j * 8 + 2 * t;
      base[(size_t)g * MT] = ct[j][0]; base[(size_t)g * MT + 1] = ct[j][1];
      base[(size_t)(g + 8) * MT] = ct[j][2]; base[(size_t)(g + 8) * MT + 1] = ct[j][3];
#pragma unroll
      for (int e = 0; e < 4; e++) ct[j][e] = 0.f;
    }
    __syncthreads();
    auto Y = [&](int r, int m) {
      float v = red[(size_t)r * MT + m];
  #pragma unroll
      for (int k = 1; k < V::NROLE; k++) v += red[((size_t)k * ROWS + r) * MT + m];
      return v;
    };
      if (EPI == EPI_RESID) {
      for (int o = tid; o < ROWS * MT; o += NTHR) {
        const int r = o % ROWS, m = o / ROWS, row = row0 + r;
        if (row < P.rows && m < P.M) {
          uint16_t* hp = P.h + (size_t)m * P.out_ld + row;
          *hp = f2bf(bf2f(*hp) + Y(r, m) * P.resid);
        }
      }
    } else if (EPI == EPI_LOGITS) {
      for (int o = tid; o < ROWS * MT; o += NTHR) {
        const int r = o % ROWS, m = o / ROWS, row = row0 + r;
        if (row < P.rows && m < P.M) P.logits[(size_t)m * P.out_ld + row] = Y(r, m) / P.logits_scaling;
      }
    } else if (EPI == EPI_SWIGLU) {
      for (int o = tid; o < (ROWS / 2) * MT; o += NTHR) {
        const int pr = o % (ROWS / 2), m = o / (ROWS / 2), row = row0 + 2 * pr;
        if (row < P.rows && m < P.M) {
          const float gg = rbf(Y(2 * pr, m)), uu = rbf(Y(2 * pr + 1, m));
          P.act_t[(size_t)m * P.out_ld + k16_pos(row >> 1)] = f2bf((gg / (1.0f + __expf(-gg))) * uu);
        }
      }
    } else {   // EPI_QKV: stream rows (2p, 2p+1) of a head are dims (p, p + HD/2); V rows keep their order
      constexpr int HP = HD / 2;
      const int QD = P.n_head * HD;
      for (int o = tid; o < (ROWS / 2) * MT; o += NTHR) {
        const int pr = o % (ROWS / 2), m = o / (ROWS / 2), rs = row0 + 2 * pr;
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
  cp_async_wait<0>();
}

}  // namespace fb
