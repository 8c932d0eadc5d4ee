// The persistent cooperative decode megakernel and the stand-alone GEMV that shares its weight pipeline.
//
// One CTA per SM: warp 16 (lane 0) is the producer, it walks the CTA's static list of weight tiles for the whole
// step and issues 1-D bulk copies into an 8-stage shared-memory ring; it never waits for activations, so weights
// for the next phase stream in while the consumers sit in a grid barrier. Warps 0..15 are consumers in 4 groups.
#pragma once
#include "fb_common.cuh"

namespace fb {

struct Pipe {
  uint8_t* stages;
  uint64_t* full;
  uint64_t* empty;
  uint32_t it;       // running tile counter; producer and consumers walk the same sequence
  uint32_t max_fly;  // producer only: bulk copies allowed in flight at once (<= kStages)
};

struct Smem {
  uint8_t* stages;
  uint8_t* scratch;
  uint16_t* x_s;       // bf16 activations of the current phase
  float* res_s;        // per-row results of the current phase
  uint64_t* full;
  uint64_t* empty;
  volatile int* s_abort;
  float* red;          // 32 floats for block reductions
  int* misc;           // 32 ints
  float* part;         // [groups][2][4 warps][4] slice partials of sliced-K phases
  float* hown;         // [kMaxOwnRows] this CTA's rows of the residual stream
  float* qpart;        // [kStages][2 blocks][4 slices][4 rows] slice partials of the block-queue GEMV
  int* tdone;          // [kStages] units finished per tile in flight
  int* bcnt;           // [kStages][2] slices finished per block
};

__device__ __forceinline__ Smem carve_smem(uint8_t* base) {
  Smem s;
  s.stages = base;
  s.scratch = base + kStages * kStageBytes;
  s.x_s = reinterpret_cast<uint16_t*>(s.scratch);
  s.res_s = reinterpret_cast<float*>(s.scratch + kXBytes);
  uint8_t* tail = s.scratch + kScratchBytes;
  s.full = reinterpret_cast<uint64_t*>(tail);
  s.empty = s.full + kStages;
  s.s_abort = reinterpret_cast<volatile int*>(tail + 128);
  s.red = reinterpret_cast<float*>(tail + 256);
  s.misc = reinterpret_cast<int*>(tail + 384);
  s.part = reinterpret_cast<float*>(tail + 512);
  s.hown = reinterpret_cast<float*>(tail + 1024);
  s.qpart = reinterpret_cast<float*>(tail + 2048);
  s.tdone = reinterpret_cast<int*>(tail + 3072);
  s.bcnt = reinterpret_cast<int*>(tail + 3104);
  return s;
}

// rows [r0, r1) of a phase that CTA b of G owns; `unit` rows stay together (2 for RoPE / gate-up pairs)
__device__ __forceinline__ void cta_rows(int rows, int unit, int b, int G, int& r0, int& r1) {
  const long long nu = rows / unit;
  r0 = (int)((nu * b) / G) * unit;
  r1 = (int)((nu * (b + 1)) / G) * unit;
}

// ------------------------------------------------------------------------------------------------ producer side
__device__ __forceinline__ bool produce_rows(Pipe& p, const uint8_t* src, int nrows, int tile_rows, int rec,
                                             const WaitCtl& wc, int layer) {
  for (int r = 0; r < nrows; r += tile_rows) {
    const int n = min(tile_rows, nrows - r);
    const uint32_t bytes = (uint32_t)n * rec;
    const int s = p.it % kStages;
    const uint32_t ph = (p.it / kStages) & 1;
    if (!mbar_wait(&p.empty[s], ph ^ 1, wc, W_EMPTY, layer)) return false;   // p.it counts issued tiles only
    // Keep the memory system's queues short: with the whole ring in flight (27 MB over 148 SMs) every small
    // latency-critical access of the consumers (flags, tagged words) waits microseconds behind bulk weight traffic.
    if (p.it >= p.max_fly) {
      const uint32_t j = p.it - p.max_fly;
      if (!mbar_wait(&p.full[j % kStages], (j / kStages) & 1, wc, W_FULL, layer)) return false;
    }
    mbar_expect_tx(&p.full[s], bytes);
    bulk_g2s(p.stages + (size_t)s * kStageBytes, src + (size_t)r * rec, bytes, &p.full[s]);
    p.it++;
  }
  return true;
}

// Before the CTA may exit, every bulk copy it issued must have landed. In a clean run the consumers have already
// waited for all of them; after a failed wait the last (up to) kStages issued tiles may still be in flight.
__device__ __forceinline__ void producer_drain(Pipe& p, const WaitCtl& wc) {
  if (*wc.s_abort == 0) return;
  const uint32_t n = p.it < (uint32_t)kStages ? p.it : (uint32_t)kStages;
  for (uint32_t k = 0; k < n; k++) {
    const uint32_t it = p.it - 1 - k;
    const int s = it % kStages;
    const uint32_t ph = (it / kStages) & 1;
    for (unsigned i = 0; i < wc.limit; i++) {
      if (mbar_try(&p.full[s], ph)) break;
      if ((i & 1023) == 1023) __nanosleep(64);
    }
  }
}

// ------------------------------------------------------------------------------------------------ consumer side
// GEMV over this CTA's `nrows` rows of one phase. Results land in res_s[row * KS + slice].
template <class KC, bool HZ>
__device__ __forceinline__ void consume_rows(Pipe& p, int nrows, const XRegs<KC>& x, float* res_s, int cw, int lane,
                                             const WaitCtl& wc, int layer) {
  constexpr int RB = KC::RB, TR = KC::TILE_ROWS;
  const int grp = cw >> 2, wg = cw & 3;
  const int slice = wg % KC::KS, sub = wg / KC::KS;
  const int rec = rec_bytes_of(KC::K, HZ);
  const int ntiles = (nrows + TR - 1) / TR;
  for (int t = 0; t < ntiles; t++) {
    const uint32_t it = p.it + t;
    if ((int)(it % kGroups) != grp) continue;
    const int s = it % kStages;
    const uint32_t ph = (it / kStages) & 1;
    const bool ok = mbar_wait(&p.full[s], ph, wc, W_FULL, layer);
    const int row0 = t * TR;
    const int tr = min(TR, nrows - row0);
    const uint8_t* tile = p.stages + (size_t)s * kStageBytes;
    if (ok) {
      for (int b = sub; b * RB < tr; b += KC::NSUB) {
        int rows[RB];
#pragma unroll
        for (int r = 0; r < RB; r++) rows[r] = min(b * RB + r, tr - 1) * rec;
        float acc[RB];
#pragma unroll
        for (int r = 0; r < RB; r++) acc[r] = 0.f;
        rowblock_dot<KC, HZ>(tile, rows, slice, lane, x, acc);
        const float c = reduce_rows<RB>(acc, lane);
        const int r = lane >> 3;
        if ((lane & 7) == 0 && r < RB && b * RB + r < tr) res_s[(row0 + b * RB + r) * KC::KS + slice] = c;
      }
    }
    named_bar_sync(kBarGroup0 + grp, kWarpsPerGroup * 32);   // the group's 4 warps are done with this tile
    if (ok && wg == 0 && lane == 0) mbar_arrive(&p.empty[s]);
  }
  p.it += ntiles;
}

// sum of slice partials of local row r
template <class KC>
__device__ __forceinline__ float row_result(const float* res_s, int r) {
  float v = res_s[r * KC::KS];
#pragma unroll
  for (int s = 1; s < KC::KS; s++) v += res_s[r * KC::KS + s];
  return v;
}

// ---- activation staging: every consumer thread calls; ends with a consumer-wide barrier ----
__device__ __forceinline__ void stage_x_plain(const uint16_t* gx, int K, uint16_t* x_s, int tid_c) {
  const int n16 = K / 8;
  for (int j = tid_c; j < n16; j += kConsumerThreads)
    reinterpret_cast<uint4*>(x_s)[j] = ld_cg_v4(reinterpret_cast<const uint4*>(gx) + j);
  named_bar_sync(kBarConsumers, kConsumerThreads);
}

// xn = bf16( (float(h) * r) * float(w) ), r = 1/sqrt(mean(h^2) + eps); up to 2 eight-value chunks per thread
__device__ __forceinline__ void stage_x_norm(const uint16_t* gh, const uint16_t* gw, int D, float eps, uint16_t* x_s,
                                             float* red, int tid_c) {
  const int n16 = D / 8;
  uint4 hv[2], wv[2];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 2; c++) {
    const int j = tid_c + c * kConsumerThreads;
    hv[c] = make_uint4(0, 0, 0, 0); wv[c] = make_uint4(0, 0, 0, 0);
    if (j < n16) {
      hv[c] = ld_cg_v4(reinterpret_cast<const uint4*>(gh) + j);
      wv[c] = __ldg(reinterpret_cast<const uint4*>(gw) + j);
    }
  }
#pragma unroll
  for (int c = 0; c < 2; c++) {
    const float hf[8] = {bflo(hv[c].x), bfhi(hv[c].x), bflo(hv[c].y), bfhi(hv[c].y), bflo(hv[c].z), bfhi(hv[c].z), bflo(hv[c].w), bfhi(hv[c].w)};
#pragma unroll
    for (int e = 0; e < 8; e++) ss = fmaf(hf[e], hf[e], ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid_c & 31) == 0) red[tid_c >> 5] = ss;
  named_bar_sync(kBarConsumers, kConsumerThreads);
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kConsumerWarps; w++) tot += red[w];
  const float r = 1.0f / sqrtf(tot / (float)D + eps);
#pragma unroll
  for (int c = 0; c < 2; c++) {
    const int j = tid_c + c * kConsumerThreads;
    if (j < n16) {
      const float hf[8] = {bflo(hv[c].x), bfhi(hv[c].x), bflo(hv[c].y), bfhi(hv[c].y), bflo(hv[c].z), bfhi(hv[c].z), bflo(hv[c].w), bfhi(hv[c].w)};
      const float wf[8] = {bflo(wv[c].x), bfhi(wv[c].x), bflo(wv[c].y), bfhi(wv[c].y), bflo(wv[c].z), bfhi(wv[c].z), bflo(wv[c].w), bfhi(wv[c].w)};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const uint32_t lo = f2bf(hf[2 * e] * r * wf[2 * e]), hi = f2bf(hf[2 * e + 1] * r * wf[2 * e + 1]);
        o[e] = lo | (hi << 16);
      }
      reinterpret_cast<uint4*>(x_s)[j] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  named_bar_sync(kBarConsumers, kConsumerThreads);
}

// ------------------------------------------------------------------------------------------------ grid barrier
struct GridBar {
  unsigned* ctr;
  unsigned target;   // meaningful in consumer thread 0 only
};

// All 512 consumer threads call. Release/acquire at gpu scope through one counter; the wait is bounded.
__device__ __forceinline__ void grid_barrier(GridBar& gb, const WaitCtl& wc, int tid_c, int layer) {
  named_bar_sync(kBarConsumers, kConsumerThreads);
  if (tid_c == 0) {
    gb.target += gridDim.x;
    if (*wc.s_abort == 0) {
      __threadfence();
      red_release_add(gb.ctr, 1u);
      bool done = false;
      unsigned seen = 0;
      for (unsigned i = 0; i < wc.limit; i++) {
        seen = ld_acquire_u32(gb.ctr);
        if ((int)(seen - gb.target) >= 0) { done = true; break; }
        if ((i & 255) == 255) {
          if (ld_volatile_s32(&wc.st->abort)) { *wc.s_abort = 1; break; }
          __nanosleep(32);
        }
      }
      if (!done && *wc.s_abort == 0) report_fail(wc, W_GRIDBAR, layer, (int)gb.target, (int)seen);
      __threadfence();
    }
  }
  named_bar_sync(kBarConsumers, kConsumerThreads);
}

// ------------------------------------------------------------------------------------------------ attention
// GQA flash-decode for one (kv head, chunk of positions) item per CTA. A row of K or V (HD bf16) is spread over
// HD/8 lanes (16 bytes each); a warp handles 32/SEG positions per step, its 16 warps stride through the chunk.
// The R query heads of the group share every K/V load.
template <int HD, int R>
struct AttnCfg {
  static constexpr int LPR = HD / 8;
  static constexpr int SEG = LPR <= 8 ? 8 : 16;
  static constexpr int PPW = 32 / SEG;
  static_assert(HD % 8 == 0 && LPR <= 16, "head_dim must be a multiple of 8 and <= 128");
};

struct AttnArgs {
  const uint16_t* qbuf;   // bf16 [NH*HD], post-RoPE queries of this step
  const uint16_t* kc;     // layer base: bf16 [max_seq, NKV, HD]
  const uint16_t* vc;
  uint16_t* ao;           // bf16 [NH*HD]
  float *pm, *pd, *pacc;  // chunk partials [NH, nchunks], [NH, nchunks, HD]
  int nkv, T, nchunks;
  float scale;
};

template <int HD, int R>
__device__ __forceinline__ void attn_phase(const AttnArgs& a, uint8_t* scratch, int cw, int lane, int tid_c) {
  using C = AttnCfg<HD, R>;
  float* wacc = reinterpret_cast<float*>(scratch);                 // [16][R][HD]
  float* wm = wacc + kConsumerWarps * R * HD;                      // [16][R]
  float* wd = wm + kConsumerWarps * R;                             // [16][R]
  const int items = a.nkv * a.nchunks;
  const int chunk_len = (a.T + a.nchunks - 1) / a.nchunks;
  const int seg = lane / C::SEG, sl = lane % C::SEG;
  const bool active = sl < C::LPR;
  const int d0 = sl * 8;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int kvh = item / a.nchunks, c = item % a.nchunks;
    const int t0 = c * chunk_len, t1 = min(a.T, t0 + chunk_len);
    float q[R][8];
#pragma unroll
    for (int r = 0; r < R; r++) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (active) v = ld_cg_v4(a.qbuf + (size_t)(kvh * R + r) * HD + d0);
      q[r][0] = bflo(v.x); q[r][1] = bfhi(v.x); q[r][2] = bflo(v.y); q[r][3] = bfhi(v.y);
      q[r][4] = bflo(v.z); q[r][5] = bfhi(v.z); q[r][6] = bflo(v.w); q[r][7] = bfhi(v.w);
    }
    float m[R], den[R], acc[R][8];
#pragma unroll
    for (int r = 0; r < R; r++) {
      m[r] = -1e30f; den[r] = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) acc[r][e] = 0.f;
    }
    for (int tb = t0 + cw * C::PPW; tb < t1; tb += kConsumerWarps * C::PPW) {
      const int t = tb + seg;
      const bool valid = t < t1;
      uint4 kk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
      if (valid && active) {
        const size_t off = ((size_t)t * a.nkv + kvh) * HD + d0;
        kk = ld_cg_v4(a.kc + off);
        vv = ld_cg_v4(a.vc + off);
      }
      const float kf[8] = {bflo(kk.x), bfhi(kk.x), bflo(kk.y), bfhi(kk.y), bflo(kk.z), bfhi(kk.z), bflo(kk.w), bfhi(kk.w)};
      const float vf[8] = {bflo(vv.x), bfhi(vv.x), bflo(vv.y), bfhi(vv.y), bflo(vv.z), bfhi(vv.z), bflo(vv.w), bfhi(vv.w)};
#pragma unroll
      for (int r = 0; r < R; r++) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) s = fmaf(q[r][e], kf[e], s);
#pragma unroll
        for (int o = C::SEG / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        s *= a.scale;
        if (valid) {
          const float m2 = fmaxf(m[r], s);
          const float corr = __expf(m[r] - m2), w = __expf(s - m2);
          den[r] = den[r] * corr + w;
#pragma unroll
          for (int e = 0; e < 8; e++) acc[r][e] = acc[r][e] * corr + w * vf[e];
          m[r] = m2;
        }
      }
    }
    // merge the warp's segments (positions were interleaved over segments)
#pragma unroll
    for (int off = C::SEG; off < 32; off <<= 1) {
#pragma unroll
      for (int r = 0; r < R; r++) {
        const float mo = __shfl_xor_sync(0xffffffffu, m[r], off);
        const float dn = __shfl_xor_sync(0xffffffffu, den[r], off);
        const float gm = fmaxf(m[r], mo);
        const float wa = __expf(m[r] - gm), wb = __expf(mo - gm);
        den[r] = den[r] * wa + dn * wb;
#pragma unroll
        for (int e = 0; e < 8; e++) {
          const float ao_ = __shfl_xor_sync(0xffffffffu, acc[r][e], off);
          acc[r][e] = acc[r][e] * wa + ao_ * wb;
        }
        m[r] = gm;
      }
    }
    if (seg == 0 && active) {
#pragma unroll
      for (int r = 0; r < R; r++) {
        float* dst = wacc + ((size_t)cw * R + r) * HD + d0;
#pragma unroll
        for (int e = 0; e < 8; e++) dst[e] = acc[r][e];
        if (sl == 0) { wm[cw * R + r] = m[r]; wd[cw * R + r] = den[r]; }
      }
    }
    named_bar_sync(kBarConsumers, kConsumerThreads);
    for (int o = tid_c; o < R * HD; o += kConsumerThreads) {
      const int r = o / HD, d = o % HD;
      float gm = -1e30f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; w++) gm = fmaxf(gm, wm[w * R + r]);
      float D = 0.f, A = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; w++) {
        const float e = __expf(wm[w * R + r] - gm);
        D += wd[w * R + r] * e;
        A += wacc[((size_t)w * R + r) * HD + d] * e;
      }
      const int qh = kvh * R + r;
      if (a.nchunks == 1) {
        a.ao[(size_t)qh * HD + d] = f2bf(A / D);
      } else {
        a.pacc[((size_t)qh * a.nchunks + c) * HD + d] = A;
        if (d == 0) { a.pm[qh * a.nchunks + c] = gm; a.pd[qh * a.nchunks + c] = D; }
      }
    }
    named_bar_sync(kBarConsumers, kConsumerThreads);
  }
}

// merge the chunk partials of every query head (one warp per head)
template <int HD>
__device__ __forceinline__ void attn_merge_phase(const AttnArgs& a, int n_head, int cw, int lane) {
  for (int qh = blockIdx.x * kConsumerWarps + cw; qh < n_head; qh += gridDim.x * kConsumerWarps) {
    float gm = -1e30f;
    for (int c = 0; c < a.nchunks; c++) gm = fmaxf(gm, ld_cg_f32(a.pm + qh * a.nchunks + c));
    float D = 0.f;
    for (int c = 0; c < a.nchunks; c++) D += ld_cg_f32(a.pd + qh * a.nchunks + c) * __expf(ld_cg_f32(a.pm + qh * a.nchunks + c) - gm);
    for (int d = lane; d < HD; d += 32) {
      float A = 0.f;
      for (int c = 0; c < a.nchunks; c++)
        A += ld_cg_f32(a.pacc + ((size_t)qh * a.nchunks + c) * HD + d) * __expf(ld_cg_f32(a.pm + qh * a.nchunks + c) - gm);
      a.ao[(size_t)qh * HD + d] = f2bf(A / D);
    }
  }
}

// ------------------------------------------------------------------------------------------------ decode kernel
struct DecodeParams {
  const uint8_t *w_qkv, *w_o, *w_gu, *w_d, *w_lm;      // streaming layout
  const uint16_t *n1, *n2, *nf, *embed;
  const float* invf;                                    // fp32 [HD/2] inverse RoPE frequencies
  uint16_t *kc, *vc;                                    // bf16 [L, max_seq, NKV, HD]
  uint16_t *h, *qbuf, *ao, *act;                        // global scratch (L2 resident)
  float *pm, *pd, *pacc;
  float* cand_val;
  int* cand_idx;
  unsigned* bar_ctr;
  DevStatus* status;
  const int32_t* d_token;
  uint16_t* d_h;                                        // optional caller residual in/out
  float* d_logits;
  int32_t* d_next;
  int32_t token, pos, max_seq;
  int32_t n_layer, dim, n_head, n_kv, ffn, vocab, nchunks;
  unsigned bar_base, spin_limit;
  float eps, attn_scale, resid, emb_mult, logits_scaling;
  long long* prof;                                      // optional phase stamps
  unsigned max_fly;
};

template <class KD, class KF, int HD, int R, bool HZ>
__global__ void __launch_bounds__(kThreads, 1) decode_mega(const DecodeParams P) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Smem sm = carve_smem(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, b = blockIdx.x;
  if (tid == 0) {
    for (int s = 0; s < kStages; s++) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    *sm.s_abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  WaitCtl wc{P.status, sm.s_abort, P.spin_limit};
  Pipe pipe{sm.stages, sm.full, sm.empty, 0u, P.max_fly};

  const int D = P.dim, FF = P.ffn, L = P.n_layer, V = P.vocab;
  const int QKV = (P.n_head + 2 * P.n_kv) * HD;
  const int recD = rec_bytes_of(KD::K, HZ), recF = rec_bytes_of(KF::K, HZ);
  int q0, q1, o0, o1, g0, g1, d0r, d1r, l0, l1;
  cta_rows(QKV, 2, b, G, q0, q1);
  cta_rows(D, 1, b, G, o0, o1);
  cta_rows(2 * FF, 2, b, G, g0, g1);
  cta_rows(D, 1, b, G, d0r, d1r);
  cta_rows(V, 1, b, G, l0, l1);

  if (warp == kConsumerWarps) {
    // ================================ producer ================================
    if (lane == 0) {
      bool ok = true;
      for (int l = 0; l < L && ok; l++) {
        ok = produce_rows(pipe, P.w_qkv + ((size_t)l * QKV + q0) * recD, q1 - q0, KD::TILE_ROWS, recD, wc, l) &&
             produce_rows(pipe, P.w_o + ((size_t)l * D + o0) * recD, o1 - o0, KD::TILE_ROWS, recD, wc, l) &&
             produce_rows(pipe, P.w_gu + ((size_t)l * 2 * FF + g0) * recD, g1 - g0, KD::TILE_ROWS, recD, wc, l) &&
             produce_rows(pipe, P.w_d + ((size_t)l * D + d0r) * recF, d1r - d0r, KF::TILE_ROWS, recF, wc, l);
      }
      if (ok) produce_rows(pipe, P.w_lm + (size_t)l0 * recD, l1 - l0, KD::TILE_ROWS, recD, wc, L);
      producer_drain(pipe, wc);
    }
  } else {
    // ================================ consumers ================================
    const int cw = warp, tid_c = tid;
    const int wg = cw & 3;
    GridBar gb{P.bar_ctr, P.bar_base};
    // ---- embedding (or caller-supplied residual) -> h ----
    {
      int tok = P.d_token ? (int)ld_cg_u32(P.d_token) : P.token;
      if ((unsigned)tok >= (unsigned)V) {
        tok = 0;
        if (tid_c == 0 && b == 0) atomicCAS(&P.status->code, 0, 6 /*FB_ERR_RANGE*/);
      }
      for (int i = b * kConsumerThreads + tid_c; i < D; i += G * kConsumerThreads) {
        if (P.d_h) P.h[i] = ld_cg_u16(P.d_h + i);
        else P.h[i] = f2bf(bf2f(__ldg(P.embed + (size_t)tok * D + i)) * P.emb_mult);
      }
    }
    grid_barrier(gb, wc, tid_c, -1);

    XRegs<KD> xd;
#define FB_STAMP(i) do { if (P.prof && tid_c == 0) P.prof[((size_t)b * L + l) * 16 + (i)] = (long long)globaltimer_ns(); } while (0)
    for (int l = 0; l < L; l++) {
      uint16_t* kcl = P.kc + (size_t)l * P.max_seq * P.n_kv * HD;
      uint16_t* vcl = P.vc + (size_t)l * P.max_seq * P.n_kv * HD;
      // ---- QKV: norm1 -> GEMV -> RoPE -> q scratch / KV append ----
      FB_STAMP(0);
      stage_x_norm(P.h, P.n1 + (size_t)l * D, D, P.eps, sm.x_s, sm.red, tid_c);
      load_x_slice<KD>(sm.x_s, wg % KD::KS, lane, xd);
      FB_STAMP(1);
      consume_rows<KD, HZ>(pipe, q1 - q0, xd, sm.res_s, cw, lane, wc, l);
      named_bar_sync(kBarConsumers, kConsumerThreads);
      FB_STAMP(2);
      for (int pr = tid_c; pr < (q1 - q0) / 2; pr += kConsumerThreads) {
        const float a = row_result<KD>(sm.res_s, 2 * pr), c = row_result<KD>(sm.res_s, 2 * pr + 1);
        const int rs = q0 + 2 * pr;
        const int head = rs / HD, within = rs % HD;
        if (head < P.n_head + P.n_kv) {
          const int i = within >> 1;
          const float x0 = rbf(a), x1 = rbf(c);
          float sn, cs;
          sincosf((float)P.pos * __ldg(P.invf + i), &sn, &cs);
          const uint16_t y0 = f2bf(x0 * cs - x1 * sn), y1 = f2bf(x1 * cs + x0 * sn);
          if (head < P.n_head) {
            P.qbuf[head * HD + i] = y0;
            P.qbuf[head * HD + i + HD / 2] = y1;
          } else {
            uint16_t* kr = kcl + ((size_t)P.pos * P.n_kv + (head - P.n_head)) * HD;
            kr[i] = y0;
            kr[i + HD / 2] = y1;
          }
        } else {
          uint16_t* vr = vcl + ((size_t)P.pos * P.n_kv + (head - P.n_head - P.n_kv)) * HD;
          vr[within] = f2bf(a);
          vr[within + 1] = f2bf(c);
        }
      }
      grid_barrier(gb, wc, tid_c, l);
      FB_STAMP(3);
      // ---- attention ----
      AttnArgs aa{P.qbuf, kcl, vcl, P.ao, P.pm, P.pd, P.pacc, P.n_kv, P.pos + 1, P.nchunks, P.attn_scale};
      attn_phase<HD, R>(aa, sm.scratch, cw, lane, tid_c);
      FB_STAMP(4);
      grid_barrier(gb, wc, tid_c, l);
      if (P.nchunks > 1) {
        attn_merge_phase<HD>(aa, P.n_head, cw, lane);
        grid_barrier(gb, wc, tid_c, l);
      }
      FB_STAMP(5);
      // ---- O projection + residual ----
      stage_x_plain(P.ao, D, sm.x_s, tid_c);
      load_x_slice<KD>(sm.x_s, wg % KD::KS, lane, xd);
      FB_STAMP(6);
      consume_rows<KD, HZ>(pipe, o1 - o0, xd, sm.res_s, cw, lane, wc, l);
      named_bar_sync(kBarConsumers, kConsumerThreads);
      FB_STAMP(7);
      for (int r = tid_c; r < o1 - o0; r += kConsumerThreads) {
        const float y = row_result<KD>(sm.res_s, r);
        P.h[o0 + r] = f2bf(bf2f(ld_cg_u16(P.h + o0 + r)) + y * P.resid);
      }
      grid_barrier(gb, wc, tid_c, l);
      FB_STAMP(8);
      // ---- gate/up + SwiGLU ----
      stage_x_norm(P.h, P.n2 + (size_t)l * D, D, P.eps, sm.x_s, sm.red, tid_c);
      load_x_slice<KD>(sm.x_s, wg % KD::KS, lane, xd);
      FB_STAMP(9);
      consume_rows<KD, HZ>(pipe, g1 - g0, xd, sm.res_s, cw, lane, wc, l);
      named_bar_sync(kBarConsumers, kConsumerThreads);
      FB_STAMP(10);
      for (int pr = tid_c; pr < (g1 - g0) / 2; pr += kConsumerThreads) {
        const float gg = rbf(row_result<KD>(sm.res_s, 2 * pr)), uu = rbf(row_result<KD>(sm.res_s, 2 * pr + 1));
        P.act[g0 / 2 + pr] = f2bf((gg / (1.0f + __expf(-gg))) * uu);
      }
      grid_barrier(gb, wc, tid_c, l);
      FB_STAMP(11);
      // ---- down projection + residual ----
      {
        XRegs<KF> xf;
        stage_x_plain(P.act, FF, sm.x_s, tid_c);
        load_x_slice<KF>(sm.x_s, wg % KF::KS, lane, xf);
        FB_STAMP(12);
        consume_rows<KF, HZ>(pipe, d1r - d0r, xf, sm.res_s, cw, lane, wc, l);
      }
      named_bar_sync(kBarConsumers, kConsumerThreads);
      FB_STAMP(13);
      for (int r = tid_c; r < d1r - d0r; r += kConsumerThreads) {
        const float y = row_result<KF>(sm.res_s, r);
        P.h[d0r + r] = f2bf(bf2f(ld_cg_u16(P.h + d0r + r)) + y * P.resid);
      }
      grid_barrier(gb, wc, tid_c, l);
      FB_STAMP(14);
    }
#undef FB_STAMP
    // ---- final norm + LM head + argmax ----
    stage_x_norm(P.h, P.nf, D, P.eps, sm.x_s, sm.red, tid_c);
    load_x_slice<KD>(sm.x_s, wg % KD::KS, lane, xd);
    consume_rows<KD, HZ>(pipe, l1 - l0, xd, sm.res_s, cw, lane, wc, L);
    named_bar_sync(kBarConsumers, kConsumerThreads);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = tid_c; r < l1 - l0; r += kConsumerThreads) {
      const float y = row_result<KD>(sm.res_s, r) / P.logits_scaling;
      if (P.d_logits) P.d_logits[l0 + r] = y;
      if (y > bv) { bv = y; bi = l0 + r; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sm.red[cw] = bv; sm.misc[cw] = bi; }
    named_bar_sync(kBarConsumers, kConsumerThreads);
    if (tid_c == 0) {
      for (int w = 1; w < kConsumerWarps; w++)
        if (sm.red[w] > bv || (sm.red[w] == bv && sm.misc[w] < bi)) { bv = sm.red[w]; bi = sm.misc[w]; }
      P.cand_val[b] = bv;
      P.cand_idx[b] = bi;
    }
    grid_barrier(gb, wc, tid_c, L);
    if (b == 0) {
      if (cw == 0) {
        float v = -INFINITY;
        int ix = 0x7fffffff;
        for (int c = lane; c < G; c += 32) {
          const float ov = ld_cg_f32(P.cand_val + c);
          const int oi = (int)ld_cg_u32(P.cand_idx + c);
          if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, o);
          const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
          if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
        }
        if (lane == 0 && P.d_next) *P.d_next = ix;
      }
      if (P.d_h)
        for (int i = tid_c; i < D; i += kConsumerThreads) P.d_h[i] = ld_cg_u16(P.h + i);
    }
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------------ stand-alone GEMV
struct GemvParams {
  const uint8_t* w;        // streaming layout, `rows` records
  const uint16_t* x;       // bf16 [K]
  float* y;                // f32 [rows], original row order
  DevStatus* status;
  int32_t rows, order, order_arg, order_rows;
  unsigned spin_limit;
};

template <class KC, bool HZ>
__global__ void __launch_bounds__(kThreads, 1) gemv_stream(const GemvParams P) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Smem sm = carve_smem(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < kStages; s++) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    *sm.s_abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  WaitCtl wc{P.status, sm.s_abort, P.spin_limit};
  Pipe pipe{sm.stages, sm.full, sm.empty, 0u, (uint32_t)kStages};
  const int rec = rec_bytes_of(KC::K, HZ);
  int r0, r1;
  cta_rows(P.rows, 1, blockIdx.x, gridDim.x, r0, r1);
  // a CTA's result buffer holds kResFloats/KS rows: walk the CTA's range in passes of that many rows
  constexpr int PASS = (kResFloats / KC::KS) / KC::TILE_ROWS * KC::TILE_ROWS;
  if (warp == kConsumerWarps) {
    if (lane == 0) {
      bool ok = true;
      for (int p0 = r0; p0 < r1 && ok; p0 += PASS)
        ok = produce_rows(pipe, P.w + (size_t)p0 * rec, min(PASS, r1 - p0), KC::TILE_ROWS, rec, wc, 0);
      producer_drain(pipe, wc);
    }
  } else {
    XRegs<KC> x;
    stage_x_plain(P.x, KC::K, sm.x_s, tid);
    load_x_slice<KC>(sm.x_s, (warp & 3) % KC::KS, lane, x);
    for (int p0 = r0; p0 < r1; p0 += PASS) {
      const int n = min(PASS, r1 - p0);
      consume_rows<KC, HZ>(pipe, n, x, sm.res_s, warp, lane, wc, 0);
      named_bar_sync(kBarConsumers, kConsumerThreads);
      for (int r = tid; r < n; r += kConsumerThreads)
        P.y[perm_row(p0 + r, P.order, P.order_arg, P.order_rows)] = row_result<KC>(sm.res_s, r);
      named_bar_sync(kBarConsumers, kConsumerThreads);
    }
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------------ layout kernels
// one CTA per stream row; blockIdx.y = layer (matrices of all layers are stacked, the row order repeats per layer)
__global__ void repack_rows(const uint32_t* q, const uint16_t* s, const uint16_t* z, int rows, int k, int order,
                            int order_arg, int order_rows, uint8_t* out) {
  const int j = blockIdx.x;
  const int src = blockIdx.y * rows + perm_row(j, order, order_arg, order_rows);
  const int rec = rec_bytes_of(k, z != nullptr);
  uint8_t* dst = out + ((size_t)blockIdx.y * rows + j) * rec;
  const int words = k / 8, groups = k / 128;
  for (int i = threadIdx.x; i < words; i += blockDim.x) reinterpret_cast<uint32_t*>(dst)[i] = q[(size_t)src * words + i];
  uint16_t* meta = reinterpret_cast<uint16_t*>(dst + k / 2);
  const int meta_n = (rec - k / 2) / 2;
  for (int i = threadIdx.x; i < meta_n; i += blockDim.x) {
    uint16_t v = 0;
    if (i < groups) v = s[(size_t)src * groups + i];
    else if (z != nullptr && i < 2 * groups) v = z[(size_t)src * groups + (i - groups)];
    meta[i] = v;
  }
}

__global__ void dequant_rows(const uint8_t* in, int rows, int k, int has_zeros, int order, int order_arg, int order_rows,
                             float* out) {
  const int j = blockIdx.x;
  const int dstrow = perm_row(j, order, order_arg, order_rows);
  const int rec = rec_bytes_of(k, has_zeros);
  const uint8_t* src = in + (size_t)j * rec;
  const uint16_t* meta = reinterpret_cast<const uint16_t*>(src + k / 2);
  for (int c = threadIdx.x; c < k; c += blockDim.x) {
    const uint32_t w = reinterpret_cast<const uint32_t*>(src)[c >> 3];
    const float nib = (float)((w >> (4 * (c & 7))) & 0xF) - 8.0f;
    float v = nib * bf2f(meta[c >> 7]);
    if (has_zeros) v = v + bf2f(meta[k / 128 + (c >> 7)]);
    out[(size_t)dstrow * k + c] = v;
  }
}

}  // namespace fb
