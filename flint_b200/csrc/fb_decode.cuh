// Decode megakernel, data-flow synchronisation.
//
// Phases of one token are chained by DATA, not by grid barriers: every vector that crosses CTAs (residual h, q / new
// k / new v, attention output, SwiGLU activations, arg-max candidates) lives in global memory as 8-byte words that
// carry their payload (two bf16 values or one fp32/int32) together with a 32-bit tag unique to (launch, layer,
// phase). A producer stores the word once; a consumer polls the word itself until the tag matches, so the value
// arrives with the same L2 round trip that a barrier would only have announced. Each hop costs about one L2 round
// trip instead of three (barrier arrive, barrier poll, data fetch).
//
// Why single buffers are enough: every phase consumes a vector that ALL CTAs contributed to, so a CTA can only be
// one full phase ahead of the slowest one; a buffer is rewritten two phases after its last reader at the earliest.
#pragma once
#include <cuda.h>

#include "fb_pipe.cuh"

#ifndef FB_ATTN_BATCH
#define FB_ATTN_BATCH 2      // K/V positions a lane group loads before it uses any of them
#endif
#ifndef FB_ATTN_PFD
#define FB_ATTN_PFD 2        // rounds ahead of its loads that a warp asks L2 for its K/V rows
#endif

namespace fb {

// GQA flash-decode geometry: a row of K or V (HD bf16) is spread over HD/8 lanes (16 bytes each); a warp handles
// 32/SEG positions per step. The R query heads of a group share every K/V load.
template <int HD, int R>
struct AttnCfg {
  static constexpr int LPR = HD / 8;
  static constexpr int SEG = LPR <= 8 ? 8 : 16;
  static constexpr int PPW = 32 / SEG;
  // long caches: K/V rows travel through the weight ring, NPS positions per stage (K rows, then V rows)
  static constexpr int NPS = 2 * 64 * HD * 2 <= kStageBytes ? 64 : 32;
  static constexpr int KV_STAGE_BYTES = 2 * NPS * HD * 2;
  static_assert(HD % 8 == 0 && LPR <= 16, "head_dim must be a multiple of 8 and <= 128");
  static_assert(KV_STAGE_BYTES <= kStageBytes && (HD * 2) % 16 == 0, "a ring stage holds one sweep of K and V rows");
};

// ------------------------------------------------------------------------------------------------ tagged words
__device__ __forceinline__ void ll_store(uint64_t* p, uint32_t payload, uint32_t tag) {
  const uint64_t v = ((uint64_t)tag << 32) | payload;
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void ll_load2(const uint64_t* p, uint64_t& a, uint64_t& b) {
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

// words exchanged between GPUs (peer stores over NVLink, polled in local memory): system scope
__device__ __forceinline__ void ll_store_sys(uint64_t* p, uint32_t payload, uint32_t tag) {
  const uint64_t v = ((uint64_t)tag << 32) | payload;
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ll_load_sys(const uint64_t* p) {
  uint64_t a;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
  return a;
}
__device__ __forceinline__ void ll_store2_sys(uint64_t* p, uint32_t pay0, uint32_t pay1, uint32_t tag) {
  const uint64_t a = ((uint64_t)tag << 32) | pay0, b = ((uint64_t)tag << 32) | pay1;
  asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ll_load2_sys(const uint64_t* p, uint64_t& a, uint64_t& b) {
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
// bounded poll of one word written by another GPU; returns the payload (0 after a failure)
__device__ __forceinline__ uint32_t ll_poll_sys(const uint64_t* p, uint32_t tag, const WaitCtl& wc, int layer) {
  for (unsigned spin = 0;; spin++) {
    const uint64_t v = ll_load_sys(p);
    if ((uint32_t)(v >> 32) == tag) return (uint32_t)v;
    if (*wc.s_abort) return 0;
    if ((spin & 255) == 255 && ld_volatile_s32(&wc.st->abort)) { *wc.s_abort = 1; return 0; }
    if (spin >= wc.limit) { report_fail(wc, W_FLAG, layer, (int)tag, -3); return 0; }
  }
}

// Poll `nwords` (even, 16-byte aligned base) tagged words into 32-bit payloads dst[0..nwords). Threads
// tid, tid+nthreads, ... each own word pairs; all of a thread's loads are issued before any is checked.
template <int MAXP>
__device__ __forceinline__ void ll_gather(const uint64_t* src, int nwords, uint32_t tag, uint32_t* dst, int tid,
                                          int nthreads, const WaitCtl& wc, int layer) {
  const int npairs = nwords >> 1;
  uint32_t pending = 0;
#pragma unroll
  for (int k = 0; k < MAXP; k++)
    if (tid + k * nthreads < npairs) pending |= 1u << k;
  for (unsigned spin = 0; pending; spin++) {
    uint64_t a[MAXP], b[MAXP];
#pragma unroll
    for (int k = 0; k < MAXP; k++)
      if (pending & (1u << k)) ll_load2(src + 2 * (size_t)(tid + k * nthreads), a[k], b[k]);
#pragma unroll
    for (int k = 0; k < MAXP; k++)
      if (pending & (1u << k)) {
        if ((uint32_t)(a[k] >> 32) == tag && (uint32_t)(b[k] >> 32) == tag) {
          const int j = 2 * (tid + k * nthreads);
          dst[j] = (uint32_t)a[k];
          dst[j + 1] = (uint32_t)b[k];
          pending &= ~(1u << k);
        }
      }
    if (pending) {
      if (*wc.s_abort) break;
      if (spin > 16) __nanosleep(40);
      if ((spin & 255) == 255 && ld_volatile_s32(&wc.st->abort)) { *wc.s_abort = 1; break; }
      if (spin >= wc.limit) { report_fail(wc, W_FLAG, layer, (int)tag, -1); break; }
    }
  }
}

// Arrival flags: polling the tagged data words directly from 75 000 threads floods the few L2 lines that hold a
// vector, so a CTA first waits (one warp, a handful of coalesced loads per round) until every producer CTA has posted
// its arrival flag, and only then gathers the words. The flag is posted without a fence, so the tags in the words
// stay the correctness check: a word that lags behind its flag is simply polled again.
__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// flags are posted with an atomic exchange: it is performed at L2 at once instead of waiting in the SM's store path
__device__ __forceinline__ void st_relaxed_u32(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.relaxed.gpu.global.exch.b32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  (void)old;
}
// all consumer threads call; warp 0 polls flags[0..n) until each equals tag
#ifndef FB_FLAG_SETS
#define FB_FLAG_SETS 1       // poll rounds kept in flight (staggered): a posted flag is seen after ~RTT/2 + RTT/(2 sets)
#endif
#ifndef FB_FLAG_SLACK_DIV
#define FB_FLAG_SLACK_DIV 3  // the gather starts when all but n / 3 producers have posted (0: wait for every flag). The tagged
#endif                       // words of the stragglers are simply polled again by the gather, so the last flags' round trip
                             // leaves the critical path: measured +2.6 % tokens/s at a third, +1.8 % at a sixth, -0.9 % with
                             // no flag wait at all (every consumer polling words floods L2)
__device__ __forceinline__ void wait_flags(const uint32_t* flags, int n, uint32_t tag, int cw, int lane, const WaitCtl& wc,
                                           int layer) {
  if (cw == 0) {
    constexpr int NS = FB_FLAG_SETS;
    uint32_t v[NS][8];
    // all loads of a round are issued before any is compared (n <= 256: at most 8 per lane)
    auto issue = [&](uint32_t (&d)[8]) {
#pragma unroll
      for (int j = 0; j < 8; j++) d[j] = (lane + 32 * j < n) ? ld_relaxed_u32(flags + lane + 32 * j) : tag;
    };
    auto all_set = [&](const uint32_t (&d)[8]) {
      if constexpr (FB_FLAG_SLACK_DIV == 0) {
        bool ok = true;
#pragma unroll
        for (int j = 0; j < 8; j++) ok = ok && (d[j] == tag);
        return __all_sync(0xffffffffu, ok) != 0;
      } else {
        unsigned miss = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) miss += (d[j] != tag);
        return __reduce_add_sync(0xffffffffu, miss) <= (unsigned)(n / FB_FLAG_SLACK_DIV);
      }
    };
#pragma unroll
    for (int s = 0; s < NS; s++) {
      if (s) __nanosleep(700 / NS);
      issue(v[s]);
    }
    bool done = false;
    for (unsigned spin = 0; !done; spin++) {
#pragma unroll
      for (int s = 0; s < NS; s++) {
        if (!done) {
          if (all_set(v[s])) done = true;
          else issue(v[s]);
        }
      }
      if (done) break;
      int stop = 0;
      if (lane == 0) {
        if (*wc.s_abort) stop = 1;
        else if ((spin & 63) == 63 && ld_volatile_s32(&wc.st->abort)) { *wc.s_abort = 1; stop = 1; }
        else if (spin >= wc.limit) { report_fail(wc, W_FLAG, layer, (int)tag, n); stop = 1; }
      }
      if (__shfl_sync(0xffffffffu, stop, 0)) break;
    }
  }
  named_bar_sync(kBarConsumers, kConsumerThreads);
}
// a warp that has finished its part of a phase calls this; the CTA's last warp posts the flag
__device__ __forceinline__ void post_when_cta_done(int* s_done, uint32_t* flag, uint32_t tag, int lane,
                                                   long long* dbg = nullptr) {
  __syncwarp();
  if (lane == 0) {
    const int old = atomicAdd(s_done, 1);
    if (old == kConsumerWarps - 1) {
      *s_done = 0;
      st_relaxed_u32(flag, tag);
      if (dbg) dbg[12] = (long long)globaltimer_ns();
    }
  }
}

// ------------------------------------------------------------------------------------------------ staging from tagged vectors
// Both functions leave the phase's activations in sm.xh / sm.xf (fp16 in B-operand order + per-group factors) and end
// with a consumer-wide barrier. A thread owns the 4 elements 4*pr .. 4*pr+3 for pr = tid_c, tid_c + kConsumerThreads, ...
// so a warp owns whole groups of 128 and converts them in place.
// xn = bf16( (float(h) * r) * float(w) ) from the tagged residual vector (dim/2 words)
template <int MAXP>
__device__ __forceinline__ void stage_norm_ll(const uint64_t* hll, const uint32_t* flags, int nflags, uint32_t tag,
                                              const uint16_t* gw, int D, float eps, const Smem& sm, int tid_c,
                                              const WaitCtl& wc, int layer, bool have_h, long long* dbg = nullptr) {
  uint32_t* xs32 = reinterpret_cast<uint32_t*>(sm.xh);
  float* red = sm.red;
  const int npairs = D / 4, lane = tid_c & 31;
  uint2 wv[MAXP];                       // norm weights do not depend on the wait: fetch them first
#pragma unroll
  for (int k = 0; k < MAXP; k++) {
    const int pr = tid_c + k * kConsumerThreads;
    wv[k] = pr < npairs ? __ldg(reinterpret_cast<const uint2*>(gw) + pr) : make_uint2(0, 0);
  }
  if (!have_h) {      // layer 0 finds the raw residual (bf16, natural order) already in place
    if (nflags > 0) wait_flags(flags, nflags, tag, tid_c >> 5, lane, wc, layer);
    else named_bar_sync(kBarConsumers, kConsumerThreads);     // every warp has left the phase that read the activations
    if (dbg && tid_c == 0) dbg[10] = (long long)globaltimer_ns();
    ll_gather<MAXP>(hll, D / 2, tag, xs32, tid_c, kConsumerThreads, wc, layer);
    if (dbg && tid_c == 0) dbg[11] = (long long)globaltimer_ns();
  }
  // each thread squares the pairs it gathered itself: no barrier needed before this
  uint2 raw[MAXP];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAXP; k++) {
    const int pr = tid_c + k * kConsumerThreads;
    raw[k] = make_uint2(0, 0);
    if (pr < npairs) {
      const uint32_t a = xs32[2 * pr], b = xs32[2 * pr + 1];
      raw[k] = make_uint2(a, b);
      ss = fmaf(bflo(a), bflo(a), ss); ss = fmaf(bfhi(a), bfhi(a), ss);
      ss = fmaf(bflo(b), bflo(b), ss); ss = fmaf(bfhi(b), bfhi(b), ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) red[tid_c >> 5] = ss;
  named_bar_sync(kBarConsumers, kConsumerThreads);
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kConsumerWarps; w++) tot += red[w];
  const float r = 1.0f / sqrtf(tot / (float)D + eps);
#pragma unroll
  for (int k = 0; k < MAXP; k++) {
    const int pr = tid_c + k * kConsumerThreads;      // warp-uniform bound: npairs is a multiple of 32
    if (pr < npairs) {
      const uint32_t a = raw[k].x, b = raw[k].y;
      const uint32_t o0 = (uint32_t)f2bf(bflo(a) * r * bflo(wv[k].x)) | ((uint32_t)f2bf(bfhi(a) * r * bfhi(wv[k].x)) << 16);
      const uint32_t o1 = (uint32_t)f2bf(bflo(b) * r * bflo(wv[k].y)) | ((uint32_t)f2bf(bfhi(b) * r * bfhi(wv[k].y)) << 16);
      const int grp = pr >> 5;
      stage_group_fp16(o0, o1, sm.xh + grp * 128, sm.xf + grp, lane);
    }
  }
  named_bar_sync(kBarConsumers, kConsumerThreads);
}

template <int MAXP>
__device__ __forceinline__ void stage_plain_ll(const uint64_t* src, const uint32_t* flags, int nflags, uint32_t tag, int K,
                                               const Smem& sm, int tid_c, const WaitCtl& wc, int layer) {
  uint32_t* xs32 = reinterpret_cast<uint32_t*>(sm.xh);
  const int npairs = K / 4, lane = tid_c & 31;
  if (nflags > 0) wait_flags(flags, nflags, tag, tid_c >> 5, lane, wc, layer);
  else named_bar_sync(kBarConsumers, kConsumerThreads);
  ll_gather<MAXP>(src, K / 2, tag, xs32, tid_c, kConsumerThreads, wc, layer);
  // a thread converts exactly the words it gathered itself
#pragma unroll
  for (int k = 0; k < MAXP; k++) {
    const int pr = tid_c + k * kConsumerThreads;
    if (pr < npairs) {
      const uint32_t a = xs32[2 * pr], b = xs32[2 * pr + 1];
      const int grp = pr >> 5;
      stage_group_fp16(a, b, sm.xh + grp * 128, sm.xf + grp, lane);
    }
  }
  named_bar_sync(kBarConsumers, kConsumerThreads);
}

// ------------------------------------------------------------------------------------------------ attention (tagged in/out)
// q and the new k live in "pair-major" tagged words: word (head*HD/2 + p) = (x[p], x[p + HD/2]), which is what one
// RoPE thread produces. A lane owns pairs 4*sl .. 4*sl+3, i.e. dims {4sl..4sl+3} and {HD/2+4sl..+3}.
struct Attn2Args {
  const uint64_t* q_ll;     // [NH * HD/2]
  const uint64_t* k_ll;     // [NKV * HD/2] new key of this step, pair-major
  const uint64_t* v_ll;     // [NKV * HD/2] new value, natural order: word w = (v[2w], v[2w+1])
  uint64_t* ao_ll;          // [NH * HD/2] natural order
  const uint16_t* kc;       // layer base: bf16 [max_seq, NKV, HD]
  const uint16_t* vc;
  uint64_t* part_ll;        // [NKV][maxchunks][R*HD + 2R] tagged chunk partials (acc, then m, then d per head)
  uint32_t* ao_flags;       // [NKV * nchunks] arrival flags of the attention output, one per (kv head, chunk) CTA
  int nkv, pos, nchunks, maxchunks;
  float scale;
  uint32_t tag_in, tag_part, tag_out;
};

template <int HD, int R, bool LONGKV = false>
__device__ __forceinline__ void attn2_phase(const Attn2Args& a, uint8_t* scratch, int* misc, int cw, int lane, int tid_c,
                                            const WaitCtl& wc, int layer, Pipe* pipe = nullptr, int* tdone = nullptr) {
  using C = AttnCfg<HD, R>;
  constexpr int HP = HD / 2;
  float* wacc = reinterpret_cast<float*>(scratch);                 // [CW][R][HD]  (dims in lane order, see below)
  float* wm = wacc + kConsumerWarps * R * HD;                      // [CW][R]
  float* wd = wm + kConsumerWarps * R;                             // [CW][R]
  uint32_t* qs = reinterpret_cast<uint32_t*>(wd + kConsumerWarps * R);   // [R*HP] q pairs, then [HP] k pairs, [HP] v words
  const int T = a.pos + 1;
  const int items = a.nkv * a.nchunks;
  const int chunk_len = (T + a.nchunks - 1) / a.nchunks;
  const int seg = lane / C::SEG, sl = lane % C::SEG;
  const bool active = sl < C::LPR;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int kvh = item / a.nchunks, c = item % a.nchunks;
    const int t0 = c * chunk_len, t1 = min(T, t0 + chunk_len);
    const bool has_new = (a.pos >= t0 && a.pos < t1);     // the chunk that contains this step's own position
    // ---- gather q (R heads) and, for the last chunk, the new k / v ----
    {
      const int nq = R * HP;
      const int total = nq + (has_new ? 2 * HP : 0);
      // one pass: every thread owns at most one word pair of each source
      uint32_t pending = 0;
      const int pr = tid_c;
      if (2 * pr < total) pending = 1;
      for (unsigned spin = 0; pending; spin++) {
        const int w = 2 * pr;
        const uint64_t* src = w < nq ? a.q_ll + (size_t)kvh * R * HP + w
                            : (w < nq + HP ? a.k_ll + (size_t)kvh * HP + (w - nq) : a.v_ll + (size_t)kvh * HP + (w - nq - HP));
        uint64_t u, v;
        ll_load2(src, u, v);
        if ((uint32_t)(u >> 32) == a.tag_in && (uint32_t)(v >> 32) == a.tag_in) {
          qs[w] = (uint32_t)u; qs[w + 1] = (uint32_t)v;
          pending = 0;
        } else {
          if (*wc.s_abort) break;
          if (spin > 16) __nanosleep(40);
          if ((spin & 255) == 255 && ld_volatile_s32(&wc.st->abort)) { *wc.s_abort = 1; break; }
          if (spin >= wc.limit) { report_fail(wc, W_FLAG, layer, (int)a.tag_in, -2); break; }
        }
      }
    }
    named_bar_sync(kBarConsumers, kConsumerThreads);
    if constexpr (LONGKV) {
      // ---- long caches: K/V stages from the ring, tensor-core flash-decode. Warp w takes units (16 positions of a stage)
      // w, w + 14, ...: the R query heads are rows 0..R-1 of one 16-row MMA tile, the positions the N dimension of Q K^T and
      // the K dimension of P V (probabilities as hi + lo bf16 pairs, ~2^-17), running maximum / denominator per row as in the scalar path.
      constexpr int KSTEPS = HD / 16, NTD = HD / 8, NPS = C::NPS, ROWB = HD * 2;
      static_assert(HD % 16 == 0 && NPS % 16 == 0 && R <= 8, "MMA flash-decode geometry");
      const int g = lane >> 2, t = lane & 3;
      uint32_t aq[KSTEPS][4];
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
          const int d = 16 * ks + 2 * t + 8 * hf;           // dims d, d + 1 of head g (pair-major words: (x[p], x[p + HP]))
          uint32_t v = 0;
          if (g < R) {
            const uint32_t w0 = qs[g * HP + (d < HP ? d : d - HP)], w1 = qs[g * HP + (d + 1 < HP ? d + 1 : d + 1 - HP)];
            v = (d < HP ? (w0 & 0xffffu) : (w0 >> 16)) | ((d + 1 < HP ? (w1 & 0xffffu) : (w1 >> 16)) << 16);
          }
          aq[ks][2 * hf] = v;
          aq[ks][2 * hf + 1] = 0u;                           // rows 8..15 of the tile are unused
        }
      }
      float o[NTD][4];
#pragma unroll
      for (int j = 0; j < NTD; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[j][e] = 0.f;
      float mrun = -1e30f, lrun = 0.f;
      // a stage is cut into units of 16 positions that different warps take: a chunk of a few stages keeps most warps busy
      constexpr int UP = 16, SPLIT = NPS / UP;
      const int nst = t1 > t0 ? (t1 - t0 + NPS - 1) / NPS : 0;
      for (int u = cw; u < nst * SPLIT; u += kConsumerWarps) {
        const int st = u / SPLIT, part = u % SPLIT;
        const uint32_t it = pipe->it + st;
        const int sslot = it % kStages;
        bool ok = true;
        if (it >= (uint32_t)kStages) {                     // the stage's previous load must be complete before its phase bit is read
          ok = false;
          for (unsigned i = 0; i < wc.limit; i++) {
            if ((uint32_t)*pipe->landed > it - kStages) { ok = true; break; }
            if ((i & 63) == 63 && *wc.s_abort) break;
          }
          if (!ok && *wc.s_abort == 0) report_fail(wc, W_LANDED, layer, (int)it, *pipe->landed);
        }
        if (ok) ok = mbar_wait(&pipe->full[sslot], (it / kStages) & 1, wc, W_FULL, layer);
        if (!ok) break;
        uint8_t* k_s = pipe->stages + (size_t)sslot * kStageBytes + (size_t)part * UP * ROWB;
        uint8_t* v_s = k_s + C::KV_STAGE_BYTES / 2;
        const int base = t0 + st * NPS + part * UP, nvalid = min(UP, t1 - base);
        if (nvalid > 0) {
          if (a.pos >= base && a.pos < base + UP) {          // this step's own row: from the tagged words, not the cache
            const uint32_t* kp = qs + R * HP;
            const uint32_t* vp = kp + HP;
            uint16_t* krow = reinterpret_cast<uint16_t*>(k_s + (size_t)(a.pos - base) * ROWB);
            uint32_t* vrow = reinterpret_cast<uint32_t*>(v_s + (size_t)(a.pos - base) * ROWB);
            for (int p2 = lane; p2 < HP; p2 += 32) {
              krow[p2] = (uint16_t)(kp[p2] & 0xffffu);
              krow[p2 + HP] = (uint16_t)(kp[p2] >> 16);
              vrow[p2] = vp[p2];
            }
          }
          // rows past the chunk are other cache rows (or never written): their V must not meet a zero probability as NaN
          for (int i = lane; i < (UP - nvalid) * (ROWB / 16); i += 32)
            *reinterpret_cast<uint4*>(v_s + (size_t)nvalid * ROWB + (size_t)i * 16) = make_uint4(0, 0, 0, 0);
          __syncwarp();
          float sc[2][4];
#pragma unroll
          for (int nt = 0; nt < 2; nt++) {
            sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
              const uint8_t* kr = k_s + (size_t)(nt * 8 + g) * ROWB + (16 * ks + 2 * t) * 2;
              mma_bf16(sc[nt], aq[ks], *reinterpret_cast<const uint32_t*>(kr), *reinterpret_cast<const uint32_t*>(kr + 16));
            }
          }
          float mx = -INFINITY;                              // row g (rows 8..15 of the tile carry nothing)
#pragma unroll
          for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
              const float v = (nt * 8 + 2 * t + e) < nvalid ? sc[nt][e] * a.scale : -INFINITY;
              sc[nt][e] = v;
              mx = fmaxf(mx, v);
            }
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float mn = fmaxf(mrun, mx);                 // finite: the running maximum starts at -1e30
          const float corr = __expf(mrun - mn);
          mrun = mn;
          lrun *= corr;
#pragma unroll
          for (int j = 0; j < NTD; j++) { o[j][0] *= corr; o[j][1] *= corr; }
          uint32_t ah[4], al[4];
#pragma unroll
          for (int e = 0; e < 2; e++) {                      // A rows g: positions 2t (+1) and + 8; rows g + 8: zero
            const float p0 = __expf(sc[e][0] - mrun), p1 = __expf(sc[e][1] - mrun);
            lrun += p0 + p1;                                 // this lane's columns; the quad is summed at the end
            const float h0 = rbf(p0), h1 = rbf(p1);
            ah[2 * e] = pack_bf16(h0, h1);
            al[2 * e] = pack_bf16(p0 - h0, p1 - h1);
            ah[2 * e + 1] = 0u;
            al[2 * e + 1] = 0u;
          }
#pragma unroll
          for (int j = 0; j < NTD; j += 2) {
            uint32_t bv[4];
            const int mat = lane >> 3;
            ldmatrix_x4_trans(bv, v_s + (size_t)((mat & 1) * 8 + (lane & 7)) * ROWB + (j + (mat >> 1)) * 16);
            mma_bf16(o[j], ah, bv[0], bv[1]);
            mma_bf16(o[j], al, bv[0], bv[1]);
            mma_bf16(o[j + 1], ah, bv[2], bv[3]);
            mma_bf16(o[j + 1], al, bv[2], bv[3]);
          }
        }
        __syncwarp();
        if (lane == 0) {                                     // the stage's last unit hands it back
          const int old = atomicAdd(tdone + sslot, 1);
          if (old == SPLIT - 1) {
            tdone[sslot] = 0;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&pipe->empty[sslot]);
          }
        }
      }
      pipe->it += (uint32_t)nst;                             // producer and consumers count alike
      lrun += __shfl_xor_sync(0xffffffffu, lrun, 1);
      lrun += __shfl_xor_sync(0xffffffffu, lrun, 2);
      if (g < R) {
        float* dst = wacc + ((size_t)cw * R + g) * HD;
#pragma unroll
        for (int j = 0; j < NTD; j++) { dst[j * 8 + 2 * t] = o[j][0]; dst[j * 8 + 2 * t + 1] = o[j][1]; }
        if (t == 0) { wm[cw * R + g] = mrun; wd[cw * R + g] = lrun; }
      }
    } else {
      float q[R][8];
#pragma unroll
      for (int r = 0; r < R; r++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const uint32_t u = active ? qs[r * HP + 4 * sl + e] : 0u;
          q[r][e] = bflo(u);        // dim 4sl+e
          q[r][4 + e] = bfhi(u);    // dim HP+4sl+e
        }
      float m[R], den[R], acc[R][8];
#pragma unroll
      for (int r = 0; r < R; r++) {
        m[r] = -1e30f; den[r] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) acc[r][e] = 0.f;
      }
      constexpr int BATCH = FB_ATTN_BATCH;
      const int stride = kConsumerWarps * C::PPW;
      for (int tb = t0 + cw * C::PPW; tb < t1; tb += BATCH * stride) {
        uint2 klo[BATCH], khi[BATCH], vlo[BATCH], vhi[BATCH];
        bool valid[BATCH];
#pragma unroll
        for (int j = 0; j < BATCH; j++) {
          const int t = tb + j * stride + seg;
          valid[j] = t < t1;
          klo[j] = khi[j] = vlo[j] = vhi[j] = make_uint2(0, 0);
          if (valid[j] && active) {
            if (t == a.pos) {      // this step's own k / v: from the tagged words (the cache row is for later steps)
              const uint32_t* kp = qs + R * HP + 4 * sl;
              const uint32_t* vp = qs + R * HP + HP;
              klo[j] = make_uint2((kp[0] & 0xffffu) | (kp[1] << 16), (kp[2] & 0xffffu) | (kp[3] << 16));
              khi[j] = make_uint2((kp[0] >> 16) | (kp[1] & 0xffff0000u), (kp[2] >> 16) | (kp[3] & 0xffff0000u));
              vlo[j] = make_uint2(vp[2 * sl], vp[2 * sl + 1]);
              vhi[j] = make_uint2(vp[HP / 2 + 2 * sl], vp[HP / 2 + 2 * sl + 1]);
            } else {
              const size_t off = ((size_t)t * a.nkv + kvh) * HD + 4 * sl;
              klo[j] = __ldcg(reinterpret_cast<const uint2*>(a.kc + off));
              khi[j] = __ldcg(reinterpret_cast<const uint2*>(a.kc + off + HP));
              vlo[j] = __ldcg(reinterpret_cast<const uint2*>(a.vc + off));
              vhi[j] = __ldcg(reinterpret_cast<const uint2*>(a.vc + off + HP));
            }
          }
        }
        // long chunks: ask L2 for the rows this warp will load two rounds from now (costs no registers)
        if (sl < (HD * 2 + 63) / 64) {
#pragma unroll
          for (int j = 0; j < BATCH; j++) {
            const int tp = tb + (FB_ATTN_PFD * BATCH + j) * stride + seg;
            if (tp < t1) {
              const size_t off = ((size_t)tp * a.nkv + kvh) * HD;
              asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(a.kc + off) + sl * 64));
              asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(a.vc + off) + sl * 64));
            }
          }
        }
        // scores of the whole batch first (independent chains), then ONE rescale per head and batch
        float sc[BATCH][R];
#pragma unroll
        for (int j = 0; j < BATCH; j++) {
          const float kf[8] = {bflo(klo[j].x), bfhi(klo[j].x), bflo(klo[j].y), bfhi(klo[j].y),
                               bflo(khi[j].x), bfhi(khi[j].x), bflo(khi[j].y), bfhi(khi[j].y)};
#pragma unroll
          for (int r = 0; r < R; r++) {
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < 8; e++) s = fmaf(q[r][e], kf[e], s);
#pragma unroll
            for (int o = C::SEG / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            sc[j][r] = valid[j] ? s * a.scale : -INFINITY;
          }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
          float mb = sc[0][r];
#pragma unroll
          for (int j = 1; j < BATCH; j++) mb = fmaxf(mb, sc[j][r]);
          const float m2 = fmaxf(m[r], mb);                 // finite: m starts at -1e30
          const float corr = __expf(m[r] - m2);
          den[r] *= corr;
#pragma unroll
          for (int e = 0; e < 8; e++) acc[r][e] *= corr;
          m[r] = m2;
        }
#pragma unroll
        for (int j = 0; j < BATCH; j++) {
          const float vf[8] = {bflo(vlo[j].x), bfhi(vlo[j].x), bflo(vlo[j].y), bfhi(vlo[j].y),
                               bflo(vhi[j].x), bfhi(vhi[j].x), bflo(vhi[j].y), bfhi(vhi[j].y)};
#pragma unroll
          for (int r = 0; r < R; r++) {
            const float w = __expf(sc[j][r] - m[r]);        // 0 for a position that does not exist
            den[r] += w;
#pragma unroll
            for (int e = 0; e < 8; e++) acc[r][e] = fmaf(w, vf[e], acc[r][e]);
          }
        }
      }
      // merge the warp's segments
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
          float* dst = wacc + ((size_t)cw * R + r) * HD;
#pragma unroll
          for (int e = 0; e < 4; e++) { dst[4 * sl + e] = acc[r][e]; dst[HP + 4 * sl + e] = acc[r][4 + e]; }
          if (sl == 0) { wm[cw * R + r] = m[r]; wd[cw * R + r] = den[r]; }
        }
      }
    }
    named_bar_sync(kBarConsumers, kConsumerThreads);
    // ---- merge the CTA's warps; one thread per (head, dim pair) ----
    constexpr int WPC = R * HD + 2 * R;                       // words of one chunk partial
    uint64_t* mine = a.part_ll + ((size_t)kvh * a.maxchunks + c) * WPC;
    for (int o = tid_c; o < R * HP; o += kConsumerThreads) {
      const int r = o / HP, d = 2 * (o % HP);
      float gm = -1e30f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; w++) gm = fmaxf(gm, wm[w * R + r]);
      float Dn = 0.f, A0 = 0.f, A1 = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; w++) {
        const float e = __expf(wm[w * R + r] - gm);
        Dn += wd[w * R + r] * e;
        A0 += wacc[((size_t)w * R + r) * HD + d] * e;
        A1 += wacc[((size_t)w * R + r) * HD + d + 1] * e;
      }
      const int qh = kvh * R + r;
      if (a.nchunks == 1) {
        ll_store(a.ao_ll + (size_t)qh * HP + (d >> 1), (uint32_t)f2bf(A0 / Dn) | ((uint32_t)f2bf(A1 / Dn) << 16), a.tag_out);
      } else {
        ll_store(mine + r * HD + d, __float_as_uint(A0), a.tag_part);
        ll_store(mine + r * HD + d + 1, __float_as_uint(A1), a.tag_part);
        if (d == 0) {
          ll_store(mine + R * HD + r, __float_as_uint(gm), a.tag_part);
          ll_store(mine + R * HD + R + r, __float_as_uint(Dn), a.tag_part);
        }
      }
    }
    if (a.nchunks > 1) {
      // Every chunk CTA of the kv head merges its share of the output: dim pairs c, c + nchunks, ... From each chunk's
      // partial it needs the 2R words (max, denominator) and its own pairs only: one 16-byte tagged load per thread,
      // no counter, no fence, a single round trip.
      named_bar_sync(kBarConsumers, kConsumerThreads);        // wacc / wm / wd are dead: scratch is free
      const int npairs = R * HP;
      const int nown = (npairs - c + a.nchunks - 1) / a.nchunks;
      const int per = R + nown;                                // loads per source chunk
      uint32_t* pg = reinterpret_cast<uint32_t*>(scratch);     // [nchunks][per][2] payloads
      const int total = a.nchunks * per;                       // <= kConsumerThreads (host checks the shape)
      if (tid_c < total) {
        const int cc = tid_c / per, sl2 = tid_c % per;
        int w;
        if (sl2 < R) {
          w = R * HD + 2 * sl2;
        } else {
          const int o = c + (sl2 - R) * a.nchunks;
          w = (o / HP) * HD + 2 * (o % HP);
        }
        const uint64_t* src = a.part_ll + ((size_t)kvh * a.maxchunks + cc) * WPC + w;
        for (unsigned spin = 0;; spin++) {
          uint64_t u, v;
          ll_load2(src, u, v);
          if ((uint32_t)(u >> 32) == a.tag_part && (uint32_t)(v >> 32) == a.tag_part) {
            pg[2 * tid_c] = (uint32_t)u; pg[2 * tid_c + 1] = (uint32_t)v;
            break;
          }
          if (*wc.s_abort) break;
          if (spin > 16) __nanosleep(40);
          if ((spin & 255) == 255 && ld_volatile_s32(&wc.st->abort)) { *wc.s_abort = 1; break; }
          if (spin >= wc.limit) { report_fail(wc, W_FLAG, layer, (int)a.tag_part, -4); break; }
        }
      }
      named_bar_sync(kBarConsumers, kConsumerThreads);
      if (tid_c < nown) {
        const float* pf = reinterpret_cast<const float*>(pg);
        const int o = c + tid_c * a.nchunks, r = o / HP, d = 2 * (o % HP);
        // words 0..R-1 of a chunk's (max, denominator) area are the maxima, R..2R-1 the denominators
        float gm = -1e30f;
        for (int cc = 0; cc < a.nchunks; cc++) gm = fmaxf(gm, pf[cc * per * 2 + r]);
        float Dn = 0.f, A0 = 0.f, A1 = 0.f;
        for (int cc = 0; cc < a.nchunks; cc++) {
          const float e = __expf(pf[cc * per * 2 + r] - gm);
          Dn += pf[cc * per * 2 + R + r] * e;
          A0 += pf[(cc * per + R + tid_c) * 2] * e;
          A1 += pf[(cc * per + R + tid_c) * 2 + 1] * e;
        }
        const int qh = kvh * R + r;
        ll_store(a.ao_ll + (size_t)qh * HP + (d >> 1), (uint32_t)f2bf(A0 / Dn) | ((uint32_t)f2bf(A1 / Dn) << 16), a.tag_out);
      }
    }
    named_bar_sync(kBarConsumers, kConsumerThreads);
    if (tid_c == 0) st_relaxed_u32(a.ao_flags + kvh * a.nchunks + c, a.tag_out);
  }
}

// Producer side of the long-cache attention: the K and V rows of this CTA's chunk(s), NPS positions per ring stage. The
// caches are [layer * max_seq + position][kv head][HD]: one 3-D tensor copy (box HD x 1 head x NPS positions) per
// matrix and stage brings the strided rows in one request. Rows past the chunk (the last stage) are real cache rows that
// nobody reads; past the end of the cache the copy fills zeros. Called by the producer lane.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
template <int HD, int R>
__device__ __forceinline__ bool produce_kv(Pipe& p, const CUtensorMap* kmap, const CUtensorMap* vmap, int row0, int nkv, int nchunks,
                                           int T, int b, int G, const WaitCtl& wc, int layer) {
  using C = AttnCfg<HD, R>;
  const int items = nkv * nchunks, chunk_len = (T + nchunks - 1) / nchunks;
  for (int item = b; item < items; item += G) {
    const int kvh = item / nchunks, c = item % nchunks, t0 = c * chunk_len, t1 = min(T, t0 + chunk_len);
    for (int ts = t0; ts < t1; ts += C::NPS) {
      const int s = (int)(p.it % kStages);
      if (!mbar_wait(&p.empty[s], ((p.it / kStages) & 1) ^ 1, wc, W_EMPTY, layer)) return false;
      mbar_expect_tx(&p.full[s], (uint32_t)C::KV_STAGE_BYTES);
      uint8_t* dst = p.stages + (size_t)s * kStageBytes;
      tma_load_3d(dst, kmap, 0, kvh, row0 + ts, &p.full[s]);
      tma_load_3d(dst + C::KV_STAGE_BYTES / 2, vmap, 0, kvh, row0 + ts, &p.full[s]);
      p.it++;
      if (p.it > p.max_fly) {                         // same trailing wait as produce_rows: keeps `landed` current
        const uint32_t j = p.it - 1 - p.max_fly;
        if (!mbar_wait(&p.full[j % kStages], (j / kStages) & 1, wc, W_FULL, layer)) return false;
        *p.landed = (int)(j + 1);
      }
    }
  }
  return true;
}

// ------------------------------------------------------------------------------------------------ kernel
struct Decode2Params {
  CUtensorMap kmap, vmap;     // long-cache variant: the K / V caches as [HD][n_kv][n_layer * max_seq] tensors (else unused)
  const uint8_t *w_qkv, *w_o, *w_gu, *w_d, *w_lm;
  const uint16_t *n1, *n2, *nf, *embed;
  const float* invf;
  uint16_t *kc, *vc;
  uint64_t *h_ll, *q_ll, *k_ll, *v_ll, *ao_ll, *act_ll, *cand_ll;   // tagged vectors
  uint64_t* part_ll;
  uint32_t *h_flags, *act_flags, *ao_flags;                          // arrival flags: [G], [G], [NKV]
  DevStatus* status;
  const int32_t* d_token;
  uint16_t* d_h;
  float* d_logits;
  int32_t* d_next;
  int32_t token, pos, max_seq;
  int32_t n_layer, dim, n_head, n_kv, ffn, vocab, nchunks, maxchunks;
  unsigned tag_base, spin_limit;
  float eps, attn_scale, resid, emb_mult, logits_scaling;
  long long* prof;
  unsigned max_fly;
  int32_t poll_words;         // 1: consumers poll the tagged words themselves instead of waiting for arrival flags first
  // tensor parallelism: this GPU holds a slice of every matrix (heads, FFN columns, vocabulary rows); the partial sums
  // of the K-sharded O and down projections are exchanged by peer stores into every rank's inbox
  int32_t tp_size, tp_rank, vocab_base;
  int32_t ao_off;             // columns between the start of this rank's O window and its own attention output (0 or 64)
  uint64_t* inbox;            // local: [2 parities][tp_size][dim] tagged fp32 partials, then [tp_size][2] arg-max candidates
  uint64_t* peer_inbox[8];    // the same buffer of every rank (peer-mapped); own entry = inbox
};

// tags: phase ids inside a layer
enum { PH_QKV = 1, PH_ATT = 2, PH_O = 3, PH_GU = 4, PH_DOWN = 5, PH_LM = 6, PH_PART = 7 };
__device__ __forceinline__ uint32_t mk_tag(unsigned base, int layer, int ph) { return base + (unsigned)(layer * 8 + ph); }

// small phases (QKV, O, down give a CTA a handful of tiles): cut long tiles in two so that more warps share them
__host__ __device__ constexpr int small_ks(int k) {
  const int rt = tile_rt(k), bq = (k / 128) / (16 / rt) * 2;
  return (rt <= 4 && bq >= 16 && bq % 2 == 0) ? 2 : 1;
}
__host__ __device__ constexpr int imax(int a, int b) { return a > b ? a : b; }

// LONGKV: the attention phase reads K/V through the weight ring (produce_kv); chosen by the host for long caches.
template <int KDIM, int KOUT, int KFFN, int HD, int R, bool HZ, bool LONGKV = false>
__global__ void __launch_bounds__(kThreads, 1) decode_mega2(const __grid_constant__ Decode2Params P) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Smem sm = carve_smem(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, b = blockIdx.x;
  // (cos, sin) of this step's position for every rotation pair: once per launch instead of a full-range sincosf in every
  // QKV epilogue of every layer
  __shared__ float2 s_rope[64];
  if (tid == 0) pipe_init(sm);
  if (tid < HD / 2) {
    float sn, cs;
    sincosf((float)P.pos * __ldg(P.invf + tid), &sn, &cs);
    s_rope[tid] = make_float2(cs, sn);
  }
  __syncthreads();
  WaitCtl wc{P.status, sm.s_abort, P.spin_limit};
  Pipe pipe{sm.stages, sm.full, sm.empty, sm.landed, 0u, P.max_fly};
  constexpr int HP = HD / 2;
  using CQ = TCfg<KDIM, small_ks(KDIM)>;      // QKV: few rows per CTA
  using CG = TCfg<KDIM>;                      // gate/up and LM head: many rows per CTA
  using CO = TCfg<KOUT, small_ks(KOUT)>;      // O projection (K = this rank's attention output width)
  using CF = TCfg<KFFN, small_ks(KFFN)>;      // down projection
  constexpr int UO = imax(CO::RT, CF::RT);    // O and down give a CTA the same rows of the residual stream
  static_assert(CG::RT % 4 == 0, "the SwiGLU epilogue packs rows (g, u, g', u') into one tagged word");
  const int D = P.dim, FF = P.ffn, L = P.n_layer, V = P.vocab;
  const int QKV = (P.n_head + 2 * P.n_kv) * HD;
  const int FG = P.poll_words ? 0 : G, FKV = P.poll_words ? 0 : P.n_kv * P.nchunks;     // arrival flags to wait for
  constexpr int recD = rec_bytes_of(KDIM, HZ), recO = rec_bytes_of(KOUT, HZ), recF = rec_bytes_of(KFFN, HZ);
  const size_t strQ = (size_t)pad_rows(QKV, KDIM) * recD, strO = (size_t)pad_rows(D, KOUT) * recO,
               strG = (size_t)pad_rows(2 * FF, KDIM) * recD, strF = (size_t)pad_rows(D, KFFN) * recF;
  const int N = P.tp_size, me = P.tp_rank;
  int q0, q1, o0, o1, g0, g1, l0, l1;
  cta_rows(QKV, CQ::RT, b, G, q0, q1);
  cta_rows(D, UO, b, G, o0, o1);         // the same rows of h belong to this CTA in the O and the down phase
  cta_rows(2 * FF, CG::RT, b, G, g0, g1);   // (g_i, u_i, g_i+1, u_i+1) stay together: one tagged word of activations
  cta_rows(V, CG::RT, b, G, l0, l1);

  if (warp == kConsumerWarps) {
    if (lane == 0) {
      bool ok = true;
      for (int l = 0; l < L && ok; l++) {
        ok = produce_rows(pipe, P.w_qkv + l * strQ + (size_t)q0 * recD, q1 - q0, CQ::TILE_ROWS, CQ::RT, recD, wc, l);
        if constexpr (LONGKV)
          ok = ok && produce_kv<HD, R>(pipe, &P.kmap, &P.vmap, l * P.max_seq, P.n_kv, P.nchunks, P.pos + 1, b, G, wc, l);
        ok = ok &&
             produce_rows(pipe, P.w_o + l * strO + (size_t)o0 * recO, o1 - o0, CO::TILE_ROWS, CO::RT, recO, wc, l) &&
             produce_rows(pipe, P.w_gu + l * strG + (size_t)g0 * recD, g1 - g0, CG::TILE_ROWS, CG::RT, recD, wc, l) &&
             produce_rows(pipe, P.w_d + l * strF + (size_t)o0 * recF, o1 - o0, CF::TILE_ROWS, CF::RT, recF, wc, l);
      }
      if (ok) produce_rows(pipe, P.w_lm + (size_t)l0 * recD, l1 - l0, CG::TILE_ROWS, CG::RT, recD, wc, L);
      producer_drain(pipe, wc);
    }
  } else {
    const int cw = warp, tid_c = tid;
    float* hown = sm.hown;                                      // this CTA's rows of the residual stream (exact bf16 values)
    int* s_done = sm.misc + 20;                                 // warps of this CTA that finished the current producing phase
    if (tid_c == 0) *s_done = 0;
    const QueueState qs_{sm.qpart, sm.tdone, sm.bcnt};
    const XStage xs_{sm.xh, sm.xf};
    float* ypart = sm.hown + kMaxOwnRows;                       // tensor parallel: this rank's partial sums of its rows
    constexpr int MAXP_O = (KOUT / 4 + kConsumerThreads - 1) / kConsumerThreads;
    // O / down epilogue. One GPU: h = bf16(h + y * resid) at once. Tensor parallel: y is a partial sum over this
    // rank's K slice: keep it, push it to every peer's inbox, finish in resid_finish once all rows are done.
    auto resid_epi = [&](int row0, float c, int nvalid, uint32_t tag, int par) {
      const int r = row0 + (lane >> 3);
      if (N > 1) {
        // lanes 0/8/16/24 hold the partial sums of rows row0..row0+3; lane j < N-1 pushes all four to one peer as two
        // 16-byte stores, so the N-1 transfers of a tile leave the SM side by side instead of one after the other
        const float c0 = __shfl_sync(0xffffffffu, c, 0), c1 = __shfl_sync(0xffffffffu, c, 8),
                    c2 = __shfl_sync(0xffffffffu, c, 16), c3 = __shfl_sync(0xffffffffu, c, 24);
        if ((lane & 7) == 0 && (lane >> 3) < nvalid) ypart[r] = c;
        if (lane < N - 1) {
          const int p = lane >= me ? lane + 1 : lane;
          uint64_t* dst = P.peer_inbox[p] + ((size_t)(par * N + me)) * D + o0 + row0;     // 32-byte aligned: row0 % 4 == 0
          if (nvalid == 4) {
            ll_store2_sys(dst, __float_as_uint(c0), __float_as_uint(c1), tag);
            ll_store2_sys(dst + 2, __float_as_uint(c2), __float_as_uint(c3), tag);
          } else {
            const float cc[4] = {c0, c1, c2, c3};
            for (int i = 0; i < nvalid; i++) ll_store_sys(dst + i, __float_as_uint(cc[i]), tag);
          }
        }
        return;
      }
      float hn = 0.f;
      if ((lane & 7) == 0 && (lane >> 3) < nvalid) {
        hn = rbf(hown[r] + c * P.resid);
        hown[r] = hn;
      }
      const float hn1 = __shfl_down_sync(0xffffffffu, hn, 8);
      if ((lane & 15) == 0 && (lane >> 3) < nvalid)
        ll_store(P.h_ll + ((o0 + r) >> 1), (uint32_t)f2bf(hn) | ((uint32_t)f2bf(hn1) << 16), tag);
    };
    // tensor parallel only: collect the peers' partials of this CTA's rows (one 16-byte load per thread and poll round,
    // all peers and row pairs in flight together), sum in rank order (identical on every rank), update h, publish
    float* yin = sm.yin;                                      // [N-1][kMaxOwnRows]
    auto resid_finish = [&](uint32_t tag, int par, int layer) {
      const int npair = (o1 - o0) / 2, nitem = npair * (N - 1);
      for (int it = tid_c; it < nitem; it += kConsumerThreads) {
        const int j = it / npair, pr = it % npair, s2 = j >= me ? j + 1 : j;
        const uint64_t* src = P.inbox + ((size_t)(par * N + s2)) * D + o0 + 2 * pr;
        for (unsigned spin = 0;; spin++) {
          uint64_t u, v;
          ll_load2_sys(src, u, v);
          if ((uint32_t)(u >> 32) == tag && (uint32_t)(v >> 32) == tag) {
            yin[j * kMaxOwnRows + 2 * pr] = __uint_as_float((uint32_t)u);
            yin[j * kMaxOwnRows + 2 * pr + 1] = __uint_as_float((uint32_t)v);
            break;
          }
          if (*wc.s_abort) break;
          if ((spin & 255) == 255 && ld_volatile_s32(&wc.st->abort)) { *wc.s_abort = 1; break; }
          if (spin >= wc.limit) { report_fail(wc, W_FLAG, layer, (int)tag, -3); break; }
        }
      }
      named_bar_sync(kBarConsumers, kConsumerThreads);        // every row's own partial and every peer's are in shared memory
      for (int pr = tid_c; pr < npair; pr += kConsumerThreads) {
        float tot0 = 0.f, tot1 = 0.f;
        for (int s2 = 0; s2 < N; s2++) {
          const float* src = s2 == me ? ypart : yin + (s2 > me ? s2 - 1 : s2) * kMaxOwnRows;
          tot0 += src[2 * pr]; tot1 += src[2 * pr + 1];
        }
        const float h0 = rbf(hown[2 * pr] + tot0 * P.resid), h1 = rbf(hown[2 * pr + 1] + tot1 * P.resid);
        hown[2 * pr] = h0; hown[2 * pr + 1] = h1;
        ll_store(P.h_ll + ((o0 >> 1) + pr), (uint32_t)f2bf(h0) | ((uint32_t)f2bf(h1) << 16), tag);
      }
      named_bar_sync(kBarConsumers, kConsumerThreads);
      if (tid_c == 0) st_relaxed_u32(P.h_flags + b, tag);
    };
    constexpr int MAXP_D = (KDIM / 4 + kConsumerThreads - 1) / kConsumerThreads;
    constexpr int MAXP_F = (KFFN / 4 + kConsumerThreads - 1) / kConsumerThreads;
    // ---- residual stream at layer 0: every CTA reads the embedding row (or the caller's h) itself ----
    {
      int tok = P.d_token ? (int)ld_cg_u32(P.d_token) : P.token;
      if ((unsigned)tok >= (unsigned)(V * N)) {                 // V is this rank's slice of the vocabulary
        tok = 0;
        if (tid_c == 0 && b == 0) atomicCAS(&P.status->code, 0, 6 /*FB_ERR_RANGE*/);
      }
      for (int i = tid_c; i < D; i += kConsumerThreads) {
        const uint16_t v = P.d_h ? ld_cg_u16(P.d_h + i) : f2bf(bf2f(__ldg(P.embed + (size_t)tok * D + i)) * P.emb_mult);
        reinterpret_cast<uint16_t*>(sm.xh)[i] = v;
        if (i >= o0 && i < o1) hown[i - o0] = bf2f(v);
      }
      named_bar_sync(kBarConsumers, kConsumerThreads);
    }
#define FB_STAMP(i) do { if (P.prof && tid_c == 0) P.prof[((size_t)b * L + l) * 16 + (i)] = (long long)globaltimer_ns(); } while (0)
    for (int l = 0; l < L; l++) {
      uint16_t* kcl = P.kc + (size_t)l * P.max_seq * P.n_kv * HD;
      uint16_t* vcl = P.vc + (size_t)l * P.max_seq * P.n_kv * HD;
      const uint32_t tg_qkv = mk_tag(P.tag_base, l, PH_QKV), tg_att = mk_tag(P.tag_base, l, PH_ATT),
                     tg_o = mk_tag(P.tag_base, l, PH_O), tg_gu = mk_tag(P.tag_base, l, PH_GU),
                     tg_dn = mk_tag(P.tag_base, l, PH_DOWN);
      // ================= QKV: norm1 -> GEMV -> RoPE -> tagged q / new k / new v, cache append =================
      FB_STAMP(0);
      if (b < P.n_kv * P.nchunks) {
        // the K/V rows this CTA will attend in this layer: pull them into L2 now, they do not depend on anything
        const int kvh = b / P.nchunks, c = b % P.nchunks;
        const int T = P.pos + 1, clen = (T + P.nchunks - 1) / P.nchunks;
        const int t0 = c * clen, t1 = min(min(T, t0 + clen), t0 + 64);
        constexpr int PER_ROW = (HD * 2 + 63) / 64;
        for (int i = tid_c; i < (t1 - t0) * PER_ROW * 2; i += kConsumerThreads) {
          const int t = t0 + (i >> 1) / PER_ROW, seg = (i >> 1) % PER_ROW;
          const uint16_t* base = ((i & 1) ? vcl : kcl) + ((size_t)t * P.n_kv + kvh) * HD;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(base) + seg * 64));
        }
      }
      stage_norm_ll<MAXP_D>(P.h_ll, P.h_flags, FG, mk_tag(P.tag_base, l - 1, PH_DOWN), P.n1 + (size_t)l * D, D, P.eps,
                            sm, tid_c, wc, l, l == 0, P.prof ? P.prof + ((size_t)b * L + l) * 16 : nullptr);
      FB_STAMP(1);
      consume_tiles<CQ, HZ, true>(pipe, q1 - q0, xs_, qs_, cw, lane, wc, l, [&](int row0, float c, int nvalid) {
        // lanes 0/8/16/24 hold rows row0..row0+3: two RoPE pairs (or four v dims)
        const float c1 = __shfl_down_sync(0xffffffffu, c, 8);
        if ((lane & 15) == 0 && (lane >> 3) < nvalid) {
          const int rs = q0 + row0 + (lane >> 3);              // stream row of the pair's first element (even)
          const int head = rs / HD, within = rs % HD;
          if (head < P.n_head + P.n_kv) {
            const int i = within >> 1;
            const float x0 = rbf(c), x1 = rbf(c1);
            const float cs = s_rope[i].x, sn = s_rope[i].y;
            const uint32_t y0 = f2bf(x0 * cs - x1 * sn), y1 = f2bf(x1 * cs + x0 * sn);
            if (head < P.n_head) {
              ll_store(P.q_ll + (size_t)head * HP + i, y0 | (y1 << 16), tg_qkv);
            } else {
              const int kvh = head - P.n_head;
              ll_store(P.k_ll + (size_t)kvh * HP + i, y0 | (y1 << 16), tg_qkv);
              uint16_t* kr = kcl + ((size_t)P.pos * P.n_kv + kvh) * HD;
              kr[i] = (uint16_t)y0;
              kr[i + HP] = (uint16_t)y1;
            }
          } else {
            const int kvh = head - P.n_head - P.n_kv;
            const uint32_t pv = (uint32_t)f2bf(c) | ((uint32_t)f2bf(c1) << 16);
            ll_store(P.v_ll + (size_t)kvh * HP + (within >> 1), pv, tg_qkv);
            *reinterpret_cast<uint32_t*>(vcl + ((size_t)P.pos * P.n_kv + kvh) * HD + within) = pv;
          }
        }
      }, P.prof ? P.prof + ((size_t)b * L + l) * 16 : nullptr);
      FB_STAMP(2);
      // ================= attention =================
      {
        if (b == 0 && KOUT != 0) {
          // columns of the O window that belong to a neighbouring rank (tensor parallel, 8-way split of the 3B-class
          // shape): the O projection must see zeros there, tagged like the real attention output
          const int used = P.n_head * HP, off = P.ao_off >> 1;
          for (int i = tid_c; i < KOUT / 2 - used; i += kConsumerThreads)
            ll_store(P.ao_ll + (i < off ? i : used + i), 0u, tg_att);
        }
        Attn2Args aa{P.q_ll, P.k_ll, P.v_ll, P.ao_ll + (P.ao_off >> 1), kcl, vcl, P.part_ll, P.ao_flags, P.n_kv, P.pos, P.nchunks,
                     P.maxchunks, P.attn_scale, tg_qkv, mk_tag(P.tag_base, l, PH_PART), tg_att};
        named_bar_sync(kBarConsumers, kConsumerThreads);        // scratch (the activations) is free: every warp left the GEMV
        attn2_phase<HD, R, LONGKV>(aa, sm.scratch, sm.misc, cw, lane, tid_c, wc, l, &pipe, sm.tdone);
      }
      FB_STAMP(3);
      // ================= O projection + residual =================
      {
        stage_plain_ll<MAXP_O>(P.ao_ll, P.ao_flags, FKV, tg_att, KOUT, sm, tid_c, wc, l);
        FB_STAMP(4);
        consume_tiles<CO, HZ, true>(pipe, o1 - o0, xs_, qs_, cw, lane, wc, l,
                                  [&](int row0, float c, int nvalid) { resid_epi(row0, c, nvalid, tg_o, 0); });
        if (N > 1) resid_finish(tg_o, 0, l);
        else post_when_cta_done(s_done, P.h_flags + b, tg_o, lane);
      }
      FB_STAMP(5);
      // ================= gate/up + SwiGLU =================
      stage_norm_ll<MAXP_D>(P.h_ll, P.h_flags, FG, tg_o, P.n2 + (size_t)l * D, D, P.eps, sm, tid_c, wc, l, false);
      FB_STAMP(6);
      consume_tiles<CG, HZ, true>(pipe, g1 - g0, xs_, qs_, cw, lane, wc, l, [&](int row0, float c, int nvalid) {
        // rows (g_i, u_i, g_{i+1}, u_{i+1}) -> act[i], act[i+1] -> one tagged word
        const float u = __shfl_down_sync(0xffffffffu, c, 8);
        float av = 0.f;
        if ((lane & 15) == 0 && (lane >> 3) < nvalid) {
          const float gg = rbf(c), uu = rbf(u);
          av = rbf((gg / (1.0f + __expf(-gg))) * uu);
        }
        const float av1 = __shfl_down_sync(0xffffffffu, av, 16);
        const int i = (g0 + row0) >> 1;                          // act index of lane 0's value: even, g0 % 4 == 0
        if (lane == 0 && nvalid == 4)
          ll_store(P.act_ll + (i >> 1), (uint32_t)f2bf(av) | ((uint32_t)f2bf(av1) << 16), tg_gu);
      });
      post_when_cta_done(s_done, P.act_flags + b, tg_gu, lane);
      FB_STAMP(7);
      // ================= down projection + residual =================
      {
        stage_plain_ll<MAXP_F>(P.act_ll, P.act_flags, FG, tg_gu, FF, sm, tid_c, wc, l);
        FB_STAMP(8);
        consume_tiles<CF, HZ, true>(pipe, o1 - o0, xs_, qs_, cw, lane, wc, l,
                                  [&](int row0, float c, int nvalid) { resid_epi(row0, c, nvalid, tg_dn, 1); });
        if (N > 1) resid_finish(tg_dn, 1, l);
        else post_when_cta_done(s_done, P.h_flags + b, tg_dn, lane, P.prof ? P.prof + ((size_t)b * L + l) * 16 : nullptr);
      }
      FB_STAMP(9);
    }
#undef FB_STAMP
    // ================= final norm + LM head + arg-max =================
    stage_norm_ll<MAXP_D>(P.h_ll, P.h_flags, FG, mk_tag(P.tag_base, L - 1, PH_DOWN), P.nf, D, P.eps, sm, tid_c, wc, L, false);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    consume_tiles<CG, HZ, true>(pipe, l1 - l0, xs_, qs_, cw, lane, wc, L, [&](int row0, float c, int nvalid) {
      if ((lane & 7) == 0 && (lane >> 3) < nvalid) {
        const int row = P.vocab_base + l0 + row0 + (lane >> 3);     // index in the full vocabulary
        const float y = c / P.logits_scaling;
        if (P.d_logits) P.d_logits[row] = y;
        if (y > bv || (y == bv && row < bi)) { bv = y; bi = row; }
      }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sm.red[cw] = bv; sm.misc[cw] = bi; }
    named_bar_sync(kBarConsumers, kConsumerThreads);
    const uint32_t tg_lm = mk_tag(P.tag_base, L, PH_LM);
    if (tid_c == 0) {
      for (int w = 1; w < kConsumerWarps; w++)
        if (sm.red[w] > bv || (sm.red[w] == bv && sm.misc[w] < bi)) { bv = sm.red[w]; bi = sm.misc[w]; }
      ll_store(P.cand_ll + 2 * b, __float_as_uint(bv), tg_lm);
      ll_store(P.cand_ll + 2 * b + 1, (uint32_t)bi, tg_lm);
    }
    if (b == 0) {
      uint32_t* cs = reinterpret_cast<uint32_t*>(sm.xh);
      named_bar_sync(kBarConsumers, kConsumerThreads);
      ll_gather<2>(P.cand_ll, 2 * G, tg_lm, cs, tid_c, kConsumerThreads, wc, L);
      named_bar_sync(kBarConsumers, kConsumerThreads);
      if (cw == 0) {
        float v = -INFINITY;
        int ix = 0x7fffffff;
        for (int c = lane; c < G; c += 32) {
          const float ov = __uint_as_float(cs[2 * c]);
          const int oi = (int)cs[2 * c + 1];
          if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, o);
          const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
          if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
        }
        if (N > 1 && lane == 0) {
          // every rank holds a slice of the vocabulary: exchange the N (value, index) candidates, reduce in rank order
          uint64_t* mine = P.inbox + (size_t)2 * N * D;
          for (int p = 0; p < N; p++) {
            uint64_t* dst = (p == me ? mine : P.peer_inbox[p] + (size_t)2 * N * D) + 2 * me;
            ll_store_sys(dst, __float_as_uint(v), tg_lm);
            ll_store_sys(dst + 1, (uint32_t)ix, tg_lm);
          }
          v = -INFINITY; ix = 0x7fffffff;
          for (int s2 = 0; s2 < N; s2++) {
            const float ov = __uint_as_float(ll_poll_sys(mine + 2 * s2, tg_lm, wc, L));
            const int oi = (int)ll_poll_sys(mine + 2 * s2 + 1, tg_lm, wc, L);
            if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
          }
        }
        if (lane == 0 && P.d_next) *P.d_next = ix;
      }
    }
    // final residual back to the caller (the reference clobbers its h argument): every CTA writes its own rows
    if (P.d_h)
      for (int r = tid_c; r < o1 - o0; r += kConsumerThreads) P.d_h[o0 + r] = f2bf(hown[r]);
  }
  __syncthreads();
}

}  // namespace fb
