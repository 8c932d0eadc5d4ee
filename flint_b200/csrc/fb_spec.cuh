// Speculative-decoding side of the decode path, all on the device: token sampling from logits (temperature / top-k,
// Gumbel-max with a counter-based generator, no host sync), chain and tree acceptance, KV compaction of an accepted
// tree path, and the EAGLE draft head (one decoder block over [target feature ; token embedding], bf16 weights as the
// reference trains and runs it).
//
// The draft head's arithmetic follows the rounding sites of bf16 PyTorch modules: every linear layer, norm, rotation,
// activation and residual addition rounds its result to bf16; accumulation inside a layer is fp32.
#pragma once
#include "fb_common.cuh"

namespace fb {

// ------------------------------------------------------------------------------------------------ random numbers
// splitmix64 finaliser over (seed, counter, index): independent streams per call (counter) and per vocabulary entry
__device__ __forceinline__ uint32_t mix32(unsigned long long seed, unsigned long long ctr, uint32_t idx) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (ctr + 1) + (((unsigned long long)idx << 1) | 1ull) * 0xD1B54A32D192ED03ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (uint32_t)(z >> 32);
}
// standard Gumbel variate from 23 random bits: u in (0, 1) exactly representable, never 0 or 1
__device__ __forceinline__ float gumbel(uint32_t bits) {
  const float u = ((float)(bits >> 9) + 0.5f) * (1.0f / 8388608.0f);
  return -logf(-logf(u));
}
// order-preserving map float -> uint32 (larger float = larger key)
__device__ __forceinline__ uint32_t fkey(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// ------------------------------------------------------------------------------------------------ sampling
struct SampleParams {
  const float* logits;          // [rows] vectors of `vocab` floats, `row_stride` elements apart (0: every row samples the same vector)
  long long row_stride;
  int32_t vocab, top_k;         // top_k <= 0: the whole vocabulary
  float temperature;            // <= 0: arg-max (first index of the maximum)
  unsigned long long seed, counter;   // row r draws from stream (seed, counter + r)
  int32_t* out;                 // [rows] token ids
};

// One CTA per row. top-k keeps every entry >= the k-th largest value (ties included, as `logits < v[-1] -> -inf` does,
// reference: engine/generate.py:41-45); the k-th largest is found exactly by a 4-pass radix select on order-preserving
// keys. The draw is arg-max of logit / T + Gumbel noise, which is a sample of softmax(logits / T) over the kept
// entries: the same distribution as arg-max(p / Exponential(1)) (reference: engine/generate.py:37-39).
__global__ void __launch_bounds__(1024) sample_rows(const SampleParams P) {
  __shared__ unsigned hist[256];
  __shared__ unsigned s_bin, s_k;
  __shared__ float s_v[32];
  __shared__ int s_i[32];
  const int tid = threadIdx.x, row = blockIdx.x;
  const float* lg = P.logits + (long long)row * P.row_stride;
  const bool draw = P.temperature > 0.f;
  uint32_t thr = 0u;
  if (draw && P.top_k > 0 && P.top_k < P.vocab) {
    uint32_t prefix = 0u, mask = 0u;
    unsigned k = (unsigned)P.top_k;
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) hist[tid] = 0u;
      __syncthreads();
      for (int i = tid; i < P.vocab; i += 1024) {
        const uint32_t key = fkey(lg[i]);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned cum = 0u;
        int b = 255;
        for (; b > 0; b--) {
          if (cum + hist[b] >= k) break;
          cum += hist[b];
        }
        s_bin = (unsigned)b;
        s_k = k - cum;
      }
      __syncthreads();
      prefix |= s_bin << shift;
      mask |= 0xFFu << shift;
      k = s_k;
      __syncthreads();
    }
    thr = prefix;                                   // key of the k-th largest value
  }
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  const float inv_t = draw ? 1.0f / P.temperature : 1.0f;
  for (int i = tid; i < P.vocab; i += 1024) {
    const float v = lg[i];
    if (fkey(v) < thr) continue;
    const float sc = draw ? v * inv_t + gumbel(mix32(P.seed, P.counter + (unsigned long long)row, (uint32_t)i)) : v;
    if (sc > bv || (sc == bv && i < bi)) { bv = sc; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((tid & 31) == 0) { s_v[tid >> 5] = bv; s_i[tid >> 5] = bi; }
  __syncthreads();
  if (tid < 32) {
    bv = s_v[tid]; bi = s_i[tid];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (tid == 0) P.out[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

// the B best entries of every row in order (value descending, first index on ties): B rounds of a block arg-max
__global__ void __launch_bounds__(1024) topb_rows(const float* logits, long long row_stride, int vocab, int B, int32_t* out_idx,
                                                  float* out_val) {
  __shared__ float s_v[32];
  __shared__ int s_i[32];
  __shared__ int chosen[16];
  const int tid = threadIdx.x, row = blockIdx.x;
  const float* lg = logits + (long long)row * row_stride;
  pdl_trigger();
  pdl_wait();
  for (int r = 0; r < B; r++) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += 1024) {
      bool taken = false;
      for (int j = 0; j < r; j++) taken = taken || (chosen[j] == i);
      const float v = lg[i];
      if (!taken && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { s_v[tid >> 5] = bv; s_i[tid >> 5] = bi; }
    __syncthreads();
    if (tid < 32) {
      bv = s_v[tid]; bi = s_i[tid];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (tid == 0) {
        chosen[r] = bi;
        out_idx[(size_t)row * B + r] = bi == 0x7fffffff ? 0 : bi;
        if (out_val) out_val[(size_t)row * B + r] = bv;
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------ acceptance
// chain: longest prefix of the K drafted tokens the target's greedy choices agree with
// (reference: spec_mega.py:106-113). out[0] = accepted count, out[1] = the target's token after the accepted prefix.
__global__ void accept_chain(const int32_t* tgt, const int32_t* draft, int K, int32_t* out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int acc = 0;
    while (acc < K && tgt[acc] == draft[acc]) acc++;
    out[0] = acc;
    out[1] = tgt[acc];
  }
}
// tree: walk from the root along the first child (lowest node index) whose token equals the target's choice at the
// current node (reference: spec_tree.py:108-118). out[0] = nodes on the path (root included), out[1] = the target's
// token at the last node, out[2 + i] = node index of path step i.
__global__ void accept_tree(const int32_t* cand, const int32_t* parent, const int32_t* tgt, int M, int32_t* out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int cur = 0, len = 1;
    out[2] = 0;
    for (;;) {
      int nxt = -1;
      for (int ch = cur + 1; ch < M; ch++)
        if (parent[ch] == cur && cand[ch] == tgt[cur]) { nxt = ch; break; }
      if (nxt < 0) break;
      out[2 + len] = nxt;
      len++;
      cur = nxt;
    }
    out[0] = len;
    out[1] = tgt[cur];
  }
}
// cache row pos + step <- row pos + path[step] for step = 1 .. len-1, K and V, every layer (reference:
// spec_tree.py:124-128). path indices grow strictly, so no row is read after it was overwritten.
// grid (n_layer, 2); `acc` is accept_tree's output.
__global__ void kv_compact(uint16_t* kc, uint16_t* vc, const int32_t* acc, int pos, size_t layer_elems, int row_elems, int max_seq) {
  uint16_t* base = (blockIdx.y ? vc : kc) + (size_t)blockIdx.x * layer_elems;
  const int len = acc[0];
  for (int step = 1; step < len; step++) {
    const int src = pos + acc[2 + step], dst = pos + step;
    if (src == dst || src >= max_seq || dst >= max_seq || src < 0) continue;
    const uint4* s = reinterpret_cast<const uint4*>(base + (size_t)src * row_elems);
    uint4* d = reinterpret_cast<uint4*>(base + (size_t)dst * row_elems);
    for (int i = threadIdx.x; i < row_elems / 8; i += blockDim.x) d[i] = s[i];
  }
}

// ------------------------------------------------------------------------------------------------ draft head
__device__ __forceinline__ float dot8(const uint4& w, const uint4& x, float acc) {
  acc = fmaf(bflo(w.x), bflo(x.x), acc); acc = fmaf(bfhi(w.x), bfhi(x.x), acc);
  acc = fmaf(bflo(w.y), bflo(x.y), acc); acc = fmaf(bfhi(w.y), bfhi(x.y), acc);
  acc = fmaf(bflo(w.z), bflo(x.z), acc); acc = fmaf(bfhi(w.z), bfhi(x.z), acc);
  acc = fmaf(bflo(w.w), bflo(x.w), acc); acc = fmaf(bfhi(w.w), bfhi(x.w), acc);
  return acc;
}

enum { DL_STORE = 0, DL_RESID = 1, DL_SWIGLU = 2, DL_LOGITS = 3 };

struct DLin {
  const uint16_t* W;            // bf16 [N, K] (torch Linear layout), K = k0 + k1
  const uint16_t* W2;           // DL_SWIGLU: the `up` matrix, same shape
  const uint16_t* x0;           // first input segment: bf16 rows of k0 elements, ldx0 apart
  const uint16_t* x1;           // second segment (k1 elements, ldx1 apart) or nullptr: the input is cat(x0, x1)
  const int32_t* x1_tokens;     // when set, segment 1 of token t is row x1_tokens[t] of x1 (an embedding table); < 0: zeros
  int ldx0, ldx1, k0, k1;
  int N, T;
  uint16_t* y;                  // bf16 [T, N] rows ldy apart (STORE / RESID / SWIGLU)
  const uint16_t* resid;        // DL_RESID: y = bf16(resid + bf16(acc)), rows ldr apart
  float* yf;                    // DL_LOGITS: f32 [T, N] = bf16(bf16(acc) / scale), rows ldy apart
  int ldy, ldr;
  float scale;
};

// y[t, n] = sum_k W[n, k] x[t, k] for TT tokens t0 .. t0+TT-1 at a time: the tokens' inputs sit in shared memory, a warp
// owns output row n and streams it with 16-byte loads. Weights are read once per TT tokens.
template <int TT, int MODE>
__global__ void __launch_bounds__(256) d_linear(const DLin P, int t0) {
  extern __shared__ __align__(16) uint16_t d_xs[];
  const int K = P.k0 + P.k1, KV = K >> 3;
  const int tid = threadIdx.x, lane = tid & 31;
  pdl_trigger();
  pdl_wait();
  for (int idx = tid; idx < TT * KV; idx += 256) {
    const int t = idx / KV, c = (idx % KV) << 3, tok = t0 + t;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tok < P.T) {
      if (c < P.k0) {
        v = *reinterpret_cast<const uint4*>(P.x0 + (size_t)tok * P.ldx0 + c);
      } else if (P.x1_tokens) {
        const int id = P.x1_tokens[tok];
        if (id >= 0) v = *reinterpret_cast<const uint4*>(P.x1 + (size_t)id * P.ldx1 + (c - P.k0));
      } else {
        v = *reinterpret_cast<const uint4*>(P.x1 + (size_t)tok * P.ldx1 + (c - P.k0));
      }
    }
    *reinterpret_cast<uint4*>(d_xs + (size_t)t * K + c) = v;
  }
  __syncthreads();
  const int warp = blockIdx.x * 8 + (tid >> 5), nwarps = gridDim.x * 8;
  for (int n = warp; n < P.N; n += nwarps) {
    float acc[TT], acc2[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) acc[t] = acc2[t] = 0.f;
    const uint4* wr = reinterpret_cast<const uint4*>(P.W + (size_t)n * K);
    const uint4* wr2 = MODE == DL_SWIGLU ? reinterpret_cast<const uint4*>(P.W2 + (size_t)n * K) : nullptr;
    // few tokens leave registers for more loads in flight per warp: a GEMV of 2560 rows gives an SM only ~17 warps
    constexpr int UNR = TT <= 2 ? 8 : (TT <= 4 ? 4 : 2);
#pragma unroll UNR
    for (int c = lane; c < KV; c += 32) {
      const uint4 w = __ldg(wr + c);
      uint4 w2 = make_uint4(0, 0, 0, 0);
      if (MODE == DL_SWIGLU) w2 = __ldg(wr2 + c);
#pragma unroll
      for (int t = 0; t < TT; t++) {
        const uint4 xv = *reinterpret_cast<const uint4*>(d_xs + (size_t)t * K + (c << 3));
        acc[t] = dot8(w, xv, acc[t]);
        if (MODE == DL_SWIGLU) acc2[t] = dot8(w2, xv, acc2[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
        if (MODE == DL_SWIGLU) acc2[t] += __shfl_xor_sync(0xffffffffu, acc2[t], o);
      }
    }
    if (lane == 0) {
#pragma unroll
      for (int t = 0; t < TT; t++) {
        const int tok = t0 + t;
        if (tok >= P.T) break;
        if (MODE == DL_STORE) {
          P.y[(size_t)tok * P.ldy + n] = f2bf(acc[t]);
        } else if (MODE == DL_RESID) {
          P.y[(size_t)tok * P.ldy + n] = f2bf(bf2f(P.resid[(size_t)tok * P.ldr + n]) + rbf(acc[t]));
        } else if (MODE == DL_SWIGLU) {
          const float g = rbf(acc[t]), u = rbf(acc2[t]);
          P.y[(size_t)tok * P.ldy + n] = f2bf(rbf(g / (1.0f + expf(-g))) * u);
        } else {
          P.yf[(size_t)tok * P.ldy + n] = rbf(rbf(acc[t]) / P.scale);
        }
      }
    }
  }
}

// y = bf16(bf16(x * r) * w), r = bf16(rsqrt(bf16(bf16(mean(bf16(x^2))) + eps))): RMSNorm as a bf16 PyTorch expression
// evaluates it (reference: train/draft_model.py:9-10). One CTA of 256 threads per row.
__global__ void __launch_bounds__(256) d_rmsnorm(const uint16_t* x, int ldx, const uint16_t* w, uint16_t* y, int ldy, int D, float eps) {
  __shared__ float red[8];
  const int tid = threadIdx.x;
  pdl_trigger();
  pdl_wait();
  const uint16_t* xr = x + (size_t)blockIdx.x * ldx;
  float ss = 0.f;
  for (int i = tid; i < D; i += 256) {
    const float v = bf2f(xr[i]);
    ss += rbf(v * v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) tot += red[i];
  const float r = rbf(rsqrtf(rbf(rbf(tot / (float)D) + eps)));
  for (int i = tid; i < D; i += 256)
    y[(size_t)blockIdx.x * ldy + i] = f2bf(rbf(bf2f(xr[i]) * r) * bf2f(w[i]));
}

// Half-split rotation of q and k (bf16 cos / sin tables as the reference casts them, reference:
// train/draft_model.py:12-22) and the cache write: token t's rotated k and its v go to cache slot slots[t].
// grid (T, n_head + n_kv), 64 threads: one CTA per (token, head), a thread per rotation pair (the angle's powf / cosf /
// sinf are the slow part: one per thread). q is rotated in place; a kv-head CTA also copies its v row.
__global__ void d_rope_store(uint16_t* q, const uint16_t* k, const uint16_t* v, const int32_t* positions, const int32_t* slots,
                             uint16_t* kc, uint16_t* vc, int nh, int nkv, int hd, float rope_base, int max_roll) {
  const int t = blockIdx.x, head = blockIdx.y, half = hd >> 1;
  pdl_trigger();
  pdl_wait();
  const float pos = (float)positions[t];
  const int slot = slots ? slots[t] : t;
  if (slot < 0 || slot >= max_roll) return;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float inv = 1.0f / powf(rope_base, (float)(2 * i) / (float)hd);
    const float ang = pos * inv;
    const float c = rbf(cosf(ang)), s = rbf(sinf(ang));
    if (head < nh) {
      uint16_t* p = q + ((size_t)t * nh + head) * hd;
      const float a = bf2f(p[i]), b = bf2f(p[i + half]);
      p[i] = f2bf(rbf(a * c) + rbf(-b * s));
      p[i + half] = f2bf(rbf(b * c) + rbf(a * s));
    } else {
      const int kh = head - nh;
      const uint16_t* p = k + ((size_t)t * nkv + kh) * hd;
      uint16_t* d = kc + ((size_t)slot * nkv + kh) * hd;
      const float a = bf2f(p[i]), b = bf2f(p[i + half]);
      d[i] = f2bf(rbf(a * c) + rbf(-b * s));
      d[i + half] = f2bf(rbf(b * c) + rbf(a * s));
    }
  }
  if (head >= nh) {
    const int kh = head - nh;
    for (int o = threadIdx.x; o < hd; o += blockDim.x)
      vc[((size_t)slot * nkv + kh) * hd + o] = v[((size_t)t * nkv + kh) * hd + o];
  }
}

// Causal attention of token t over cache slots 0 .. slots[t] (the rows of a lower-triangular mask, reference:
// train/draft_model.py:43,57-59). grid (T, nh), 128 threads; softmax in fp32, output bf16.
__global__ void __launch_bounds__(128) d_attn(const uint16_t* q, const int32_t* slots, const uint16_t* kc, const uint16_t* vc,
                                              uint16_t* out, int nh, int nkv, int hd, int max_roll) {
  extern __shared__ float d_sc[];                  // [max_roll] scores, then [hd] is not needed: threads own dims
  __shared__ float red[4];
  const int t = blockIdx.x, head = blockIdx.y, kh = head / (nh / nkv), tid = threadIdx.x;
  pdl_trigger();
  pdl_wait();
  const int last = min(slots ? slots[t] : t, max_roll - 1);
  if (last < 0) return;
  const uint16_t* qr = q + ((size_t)t * nh + head) * hd;
  const float scale = rsqrtf((float)hd);
  float mx = -INFINITY;
  for (int s = tid; s <= last; s += 128) {
    const uint16_t* kr = kc + ((size_t)s * nkv + kh) * hd;
    float d = 0.f;
    for (int i = 0; i < hd; i++) d = fmaf(bf2f(qr[i]), bf2f(kr[i]), d);
    d *= scale;
    d_sc[s] = d;
    mx = fmaxf(mx, d);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  float den = 0.f;
  for (int s = tid; s <= last; s += 128) {
    const float e = expf(d_sc[s] - mx);
    d_sc[s] = e;
    den += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
  if ((tid & 31) == 0) red[tid >> 5] = den;
  __syncthreads();
  den = red[0] + red[1] + red[2] + red[3];
  for (int i = tid; i < hd; i += 128) {
    float a = 0.f;
    for (int s = 0; s <= last; s++) a = fmaf(d_sc[s], bf2f(vc[((size_t)s * nkv + kh) * hd + i]), a);
    out[((size_t)t * nh + head) * hd + i] = f2bf(a / den);
  }
}

}  // namespace fb
