// extern "C" entry points of the speculative-decoding side: sampling, acceptance, KV compaction, the EAGLE draft head.
// No torch types, no CPU fallback: a failed CUDA call or an unsupported shape is an error code.
#include <string.h>

#include <new>

#include "../../include/flint_b200.h"
#include "fb_ctx.hpp"
#include "fb_spec.cuh"

using namespace fb;

struct fb_draft {
  fb_draft_desc d;
  int device, sm_count;
  fb_draft_weights w;
  bool bound;
  uint16_t *x, *h, *q, *k, *v, *att, *x2, *act, *hh, *fn;     // [max_tokens] rows of activations
  uint16_t *kc, *vc;                                           // [max_roll, n_kv, hd]
  float* logits;                                               // [max_heads rows, vocab]
  int last_cuda_error;
};

namespace {

constexpr int kMaxHeadRows = 16;

template <class T>
cudaError_t dmalloc(T** p, size_t n) { return cudaMalloc(reinterpret_cast<void**>(p), n); }

struct DeviceGuard {
  int prev;
  bool ok;
  explicit DeviceGuard(int dev) : prev(0), ok(false) {
    if (cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) ok = true;
  }
  ~DeviceGuard() { if (ok) cudaSetDevice(prev); }
};

template <int TT, int MODE>
cudaError_t launch_linear_tt(const DLin& p, int t0, int sms, cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  const size_t smem = (size_t)TT * (p.k0 + p.k1) * 2;
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(d_linear<TT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  int per_sm = (int)((220 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
  int grid = (p.N + 7) / 8;
  if (grid > sms * per_sm) grid = sms * per_sm;
  return launch_pdl(d_linear<TT, MODE>, dim3(grid), dim3(256), smem, st, p, t0);
}

// all T tokens, in blocks of up to 16 where two CTAs of 16 input rows still share an SM, else up to 8 (fewer tokens per
// block where 8 rows of inputs do not fit shared memory): the weights are read once per block
template <int MODE>
cudaError_t launch_linear(const DLin& p, int sms, cudaStream_t st) {
  const int K = p.k0 + p.k1;
  if (K % 8 || p.k0 % 8 || p.N <= 0 || p.T <= 0) return cudaErrorInvalidValue;
  const int cap = K * 2 * 8 <= 200 * 1024 ? 8 : (K * 2 * 4 <= 200 * 1024 ? 4 : (K * 2 * 2 <= 200 * 1024 ? 2 : 1));
  for (int t0 = 0; t0 < p.T;) {
    const int left = p.T - t0;
    cudaError_t e;
    if (left >= 16 && K * 2 * 16 <= 100 * 1024) { e = launch_linear_tt<16, MODE>(p, t0, sms, st); t0 += 16; }
    else if (left >= 8 && cap >= 8) { e = launch_linear_tt<8, MODE>(p, t0, sms, st); t0 += 8; }
    else if (left >= 4 && cap >= 4) { e = launch_linear_tt<4, MODE>(p, t0, sms, st); t0 += 4; }
    else if (left >= 2 && cap >= 2) { e = launch_linear_tt<2, MODE>(p, t0, sms, st); t0 += 2; }
    else { e = launch_linear_tt<1, MODE>(p, t0, sms, st); t0 += 1; }
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

int dfail(fb_draft* d, cudaError_t e) {
  if (d) d->last_cuda_error = (int)e;
  return FB_ERR_CUDA;
}
#define FB_DCUDA(d, call)                                 \
  do {                                                    \
    cudaError_t e__ = (call);                             \
    if (e__ != cudaSuccess) return dfail((d), e__);       \
  } while (0)

}  // namespace

extern "C" {

int fb_sample(const float* d_logits, int32_t vocab, int32_t rows, int64_t row_stride, float temperature, int32_t top_k,
              uint64_t seed, uint64_t counter, int32_t* d_out, void* stream) {
  if (!d_logits || !d_out || vocab <= 0 || rows <= 0 || row_stride < 0) return FB_ERR_ARG;
  SampleParams p{d_logits, (long long)row_stride, vocab, top_k, temperature, (unsigned long long)seed,
                 (unsigned long long)counter, d_out};
  sample_rows<<<rows, 1024, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_CUDA;
}

int fb_accept_chain(const int32_t* d_target, const int32_t* d_draft, int32_t k, int32_t* d_out, void* stream) {
  if (!d_target || !d_out || k < 0 || (k > 0 && !d_draft)) return FB_ERR_ARG;
  accept_chain<<<1, 32, 0, (cudaStream_t)stream>>>(d_target, d_draft, k, d_out);
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_CUDA;
}

int fb_accept_tree(const int32_t* d_cand, const int32_t* d_parent, const int32_t* d_target, int32_t m, int32_t* d_out,
                   void* stream) {
  if (!d_cand || !d_parent || !d_target || !d_out || m < 1 || m > 64) return FB_ERR_ARG;
  accept_tree<<<1, 32, 0, (cudaStream_t)stream>>>(d_cand, d_parent, d_target, m, d_out);
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_CUDA;
}

int fb_kv_compact(fb_ctx* c, const int32_t* d_accept, int32_t pos, void* stream) {
  if (!c || !c->kc || !d_accept) return FB_ERR_ARG;
  if (pos < 0 || pos >= c->max_seq) return FB_ERR_RANGE;
  const fb_model_desc& d = c->d;
  DeviceGuard g(c->device);
  const int row = d.n_kv_head * d.head_dim;
  if (row % 8) return FB_ERR_SHAPE;
  kv_compact<<<dim3(d.n_layer, 2), 128, 0, (cudaStream_t)stream>>>((uint16_t*)c->kc, (uint16_t*)c->vc, d_accept, pos,
                                                                  (size_t)c->max_seq * row, row, c->max_seq);
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_CUDA;
}

int fb_draft_create(const fb_draft_desc* desc, int device, fb_draft** out) {
  if (!desc || !out) return FB_ERR_ARG;
  *out = nullptr;
  const fb_draft_desc& d = *desc;
  if (d.dim <= 0 || d.n_head <= 0 || d.n_kv_head <= 0 || d.dim % d.n_head || d.n_head % d.n_kv_head || d.inter <= 0 ||
      d.fuse < 1 || d.vocab <= 0 || d.max_roll < 1 || d.max_tokens < 1)
    return FB_ERR_SHAPE;
  const int hd = d.dim / d.n_head;
  if (d.dim % 8 || d.inter % 8 || hd % 2 || (d.n_kv_head * hd) % 8) return FB_ERR_SHAPE;
  DeviceGuard g(device);
  if (!g.ok) return FB_ERR_CUDA;
  fb_draft* r = new (std::nothrow) fb_draft();
  if (!r) return FB_ERR_ARG;
  memset(r, 0, sizeof(*r));
  r->d = d;
  r->device = device;
  if (cudaDeviceGetAttribute(&r->sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) { delete r; return FB_ERR_CUDA; }
  const size_t T = d.max_tokens, D = d.dim, kvd = (size_t)d.n_kv_head * hd, F = (size_t)d.fuse * d.dim;
  cudaError_t e = cudaSuccess;
  auto A = [&](cudaError_t x) { if (e == cudaSuccess) e = x; };
  A(dmalloc(&r->x, T * D * 2)); A(dmalloc(&r->h, T * D * 2)); A(dmalloc(&r->q, T * D * 2));
  A(dmalloc(&r->k, T * kvd * 2)); A(dmalloc(&r->v, T * kvd * 2)); A(dmalloc(&r->att, T * D * 2));
  A(dmalloc(&r->x2, T * D * 2)); A(dmalloc(&r->act, T * (size_t)d.inter * 2)); A(dmalloc(&r->hh, T * D * 2));
  A(dmalloc(&r->fn, (size_t)kMaxHeadRows * D * 2));
  A(dmalloc(&r->kc, (size_t)d.max_roll * kvd * 2)); A(dmalloc(&r->vc, (size_t)d.max_roll * kvd * 2));
  A(dmalloc(&r->logits, (size_t)kMaxHeadRows * d.vocab * 4));
  if (e == cudaSuccess) A(cudaMemset(r->kc, 0, (size_t)d.max_roll * kvd * 2));
  if (e == cudaSuccess) A(cudaMemset(r->vc, 0, (size_t)d.max_roll * kvd * 2));
  (void)F;
  if (e != cudaSuccess) { fb_draft_destroy(r); return FB_ERR_CUDA; }
  *out = r;
  return FB_OK;
}

int fb_draft_destroy(fb_draft* r) {
  if (!r) return FB_ERR_ARG;
  DeviceGuard g(r->device);
  void* ptrs[] = {r->x, r->h, r->q, r->k, r->v, r->att, r->x2, r->act, r->hh, r->fn, r->kc, r->vc, r->logits};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  delete r;
  return FB_OK;
}

int fb_draft_bind(fb_draft* r, const fb_draft_weights* w) {
  if (!r || !w) return FB_ERR_ARG;
  const void* need[] = {w->merge, w->n1, w->n2, w->q, w->k, w->v, w->o, w->gate, w->up, w->down, w->fout, w->nf, w->embed};
  for (const void* p : need)
    if (!p || ((uintptr_t)p & 15)) return FB_ERR_ARG;
  r->w = *w;
  r->bound = true;
  return FB_OK;
}

int fb_draft_forward(fb_draft* r, const void* d_feat, const void* d_emb, const int32_t* d_tokens, const int32_t* d_positions,
                     const int32_t* d_slots, int32_t T, void* d_out, void* stream) {
  if (!r || !d_feat || !d_positions || !d_out || (!d_emb && !d_tokens)) return FB_ERR_ARG;
  if (!r->bound) return FB_ERR_STATE;
  const fb_draft_desc& d = r->d;
  if (T < 1 || T > d.max_tokens || (!d_slots && T > d.max_roll)) return FB_ERR_RANGE;
  if (((uintptr_t)d_feat & 15) || ((uintptr_t)d_emb & 15) || ((uintptr_t)d_out & 1)) return FB_ERR_ARG;
  DeviceGuard g(r->device);
  cudaStream_t st = (cudaStream_t)stream;
  const int D = d.dim, F = d.fuse * d.dim, hd = D / d.n_head, kvd = d.n_kv_head * hd, sms = r->sm_count;
  const uint16_t* W = nullptr;
  DLin p;
  // x = merge(cat(feat, emb))
  memset(&p, 0, sizeof(p));
  p.W = (const uint16_t*)r->w.merge; p.x0 = (const uint16_t*)d_feat; p.ldx0 = F; p.k0 = F;
  if (d_emb) { p.x1 = (const uint16_t*)d_emb; p.ldx1 = D; }
  else { p.x1 = (const uint16_t*)r->w.embed; p.ldx1 = D; p.x1_tokens = d_tokens; }
  p.k1 = D; p.N = D; p.T = T; p.y = r->x; p.ldy = D;
  FB_DCUDA(r, launch_linear<DL_STORE>(p, sms, st));
  FB_DCUDA(r, launch_pdl(d_rmsnorm, dim3(T), dim3(256), 0, st, (const uint16_t*)r->x, D, (const uint16_t*)r->w.n1, r->h, D, D, d.rms_eps));
  // q, k, v
  const void* qkvw[3] = {r->w.q, r->w.k, r->w.v};
  uint16_t* qkvo[3] = {r->q, r->k, r->v};
  const int qkvn[3] = {D, kvd, kvd};
  for (int i = 0; i < 3; i++) {
    memset(&p, 0, sizeof(p));
    p.W = (const uint16_t*)qkvw[i]; p.x0 = r->h; p.ldx0 = D; p.k0 = D; p.N = qkvn[i]; p.T = T; p.y = qkvo[i]; p.ldy = qkvn[i];
    FB_DCUDA(r, launch_linear<DL_STORE>(p, sms, st));
  }
  FB_DCUDA(r, launch_pdl(d_rope_store, dim3(T, d.n_head + d.n_kv_head), dim3(64), 0, st, r->q, (const uint16_t*)r->k, (const uint16_t*)r->v, d_positions,
                         d_slots, r->kc, r->vc, d.n_head, d.n_kv_head, hd, d.rope_base, d.max_roll));
  FB_DCUDA(r, launch_pdl(d_attn, dim3(T, d.n_head), dim3(128), (size_t)d.max_roll * 4, st, (const uint16_t*)r->q, d_slots,
                         (const uint16_t*)r->kc, (const uint16_t*)r->vc, r->att, d.n_head, d.n_kv_head, hd, d.max_roll));
  // x2 = x + o(att)
  memset(&p, 0, sizeof(p));
  p.W = (const uint16_t*)r->w.o; p.x0 = r->att; p.ldx0 = D; p.k0 = D; p.N = D; p.T = T; p.y = r->x2; p.ldy = D;
  p.resid = r->x; p.ldr = D;
  FB_DCUDA(r, launch_linear<DL_RESID>(p, sms, st));
  FB_DCUDA(r, launch_pdl(d_rmsnorm, dim3(T), dim3(256), 0, st, (const uint16_t*)r->x2, D, (const uint16_t*)r->w.n2, r->h, D, D, d.rms_eps));
  // act = silu(gate h) * up h
  memset(&p, 0, sizeof(p));
  p.W = (const uint16_t*)r->w.gate; p.W2 = (const uint16_t*)r->w.up; p.x0 = r->h; p.ldx0 = D; p.k0 = D; p.N = d.inter; p.T = T;
  p.y = r->act; p.ldy = d.inter;
  FB_DCUDA(r, launch_linear<DL_SWIGLU>(p, sms, st));
  // hh = x2 + down(act)
  memset(&p, 0, sizeof(p));
  p.W = (const uint16_t*)r->w.down; p.x0 = r->act; p.ldx0 = d.inter; p.k0 = d.inter; p.N = D; p.T = T; p.y = r->hh; p.ldy = D;
  p.resid = r->x2; p.ldr = D;
  FB_DCUDA(r, launch_linear<DL_RESID>(p, sms, st));
  // out = fout(hh)
  memset(&p, 0, sizeof(p));
  p.W = (const uint16_t*)r->w.fout; p.x0 = r->hh; p.ldx0 = D; p.k0 = D; p.N = F; p.T = T; p.y = (uint16_t*)d_out; p.ldy = F;
  FB_DCUDA(r, launch_linear<DL_STORE>(p, sms, st));
  (void)W;
  FB_DCUDA(r, cudaGetLastError());
  return FB_OK;
}

int fb_draft_head(fb_draft* r, const void* d_feat_rows, int32_t n, int32_t top_b, int32_t* d_tokens, float* d_scores,
                  void* stream) {
  if (!r || !d_feat_rows || !d_tokens) return FB_ERR_ARG;
  if (!r->bound) return FB_ERR_STATE;
  const fb_draft_desc& d = r->d;
  if (n < 1 || n > kMaxHeadRows || top_b < 1 || top_b > 16 || top_b > d.vocab) return FB_ERR_RANGE;
  DeviceGuard g(r->device);
  cudaStream_t st = (cudaStream_t)stream;
  const int D = d.dim, F = d.fuse * d.dim;
  // the token head reads the HIGH slice (last dim elements) of the fused feature (reference: spec_mega.py:43-44)
  FB_DCUDA(r, launch_pdl(d_rmsnorm, dim3(n), dim3(256), 0, st, (const uint16_t*)d_feat_rows + (F - D), F, (const uint16_t*)r->w.nf, r->fn, D, D,
                         d.rms_eps));
  DLin p;
  memset(&p, 0, sizeof(p));
  p.W = (const uint16_t*)r->w.embed; p.x0 = r->fn; p.ldx0 = D; p.k0 = D; p.N = d.vocab; p.T = n; p.yf = r->logits; p.ldy = d.vocab;
  p.scale = d.logits_scaling;
  FB_DCUDA(r, launch_linear<DL_LOGITS>(p, r->sm_count, st));
  FB_DCUDA(r, launch_pdl(topb_rows, dim3(n), dim3(1024), 0, st, (const float*)r->logits, (long long)d.vocab, d.vocab, top_b, d_tokens,
                         d_scores));
  FB_DCUDA(r, cudaGetLastError());
  return FB_OK;
}

}  // extern "C"
