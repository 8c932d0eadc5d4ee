/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's batch-1 int4 decode step and of its
 * M-token tree-verify step. It is the checker the CUDA path is compared with (tests/, the smoke
 * check and the CPU-baseline leg of the benchmark); no product code path may call it.
 *
 * What is restated, and from where (paths are inside the reference project):
 *   int4 dequant  (nibble-8)*scale [+zero]        kernels/megakernel_decode.cu:30,34 ; engine/quantize.py:150-153
 *   RMSNorm, eps inside the sqrt, ONE bf16 round  kernels/megakernel_decode.cu:47-63
 *   QKV store as bf16                             kernels/megakernel_decode.cu:76-79
 *   half-split (HF/NEOX) RoPE on bf16 q,k         kernels/megakernel_decode.cu:82-89
 *   KV append at row pos (+m for verify)          kernels/megakernel_decode.cu:91-94 ; kernels/verify_mega.cu:153-158
 *   GQA attention, softmax over visible keys      kernels/megakernel_decode.cu:96-131 ; kernels/verify_mega.cu:163-198
 *   tree semantics: RoPE at pos+depth[m], key t>=pos visible iff amask[m][t-pos]   kernels/verify_mega.cu:143,169
 *   O-proj + scaled residual, bf16 store          kernels/megakernel_decode.cu:133-136
 *   gate/up, SwiGLU on bf16 g,u, down + residual  kernels/megakernel_decode.cu:147-160
 *   final norm, LM head / logits_scaling (fp32)   kernels/megakernel_decode.cu:195-200
 *   post-final-norm feature output                kernels/verify_mega.cu:282
 *
 * Where this file deliberately departs from the reference kernel: dot products and softmax are summed
 * in double (the kernel's fp32 lane-strided order is not reproducible by any other schedule), exp is
 * exact (the kernel uses __expf), and the RoPE angle is float(pos)*inv_freq with an fp32 inv_freq table
 * and exact sin/cos (the kernel uses fast-math powf/cosf/sinf, whose error grows with the angle).
 * Stores round to bf16 (round-to-nearest-even) at exactly the kernel's store sites.
 *
 * Pinning: this restatement is checked against (1) the reference's own packer and quantiser outputs,
 * (2) the reference's PyTorch engine (engine/model.py) run on CPU with the same dequantised weights
 * (committed fixtures under tests/golden/) and (3), on a GPU host where the reference kernels were built
 * into oracle/_ref, the reference megakernel itself at its native head shape.
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
  int32_t n_layer, dim, n_head, n_kv, head_dim, ffn, vocab, max_seq;
  int32_t has_zeros;
  float eps, rope_base, attn_scale, resid, logits_scaling;
} fo_desc;

/* Stacked per-layer tensors exactly as the reference boundary takes them (kernels/megakernel_decode.cu:204-211):
 * q words int32 [L, OUT, IN/8], scales/zeros bf16 [L, OUT, IN/128]; norm weights bf16. */
typedef struct {
  const uint32_t *qkv_q, *o_q, *gu_q, *d_q, *lm_q;
  const uint16_t *qkv_s, *o_s, *gu_s, *d_s, *lm_s;
  const uint16_t *qkv_z, *o_z, *gu_z, *d_z, *lm_z; /* NULL unless has_zeros */
  const uint16_t *n1, *n2, *nf;
} fo_weights;

static inline float bf2f(uint16_t b) {
  uint32_t u = ((uint32_t)b) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f2bf(float f) { /* round-to-nearest-even, NaN kept quiet */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* y[m*ldy + r] = sum_k ((nib-8)*s + z) * x[m*k + ...]   for r in [0, rows), m in [0, M).
 * x is the fp32 image of bf16 activations. Group partial sums are fp32 over exact products
 * (4-bit x 8-bit mantissas), group results are combined in double. */
void fo_gemv(const uint32_t *q, const uint16_t *s, const uint16_t *z, int rows, int k, const float *x, int M,
             float *y, int ldy) {
  const int words = k / 8, groups = k / 128;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; r++) {
    const uint32_t *qr = q + (size_t)r * words;
    const uint16_t *sr = s + (size_t)r * groups;
    const uint16_t *zr = z ? z + (size_t)r * groups : NULL;
    float wf[128];
    double acc[64];
    for (int m = 0; m < M; m++) acc[m] = 0.0;
    for (int g = 0; g < groups; g++) {
      for (int w = 0; w < 16; w++) {
        const uint32_t word = qr[g * 16 + w];
        for (int n = 0; n < 8; n++) wf[w * 8 + n] = (float)((word >> (4 * n)) & 0xF) - 8.0f;
      }
      const double sc = (double)bf2f(sr[g]);
      const double zc = zr ? (double)bf2f(zr[g]) : 0.0;
      for (int m = 0; m < M; m++) {
        const float *xm = x + (size_t)m * k + g * 128;
        float dot = 0.f, xs = 0.f;
#pragma omp simd reduction(+ : dot, xs)
        for (int i = 0; i < 128; i++) {
          dot += wf[i] * xm[i];
          xs += xm[i];
        }
        acc[m] += sc * (double)dot + zc * (double)xs;
      }
    }
    for (int m = 0; m < M; m++) y[(size_t)m * ldy + r] = (float)acc[m];
  }
}

/* xn = bf16( float(h) * r * float(w) ),  r = 1/sqrt(mean(h^2)+eps), product evaluated left to right in fp32. */
static void rmsnorm_row(const uint16_t *h, const uint16_t *w, int dim, float eps, uint16_t *xn) {
  double ss = 0.0;
  for (int i = 0; i < dim; i++) {
    const double v = bf2f(h[i]);
    ss += v * v;
  }
  const float r = (float)(1.0 / sqrt(ss / dim + (double)eps));
  for (int i = 0; i < dim; i++) xn[i] = f2bf(bf2f(h[i]) * r * bf2f(w[i]));
}

static void to_f32(const uint16_t *src, float *dst, size_t n) {
  for (size_t i = 0; i < n; i++) dst[i] = bf2f(src[i]);
}

/* One M-token step. h [M, dim] bf16 is the (already multiplied) embedding on entry and the final residual
 * on exit. kc/vc bf16 [L, max_seq, n_kv, head_dim]. depth int32 [M], amask uint8 [M, M].
 * logits f32 [M, vocab] (may be NULL), feat bf16 [M, dim] (may be NULL). Decode is M=1, depth={0}, amask={1}.
 * Returns 0, or a negative code on a bad argument. */
int fo_step(const fo_desc *d, const fo_weights *W, uint16_t *h, uint16_t *kc, uint16_t *vc, const int32_t *depth,
            const uint8_t *amask, int pos, int M, float *logits, uint16_t *feat) {
  const int D = d->dim, NH = d->n_head, NKV = d->n_kv, HD = d->head_dim, FF = d->ffn, V = d->vocab;
  const int QD = NH * HD, KVD = NKV * HD, QKV = QD + 2 * KVD, T = pos + M, rep = NH / NKV;
  if (M < 1 || M > 64 || pos < 0 || T > d->max_seq || D % 128 || FF % 128 || QD % 128) return -1;
  const int xmax = (FF > D ? FF : D) > QD ? (FF > D ? FF : D) : QD;
  uint16_t *xn = malloc(sizeof(uint16_t) * (size_t)M * xmax);
  float *xf = malloc(sizeof(float) * (size_t)M * xmax);
  float *y = malloc(sizeof(float) * (size_t)M * (2 * FF > QKV ? 2 * FF : QKV));
  uint16_t *qkv = malloc(sizeof(uint16_t) * (size_t)M * QKV);
  uint16_t *ao = malloc(sizeof(uint16_t) * (size_t)M * QD);
  uint16_t *act = malloc(sizeof(uint16_t) * (size_t)M * FF);
  float *invf = malloc(sizeof(float) * (HD / 2));
  double *sc = malloc(sizeof(double) * (size_t)T);
  for (int i = 0; i < HD / 2; i++) invf[i] = (float)pow((double)d->rope_base, -2.0 * i / HD);
  const size_t kst = (size_t)d->max_seq * KVD;

  for (int l = 0; l < d->n_layer; l++) {
    /* ---- attention block ---- */
    for (int m = 0; m < M; m++) rmsnorm_row(h + (size_t)m * D, W->n1 + (size_t)l * D, D, d->eps, xn + (size_t)m * D);
    to_f32(xn, xf, (size_t)M * D);
    fo_gemv(W->qkv_q + (size_t)l * QKV * (D / 8), W->qkv_s + (size_t)l * QKV * (D / 128),
            W->qkv_z ? W->qkv_z + (size_t)l * QKV * (D / 128) : NULL, QKV, D, xf, M, y, QKV);
    for (size_t i = 0; i < (size_t)M * QKV; i++) qkv[i] = f2bf(y[i]);
    for (int m = 0; m < M; m++) {
      const float p = (float)(pos + depth[m]);
      for (int hh = 0; hh < NH + NKV; hh++) {
        uint16_t *b = qkv + (size_t)m * QKV + (hh < NH ? hh * HD : QD + (hh - NH) * HD);
        for (int i = 0; i < HD / 2; i++) {
          const float ang = p * invf[i];
          const double c = (double)(float)cos((double)ang), s = (double)(float)sin((double)ang);
          const double x0 = bf2f(b[i]), x1 = bf2f(b[i + HD / 2]);
          b[i] = f2bf((float)(x0 * c - x1 * s));
          b[i + HD / 2] = f2bf((float)(x1 * c + x0 * s));
        }
      }
      memcpy(kc + l * kst + (size_t)(pos + m) * KVD, qkv + (size_t)m * QKV + QD, sizeof(uint16_t) * KVD);
      memcpy(vc + l * kst + (size_t)(pos + m) * KVD, qkv + (size_t)m * QKV + QD + KVD, sizeof(uint16_t) * KVD);
    }
    for (int m = 0; m < M; m++) {
      for (int qh = 0; qh < NH; qh++) {
        const int kv = qh / rep;
        const uint16_t *qv = qkv + (size_t)m * QKV + qh * HD;
        double mx = -INFINITY;
        for (int t = 0; t < T; t++) {
          if (t >= pos && !amask[m * M + (t - pos)]) {
            sc[t] = -INFINITY;
            continue;
          }
          const uint16_t *kt = kc + l * kst + ((size_t)t * NKV + kv) * HD;
          double dot = 0.0;
          for (int e = 0; e < HD; e++) dot += (double)bf2f(qv[e]) * (double)bf2f(kt[e]);
          sc[t] = (double)((float)dot * d->attn_scale);
          if (sc[t] > mx) mx = sc[t];
        }
        double den = 0.0;
        for (int t = 0; t < T; t++) {
          sc[t] = (sc[t] == -INFINITY) ? 0.0 : exp(sc[t] - mx);
          den += sc[t];
        }
        for (int e = 0; e < HD; e++) {
          double o = 0.0;
          for (int t = 0; t < T; t++)
            if (sc[t] != 0.0) o += sc[t] * (double)bf2f(vc[l * kst + ((size_t)t * NKV + kv) * HD + e]);
          ao[(size_t)m * QD + qh * HD + e] = f2bf((float)(o / den));
        }
      }
    }
    to_f32(ao, xf, (size_t)M * QD);
    fo_gemv(W->o_q + (size_t)l * D * (QD / 8), W->o_s + (size_t)l * D * (QD / 128),
            W->o_z ? W->o_z + (size_t)l * D * (QD / 128) : NULL, D, QD, xf, M, y, D);
    for (size_t i = 0; i < (size_t)M * D; i++) h[i] = f2bf((float)((double)bf2f(h[i]) + (double)y[i] * (double)d->resid));
    /* ---- MLP block ---- */
    for (int m = 0; m < M; m++) rmsnorm_row(h + (size_t)m * D, W->n2 + (size_t)l * D, D, d->eps, xn + (size_t)m * D);
    to_f32(xn, xf, (size_t)M * D);
    fo_gemv(W->gu_q + (size_t)l * 2 * FF * (D / 8), W->gu_s + (size_t)l * 2 * FF * (D / 128),
            W->gu_z ? W->gu_z + (size_t)l * 2 * FF * (D / 128) : NULL, 2 * FF, D, xf, M, y, 2 * FF);
    for (int m = 0; m < M; m++)
      for (int i = 0; i < FF; i++) {
        const float g = bf2f(f2bf(y[(size_t)m * 2 * FF + i])), u = bf2f(f2bf(y[(size_t)m * 2 * FF + FF + i]));
        act[(size_t)m * FF + i] = f2bf((float)(((double)g / (1.0 + exp(-(double)g))) * (double)u));
      }
    to_f32(act, xf, (size_t)M * FF);
    fo_gemv(W->d_q + (size_t)l * D * (FF / 8), W->d_s + (size_t)l * D * (FF / 128),
            W->d_z ? W->d_z + (size_t)l * D * (FF / 128) : NULL, D, FF, xf, M, y, D);
    for (size_t i = 0; i < (size_t)M * D; i++) h[i] = f2bf((float)((double)bf2f(h[i]) + (double)y[i] * (double)d->resid));
  }
  /* ---- final norm + LM head ---- */
  for (int m = 0; m < M; m++) rmsnorm_row(h + (size_t)m * D, W->nf, D, d->eps, xn + (size_t)m * D);
  if (feat) memcpy(feat, xn, sizeof(uint16_t) * (size_t)M * D);
  if (logits) {
    to_f32(xn, xf, (size_t)M * D);
    fo_gemv(W->lm_q, W->lm_s, W->lm_z, V, D, xf, M, logits, V);
    for (size_t i = 0; i < (size_t)M * V; i++) logits[i] = logits[i] / d->logits_scaling;
  }
  free(xn); free(xf); free(y); free(qkv); free(ao); free(act); free(invf); free(sc);
  return 0;
}

/* fp32 [rows, k] = (nibble-8)*float(s) + float(z): the dequantisation contract. */
void fo_dequant(const uint32_t *q, const uint16_t *s, const uint16_t *z, int rows, int k, float *out) {
  const int words = k / 8, groups = k / 128;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; r++)
    for (int c = 0; c < k; c++) {
      const uint32_t word = q[(size_t)r * words + c / 8];
      const float nib = (float)((word >> (4 * (c % 8))) & 0xF) - 8.0f;
      const float sc = bf2f(s[(size_t)r * groups + c / 128]);
      const float v = nib * sc;
      out[(size_t)r * k + c] = z ? v + bf2f(z[(size_t)r * groups + c / 128]) : v;
    }
}

/* Launchers export OMP_NUM_THREADS=1 to their children (torch.distributed.run does): the timed CPU baseline sets the
 * thread count itself. Returns the count in force. */
int fo_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

int fo_argmax(const float *v, int n) { /* first index of the maximum (torch.argmax tie rule) */
  int best = 0;
  for (int i = 1; i < n; i++)
    if (v[i] > v[best]) best = i;
  return best;
}
