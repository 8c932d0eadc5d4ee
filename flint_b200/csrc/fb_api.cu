// extern "C" boundary of libflintb200.so: context management, weight re-layout and the launches.
// No torch types, no CPU fallback: a failed CUDA call or an unsupported shape is an error code.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <new>

#include "../../include/flint_b200.h"
#include "fb_ctx.hpp"
#include "fb_decode.cuh"
#include "fb_verify.cuh"
#include "fb_vsub.cuh"
#include "fb_vtc.cuh"

using namespace fb;


namespace {

struct KernelEntry {
  int dim, ko, ffn, head_dim, rgqa, hz;
  const void* fn2;
  const void* fn_long;     // the variant whose attention reads K/V through the weight ring (long caches), or NULL
};

// KD: model width, KO: attention output width of this rank, KF: FFN width of this rank
#define FB_DECODE_ENTRY(KD, KO, KF, HD, R)                                              \
  {KD, KO, KF, HD, R, 0, (const void*)decode_mega2<KD, KO, KF, HD, R, false>, nullptr},  \
  {KD, KO, KF, HD, R, 1, (const void*)decode_mega2<KD, KO, KF, HD, R, true>, nullptr}
// ... with the long-cache variant as well
#define FB_DECODE_ENTRY_LONG(KD, KO, KF, HD, R)                                                            \
  {KD, KO, KF, HD, R, 0, (const void*)decode_mega2<KD, KO, KF, HD, R, false>,                               \
   (const void*)decode_mega2<KD, KO, KF, HD, R, false, true>},                                             \
  {KD, KO, KF, HD, R, 1, (const void*)decode_mega2<KD, KO, KF, HD, R, true>,                                \
   (const void*)decode_mega2<KD, KO, KF, HD, R, true, true>}

const KernelEntry kDecodeKernels[] = {
    FB_DECODE_ENTRY_LONG(512, 512, 1408, 64, 4),  // tiny test decoder
    FB_DECODE_ENTRY(512, 512, 1536, 64, 4),       // tiny decoder whose FFN splits into whole groups over 2 ranks
    FB_DECODE_ENTRY(512, 256, 768, 64, 4),        // ... and its 2-rank slice
    FB_DECODE_ENTRY(640, 640, 1024, 80, 4),       // small decoder with heads of 80 ...
    FB_DECODE_ENTRY(640, 384, 512, 80, 4),        // ... whose 2-rank slice reads a widened O window (320 columns in 3 groups)
    FB_DECODE_ENTRY_LONG(2560, 2560, 8192, 80, 4),   // 3B-class (32 q / 8 kv heads of 80)
#ifndef FB_KERNELS_MINIMAL                        // (a build for kernel experiments keeps only the shapes above)
    FB_DECODE_ENTRY(2560, 2560, 8192, 64, 5),     // the reference's native Granite shape (40 q / 8 kv heads of 64)
    FB_DECODE_ENTRY_LONG(4096, 4096, 14336, 128, 4),   // 8B-class
    FB_DECODE_ENTRY(2560, 1280, 4096, 80, 4),     // 3B-class over 2 GPUs
    FB_DECODE_ENTRY(2560, 640, 2048, 80, 4),      // 3B-class over 4 GPUs
    FB_DECODE_ENTRY(2560, 384, 1024, 80, 4),      // 3B-class over 8 GPUs (320 attention columns inside 3 whole groups)
    FB_DECODE_ENTRY(4096, 2048, 7168, 128, 4),    // 8B-class over 2 GPUs
    FB_DECODE_ENTRY(4096, 1024, 3584, 128, 4),    // 8B-class over 4 GPUs
    FB_DECODE_ENTRY(4096, 512, 1792, 128, 4),     // 8B-class over 8 GPUs
    FB_DECODE_ENTRY(2048, 2048, 8192, 64, 4),     // 1B-class (32 q / 8 kv heads of 64)
#endif
#ifdef FB_EXTRA_DECODE_ENTRIES                    // further shapes named at build time (csrc/build.py: FLINT_B200_EXTRA_SHAPES)
    FB_EXTRA_DECODE_ENTRIES
#endif
};
constexpr int kNumDecodeKernels = sizeof(kDecodeKernels) / sizeof(kDecodeKernels[0]);
constexpr int kLongKvMin = 1;                     // cached positions from which the long-cache variant runs (fb_set_option 8 overrides)

// columns of the O projection a rank reads: its heads' columns widened to whole int4 groups (a rank of the 3B-class
// model split 8 ways owns 320 columns = 2.5 groups: it reads 384 and feeds zeros for its neighbour's 64)
void o_window(int width, int rank, int* ko, int* off) {
  const int start = rank * width, lo = start / 128 * 128, hi = (start + width + 127) / 128 * 128;
  *ko = hi - lo;
  *off = start - lo;
}

int find_kernel(const fb_model_desc& d, int ko) {
  if (d.n_kv_head <= 0 || d.n_head % d.n_kv_head) return -1;
  for (int i = 0; i < kNumDecodeKernels; i++) {
    const KernelEntry& e = kDecodeKernels[i];
    if (e.dim == d.dim && e.ko == ko && e.ffn == d.ffn && e.head_dim == d.head_dim &&
        e.rgqa == d.n_head / d.n_kv_head && e.hz == (d.has_zeros ? 1 : 0))
      return i;
  }
  return -1;
}

int cuda_fail(fb_ctx* c, cudaError_t e) {
  if (c) c->last_cuda_error = (int)e;
  return FB_ERR_CUDA;
}

#define FB_CUDA(c, call)                                   \
  do {                                                     \
    cudaError_t e__ = (call);                              \
    if (e__ != cudaSuccess) return cuda_fail((c), e__);    \
  } while (0)

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

int chunks_for(const fb_ctx* c, int T) {
  if (c->force_chunks > 0) return c->force_chunks < c->maxchunks ? c->force_chunks : c->maxchunks;
  // spread every kv head over as many CTAs as there are (one sweep of the consumer warps covers ~32 positions)
  int n = (T + 15) / 16;
  if (n < 1) n = 1;
  return n < c->maxchunks ? n : c->maxchunks;
}

// every K the stand-alone entry points (re-layout, dequantise, GEMV) are built for
#ifndef FB_EXTRA_K
#define FB_EXTRA_K(X)                             // widths of the build-time extra shapes that this list lacks
#endif
#define FB_FOR_EACH_K(X) X(256) X(384) X(512) X(640) X(768) X(1024) X(1280) X(1408) X(1536) X(1792) X(2048) X(2560) X(3584) X(4096) X(7168) X(8192) X(14336) FB_EXTRA_K(X)

template <int K>
int launch_gemv_k(bool hz, const GemvParams& p, int grid, cudaStream_t st) {
  cudaError_t e;
  if (hz) {
    e = cudaFuncSetAttribute(gemv_stream<TCfg<K>, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    gemv_stream<TCfg<K>, true><<<grid, kThreads, kSmemBytes, st>>>(p);
  } else {
    e = cudaFuncSetAttribute(gemv_stream<TCfg<K>, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    gemv_stream<TCfg<K>, false><<<grid, kThreads, kSmemBytes, st>>>(p);
  }
  return (int)cudaGetLastError();
}

bool supported_k(int k) {
  switch (k) {
#define X(K_) case K_:
    FB_FOR_EACH_K(X)
#undef X
    return true;
  }
  return false;
}

// caller layout -> tiles, for `layers` stacked matrices of `rows` rows each
cudaError_t launch_repack(const void* q, const void* s, const void* z, int layers, int rows, int k, int order, int arg,
                          int orows, uint8_t* out, cudaStream_t st) {
  const int tiles = (rows + tile_rt(k) - 1) / tile_rt(k);
  switch (k) {
#define X(K_)                                                                                                          \
  case K_:                                                                                                             \
    repack_tiles<K_><<<dim3(tiles, layers), 128, 0, st>>>((const uint32_t*)q, (const uint16_t*)s, (const uint16_t*)z, rows, \
                                                          order, arg, orows, out);                                     \
    break;
    FB_FOR_EACH_K(X)
#undef X
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

template <int MT, int K, int EPI, int HD, int ROWS>
cudaError_t launch_vgemm_r(const VGemmParams& p, int sms, cudaStream_t st) {
  static bool configured[64] = {};        // the attribute belongs to a device's copy of the function: once per device
  using V = VG<MT, K, ROWS>;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(v_gemm<MT, K, EPI, HD, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, V::smem());
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int per_sm = (227 * 1024) / (V::smem() + 1024) >= 2 ? 2 : 1;      // persistent CTAs: as many as are resident
  const int nrb = (p.rows + V::ROWS - 1) / V::ROWS;
  const int grid = nrb < sms * per_sm ? nrb : sms * per_sm;
  return launch_pdl(v_gemm<MT, K, EPI, HD, ROWS>, dim3(grid), dim3(V::NTHR), V::smem(), st, p);
}
template <int MT, int K, int EPI, int HD>
cudaError_t launch_vgemm_k(const VGemmParams& p, int sms, cudaStream_t st) {
  // tall matrices (gate/up, LM head) with few tokens: 64-row blocks halve the per-chunk overhead per MMA and still
  // give every SM at least one block
  if constexpr (MT == 16 && (EPI == EPI_SWIGLU || EPI == EPI_LOGITS)) {
    if (p.rows >= 64 * sms) return launch_vgemm_r<MT, K, EPI, HD, 64>(p, sms, st);
  }
  return launch_vgemm_r<MT, K, EPI, HD, 32>(p, sms, st);
}
// the shapes the decode kernel table knows: K = model width for QKV / gate-up / LM head and O, FFN width for down
// whether the bf16 warp-level verify GEMM is instantiated for a model's widths (the other verify kernels take them at
// run time)
bool vgemm_known(int D, int QD, int FF, int HD) {
  const bool qkv = (D == 512 && HD == 64) || (D == 2560 && (HD == 80 || HD == 64)) || (D == 4096 && HD == 128);
  const bool kd = D == 512 || D == 2560 || D == 4096, kq = QD == 512 || QD == 2560 || QD == 4096;
  const bool kf = FF == 1408 || FF == 8192 || FF == 14336 || FF == 512 || FF == 2560 || FF == 4096;
  return qkv && kd && kq && kf;
}

template <int MT, int EPI>
cudaError_t launch_vgemm_shape(const VGemmParams& p, int k, int hd, int sms, cudaStream_t st) {
  if constexpr (EPI == EPI_QKV) {
    if (k == 512 && hd == 64) return launch_vgemm_k<MT, 512, EPI, 64>(p, sms, st);
    if (k == 2560 && hd == 80) return launch_vgemm_k<MT, 2560, EPI, 80>(p, sms, st);
    if (k == 2560 && hd == 64) return launch_vgemm_k<MT, 2560, EPI, 64>(p, sms, st);
    if (k == 4096 && hd == 128) return launch_vgemm_k<MT, 4096, EPI, 128>(p, sms, st);
    return cudaErrorInvalidValue;
  } else {
    switch (k) {
      case 512: return launch_vgemm_k<MT, 512, EPI, 64>(p, sms, st);
      case 2560: return launch_vgemm_k<MT, 2560, EPI, 64>(p, sms, st);
      case 4096: return launch_vgemm_k<MT, 4096, EPI, 64>(p, sms, st);
    }
    if constexpr (EPI == EPI_RESID) {
      switch (k) {
        case 1408: return launch_vgemm_k<MT, 1408, EPI_RESID, 64>(p, sms, st);
        case 8192: return launch_vgemm_k<MT, 8192, EPI_RESID, 64>(p, sms, st);
        case 14336: return launch_vgemm_k<MT, 14336, EPI_RESID, 64>(p, sms, st);
      }
    }
    return cudaErrorInvalidValue;
  }
}
template <int EPI>
cudaError_t launch_vgemm_mt(const VGemmParams& p, int mt, int k, int hd, int sms, cudaStream_t st) {
  switch (mt) {
    case 16: return launch_vgemm_shape<16, EPI>(p, k, hd, sms, st);
    case 32: return launch_vgemm_shape<32, EPI>(p, k, hd, sms, st);
    case 64: return launch_vgemm_shape<64, EPI>(p, k, hd, sms, st);
  }
  return cudaErrorInvalidValue;
}
constexpr int kTcMaxItems = 256;      // split-K work items whose partial sums the context can hold

// K splits of one verify GEMM: enough (row block, split) items to occupy the GPU, whole groups per split, at most 4
// partials to add, at most kTcMaxGroups groups per item
int tc_splits(int rows, int k, int sms) {
  const int rb = (rows + kTcRowBlock - 1) / kTcRowBlock, G = k / 128;
  int ns = 1;
  while (ns < 4 && rb * ns < sms * 3 / 4 && G / (ns * 2) >= 2 && rb * ns * 2 <= kTcMaxItems) ns *= 2;
  while ((G + ns - 1) / ns > kTcMaxGroups && ns < 64) ns *= 2;
  return ns;
}

template <int NT, int EPI>
cudaError_t launch_vsub_nt(const VsubParams& p, int sms, cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(v_gemm_sub<NT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kVsSmem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return launch_pdl(v_gemm_sub<NT, EPI>, dim3(sms), dim3(kVsThreads), (size_t)p.plan.bar_off + 512, st, p);
}
template <int EPI>
cudaError_t launch_vsub(const VsubParams& p, int sms, cudaStream_t st) {
  switch ((p.M + 7) / 8) {
    case 1: return launch_vsub_nt<1, EPI>(p, sms, st);
    case 2: return launch_vsub_nt<2, EPI>(p, sms, st);
    case 3: return launch_vsub_nt<3, EPI>(p, sms, st);
    case 4: return launch_vsub_nt<4, EPI>(p, sms, st);
  }
  return cudaErrorInvalidValue;
}

template <int MT, int EPI, bool HZ>
cudaError_t launch_vtc_hz(VtcParams& p, int sms, cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(v_gemm_tc<MT, EPI, HZ>, cudaFuncAttributeMaxDynamicSharedMemorySize, VtcSmem<MT, HZ>::TOTAL);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  p.nsplit = tc_splits(p.rows, p.K, sms);
  const int items = ((p.rows + kTcRowBlock - 1) / kTcRowBlock) * p.nsplit;
  if (p.K % 128 || (p.K / 128 + p.nsplit - 1) / p.nsplit > kTcMaxGroups || (p.nsplit > 1 && items > kTcMaxItems))
    return cudaErrorInvalidValue;
  return launch_pdl(v_gemm_tc<MT, EPI, HZ>, dim3(items < sms ? items : sms), dim3(kTcThreads), (size_t)VtcSmem<MT, HZ>::TOTAL, st, p);
}
template <int MT, int EPI>
cudaError_t launch_vtc_mt(VtcParams& p, int sms, cudaStream_t st) {
  return p.has_zeros ? launch_vtc_hz<MT, EPI, true>(p, sms, st) : launch_vtc_hz<MT, EPI, false>(p, sms, st);
}
template <int EPI>
cudaError_t launch_vtc(VtcParams& p, int mt, int sms, cudaStream_t st) {
  switch (mt) {
    case 16: return launch_vtc_mt<16, EPI>(p, sms, st);
    case 32: return launch_vtc_mt<32, EPI>(p, sms, st);
    case 64: return launch_vtc_mt<64, EPI>(p, sms, st);
  }
  return cudaErrorInvalidValue;
}

template <int MT, bool HZ>
cudaError_t launch_vchain_hz(VchainParams& p, int sms, cudaStream_t st) {
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(v_chain_tc<MT, HZ>, cudaFuncAttributeMaxDynamicSharedMemorySize, VtcSmem<MT, HZ>::TOTAL);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  for (int i = 0; i < p.nph; i++) {
    VtcPhase& f = p.ph[i];
    f.nsplit = tc_splits(f.rows, f.K, sms);
    const int items = ((f.rows + kTcRowBlock - 1) / kTcRowBlock) * f.nsplit;
    if (f.K % 128 || (f.K / 128 + f.nsplit - 1) / f.nsplit > kTcMaxGroups || (f.nsplit > 1 && items > kTcMaxItems) ||
        (f.rows + kTcRowBlock - 1) / kTcRowBlock * 4 > 4096)
      return cudaErrorInvalidValue;
  }
  void* args[] = {&p};
  // every CTA must be resident: the loaders of a phase wait for the epilogue warps of the whole grid
  return cudaLaunchCooperativeKernel((const void*)v_chain_tc<MT, HZ>, dim3(sms), dim3(kTcThreads), args,
                                     (size_t)VtcSmem<MT, HZ>::TOTAL, st);
}
cudaError_t launch_vchain(VchainParams& p, int mt, bool hz, int sms, cudaStream_t st) {
  switch (mt) {
    case 16: return hz ? launch_vchain_hz<16, true>(p, sms, st) : launch_vchain_hz<16, false>(p, sms, st);
    case 32: return hz ? launch_vchain_hz<32, true>(p, sms, st) : launch_vchain_hz<32, false>(p, sms, st);
    case 64: return hz ? launch_vchain_hz<64, true>(p, sms, st) : launch_vchain_hz<64, false>(p, sms, st);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_vnorm(const uint16_t* h, const uint16_t* w, uint16_t* xn_t, uint16_t* xn_nat, int D, int M, float eps,
                         cudaStream_t st) {
  if (D % 16 || D > 8 * 256 * 2) return cudaErrorInvalidValue;
  if (D <= 8 * 256) return launch_pdl(v_rmsnorm<1>, dim3(M), dim3(256), 0, st, h, w, xn_t, xn_nat, D, eps);
  return launch_pdl(v_rmsnorm<2>, dim3(M), dim3(256), 0, st, h, w, xn_t, xn_nat, D, eps);
}
constexpr int kVSpans = 32;       // most spans of positions a kv head's attention is cut into

cudaError_t launch_vattn(const fb_ctx* c, const uint16_t* q, const uint16_t* kc, const uint16_t* vc, const uint8_t* amask,
                         uint16_t* ao, int pos, int M, int natural, cudaStream_t st) {
  const fb_model_desc& d = c->d;
  const int T = pos + M;
  // a CTA takes 64 query rows (four 16-row tiles); spans of positions are sized so that about two CTAs per SM exist
  const int mgroups = (M * c->rgqa + 63) / 64;
  int smax = (2 * c->sm_count) / (d.n_kv_head * mgroups);
  if (smax < 1) smax = 1;
  if (smax > kVSpans) smax = kVSpans;
  int S = (T + 63) / 64;
  if (S > smax) S = smax;
  const int span = ((T + S - 1) / S + 63) / 64 * 64;
  S = (T + span - 1) / span;
#define FB_VATTN(HD_, R_)                                                                                               \
  if (d.head_dim == HD_ && c->rgqa == R_) {                                                                             \
    cudaError_t e = launch_pdl(v_attn_mma<HD_, R_>, dim3(d.n_kv_head, S, mgroups), dim3(128), 0, st, q, kc, vc, amask, c->vpart,  \
                               d.n_head, d.n_kv_head, pos, M, d.attn_scale, span);                                      \
    if (e != cudaSuccess) return e;                                                                                     \
    return launch_pdl(v_attn_merge<HD_, R_>, dim3(M, d.n_kv_head), dim3(256), 0, st, (const float*)c->vpart, ao, d.n_head, \
                      d.n_kv_head, M, S, natural);                                                                      \
  }
  FB_VATTN(64, 4) FB_VATTN(80, 4) FB_VATTN(64, 5) FB_VATTN(128, 4)
#undef FB_VATTN
  return cudaErrorInvalidValue;
}

}  // namespace

extern "C" {

int fb_query(int device, fb_caps* out) {
  if (!out) return FB_ERR_ARG;
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) return FB_ERR_CUDA;
  memset(out, 0, sizeof(*out));
  out->device = device;
  out->sm_count = p.multiProcessorCount;
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->smem_per_block_optin = (int32_t)p.sharedMemPerBlockOptin;
  out->l2_bytes = p.l2CacheSize;
  out->cooperative_launch = p.cooperativeLaunch;
  out->total_mem_bytes = (int64_t)p.totalGlobalMem;
  cudaFuncAttributes fa;
  for (int i = 0; i < kNumDecodeKernels; i++)      /* registers of the 3B-class instantiation, the one the benchmark runs */
    if (kDecodeKernels[i].dim == 2560 && kDecodeKernels[i].head_dim == 80 && kDecodeKernels[i].ko == 2560 && !kDecodeKernels[i].hz) {
      if (cudaFuncGetAttributes(&fa, kDecodeKernels[i].fn2) == cudaSuccess) out->regs_decode_kernel = fa.numRegs;
      break;
    }
  return FB_OK;
}

int fb_ctx_create(const fb_model_desc* desc, int device, fb_ctx** out) {
  return fb_ctx_create_tp(desc, device, 0, 1, 0, out);
}

int fb_ctx_create_tp(const fb_model_desc* desc, int device, int32_t tp_rank, int32_t tp_size, int32_t vocab_base,
                     fb_ctx** out) {
  if (!desc || !out) return FB_ERR_ARG;
  *out = nullptr;
  const fb_model_desc& d = *desc;
  if (tp_size < 1 || tp_size > 8 || tp_rank < 0 || tp_rank >= tp_size) return FB_ERR_ARG;
  if (d.n_layer <= 0 || d.vocab <= 0 || d.dim % 128 || d.ffn % 128 || d.n_head <= 0 || d.head_dim <= 0) return FB_ERR_SHAPE;
  if (tp_size == 1 && d.n_head * d.head_dim != d.dim) return FB_ERR_SHAPE;
  int ko = 0, ao_off = 0;
  o_window(d.n_head * d.head_dim, tp_rank, &ko, &ao_off);
  if (tp_size == 1 && ao_off) return FB_ERR_SHAPE;
  const int kid = find_kernel(d, ko);
  if (kid < 0) return FB_ERR_SHAPE;
  DeviceGuard g(device);
  if (!g.ok) return FB_ERR_CUDA;
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) return FB_ERR_CUDA;
  if (p.major < 10 || !p.cooperativeLaunch || (int)p.sharedMemPerBlockOptin < kSmemBytes) return FB_ERR_SHAPE;
  fb_ctx* c = new (std::nothrow) fb_ctx();
  if (!c) return FB_ERR_ARG;
  memset(c, 0, sizeof(*c));
  c->d = d;
  c->device = device;
  c->sm_count = p.multiProcessorCount;
  c->kernel_id = kid;
  c->rgqa = d.n_head / d.n_kv_head;
  c->spin_limit = 4000000u;
  c->max_fly = 4;
  c->tp_size = tp_size; c->tp_rank = tp_rank; c->vocab_base = vocab_base; c->ko = ko; c->ao_off = ao_off;
  c->tag_base = 8;
  c->maxchunks = c->sm_count / d.n_kv_head;
  if (c->maxchunks < 1) c->maxchunks = 1;
  if (c->maxchunks > 64) c->maxchunks = 64;
  {  // every chunk CTA merges its share of the attention output with one tagged load per thread:
     // chunks * (R + ceil(R * HD/2 / chunks)) loads must fit the consumer threads
    const int pairs = c->rgqa * d.head_dim / 2;
    const int cap = (kConsumerThreads - pairs) / (c->rgqa + 1);
    if (c->maxchunks > cap) c->maxchunks = cap;
    if (c->maxchunks < 1) c->maxchunks = 1;
  }
  const int QD = d.n_head * d.head_dim;
  cudaError_t e = cudaSuccess;
  auto A = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
  A(dmalloc(&c->invf, sizeof(float) * (d.head_dim / 2)));
  A(dmalloc(&c->status, sizeof(DevStatus)));
  {
    const size_t inbox_words = (size_t)2 * tp_size * d.dim + 2 * (size_t)tp_size + 16;
    A(dmalloc(&c->inbox, inbox_words * 8));
    if (e == cudaSuccess) A(cudaMemset(c->inbox, 0, inbox_words * 8));
    c->peer_inbox[tp_rank] = c->inbox;
  }
  const size_t hp = d.head_dim / 2;
  const size_t wpc = (size_t)c->rgqa * d.head_dim + 2 * c->rgqa;
  const size_t ll_words[8] = {(size_t)d.dim / 2, d.n_head * hp, d.n_kv_head * hp, d.n_kv_head * hp, (size_t)ko / 2,
                              (size_t)d.ffn / 2, 2 * (size_t)c->sm_count, (size_t)d.n_kv_head * c->maxchunks * wpc};
  uint64_t** ll_ptrs[8] = {&c->h_ll, &c->q_ll, &c->k_ll, &c->v_ll, &c->ao_ll, &c->act_ll, &c->cand_ll, &c->part_ll};
  for (int i = 0; i < 8; i++) {
    A(dmalloc(ll_ptrs[i], 8 * ll_words[i] + 16));
    if (e == cudaSuccess) A(cudaMemset(*ll_ptrs[i], 0, 8 * ll_words[i] + 16));
  }
  {
    const size_t rowsz[5] = {(size_t)d.dim, (size_t)d.dim, (size_t)QD, (size_t)QD, (size_t)d.ffn};
    uint16_t** vp[5] = {&c->vh, &c->vxn, &c->vq, &c->vao, &c->vact};
    for (int i = 0; i < 5; i++) {
      A(dmalloc(vp[i], 64 * rowsz[i] * 2));
      if (e == cudaSuccess) A(cudaMemset(*vp[i], 0, 64 * rowsz[i] * 2));
    }
  }
  A(dmalloc(&c->vpart, (size_t)d.n_kv_head * 32 * 64 * c->rgqa * (d.head_dim + 2) * 4));
  A(dmalloc(&c->vsplit, (size_t)kTcMaxItems * 64 * 128 * 4));
  A(dmalloc(&c->vcount, kVsCounters * 4));
  if (e == cudaSuccess) A(cudaMemset(c->vcount, 0, kVsCounters * 4));
  A(cudaMalloc(&c->vrope, (size_t)64 * (d.head_dim / 2) * 8));
  A(dmalloc(&c->vssq, (size_t)2 * 256 * 64 * 4));
  A(dmalloc(&c->vgbar, (size_t)(d.n_layer + 2) * 4 * 4));
  A(dmalloc(&c->flags, 3 * 256 * 4));
  if (e == cudaSuccess) A(cudaMemset(c->flags, 0, 3 * 256 * 4));
  if (c->sm_count > 256) e = cudaErrorInvalidValue;
  {  // rows of the residual stream one CTA owns (whole tiles of the O and the down matrix)
    const int uo = tile_rt(ko) > tile_rt(d.ffn) ? tile_rt(ko) : tile_rt(d.ffn);
    const int units = (d.dim + uo - 1) / uo;
    if (((units + c->sm_count - 1) / c->sm_count + 1) * uo > kMaxOwnRows || (2 * d.ffn) % 4) e = cudaErrorInvalidValue;
  }
  if (e == cudaSuccess) {
    float invf[128];
    for (int i = 0; i < d.head_dim / 2; i++) invf[i] = (float)pow((double)d.rope_base, -2.0 * i / d.head_dim);
    A(cudaMemcpy(c->invf, invf, sizeof(float) * (d.head_dim / 2), cudaMemcpyHostToDevice));
    A(cudaMemset(c->status, 0, sizeof(DevStatus)));
    A(cudaFuncSetAttribute(kDecodeKernels[kid].fn2, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    if (kDecodeKernels[kid].fn_long)
      A(cudaFuncSetAttribute(kDecodeKernels[kid].fn_long, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  }
  if (e != cudaSuccess) {
    fb_ctx_destroy(c);
    return FB_ERR_CUDA;
  }
  *out = c;
  return FB_OK;
}

int fb_ctx_destroy(fb_ctx* c) {
  if (!c) return FB_ERR_ARG;
  DeviceGuard g(c->device);
  for (int p = 0; p < 8; p++)
    if (c->peers_open[p] && c->peer_inbox[p]) cudaIpcCloseMemHandle(c->peer_inbox[p]);
  void* ptrs[] = {c->w_qkv, c->w_o, c->w_gu, c->w_d, c->w_lm, c->invf,
                  c->status, c->h_ll, c->q_ll, c->k_ll, c->v_ll, c->ao_ll, c->act_ll, c->cand_ll, c->flags,
                  c->part_ll, c->vh, c->vxn, c->vq, c->vao, c->vact, c->vpart, c->inbox,
                  c->t_qkv, c->t_o, c->t_gu, c->t_d, c->t_lm, c->s_qkv, c->s_o, c->s_gu, c->s_d, c->s_lm, c->vsplit, c->vcount, c->vrope, c->vssq, c->vgbar};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  delete c;
  return FB_OK;
}

int fb_set_option(fb_ctx* c, int32_t what, int64_t value) {
  if (!c) return FB_ERR_ARG;
  if (what == 0) { c->spin_limit = (unsigned)value; return FB_OK; }       // spin limit of every device-side wait
  if (what == 1) { c->force_chunks = (int)value; return FB_OK; }          // attention chunks per kv head (0 = auto)
  if (what == 5) { c->poll_words = value != 0; return FB_OK; }
  if (what == 8) { if (value < 0 || value > 2) return FB_ERR_ARG; c->long_kv = (int)value; return FB_OK; }
  if (what == 7) { if (value < 0 || value > 4) return FB_ERR_ARG; c->verify_path = (int)value; return FB_OK; }
  if (what == 4) { if (value < 1 || value > kStages / 2) return FB_ERR_ARG; c->max_fly = (int)value; return FB_OK; }
  if (what == 2) { c->prof = (long long*)(uintptr_t)value; return FB_OK; } // device int64[sm_count * n_layer * 16] phase stamps (ns), 0 = off
  return FB_ERR_ARG;
}

int fb_last_status(fb_ctx* c, fb_status* out) {
  if (!c || !out) return FB_ERR_ARG;
  DeviceGuard g(c->device);
  DevStatus s;
  cudaError_t e = cudaMemcpy(&s, c->status, sizeof(s), cudaMemcpyDeviceToHost);
  memset(out, 0, sizeof(*out));
  out->cuda_error = c->last_cuda_error;
  if (e != cudaSuccess) {
    out->code = FB_ERR_CUDA;
    out->cuda_error = (int)e;
    return FB_ERR_CUDA;
  }
  out->code = s.code;
  out->where = s.where;
  out->layer = s.layer;
  out->block = s.block;
  out->expected = s.expected;
  out->seen = s.seen;
  if (s.code != 0) {   // a launch gave up: clear the report so that the next launch starts clean
    cudaMemset(c->status, 0, sizeof(DevStatus));
  }
  return FB_OK;
}

size_t fb_stream_bytes(int32_t rows, int32_t k, int32_t has_zeros) {
  if (rows < 0 || !supported_k(k)) return 0;
  return (size_t)pad_rows(rows, k) * rec_bytes_of(k, has_zeros);
}

int fb_repack(const void* d_q, const void* d_s, const void* d_z, int32_t rows, int32_t k, int32_t order, int32_t order_arg,
              int32_t order_rows, void* d_out, void* stream) {
  if (!d_q || !d_s || !d_out || rows <= 0 || k <= 0 || k % 128 || order < 0 || order > 2) return FB_ERR_ARG;
  if (order == 1 && (order_arg <= 0 || order_arg % 2 || order_rows % order_arg || order_rows > rows)) return FB_ERR_ARG;
  if (order == 2 && (order_arg * 2 != rows)) return FB_ERR_ARG;
  if (!supported_k(k)) return FB_ERR_SHAPE;
  return launch_repack(d_q, d_s, d_z, 1, rows, k, order, order_arg, order_rows, (uint8_t*)d_out, (cudaStream_t)stream) ==
                 cudaSuccess
             ? FB_OK
             : FB_ERR_CUDA;
}

int fb_dequant(const void* d_in, int32_t rows, int32_t k, int32_t has_zeros, int32_t order, int32_t order_arg,
               int32_t order_rows, float* d_out, void* stream) {
  if (!d_in || !d_out || rows <= 0 || k <= 0 || k % 128 || order < 0 || order > 2) return FB_ERR_ARG;
  switch (k) {
#define X(K_)                                                                                                         \
  case K_:                                                                                                            \
    dequant_tiles<K_><<<rows, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)d_in, rows, has_zeros, order, order_arg, \
                                                              order_rows, d_out);                                     \
    break;
    FB_FOR_EACH_K(X)
#undef X
    default: return FB_ERR_SHAPE;
  }
  return cudaGetLastError() == cudaSuccess ? FB_OK : FB_ERR_CUDA;
}

int fb_gemv(const void* d_in, int32_t rows, int32_t k, int32_t has_zeros, int32_t order, int32_t order_arg,
            int32_t order_rows, const void* d_x, float* d_y, void* d_status, void* stream) {
  if (!d_in || !d_x || !d_y || !d_status || rows <= 0) return FB_ERR_ARG;
  if (((uintptr_t)d_in & 15) || ((uintptr_t)d_x & 15)) return FB_ERR_ARG;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return FB_ERR_CUDA;
  GemvParams p{(const uint8_t*)d_in, (const uint16_t*)d_x, d_y, (DevStatus*)d_status, rows, order, order_arg, order_rows,
               4000000u};
  const bool hz = has_zeros != 0;
  cudaStream_t st = (cudaStream_t)stream;
  int e;
  switch (k) {
#define X(K_) case K_: e = launch_gemv_k<K_>(hz, p, sms, st); break;
    FB_FOR_EACH_K(X)
#undef X
    default: return FB_ERR_SHAPE;
  }
  return e == 0 ? FB_OK : FB_ERR_CUDA;
}

// ---- GEMV for callers that must not allocate ----------------------------------------------------------------------
// The streaming-layout copy of the matrix is the scratch of this path. Here it lives in one fixed array inside the
// library image instead of a buffer from cudaMalloc: every GPU that loads the library carries these 9 MiB until the
// process exits. `g_static_scratch` in HOST code is only a stand-in for the symbol, not a device address: the address
// a kernel can use comes from cudaGetSymbolAddress, once per device, with that device current.
constexpr size_t kStaticScratchBytes = (size_t)9 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static void* g_static_scratch_addr[64];      // per device ordinal, filled by the first call on that device

int fb_gemv_static(const void* d_q, const void* d_s, const void* d_z, int32_t rows, int32_t k, const void* d_x, float* d_y,
                   void* d_status, void* stream) {
  if (!d_q || !d_s || !d_x || !d_y || !d_status || rows <= 0 || k <= 0 || k % 128) return FB_ERR_ARG;
  const int hz = d_z != nullptr;
  if (!supported_k(k)) return FB_ERR_SHAPE;
  const size_t need = fb_stream_bytes(rows, k, hz);
  if (need > kStaticScratchBytes) return FB_ERR_RANGE;       /* matrix larger than the built-in scratch: use fb_gemv */
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FB_ERR_CUDA;
  if (!g_static_scratch_addr[dev]) {                          /* set-up, once per device, with that device current */
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return FB_ERR_CUDA;
    g_static_scratch_addr[dev] = p;
  }
  void* scratch = g_static_scratch_addr[dev];
  cudaStream_t st = (cudaStream_t)stream;
  /* the caller's status words must start at zero; the scratch itself needs no clearing: every byte of the rows*record
     range that the GEMV reads is rewritten by the re-layout below (padding included) */
  if (cudaMemsetAsync(d_status, 0, 32, st) != cudaSuccess) return FB_ERR_CUDA;
  int rc = fb_repack(d_q, d_s, d_z, rows, k, 0, 0, 0, scratch, stream);
  if (rc != FB_OK) return rc;
  return fb_gemv(scratch, rows, k, hz, 0, 0, 0, d_x, d_y, d_status, stream);
}

int fb_bind_weights(fb_ctx* c, const fb_weight_ptrs* w, void* stream) {
  if (!c || !w) return FB_ERR_ARG;
  const fb_model_desc& d = c->d;
  const bool hz = d.has_zeros != 0;
  const void* need[] = {w->qkv_q, w->qkv_s, w->o_q, w->o_s, w->gu_q, w->gu_s, w->d_q, w->d_s, w->lm_q, w->lm_s,
                        w->n1, w->n2, w->nf};   /* embed may be NULL when every step supplies its own residual */
  for (const void* p : need)
    if (!p) return FB_ERR_ARG;
  if (hz && (!w->qkv_z || !w->o_z || !w->gu_z || !w->d_z || !w->lm_z)) return FB_ERR_ARG;
  if (((uintptr_t)w->n1 & 15) || ((uintptr_t)w->n2 & 15) || ((uintptr_t)w->nf & 15)) return FB_ERR_ARG;
  DeviceGuard g(c->device);
  cudaStream_t st = (cudaStream_t)stream;
  const int L = d.n_layer, D = d.dim, FF = d.ffn, HD = d.head_dim;
  const int QKV = (d.n_head + 2 * d.n_kv_head) * HD, QD = d.n_head * HD;
  struct M { uint8_t** dst; uint8_t** tdst; uint8_t** sdst; const void *q, *s, *z; int layers, rows, k, order, arg, orows; };
  M ms[] = {
      {&c->w_qkv, &c->t_qkv, &c->s_qkv, w->qkv_q, w->qkv_s, w->qkv_z, L, QKV, D, 1, HD, (d.n_head + d.n_kv_head) * HD},
      {&c->w_o, &c->t_o, &c->s_o, w->o_q, w->o_s, w->o_z, L, D, c->ko, 0, 0, 0},
      {&c->w_gu, &c->t_gu, &c->s_gu, w->gu_q, w->gu_s, w->gu_z, L, 2 * FF, D, 2, FF, 0},
      {&c->w_d, &c->t_d, &c->s_d, w->d_q, w->d_s, w->d_z, L, D, FF, 0, 0, 0},
      {&c->w_lm, &c->t_lm, &c->s_lm, w->lm_q, w->lm_s, w->lm_z, 1, d.vocab, D, 0, 0, 0},
  };
  for (M& m : ms) {
    const size_t bytes = (size_t)m.layers * pad_rows(m.rows, m.k) * rec_bytes_of(m.k, hz);
    if (*m.dst) { cudaFree(*m.dst); *m.dst = nullptr; }
    FB_CUDA(c, dmalloc(m.dst, bytes + 16));
    FB_CUDA(c, launch_repack(m.q, m.s, hz ? m.z : nullptr, m.layers, m.rows, m.k, m.order, m.arg, m.orows, *m.dst, st));
    if (*m.tdst) { cudaFree(*m.tdst); *m.tdst = nullptr; }
    if (c->tp_size == 1) {     // the verify path's own copy, in the layout the tcgen05 GEMM streams
      const int nrb = (m.rows + kTcRowBlock - 1) / kTcRowBlock;
      FB_CUDA(c, dmalloc(m.tdst, (size_t)m.layers * tc_matrix_bytes(m.rows, m.k, hz) + 16));
      tc_repack<<<dim3(nrb, m.layers), 256, 0, st>>>((const uint32_t*)m.q, (const uint16_t*)m.s, hz ? (const uint16_t*)m.z : nullptr,
                                                     m.rows, m.k, m.order, m.arg, m.orows, *m.tdst);
      FB_CUDA(c, cudaGetLastError());
    }
    if (*m.sdst) { cudaFree(*m.sdst); *m.sdst = nullptr; }
    const int tiles32 = (m.rows + 31) / 32;
    const VsPlan vp = vs_plan(m.k, 1, tiles32);
    if (c->tp_size == 1 && !hz && vp.ok &&
        (size_t)tiles32 * vp.nkc * 8 * 512 <= (size_t)kTcMaxItems * 64 * 128 * 4) {   // K-split partials fit the shared buffer
      // the small-tree verify GEMM's copy (symmetric layout only; other shapes keep the bf16 warp-level kernel)
      FB_CUDA(c, dmalloc(m.sdst, (size_t)m.layers * vs_matrix_bytes(m.rows, m.k) + 16));
      vs_repack<<<dim3(tiles32, m.layers), 256, 0, st>>>((const uint32_t*)m.q, (const uint16_t*)m.s, m.rows, m.k, vp.ug, m.order,
                                                         m.arg, m.orows, *m.sdst);
      FB_CUDA(c, cudaGetLastError());
    }
  }
  c->n1 = w->n1; c->n2 = w->n2; c->nf = w->nf; c->embed = w->embed;
  c->weights_bound = true;
  return FB_OK;
}

// The caches as 3-D tensors for the long-cache decode variant: [n_layer * max_seq rows][n_kv heads][HD], box = HD x 1 head x
// one stage of positions. Returns false where the driver entry point is missing or refuses the shape: the plain variant runs.
static bool make_kv_maps(fb_ctx* c) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
      qres != cudaDriverEntryPointSuccess)
    return false;
  const fb_model_desc& d = c->d;
  const int HD = d.head_dim, R = d.n_head / d.n_kv_head;
  int nps = 0;
  if (HD == 64 && R == 4) nps = AttnCfg<64, 4>::NPS;
  else if (HD == 80 && R == 4) nps = AttnCfg<80, 4>::NPS;
  else if (HD == 128 && R == 4) nps = AttnCfg<128, 4>::NPS;
  else return false;
  const cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)d.n_kv_head, (cuuint64_t)d.n_layer * (cuuint64_t)c->max_seq};
  const cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)d.n_kv_head * HD * 2};
  const cuuint32_t box[3] = {(cuuint32_t)HD, 1u, (cuuint32_t)nps};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  void* bases[2] = {c->kc, c->vc};
  CUtensorMap* maps[2] = {&c->kmap, &c->vmap};
  for (int i = 0; i < 2; i++) {
    const CUresult r = ((EncodeFn)fn)(maps[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, bases[i], dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
  }
  return true;
}

int fb_bind_kv(fb_ctx* c, void* d_k, void* d_v, int32_t max_seq) {
  if (!c || !d_k || !d_v || max_seq <= 0) return FB_ERR_ARG;
  if (((uintptr_t)d_k & 15) || ((uintptr_t)d_v & 15)) return FB_ERR_ARG;
  c->kc = d_k; c->vc = d_v; c->max_seq = max_seq;
  DeviceGuard g(c->device);
  c->kv_maps = kDecodeKernels[c->kernel_id].fn_long != nullptr && c->tp_size == 1 && make_kv_maps(c);
  return FB_OK;
}

int fb_decode(fb_ctx* c, int32_t token, const int32_t* d_token, void* d_h, int32_t pos, float* d_logits, int32_t* d_next,
              void* stream) {
  if (!c) return FB_ERR_ARG;
  if (!c->weights_bound || !c->kc) return FB_ERR_STATE;
  const fb_model_desc& d = c->d;
  if (pos < 0 || pos >= c->max_seq) return FB_ERR_RANGE;
  if (!d_token && !d_h && (token < 0 || (c->tp_size == 1 && token >= d.vocab))) return FB_ERR_RANGE;
  if (!d_h && !c->embed) return FB_ERR_STATE;
  if (d_h && ((uintptr_t)d_h & 1)) return FB_ERR_ARG;
  DeviceGuard g(c->device);
  Decode2Params Q;
  memset(&Q, 0, sizeof(Q));
  Q.w_qkv = c->w_qkv; Q.w_o = c->w_o; Q.w_gu = c->w_gu; Q.w_d = c->w_d; Q.w_lm = c->w_lm;
  Q.n1 = (const uint16_t*)c->n1; Q.n2 = (const uint16_t*)c->n2; Q.nf = (const uint16_t*)c->nf;
  Q.embed = (const uint16_t*)c->embed; Q.invf = c->invf;
  Q.kc = (uint16_t*)c->kc; Q.vc = (uint16_t*)c->vc;
  if (c->kv_maps) { Q.kmap = c->kmap; Q.vmap = c->vmap; }
  Q.h_ll = c->h_ll; Q.q_ll = c->q_ll; Q.k_ll = c->k_ll; Q.v_ll = c->v_ll; Q.ao_ll = c->ao_ll; Q.act_ll = c->act_ll;
  Q.h_flags = c->flags; Q.act_flags = c->flags + 256; Q.ao_flags = c->flags + 512;
  Q.cand_ll = c->cand_ll; Q.part_ll = c->part_ll; Q.status = c->status;
  Q.d_token = d_token; Q.d_h = (uint16_t*)d_h; Q.d_logits = d_logits; Q.d_next = d_next;
  Q.token = token; Q.pos = pos; Q.max_seq = c->max_seq;
  Q.n_layer = d.n_layer; Q.dim = d.dim; Q.n_head = d.n_head; Q.n_kv = d.n_kv_head; Q.ffn = d.ffn; Q.vocab = d.vocab;
  Q.nchunks = chunks_for(c, pos + 1);
  Q.maxchunks = c->maxchunks;
  const unsigned span = (unsigned)(d.n_layer + 1) * 8u;
  if (c->tag_base > 0xffffffffu - 2 * span) c->tag_base = 8;      // tags never reach 0 (the value of fresh buffers)
  Q.tag_base = c->tag_base; Q.spin_limit = c->spin_limit;
  Q.eps = d.rms_eps; Q.attn_scale = d.attn_scale; Q.resid = d.resid_mult; Q.emb_mult = d.emb_mult;
  Q.logits_scaling = d.logits_scaling; Q.prof = c->prof; Q.max_fly = (unsigned)c->max_fly; Q.poll_words = c->poll_words;
  Q.tp_size = c->tp_size; Q.tp_rank = c->tp_rank; Q.vocab_base = c->vocab_base; Q.inbox = c->inbox; Q.ao_off = c->ao_off;
  for (int p = 0; p < c->tp_size; p++) {
    if (!c->peer_inbox[p]) return FB_ERR_STATE;       /* fb_tp_connect has not been called */
    Q.peer_inbox[p] = c->peer_inbox[p];
  }
  void* args2[] = {&Q};
  // long caches: the variant whose producer warp streams the K/V rows through the ring (8 x the bytes in flight)
  const KernelEntry& ke = kDecodeKernels[c->kernel_id];
  const bool long_kv = ke.fn_long && c->kv_maps && (c->long_kv == 1 || (c->long_kv == 0 && pos + 1 >= kLongKvMin));
  FB_CUDA(c, cudaLaunchCooperativeKernel(long_kv ? ke.fn_long : ke.fn2, dim3(c->sm_count), dim3(kThreads), args2,
                                         (size_t)kSmemBytes, (cudaStream_t)stream));
  c->tag_base += span;
  return FB_OK;
}

int fb_verify(fb_ctx* c, const int32_t* d_tokens, const void* d_h, const int32_t* d_depth, const uint8_t* d_amask,
              int32_t M, int32_t pos, float* d_logits, void* d_feat, void* stream) {
  if (!c || !d_depth || !d_amask || (!d_tokens && !d_h)) return FB_ERR_ARG;
  if (!c->weights_bound || !c->kc) return FB_ERR_STATE;
  if (c->tp_size > 1) return FB_ERR_STATE;           /* a tensor-parallel rank holds slices only */
  if (!d_h && !c->embed) return FB_ERR_STATE;
  if (M < 1 || M > 64) return FB_ERR_RANGE;          /* never fall through to another M (reference: result.md:112-113) */
  if (pos < 0 || pos + M > c->max_seq) return FB_ERR_RANGE;
  const fb_model_desc& d = c->d;
  DeviceGuard g(c->device);
  cudaStream_t st = (cudaStream_t)stream;
  const int MT = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  const int D = d.dim, FF = d.ffn, HD = d.head_dim, QD = d.n_head * HD, QKV = (d.n_head + 2 * d.n_kv_head) * HD;
  const bool hz = d.has_zeros != 0;
  const size_t strQ = (size_t)pad_rows(QKV, D) * rec_bytes_of(D, hz), strO = (size_t)pad_rows(D, QD) * rec_bytes_of(QD, hz),
               strG = (size_t)pad_rows(2 * FF, D) * rec_bytes_of(D, hz), strF = (size_t)pad_rows(D, FF) * rec_bytes_of(FF, hz);
  FB_CUDA(c, launch_pdl(v_embed, dim3(M), dim3(256), 0, st, d_tokens, (const uint16_t*)c->embed, (const uint16_t*)d_h, c->vh,
                        D, d.vocab, d.emb_mult, &c->status->code));
  if (c->verify_path == 3) {
    // ---- tcgen05 GEMM chains: per layer one launch covers O -> gate/up -> down -> the next layer's QKV (or the LM head)
    const size_t tQ = tc_matrix_bytes(QKV, D, hz), tO = tc_matrix_bytes(D, QD, hz), tG = tc_matrix_bytes(2 * FF, D, hz),
                 tF = tc_matrix_bytes(D, FF, hz);
    const int L = d.n_layer, nssq = (D + kTcRowBlock - 1) / kTcRowBlock * 4;
    float *ssqA = c->vssq, *ssqB = c->vssq + 256 * 64;
    if (nssq > 256) return FB_ERR_SHAPE;
    FB_CUDA(c, cudaMemsetAsync(c->vgbar, 0, (size_t)(L + 2) * 16, st));
    FB_CUDA(c, launch_pdl(v_rope_table, dim3(M), dim3(64), 0, st, d_depth, (const float*)c->invf, (int)pos, HD / 2, (float2*)c->vrope));
    VchainParams t;
    memset(&t, 0, sizeof(t));
    t.M = M; t.part = c->vsplit; t.counters = c->vcount; t.status = c->status; t.spin_limit = c->spin_limit;
    t.rope = (const float2*)c->vrope; t.n_head = d.n_head; t.nkv = d.n_kv_head; t.pos = pos; t.head_dim = HD; t.dim = D;
    t.resid = d.resid_mult; t.logits_scaling = d.logits_scaling; t.eps = d.rms_eps;
    auto kcl = [&](int l) { return (uint16_t*)c->kc + (size_t)l * c->max_seq * d.n_kv_head * HD; };
    auto vcl = [&](int l) { return (uint16_t*)c->vc + (size_t)l * c->max_seq * d.n_kv_head * HD; };
    auto qkv_phase = [&](int l, bool normed) {
      VtcPhase f;
      memset(&f, 0, sizeof(f));
      f.w = c->t_qkv + l * tQ; f.rows = QKV; f.K = D; f.epi = EPI_QKV; f.q = c->vq; f.kc = kcl(l); f.vc = vcl(l);
      if (normed) { f.x = c->vh; f.norm_w = (const uint16_t*)c->n1 + (size_t)l * D; f.ssq_in = ssqB; f.n_ssq = nssq; }
      else f.x = c->vxn;
      return f;
    };
    // layer 0's QKV reads the embeddings through the stand-alone norm kernel
    FB_CUDA(c, launch_vnorm(c->vh, (const uint16_t*)c->n1, nullptr, c->vxn, D, M, d.rms_eps, st));
    t.nph = 1; t.ph[0] = qkv_phase(0, false); t.gbar = c->vgbar;
    FB_CUDA(c, launch_vchain(t, MT, hz, c->sm_count, st));
    for (int l = 0; l < L; l++) {
      FB_CUDA(c, launch_vattn(c, c->vq, kcl(l), vcl(l), d_amask, c->vao, pos, M, 1, st));
      VtcPhase f;
      memset(&f, 0, sizeof(f));
      f.w = c->t_o + l * tO; f.x = c->vao; f.rows = D; f.K = QD; f.epi = EPI_RESID; f.h = c->vh; f.out_ld = D; f.ssq_out = ssqA;
      t.ph[0] = f;
      memset(&f, 0, sizeof(f));
      f.w = c->t_gu + l * tG; f.x = c->vh; f.norm_w = (const uint16_t*)c->n2 + (size_t)l * D; f.ssq_in = ssqA; f.n_ssq = nssq;
      f.rows = 2 * FF; f.K = D; f.epi = EPI_SWIGLU; f.act = c->vact; f.out_ld = FF;
      t.ph[1] = f;
      memset(&f, 0, sizeof(f));
      f.w = c->t_d + l * tF; f.x = c->vact; f.rows = D; f.K = FF; f.epi = EPI_RESID; f.h = c->vh; f.out_ld = D; f.ssq_out = ssqB;
      t.ph[2] = f;
      t.nph = 3;
      if (l + 1 < L) {
        t.ph[3] = qkv_phase(l + 1, true);
        t.nph = 4;
      } else if (d_logits) {
        memset(&f, 0, sizeof(f));
        f.w = c->t_lm; f.x = c->vh; f.norm_w = (const uint16_t*)c->nf; f.ssq_in = ssqB; f.n_ssq = nssq; f.xn_out = (uint16_t*)d_feat;
        f.rows = d.vocab; f.K = D; f.epi = EPI_LOGITS; f.logits = d_logits; f.out_ld = d.vocab;
        t.ph[3] = f;
        t.nph = 4;
      }
      t.gbar = c->vgbar + 4 * (l + 1);
      t.dbg = (c->prof && l == 1) ? c->prof : nullptr;
      FB_CUDA(c, launch_vchain(t, MT, hz, c->sm_count, st));
    }
    if (!d_logits && d_feat)
      FB_CUDA(c, launch_vnorm(c->vh, (const uint16_t*)c->nf, nullptr, (uint16_t*)d_feat, D, M, d.rms_eps, st));
    FB_CUDA(c, cudaGetLastError());
    return FB_OK;
  }
  if (c->verify_path == 2 || (c->verify_path == 0 && M > 16) || (c->verify_path != 3 && !vgemm_known(D, QD, FF, HD))) {
    // ---- tcgen05 path: natural-order activations, the matrices in the TC layout ----
    const size_t tQ = tc_matrix_bytes(QKV, D, hz), tO = tc_matrix_bytes(D, QD, hz), tG = tc_matrix_bytes(2 * FF, D, hz),
                 tF = tc_matrix_bytes(D, FF, hz);
    FB_CUDA(c, launch_pdl(v_rope_table, dim3(M), dim3(64), 0, st, d_depth, (const float*)c->invf, (int)pos, HD / 2, (float2*)c->vrope));
    VtcParams t;
    memset(&t, 0, sizeof(t));
    t.M = M; t.has_zeros = hz; t.part = c->vsplit; t.counters = c->vcount; t.status = c->status; t.spin_limit = c->spin_limit;
    t.rope = (const float2*)c->vrope; t.n_head = d.n_head; t.nkv = d.n_kv_head; t.pos = pos; t.head_dim = HD;
    t.resid = d.resid_mult; t.logits_scaling = d.logits_scaling;
    for (int l = 0; l < d.n_layer; l++) {
      uint16_t* kcl = (uint16_t*)c->kc + (size_t)l * c->max_seq * d.n_kv_head * HD;
      uint16_t* vcl = (uint16_t*)c->vc + (size_t)l * c->max_seq * d.n_kv_head * HD;
      FB_CUDA(c, launch_vnorm(c->vh, (const uint16_t*)c->n1 + (size_t)l * D, nullptr, c->vxn, D, M, d.rms_eps, st));
      t.w = c->t_qkv + l * tQ; t.x = c->vxn; t.rows = QKV; t.K = D; t.q = c->vq; t.kc = kcl; t.vc = vcl;
      FB_CUDA(c, launch_vtc<EPI_QKV>(t, MT, c->sm_count, st));
      FB_CUDA(c, launch_vattn(c, c->vq, kcl, vcl, d_amask, c->vao, pos, M, 1, st));
      t.w = c->t_o + l * tO; t.x = c->vao; t.rows = D; t.K = QD; t.h = c->vh; t.out_ld = D;
      FB_CUDA(c, launch_vtc<EPI_RESID>(t, MT, c->sm_count, st));
      FB_CUDA(c, launch_vnorm(c->vh, (const uint16_t*)c->n2 + (size_t)l * D, nullptr, c->vxn, D, M, d.rms_eps, st));
      t.w = c->t_gu + l * tG; t.x = c->vxn; t.rows = 2 * FF; t.K = D; t.act = c->vact; t.out_ld = FF;
      FB_CUDA(c, launch_vtc<EPI_SWIGLU>(t, MT, c->sm_count, st));
      t.w = c->t_d + l * tF; t.x = c->vact; t.rows = D; t.K = FF; t.out_ld = D;
      FB_CUDA(c, launch_vtc<EPI_RESID>(t, MT, c->sm_count, st));
    }
    // the feature goes to the caller in natural order; the LM head reads the same rows
    uint16_t* feat = d_feat ? (uint16_t*)d_feat : c->vxn;
    FB_CUDA(c, launch_vnorm(c->vh, (const uint16_t*)c->nf, nullptr, feat, D, M, d.rms_eps, st));
    if (d_logits) {
      t.w = c->t_lm; t.x = feat; t.rows = d.vocab; t.K = D; t.logits = d_logits; t.out_ld = d.vocab;
      FB_CUDA(c, launch_vtc<EPI_LOGITS>(t, MT, c->sm_count, st));
    }
    FB_CUDA(c, cudaGetLastError());
    return FB_OK;
  }
  VGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.has_zeros = hz; p.depth = d_depth; p.invf = c->invf; p.n_head = d.n_head; p.nkv = d.n_kv_head; p.pos = pos;
  p.resid = d.resid_mult; p.logits_scaling = d.logits_scaling;
  // small trees: every GEMM whose matrix has an R32 copy runs on the subnormal-operand kernel. It reads the same
  // activation buffers; the QKV and gate/up GEMMs read the residual rows and apply the RMSNorm themselves
  // by tree size: up to 8 tokens (one B tile) this kernel wins (2.07 vs 2.40 ms per pass of the 3B model); above, its
  // per-CTA conversion of the activations (linear in the tokens) costs more than the dequantisation it saves
  const bool use_sub = (c->verify_path == 4 || (c->verify_path == 0 && M <= 8)) && M <= kVsMaxTokens && !hz;
  VsubParams sp;
  memset(&sp, 0, sizeof(sp));
  sp.M = M; sp.part = c->vsplit; sp.counters = (int*)c->vcount; sp.status = c->status; sp.spin_limit = c->spin_limit;
  sp.rope = (const float2*)c->vrope; sp.n_head = d.n_head; sp.nkv = d.n_kv_head; sp.pos = pos; sp.head_dim = HD;
  sp.resid = d.resid_mult; sp.logits_scaling = d.logits_scaling; sp.eps = d.rms_eps;
  if (use_sub && c->s_qkv)
    FB_CUDA(c, launch_pdl(v_rope_table, dim3(M), dim3(64), 0, st, d_depth, (const float*)c->invf, (int)pos, HD / 2, (float2*)c->vrope));
  int nsub = 0;
  auto sub = [&](const uint8_t* sw, size_t layer, int rows, int K) -> bool {
    if (!use_sub || !sw) return false;
    sp.plan = vs_plan(K, M, (rows + 31) / 32);
    if (!sp.plan.ok) return false;
    sp.w = sw + layer * vs_matrix_bytes(rows, K); sp.rows = rows; sp.K = K; sp.norm_w = nullptr;
    sp.dbg = (c->prof && layer == 1) ? c->prof + 8 * (nsub++ & 7) : nullptr;   // stamps of the second layer's GEMMs
    return true;
  };
  for (int l = 0; l < d.n_layer; l++) {
    uint16_t* kcl = (uint16_t*)c->kc + (size_t)l * c->max_seq * d.n_kv_head * HD;
    uint16_t* vcl = (uint16_t*)c->vc + (size_t)l * c->max_seq * d.n_kv_head * HD;
    if (sub(c->s_qkv, l, QKV, D)) {
      if (sp.plan.nkc == 1) { sp.x = c->vh; sp.norm_w = (const uint16_t*)c->n1 + (size_t)l * D; }
      else {
        FB_CUDA(c, launch_vnorm(c->vh, (const uint16_t*)c->n1 + (size_t)l * D, c->vxn, nullptr, D, M, d.rms_eps, st));
        sp.x = c->vxn;
      }
      sp.q = c->vq; sp.kc = kcl; sp.vc = vcl;
      FB_CUDA(c, launch_vsub<EPI_QKV>(sp, c->sm_count, st));
    } else {
      FB_CUDA(c, launch_vnorm(c->vh, (const uint16_t*)c->n1 + (size_t)l * D, c->vxn, nullptr, D, M, d.rms_eps, st));
      p.w = c->w_qkv + l * strQ; p.x_t = c->vxn; p.rows = QKV;
      p.q = c->vq; p.kc = kcl; p.vc = vcl;
      FB_CUDA(c, launch_vgemm_mt<EPI_QKV>(p, MT, D, HD, c->sm_count, st));
    }
    FB_CUDA(c, launch_vattn(c, c->vq, kcl, vcl, d_amask, c->vao, pos, M, 0, st));
    if (sub(c->s_o, l, D, QD)) {
      sp.x = c->vao; sp.h = c->vh; sp.out_ld = D;
      FB_CUDA(c, launch_vsub<EPI_RESID>(sp, c->sm_count, st));
    } else {
      p.w = c->w_o + l * strO; p.x_t = c->vao; p.rows = D; p.h = c->vh; p.out_ld = D;
      FB_CUDA(c, launch_vgemm_mt<EPI_RESID>(p, MT, QD, HD, c->sm_count, st));
    }
    if (sub(c->s_gu, l, 2 * FF, D)) {
      if (sp.plan.nkc == 1) { sp.x = c->vh; sp.norm_w = (const uint16_t*)c->n2 + (size_t)l * D; }
      else {
        FB_CUDA(c, launch_vnorm(c->vh, (const uint16_t*)c->n2 + (size_t)l * D, c->vxn, nullptr, D, M, d.rms_eps, st));
        sp.x = c->vxn;
      }
      sp.act_t = c->vact; sp.out_ld = FF;
      FB_CUDA(c, launch_vsub<EPI_SWIGLU>(sp, c->sm_count, st));
    } else {
      FB_CUDA(c, launch_vnorm(c->vh, (const uint16_t*)c->n2 + (size_t)l * D, c->vxn, nullptr, D, M, d.rms_eps, st));
      p.w = c->w_gu + l * strG; p.x_t = c->vxn; p.rows = 2 * FF; p.act_t = c->vact;
      p.out_ld = FF;
      FB_CUDA(c, launch_vgemm_mt<EPI_SWIGLU>(p, MT, D, HD, c->sm_count, st));
    }
    if (sub(c->s_d, l, D, FF)) {
      sp.x = c->vact; sp.h = c->vh; sp.out_ld = D;
      FB_CUDA(c, launch_vsub<EPI_RESID>(sp, c->sm_count, st));
    } else {
      p.w = c->w_d + l * strF; p.x_t = c->vact; p.rows = D; p.h = c->vh; p.out_ld = D;
      FB_CUDA(c, launch_vgemm_mt<EPI_RESID>(p, MT, FF, HD, c->sm_count, st));
    }
  }
  FB_CUDA(c, launch_vnorm(c->vh, (const uint16_t*)c->nf, c->vxn, (uint16_t*)d_feat, D, M, d.rms_eps, st));
  if (d_logits) {
    if (sub(c->s_lm, 0, d.vocab, D)) {
      sp.x = c->vxn; sp.logits = d_logits; sp.out_ld = d.vocab;
      FB_CUDA(c, launch_vsub<EPI_LOGITS>(sp, c->sm_count, st));
    } else {
      p.w = c->w_lm; p.x_t = c->vxn; p.rows = d.vocab; p.logits = d_logits; p.out_ld = d.vocab;
      FB_CUDA(c, launch_vgemm_mt<EPI_LOGITS>(p, MT, D, HD, c->sm_count, st));
    }
  }
  FB_CUDA(c, cudaGetLastError());
  return FB_OK;
}

int fb_tp_export(fb_ctx* c, void* handle_out64) {
  if (!c || !handle_out64) return FB_ERR_ARG;
  DeviceGuard g(c->device);
  cudaIpcMemHandle_t h;
  FB_CUDA(c, cudaIpcGetMemHandle(&h, c->inbox));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle_out64, &h, 64);
  return FB_OK;
}

int fb_tp_connect(fb_ctx* c, const void* handles, int32_t n) {
  if (!c || !handles || n != c->tp_size) return FB_ERR_ARG;
  DeviceGuard g(c->device);
  for (int p = 0; p < n; p++) {
    if (p == c->tp_rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char*)handles + 64 * p, 64);
    void* ptr = nullptr;
    FB_CUDA(c, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    c->peer_inbox[p] = (uint64_t*)ptr;
    c->peers_open[p] = true;
  }
  return FB_OK;
}

int fb_tp_connect_local(fb_ctx* c, fb_ctx* const* ranks, int32_t n) {
  if (!c || !ranks || n != c->tp_size) return FB_ERR_ARG;
  DeviceGuard g(c->device);
  for (int p = 0; p < n; p++) {
    if (p == c->tp_rank) continue;
    fb_ctx* o = ranks[p];
    if (!o || o == c || o->tp_size != n || o->tp_rank != p || o->d.dim != c->d.dim) return FB_ERR_ARG;
    if (o->device != c->device) {
      int can = 0;
      FB_CUDA(c, cudaDeviceCanAccessPeer(&can, c->device, o->device));
      if (!can) return FB_ERR_STATE;
      cudaError_t e = cudaDeviceEnablePeerAccess(o->device, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
      else if (e != cudaSuccess) return cuda_fail(c, e);
    }
    c->peer_inbox[p] = o->inbox;
    c->peers_open[p] = false;                          /* not an IPC mapping: the owner frees it */
  }
  return FB_OK;
}

int fb_kv_move(fb_ctx* c, const int32_t* src, const int32_t* dst, int32_t n, void* stream) {
  if (!c || !c->kc || (n > 0 && (!src || !dst))) return FB_ERR_ARG;
  const fb_model_desc& d = c->d;
  DeviceGuard g(c->device);
  const size_t row = (size_t)d.n_kv_head * d.head_dim * 2, layer = (size_t)c->max_seq * row;
  for (int i = 0; i < n; i++) {     /* sequential, like the reference loop (reference: spec_tree.py:126-128) */
    if (src[i] < 0 || dst[i] < 0 || src[i] >= c->max_seq || dst[i] >= c->max_seq) return FB_ERR_RANGE;
    if (src[i] == dst[i]) continue;
    for (void* base : {c->kc, c->vc})
      FB_CUDA(c, cudaMemcpy2DAsync((char*)base + dst[i] * row, layer, (char*)base + src[i] * row, layer, row, d.n_layer,
                                   cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  }
  return FB_OK;
}

}  // extern "C"
