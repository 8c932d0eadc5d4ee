// The weight pipeline every streaming kernel of this library shares, the stand-alone GEMV built on it and the kernels
// that convert between the caller's weight layout and the tiled streaming layout.
//
// One CTA per SM: the last warp (lane 0) is the producer; it walks the CTA's static list of weight tiles and issues
// 1-D bulk copies into an 8-stage shared-memory ring. It never waits for activations, so the weights of the next
// phase stream in while the consumers are still waiting for their inputs. The other warps are consumers: warp w takes
// tiles w, w + n, ... straight off the ring; there are no warp groups and no block-wide barriers in the steady state.
#pragma once
#include "fb_common.cuh"

namespace fb {

struct Pipe {
  uint8_t* stages;
  uint64_t* full;
  uint64_t* empty;
  volatile int* landed;  // stage loads that are known to be complete (written by the producer, read by consumers)
  uint32_t it;           // running stage-load counter; producer and consumers walk the same sequence
  uint32_t max_fly;      // producer only: bulk copies allowed in flight at once (1..kStages/2)
};

struct Smem {
  uint8_t* stages;
  uint8_t* scratch;
  __half* xh;          // activations of the current phase (fp16, B-operand order); bf16 while they are being gathered
  uint64_t* full;
  uint64_t* empty;
  volatile int* s_abort;
  volatile int* landed;
  float* red;          // 32 floats for block reductions
  int* misc;           // 32 ints
  float* hown;         // [2 * kMaxOwnRows] this CTA's rows of the residual stream, then tensor-parallel partial sums
  float* qpart;        // [kStages][2 tiles][4 slices][4 rows] slice partials
  int* tdone;          // [kStages] units finished per stage in flight
  int* bcnt;           // [kStages][2] slices finished per tile
  float4* xf;          // [kMaxGroups] per-group activation factors
  float* yin;          // [7][kMaxOwnRows] tensor parallel: the peers' partial sums of this CTA's rows
};

__device__ __forceinline__ Smem carve_smem(uint8_t* base) {
  Smem s;
  s.stages = base;
  s.scratch = base + kStages * kStageBytes;
  s.xh = reinterpret_cast<__half*>(s.scratch);
  uint8_t* tail = s.scratch + kScratchBytes;
  s.full = reinterpret_cast<uint64_t*>(tail);
  s.empty = s.full + kStages;
  s.s_abort = reinterpret_cast<volatile int*>(tail + 128);
  s.landed = reinterpret_cast<volatile int*>(tail + 132);
  s.red = reinterpret_cast<float*>(tail + 256);
  s.misc = reinterpret_cast<int*>(tail + 384);
  s.hown = reinterpret_cast<float*>(tail + 512);
  s.qpart = reinterpret_cast<float*>(tail + 1024);
  s.tdone = reinterpret_cast<int*>(tail + 2048);
  s.bcnt = reinterpret_cast<int*>(tail + 2080);
  s.yin = reinterpret_cast<float*>(tail + 2176);
  s.xf = reinterpret_cast<float4*>(tail + 4096);
  return s;
}
static_assert(kMaxGroups * 16 + 4096 <= kTailBytes && 2 * kMaxOwnRows * 4 <= 512 && 2176 + 7 * kMaxOwnRows * 4 <= 4096, "tail layout");

// called by one thread before the CTA-wide barrier that opens the kernel
__device__ __forceinline__ void pipe_init(const Smem& sm) {
  for (int s = 0; s < kStages; s++) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); sm.tdone[s] = 0; }
  for (int i = 0; i < 2 * kStages; i++) sm.bcnt[i] = 0;
  *sm.s_abort = 0;
  *sm.landed = 0;
  mbar_fence_init();
}

// rows [r0, r1) of a phase that CTA b of G owns; `unit` rows stay together (the tile height of the matrix)
__device__ __forceinline__ void cta_rows(int rows, int unit, int b, int G, int& r0, int& r1) {
  const long long nu = (rows + unit - 1) / unit;
  r0 = min(rows, (int)((nu * b) / G) * unit);
  r1 = min(rows, (int)((nu * (b + 1)) / G) * unit);
}

// ------------------------------------------------------------------------------------------------ producer side
// `src` points at the tile that holds the first of `nrows` rows; `tile_rows` rows (whole tiles) travel per stage.
__device__ __forceinline__ bool produce_rows(Pipe& p, const uint8_t* src, int nrows, int tile_rows, int rt, int rec,
                                             const WaitCtl& wc, int layer) {
  for (int r = 0; r < nrows; r += tile_rows) {
    const int n = (min(tile_rows, nrows - r) + rt - 1) / rt * rt;             // the last tile may be partly padding
    const uint32_t bytes = (uint32_t)n * rec;
    const int s = p.it % kStages;
    const uint32_t ph = (p.it / kStages) & 1;
    if (!mbar_wait(&p.empty[s], ph ^ 1, wc, W_EMPTY, layer)) return false;   // p.it counts issued loads only
    mbar_expect_tx(&p.full[s], bytes);
    bulk_g2s(p.stages + (size_t)s * kStageBytes, src + (size_t)r * rec, bytes, &p.full[s]);
    p.it++;
    // Keep the memory system's queues short: with the whole ring in flight (27 MB over 148 SMs) every small
    // latency-critical access of the consumers (flags, tagged words) waits microseconds behind bulk weight traffic.
    // The same wait tells the consumers which loads have landed: a consumer may only wait for load i on a stage's
    // one-bit phase once load i - kStages is known to be complete.
    if (p.it > p.max_fly) {
      const uint32_t j = p.it - 1 - p.max_fly;
      if (!mbar_wait(&p.full[j % kStages], (j / kStages) & 1, wc, W_FULL, layer)) return false;
      *p.landed = (int)(j + 1);
    }
  }
  return true;
}

// Before the CTA may exit, every bulk copy it issued must have landed. In a clean run the consumers have already
// waited for all of them; after a failed wait the last (up to) kStages issued loads may still be in flight.
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
struct QueueState {
  float* qpart;
  int* tdone;
  int* bcnt;
};

// GEMV over this CTA's `nrows` rows of one phase (they start on a tile boundary). Warp w takes slice w % KS of tiles
// w / KS, w / KS + NL, ... in order. Every finished group of up to 4 rows is handed to `epi(row0_local, c, nvalid)` by
// the whole warp, lane r << 3 holding the total of row row0_local + r, so results leave the CTA as soon as they exist.
// A stage goes back to the producer when its last unit finishes (shared-memory counter); for sliced tiles the warp
// that finishes the last slice adds the partials in slice order and runs the epilogue.
template <class C, bool HZ, bool ROLL = false, class Epi>
__device__ __forceinline__ void consume_tiles(Pipe& p, int nrows, const XStage& x, const QueueState& q, int cw, int lane,
                                              const WaitCtl& wc, int layer, Epi epi, long long* dbg = nullptr) {
  constexpr int RT = C::RT, KS = C::KS, TPS = C::TPS;
  constexpr int NL = kConsumerWarps / KS;            // tile lanes; warps beyond NL * KS sit this phase out
  constexpr int TILE = C::tile(HZ);
  const int nt = (nrows + RT - 1) / RT;
  const int nst = (nt + TPS - 1) / TPS;
  if (cw < NL * KS) {
    const int slice = cw % KS;
    for (int tl = cw / KS; tl < nt; tl += NL) {
      const int st = tl / TPS, blk = tl % TPS;
      const uint32_t it = p.it + st;
      const int s = it % kStages;
      if (it >= (uint32_t)kStages) {                 // the stage's previous load must be complete before its phase bit is read
        bool ok = false;
        for (unsigned i = 0; i < wc.limit; i++) {
          if ((uint32_t)*p.landed > it - kStages) { ok = true; break; }
          if ((i & 63) == 63 && *wc.s_abort) break;
        }
        if (!ok) {
          if (*wc.s_abort == 0) report_fail(wc, W_LANDED, layer, (int)it, *p.landed);
          break;
        }
      }
      if (!mbar_wait(&p.full[s], (it / kStages) & 1, wc, W_FULL, layer)) break;
      if (dbg && cw == 0 && lane == 0 && tl == 0) dbg[13] = (long long)globaltimer_ns();
      const uint8_t* tile = p.stages + (size_t)s * kStageBytes + (size_t)blk * TILE;
      const int nvalid_tile = min(RT, nrows - tl * RT);
      float lo, hi;
      tile_dot<C, HZ, ROLL>(tile, slice, x, lane, lo, hi);
      if (dbg && cw == 0 && lane == 0 && tl == 0) dbg[14] = (long long)globaltimer_ns();
      if (KS == 1) {
        if (RT <= 4) {
          epi(tl * RT, __shfl_sync(0xffffffffu, lo, (lane >> 3) * 4), nvalid_tile);
        } else if (RT == 8) {
          epi(tl * RT, __shfl_sync(0xffffffffu, lo, (lane >> 3) * 4), min(4, nvalid_tile));
          epi(tl * RT + 4, __shfl_sync(0xffffffffu, lo, (4 + (lane >> 3)) * 4), min(4, nvalid_tile - 4));
        } else {
#pragma unroll
          for (int qd = 0; qd < 4; qd++) {
            const float v = qd < 2 ? lo : hi;
            epi(tl * RT + 4 * qd, __shfl_sync(0xffffffffu, v, (4 * (qd & 1) + (lane >> 3)) * 4), min(4, nvalid_tile - 4 * qd));
          }
        }
      } else {
        float* part = q.qpart + ((s * 2 + blk) * 4) * 4;         // [slice][row]
        if ((lane & 3) == 0 && (lane >> 2) < RT) part[slice * 4 + (lane >> 2)] = lo;
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          __threadfence_block();
          const int old = atomicAdd(q.bcnt + s * 2 + blk, 1);
          last = (old == KS - 1);
          if (last) q.bcnt[s * 2 + blk] = 0;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {                                              // every slice of this tile is in: combine, epilogue
          __threadfence_block();
          float c = 0.f;
#pragma unroll
          for (int sl = 0; sl < KS; sl++) c += part[sl * 4 + (lane >> 3)];
          epi(tl * RT, c, nvalid_tile);
        }
      }
      __syncwarp();
      if (lane == 0) {                                           // the stage's last unit hands the slot back
        const int units = min(TPS, nt - st * TPS) * KS;
        const int old = atomicAdd(q.tdone + s, 1);
        if (old == units - 1) {
          q.tdone[s] = 0;
          mbar_arrive(&p.empty[s]);
        }
      }
    }
  }
  p.it += nst;
}

// ------------------------------------------------------------------------------------------------ stand-alone GEMV
struct GemvParams {
  const uint8_t* w;        // streaming layout
  const uint16_t* x;       // bf16 [K]
  float* y;                // f32 [rows], original row order
  DevStatus* status;
  int32_t rows, order, order_arg, order_rows;
  unsigned spin_limit;
};

// every consumer thread calls; ends with a consumer-wide barrier
template <int K>
__device__ __forceinline__ void stage_x_global(const uint16_t* gx, const Smem& sm, int tid_c) {
  const int warp = tid_c >> 5, lane = tid_c & 31;
  for (int grp = warp; grp < K / 128; grp += kConsumerWarps) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(gx + grp * 128) + lane);
    stage_group_fp16(v.x, v.y, sm.xh + grp * 128, sm.xf + grp, lane);
  }
  named_bar_sync(kBarConsumers, kConsumerThreads);
}

template <class C, bool HZ>
__global__ void __launch_bounds__(kThreads, 1) gemv_stream(const GemvParams P) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Smem sm = carve_smem(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) pipe_init(sm);
  __syncthreads();
  WaitCtl wc{P.status, sm.s_abort, P.spin_limit};
  Pipe pipe{sm.stages, sm.full, sm.empty, sm.landed, 0u, 4u};
  constexpr int rec = rec_bytes_of(C::K, HZ);
  int r0, r1;
  cta_rows(P.rows, C::RT, blockIdx.x, gridDim.x, r0, r1);
  if (warp == kConsumerWarps) {
    if (lane == 0) {
      produce_rows(pipe, P.w + (size_t)r0 * rec, r1 - r0, C::TILE_ROWS, C::RT, rec, wc, 0);
      producer_drain(pipe, wc);
    }
  } else {
    stage_x_global<C::K>(P.x, sm, tid);
    const XStage xs{sm.xh, sm.xf};
    const QueueState qs{sm.qpart, sm.tdone, sm.bcnt};
    consume_tiles<C, HZ>(pipe, r1 - r0, xs, qs, warp, lane, wc, 0, [&](int row0, float c, int nvalid) {
      if ((lane & 7) == 0 && (lane >> 3) < nvalid)
        P.y[perm_row(r0 + row0 + (lane >> 3), P.order, P.order_arg, P.order_rows)] = c;
    });
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------------ layout kernels
// Caller layout -> tiles. One CTA per tile; blockIdx.y = layer (the matrices of all layers are stacked; every layer
// starts on a tile boundary and repeats the row order). Rows beyond `rows` are padding: nibble 8 (value 0), scale 0.
template <int K>
__global__ void repack_tiles(const uint32_t* q, const uint16_t* sc, const uint16_t* zr, int rows, int order, int order_arg,
                             int order_rows, uint8_t* out) {
  using C = TCfg<K>;
  constexpr int RT = C::RT;
  const bool hz = zr != nullptr;
  const int T = blockIdx.x, tiles = (rows + RT - 1) / RT;
  uint8_t* tile = out + ((size_t)blockIdx.y * tiles + T) * tile_bytes(K, hz);
  __shared__ int src_row[16];
  if (threadIdx.x < RT) {
    const int j = T * RT + threadIdx.x;
    src_row[threadIdx.x] = j < rows ? (int)blockIdx.y * rows + perm_row(j, order, order_arg, order_rows) : -1;
  }
  __syncthreads();
  auto nib = [&](int r, int col) -> uint32_t {
    const int row = src_row[r];
    if (row < 0) return 8u;
    return (__ldg(q + (size_t)row * (K / 8) + (col >> 3)) >> (4 * (col & 7))) & 15u;
  };
  for (int wi = threadIdx.x; wi < C::NIB / 4; wi += blockDim.x) {
    const int i = wi & 3, lane = (wi >> 2) & 31, bq = wi >> 7;
    const int s = 4 * bq + i, g = lane >> 2, t = lane & 3;
    const int rl = g % RT, rh = (g + 8) % RT, jl = g / RT, jh = (g + 8) / RT;
    const int cl = jl * (K / C::NJ) + 16 * local_step(s, jl) + 2 * t, ch = jh * (K / C::NJ) + 16 * local_step(s, jh) + 2 * t;
    reinterpret_cast<uint32_t*>(tile)[wi] = nib(rl, cl) | nib(rh, ch) << 4 | nib(rl, cl + 8) << 8 | nib(rh, ch + 8) << 12 |
                                            nib(rl, cl + 1) << 16 | nib(rh, ch + 1) << 20 | nib(rl, cl + 9) << 24 |
                                            nib(rh, ch + 9) << 28;
  }
  uint16_t* meta = reinterpret_cast<uint16_t*>(tile + C::NIB);
  for (int i = threadIdx.x; i < RT * C::G; i += blockDim.x) {
    const int grp = i / RT, row = src_row[i % RT];
    meta[i] = row >= 0 ? sc[(size_t)row * C::G + grp] : 0;
    if (hz) meta[RT * C::G + i] = row >= 0 ? zr[(size_t)row * C::G + grp] : 0;
  }
}

// tiles -> f32 [rows][K] in the caller's row order: (nib - 8) * scale (+ zero). One CTA per stream row.
template <int K>
__global__ void dequant_tiles(const uint8_t* in, int rows, int has_zeros, int order, int order_arg, int order_rows, float* out) {
  using C = TCfg<K>;
  constexpr int RT = C::RT;
  const int j = blockIdx.x, T = j / RT, r = j % RT;
  const int dstrow = perm_row(j, order, order_arg, order_rows);
  const uint8_t* tile = in + (size_t)T * tile_bytes(K, has_zeros);
  const uint16_t* meta = reinterpret_cast<const uint16_t*>(tile + C::NIB);
  for (int c = threadIdx.x; c < K; c += blockDim.x) {
    const int jr = c / (K / C::NJ), cl = c % (K / C::NJ), sp = cl >> 4, c16 = cl & 15;
    const int s = (sp & ~3) | ((sp - jr) & 3);                 // the MMA step whose local step for range jr is sp
    const int mrow = r + RT * jr;                              // MMA row
    const int g = mrow & 7, hi = mrow >> 3;
    const int t = (c16 & 7) >> 1, odd = c16 & 1, second = c16 >> 3;
    const int lane = 4 * g + t;
    const uint32_t w = reinterpret_cast<const uint32_t*>(tile)[(((s >> 2) * 32 + lane) << 2) + (s & 3)];
    const float nibv = (float)((w >> (4 * (odd * 4 + second * 2 + hi))) & 0xF) - 8.0f;
    const int grp = c >> 7;
    float v = nibv * bf2f(meta[grp * RT + r]);
    if (has_zeros) v = v + bf2f(meta[RT * C::G + grp * RT + r]);
    out[(size_t)dstrow * K + c] = v;
  }
}

}  // namespace fb
