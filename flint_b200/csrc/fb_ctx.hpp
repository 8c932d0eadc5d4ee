// The context object behind the C ABI's opaque `fb_ctx`, shared by the translation units of the library.
#pragma once
#include <cuda.h>
#include <stdint.h>

#include "../../include/flint_b200.h"

namespace fb { struct DevStatus; }
using fb::DevStatus;

struct fb_ctx {
  fb_model_desc d;
  int device, sm_count, kernel_id, rgqa;
  uint8_t *w_qkv, *w_o, *w_gu, *w_d, *w_lm;
  const void *n1, *n2, *nf, *embed;
  float* invf;
  DevStatus* status;
  void *kc, *vc;
  int max_seq, maxchunks;
  unsigned spin_limit;
  bool weights_bound;
  int last_cuda_error;
  int force_chunks;
  long long* prof;
  uint64_t *h_ll, *q_ll, *k_ll, *v_ll, *ao_ll, *act_ll, *cand_ll, *part_ll;   // tagged vectors of the data-flow kernel
  uint32_t* flags;                                                  // [3][256] arrival flags: h, act, ao
  unsigned tag_base;
  int tp_size, tp_rank, vocab_base, ko, ao_off;                     // tensor parallelism (1 GPU: tp_size 1, ko = dim)
  uint64_t* inbox;                                                  // [2][tp][dim] partial words + [tp][2] candidates
  uint64_t* peer_inbox[8];
  bool peers_open[8];
  uint16_t *vh, *vxn, *vq, *vao, *vact;                             // verify activations, 64 token rows each
  float* vpart;                                                     // verify attention: per-span partials
  uint8_t *t_qkv, *t_o, *t_gu, *t_d, *t_lm;                          // verify: the matrices in the tensor-core (TC) layout
  uint8_t *s_qkv, *s_o, *s_gu, *s_d, *s_lm;                          // verify: the matrices in the R32 layout (small trees); NULL = not built
  float* vsplit;                                                    // verify: split-K partial sums
  unsigned* vcount;                                                 // verify: arrivals per (row block, row quadrant)
  float* vssq;                                                      // verify chain: partial sums of squares, 2 x [256][64]
  unsigned* vgbar;                                                  // verify chain: grid arrival counters per launch and phase
  void* vrope;                                                      // verify: (cos, sin) per (token, rotation pair)
  int verify_path;                                                  // 0: by tree size, 1: warp-level MMA GEMMs (bf16), 2: tcgen05 GEMMs, 3: tcgen05 GEMM chains, 4: warp-level MMA GEMMs on fp16 subnormals
  int max_fly, poll_words;
  CUtensorMap kmap, vmap;                                           // the caches as tensors for the long-cache variant
  bool kv_maps;
  int long_kv;                                                      // 0: long-cache decode variant by cached length, 1: always (where built), 2: never
};
