/*
 * flint_b200 -- C ABI of the B200 (sm_100a) batch-1 int4 decode engine.
 *
 * Plain pointers and sizes only: every `d_*` argument is a device pointer owned by the caller, `stream` is a
 * cudaStream_t passed as void* (NULL = default stream). Every entry point returns an int status, 0 = FB_OK.
 * Launches are asynchronous on `stream`; FB_ERR_TIMEOUT and friends are reported by fb_last_status() after the
 * stream has been synchronised. Nothing here falls back to the CPU.
 *
 * Each declaration names the reference interface it replaces (paths inside the reference project).
 */
#ifndef FLINT_B200_H_
#define FLINT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FB_OK = 0,
  FB_ERR_ARG = 1,          /* NULL pointer, misaligned pointer, bad size */
  FB_ERR_SHAPE = 2,        /* model shape this build has no kernel for */
  FB_ERR_CUDA = 3,         /* a CUDA runtime call failed; fb_last_status() carries the cudaError_t */
  FB_ERR_STATE = 4,        /* weights / KV cache not bound yet, or context poisoned by an earlier device error */
  FB_ERR_TIMEOUT = 5,      /* a bounded device-side wait ran out (copy barrier, arrival flag, tagged word, peer word) */
  FB_ERR_RANGE = 6         /* pos / M / token outside the bound cache or vocabulary */
};

/* Device facts the host side sizes things by. Replaces decode_occupancy()/verify_occupancy()
 * (reference: kernels/megakernel_decode.cu:239-245, kernels/verify_mega.cu:285-293). */
typedef struct fb_caps {
  int32_t device, sm_count, cc_major, cc_minor;
  int32_t smem_per_block_optin, l2_bytes, cooperative_launch, regs_decode_kernel;
  int64_t total_mem_bytes;
} fb_caps;
int fb_query(int device, fb_caps* out);

/* Model shape and scalar multipliers: the module globals of the reference front-end
 * (reference: chat.py:19-21) and the trailing scalar arguments of decode_mega_launch
 * (reference: kernels/megakernel_decode.cu:204-211). ffn must be a multiple of 128 (pad with zero weights). */
typedef struct fb_model_desc {
  int32_t n_layer, dim, n_head, n_kv_head, head_dim, ffn, vocab;
  int32_t has_zeros;       /* 0: (nib-8)*s  (reference: chat.py:23-30); 1: (nib-8)*s+z (reference: engine/quantize.py:138-155) */
  float rms_eps, rope_base, attn_scale, resid_mult, emb_mult, logits_scaling;
} fb_model_desc;

/* The 13 weight tensors of the reference boundary in the reference's own layout
 * (reference: chat.py:32-52, kernels/megakernel_decode.cu:204-208): q int32 [L, OUT, IN/8],
 * s (and z) bf16 [L, OUT, IN/128]; lm_* have no layer dimension; norms bf16; embed bf16 [vocab, dim].
 * *_z may be NULL when has_zeros == 0. */
typedef struct fb_weight_ptrs {
  const void *qkv_q, *qkv_s, *qkv_z;
  const void *o_q, *o_s, *o_z;
  const void *gu_q, *gu_s, *gu_z;
  const void *d_q, *d_s, *d_z;
  const void *lm_q, *lm_s, *lm_z;
  const void *n1, *n2, *nf;
  const void *embed;
} fb_weight_ptrs;

typedef struct fb_ctx fb_ctx;

typedef struct fb_status {
  int32_t code;            /* FB_* */
  int32_t cuda_error;      /* last cudaError_t seen by the host side, 0 if none */
  int32_t where;           /* device side: phase id that gave up */
  int32_t layer, block, expected, seen;
} fb_status;

/* Context: scratch, barrier words and status buffer on `device`. Replaces the per-call torch::empty scratch
 * allocations and occupancy queries of the reference launcher (reference: kernels/megakernel_decode.cu:213-223). */
int fb_ctx_create(const fb_model_desc* desc, int device, fb_ctx** out);
int fb_ctx_destroy(fb_ctx* ctx);

/* Tensor parallelism over 2/4/8 GPUs of one box, one process per GPU (no counterpart in the reference: its
 * generate.py imports a `tp` module that the repository does not contain, reference: engine/generate.py:238-241).
 * `desc` describes THIS RANK'S slice: n_head / n_kv_head = local heads, ffn = local FFN columns, vocab = local
 * vocabulary rows, dim = the full model width. vocab_base = first vocabulary row of this rank. Every rank exports the
 * IPC handle of its inbox, the host side exchanges the handles (any transport), and every rank connects to all of
 * them before the first fb_decode. The partial sums of the K-sharded O and down projections and the arg-max
 * candidates then travel by peer stores over NVLink inside the kernel; no NCCL launch is involved.
 *   fb_tp_export : 64-byte cudaIpcMemHandle_t of this rank's inbox
 *   fb_tp_connect: handles = n * 64 bytes, entry p = rank p's handle (the own entry is ignored)
 *   fb_tp_connect_local: the single-process form (one host process that drives several GPUs, or several ranks of a
 *                  test on one GPU): ranks[p] = rank p's context of THIS process; peer access is enabled between the
 *                  devices, no IPC handle is involved. Every rank's context must outlive the others' launches. */
int fb_ctx_create_tp(const fb_model_desc* desc, int device, int32_t tp_rank, int32_t tp_size, int32_t vocab_base,
                     fb_ctx** out);
int fb_tp_export(fb_ctx* ctx, void* handle_out64);
int fb_tp_connect(fb_ctx* ctx, const void* handles, int32_t n);
int fb_tp_connect_local(fb_ctx* ctx, fb_ctx* const* ranks, int32_t n);
int fb_last_status(fb_ctx* ctx, fb_status* out);

/* Re-lays the caller's int4 tensors out into the context's streaming layout (one pass on the GPU, once).
 * The caller's tensors are not referenced afterwards, except n1/n2/nf/embed which must stay alive.
 * Replaces load_packed's stacked tensors as kernel operands (reference: chat.py:32-52). */
int fb_bind_weights(fb_ctx* ctx, const fb_weight_ptrs* w, void* stream);

/* Caller-owned KV cache, bf16 [n_layer, max_seq, n_kv_head, head_dim], dimension 1 = position
 * (reference: chat.py:68-69; the cache is indexed by position from Python in spec_tree.py:126-128). */
int fb_bind_kv(fb_ctx* ctx, void* d_k, void* d_v, int32_t max_seq);

/* One decode step in one cooperative launch: embedding (or a caller-supplied residual), all layers, final norm,
 * LM head, argmax. Replaces decode_mega_launch (reference: kernels/megakernel_decode.cu:204-237) plus the
 * host-side embedding lookup and argmax around it (reference: chat.py:71-77).
 *   token     : used when d_token == NULL and d_h == NULL
 *   d_token   : device int32, read by the kernel (lets step t+1 consume step t's d_next without a host sync)
 *   d_h       : bf16 [dim], the already multiplied embedding, as the reference boundary takes it; it receives the
 *               final residual stream (the reference clobbers its h argument too); NULL to use the token
 *   d_logits  : f32 [vocab] or NULL
 *   d_next    : int32 argmax (first index of the maximum) or NULL */
int fb_decode(fb_ctx* ctx, int32_t token, const int32_t* d_token, void* d_h, int32_t pos, float* d_logits,
              int32_t* d_next, void* stream);

/* M-token tree verification: every weight row is read once for all M candidate tokens. Replaces verify_mega_launch
 * (reference: kernels/verify_mega.cu:246-283) with its tree semantics (reference: kernels/verify_mega.cu:143,153-158,169):
 * token m is written to cache slot pos+m, rotated at position pos+depth[m], and sees every slot < pos plus the new
 * slots j with amask[m*M + j] != 0. M is 1..64 (any value, padded internally to 16/32/64); other M is FB_ERR_RANGE.
 *   d_tokens : device int32[M], or NULL when d_h is given
 *   d_h      : bf16 [M, dim] already multiplied embeddings (the reference's argument), or NULL
 *   d_logits : f32 [M, vocab] or NULL;   d_feat : bf16 [M, dim] post-final-norm feature (the draft head's input) or NULL */
int fb_verify(fb_ctx* ctx, const int32_t* d_tokens, const void* d_h, const int32_t* d_depth, const uint8_t* d_amask,
              int32_t M, int32_t pos, float* d_logits, void* d_feat, void* stream);

/* Tree KV surgery after acceptance: cache row dst[i] <- row src[i] in every layer, in order, for K and V.
 * src/dst are HOST arrays. Replaces `kc[:, dst] = kc[:, src]` (reference: spec_tree.py:126-128). */
int fb_kv_move(fb_ctx* ctx, const int32_t* src, const int32_t* dst, int32_t n, void* stream);

/* On-device KV compaction after a tree acceptance: the device-side form of fb_kv_move. d_accept is fb_accept_tree's
 * output (device int32: [0] = nodes on the accepted path, [2 + i] = node index of path step i); cache row pos + i
 * receives row pos + path[i] for i = 1 .. len-1, K and V, every layer. No host copy of the path is needed. */
int fb_kv_compact(fb_ctx* ctx, const int32_t* d_accept, int32_t pos, void* stream);

/* Token choice on the device, no host sync (replaces the host-side pick() / sample(), reference: chat.py:76-81,
 * engine/generate.py:37-55). One token per row of d_logits (f32, `vocab` entries, rows `row_stride` elements apart; a
 * stride of 0 draws every row from the same vector).
 *   temperature <= 0 : arg-max, first index of the maximum
 *   temperature  > 0 : a sample of softmax(logits / temperature) restricted, when 0 < top_k < vocab, to the entries
 *                      >= the top_k-th largest (ties kept, as the reference's masking does)
 *   seed, counter    : row r uses the random stream (seed, counter + r): equal arguments give equal tokens; advance
 *                      `counter` by `rows` per call */
int fb_sample(const float* d_logits, int32_t vocab, int32_t rows, int64_t row_stride, float temperature, int32_t top_k,
              uint64_t seed, uint64_t counter, int32_t* d_out, void* stream);

/* Acceptance walks on the device (replace the host loops, reference: spec_mega.py:106-113, spec_tree.py:108-118).
 *   fb_accept_chain: d_target int32[k+1] = the target's greedy token at every candidate position, d_draft int32[k];
 *                    d_out[0] = accepted count a (longest agreeing prefix), d_out[1] = d_target[a]
 *   fb_accept_tree : d_cand / d_parent / d_target int32[m] (node 0 = root, parent[0] = -1, parents before children);
 *                    d_out int32[2 + m]: [0] = nodes on the accepted path incl. the root, [1] = the target's token at
 *                    its last node, [2 + i] = node index of path step i */
int fb_accept_chain(const int32_t* d_target, const int32_t* d_draft, int32_t k, int32_t* d_out, void* stream);
int fb_accept_tree(const int32_t* d_cand, const int32_t* d_parent, const int32_t* d_target, int32_t m, int32_t* d_out,
                   void* stream);

/* EAGLE draft head inside the library: one decoder block over [target feature ; token embedding] with bf16 weights in
 * torch.nn.Linear layout, the computation of the reference's DraftHead.forward (reference: train/draft_model.py:24-64)
 * and of its token head (reference: spec_mega.py:43-44), rounding to bf16 where bf16 PyTorch modules round.
 * fuse * dim is the width of the (fused) feature; n_kv_head == n_head is the reference's multi-head form.
 *   fb_draft_forward: T rows. d_feat bf16 [T, fuse*dim]; the token embedding of row t is d_emb[t] (bf16 [T, dim]) or,
 *                     when d_emb is NULL, row d_tokens[t] of the bound embedding table (a negative id = zeros), read on
 *                     the device; d_positions int32[T] rotation positions; d_slots int32[T] = cache slot of every row
 *                     (its k/v are written there and row t attends slots 0..d_slots[t]) or NULL (slot t: plain causal
 *                     attention over the T rows); d_out bf16 [T, fuse*dim] = predicted next features
 *   fb_draft_head   : n <= 16 feature rows -> the top_b <= 16 tokens of each (d_tokens int32 [n, top_b], best first) and
 *                     optionally their logits (d_scores f32 [n, top_b]); logits are rounded to bf16 as the reference's
 *                     bf16 head computes them */
typedef struct fb_draft_desc {
  int32_t dim, n_head, n_kv_head, inter, fuse, vocab;
  int32_t max_roll;        /* cache slots (window + rollout depth) */
  int32_t max_tokens;      /* most rows one fb_draft_forward call takes */
  float rope_base, rms_eps, logits_scaling;
} fb_draft_desc;
typedef struct fb_draft_weights {
  const void *merge, *n1, *n2, *q, *k, *v, *o, *gate, *up, *down, *fout;   /* the draft head's own tensors */
  const void *nf, *embed;                                                  /* the target's final norm and embedding table */
} fb_draft_weights;
typedef struct fb_draft fb_draft;
int fb_draft_create(const fb_draft_desc* desc, int device, fb_draft** out);
int fb_draft_destroy(fb_draft* draft);
int fb_draft_bind(fb_draft* draft, const fb_draft_weights* w);
int fb_draft_forward(fb_draft* draft, const void* d_feat, const void* d_emb, const int32_t* d_tokens,
                     const int32_t* d_positions, const int32_t* d_slots, int32_t T, void* d_out, void* stream);
int fb_draft_head(fb_draft* draft, const void* d_feat_rows, int32_t n, int32_t top_b, int32_t* d_tokens, float* d_scores,
                  void* stream);

/* Stand-alone slices of the same path, on the streaming layout (unit-test granularity; they replace the
 * reference's GEMV family, reference: kernels/int4_gemv.cu:384-424).
 *   fb_stream_bytes : bytes of the streaming layout for one [rows, k] matrix
 *   fb_repack       : caller layout -> streaming layout (order: 0 plain, 1 RoPE pair interleave with head_dim,
 *                     2 gate/up interleave: stream rows (2i, 2i+1) hold source rows (i, i+order_arg))
 *   fb_dequant      : streaming layout -> f32 [rows, k] in ORIGINAL row order: (nib-8)*s+z, bit for bit
 *   fb_gemv         : y f32 [rows] (original row order) = W x, x bf16 [k]; d_status is a zeroed 32-byte device
 *                     buffer (int32[8]) whose first word becomes FB_ERR_TIMEOUT if a bounded wait ran out */
size_t fb_stream_bytes(int32_t rows, int32_t k, int32_t has_zeros);
int fb_repack(const void* d_q, const void* d_s, const void* d_z, int32_t rows, int32_t k, int32_t order,
              int32_t order_arg, int32_t order_rows, void* d_stream_out, void* stream);
int fb_dequant(const void* d_stream_in, int32_t rows, int32_t k, int32_t has_zeros, int32_t order, int32_t order_arg,
               int32_t order_rows, float* d_out, void* stream);
int fb_gemv(const void* d_stream_in, int32_t rows, int32_t k, int32_t has_zeros, int32_t order, int32_t order_arg,
            int32_t order_rows, const void* d_x, float* d_y, void* d_status, void* stream);

/* The same GEMV for callers that are not allowed to allocate device memory. This entry point has no counterpart in the
 * reference. Who needs it: a host that hands this library a fixed device arena and forbids any further cudaMalloc
 * (inference servers that pre-reserve all of HBM), and code that runs where an allocation would be an error or a stall,
 * e.g. while a stream is being captured or inside a latency-critical loop. fb_gemv needs a caller-allocated copy of the
 * matrix in the streaming layout; here that copy goes into ONE array built into the library (9 MiB, 256-byte aligned,
 * held by every GPU that loads the library until the process exits), so nothing is allocated or freed, here or in any
 * library this calls.
 *   inputs   : d_q int32 [rows, k/8], d_s bf16 [rows, k/128], d_z bf16 [rows, k/128] or NULL (caller layout), d_x bf16 [k]
 *   outputs  : d_y f32 [rows]; d_status int32[8] (cleared by this call; word 0 becomes FB_ERR_TIMEOUT if a wait ran out)
 *   limit    : fb_stream_bytes(rows, k, zeros) <= 9 MiB, else FB_ERR_RANGE (nothing is launched);
 *              k must be one of the widths fb_gemv supports, else FB_ERR_SHAPE
 *   set-up   : the first call on a device resolves the array's device address; make that first call before any stream
 *              capture begins on that device
 *   sharing  : every call uses the same array and leaves its contents behind; two calls that overlap on the GPU
 *              (different streams, or another thread) race on it — order them on one stream */
int fb_gemv_static(const void* d_q, const void* d_s, const void* d_z, int32_t rows, int32_t k, const void* d_x, float* d_y,
                   void* d_status, void* stream);

/* Tuning / test knobs (no reference counterpart: the reference has no bounded waits and a fixed split).
 *   what 0: iteration limit of every device-side wait (default 4000000); a tiny value makes a launch give up
 *           with FB_ERR_TIMEOUT, which is how the time-out path is tested without hanging a GPU
 *   what 1: force the number of attention chunks per kv head (0 = choose from the cached length)
 *   what 2: value = device pointer to int64[sm_count * n_layer * 16] (0 = off): %globaltimer stamps (ns) of every CTA
 *           at the phase boundaries of every layer, the run-time replacement of the reference's -DNOSYNC/-DNOATTN diagnostic
 *           builds (reference: kernels/megakernel_decode.cu:15-24)
 *   what 4: bulk weight copies one CTA keeps in flight at once (1..4, default 4)
 *   what 5: 1 = consumers poll the tagged activation words directly; 0 = they wait for the producers' arrival flags first
 *   what 8: decode variant whose attention reads K/V through the weight ring: 0 = always where the shape has it (default),
 *           1 = always (shapes built with it: tiny, 3B-class, 8B-class on one GPU), 2 = never
 *   what 7: GEMMs of fb_verify: 0 = chosen by tree size (default: more than 16 tokens run the tcgen05 kernels with
 *           accumulators in tensor memory; smaller trees, latency-bound, run the warp-level mma.sync kernels: up to
 *           8 tokens on fp16-subnormal operands, 9 to 16 on bf16 operands), 1 = warp-level on bf16 operands, 2 = tcgen05,
 *           3 = tcgen05 with four GEMMs chained per launch, 4 = warp-level on fp16-subnormal operands (the decode
 *           kernel's arithmetic; symmetric weights, up to 26 tokens, other cases fall back to 1) */
int fb_set_option(fb_ctx* ctx, int32_t what, int64_t value);

#ifdef __cplusplus
}
#endif
#endif /* FLINT_B200_H_ */
