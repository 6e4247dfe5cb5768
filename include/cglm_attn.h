/*
 * cglm_attn.h -- C ABI of the B200 (sm_100a) attention KV-cache path.
 *
 * The library replaces what chatglm::BasicAttention::forward records between its two Linears
 * (li-plus/chatglm.cpp, chatglm.cpp:636-717): qkv split views, RoPE on q and k, the f16 append of K
 * into k_cache [kv_heads, max_len, head_dim] and of V into the transposed v_cache
 * [kv_heads, head_dim, max_len] at n_past, and scaled-dot-product attention over the cache.
 *
 * Conventions
 *  - every entry point returns CGLM_OK (0) or a negative CGLM_ERR_*; nothing throws, aborts or waits
 *    without a bound; work is enqueued on the given CUDA stream and the host never synchronises
 *    unless the function says so;
 *  - there is no CPU fallback: without a usable CUDA device every compute entry point fails;
 *  - pointers named *_host are host memory, all others are device memory;
 *  - strides are in elements, not bytes.
 */
#ifndef CGLM_ATTN_H
#define CGLM_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    CGLM_OK = 0,
    CGLM_ERR_INVALID_ARG = -1,   /* bad shape, null pointer, n_past + qlen beyond the cache ... */
    CGLM_ERR_CUDA = -2,          /* a CUDA runtime/driver call failed; see cglm_last_error_string */
    CGLM_ERR_WORKSPACE = -3,     /* workspace missing, too small or not initialised */
    CGLM_ERR_UNSUPPORTED = -4,   /* shape outside what the kernels cover (head_dim > 256, ...) */
    CGLM_ERR_TIMEOUT = -5,       /* a bounded device-side wait ran out; results of that call are invalid */
    CGLM_ERR_NO_DEVICE = -6      /* no CUDA device / wrong architecture */
};

/* values of chatglm::RopeType (chatglm.h:93-99) */
enum {
    CGLM_ROPE_GPTJ = 0,       /* full head, adjacent pairs      (apply_rotary_emb_basic, chatglm.cpp:523-537) */
    CGLM_ROPE_NEOX = 2,       /* full head, split-half pairs    (apply_rotary_emb_basic) */
    CGLM_ROPE_CHATGLM = 4,    /* 2-D: position / block position (apply_rotary_emb_glm,  chatglm.cpp:539-574) */
    CGLM_ROPE_CHATGLM2 = 8,   /* first half of the head, adjacent pairs (apply_rotary_emb_glm2, chatglm.cpp:576-601) */
    CGLM_ROPE_DISABLED = 10000
};

/* values of chatglm::AttentionMaskType (chatglm.h:101-104) */
enum {
    CGLM_MASK_CAUSAL = 0,     /* ggml_diag_mask_inf at n_past == 0 (chatglm.cpp:696-697) */
    CGLM_MASK_CHATGLM = 1     /* prefix-bidirectional: scores[:, :-1, -1] = -inf at n_past == 0 (chatglm.cpp:1126-1140) */
};

/* What the BasicAttention constructor fixes per model (chatglm.h:443-455). */
typedef struct cglm_attn_desc {
    int n_head;        /* num_attention_heads */
    int n_kv_head;     /* num_key_value_heads */
    int head_dim;      /* hidden_size / num_attention_heads */
    int max_len;       /* cache capacity in tokens = max_length + num_virtual_tokens */
    int n_virtual;     /* num_virtual_tokens (P-Tuning v2 prefix held in cache slots [0, n_virtual)) */
    int rope_type;     /* CGLM_ROPE_* */
    float rope_theta;
    int mask_type;     /* CGLM_MASK_* */
} cglm_attn_desc;

/*
 * KV arena: one device allocation holding the k_cache / v_cache pairs ("slots") of every layer and
 * every sequence, the counterpart of ModelContext::ctx_kv + buf_kv (chatglm.h:337,345,627-628).
 * Slot s holds k_cache f16 [n_kv_head][max_len][head_dim] and v_cache f16 [n_kv_head][head_dim][max_len],
 * exactly the two tensors BasicAttention owns (chatglm.h:452-455,470-471).  All K slabs are contiguous,
 * then all V slabs, so that two TMA tensor maps cover the whole arena.
 */
typedef struct cglm_kv_arena cglm_kv_arena;

/* Allocates and zero-fills the arena on the current CUDA device.  Synchronous. */
int cglm_kv_arena_create(const cglm_attn_desc *desc, int n_slots, cglm_kv_arena **out);
/* The same object over caches the CALLER owns, for a host that already has its kv buffer (the reference allocates one
 * for all layers, chatglm.h:627-628) and cannot move it: k_base = f16 [n_slots][n_kv_head][max_len][head_dim], every
 * slot's k_cache back to back; v_base = f16 [n_slots][n_kv_head][head_dim][max_len], every slot's v_cache back to back
 * (in ggml terms: create all k_cache tensors, then all v_cache tensors, before ggml_backend_alloc_ctx_tensors).  Both
 * device memory of the current device, 128-byte aligned; nothing is zero-filled, copied or freed by the library.
 * angle_table: optional device memory of cglm_kv_angle_table_bytes(desc) bytes (128-byte aligned) that the library
 * fills once with the (cos, sin) of every cache position; NULL makes the kernels evaluate the angles on the fly
 * (same values, a few microseconds more per decode launch).  cglm_kv_arena_destroy releases only the handle. */
int cglm_kv_arena_adopt(const cglm_attn_desc *desc, int n_slots, void *k_base, void *v_base, void *angle_table,
                        cglm_kv_arena **out);
size_t cglm_kv_angle_table_bytes(const cglm_attn_desc *desc);
int cglm_kv_arena_destroy(cglm_kv_arena *arena);
/* Device pointers of one slot's tensors (the public k_cache / v_cache members, chatglm.h:470-471). */
void *cglm_kv_arena_k_cache(const cglm_kv_arena *arena, int slot);
void *cglm_kv_arena_v_cache(const cglm_kv_arena *arena, int slot);
int cglm_kv_arena_n_slots(const cglm_kv_arena *arena);
const cglm_attn_desc *cglm_kv_arena_desc(const cglm_kv_arena *arena);
/* Tokens between two rows of a cache as laid out: k_cache is [n_kv_head][pitch][head_dim], v_cache
 * [n_kv_head][head_dim][pitch], of which the first max_len tokens are used.  pitch = max_len for adopted caches; an arena
 * of the library's own rounds it up to a multiple of 8 at head_dim 128 (TMA wants 16-byte row pitches), so that a model
 * whose max_length + num_virtual_tokens is not a multiple of 8 (P-Tuning v2) keeps the fused kernels. */
int cglm_kv_arena_pitch(const cglm_kv_arena *arena);
/* Bytes of one slot (k_cache + v_cache). */
size_t cglm_kv_slot_bytes(const cglm_attn_desc *desc);
/* Whole-slot copies between host and device, the counterpart of ggml_backend_tensor_set/get on the cache
 * tensors (e.g. chatglm.h:588).  k_host: f16 [n_kv_head][max_len][head_dim]; v_host: f16
 * [n_kv_head][head_dim][max_len]; either may be NULL.  to_device != 0 uploads.  Asynchronous on cuda_stream. */
int cglm_kv_slot_copy(cglm_kv_arena *arena, int slot, void *k_host, void *v_host, int to_device,
                      void *cuda_stream);

/*
 * One BasicAttention::forward call for one sequence (chatglm.cpp:620-721 minus the two Linears).
 * q/k/v point into the fused qkv activation; the (token, head) strides express both layouts of
 * chatglm.cpp:636-653 without a copy:
 *   blocked     (ChatGLM2/3/4): q = qkv, k = qkv + H*D, v = qkv + (H+G)*D, tok_stride = (H+2G)*D, head_stride = D
 *   interleaved (ChatGLM-6B v1): q = qkv, k = qkv + D,  v = qkv + 2*D,     tok_stride = 3*H*D,    head_stride = 3*D
 */
typedef struct cglm_attn_seq {
    const float *q, *k, *v;           /* f32 [qlen][heads][head_dim] through the strides below (f16 data behind the
                                         same pointers with CGLM_SEQ_QKV_F16; strides stay in elements) */
    long long q_tok_stride, q_head_stride;
    long long kv_tok_stride, kv_head_stride;
    int slot;                         /* which cache pair of the arena */
    int qlen;                         /* tokens in this call; masks apply only at n_past == 0 (chatglm.cpp:689) */
    int n_past;
    int n_ctx;                        /* prompt length; only CGLM_ROPE_CHATGLM derives ids from it (chatglm.cpp:1147-1151) */
    const int *position_ids;          /* optional [qlen] (or [2*qlen] for CGLM_ROPE_CHATGLM); NULL: derived from n_past, n_ctx */
    float *out;                       /* context_layer f32 [qlen][n_head*head_dim] (chatglm.cpp:716-717); 16-byte aligned
                                         (f16, 8-byte aligned, with CGLM_SEQ_OUT_F16) */
    float *q_roped;                   /* optional f32 [qlen][n_head][head_dim]: q after RoPE, before the 1/sqrt(d) scale */
    float *k_roped;                   /* optional f32 [qlen][n_kv_head][head_dim]: k after RoPE (the reference ropes in place) */
    /* split-KV use only (zero otherwise) */
    int kv_local;                     /* >0: tokens of this sequence present in this arena slot before the call */
    int flags;                        /* CGLM_SEQ_* */
    float *partial;                   /* with CGLM_SEQ_PARTIAL: f32 [n_head][head_dim+2] = acc | m | l instead of out */
    /* step-graph use only (NULL otherwise) */
    const int *n_past_dev;            /* with CGLM_SEQ_N_PAST_DEVICE: device word holding this sequence's n_past */
} cglm_attn_seq;

enum {
    CGLM_SEQ_NO_APPEND = 1,   /* this rank does not own position n_past: attend only */
    CGLM_SEQ_PARTIAL = 2,     /* emit un-normalised (acc, m, l) into .partial; .out is not written */
    CGLM_SEQ_USE_KV_LOCAL = 4,/* attend over kv_local cached tokens (+ the appended one) instead of n_virtual + n_past */
    /* Decode step whose position is a device-side scalar, so that a CUDA graph holding the layer calls of one
     * decode step can be replayed for the next token without being rebuilt (the reference rebuilds its ggml graph
     * every token, chatglm.cpp:728-729): the kernel reads n_past from *n_past_dev when it runs; the host field
     * n_past is only an upper bound (capacity check, launch sizing).  qlen 1, fused-decode shapes only
     * (CGLM_ERR_UNSUPPORTED otherwise); a device value outside [0, capacity) is clamped and reported through the
     * workspace status word as CGLM_ERR_INVALID_ARG.  cglm_seq_advance bumps the words between steps. */
    CGLM_SEQ_N_PAST_DEVICE = 8,
    /* A promise by the caller: no kernel that precedes this call on its stream and can still be running when this
     * call's kernel starts writes cache positions [0, n_virtual + n_past) of this sequence's slot.  The library launches its kernels as programmatic
     * dependents, so "can still be running" means the kernel enqueued immediately before (and, behind a kernel that
     * releases its dependents before it has waited for its own predecessor, that predecessor too).  The promise holds
     * for the layer calls of a decode step: what precedes is the qkv projection or another layer's attention.  It does
     * not hold for a call that directly follows a prefill, a cglm_kv_load_prefix or any other kernel that writes the
     * same slot.  When every one-token sequence of a call carries the flag, the fused decode kernel starts streaming
     * cache tiles (and pulls a few more into L2) while the previous kernel is still draining; q, k, v and the appended
     * row are still read and written only after that kernel has completed.  Without the flag nothing is read early. */
    CGLM_SEQ_CACHE_SETTLED = 16,
    /* f16 hand-off at either end of the path, for callers whose two Linears (chatglm.cpp:629, :719) produce and
     * consume half precision: with CGLM_SEQ_QKV_F16 q, k and v point at f16 values (what an f16 query_key_value GEMM
     * writes), with CGLM_SEQ_OUT_F16 out receives f16 (what an f16 dense GEMM reads).  RoPE, the 1/sqrt(d) scale and
     * the softmax still run in f32 and the cache bits are those of the f32 path fed the same (f16-representable)
     * values; the output is the f32 result rounded to nearest even.  q_roped / k_roped stay f32. */
    CGLM_SEQ_QKV_F16 = 32,
    CGLM_SEQ_OUT_F16 = 64,
    /* q has been through RoPE already (cglm_qkv_linear_forward ropes it in its epilogue): the kernels skip the rotation.
     * One-token sequences only.  Combined with CGLM_SEQ_NO_APPEND | CGLM_SEQ_USE_KV_LOCAL (kv_local = n_virtual + n_past
     * + 1) it is the attention call that follows the fused qkv Linear, which has appended K and V itself; k and v are
     * then not read and may alias q. */
    CGLM_SEQ_Q_ROPED = 128
};

/* Scratch the kernels need for n_seq sequences per call with at most max_qlen tokens each: a 256-byte header (status
 * word, counters), 9.7 MB of scratch for the Linear kernels (see cglm_linear_forward), then the attention kernels'
 * counters, partial results and staging.  One workspace serves one stream at a time. */
size_t cglm_attn_workspace_bytes(const cglm_attn_desc *desc, int n_seq, int max_qlen);
/* Zeroes the control words of a workspace.  Call once before first use and after any CGLM_ERR_TIMEOUT. */
int cglm_attn_workspace_init(void *workspace, size_t workspace_bytes, void *cuda_stream);
/* Synchronises the stream, returns the device-side status accumulated since the last query, clears it. */
int cglm_attn_workspace_status(void *workspace, void *cuda_stream);

/*
 * RoPE(q,k) -> f16 append -> attention for n_seq independent sequences (host array of descriptors).
 * Replaces the graph nodes of chatglm.cpp:636-717.  Decode (qlen 1) and prefill (n_past 0) may be mixed.
 * Asynchronous on cuda_stream.
 */
int cglm_attn_forward(cglm_kv_arena *arena, const cglm_attn_seq *seqs, int n_seq, void *workspace,
                      size_t workspace_bytes, void *cuda_stream);
/*
 * query_key_value Linear of a decode step with the front half of the attention path in its epilogue (chatglm.cpp:629 =
 * Linear::forward, chatglm.cpp:418-426, then :655-656 and :668-675): for n_seq one-token sequences
 *   qkv = x . weight^T + bias           x f16 [n_seq][hidden] (device), weight f16 [(H + 2G) * D][hidden] as the model file
 *                                       stores it, bias f32 [(H + 2G) * D] or NULL; tcgen05 tensor cores, f32 accumulation
 *   q_roped[i] = RoPE(q part)           f32 [n_seq][H * D], what the following attention call takes as q with
 *                                       CGLM_SEQ_Q_ROPED | CGLM_SEQ_NO_APPEND | CGLM_SEQ_USE_KV_LOCAL
 *   k_cache / v_cache of seqs[i].slot   RoPE(k part) and the v part appended as f16 at position n_virtual + n_past
 * The fused qkv activation itself is never written.  Only slot and n_past of each descriptor are read.  Arenas with
 * head_dim 128, blocked qkv layout and CGLM_ROPE_CHATGLM2 or CGLM_ROPE_DISABLED; hidden a multiple of 64; at most 128
 * sequences per call; other shapes return CGLM_ERR_UNSUPPORTED (run the Linear elsewhere and call cglm_attn_forward).
 * x, weight and q_roped 16-byte aligned.  Asynchronous on cuda_stream; workspace as for cglm_attn_forward (status word).
 */
int cglm_qkv_linear_forward(cglm_kv_arena *arena, const cglm_attn_seq *seqs, int n_seq, const void *x_f16, int hidden,
                            const void *weight_f16, const float *bias, float *q_roped, void *workspace,
                            size_t workspace_bytes, void *cuda_stream);
/*
 * Linear::forward (chatglm.cpp:418-426) on its own: out = x . weight^T + bias, the same tcgen05 GEMM with a plain
 * epilogue.  It is the dense projection behind the attention path (chatglm.cpp:719), fed by the f16 context_layer that
 * the attention kernels store with CGLM_SEQ_OUT_F16, and the query_key_value projection (chatglm.cpp:629) of prompts and
 * of shapes that cglm_qkv_linear_forward does not cover.
 *   x_f16 f16 [n_tok][in_features], weight_f16 f16 [out_features][in_features] as the model file stores it, bias f32
 *   [out_features] or NULL, out f32 (out_is_f16 == 0) or f16 [n_tok][out_features]; all on the device, x, weight and
 *   out 16-byte aligned; in_features a multiple of 64, out_features of 32 (else CGLM_ERR_UNSUPPORTED); any n_tok > 0.
 * f32 accumulation; the f32 result is rounded to nearest even when out is f16.  Runs on the current device.
 * workspace: an initialised workspace of at least cglm_linear_workspace_bytes(), which every workspace sized by
 * cglm_attn_workspace_bytes is.  Out-features that are a multiple of 128 run with the features on the M side of the MMA
 * and k split over several thread blocks per 128-feature tile, whose partial sums pass through the workspace; with a
 * smaller workspace (at least the 256-byte header) or other out-features the kernel with the tokens on the M side runs.
 * Asynchronous on cuda_stream; calls that share a workspace must be ordered on one stream.
 */
size_t cglm_linear_workspace_bytes(void);
/* How cglm_linear_forward would run a shape on a device of n_sm multiprocessors, without running it (host arithmetic only;
 * for tests and tuning).  Returns 1 and fills plan[8] = {tokens per tile, feature tiles, token tiles, k splits, 64-k blocks
 * per thread block, 64-k blocks per TMA box, ring stages, tensor-memory columns} when the kernel with the features on the
 * M side takes the shape, 0 when the kernel with the tokens on the M side does. */
int cglm_linear_kernel_plan(int n_tok, int in_features, int out_features, int n_sm, int plan[8]);
int cglm_linear_forward(const void *x_f16, int n_tok, int in_features, const void *weight_f16, int out_features,
                        const float *bias, void *out, int out_is_f16, void *workspace, size_t workspace_bytes,
                        void *cuda_stream);
/* dst_f16[i] = f16(src[i]), round to nearest even, for i in [0, n): the cast ggml applies to an f32 activation in front
 * of an f16 matrix (device pointers; asynchronous on cuda_stream). */
int cglm_convert_f32_to_f16(const float *src, void *dst_f16, size_t n, void *cuda_stream);
/* n_past_dev[i] += delta for i in [0, n): the last node of a captured decode step (see CGLM_SEQ_N_PAST_DEVICE). */
int cglm_seq_advance(int *n_past_dev, int n, int delta, void *cuda_stream);

/*
 * The same call for callers whose activations live in host memory, as ggml_backend_tensor_set /
 * ggml_backend_tensor_get move them in the reference (chatglm.cpp:743, 764): copies the fused qkv rows
 * host->device, runs cglm_attn_forward, copies context_layer device->host, all on cuda_stream.
 *   qkv_host  f32 (or f16) [n_tokens][(H+2G)*D], the rows of all sequences back to back (sequence i owns rows
 *             [tok_begin_i, tok_begin_i + qlen_i)); out_host f32 (or f16) [n_tokens][H*D].
 * layout: CGLM_HOST_INTERLEAVED_QKV selects the v1 layout; CGLM_HOST_F16 says that all four buffers hold f16 instead of
 * f32 (half the bytes across the bus; the kernels convert on load and store, see CGLM_SEQ_QKV_F16 / CGLM_SEQ_OUT_F16).
 * dev_qkv / dev_out are device staging buffers of at least those sizes.
 * Only n_past / qlen / n_ctx / slot (and CGLM_SEQ_CACHE_SETTLED of flags) of each descriptor are read.
 * The two copies run on streams of the arena's own and the kernels on cuda_stream, so that the
 * upload of one call and the download of another overlap the kernels between them (one call per layer: give
 * neighbouring calls different staging buffers, two or three pairs are enough; reuse of a staging buffer is ordered
 * by the library).  The copies are chained to the kernels by events, except that a fused decode launch does not make
 * cuda_stream wait for its input copy: it polls, with a bound, a device word that the copy stream writes right behind
 * the data, because a wait on the stream between two launches would end their programmatic overlap (measured: 2.79 ->
 * 2.57 ms per 40-layer step).  out_host is valid once cglm_attn_host_drain has been enqueued on a stream and that stream has
 * been synchronised.  Use pinned host memory for truly asynchronous copies.
 * Pinned host buffers are always staged, never read by the kernels across the bus: with the gated copies the staged
 * pipeline measured faster at every call size (8 sequences: 1.45 against 3.45 ms per 40-layer step).
 * The call uses streams and events of its own, so it cannot be issued while cuda_stream is being captured: capture
 * cglm_attn_forward on device buffers instead.
 */
enum { CGLM_HOST_INTERLEAVED_QKV = 1, CGLM_HOST_F16 = 2 };
int cglm_attn_forward_host(cglm_kv_arena *arena, const cglm_attn_seq *seqs, int n_seq, int layout,
                           const void *qkv_host, void *out_host, void *dev_qkv, void *dev_out,
                           void *workspace, size_t workspace_bytes, void *cuda_stream);

/* Makes cuda_stream wait for every device-to-host copy that cglm_attn_forward_host has enqueued for this arena: the
 * point where a step's results are read back (ggml_backend_tensor_get at the end of a step, chatglm.cpp:764).
 * cuda_stream may be any stream. */
int cglm_attn_host_drain(cglm_kv_arena *arena, void *cuda_stream);

/*
 * Decode step that brings its own scratch memory.  No counterpart in the reference; it exists for hosts that
 * cannot hand the library a workspace when they call it: a server whose allocator already owns the whole GPU, a
 * plugin sandbox where cudaMalloc is off limits, a loop that must stay clear of the allocator once it runs.
 * Same work and same results as cglm_attn_forward for one-token sequences (qlen 1, flags 0, no partial output)
 * on an arena with head_dim 128, at most 16 q heads per kv head and a cache capacity that is a multiple of 8;
 * other shapes return CGLM_ERR_UNSUPPORTED.  The scratch is a fixed ~5 MiB (5 258 496 bytes) array inside the library image, held
 * by every GPU that loads the library until the process exits.  Limits per call: 128 sequences, 32 kv heads,
 * a GPU of at most 148 SMs; beyond them the call fails with CGLM_ERR_WORKSPACE.
 * The call allocates nothing.  The first call on each device looks up the array's device address (with that
 * device current); make that first call before any stream capture begins.  All calls on a device share the
 * array: two calls whose kernels can overlap on the GPU (different streams) race on it, so keep them on one
 * stream or order them yourself.  wait_and_check != 0 synchronises the stream and returns the device-side
 * status (0 or CGLM_ERR_TIMEOUT); otherwise the call is asynchronous like cglm_attn_forward.
 */
int cglm_attn_decode_static(cglm_kv_arena *arena, const cglm_attn_seq *seqs, int n_seq, int wait_and_check,
                            void *cuda_stream);

/*
 * Split-KV combine: log-sum-exp merge of n_part partials of one query token, each laid out
 * f32 [n_head][head_dim+2] (acc | m | l), all in this GPU's memory -> out f32 [n_head*head_dim].
 * The per-GPU partials come from cglm_attn_forward with CGLM_SEQ_PARTIAL.
 */
int cglm_attn_splitkv_combine(const float *partials, int n_part, int n_head, int head_dim, float *out,
                              void *cuda_stream);

/*
 * Fused split-KV step over peer memory: ONE launch per rank and decode step.  (The reference runs on one device; this
 * is the exchange step of a KV length split over the GPUs of one NVLink box, done inside the attention kernel.)
 *
 * Every rank owns an exchange buffer of cglm_attn_splitkv_xchg_bytes(n_rank, n_head, head_dim) bytes in its own
 * memory, zero-filled once, and mapped into its peers by the host (cglm_xchg_export / cglm_xchg_import between
 * processes, plain pointers when the ranks are contexts of one process).  The buffer holds a step counter, two sets
 * (alternating by step) of arrival words [rank][kv head] and two sets of n_rank partial slots [n_head][head_dim+2].
 *
 * cglm_attn_splitkv_step runs the fused decode kernel over this rank's slice of the sequence (seq as for
 * cglm_attn_forward with CGLM_SEQ_USE_KV_LOCAL and, on ranks that do not own position n_past, CGLM_SEQ_NO_APPEND;
 * .out and .partial are ignored).  Step number e = the local buffer's counter + 1.  The thread block that completes a
 * kv head writes its un-normalised (acc, m, l) rows into slot `rank` of set e & 1 of EVERY rank's buffer
 * (xchg[0..n_rank), device pointers valid on this GPU, entry `rank` the local one) with plain stores, fences at system
 * scope and publishes e in the arrival words (release).  With combine != 0 the block that publishes this rank's last
 * kv head then waits until every arrival word of set e & 1 of the LOCAL buffer holds e, merges the n_rank partials
 * (log-sum-exp) into out f32 [n_head * head_dim] and advances the local counter to e; with combine == 0 it only
 * advances the counter (gather-to-root: only the ranks that need the result combine).  The wait is bounded: after
 * timeout_us (0: 20 ms) the kernel records CGLM_ERR_TIMEOUT in the workspace status word, leaves out untouched and
 * still advances the counter.  A host that reads CGLM_ERR_TIMEOUT from cglm_attn_workspace_status must stop stepping:
 * the ranks are no longer in the same step, and every further combine would run into its bound as well.
 * The waiting block waits for other GPUs only, never for another block or launch of its own GPU; ranks that share a
 * GPU (tests) must therefore be launched with combine == 0 for all but the last of them.
 * Two sets suffice: a rank cannot publish step e+2 before its own combine of step e+1, which needs every peer's step
 * e+1, which that peer launched after its own combine of step e had completed.  Because the step counter lives on the
 * device, a captured CUDA graph of the step can be replayed.  No TMA multicast and no library kernel touch peer memory.
 */
size_t cglm_attn_splitkv_xchg_bytes(int n_rank, int n_head, int head_dim);
/* Host plumbing for ranks that are separate processes (one per GPU): the owner allocates its zero-filled buffer
 * and exports a 64-byte CUDA IPC handle, which travels to the peers by any host channel; a peer imports it WITH ITS
 * OWN DEVICE CURRENT, which maps the owner's memory into the importing device's context (peer access is enabled
 * as part of the import; CGLM_ERR_UNSUPPORTED when the two devices have no peer path) and checks the mapping with
 * a 4-byte copy through the runtime before any kernel touches it.  Imported mappings live until the process
 * exits. */
int cglm_xchg_alloc(size_t bytes, void **ptr);
int cglm_xchg_free(void *ptr);
/* Diagnostics: waits for the device, then copies the first `bytes` bytes of a buffer (step counter at word 0, arrival
 * words [set][rank 0..15][kv head 0..31] from word 32) to host memory. */
int cglm_xchg_read(const void *ptr, void *host, size_t bytes);
int cglm_xchg_export(void *ptr, unsigned char handle[64]);
int cglm_xchg_import(const unsigned char handle[64], int owner_device, void **ptr);
int cglm_attn_splitkv_step(cglm_kv_arena *arena, const cglm_attn_seq *seq, void *const *xchg, int n_rank, int rank,
                           float *out, int combine, unsigned int timeout_us, void *workspace, size_t workspace_bytes,
                           void *cuda_stream);

/* P-Tuning v2 prefix load for one slot (BasicModel::load_prefix_cache, chatglm.h:580-615):
 * past_kv f16 [2][n_kv_head][n_virtual][head_dim] (device) -> cache positions [0, n_virtual), V transposed. */
int cglm_kv_load_prefix(cglm_kv_arena *arena, int slot, const void *past_kv, void *cuda_stream);

/*
 * Counter-based synthetic data (no counterpart in the reference; for benchmarks and tests): element first + i of tensor
 * tensor_id under a seed is table[splitmix64(seed * 0x9E3779B97F4A7C15 + tensor_id * 0xBF58476D1CE4E5B9 + first + i) >> 48],
 * table being 65536 values in device memory (e.g. the N(0,1) quantiles).  Integer arithmetic only: a host loop over
 * the same expression yields the same bits, so a CPU arm can rebuild any part of a 20 GiB cache without a download.
 */
int cglm_synth_fill_f16(void *dst, long long n, unsigned long long seed, unsigned long long tensor_id, long long first,
                        const void *table_f16, void *cuda_stream);
int cglm_synth_fill_f32(float *dst, long long n, unsigned long long seed, unsigned long long tensor_id, long long first,
                        const float *table_f32, void *cuda_stream);

const char *cglm_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char *cglm_last_error_string(void);
/* Number of kernels the library launched since load (all threads); for launch accounting in benchmarks. */
unsigned long long cglm_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* CGLM_ATTN_H */
