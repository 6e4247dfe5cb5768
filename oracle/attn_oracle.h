/*
 * CPU oracle for the attention KV-cache path of li-plus/chatglm.cpp.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It is a restatement, op by op, of what
 * BasicAttention::forward (chatglm.cpp:620-721) and the RoPE helpers (chatglm.cpp:523-618)
 * record as a ggml graph, plus the two set_graph_inputs producers (chatglm.cpp:1123-1154,
 * 1315-1327).  Only tests, the smoke check and the bench's CPU-baseline leg may link it; the
 * shipped library never does.
 *
 * The arithmetic of the reference lives in ggml (module ggerganov/ggml, revision unpinned in
 * .gitmodules:8-10, sources absent), so the numerics that ggml's CPU backend chooses are
 * carried as switches in oracle_numerics:
 *   - the f32 operand of a mul_mat against an f16 matrix is rounded to f16 first,
 *   - the softmax denominator is accumulated in double,
 *   - the RoPE angle ladder is an iterated f32 product theta *= theta_scale.
 * Parity of this restatement is pinned by the reference's own golden fixtures
 * (tests/data/{glm,glm_ptuning_v2,glm2,glm3,glm3_ptuning_v2,glm4}_model.data, tolerance 5e-4 from
 * chatglm_test.cpp:338).  Those fixtures use head_dim 4, so the pair pattern and frequency
 * ladder at head_dim 128 are "parity unpinned" by the reference's tests; they follow the
 * call-site arguments (chatglm.cpp:563-564, 593-594) and are cross-checked against the
 * published GLM rotary formulation.
 */
#ifndef ATTN_ORACLE_H
#define ATTN_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* values of chatglm::RopeType (chatglm.h:93-99) */
enum {
    ORACLE_ROPE_GPTJ = 0,
    ORACLE_ROPE_NEOX = 2,
    ORACLE_ROPE_CHATGLM = 4,
    ORACLE_ROPE_CHATGLM2 = 8,
    ORACLE_ROPE_DISABLED = 10000
};

/* values of chatglm::AttentionMaskType (chatglm.h:101-104) */
enum { ORACLE_MASK_CAUSAL = 0, ORACLE_MASK_CHATGLM = 1 };

typedef struct {
    int round_q_f16;     /* 1: scaled q is rounded to f16 before QK^T (ggml CPU mul_mat with an f16 src0) */
    int round_p_f16;     /* 1: probabilities are rounded to f16 before PV */
    int softmax_double;  /* 1: softmax denominator accumulated in double */
    int theta_powf;      /* 0: iterated product ladder (ggml); 1: powf(theta, -2i/n) per pair */
} oracle_numerics;

typedef struct {
    int n_head;      /* H  */
    int n_kv_head;   /* G  */
    int head_dim;    /* D  */
    int max_len;     /* M = max_length + n_virtual, the cache capacity in tokens (chatglm.h:452-455) */
    int n_virtual;   /* V, P-Tuning v2 prefix length */
    int rope_type;   /* ORACLE_ROPE_* */
    float rope_theta;
    int mask_type;   /* ORACLE_MASK_* */
    oracle_numerics num;
} oracle_cfg;

/* The numerics ggml's CPU backend uses (f16 operand rounding, double softmax sum, iterated ladder). */
oracle_numerics oracle_numerics_ggml(void);
/* Plain f32 attention over the f16 cache: no operand rounding. */
oracle_numerics oracle_numerics_f32(void);

/* IEEE binary16 <-> binary32, round to nearest even (what ggml_cpy f32->f16 stores). */
uint16_t oracle_f32_to_f16(float x);
float oracle_f16_to_f32(uint16_t h);

/* chatglm.cpp:1319-1327 : ids = n_past .. n_past+qlen-1 */
void oracle_position_ids_glm2(int qlen, int n_past, int *ids /* [qlen] */);
/* chatglm.cpp:1142-1153 : ids[i] = min(p, n_ctx-2), ids[qlen+i] = max(p-(n_ctx-2), 0), p = n_past+i */
void oracle_position_ids_glm(int qlen, int n_past, int n_ctx, int *ids /* [2*qlen] */);
/* chatglm.cpp:1126-1140 : additive mask [qlen, kvlen], -inf at [i < qlen-1][kvlen-1] */
void oracle_attention_mask_glm(int qlen, int kvlen, float *mask /* [qlen*kvlen] */);

/* RoPE in place on x[s][h][:] (chatglm.cpp:523-618).  Strides in elements. */
void oracle_apply_rotary_emb(const oracle_cfg *cfg, float *x, long tok_stride, long head_stride, int n_heads,
                             int qlen, const int *position_ids);

/*
 * One BasicAttention::forward without the two Linears: from the split q/k/v activations to
 * context_layer [qlen, H*D] (chatglm.cpp:636-717).
 *   q,k,v          f32, read through (token, head) element strides so that both the blocked
 *                  (chatglm.cpp:646-652) and interleaved (chatglm.cpp:638-644) qkv layouts pass.
 *   k_cache        f16 [G][M][D]; v_cache f16 [G][D][M] (chatglm.h:452-455); updated in place.
 *   position_ids   [qlen] or, for ORACLE_ROPE_CHATGLM, [2*qlen].
 *   attention_mask [qlen][V+qlen] additive, used only when n_past==0 and mask_type==CHATGLM.
 *   out            f32 [qlen][H*D].
 *   q_roped/k_roped optional f32 [qlen][H*D] / [qlen][G*D]: the activations after RoPE (before the
 *                  1/sqrt(D) scale), which the reference leaves in place in the qkv buffer.
 * Returns 0, or -1 on an argument error.
 */
int oracle_attn_forward(const oracle_cfg *cfg, const float *q, long q_tok_stride, long q_head_stride,
                        const float *k, const float *v, long kv_tok_stride, long kv_head_stride,
                        uint16_t *k_cache, uint16_t *v_cache, const int *position_ids,
                        const float *attention_mask, int qlen, int n_past, float *out, float *q_roped,
                        float *k_roped);

/* P-Tuning v2 prefix load (chatglm.h:580-615): past_key_values f16 [2][G][V][D] for one layer. */
void oracle_load_prefix_cache(const oracle_cfg *cfg, const uint16_t *past_kv, uint16_t *k_cache,
                              uint16_t *v_cache);

/*
 * Attention over positions [kv_begin, kv_end) of an already-filled cache for one query token,
 * returning un-normalised partials: acc [H][D], m [H], l [H]  (the split-KV building block).
 * q must already be roped; it is scaled here.
 */
int oracle_attn_partial(const oracle_cfg *cfg, const float *q_roped /* [H][D] */, const uint16_t *k_cache,
                        const uint16_t *v_cache, int kv_begin, int kv_end, float *acc, float *m, float *l);
/* log-sum-exp merge of n partials laid out [n][H][D], [n][H], [n][H] -> out [H][D] */
void oracle_attn_combine(int n_head, int head_dim, int n, const float *acc, const float *m, const float *l,
                         float *out);

/*
 * Batched decode used for the timed CPU baseline: n_seq independent sequences, one token each,
 * OpenMP-parallel over (sequence, kv head).  Every array is indexed by sequence.
 */
int oracle_attn_decode_batch(const oracle_cfg *cfg, int n_seq, const float *const *q, const float *const *k,
                             const float *const *v, long q_head_stride, long kv_head_stride,
                             uint16_t *const *k_cache, uint16_t *const *v_cache, const int *n_past,
                             const int *n_ctx, float *const *out, int n_threads);

/* Host twin of the library's counter-based synthetic data (cglm_synth_fill_f16 / _f32): same integer expression,
 * same bits.  table: 65536 values. */
void oracle_synth_fill_f16(uint16_t *dst, long long n, unsigned long long seed, unsigned long long tensor_id, long long first,
                           const uint16_t *table);
void oracle_synth_fill_f32(float *dst, long long n, unsigned long long seed, unsigned long long tensor_id, long long first,
                           const float *table);

/* Linear::forward (chatglm.cpp:418-426): y [n_tok][out] = x [n_tok][in] . weight[out][in]^T (+ bias).  weight is f32, or
 * f16 bits with w_is_f16; round_x_f16 rounds the activations to f16 first, as ggml's CPU backend does against an f16
 * matrix; accumulation in f32. */
void oracle_linear(const float *x, int n_tok, int in, const void *weight, int w_is_f16, const float *bias, int out,
                   int round_x_f16, float *y);

#ifdef __cplusplus
}
#endif
#endif
