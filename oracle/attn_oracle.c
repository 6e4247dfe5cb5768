/*
 * CPU oracle for the attention KV-cache path of li-plus/chatglm.cpp -- test infrastructure only.
 * See attn_oracle.h for what it restates and how its parity is pinned.
 *
 * Build with -ffp-contract=off so that the RoPE rotation keeps its four products and two sums as
 * separately rounded f32 operations.
 */
#include "attn_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

oracle_numerics oracle_numerics_ggml(void) {
    oracle_numerics n = {1, 1, 1, 0};
    return n;
}

oracle_numerics oracle_numerics_f32(void) {
    oracle_numerics n = {0, 0, 1, 0};
    return n;
}

/* ---- binary16 conversion, round to nearest even ------------------------------------------- */

uint16_t oracle_f32_to_f16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t absu = u & 0x7fffffffu;
    if (absu >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | (absu > 0x7f800000u ? (0x0200u | ((absu >> 13) & 0x3ffu)) : 0u));
    }
    if (absu >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absu < 0x33000001u) { /* <= 2^-25 rounds to zero (tie at exactly 2^-25 goes to even = 0) */
        return (uint16_t)sign;
    }
    int exp = (int)(absu >> 23) - 127;
    uint32_t man = (absu & 0x7fffffu) | 0x800000u; /* 24-bit significand */
    int shift;                                     /* bits dropped from the 24-bit significand */
    uint32_t base;
    if (exp < -14) { /* subnormal half */
        shift = 13 + (-14 - exp);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(exp + 15) << 10;
        man &= 0x7fffffu;
    }
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) {
        q++;
    }
    return (uint16_t)(sign | (base + q)); /* a carry out of the mantissa bumps the exponent */
}

float oracle_f16_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* ---- graph inputs ---------------------------------------------------------------------------- */

/* chatglm.cpp:1319-1327 */
void oracle_position_ids_glm2(int qlen, int n_past, int *ids) {
    for (int i = 0; i < qlen; i++) {
        ids[i] = n_past + i;
    }
}

/* chatglm.cpp:1142-1153 */
void oracle_position_ids_glm(int qlen, int n_past, int n_ctx, int *ids) {
    for (int i = 0; i < qlen; i++) {
        const int p = n_past + i;
        ids[i] = p < n_ctx - 2 ? p : n_ctx - 2;
        ids[qlen + i] = p - (n_ctx - 2) > 0 ? p - (n_ctx - 2) : 0;
    }
}

/* chatglm.cpp:1126-1140 */
void oracle_attention_mask_glm(int qlen, int kvlen, float *mask) {
    for (long i = 0; i < (long)qlen * kvlen; i++) {
        mask[i] = 0.f;
    }
    for (int i = 0; i < qlen - 1; i++) {
        mask[(long)i * kvlen + (kvlen - 1)] = -INFINITY;
    }
}

/* ---- RoPE ------------------------------------------------------------------------------------ */

/*
 * cos/sin of the n_dims/2 angles of one position, the way ggml fills its per-position cache:
 * theta_0 = pos, theta_{i+1} = theta_i * theta_scale with theta_scale = powf(base, -2/n_dims).
 */
static void rope_cache(const oracle_cfg *cfg, int pos, int n_dims, float base, float *cs /* [n_dims] */) {
    const float theta_scale = powf(base, -2.0f / (float)n_dims);
    float theta = (float)pos;
    for (int i0 = 0; i0 < n_dims; i0 += 2) {
        float t = theta;
        if (cfg->num.theta_powf) {
            t = (float)pos * powf(base, -(float)i0 / (float)n_dims);
        }
        /* cosf/sinf taken as the correctly rounded values (evaluated in double, rounded once), so that the
         * pin does not hang on one C library's last-bit behaviour: libm float versions differ by an ulp
         * between platforms, and an ulp in cos is unbounded in ulps of x0*cos - x1*sin under cancellation. */
        cs[i0] = (float)cos((double)t);
        cs[i0 + 1] = (float)sin((double)t);
        theta *= theta_scale;
    }
}

/* ggml rope mode 0 ("GPTJ"/norm): adjacent pairs (2i, 2i+1) within the first n_dims of the row */
static void rope_row_adjacent(float *x, int n_dims, const float *cs) {
    for (int i0 = 0; i0 < n_dims; i0 += 2) {
        const float c = cs[i0], s = cs[i0 + 1];
        const float x0 = x[i0], x1 = x[i0 + 1];
        x[i0] = x0 * c - x1 * s;
        x[i0 + 1] = x0 * s + x1 * c;
    }
}

/* ggml rope mode 2 ("NEOX"): pairs (i, i + n_dims/2) within the first n_dims of the row */
static void rope_row_split(float *x, int n_dims, const float *cs) {
    const int half = n_dims / 2;
    for (int i0 = 0; i0 < n_dims; i0 += 2) {
        const int ic = i0 / 2;
        const float c = cs[i0], s = cs[i0 + 1];
        const float x0 = x[ic], x1 = x[ic + half];
        x[ic] = x0 * c - x1 * s;
        x[ic + half] = x0 * s + x1 * c;
    }
}

void oracle_apply_rotary_emb(const oracle_cfg *cfg, float *x, long tok_stride, long head_stride, int n_heads,
                             int qlen, const int *position_ids) {
    const int D = cfg->head_dim;
    if (cfg->rope_type == ORACLE_ROPE_DISABLED) { /* chatglm.cpp:613-614 */
        return;
    }
    float *cs = (float *)malloc(sizeof(float) * (size_t)D * 2);
    for (int s = 0; s < qlen; s++) {
        switch (cfg->rope_type) {
        case ORACLE_ROPE_GPTJ: /* chatglm.cpp:523-537, full head, n_dims = head_size */
        case ORACLE_ROPE_NEOX:
            rope_cache(cfg, position_ids[s], D, cfg->rope_theta, cs);
            for (int h = 0; h < n_heads; h++) {
                float *row = x + s * tok_stride + h * head_stride;
                if (cfg->rope_type == ORACLE_ROPE_GPTJ) {
                    rope_row_adjacent(row, D, cs);
                } else {
                    rope_row_split(row, D, cs);
                }
            }
            break;
        case ORACLE_ROPE_CHATGLM2: /* chatglm.cpp:576-601: first D/2 dims, adjacent pairs, base rope_theta */
            rope_cache(cfg, position_ids[s], D / 2, cfg->rope_theta, cs);
            for (int h = 0; h < n_heads; h++) {
                rope_row_adjacent(x + s * tok_stride + h * head_stride, D / 2, cs);
            }
            break;
        case ORACLE_ROPE_CHATGLM: /* chatglm.cpp:539-574: two halves, split pairs, default base 10000 */
            rope_cache(cfg, position_ids[s], D / 2, 10000.f, cs);
            rope_cache(cfg, position_ids[qlen + s], D / 2, 10000.f, cs + D);
            for (int h = 0; h < n_heads; h++) {
                float *row = x + s * tok_stride + h * head_stride;
                rope_row_split(row, D / 2, cs);
                rope_row_split(row + D / 2, D / 2, cs + D);
            }
            break;
        default:
            break;
        }
    }
    free(cs);
}

/* ---- attention ------------------------------------------------------------------------------- */

static inline float maybe_round_f16(float x, int on) { return on ? oracle_f16_to_f32(oracle_f32_to_f16(x)) : x; }

/* dot(f16 row, f32 vector) with f32 accumulation: the inner product of both mul_mats */
static float dot_f16_f32_scalar(const uint16_t *a, const float *b, int n) {
    float acc = 0.f;
    for (int i = 0; i < n; i++) {
        acc += oracle_f16_to_f32(a[i]) * b[i];
    }
    return acc;
}

#if defined(__x86_64__) && defined(__GNUC__)
#include <immintrin.h>
/* SIMD form (F16C convert + FMA, eight lanes), as ggml's CPU vec_dot does on x86; chosen at run time */
__attribute__((target("avx2,f16c,fma"))) static float dot_f16_f32_avx2(const uint16_t *a, const float *b, int n) {
    __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
    int i = 0;
    for (; i + 16 <= n; i += 16) {
        const __m256 a0 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(a + i)));
        const __m256 a1 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(a + i + 8)));
        acc0 = _mm256_fmadd_ps(a0, _mm256_loadu_ps(b + i), acc0);
        acc1 = _mm256_fmadd_ps(a1, _mm256_loadu_ps(b + i + 8), acc1);
    }
    for (; i + 8 <= n; i += 8) {
        const __m256 a0 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(a + i)));
        acc0 = _mm256_fmadd_ps(a0, _mm256_loadu_ps(b + i), acc0);
    }
    acc0 = _mm256_add_ps(acc0, acc1);
    __m128 lo = _mm_add_ps(_mm256_castps256_ps128(acc0), _mm256_extractf128_ps(acc0, 1));
    lo = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
    lo = _mm_add_ss(lo, _mm_shuffle_ps(lo, lo, 1));
    float acc = _mm_cvtss_f32(lo);
    for (; i < n; i++) {
        acc += oracle_f16_to_f32(a[i]) * b[i];
    }
    return acc;
}
static int have_avx2_f16c(void) {
    static int cached = -1;
    if (cached < 0) {
        cached = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("f16c") && __builtin_cpu_supports("fma");
    }
    return cached;
}
static inline float dot_f16_f32(const uint16_t *a, const float *b, int n) {
    return have_avx2_f16c() ? dot_f16_f32_avx2(a, b, n) : dot_f16_f32_scalar(a, b, n);
}
#else
static inline float dot_f16_f32(const uint16_t *a, const float *b, int n) { return dot_f16_f32_scalar(a, b, n); }
#endif

/* softmax over one row in place (ggml_soft_max: max-subtract, exp, sum, scale by 1/sum) */
static void softmax_row(float *row, int n, int sum_double) {
    float mx = -INFINITY;
    for (int j = 0; j < n; j++) {
        mx = row[j] > mx ? row[j] : mx;
    }
    if (sum_double) {
        double sum = 0.0;
        for (int j = 0; j < n; j++) {
            const float e = row[j] == -INFINITY ? 0.f : expf(row[j] - mx);
            row[j] = e;
            sum += (double)e;
        }
        const float inv = (float)(1.0 / sum);
        for (int j = 0; j < n; j++) {
            row[j] *= inv;
        }
    } else {
        float sum = 0.f;
        for (int j = 0; j < n; j++) {
            const float e = row[j] == -INFINITY ? 0.f : expf(row[j] - mx);
            row[j] = e;
            sum += e;
        }
        const float inv = 1.f / sum;
        for (int j = 0; j < n; j++) {
            row[j] *= inv;
        }
    }
}

/*
 * Attention of one q head over cache positions [0, L) for qlen query rows.
 * qh: [qlen][D] roped, unscaled (row stride D).  scores: scratch [qlen][L].  out row stride out_stride.
 */
static void attend_head(const oracle_cfg *cfg, const float *qh, int qlen, int n_past, const uint16_t *kc,
                        const uint16_t *vc, const float *attention_mask, float *scores, float *qs, float *out,
                        long out_stride) {
    const int D = cfg->head_dim, M = cfg->max_len, V = cfg->n_virtual;
    const int L = V + n_past + qlen;
    const float scale = 1.f / sqrtf((float)D); /* chatglm.cpp:686 */
    for (int s = 0; s < qlen; s++) {
        float *row = scores + (long)s * L;
        for (int d = 0; d < D; d++) {
            qs[d] = maybe_round_f16(qh[(long)s * D + d] * scale, cfg->num.round_q_f16);
        }
        /* chatglm.cpp:687: scores = K . q over [0, L) */
        for (int j = 0; j < L; j++) {
            row[j] = dot_f16_f32(kc + (long)j * D, qs, D);
        }
        /* chatglm.cpp:689-707: masks only while n_past == 0 */
        if (n_past == 0) {
            if (cfg->mask_type == ORACLE_MASK_CAUSAL) {
                for (int j = V + s + 1; j < L; j++) { /* ggml_diag_mask_inf(n_past = V): j > V + s */
                    row[j] = -INFINITY;
                }
            } else if (attention_mask) {
                for (int j = 0; j < L; j++) {
                    row[j] += attention_mask[(long)s * L + j];
                }
            }
        }
        softmax_row(row, L, cfg->num.softmax_double); /* chatglm.cpp:709 */
        /* chatglm.cpp:711: context = V^T . p */
        if (cfg->num.round_p_f16) {
            for (int j = 0; j < L; j++) {
                row[j] = maybe_round_f16(row[j], 1);
            }
        }
        for (int d = 0; d < D; d++) {
            out[(long)s * out_stride + d] = dot_f16_f32(vc + (long)d * M, row, L);
        }
    }
}

int oracle_attn_forward(const oracle_cfg *cfg, const float *q, long q_tok_stride, long q_head_stride,
                        const float *k, const float *v, long kv_tok_stride, long kv_head_stride,
                        uint16_t *k_cache, uint16_t *v_cache, const int *position_ids,
                        const float *attention_mask, int qlen, int n_past, float *out, float *q_roped,
                        float *k_roped) {
    const int H = cfg->n_head, G = cfg->n_kv_head, D = cfg->head_dim, M = cfg->max_len, V = cfg->n_virtual;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || (D & 1) || qlen <= 0 || n_past < 0 || V + n_past + qlen > M) {
        return -1;
    }
    const int R = H / G;
    const int L = V + n_past + qlen;

    /* contiguous working copies: [qlen][H][D] and [qlen][G][D] */
    float *qw = (float *)malloc(sizeof(float) * (size_t)qlen * H * D);
    float *kw = (float *)malloc(sizeof(float) * (size_t)qlen * G * D);
    for (int s = 0; s < qlen; s++) {
        for (int h = 0; h < H; h++) {
            memcpy(qw + ((long)s * H + h) * D, q + s * q_tok_stride + h * q_head_stride, sizeof(float) * D);
        }
        for (int g = 0; g < G; g++) {
            memcpy(kw + ((long)s * G + g) * D, k + s * kv_tok_stride + g * kv_head_stride, sizeof(float) * D);
        }
    }
    /* chatglm.cpp:655-656 */
    oracle_apply_rotary_emb(cfg, qw, (long)H * D, D, H, qlen, position_ids);
    oracle_apply_rotary_emb(cfg, kw, (long)G * D, D, G, qlen, position_ids);
    if (q_roped) {
        memcpy(q_roped, qw, sizeof(float) * (size_t)qlen * H * D);
    }
    if (k_roped) {
        memcpy(k_roped, kw, sizeof(float) * (size_t)qlen * G * D);
    }

    /* chatglm.cpp:668-675: append f16(k) at rows V+n_past.., f16(v) transposed at columns V+n_past.. */
    for (int g = 0; g < G; g++) {
        for (int s = 0; s < qlen; s++) {
            uint16_t *krow = k_cache + ((long)g * M + (V + n_past + s)) * D;
            const float *vsrc = v + s * kv_tok_stride + g * kv_head_stride;
            for (int d = 0; d < D; d++) {
                krow[d] = oracle_f32_to_f16(kw[((long)s * G + g) * D + d]);
                v_cache[((long)g * D + d) * M + (V + n_past + s)] = oracle_f32_to_f16(vsrc[d]);
            }
        }
    }

    /* chatglm.cpp:658-662, 678-717: per q head h of group g = h / R */
    int err = 0;
#pragma omp parallel
    {
        float *scores = (float *)malloc(sizeof(float) * (size_t)qlen * L);
        float *qh = (float *)malloc(sizeof(float) * (size_t)qlen * D);
        float *qs = (float *)malloc(sizeof(float) * (size_t)D);
#pragma omp for schedule(dynamic, 1)
        for (int h = 0; h < H; h++) {
            const int g = h / R;
            for (int s = 0; s < qlen; s++) {
                memcpy(qh + (long)s * D, qw + ((long)s * H + h) * D, sizeof(float) * D);
            }
            attend_head(cfg, qh, qlen, n_past, k_cache + (long)g * M * D, v_cache + (long)g * D * M,
                        attention_mask, scores, qs, out + (long)h * D, (long)H * D);
        }
        free(scores);
        free(qh);
        free(qs);
    }
    free(qw);
    free(kw);
    return err;
}

/* chatglm.h:580-615 */
void oracle_load_prefix_cache(const oracle_cfg *cfg, const uint16_t *past_kv, uint16_t *k_cache,
                              uint16_t *v_cache) {
    const int G = cfg->n_kv_head, D = cfg->head_dim, M = cfg->max_len, V = cfg->n_virtual;
    const uint16_t *pk = past_kv;                     /* [G][V][D] */
    const uint16_t *pv = past_kv + (long)G * V * D;   /* [G][V][D] */
    for (int g = 0; g < G; g++) {
        for (int t = 0; t < V; t++) {
            for (int d = 0; d < D; d++) {
                k_cache[((long)g * M + t) * D + d] = pk[((long)g * V + t) * D + d];
                v_cache[((long)g * D + d) * M + t] = pv[((long)g * V + t) * D + d];
            }
        }
    }
}

/* ---- split-KV building blocks ---------------------------------------------------------------- */

int oracle_attn_partial(const oracle_cfg *cfg, const float *q_roped, const uint16_t *k_cache,
                        const uint16_t *v_cache, int kv_begin, int kv_end, float *acc, float *m, float *l) {
    const int H = cfg->n_head, G = cfg->n_kv_head, D = cfg->head_dim, M = cfg->max_len;
    if (kv_begin < 0 || kv_end > M || kv_begin > kv_end) {
        return -1;
    }
    const int R = H / G;
    const float scale = 1.f / sqrtf((float)D);
    const int n = kv_end - kv_begin;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < H; h++) {
        const int g = h / R;
        const uint16_t *kc = k_cache + (long)g * M * D;
        const uint16_t *vc = v_cache + (long)g * D * M;
        float *sc = (float *)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
        float *qs = (float *)malloc(sizeof(float) * (size_t)D);
        for (int d = 0; d < D; d++) {
            qs[d] = maybe_round_f16(q_roped[(long)h * D + d] * scale, cfg->num.round_q_f16);
        }
        float mx = -INFINITY;
        for (int j = 0; j < n; j++) {
            const float a = dot_f16_f32(kc + (long)(kv_begin + j) * D, qs, D);
            sc[j] = a;
            mx = a > mx ? a : mx;
        }
        double sum = 0.0;
        for (int j = 0; j < n; j++) {
            sc[j] = expf(sc[j] - mx);
            sum += sc[j];
        }
        for (int j = 0; j < n; j++) {
            sc[j] = maybe_round_f16(sc[j], cfg->num.round_p_f16);
        }
        for (int d = 0; d < D; d++) {
            acc[(long)h * D + d] = dot_f16_f32(vc + (long)d * M + kv_begin, sc, n);
        }
        m[h] = mx;
        l[h] = (float)sum;
        free(sc);
        free(qs);
    }
    return 0;
}

void oracle_attn_combine(int n_head, int head_dim, int n, const float *acc, const float *m, const float *l,
                         float *out) {
    for (int h = 0; h < n_head; h++) {
        float mx = -INFINITY;
        for (int r = 0; r < n; r++) {
            mx = m[(long)r * n_head + h] > mx ? m[(long)r * n_head + h] : mx;
        }
        double den = 0.0;
        for (int r = 0; r < n; r++) {
            const float mr = m[(long)r * n_head + h];
            den += mr == -INFINITY ? 0.0 : (double)l[(long)r * n_head + h] * exp((double)(mr - mx));
        }
        for (int d = 0; d < head_dim; d++) {
            double num = 0.0;
            for (int r = 0; r < n; r++) {
                const float mr = m[(long)r * n_head + h];
                if (mr != -INFINITY) {
                    num += (double)acc[((long)r * n_head + h) * head_dim + d] * exp((double)(mr - mx));
                }
            }
            out[(long)h * head_dim + d] = (float)(num / den);
        }
    }
}

/* ---- batched decode for the timed CPU baseline ------------------------------------------------ */

int oracle_attn_decode_batch(const oracle_cfg *cfg, int n_seq, const float *const *q, const float *const *k,
                             const float *const *v, long q_head_stride, long kv_head_stride,
                             uint16_t *const *k_cache, uint16_t *const *v_cache, const int *n_past,
                             const int *n_ctx, float *const *out, int n_threads) {
    const int H = cfg->n_head, G = cfg->n_kv_head, D = cfg->head_dim, M = cfg->max_len, V = cfg->n_virtual;
    const int R = H / G;
    int bad = 0;
    for (int i = 0; i < n_seq; i++) {
        if (n_past[i] < 0 || V + n_past[i] + 1 > M) {
            bad = 1;
        }
    }
    if (bad) {
        return -1;
    }
#ifdef _OPENMP
    if (n_threads > 0) {
        omp_set_num_threads(n_threads);
    }
#else
    (void)n_threads;
#endif
    /* pass 1: RoPE + append per (sequence, kv head): chatglm.cpp:655-675 */
    float *qr = (float *)malloc(sizeof(float) * (size_t)n_seq * H * D);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < n_seq; i++) {
        int ids[2];
        if (cfg->rope_type == ORACLE_ROPE_CHATGLM) {
            oracle_position_ids_glm(1, n_past[i], n_ctx ? n_ctx[i] : n_past[i], ids);
        } else {
            ids[0] = n_past[i];
        }
        float *qi = qr + (long)i * H * D;
        float kr[G * D];
        for (int h = 0; h < H; h++) {
            memcpy(qi + (long)h * D, q[i] + h * q_head_stride, sizeof(float) * D);
        }
        for (int g = 0; g < G; g++) {
            memcpy(kr + (long)g * D, k[i] + g * kv_head_stride, sizeof(float) * D);
        }
        oracle_apply_rotary_emb(cfg, qi, (long)H * D, D, H, 1, ids);
        oracle_apply_rotary_emb(cfg, kr, (long)G * D, D, G, 1, ids);
        const int pos = V + n_past[i];
        for (int g = 0; g < G; g++) {
            for (int d = 0; d < D; d++) {
                k_cache[i][((long)g * M + pos) * D + d] = oracle_f32_to_f16(kr[(long)g * D + d]);
                v_cache[i][((long)g * D + d) * M + pos] = oracle_f32_to_f16(v[i][g * kv_head_stride + d]);
            }
        }
    }
    /* pass 2: scores / softmax / PV per (sequence, q head), scores materialised: chatglm.cpp:686-717 */
#pragma omp parallel
    {
        float *scores = (float *)malloc(sizeof(float) * (size_t)M);
        float *qs = (float *)malloc(sizeof(float) * (size_t)D);
#pragma omp for schedule(dynamic, 1) collapse(2)
        for (int i = 0; i < n_seq; i++) {
            for (int h = 0; h < H; h++) {
                const int g = h / R;
                attend_head(cfg, qr + ((long)i * H + h) * D, 1, n_past[i], k_cache[i] + (long)g * M * D,
                            v_cache[i] + (long)g * D * M, NULL, scores, qs, out[i] + (long)h * D, (long)H * D);
            }
        }
        free(scores);
        free(qs);
    }
    free(qr);
    return 0;
}

/* ---- counter-based synthetic data: the host twin of the library's cglm_synth_fill_* (test infrastructure) --------
 * element first + i of tensor tensor_id under seed = table[splitmix64(seed * C1 + tensor_id * C2 + first + i) >> 48].
 * Integer arithmetic only, so host and device agree bit for bit; the reference has no counterpart (its tests read
 * fixtures from files, chatglm_test.cpp:296-304). */
static inline uint64_t synth_mix(uint64_t z) {
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

void oracle_synth_fill_f16(uint16_t *dst, long long n, unsigned long long seed, unsigned long long tensor_id, long long first,
                           const uint16_t *table) {
    const uint64_t base = (uint64_t)seed * 0x9E3779B97F4A7C15ull + (uint64_t)tensor_id * 0xBF58476D1CE4E5B9ull;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; i++) {
        dst[i] = table[synth_mix(base + (uint64_t)(first + i)) >> 48];
    }
}

void oracle_synth_fill_f32(float *dst, long long n, unsigned long long seed, unsigned long long tensor_id, long long first,
                           const float *table) {
    const uint64_t base = (uint64_t)seed * 0x9E3779B97F4A7C15ull + (uint64_t)tensor_id * 0xBF58476D1CE4E5B9ull;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; i++) {
        dst[i] = table[synth_mix(base + (uint64_t)(first + i)) >> 48];
    }
}

/* ---- Linear (chatglm.cpp:418-426): y = ggml_mul_mat(weight, x) (+ bias), the module either side of the attention path ---
 * x [n_tok][in] f32, weight [out][in] (f32, or f16 bits when w_is_f16), bias [out] or NULL, y [n_tok][out] f32.
 * round_x_f16: ggml's CPU mul_mat against an f16 matrix first converts the activation row to f16 [ggml-recall];
 * products are accumulated in f32. */
void oracle_linear(const float *x, int n_tok, int in, const void *weight, int w_is_f16, const float *bias, int out,
                   int round_x_f16, float *y) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int t = 0; t < n_tok; t++) {
        for (int o = 0; o < out; o++) {
            float acc = 0.f;
            for (int k = 0; k < in; k++) {
                const float w = w_is_f16 ? oracle_f16_to_f32(((const uint16_t *)weight)[(long)o * in + k])
                                         : ((const float *)weight)[(long)o * in + k];
                const float xv = round_x_f16 ? oracle_f16_to_f32(oracle_f32_to_f16(x[(long)t * in + k])) : x[(long)t * in + k];
                acc += w * xv;
            }
            y[(long)t * out + o] = acc + (bias ? bias[o] : 0.f);
        }
    }
}
