// Generic CUDA path of the attention KV-cache step: any head_dim <= 256, any cache capacity, prefill and
// decode, every rope and mask mode.  It covers the shapes the specialised kernels do not (the reference's
// head_dim-4 test models, P-Tuning capacities that are not a multiple of 8, more than 16 q heads per kv
// head) with plain loads and CUDA-core math.
//
//   rope_append_kernel : chatglm.cpp:655-656 (RoPE on q and k) + :668-675 (f16 append, V transposed)
//                        + :686 (q * 1/sqrt(d)), q staged in f32
//   attend_kernel      : chatglm.cpp:687-717 (QK^T, mask at n_past == 0, softmax, PV, [s, h*d] output)
#include "common.cuh"

namespace cglm {

namespace {

constexpr int kRopeThreads = 128;
constexpr int kMaxHeadDim = 256;

// One CTA per (sequence, token).  cos/sin of the token's angle ladders are computed once into shared
// memory, then every (head, pair) is rotated by one thread.
__global__ void __launch_bounds__(kRopeThreads)
rope_append_kernel(AttnShape sh, const SeqDev *__restrict__ seqs, int n_seq, uint16_t *__restrict__ k_base,
                   uint16_t *__restrict__ v_base, float *__restrict__ q_stage) {
    __shared__ float cs[2][kMaxHeadDim / 2][2];   // [stream][ladder index][cos, sin]
    __shared__ int s_seq, s_tok;
    if (threadIdx.x == 0) {
        // blockIdx.x is a global token index; find its sequence (sequences are few, tokens many)
        int lo = 0, hi = n_seq - 1;
        const int t = blockIdx.x;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (seqs[mid].tok_begin <= t) lo = mid; else hi = mid - 1;
        }
        s_seq = lo;
        s_tok = t - seqs[lo].tok_begin;
    }
    __syncthreads();
    const SeqDev sq = seqs[s_seq];
    const int s = s_tok;
    const int D = sh.D, H = sh.H, G = sh.G, M = sh.M;
    const int n_pairs = (sq.flags & CGLM_SEQ_Q_ROPED) ? 0 : rope_n_pairs(sh.rope_type, D);
    const int ladder_len = rope_n_dims(sh.rope_type, D) / 2;

    int pos, block;
    derive_positions(sq, sh.rope_type, s, pos, block);
    const int n_streams = sh.rope_type == CGLM_ROPE_CHATGLM ? 2 : 1;
    if (n_pairs > 0) {
        for (int i = threadIdx.x; i < n_streams * ladder_len; i += blockDim.x) {
            const int st = i / ladder_len, li = i % ladder_len;
            rope_cos_sin(st ? block : pos, li, sh.theta_scale, cs[st][li][0], cs[st][li][1]);
        }
    }
    __syncthreads();

    const int cache_pos = sq.kv_before + s;
    const bool do_append = !(sq.flags & CGLM_SEQ_NO_APPEND);
    const bool in_f16 = (sq.flags & CGLM_SEQ_QKV_F16) != 0;
    const int half_pairs = D / 2;   // every head is walked as D/2 (i0, i1) pairs, rotated or not
    // q heads then k heads
    for (int idx = threadIdx.x; idx < (H + G) * half_pairs; idx += blockDim.x) {
        const int head = idx / half_pairs, p = idx % half_pairs;
        const bool is_q = head < H;
        const int hh = is_q ? head : head - H;
        const float *base = is_q ? sq.q : sq.k;
        const long long row = is_q ? s * sq.q_tok_stride + hh * sq.q_head_stride : s * sq.kv_tok_stride + hh * sq.kv_head_stride;
        int i0, i1;
        float y0, y1;
        if (p < n_pairs) {
            const RopePair rp = rope_pair(sh.rope_type, D, p);
            i0 = rp.i0; i1 = rp.i1;
            rope_rotate(ld_act(base, row + i0, in_f16), ld_act(base, row + i1, in_f16), cs[rp.stream][rp.ladder][0],
                        cs[rp.stream][rp.ladder][1], y0, y1);
        } else {
            // elements no pair rotates: for CHATGLM2 the second half of the head, for DISABLED all of it
            const int first_free = sh.rope_type == CGLM_ROPE_CHATGLM2 ? D / 2 : 0;
            i0 = first_free + 2 * (p - n_pairs); i1 = i0 + 1;
            y0 = ld_act(base, row + i0, in_f16); y1 = ld_act(base, row + i1, in_f16);
        }
        if (is_q) {
            float *dst = q_stage + (static_cast<long long>(sq.tok_begin + s) * H + hh) * D;
            dst[i0] = __fmul_rn(y0, sh.scale);
            dst[i1] = __fmul_rn(y1, sh.scale);
            if (sq.q_roped) {
                float *qr = sq.q_roped + (static_cast<long long>(s) * H + hh) * D;
                qr[i0] = y0; qr[i1] = y1;
            }
        } else {
            if (do_append) {
                uint16_t *krow = k_base + (static_cast<long long>(sq.slot * G + hh) * M + cache_pos) * D;
                krow[i0] = __half_as_ushort(__float2half_rn(y0));
                krow[i1] = __half_as_ushort(__float2half_rn(y1));
            }
            if (sq.k_roped) {
                float *kr = sq.k_roped + (static_cast<long long>(s) * G + hh) * D;
                kr[i0] = y0; kr[i1] = y1;
            }
        }
    }
    if (do_append) {
        for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
            const int g = idx / D, d = idx % D;
            const float x = ld_act(sq.v, s * sq.kv_tok_stride + g * sq.kv_head_stride + d, in_f16);
            v_base[(static_cast<long long>(sq.slot * G + g) * D + d) * M + cache_pos] =
                __half_as_ushort(__float2half_rn(x));
        }
    }
}

constexpr int kAttendWarps = 4;

// One warp per (token, q head).  Tokens of the cache are walked 32 at a time: lane j scores token j,
// the warp updates the running max / sum, then lane d accumulates dims d, d+32, ... of P.V.
__global__ void __launch_bounds__(kAttendWarps * 32)
attend_kernel(AttnShape sh, const SeqDev *__restrict__ seqs, int n_seq, int total_rows,
              const uint16_t *__restrict__ k_base, const uint16_t *__restrict__ v_base,
              const float *__restrict__ q_stage) {
    __shared__ float q_sm[kAttendWarps][kMaxHeadDim];
    __shared__ float p_sm[kAttendWarps][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kAttendWarps + warp;   // (global token, head)
    if (row >= total_rows) {
        return;
    }
    const int H = sh.H, D = sh.D, M = sh.M;
    const int tok = row / H, h = row % H;
    int lo = 0, hi = n_seq - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (seqs[mid].tok_begin <= tok) lo = mid; else hi = mid - 1;
    }
    const SeqDev sq = seqs[lo];
    const int s = tok - sq.tok_begin;
    const int g = h / sh.R;
    const int L = sq.kv_before + ((sq.flags & CGLM_SEQ_NO_APPEND) ? 0 : sq.qlen);
    // visible prefix of this row: masks exist only at n_past == 0 (chatglm.cpp:689-707)
    int vis = L;
    if (sq.n_past == 0 && !(sq.flags & CGLM_SEQ_USE_KV_LOCAL)) {
        if (sh.mask_type == CGLM_MASK_CAUSAL) {
            vis = sh.V + s + 1;                       // ggml_diag_mask_inf(n_past = V): j > V + s is masked
        } else if (s < sq.qlen - 1) {
            vis = L - 1;                              // every row but the last is blocked from the last column
        }
    }
    for (int d = lane; d < D; d += 32) {
        q_sm[warp][d] = q_stage[(static_cast<long long>(tok) * H + h) * D + d];
    }
    __syncwarp();
    const uint16_t *kc = k_base + static_cast<long long>(sq.slot * sh.G + g) * M * D;
    const uint16_t *vc = v_base + static_cast<long long>(sq.slot * sh.G + g) * D * M;

    float m_run = -INFINITY, l_run = 0.f;
    float acc[kMaxHeadDim / 32];
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.f;

    for (int j0 = 0; j0 < vis; j0 += 32) {
        const int j = j0 + lane;
        float sc = -INFINITY;
        if (j < vis) {
            const __half2 *kr = reinterpret_cast<const __half2 *>(kc + static_cast<long long>(j) * D);
            float a = 0.f;
            for (int d2 = 0; d2 < D / 2; ++d2) {
                const float2 kv = __half22float2(kr[d2]);
                a = fmaf(kv.x, q_sm[warp][2 * d2], a);
                a = fmaf(kv.y, q_sm[warp][2 * d2 + 1], a);
            }
            sc = a;
        }
        float mx = sc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m_run, mx);
        const float alpha = __expf(m_run - m_new);   // 0 on the first chunk (m_run = -inf)
        const float p = j < vis ? __expf(sc - m_new) : 0.f;
        float ps = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l_run = l_run * alpha + ps;
        m_run = m_new;
        const int n_here = min(32, vis - j0);
        p_sm[warp][lane] = p;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < kMaxHeadDim / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < D) {
                float a = acc[i] * alpha;
                const uint16_t *vr = vc + static_cast<long long>(d) * M + j0;
                for (int jj = 0; jj < n_here; ++jj) {
                    a = fmaf(__half2float(__ushort_as_half(vr[jj])), p_sm[warp][jj], a);
                }
                acc[i] = a;
            }
        }
        __syncwarp();
    }
    if (sq.flags & CGLM_SEQ_PARTIAL) {
        float *pp = sq.partial + static_cast<long long>(h) * (D + 2);
#pragma unroll
        for (int i = 0; i < kMaxHeadDim / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < D) pp[d] = acc[i];
        }
        if (lane == 0) { pp[D] = m_run; pp[D + 1] = l_run; }
    } else {
        const float inv = 1.f / l_run;
        const long long o = (static_cast<long long>(s) * H + h) * D;
        const bool out_f16 = (sq.flags & CGLM_SEQ_OUT_F16) != 0;
#pragma unroll
        for (int i = 0; i < kMaxHeadDim / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < D) st_out(sq.out, o + d, out_f16, acc[i] * inv);
        }
    }
}

}  // namespace

cudaError_t launch_generic(const LaunchCtx &cx, const SeqDev *seqs_dev, int n_seq, int total_tokens) {
    if (n_seq == 0 || total_tokens == 0) {
        return cudaSuccess;
    }
    rope_append_kernel<<<total_tokens, kRopeThreads, 0, cx.stream>>>(cx.shape, seqs_dev, n_seq, cx.k_base,
                                                                     cx.v_base, cx.q_stage);
    const int rows = total_tokens * cx.shape.H;
    attend_kernel<<<(rows + kAttendWarps - 1) / kAttendWarps, kAttendWarps * 32, 0, cx.stream>>>(
        cx.shape, seqs_dev, n_seq, rows, cx.k_base, cx.v_base, cx.q_stage);
    g_launch_count += 2;
    return cudaGetLastError();
}

}  // namespace cglm
