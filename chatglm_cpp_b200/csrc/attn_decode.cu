// Fused RoPE + f16 KV append + split-KV decode attention for head_dim 128 (sm_100a).
//
// One launch covers chatglm.cpp:655-717 for a batch of one-token sequences:
//   RoPE on the new q and k (:655-656), f16 append of K row / V^T column at n_past (:668-675),
//   q * 1/sqrt(d) (:686), QK^T over the whole cache (:687), softmax (:709), PV (:711), [h*d] output (:712-717).
// Decode applies no mask (the reference masks only at n_past == 0, :689).
//
// Work decomposition.  The cache of (sequence i, kv head g) is cut into tiles of 64 tokens; all tiles of
// all (i, g) items form one line, and each persistent CTA owns an equal contiguous span of it, so that
// every SM streams the same number of bytes whatever the mix of sequence lengths.  A span crosses item
// boundaries; the part of an item inside one span is a segment.  A segment that is the whole item writes
// the output directly; otherwise it leaves an un-normalised (acc, m, l) partial in scratch memory and the
// CTA that completes the item (an atomic counter per item, no CTA ever waits for another) merges them.
//
// Inside a CTA a producer warp issues TMA tile loads (two 64x64 K boxes, one 128x64 V^T box, 128-byte
// swizzle, no multicast) into a 3-stage ring guarded by mbarriers; four consumer warps take 16 tokens of
// each tile, run QK^T and PV on tensor cores (mma.sync m16n8k16, the <=16 q heads of the kv head are the M
// rows) with a warp-shuffle online softmax.  Both caches are already contraction-contiguous for the B
// operand: K is [token][d] for QK^T and V^T is [d][token] for PV.
#include "common.cuh"

namespace cglm {

unsigned long long g_launch_count = 0;

namespace {

constexpr int kTile = 64;              // tokens per stage
constexpr int kStages = 3;
constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kD = 128;
constexpr int kRows = 16;              // MMA M = q heads per kv head, zero padded
constexpr int kKHalfBytes = kTile * 128;            // one 64-dim half of a K tile: 64 lines of 128 B
constexpr int kVBytes = kD * 128;                   // V^T tile: 128 lines (dims) of 64 tokens
constexpr int kStageBytes = 2 * kKHalfBytes + kVBytes;   // 32 KiB
constexpr int kXchgStride = 132;                    // floats per row of the merge buffer (padded)
constexpr int kQStride = 136;                       // halfs per row of the q tile (272 B, ldmatrix conflict-free)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct __align__(1024) DecodeSmem {
    uint8_t stage[kStages][kStageBytes];
    float xchg[kRows * kXchgStride + 2 * kRows];
    __half q[kRows][kQStride];
    float cs[2][32][2];
    __half newk[kD];
    __half newv[kD];
    int prefix[kDecodeMaxSeqPerLaunch + 1];   // tiles of sequences [0, i), per kv head
    uint64_t full[kStages];
    uint64_t empty[kStages];
    int abort_flag;
    int last_flag;
};

struct Span {
    long long lo, hi;   // tile range of this CTA on the line of all tiles
};

__device__ __forceinline__ long long span_start(long long b, long long total, long long nb) {
    return b * total / nb;
}

// Position on the line -> (sequence, kv head, tile) using the per-sequence prefix of tile counts.
struct ItemPos {
    int seq, g, tile, n_tiles;
    long long item_begin;   // line position of tile 0 of this item
};
__device__ __forceinline__ ItemPos locate(const int *prefix, int n_seq, int G, long long pos) {
    int lo = 0, hi = n_seq - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (static_cast<long long>(prefix[mid]) * G <= pos) lo = mid; else hi = mid - 1;
    }
    ItemPos ip;
    ip.seq = lo;
    ip.n_tiles = prefix[lo + 1] - prefix[lo];
    const long long off = pos - static_cast<long long>(prefix[lo]) * G;
    ip.g = static_cast<int>(off / ip.n_tiles);
    ip.tile = static_cast<int>(off % ip.n_tiles);
    ip.item_begin = pos - ip.tile;
    return ip;
}

__device__ __forceinline__ int attended_len(const SeqDev &sq) {
    return sq.kv_before + ((sq.flags & CGLM_SEQ_NO_APPEND) ? 0 : 1);
}

__global__ void __launch_bounds__(kThreads, 2)
decode_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map, AttnShape sh,
              const SeqDev *__restrict__ seqs, int n_seq, uint16_t *__restrict__ k_base,
              uint16_t *__restrict__ v_base, WsHeader *hdr, int *counters, float *partials) {
    extern __shared__ uint8_t smem_raw[];
    DecodeSmem &sm = *reinterpret_cast<DecodeSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = sh.G, R = sh.R, M = sh.M;

    // ---- tiles per sequence and their prefix sums ------------------------------------------------------
    for (int i = tid; i < n_seq; i += kThreads) {
        sm.prefix[i + 1] = (attended_len(seqs[i]) + kTile - 1) / kTile;
    }
    if (tid == 0) {
        sm.prefix[0] = 0;
        sm.abort_flag = 0;
        sm.last_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], kConsumerWarps);
        }
        fence_mbar_init();
    }
    __syncthreads();
    if (warp == 0) {   // inclusive scan of prefix[1..n_seq], 32 entries per step
        int carry = 0;
        for (int base = 1; base <= n_seq; base += 32) {
            const int idx = base + lane;
            int v = idx <= n_seq ? sm.prefix[idx] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += t;
            }
            if (idx <= n_seq) sm.prefix[idx] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    const long long total = static_cast<long long>(sm.prefix[n_seq]) * G;
    const long long nb = gridDim.x;
    Span span{span_start(blockIdx.x, total, nb), span_start(blockIdx.x + 1, total, nb)};
    if (span.lo >= span.hi) {
        return;
    }

    if (warp == kConsumerWarps) {
        // ================================ producer warp ================================================
        if (lane == 0) {
            tma_prefetch_desc(&k_map);
            tma_prefetch_desc(&v_map);
            long long pos = span.lo;
            unsigned int n = 0;
            while (pos < span.hi) {
                const ItemPos ip = locate(sm.prefix, n_seq, G, pos);
                const int row = seqs[ip.seq].slot * G + ip.g;
                const long long seg_end = min(span.hi, ip.item_begin + ip.n_tiles);
                for (int t = ip.tile; pos < seg_end; ++t, ++pos, ++n) {
                    const int st = n % kStages;
                    mbar_wait_bounded(&sm.empty[st], ((n / kStages) & 1u) ^ 1u, &sm.abort_flag);
                    if (sm.abort_flag) break;
                    uint8_t *dst = sm.stage[st];
                    mbar_arrive_expect_tx(&sm.full[st], kStageBytes);
                    tma_load_3d(dst, &k_map, 0, t * kTile, row, &sm.full[st]);
                    tma_load_3d(dst + kKHalfBytes, &k_map, 64, t * kTile, row, &sm.full[st]);
                    tma_load_2d(dst + 2 * kKHalfBytes, &v_map, t * kTile, row * kD, &sm.full[st]);
                }
                if (sm.abort_flag) break;
            }
        }
    } else {
        // ================================ consumer warps ===============================================
        const int quad_row = lane >> 2, c = lane & 3;
        long long pos = span.lo;
        unsigned int n = 0;
        bool first_segment = true;
        while (pos < span.hi) {
            const ItemPos ip = locate(sm.prefix, n_seq, G, pos);
            const SeqDev sq = seqs[ip.seq];
            const int g = ip.g;
            const int row = sq.slot * G + g;
            const long long item_end = ip.item_begin + ip.n_tiles;
            const long long seg_end = min(span.hi, item_end);
            const int L = attended_len(sq);
            const bool has_last_tile = seg_end == item_end;
            const bool appender = has_last_tile && !(sq.flags & CGLM_SEQ_NO_APPEND);
            const bool whole_item = pos == ip.item_begin && has_last_tile;

            // ---- segment prologue: RoPE, scaled f16 q tile, append ---------------------------------------
            // Every global load of the prologue is issued before the first barrier so that the loads and the
            // cos/sin ladder overlap instead of queueing behind one another.
            const int n_pairs = rope_n_pairs(sh.rope_type, kD);   // 0, 32 (CHATGLM2) or 64 (CHATGLM)
            const int pr = tid & 63;                               // this thread's pair of the head, rows r0 + 2j
            int i0, i1, cs_stream = 0, cs_ladder = 0;
            if (pr < n_pairs) {
                const RopePair rp = rope_pair(sh.rope_type, kD, pr);
                i0 = rp.i0; i1 = rp.i1; cs_stream = rp.stream; cs_ladder = rp.ladder;
            } else {
                const int first_free = sh.rope_type == CGLM_ROPE_CHATGLM2 ? kD / 2 : 0;
                i0 = first_free + 2 * (pr - n_pairs); i1 = i0 + 1;
            }
            const bool k_needed = appender || (has_last_tile && sq.k_roped);
            float qx0[8], qx1[8], kx0 = 0.f, kx1 = 0.f, vx = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int r = (tid >> 6) + 2 * j;
                qx0[j] = qx1[j] = 0.f;
                if (r < R) {
                    const float *src = sq.q + (g * R + r) * sq.q_head_stride;
                    qx0[j] = __ldg(src + i0);
                    qx1[j] = __ldg(src + i1);
                }
            }
            if (k_needed && tid < 64) {
                const float *src = sq.k + g * sq.kv_head_stride;
                kx0 = __ldg(src + i0);
                kx1 = __ldg(src + i1);
            }
            if (appender) {
                vx = __ldg(sq.v + g * sq.kv_head_stride + tid);   // 128 consumer threads, 128 dims
            }
            int pos_id, block_id;
            derive_positions(sq, sh.rope_type, 0, pos_id, block_id);
            named_bar_sync(1, kConsumerThreads);   // previous segment is done with q / cs / newk / newv / xchg
            if (tid < 64 && n_pairs > 0) {
                const int st = tid >> 5;
                if (st == 0 || sh.rope_type == CGLM_ROPE_CHATGLM) {
                    rope_cos_sin(st ? block_id : pos_id, tid & 31, sh.theta_scale, sm.cs[st][tid & 31][0],
                                 sm.cs[st][tid & 31][1]);
                }
            }
            named_bar_sync(1, kConsumerThreads);
            float rc = 1.f, rs = 0.f;
            if (pr < n_pairs) {
                rc = sm.cs[cs_stream][cs_ladder][0];
                rs = sm.cs[cs_stream][cs_ladder][1];
            }
            // q: 16 rows x 64 pairs; rows >= R are zero
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int r = (tid >> 6) + 2 * j;
                float y0 = qx0[j], y1 = qx1[j];
                if (pr < n_pairs) {
                    rope_rotate(qx0[j], qx1[j], rc, rs, y0, y1);
                }
                sm.q[r][i0] = __float2half_rn(__fmul_rn(y0, sh.scale));
                sm.q[r][i1] = __float2half_rn(__fmul_rn(y1, sh.scale));
                if (has_last_tile && sq.q_roped && r < R) {
                    float *qr = sq.q_roped + static_cast<long long>(g * R + r) * kD;
                    qr[i0] = y0; qr[i1] = y1;
                }
            }
            if (k_needed && tid < 64) {
                float y0 = kx0, y1 = kx1;
                if (pr < n_pairs) {
                    rope_rotate(kx0, kx1, rc, rs, y0, y1);
                }
                if (sq.k_roped) {
                    float *kr = sq.k_roped + static_cast<long long>(g) * kD;
                    kr[i0] = y0; kr[i1] = y1;
                }
                if (appender) {
                    const __half h0 = __float2half_rn(y0), h1 = __float2half_rn(y1);
                    sm.newk[i0] = h0; sm.newk[i1] = h1;
                    uint16_t *krow = k_base + (static_cast<long long>(row) * M + sq.kv_before) * kD;
                    krow[i0] = __half_as_ushort(h0);
                    krow[i1] = __half_as_ushort(h1);
                }
            }
            if (appender) {
                const __half hv = __float2half_rn(vx);
                sm.newv[tid] = hv;
                v_base[(static_cast<long long>(row) * kD + tid) * M + sq.kv_before] = __half_as_ushort(hv);
            }
            named_bar_sync(1, kConsumerThreads);
            // A fragments of the q tile: 8 k-steps of 16 dims
            uint32_t qa[8][4];
            {
                const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const int rr = r8 + 8 * (mi & 1);
                    const int col = 16 * ks + 8 * (mi >> 1);
                    ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], smem_u32(&sm.q[rr][col]));
                }
            }

            float o[16][4];
#pragma unroll
            for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
            float m_run[2] = {-INFINITY, -INFINITY};   // rows quad_row and quad_row + 8, log2 domain
            float l_run[2] = {0.f, 0.f};               // this thread's share of the row sums

            // ---- tiles of the segment -------------------------------------------------------------------
            for (int t = ip.tile; pos < seg_end; ++t, ++pos, ++n) {
                const int st = n % kStages;
                mbar_wait_bounded(&sm.full[st], (n / kStages) & 1u, &sm.abort_flag);
                const uint32_t kb = smem_u32(sm.stage[st]);
                const uint32_t vb = kb + 2 * kKHalfBytes;
                const int tok0 = t * kTile + 16 * warp;           // first token of this warp's slice
                const int n_valid = min(16, L - tok0);
                if (n_valid > 0) {
                    if (n_valid < 16 || (appender && t == ip.n_tiles - 1)) {
                        // last tile of the item: splice in the token appended by this call and blank the
                        // V^T columns of tokens beyond the attended length (stale cache contents)
                        const int new_local = appender ? sq.kv_before - tok0 : -1;   // in [0,16) if ours
                        if (new_local >= 0 && new_local < 16) {
                            const int tk = 16 * warp + new_local;
                            const int ch = lane >> 1;   // 16-byte chunk of the 256-byte row
                            const uint32_t addr = kb + (ch >> 3) * kKHalfBytes + tk * 128 +
                                                  (((ch & 7) ^ (tk & 7)) << 4) + (lane & 1) * 8;
                            const uint2 val = *reinterpret_cast<const uint2 *>(&sm.newk[ch * 8 + (lane & 1) * 4]);
                            asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(val.x), "r"(val.y));
                        }
                        for (int d = lane; d < kD; d += 32) {
                            for (int j = (new_local >= 0 && new_local < 16) ? new_local : n_valid; j < 16; ++j) {
                                const int tk = 16 * warp + j;
                                const uint32_t addr = vb + d * 128 + (((tk >> 3) ^ (d & 7)) << 4) + (tk & 7) * 2;
                                const uint16_t hv = j == new_local ? __half_as_ushort(sm.newv[d]) : (uint16_t)0;
                                asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(hv));
                            }
                        }
                        __syncwarp();
                    }
                    // ---- S = Q K^T for 16 tokens: two n-blocks of 8 -------------------------------------
                    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                    {
                        const int mi = lane >> 3, r8 = lane & 7;
                        const int tk = 16 * warp + 8 * (mi >> 1) + r8;
                        const uint32_t rowaddr = kb + tk * 128;
                        const int sw = tk & 7;
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {
                            const int ch = 2 * ks + (mi & 1);
                            uint32_t b0, b1, b2, b3;
                            ldmatrix_x4(b0, b1, b2, b3, rowaddr + (ch >> 3) * kKHalfBytes + (((ch & 7) ^ sw) << 4));
                            mma_m16n8k16(s[0], qa[ks], b0, b1);
                            mma_m16n8k16(s[1], qa[ks], b2, b3);
                        }
                    }
                    // ---- online softmax (log2 domain) ---------------------------------------------------
#pragma unroll
                    for (int nbk = 0; nbk < 2; ++nbk) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = 8 * nbk + 2 * c + (e & 1);
                            s[nbk][e] = j < n_valid ? s[nbk][e] * kLog2e : -INFINITY;
                        }
                    }
                    float mx[2];
                    mx[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
                    mx[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
                    float alpha[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                        const float m_new = fmaxf(m_run[h], mx[h]);
                        alpha[h] = ex2_approx(m_run[h] - m_new);
                        m_run[h] = m_new;
                    }
                    float p[2][4];
#pragma unroll
                    for (int nbk = 0; nbk < 2; ++nbk) {
                        p[nbk][0] = ex2_approx(s[nbk][0] - m_run[0]);
                        p[nbk][1] = ex2_approx(s[nbk][1] - m_run[0]);
                        p[nbk][2] = ex2_approx(s[nbk][2] - m_run[1]);
                        p[nbk][3] = ex2_approx(s[nbk][3] - m_run[1]);
                    }
                    l_run[0] = l_run[0] * alpha[0] + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
                    l_run[1] = l_run[1] * alpha[1] + (p[0][2] + p[0][3] + p[1][2] + p[1][3]);
                    uint32_t pa[4];
                    pa[0] = pack_half2(p[0][0], p[0][1]);
                    pa[1] = pack_half2(p[0][2], p[0][3]);
                    pa[2] = pack_half2(p[1][0], p[1][1]);
                    pa[3] = pack_half2(p[1][2], p[1][3]);
                    // ---- O = O * alpha + P V ------------------------------------------------------------
                    {
                        const int mi = lane >> 3, r8 = lane & 7;
                        const int ch = 2 * warp + (mi & 1);
#pragma unroll
                        for (int ndp = 0; ndp < 8; ++ndp) {
                            const int d = 8 * (2 * ndp + (mi >> 1)) + r8;
                            uint32_t b0, b1, b2, b3;
                            ldmatrix_x4(b0, b1, b2, b3, vb + d * 128 + ((ch ^ (d & 7)) << 4));
                            float(&o0)[4] = o[2 * ndp];
                            float(&o1)[4] = o[2 * ndp + 1];
                            o0[0] *= alpha[0]; o0[1] *= alpha[0]; o0[2] *= alpha[1]; o0[3] *= alpha[1];
                            o1[0] *= alpha[0]; o1[1] *= alpha[0]; o1[2] *= alpha[1]; o1[3] *= alpha[1];
                            mma_m16n8k16(o0, pa, b0, b1);
                            mma_m16n8k16(o1, pa, b2, b3);
                        }
                    }
                    if (n_valid < 16 || (appender && t == ip.n_tiles - 1)) {
                        fence_proxy_async();   // our plain stores into the stage precede its next TMA fill
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&sm.empty[st]);
                }
            }

            // ---- fold the four warps' states into warp 0 ------------------------------------------------
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
                l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
            }
            for (int src = 1; src < kConsumerWarps; ++src) {
                named_bar_sync(1, kConsumerThreads);
                if (warp == src) {
#pragma unroll
                    for (int nd = 0; nd < 16; ++nd) {
                        *reinterpret_cast<float2 *>(&sm.xchg[quad_row * kXchgStride + 8 * nd + 2 * c]) =
                            make_float2(o[nd][0], o[nd][1]);
                        *reinterpret_cast<float2 *>(&sm.xchg[(quad_row + 8) * kXchgStride + 8 * nd + 2 * c]) =
                            make_float2(o[nd][2], o[nd][3]);
                    }
                    if (c == 0) {
                        sm.xchg[kRows * kXchgStride + quad_row] = m_run[0];
                        sm.xchg[kRows * kXchgStride + quad_row + 8] = m_run[1];
                        sm.xchg[kRows * kXchgStride + kRows + quad_row] = l_run[0];
                        sm.xchg[kRows * kXchgStride + kRows + quad_row + 8] = l_run[1];
                    }
                }
                named_bar_sync(1, kConsumerThreads);
                if (warp == 0) {
                    float a_me[2], a_src[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float m_src = sm.xchg[kRows * kXchgStride + quad_row + 8 * h];
                        const float l_src = sm.xchg[kRows * kXchgStride + kRows + quad_row + 8 * h];
                        const float m_new = fmaxf(m_run[h], m_src);
                        a_me[h] = ex2_approx(m_run[h] - m_new);
                        a_src[h] = ex2_approx(m_src - m_new);
                        l_run[h] = l_run[h] * a_me[h] + l_src * a_src[h];
                        m_run[h] = m_new;
                    }
#pragma unroll
                    for (int nd = 0; nd < 16; ++nd) {
                        const float2 lo2 = *reinterpret_cast<const float2 *>(&sm.xchg[quad_row * kXchgStride + 8 * nd + 2 * c]);
                        const float2 hi2 = *reinterpret_cast<const float2 *>(&sm.xchg[(quad_row + 8) * kXchgStride + 8 * nd + 2 * c]);
                        o[nd][0] = o[nd][0] * a_me[0] + lo2.x * a_src[0];
                        o[nd][1] = o[nd][1] * a_me[0] + lo2.y * a_src[0];
                        o[nd][2] = o[nd][2] * a_me[1] + hi2.x * a_src[1];
                        o[nd][3] = o[nd][3] * a_me[1] + hi2.y * a_src[1];
                    }
                }
            }

            // ---- emit: final rows, or a partial plus the completion protocol -----------------------------
            const bool want_partial = (sq.flags & CGLM_SEQ_PARTIAL) != 0;
            if (whole_item) {
                if (warp == 0) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int r = quad_row + 8 * h;
                        if (r < R) {
                            const int head = g * R + r;
                            if (want_partial) {
                                float *pp = sq.partial + static_cast<long long>(head) * (kD + 2);
#pragma unroll
                                for (int nd = 0; nd < 16; ++nd) {
                                    *reinterpret_cast<float2 *>(&pp[8 * nd + 2 * c]) =
                                        make_float2(o[nd][2 * h], o[nd][2 * h + 1]);
                                }
                                if (c == 0) { pp[kD] = m_run[h] * kLn2; pp[kD + 1] = l_run[h]; }
                            } else {
                                const float inv = 1.f / l_run[h];
                                float *op = sq.out + static_cast<long long>(head) * kD;
#pragma unroll
                                for (int nd = 0; nd < 16; ++nd) {
                                    *reinterpret_cast<float2 *>(&op[8 * nd + 2 * c]) =
                                        make_float2(o[nd][2 * h] * inv, o[nd][2 * h + 1] * inv);
                                }
                            }
                        }
                    }
                }
            } else {
                // CTAs b0..b1 hold parts of this item
                long long b0 = ip.item_begin * nb / total;
                while (span_start(b0 + 1, total, nb) <= ip.item_begin) ++b0;
                long long b1 = (item_end - 1) * nb / total;
                while (span_start(b1 + 1, total, nb) <= item_end - 1) ++b1;
                const int n_parts = static_cast<int>(b1 - b0 + 1);
                const int item = ip.seq * G + g;
                if (warp == 0) {
                    float *pp = partials + (static_cast<long long>(blockIdx.x) * 2 + (first_segment ? 0 : 1)) * kDecodePartialFloats;
#pragma unroll
                    for (int nd = 0; nd < 16; ++nd) {
                        __stcg(reinterpret_cast<float2 *>(&pp[quad_row * kD + 8 * nd + 2 * c]), make_float2(o[nd][0], o[nd][1]));
                        __stcg(reinterpret_cast<float2 *>(&pp[(quad_row + 8) * kD + 8 * nd + 2 * c]), make_float2(o[nd][2], o[nd][3]));
                    }
                    if (c == 0) {
                        __stcg(&pp[kRows * kD + quad_row], m_run[0]);
                        __stcg(&pp[kRows * kD + quad_row + 8], m_run[1]);
                        __stcg(&pp[kRows * kD + kRows + quad_row], l_run[0]);
                        __stcg(&pp[kRows * kD + kRows + quad_row + 8], l_run[1]);
                    }
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) {
                        const int old = atomicAdd(&counters[item], 1);
                        const int last = old == n_parts - 1;
                        if (last) {
                            atomicExch(&counters[item], 0);   // ready for the next launch
                        }
                        sm.last_flag = last;
                    }
                }
                named_bar_sync(1, kConsumerThreads);
                if (sm.last_flag) {
                    __threadfence();
                    // thread (r, c8) merges 16 dims of row r over all parts; loads are issued in batches so that
                    // L2 round trips overlap instead of adding up
                    const int r = tid >> 3, d0 = (tid & 7) * 16;
                    if (r < R) {
                        auto part_ptr = [&](long long b) -> const float * {
                            const int slot = span_start(b, total, nb) >= ip.item_begin ? 0 : 1;
                            return partials + (b * 2 + slot) * kDecodePartialFloats;
                        };
                        float m_star = -INFINITY;
                        for (long long b = b0; b <= b1; b += 8) {
                            float mv[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                mv[u] = b + u <= b1 ? __ldcg(part_ptr(b + u) + kRows * kD + r) : -INFINITY;
                            }
#pragma unroll
                            for (int u = 0; u < 8; ++u) m_star = fmaxf(m_star, mv[u]);
                        }
                        float acc[16];
#pragma unroll
                        for (int e = 0; e < 16; ++e) acc[e] = 0.f;
                        float den = 0.f;
                        for (long long b = b0; b <= b1; b += 4) {
                            float mv[4], lv[4];
                            float4 av[4][4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const bool ok = b + u <= b1;
                                const float *pp = part_ptr(ok ? b + u : b);
                                mv[u] = ok ? __ldcg(pp + kRows * kD + r) : -INFINITY;
                                lv[u] = __ldcg(pp + kRows * kD + kRows + r);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    av[u][e] = __ldcg(reinterpret_cast<const float4 *>(pp + r * kD + d0) + e);
                                }
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const float w = ex2_approx(mv[u] - m_star);   // 0 for the padding entries
                                den += w * lv[u];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    acc[4 * e + 0] += w * av[u][e].x; acc[4 * e + 1] += w * av[u][e].y;
                                    acc[4 * e + 2] += w * av[u][e].z; acc[4 * e + 3] += w * av[u][e].w;
                                }
                            }
                        }
                        const int head = g * R + r;
                        if (want_partial) {
                            float *po = sq.partial + static_cast<long long>(head) * (kD + 2);
#pragma unroll
                            for (int e = 0; e < 16; ++e) po[d0 + e] = acc[e];   // row stride 130 floats: not 16-byte aligned
                            if (d0 == 0) { po[kD] = m_star * kLn2; po[kD + 1] = den; }
                        } else {
                            const float inv = 1.f / den;
                            float4 *op = reinterpret_cast<float4 *>(sq.out + static_cast<long long>(head) * kD + d0);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                op[e] = make_float4(acc[4 * e] * inv, acc[4 * e + 1] * inv, acc[4 * e + 2] * inv,
                                                    acc[4 * e + 3] * inv);
                            }
                        }
                    }
                }
            }
            first_segment = false;
        }
    }
    if (sm.abort_flag && (tid == 0 || tid == kConsumerThreads)) {
        atomicExch(&hdr->status, static_cast<int>(CGLM_ERR_TIMEOUT));
    }
}

}  // namespace

int decode_max_ctas(int n_sm) { return 2 * n_sm; }

cudaError_t launch_decode(const LaunchCtx &cx, const SeqDev *seqs_dev, int n_seq, long long total_tiles) {
    if (n_seq == 0 || total_tiles == 0) {
        return cudaSuccess;
    }
    static bool configured = false;
    const int smem_bytes = static_cast<int>(sizeof(DecodeSmem)) + 1024;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const long long max_ctas = decode_max_ctas(cx.n_sm);
    const int grid = static_cast<int>(total_tiles < max_ctas ? total_tiles : max_ctas);
    decode_kernel<<<grid, kThreads, smem_bytes, cx.stream>>>(*cx.k_map, *cx.v_map, cx.shape, seqs_dev, n_seq, cx.k_base,
                                                            cx.v_base, cx.hdr, cx.counters, cx.partials);
    g_launch_count += 1;
    return cudaGetLastError();
}

}  // namespace cglm
