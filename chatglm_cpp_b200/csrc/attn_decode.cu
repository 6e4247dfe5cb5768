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
// the output directly; otherwise it leaves an un-normalised (acc, m, l) partial in scratch memory and the CTA
// that completes the item (an atomic counter per item; no CTA ever waits for another) merges the partials.
//
// Inside a CTA (six warps):
//   producer warp   issues the TMA tile loads (two 64x64 K boxes, one 128x64 V^T box, 128-byte swizzle, no
//                   multicast) into a 3-stage ring guarded by mbarriers, running ahead across segments;
//   helper warp     prepares the NEXT segment while the consumers stream the current one (RoPE of q and of
//                   the new k, the scaled f16 q tile, the f16 append into the cache) and finishes the PREVIOUS
//                   one (completion counter, merge of a split item), so that a segment switch costs the
//                   consumers no global-memory round trip;
//   4 consumer warps take 16 tokens of each tile, run QK^T and PV on tensor cores (mma.sync m16n8k16, the
//                   <=16 q heads of the kv head are the M rows) with a warp-shuffle online softmax.
// Both caches are already contraction-contiguous for the B operand: K is [token][d] for QK^T and V^T is
// [d][token] for PV.
#include "common.cuh"

namespace cglm {

unsigned long long g_launch_count = 0;

namespace {

constexpr int kTile = kDecodeTile;     // tokens per stage
constexpr int kStages = 3;
constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kProducerWarp = kConsumerWarps;
constexpr int kHelperWarp = kConsumerWarps + 1;
constexpr int kThreads = (kConsumerWarps + 2) * 32;
constexpr int kD = 128;
constexpr int kRows = 16;              // MMA M = q heads per kv head, zero padded
constexpr int kKHalfBytes = kTile * 128;            // one 64-dim half of a K tile: 64 lines of 128 B
constexpr int kVBytes = kD * 128;                   // V^T tile: 128 lines (dims) of 64 tokens
constexpr int kStageBytes = 2 * kKHalfBytes + kVBytes;   // 32 KiB
constexpr int kXchgStride = 68;                     // floats per row of the fold buffer (64 dims + pad)
constexpr int kQStride = 136;                       // halfs per row of the q tile (272 B, ldmatrix conflict-free)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// What the helper warp hands to the consumers for one segment.
struct alignas(16) QBuf {
    __half q[kRows][kQStride];   // roped, scaled q heads of the kv head (rows >= R zero)
    __half newk[kD];             // f16 of the roped k appended by this call
    __half newv[kD];             // f16 of the v appended by this call
    float *out;                  // the sequence's output row / partial row, attended length inputs
    float *partial;
    int kv_before;
    int flags;
};

struct __align__(1024) DecodeSmem {
    uint8_t stage[kStages][kStageBytes];
    QBuf qb[2];
    float xchg[kRows * kXchgStride + 2 * kRows];   // fold buffer: one 64-dim half of a warp's O, its m and l
    int prefix[kDecodeMaxSeqPerLaunch + 2];        // copy of the launch's tile prefix sums (parameter space is slow to index)
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t qfull[2];
    uint64_t qempty[2];
    uint64_t hstart;                               // helper -> producer: the first segment's loads are on their way
    int last_flag;                                 // end-of-span partial: this CTA completed the item
    uint64_t pdone[2];                             // consumers -> helper: partial 0 / 1 of this CTA is in scratch
    int abort_flag;
};

static_assert(sizeof(QBuf) % 16 == 0, "ldmatrix rows of the second q tile stay 16-byte aligned");
// two CTAs per SM: 2 * (dynamic shared memory + 1 KiB alignment slack + 1 KiB reserved per CTA) <= 228 KiB
static_assert(2 * (sizeof(DecodeSmem) + 2048) <= 233472, "two decode CTAs must fit one SM");

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

__device__ __forceinline__ int attended_len(int kv_before, int flags) {
    return kv_before + ((flags & CGLM_SEQ_NO_APPEND) ? 0 : 1);
}

// CTAs b0..b1 of an nb-CTA launch hold parts of the item spanning [item_begin, item_end) on the line.
__device__ __forceinline__ void item_ctas(long long item_begin, long long item_end, long long total, long long nb,
                                          long long &b0, long long &b1) {
    b0 = item_begin * nb / total;
    while (span_start(b0 + 1, total, nb) <= item_begin) ++b0;
    b1 = (item_end - 1) * nb / total;
    while (span_start(b1 + 1, total, nb) <= item_end - 1) ++b1;
}
// A CTA keeps at most two partials: slot 0 for its first segment, slot 1 for its last.
__device__ __forceinline__ const float *part_ptr(const float *partials, long long b, long long item_begin,
                                                 long long total, long long nb) {
    const int slot = span_start(b, total, nb) >= item_begin ? 0 : 1;
    return partials + (b * 2 + slot) * kDecodePartialFloats;
}

// ---- per-warp tile math ---------------------------------------------------------------------------------
// A consumer warp owns 16 tokens of every 64-token tile: tokens 16*warp .. 16*warp+15.

// S[16 q rows][16 tokens] = Q K^T as two n-blocks of 8 tokens; kb = shared address of the stage's K halves.
__device__ __forceinline__ void qk_slice(uint32_t kb, int warp, int lane, const uint32_t (&qa)[8][4], float (&s)[2][4]) {
    const int mi = lane >> 3, r8 = lane & 7;
    const int tk = 16 * warp + 8 * (mi >> 1) + r8;
    const uint32_t rowaddr = kb + tk * 128;
    const int sw = tk & 7;
#pragma unroll
    for (int e = 0; e < 4; ++e) { s[0][e] = 0.f; s[1][e] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const int ch = 2 * ks + (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, rowaddr + (ch >> 3) * kKHalfBytes + (((ch & 7) ^ sw) << 4));
        mma_m16n8k16(s[0], qa[ks], b0, b1);
        mma_m16n8k16(s[1], qa[ks], b2, b3);
    }
}

// Online softmax over the slice's 16 scores per row (log2 domain) and O = O * alpha + P V.
// kFull: all 16 tokens are attended (every tile but an item's last).
template <bool kFull>
__device__ __forceinline__ void softmax_pv_slice(uint32_t vb, int warp, int lane, int n_valid, float (&s)[2][4],
                                                 float (&m_run)[2], float (&l_run)[2], float (&o)[16][4]) {
    const int c = lane & 3;
#pragma unroll
    for (int nbk = 0; nbk < 2; ++nbk) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = 8 * nbk + 2 * c + (e & 1);
            s[nbk][e] = (kFull || j < n_valid) ? s[nbk][e] * kLog2e : -INFINITY;
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

// Last tile of an item: splice in the token appended by this call (new_local = its index inside this warp's
// slice, or outside [0,16)) and blank the V^T columns of tokens past the attended length, whose cache contents
// are stale.  Plain stores into a TMA-filled stage, so a proxy fence follows.
__device__ __forceinline__ void patch_last_tile(uint32_t kb, uint32_t vb, int warp, int lane, int n_valid, int new_local,
                                                const __half *newk, const __half *newv) {
    const bool ours = new_local >= 0 && new_local < 16;
    if (ours) {
        const int tk = 16 * warp + new_local;
        const int ch = lane >> 1;   // 16-byte chunk of the 256-byte row
        const uint32_t addr = kb + (ch >> 3) * kKHalfBytes + tk * 128 + (((ch & 7) ^ (tk & 7)) << 4) + (lane & 1) * 8;
        const uint2 val = *reinterpret_cast<const uint2 *>(&newk[ch * 8 + (lane & 1) * 4]);
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(val.x), "r"(val.y) : "memory");
    }
    for (int d = lane; d < kD; d += 32) {
        for (int j = ours ? new_local : n_valid; j < 16; ++j) {
            const int tk = 16 * warp + j;
            const uint32_t addr = vb + d * 128 + (((tk >> 3) ^ (d & 7)) << 4) + (tk & 7) * 2;
            const uint16_t hv = j == new_local ? __half_as_ushort(newv[d]) : (uint16_t)0;
            asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(hv) : "memory");
        }
    }
    fence_proxy_async();
    __syncwarp();
}

// ---- helper warp: everything a segment needs before its first tile -----------------------------------------
// RoPE on the 16 q heads of the kv head and on the new k (chatglm.cpp:655-656), q * 1/sqrt(d) in f16
// (chatglm.cpp:686), and, when the segment holds the item's last tile, the f16 append of K row and V^T column
// (chatglm.cpp:668-675).  One warp: lane l owns pairs l and l+32 of every head.
__device__ __forceinline__ void prepare_segment(QBuf &qb, const AttnShape &sh, const SeqDev &sq, int g,
                                                int row, bool has_last_tile, bool appender, int lane,
                                                uint16_t *__restrict__ k_base, uint16_t *__restrict__ v_base,
                                                uint64_t *loads_issued) {
    const int R = sh.R, M = sh.M;
    const int n_pairs = rope_n_pairs(sh.rope_type, kD);   // 0, 32 (CHATGLM2) or 64 (CHATGLM)
    if (lane == 0) {
        qb.out = sq.out; qb.partial = sq.partial; qb.kv_before = sq.kv_before; qb.flags = sq.flags;
    }
    const bool k_needed = appender || (has_last_tile && sq.k_roped);
    // element indices of this lane's two pairs
    int i0[2], i1[2];
    bool rotated[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int pr = lane + 32 * half;   // pair index inside the head
        rotated[half] = pr < n_pairs;
        if (rotated[half]) {
            const RopePair rp = rope_pair(sh.rope_type, kD, pr);   // rp.ladder == lane, rp.stream == half
            i0[half] = rp.i0; i1[half] = rp.i1;
        } else {
            const int first_free = sh.rope_type == CGLM_ROPE_CHATGLM2 ? kD / 2 : 0;
            i0[half] = first_free + 2 * (pr - n_pairs); i1[half] = i0[half] + 1;
        }
    }
    // every global load of the segment is issued before anything depends on one: a single round trip
    float x0[2][kRows], x1[2][kRows], kx0[2] = {0.f, 0.f}, kx1[2] = {0.f, 0.f}, vx[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            x0[half][r] = x1[half][r] = 0.f;
            if (r < R) {
                const float *src = sq.q + (g * R + r) * sq.q_head_stride;
                x0[half][r] = __ldg(src + i0[half]);
                x1[half][r] = __ldg(src + i1[half]);
            }
        }
        if (k_needed) {
            const float *src = sq.k + g * sq.kv_head_stride;
            kx0[half] = __ldg(src + i0[half]);
            kx1[half] = __ldg(src + i1[half]);
        }
    }
    if (appender) {
#pragma unroll
        for (int j = 0; j < 4; ++j) vx[j] = __ldg(sq.v + g * sq.kv_head_stride + lane + 32 * j);
    }
    if (loads_issued) {   // first segment of the CTA: only now may the producer start its burst of tile loads,
        __syncwarp();     // so that these few small loads do not queue behind 96 KiB of them
        if (lane == 0) mbar_arrive(loads_issued);
    }
    // In both GLM modes pair l and pair l+32 of a head use ladder index l (of the position stream for the first,
    // of the block-position stream for the second), so every lane needs only its own cos/sin.
    int pos_id, block_id;
    derive_positions(sq, sh.rope_type, 0, pos_id, block_id);
    float cs_c[2] = {1.f, 1.f}, cs_s[2] = {0.f, 0.f};
    if (n_pairs > 0) {
        rope_cos_sin(pos_id, lane, sh.theta_scale, cs_c[0], cs_s[0]);
        if (sh.rope_type == CGLM_ROPE_CHATGLM) {
            rope_cos_sin(block_id, lane, sh.theta_scale, cs_c[1], cs_s[1]);
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const float rc = cs_c[half], rs = cs_s[half];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            float y0 = x0[half][r], y1 = x1[half][r];
            if (rotated[half]) rope_rotate(x0[half][r], x1[half][r], rc, rs, y0, y1);
            qb.q[r][i0[half]] = __float2half_rn(__fmul_rn(y0, sh.scale));
            qb.q[r][i1[half]] = __float2half_rn(__fmul_rn(y1, sh.scale));
            if (has_last_tile && sq.q_roped && r < R) {
                float *qr = sq.q_roped + static_cast<long long>(g * R + r) * kD;
                qr[i0[half]] = y0; qr[i1[half]] = y1;
            }
        }
        if (k_needed) {
            float y0 = kx0[half], y1 = kx1[half];
            if (rotated[half]) rope_rotate(kx0[half], kx1[half], rc, rs, y0, y1);
            if (sq.k_roped) {
                float *kr = sq.k_roped + static_cast<long long>(g) * kD;
                kr[i0[half]] = y0; kr[i1[half]] = y1;
            }
            if (appender) {
                const __half h0 = __float2half_rn(y0), h1 = __float2half_rn(y1);
                qb.newk[i0[half]] = h0; qb.newk[i1[half]] = h1;
                uint16_t *krow = k_base + (static_cast<long long>(row) * M + sq.kv_before) * kD;
                krow[i0[half]] = __half_as_ushort(h0);
                krow[i1[half]] = __half_as_ushort(h1);
            }
        }
    }
    if (appender) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int d = lane + 32 * j;
            const __half hv = __float2half_rn(vx[j]);
            qb.newv[d] = hv;
            v_base[(static_cast<long long>(row) * kD + d) * M + sq.kv_before] = __half_as_ushort(hv);
        }
    }
}

// ---- completion of split items ------------------------------------------------------------------------------
// An item cut across CTAs is completed by whichever CTA delivers its last part (atomic counters, nobody waits).
// Items of up to kMergeFan parts are merged in one step.  Longer ones (one very long sequence covers hundreds of
// CTAs) go through a two-level tree so that no thread walks hundreds of parts one batch after another: CTAs are
// grouped kMergeFan at a time by their index; the last CTA of a group to finish merges the item's parts inside the
// group into a group partial, and the last group to finish merges the group partials.
constexpr int kMergeFan = kDecodeMergeFan;

struct MergeCtx {
    long long total, nb;   // tiles on the line, CTAs of the launch
    int *counters;         // per item: parts delivered (short items) or groups delivered (long items)
    int *gcounters;        // per (CTA group, slot): parts of the long item in that slot delivered
    float *partials;       // per (CTA, slot)
    float *gpartials;      // per (CTA group, slot)
};
// A CTA group holds parts of at most two long items: one that began in an earlier group (slot 0) and one that
// begins inside the group (slot 1).
__device__ __forceinline__ int group_slot(long long grp, long long b0) { return b0 < grp * kMergeFan ? 0 : 1; }

// 16 dims of one q row merged over sources k0..k1 in one pass with a running maximum, four sources in flight at a
// time.  Sources are CTA partials (level 0) or group partials (level 1).  Every caller goes through this routine
// with the same source order, so the result does not depend on which CTA or warp happens to complete the item.
// to_group >= 0: the result is itself a group partial (un-normalised); otherwise it is the item's output.
__device__ __forceinline__ void merge_row_chunk(const ItemPos &ip, const SeqDev &sq, const AttnShape &sh, const MergeCtx &mc,
                                                bool from_groups, long long b0, long long k0, long long k1, long long to_group,
                                                int r, int d0) {
    auto source = [&](long long k) -> const float * {
        return from_groups ? mc.gpartials + (k * 2 + group_slot(k, b0)) * kDecodePartialFloats
                           : part_ptr(mc.partials, k, ip.item_begin, mc.total, mc.nb);
    };
    float m_run = -INFINITY, den = 0.f;
    float acc[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) acc[e] = 0.f;
    for (long long k = k0; k <= k1; k += 4) {
        float mv[4], lv[4];
        float4 av[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const bool ok = k + u <= k1;
            const float *pp = source(ok ? k + u : k);
            mv[u] = ok ? __ldcg(pp + kRows * kD + r) : -INFINITY;
            lv[u] = __ldcg(pp + kRows * kD + kRows + r);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                av[u][e] = __ldcg(reinterpret_cast<const float4 *>(pp + r * kD + d0) + e);
            }
        }
        const float m_new = fmaxf(fmaxf(m_run, fmaxf(mv[0], mv[1])), fmaxf(mv[2], mv[3]));
        const float keep = ex2_approx(m_run - m_new);   // 0 on the first batch
        den *= keep;
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[e] *= keep;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float w = ex2_approx(mv[u] - m_new);   // 0 for the padding entries
            den += w * lv[u];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[4 * e + 0] += w * av[u][e].x; acc[4 * e + 1] += w * av[u][e].y;
                acc[4 * e + 2] += w * av[u][e].z; acc[4 * e + 3] += w * av[u][e].w;
            }
        }
        m_run = m_new;
    }
    const int head = ip.g * sh.R + r;
    if (to_group >= 0) {
        float *gp = mc.gpartials + (to_group * 2 + group_slot(to_group, b0)) * kDecodePartialFloats;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __stcg(reinterpret_cast<float4 *>(gp + r * kD + d0) + e,
                   make_float4(acc[4 * e], acc[4 * e + 1], acc[4 * e + 2], acc[4 * e + 3]));
        }
        if (d0 == 0) { __stcg(gp + kRows * kD + r, m_run); __stcg(gp + kRows * kD + kRows + r, den); }
    } else if (sq.flags & CGLM_SEQ_PARTIAL) {
        float *po = sq.partial + static_cast<long long>(head) * (kD + 2);   // row stride 130 floats: scalar stores
#pragma unroll
        for (int e = 0; e < 16; ++e) po[d0 + e] = acc[e];
        if (d0 == 0) { po[kD] = m_run * kLn2; po[kD + 1] = den; }
    } else {
        const float inv = 1.f / den;
        float4 *op = reinterpret_cast<float4 *>(sq.out + static_cast<long long>(head) * kD + d0);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            op[e] = make_float4(acc[4 * e] * inv, acc[4 * e + 1] * inv, acc[4 * e + 2] * inv, acc[4 * e + 3] * inv);
        }
    }
}

__device__ __forceinline__ int count_part(int *ctr, int expected) {
    int old;   // release: this CTA's partial stores; acquire: the other CTAs'
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(ctr) : "memory");
    const int last = old == expected - 1;
    if (last) atomicExch(ctr, 0);   // ready for the next launch
    return last;
}

// Called by a team of n_thr threads (the four consumer warps at the end of a span, or the helper warp in the
// middle of one) after CTA `b` stored its part of item `ip`.  t: index inside the team; lead(f): synchronises the
// team (ordering its memory operations), lets the team leader evaluate f() and hands the result to every member.
template <class Lead>
__device__ __forceinline__ void deliver_part(const ItemPos &ip, const SeqDev &sq, const AttnShape &sh, const MergeCtx &mc,
                                             long long b, int t, int n_thr, Lead lead) {
    long long b0, b1;
    item_ctas(ip.item_begin, ip.item_begin + ip.n_tiles, mc.total, mc.nb, b0, b1);
    const int n_parts = static_cast<int>(b1 - b0 + 1);
    const int item = ip.seq * sh.G + ip.g;
    auto merge = [&](bool from_groups, long long k0, long long k1, long long to_group) {
        for (int chunk = t; chunk < kRows * 8; chunk += n_thr) {
            const int r = chunk >> 3;
            if (r < sh.R) merge_row_chunk(ip, sq, sh, mc, from_groups, b0, k0, k1, to_group, r, (chunk & 7) * 16);
        }
    };
    if (n_parts <= kMergeFan) {
        if (!lead([&] { return count_part(mc.counters + item, n_parts); })) return;
        __threadfence();
        merge(false, b0, b1, -1);
        return;
    }
    const long long grp = b / kMergeFan;
    const long long gb0 = max(b0, grp * kMergeFan), gb1 = min(b1, grp * kMergeFan + kMergeFan - 1);
    if (!lead([&] { return count_part(mc.gcounters + grp * 2 + group_slot(grp, b0), static_cast<int>(gb1 - gb0 + 1)); })) return;
    __threadfence();
    merge(false, gb0, gb1, grp);
    __threadfence();   // every member publishes its piece of the group partial before the leader counts the group
    const long long g0 = b0 / kMergeFan, g1 = b1 / kMergeFan;
    if (!lead([&] { return count_part(mc.counters + item, static_cast<int>(g1 - g0 + 1)); })) return;
    __threadfence();
    merge(true, g0, g1, -1);
}

__global__ void __launch_bounds__(kThreads, 2)
decode_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
              const __grid_constant__ DecodeTable tab, AttnShape sh, uint16_t *__restrict__ k_base,
              uint16_t *__restrict__ v_base, WsHeader *hdr, int *counters, int *gcounters, float *partials,
              float *gpartials) {
    extern __shared__ uint8_t smem_raw[];
    DecodeSmem &sm = *reinterpret_cast<DecodeSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = sh.G, R = sh.R;

    if (tid == 0) {
        sm.abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], kConsumerWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.qfull[b], 1);
            mbar_init(&sm.qempty[b], kConsumerWarps);
        }
        mbar_init(&sm.hstart, 1);
        mbar_init(&sm.pdone[0], 1);
        mbar_init(&sm.pdone[1], 1);
        fence_mbar_init();
    }
    // The sequence descriptors and the prefix sums of their tile counts arrive as kernel parameters: no upload
    // precedes the launch.  The prefix sums are searched by every role, so they are copied to shared memory once
    // (dependent reads of parameter space miss the small constant cache one after another).
    const int n_seq = tab.n_seq;
    for (int i = tid; i <= n_seq; i += kThreads) {
        sm.prefix[i] = tab.prefix[i];
    }
    // Launched with programmatic stream serialization: everything above (barrier set-up, parameter reads) may run
    // while the previous kernel of the stream is still draining; from here on this grid touches global memory, so
    // it waits until that kernel has completed and its writes are visible.  Stream order is preserved.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __syncthreads();
    const long long total = static_cast<long long>(sm.prefix[n_seq]) * G;
    const long long nb = gridDim.x;
    const long long span_lo = span_start(blockIdx.x, total, nb), span_hi = span_start(blockIdx.x + 1, total, nb);
    if (span_lo >= span_hi) {
        return;
    }

    if (warp == kProducerWarp) {
        // ================================ producer warp ================================================
        if (lane == 0) {
            tma_prefetch_desc(&k_map);
            tma_prefetch_desc(&v_map);
            long long pos = span_lo;
            unsigned int n = 0;
            while (pos < span_hi && !sm.abort_flag) {
                const ItemPos ip = locate(sm.prefix, n_seq, G, pos);
                const int row = tab.seqs[ip.seq].slot * G + ip.g;
                const long long seg_end = min(span_hi, ip.item_begin + ip.n_tiles);
                for (int t = ip.tile; pos < seg_end; ++t, ++pos, ++n) {
                    const int st = n % kStages;
                    if (n == 1) {
                        // The first tile goes out at once; the rest of the ring's initial burst waits until the helper
                        // warp has issued the first segment's few small loads, so that they do not queue behind it.
                        mbar_wait_bounded(&sm.hstart, 0, &sm.abort_flag);
                    }
                    if (!mbar_wait_bounded(&sm.empty[st], ((n / kStages) & 1u) ^ 1u, &sm.abort_flag)) break;
                    uint8_t *dst = sm.stage[st];
                    mbar_arrive_expect_tx(&sm.full[st], kStageBytes);
                    tma_load_3d(dst, &k_map, 0, t * kTile, row, &sm.full[st]);
                    tma_load_3d(dst + kKHalfBytes, &k_map, 64, t * kTile, row, &sm.full[st]);
                    tma_load_2d(dst + 2 * kKHalfBytes, &v_map, t * kTile, row * kD, &sm.full[st]);
                }
                if (pos < seg_end) break;   // a wait ran out
            }
        }
    } else if (warp == kHelperWarp) {
        // ================================ helper warp ==================================================
        const MergeCtx mc{total, nb, counters, gcounters, partials, gpartials};
        auto warp_lead = [&](auto f) {
            __syncwarp();
            int v = 0;
            if (lane == 0) v = f();
            return __shfl_sync(0xffffffffu, v, 0);
        };
        long long pos = span_lo;
        unsigned int sidx = 0;
        int prev_slot = 0;   // partial slot of the previous segment: 0 for the CTA's first segment, else 1
        bool prev_partial = false;
        ItemPos prev_ip{};
        SeqDev prev_sq{};
        while (pos < span_hi && !sm.abort_flag) {
            const ItemPos ip = locate(sm.prefix, n_seq, G, pos);
            const SeqDev sq = tab.seqs[ip.seq];
            const long long item_end = ip.item_begin + ip.n_tiles;
            const long long seg_end = min(span_hi, item_end);
            const bool has_last_tile = seg_end == item_end;
            const bool appender = has_last_tile && !(sq.flags & CGLM_SEQ_NO_APPEND);
            const int b = sidx & 1;
            mbar_wait_bounded(&sm.qempty[b], ((sidx >> 1) & 1u) ^ 1u, &sm.abort_flag);
            prepare_segment(sm.qb[b], sh, sq, ip.g, sq.slot * G + ip.g, has_last_tile, appender, lane, k_base, v_base,
                            sidx == 0 ? &sm.hstart : nullptr);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.qfull[b]);
            if (prev_partial) {   // the consumers are still on the previous segment, or just left it
                mbar_wait_bounded(&sm.pdone[prev_slot], 0, &sm.abort_flag);   // each used once: a CTA has <= 2 partials
                deliver_part(prev_ip, prev_sq, sh, mc, blockIdx.x, lane, 32, warp_lead);
            }
            // the span's final segment is finished by the consumer warps themselves
            prev_partial = !(pos == ip.item_begin && has_last_tile) && seg_end < span_hi;
            prev_slot = sidx == 0 ? 0 : 1;
            prev_ip = ip;
            prev_sq = sq;
            pos = seg_end;
            ++sidx;
        }
        if (prev_partial && !sm.abort_flag) {
            mbar_wait_bounded(&sm.pdone[prev_slot], 0, &sm.abort_flag);
            deliver_part(prev_ip, prev_sq, sh, mc, blockIdx.x, lane, 32, warp_lead);
        }
    } else {
        // ================================ consumer warps ===============================================
        const int quad_row = lane >> 2, c = lane & 3;
        long long pos = span_lo;
        unsigned int n = 0, sidx = 0;
        bool first_segment = true;
        while (pos < span_hi) {
            const ItemPos ip = locate(sm.prefix, n_seq, G, pos);
            const int g = ip.g;
            const long long item_end = ip.item_begin + ip.n_tiles;
            const long long seg_end = min(span_hi, item_end);
            const bool has_last_tile = seg_end == item_end;
            const bool whole_item = pos == ip.item_begin && has_last_tile;
            const int last_tile = ip.n_tiles - 1;
            const QBuf &qb = sm.qb[sidx & 1];

            // what the helper warp prepared: the sequence's scalars and the q tile (A fragments: 8 k-steps of 16 dims)
            mbar_wait_bounded(&sm.qfull[sidx & 1], (sidx >> 1) & 1u, &sm.abort_flag);
            const int kv_before = qb.kv_before, flags = qb.flags;
            float *const out_ptr = qb.out, *const partial_ptr = qb.partial;
            const int L = attended_len(kv_before, flags);
            const bool appender = has_last_tile && !(flags & CGLM_SEQ_NO_APPEND);
            uint32_t qa[8][4];
            {
                const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const int rr = r8 + 8 * (mi & 1);
                    const int col = 16 * ks + 8 * (mi >> 1);
                    ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], smem_u32(&qb.q[rr][col]));
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
                float s[2][4];
                if (t != last_tile) {
                    qk_slice(kb, warp, lane, qa, s);
                    softmax_pv_slice<true>(vb, warp, lane, 16, s, m_run, l_run, o);
                } else {
                    const int tok0 = t * kTile + 16 * warp;   // first token of this warp's slice
                    const int n_valid = min(16, L - tok0);
                    if (n_valid > 0) {
                        patch_last_tile(kb, vb, warp, lane, n_valid, appender ? kv_before - tok0 : -1, qb.newk, qb.newv);
                        qk_slice(kb, warp, lane, qa, s);
                        softmax_pv_slice<false>(vb, warp, lane, n_valid, s, m_run, l_run, o);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.empty[st]);
            }
            // the q tile, newk and newv of this segment are no longer needed
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.qempty[sidx & 1]);

            // ---- fold the four warps' states into warp 0, one 64-dim half at a time ----------------------
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
                l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
            }
            if (seg_end == span_hi) {
                // Last segment of the span: the tile ring is idle (every tile has been loaded and consumed), so it
                // serves as one exchange area per warp and the fold takes two barriers instead of twelve.
                constexpr int kStride = 132;
                float *area = reinterpret_cast<float *>(sm.stage[0]);   // [3 warps][16 rows * 132 + 32]
                named_bar_sync(1, kConsumerThreads);                     // every warp has finished reading its tiles
                if (warp > 0) {
                    float *mine = area + (warp - 1) * (kRows * kStride + 2 * kRows);
#pragma unroll
                    for (int nd = 0; nd < 16; ++nd) {
                        *reinterpret_cast<float2 *>(&mine[quad_row * kStride + 8 * nd + 2 * c]) = make_float2(o[nd][0], o[nd][1]);
                        *reinterpret_cast<float2 *>(&mine[(quad_row + 8) * kStride + 8 * nd + 2 * c]) = make_float2(o[nd][2], o[nd][3]);
                    }
                    if (c == 0) {
                        mine[kRows * kStride + quad_row] = m_run[0];
                        mine[kRows * kStride + quad_row + 8] = m_run[1];
                        mine[kRows * kStride + kRows + quad_row] = l_run[0];
                        mine[kRows * kStride + kRows + quad_row + 8] = l_run[1];
                    }
                }
                named_bar_sync(1, kConsumerThreads);
                if (warp == 0) {
                    for (int src = 1; src < kConsumerWarps; ++src) {
                        const float *theirs = area + (src - 1) * (kRows * kStride + 2 * kRows);
                        float a_me[2], a_src[2];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const float m_src = theirs[kRows * kStride + quad_row + 8 * h];
                            const float l_src = theirs[kRows * kStride + kRows + quad_row + 8 * h];
                            const float m_new = fmaxf(m_run[h], m_src);
                            a_me[h] = ex2_approx(m_run[h] - m_new);
                            a_src[h] = ex2_approx(m_src - m_new);
                            l_run[h] = l_run[h] * a_me[h] + l_src * a_src[h];
                            m_run[h] = m_new;
                        }
#pragma unroll
                        for (int nd = 0; nd < 16; ++nd) {
                            const float2 lo2 = *reinterpret_cast<const float2 *>(&theirs[quad_row * kStride + 8 * nd + 2 * c]);
                            const float2 hi2 = *reinterpret_cast<const float2 *>(&theirs[(quad_row + 8) * kStride + 8 * nd + 2 * c]);
                            o[nd][0] = o[nd][0] * a_me[0] + lo2.x * a_src[0];
                            o[nd][1] = o[nd][1] * a_me[0] + lo2.y * a_src[0];
                            o[nd][2] = o[nd][2] * a_me[1] + hi2.x * a_src[1];
                            o[nd][3] = o[nd][3] * a_me[1] + hi2.y * a_src[1];
                        }
                    }
                }
            } else
            for (int src = 1; src < kConsumerWarps; ++src) {
                float a_me[2] = {1.f, 1.f}, a_src[2] = {0.f, 0.f};
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    named_bar_sync(1, kConsumerThreads);
                    if (warp == src) {
#pragma unroll
                        for (int nd = 0; nd < 8; ++nd) {
                            *reinterpret_cast<float2 *>(&sm.xchg[quad_row * kXchgStride + 8 * nd + 2 * c]) =
                                make_float2(o[8 * half + nd][0], o[8 * half + nd][1]);
                            *reinterpret_cast<float2 *>(&sm.xchg[(quad_row + 8) * kXchgStride + 8 * nd + 2 * c]) =
                                make_float2(o[8 * half + nd][2], o[8 * half + nd][3]);
                        }
                        if (half == 0 && c == 0) {
                            sm.xchg[kRows * kXchgStride + quad_row] = m_run[0];
                            sm.xchg[kRows * kXchgStride + quad_row + 8] = m_run[1];
                            sm.xchg[kRows * kXchgStride + kRows + quad_row] = l_run[0];
                            sm.xchg[kRows * kXchgStride + kRows + quad_row + 8] = l_run[1];
                        }
                    }
                    named_bar_sync(1, kConsumerThreads);
                    if (warp == 0) {
                        if (half == 0) {
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
                        }
#pragma unroll
                        for (int nd = 0; nd < 8; ++nd) {
                            const float2 lo2 = *reinterpret_cast<const float2 *>(&sm.xchg[quad_row * kXchgStride + 8 * nd + 2 * c]);
                            const float2 hi2 = *reinterpret_cast<const float2 *>(&sm.xchg[(quad_row + 8) * kXchgStride + 8 * nd + 2 * c]);
                            float(&oo)[4] = o[8 * half + nd];
                            oo[0] = oo[0] * a_me[0] + lo2.x * a_src[0];
                            oo[1] = oo[1] * a_me[0] + lo2.y * a_src[0];
                            oo[2] = oo[2] * a_me[1] + hi2.x * a_src[1];
                            oo[3] = oo[3] * a_me[1] + hi2.y * a_src[1];
                        }
                    }
                }
            }

            // ---- emit: final rows, or a partial for the merge kernel --------------------------------------
            if (warp == 0) {
                const bool want_partial = (flags & CGLM_SEQ_PARTIAL) != 0;
                if (whole_item) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int r = quad_row + 8 * h;
                        if (r < R) {
                            const int head = g * R + r;
                            if (want_partial) {
                                float *pp = partial_ptr + static_cast<long long>(head) * (kD + 2);
#pragma unroll
                                for (int nd = 0; nd < 16; ++nd) {
                                    *reinterpret_cast<float2 *>(&pp[8 * nd + 2 * c]) =
                                        make_float2(o[nd][2 * h], o[nd][2 * h + 1]);
                                }
                                if (c == 0) { pp[kD] = m_run[h] * kLn2; pp[kD + 1] = l_run[h]; }
                            } else {
                                const float inv = 1.f / l_run[h];
                                float *op = out_ptr + static_cast<long long>(head) * kD;
#pragma unroll
                                for (int nd = 0; nd < 16; ++nd) {
                                    *reinterpret_cast<float2 *>(&op[8 * nd + 2 * c]) =
                                        make_float2(o[nd][2 * h] * inv, o[nd][2 * h + 1] * inv);
                                }
                            }
                        }
                    }
                } else {
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
                    __syncwarp();
                    if (seg_end < span_hi) {
                        // more segments follow: the helper warp counts and merges while we stream on
                        if (lane == 0) mbar_arrive(&sm.pdone[first_segment ? 0 : 1]);
                    }
                }
            }
            if (!whole_item && seg_end == span_hi) {
                // end of the span: nothing left to overlap with, all four warps complete the item if it is theirs to
                // complete.  The barrier inside cta_lead also orders warp 0's partial stores before the count.
                const MergeCtx mc{total, nb, counters, gcounters, partials, gpartials};
                auto cta_lead = [&](auto f) {
                    named_bar_sync(1, kConsumerThreads);
                    if (tid == 0) sm.last_flag = f();
                    named_bar_sync(1, kConsumerThreads);
                    return sm.last_flag;
                };
                deliver_part(ip, tab.seqs[ip.seq], sh, mc, blockIdx.x, tid, kConsumerThreads, cta_lead);
            }
            first_segment = false;
            ++sidx;
        }
    }
    if (sm.abort_flag && lane == 0) {
        atomicExch(&hdr->status, static_cast<int>(CGLM_ERR_TIMEOUT));
    }
}

}  // namespace

int decode_max_ctas(int n_sm) { return 2 * n_sm; }

cudaError_t launch_decode(const LaunchCtx &cx, const DecodeTable &tab) {
    const long long total_tiles = static_cast<long long>(tab.prefix[tab.n_seq]) * cx.shape.G;
    if (tab.n_seq == 0 || total_tiles == 0) {
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = cx.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see griddepcontrol.wait in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_kernel, *cx.k_map, *cx.v_map, tab, cx.shape, cx.k_base, cx.v_base, cx.hdr,
                                       cx.counters, cx.gcounters, cx.partials, cx.gpartials);
    g_launch_count += 1;
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace cglm
