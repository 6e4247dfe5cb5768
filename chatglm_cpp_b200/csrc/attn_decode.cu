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
//                   the new k with angles from the arena's table, the scaled f16 q tile, the f16 append into the
//                   cache) and finishes the PREVIOUS one (completion counter, merge of a split item), so that a
//                   segment switch costs the consumers no global-memory round trip;
//   4 consumer warps take 16 tokens of each tile, run QK^T and PV on tensor cores (mma.sync m16n8k16, the
//                   <=16 q heads of the kv head are the M rows) with a warp-shuffle online softmax; at the end
//                   of a segment they fold their four states through the stage of the segment's last tile.
// What shaped the code around the tile loop: straight-line code that runs once per launch (or once per item) is
// paid for in instruction-fetch misses, about a microsecond per 5 KiB, while every other SM waits.  Hence one body
// for full and partial tiles, the merge code out of line in a single copy, reads of parameter space and a dry pass
// of the helper's first segment placed before the programmatic-dependency wait, and no sincos between the start of
// the kernel and its first tile.
// Both caches are already contraction-contiguous for the B operand: K is [token][d] for QK^T and V^T is
// [d][token] for PV.
#include <cstdlib>

#include <type_traits>

#include "common.cuh"

namespace cglm {

std::atomic<unsigned long long> g_launch_count{0};

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
    int seq, g, tile, n_tiles;   // the segment's ItemPos: the consumers take it from here instead of searching the
    long long item_begin;        // tile prefix themselves between two segments (0.7 us, measured)
};

// A position on the line of tiles: which (sequence, kv head) item it falls in and where.
struct ItemPos {
    int seq, g, tile, n_tiles;
    long long item_begin;   // line position of tile 0 of this item
};

// Where a completed item goes: the sequence's output row, or its (acc, m, l) row for a split-KV combine.
struct ItemOut {
    float *out, *partial;
    int flags;
};
// How the line of tiles is cut into the CTAs' spans.  Every item start inside a span costs the CTA a switch (fold of the
// four warps' states, partial store, a new q tile): about the time of two or three tiles.  The cut therefore balances
// cost, not tiles: on the *charged* line every item is preceded by `charge` pseudo-tiles, the charged line is cut into
// nb equal pieces, and a piece's pseudo-tiles are dropped again.  A span that contains an item start gets that many
// fewer tiles.  charge = 0 gives the plain equal-tile cut.  The cut depends on (prefix, G, nb, charge) only.
struct Geo {
    const int *prefix;     // shared-memory copy of the launch's tile prefix sums (per sequence, per kv head)
    long long total, nb;   // tiles on the line, CTAs with work
    int n_seq, G, charge;
    // tile position of charged position x
    __device__ __forceinline__ long long uncharge(long long x) const {
        if (charge == 0) return x;
        int lo = 0, hi = n_seq - 1;   // last sequence whose charged start is <= x
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (static_cast<long long>(prefix[mid] + mid * charge) * G <= x) lo = mid; else hi = mid - 1;
        }
        const int n = prefix[lo + 1] - prefix[lo];
        const int off = static_cast<int>(x - static_cast<long long>(prefix[lo] + lo * charge) * G);   // < G * (n + charge)
        const int g = off / (n + charge);
        const int o2 = off - g * (n + charge);
        return static_cast<long long>(prefix[lo]) * G + static_cast<long long>(g) * n + (o2 > charge ? o2 - charge : 0);
    }
    __device__ __forceinline__ long long charged_total() const { return total + static_cast<long long>(n_seq) * G * charge; }
    __device__ __forceinline__ long long span_start(long long b) const { return b >= nb ? total : uncharge(b * charged_total() / nb); }
    // the span that holds tile `tile` of item (seq, g), whose first tile sits at item_begin on the line
    __device__ __forceinline__ long long span_of(int seq, int g, long long item_begin, int tile) const {
        const long long x = item_begin + static_cast<long long>(seq * G + g + 1) * charge + tile;
        long long b = x * nb / charged_total();
        while (span_start(b + 1) <= item_begin + tile) ++b;
        return b;
    }
};

struct MergeCtx {
    Geo geo;
    int *counters;         // per item: parts delivered (short items) or groups delivered (long items)
    int *gcounters;        // per (CTA group, slot): parts of the long item in that slot delivered
    float *partials;       // per (CTA, slot)
    float *gpartials;      // per (CTA group, slot)
};

// What a team hands to deliver_part, parked in shared memory: the function is kept out of line (one copy of the
// merge code for its three callers), and a stack frame in local memory would put loads from a saturated memory
// system on the critical path of the launch's last microseconds.
// Exchange state of a fused split-KV step, in shared memory: the kernel parameter plus what the helper warp reads
// after the dependency wait.
struct XchgShared {
    XchgDev xd;
    WsHeader *hdr;
    unsigned int epoch;    // this step's number = the local buffer's counter + 1
    int slot_words;        // kv heads * kDecodePartialFloats
    int H, G, R;
};

// Which CTAs hold parts of an item, worked out (a few 64-bit divisions and a search of the tile prefix) when a segment
// starts, i.e. while its tiles are still on their way, not between its last tile and the merge.
struct ItemSpans {
    long long b0, b1;   // CTAs b0..b1 hold parts of the item
    int first_slot;     // CTA b0 holds its part in its second slot unless the item begins exactly where b0's span does
};
__device__ __forceinline__ ItemSpans item_spans(const Geo &geo, const ItemPos &ip) {
    ItemSpans is;
    is.b0 = geo.span_of(ip.seq, ip.g, ip.item_begin, 0);
    is.b1 = geo.span_of(ip.seq, ip.g, ip.item_begin, ip.n_tiles - 1);
    is.first_slot = geo.span_start(is.b0) >= ip.item_begin ? 0 : 1;
    return is;
}

struct DeliverArgs {
    ItemPos ip;
    ItemSpans is;
    ItemOut io;
    MergeCtx mc;
    int G, R;
    const XchgShared *xs;   // non-null: the item's (acc, m, l) rows go to every rank's exchange buffer
};

struct __align__(1024) DecodeSmem {
    uint8_t stage[kStages][kStageBytes];
    QBuf qb[2];
    float xchg[kConsumerWarps * 2 * kRows];        // fold: every warp's row maxima and row sums
    int prefix[kDecodeMaxSeqPerLaunch + 2];        // copy of the launch's tile prefix sums (parameter space is slow to index)
    int slot[kDecodeMaxSeqPerLaunch];              // copy of every sequence's arena slot, for the producer
    SeqDev sq;                                     // the helper warp's copy of the descriptor it is preparing
    int npast[kDecodeMaxSeqPerLaunch];             // kDynPast: every sequence's n_past as read from the device
    DeliverArgs dargs[kConsumerWarps + 1];         // per calling warp: arguments of deliver_part
    XchgShared xs;                                 // exchange instantiation only
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t qfull[2];
    uint64_t qempty[2];
    uint64_t hstart;                               // helper -> producer: the first segment's loads are on their way
    int last_flag;                                 // end-of-span partial: this CTA completed the item
    uint64_t pdone[2];                             // consumers -> helper: partial 0 / 1 of this CTA is in scratch
    uint64_t isready;                              // helper -> consumers: last_is holds the geometry of the span's final item
    ItemSpans last_is;
    int abort_flag;
    int gated;                                     // this launch has gate words to poll (host-buffer call)
};

static_assert(sizeof(QBuf) % 16 == 0, "ldmatrix rows of the second q tile stay 16-byte aligned");
// two CTAs per SM: 2 * (dynamic shared memory + 1 KiB alignment slack + 1 KiB reserved per CTA) <= 228 KiB
static_assert(2 * (sizeof(DecodeSmem) + 2048) <= 233472, "two decode CTAs must fit one SM");


// Position on the line -> (sequence, kv head, tile) using the per-sequence prefix of tile counts.
__device__ __forceinline__ ItemPos locate(const int *prefix, int n_seq, int G, long long pos) {
    int lo = 0, hi = n_seq - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (static_cast<long long>(prefix[mid]) * G <= pos) lo = mid; else hi = mid - 1;
    }
    ItemPos ip;
    ip.seq = lo;
    ip.n_tiles = prefix[lo + 1] - prefix[lo];
    const int off = static_cast<int>(pos - static_cast<long long>(prefix[lo]) * G);   // < G * n_tiles
    ip.g = off / ip.n_tiles;
    ip.tile = off - ip.g * ip.n_tiles;
    ip.item_begin = pos - ip.tile;
    return ip;
}

__device__ __forceinline__ int attended_len(int kv_before, int flags) {
    return kv_before + ((flags & CGLM_SEQ_NO_APPEND) ? 0 : 1);
}

// A CTA keeps at most two partials: slot 0 for its first segment, slot 1 for its last.

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

// Online softmax over the slice's 16 scores per row (log2 domain) and O = O * alpha + P V.  n_valid: attended
// tokens of the slice, 16 for every tile but an item's last.  One body for both cases: code that runs once per
// item costs more in instruction fetch than eight selects per tile do.
__device__ __forceinline__ void softmax_pv_slice(uint32_t vb, int warp, int lane, int n_valid, float (&s)[2][4],
                                                 float (&m_run)[2], float (&l_run)[2], float (&o)[16][4]) {
    const int c = lane & 3;
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
    // V^T: the slice's 16 tokens of a dim are 8 words (two 16-byte chunks of the dim's 128-byte line).  Word w
    // keeps tokens 2w, 2w+1 below keep_n; the new token's half takes the new v.  Lane l patches dims l, l+32, ...
    const int keep_n = ours ? new_local : n_valid;
    uint32_t keep[8], ins[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        keep[w] = (2 * w < keep_n ? 0x0000ffffu : 0u) | (2 * w + 1 < keep_n ? 0xffff0000u : 0u);
        ins[w] = (ours && (new_local >> 1) == w) ? ((new_local & 1) ? 0xffff0000u : 0x0000ffffu) : 0u;
    }
#pragma unroll 1
    for (int d = lane; d < kD; d += 32) {
        const uint32_t nv = __half_as_ushort(newv[d]) * 0x00010001u;
        const uint32_t line = vb + d * 128;
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
            const uint32_t addr = line + (((2 * warp + hc) ^ (d & 7)) << 4);
            uint32_t x0, x1, x2, x3;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(addr) : "memory");
            x0 = (x0 & keep[4 * hc + 0]) | (nv & ins[4 * hc + 0]);
            x1 = (x1 & keep[4 * hc + 1]) | (nv & ins[4 * hc + 1]);
            x2 = (x2 & keep[4 * hc + 2]) | (nv & ins[4 * hc + 2]);
            x3 = (x3 & keep[4 * hc + 3]) | (nv & ins[4 * hc + 3]);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x0), "r"(x1), "r"(x2), "r"(x3) : "memory");
        }
    }
    fence_proxy_async();
    __syncwarp();
}

// One warp copies a sequence descriptor from parameter space to shared memory, a word per lane: one trip instead
// of one per field read.
__device__ __forceinline__ void load_seq_desc(SeqDev &dst, const SeqDev &src, int lane) {
    static_assert(sizeof(SeqDev) == 32 * sizeof(uint32_t), "one word per lane");
    reinterpret_cast<uint32_t *>(&dst)[lane] = reinterpret_cast<const uint32_t *>(&src)[lane];
    __syncwarp();
}

// ---- helper warp: everything a segment needs before its first tile -----------------------------------------
// RoPE on the 16 q heads of the kv head and on the new k (chatglm.cpp:655-656), q * 1/sqrt(d) in f16
// (chatglm.cpp:686), and, when the segment holds the item's last tile, the f16 append of K row and V^T column
// (chatglm.cpp:668-675).  One warp, lane l owns dims 4l..4l+3 of every head: 18 sixteen-byte loads per lane, all
// issued before anything depends on one (a single round trip), and as few instructions as possible, because this
// runs between the start of the kernel and its first tile.  The callers guarantee 16-byte aligned rows.
// dry: touch no global memory (loads and stores are predicated off); a dry pass before the real one only pulls
// this code into the instruction cache, which the first execution of straight-line code otherwise pays for with
// a few microseconds of fetch misses.
//   CHATGLM2: dims [0, 64) rotate as adjacent pairs (2p, 2p+1) by ladder angle p: both pairs of lanes 0..15 stay
//             inside the lane.
//   CHATGLM:  each 64-dim half rotates as pairs (i, i+32) by ladder angle i, the first half by the position id and
//             the second by the block position id: the partner of lane l sits in lane l ^ 8.
__device__ __forceinline__ float4 ldg4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
// four consecutive outputs at element index e of an f32 row, or of an f16 row with CGLM_SEQ_OUT_F16
__device__ __forceinline__ void st_out4(float *row, long long e, bool f16, float a, float b, float c, float d) {
    if (f16) {
        *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(row) + e) = make_uint2(pack_half2(a, b), pack_half2(c, d));
    } else {
        *reinterpret_cast<float4 *>(row + e) = make_float4(a, b, c, d);
    }
}
__device__ __forceinline__ uint2 pack_half4(float a, float b, float c, float d) {
    return make_uint2(pack_half2(a, b), pack_half2(c, d));
}
// Angle of a position the arena's table does not hold (explicit position ids beyond the cache capacity): out of
// line, so that the double-precision sincos stays out of the instruction stream of the common case.
__device__ __noinline__ float2 rope_angle_uncached(int pos, int i, float theta_scale) {
    float2 cs;
    rope_cos_sin(pos, i, theta_scale, cs.x, cs.y);
    return cs;
}

__device__ __forceinline__ void prepare_segment(QBuf &qb, const AttnShape &sh, const SeqDev &sq, int g,
                                                int row, bool has_last_tile, bool appender, int lane,
                                                uint16_t *__restrict__ k_base, uint16_t *__restrict__ v_base,
                                                const float2 *__restrict__ rope_tab, int rope_tab_len,
                                                uint64_t *loads_issued, bool dry) {
    const int R = sh.R, M = sh.M;
    if (lane == 0) {
        qb.out = sq.out; qb.partial = sq.partial; qb.kv_before = sq.kv_before; qb.flags = sq.flags;
    }
    const bool k_needed = appender || (has_last_tile && sq.k_roped);
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 x[kRows + 1], xv = zero4;   // x[kRows]: the new k row
    const bool in_f16 = (sq.flags & CGLM_SEQ_QKV_F16) != 0;   // element strides either way
    // one branch around each batch of loads, not one per load: all 18 requests leave before anything waits for one
    if (in_f16) {
        uint2 raw[kRows + 2];
        const __half *qh = reinterpret_cast<const __half *>(sq.q) + static_cast<long long>(g) * R * sq.q_head_stride + 4 * lane;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            raw[r] = (r < R && !dry) ? __ldg(reinterpret_cast<const uint2 *>(qh)) : make_uint2(0u, 0u);
            qh += sq.q_head_stride;
        }
        raw[kRows] = (k_needed && !dry) ? __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const __half *>(sq.k) + g * sq.kv_head_stride + 4 * lane))
                                        : make_uint2(0u, 0u);
        raw[kRows + 1] = (appender && !dry) ? __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const __half *>(sq.v) + g * sq.kv_head_stride + 4 * lane))
                                            : make_uint2(0u, 0u);
        auto widen = [](uint2 u) {
            const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
            const float2 c = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
            return make_float4(a.x, a.y, c.x, c.y);
        };
#pragma unroll
        for (int r = 0; r <= kRows; ++r) x[r] = widen(raw[r]);
        xv = widen(raw[kRows + 1]);
    } else {
        const float *src = sq.q + static_cast<long long>(g) * R * sq.q_head_stride + 4 * lane;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            x[r] = (r < R && !dry) ? ldg4(src) : zero4;
            src += sq.q_head_stride;
        }
        x[kRows] = (k_needed && !dry) ? ldg4(sq.k + g * sq.kv_head_stride + 4 * lane) : zero4;
        if (appender && !dry) xv = ldg4(sq.v + g * sq.kv_head_stride + 4 * lane);
    }
    // Lane l fetches ladder angle l of the position stream (and of the block-position stream in CHATGLM mode) from
    // the arena's table in the same round trip.
    int pos_id = 0, block_id = 0;
    float2 cs0 = make_float2(1.f, 0.f), cs1 = make_float2(1.f, 0.f);
    const int mode = (sq.flags & CGLM_SEQ_Q_ROPED) ? static_cast<int>(CGLM_ROPE_DISABLED) : sh.rope_type;
    if (mode != CGLM_ROPE_DISABLED && !dry) {
        derive_positions(sq, mode, 0, pos_id, block_id);
        const bool tab0 = pos_id >= 0 && pos_id < rope_tab_len;
        const bool tab1 = block_id >= 0 && block_id < rope_tab_len;
        if (tab0) cs0 = __ldg(rope_tab + static_cast<long long>(pos_id) * 32 + lane);
        else cs0 = rope_angle_uncached(pos_id, lane, sh.theta_scale);
        if (mode == CGLM_ROPE_CHATGLM) {
            if (tab1) cs1 = __ldg(rope_tab + static_cast<long long>(block_id) * 32 + lane);
            else cs1 = rope_angle_uncached(block_id, lane, sh.theta_scale);
        }
    }
    if (loads_issued) {   // first segment of the CTA: only now may the producer start its burst of tile loads,
        __syncwarp();     // so that these few small loads do not queue behind 96 KiB of them
        if (lane == 0) mbar_arrive(loads_issued);
    }
    // Rotation of the 17 rows, in place.  Every product and sum is rounded separately and in the order of
    // rope_rotate(): y0 = x0 c - x1 s, y1 = x0 s + x1 c.
    if (mode == CGLM_ROPE_CHATGLM2) {
        // lanes 0..15 hold pairs 2l and 2l+1 entirely; lanes 16..31 hold dims that do not rotate
        const int a = (2 * lane) & 31;
        const float ca = __shfl_sync(0xffffffffu, cs0.x, a), sa = __shfl_sync(0xffffffffu, cs0.y, a);
        const float cb = __shfl_sync(0xffffffffu, cs0.x, a + 1), sb = __shfl_sync(0xffffffffu, cs0.y, a + 1);
        const bool rot = lane < 16;
#pragma unroll
        for (int r = 0; r <= kRows; ++r) {
            float4 y;
            rope_rotate(x[r].x, x[r].y, ca, sa, y.x, y.y);
            rope_rotate(x[r].z, x[r].w, cb, sb, y.z, y.w);
            if (rot) x[r] = y;
        }
    } else if (mode == CGLM_ROPE_CHATGLM) {
        // lane l holds x_i (bit 3 of l clear) or x_{i+32} (set) of four pairs; the other element sits in lane l ^ 8
        const bool second = lane >= 16, upper = (lane & 8) != 0;
        float c[4], sg[4];   // sg: the sine with the sign this lane's element takes (-s for x_i, +s for x_{i+32})
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int a = 4 * (lane & 7) + e;
            const float c0 = __shfl_sync(0xffffffffu, cs0.x, a), s0 = __shfl_sync(0xffffffffu, cs0.y, a);
            const float c1 = __shfl_sync(0xffffffffu, cs1.x, a), s1 = __shfl_sync(0xffffffffu, cs1.y, a);
            c[e] = second ? c1 : c0;
            sg[e] = second ? s1 : s0;
        }
#pragma unroll
        for (int r = 0; r <= kRows; ++r) {
            const float ox = __shfl_xor_sync(0xffffffffu, x[r].x, 8), oy = __shfl_xor_sync(0xffffffffu, x[r].y, 8);
            const float oz = __shfl_xor_sync(0xffffffffu, x[r].z, 8), ow = __shfl_xor_sync(0xffffffffu, x[r].w, 8);
            // x_i:      y = x c - o s  (rope_rotate's y0 with x0 = x, x1 = o)
            // x_{i+32}: y = o s + x c  (rope_rotate's y1 with x0 = o, x1 = x); the sum commutes exactly
            const float px = __fmul_rn(ox, sg[0]), py = __fmul_rn(oy, sg[1]), pz = __fmul_rn(oz, sg[2]), pw = __fmul_rn(ow, sg[3]);
            x[r].x = upper ? __fadd_rn(px, __fmul_rn(x[r].x, c[0])) : __fsub_rn(__fmul_rn(x[r].x, c[0]), px);
            x[r].y = upper ? __fadd_rn(py, __fmul_rn(x[r].y, c[1])) : __fsub_rn(__fmul_rn(x[r].y, c[1]), py);
            x[r].z = upper ? __fadd_rn(pz, __fmul_rn(x[r].z, c[2])) : __fsub_rn(__fmul_rn(x[r].z, c[2]), pz);
            x[r].w = upper ? __fadd_rn(pw, __fmul_rn(x[r].w, c[3])) : __fsub_rn(__fmul_rn(x[r].w, c[3]), pw);
        }
    }
    const bool want_q = has_last_tile && sq.q_roped != nullptr && !dry;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        *reinterpret_cast<uint2 *>(&qb.q[r][4 * lane]) =
            pack_half4(__fmul_rn(x[r].x, sh.scale), __fmul_rn(x[r].y, sh.scale), __fmul_rn(x[r].z, sh.scale), __fmul_rn(x[r].w, sh.scale));
        if (want_q && r < R) {
            *reinterpret_cast<float4 *>(sq.q_roped + static_cast<long long>(g * R + r) * kD + 4 * lane) = x[r];
        }
    }
    if (k_needed && !dry) {
        const float4 y = x[kRows];
        if (sq.k_roped) *reinterpret_cast<float4 *>(sq.k_roped + static_cast<long long>(g) * kD + 4 * lane) = y;
        if (appender) {
            const uint2 h = pack_half4(y.x, y.y, y.z, y.w);
            *reinterpret_cast<uint2 *>(&qb.newk[4 * lane]) = h;
            *reinterpret_cast<uint2 *>(k_base + (static_cast<long long>(row) * M + sq.kv_before) * kD + 4 * lane) = h;
        }
    }
    if (appender && !dry) {
        const uint2 h = pack_half4(xv.x, xv.y, xv.z, xv.w);
        *reinterpret_cast<uint2 *>(&qb.newv[4 * lane]) = h;
        uint16_t *col = v_base + (static_cast<long long>(row) * kD + 4 * lane) * M + sq.kv_before;
        col[0] = static_cast<uint16_t>(h.x & 0xffffu);
        col[M] = static_cast<uint16_t>(h.x >> 16);
        col[2 * static_cast<long long>(M)] = static_cast<uint16_t>(h.y & 0xffffu);
        col[3 * static_cast<long long>(M)] = static_cast<uint16_t>(h.y >> 16);
    }
}

// ---- completion of split items ------------------------------------------------------------------------------
// An item cut across CTAs is completed by whichever CTA delivers its last part (atomic counters, nobody waits).
// Items of up to kMergeFan parts are merged in one step.  Longer ones (one very long sequence covers hundreds of
// CTAs) go through a two-level tree so that no thread walks hundreds of parts one batch after another: CTAs are
// grouped kMergeFan at a time by their index; the last CTA of a group to finish merges the item's parts inside the
// group into a group partial, and the last group to finish merges the group partials.
constexpr int kMergeFan = kDecodeMergeFan;

// A CTA group holds parts of at most two long items: one that began in an earlier group (slot 0) and one that
// begins inside the group (slot 1).
__device__ __forceinline__ int group_slot(long long grp, long long b0) { return b0 < grp * kMergeFan ? 0 : 1; }

// 16 dims of one q row merged over sources k0..k1 in one pass with a running maximum, four sources in flight at a
// time.  Sources are CTA partials (level 0) or group partials (level 1): source k sits at base + 2k slots (stride 2),
// except that source k_first uses its second slot when first_slot is 1 (the CTA or group in which the item begins
// holds the end of the previous item in its first slot).  The fused split-KV step merges the ranks' copies of a kv
// head with the same routine: source = rank, stride = kv heads per rank slot.  Every caller goes through this routine with the same source
// order, so the result does not depend on which CTA or warp happens to complete the item.
// dst_kind 0: the result is a group partial (un-normalised) at dst; 1: the sequence's (acc, m, l) row; 2: its f32
// output; 3: its f16 output.
__device__ __forceinline__ void merge_row_chunk(const float *base, int stride, long long k_first, int first_slot, long long k0,
                                                long long k1, float *dst, int dst_kind, int r, int d0) {
    float m_run = -INFINITY, den = 0.f;
    float acc[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) acc[e] = 0.f;
#pragma unroll 1
    for (long long k = k0; k <= k1; k += 4) {
        float mv[4], lv[4];
        float4 av[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const bool ok = k + u <= k1;
            const long long ks = ok ? k + u : k;
            const float *pp = base + (ks * stride + (ks == k_first ? first_slot : 0)) * kDecodePartialFloats;
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
    if (dst_kind == 0) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            __stcg(reinterpret_cast<float4 *>(dst + r * kD + d0) + e,
                   make_float4(acc[4 * e], acc[4 * e + 1], acc[4 * e + 2], acc[4 * e + 3]));
        }
        if (d0 == 0) { __stcg(dst + kRows * kD + r, m_run); __stcg(dst + kRows * kD + kRows + r, den); }
    } else if (dst_kind == 1) {
        float *po = dst + static_cast<long long>(r) * (kD + 2);   // row stride 130 floats: 8-byte aligned only
#pragma unroll
        for (int e = 0; e < 8; ++e) *reinterpret_cast<float2 *>(po + d0 + 2 * e) = make_float2(acc[2 * e], acc[2 * e + 1]);
        if (d0 == 0) { po[kD] = m_run * kLn2; po[kD + 1] = den; }
    } else {   // 2: f32 output row, 3: f16 output row (dst addresses row 0 of the kv head in the output's own type)
        const float inv = 1.f / den;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            st_out4(dst, static_cast<long long>(r) * kD + d0 + 4 * e, dst_kind == 3, acc[4 * e] * inv, acc[4 * e + 1] * inv,
                    acc[4 * e + 2] * inv, acc[4 * e + 3] * inv);
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


// Out of line for the combine of a fused split-KV step (inlined into the item merge above, where a call per chunk
// cost batch-1 decode 0.4 us per launch).
__device__ __noinline__ void merge_row_chunk_ool(const float *base, int stride, long long k1, float *dst, int dst_kind, int r, int d0) {
    merge_row_chunk(base, stride, -1, 0, 0, k1, dst, dst_kind, r, d0);
}

// ---- fused split-KV step: publish an item's rows to the peers, combine when everything has arrived --------------------
// A rank's slot of an exchange buffer holds, per kv head, one block in the layout of a CTA partial
// (acc[16][128] | m[16] | l[16], un-normalised, log2 domain): what the ranks exchange is what the CTAs of one
// launch exchange, and the final combine is merge_row_chunk with source = rank.
// Called by the team (n_thr threads, index t) that has just written the block of kv head g into this rank's slot of
// the LOCAL exchange buffer.  The team copies the block into the same slot of every peer's buffer with plain peer
// stores; after a team barrier its leader fences at system scope and writes the step number into the arrival word
// [rank][g] of every buffer.  The team that publishes this rank's last kv head then waits, with a bound, until the
// arrival words of every rank and kv head in the local buffer hold the step number, merges the n_rank blocks of
// every kv head into xd.out and advances the local step counter.  Nothing here waits for another CTA of this grid,
// only for other GPUs.
__device__ __noinline__ void xchg_finish(const XchgShared *xs, int g, int t, int n_thr, int *cta_flag) {
    const XchgDev &xd = xs->xd;
    const unsigned int e = xs->epoch;
    const int set = static_cast<int>(e & 1u), n_rank = xd.n_rank, rank = xd.rank, G = xs->G, R = xs->R;
    auto team_sync = [&]() {
        if (cta_flag) named_bar_sync(1, n_thr); else __syncwarp();
    };
    auto team_and = [&](int v) -> int {   // logical AND over the team; every member calls it
        if (cta_flag) {
            named_bar_sync(1, n_thr);
            if (t == 0) *cta_flag = 1;
            named_bar_sync(1, n_thr);
            if (!v) *cta_flag = 0;
            named_bar_sync(1, n_thr);
            return *cta_flag;
        }
        return __all_sync(0xffffffffu, v != 0);
    };
    team_sync();   // the block written by the other members is visible
    unsigned int *local = xd.peer[rank];
    const size_t blk0 = xchg_slot_word(set, rank, n_rank, xs->slot_words) + static_cast<size_t>(g) * kDecodePartialFloats;
    if (n_rank > 1) {
        // every member reads its share once (all loads in flight together: one trip to L2), then stores it to every peer
        constexpr int kShare = 5, kUnits = kDecodePartialFloats / 4;   // 520 float4 over >= 128 threads; a warp team takes 4 passes
        const float4 *src = reinterpret_cast<const float4 *>(local + blk0);
#pragma unroll 1
        for (int i0 = 0; i0 < kUnits; i0 += kShare * n_thr) {
            float4 mine[kShare];
#pragma unroll
            for (int c = 0; c < kShare; ++c) {
                const int i = i0 + c * n_thr + t;
                mine[c] = i < kUnits ? __ldcg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll 1
            for (int p = 0; p < n_rank; ++p) {
                if (p == rank) continue;
                float4 *dst = reinterpret_cast<float4 *>(xd.peer[p] + blk0);
#pragma unroll
                for (int c = 0; c < kShare; ++c) {
                    const int i = i0 + c * n_thr + t;
                    if (i < kUnits) dst[i] = mine[c];
                }
            }
        }
    }
    team_sync();   // every member's peer stores precede the leader's fence
    int last = 0;
    if (t == 0) {
        __threadfence_system();   // one fence, then the words: a release per word would wait for each peer in turn
        for (int p = 0; p < n_rank; ++p) {
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(xd.peer[p] + xchg_flag_word(set, rank, g)), "r"(e) : "memory");
        }
        last = atomicAdd(&xs->hdr->xchg_items, 1) == G - 1;
        if (last) atomicExch(&xs->hdr->xchg_items, 0);   // ready for the next step
    }
    if (cta_flag) {
        if (t == 0) *cta_flag = last;
        named_bar_sync(1, n_thr);
        last = *cta_flag;
    } else {
        last = __shfl_sync(0xffffffffu, last, 0);
    }
    if (!last) return;
    int ok = 1;
    if (xd.combine) {
        long long t0, now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        const long long limit = static_cast<long long>(xd.timeout_us) * 1000;
        for (int w = t; w < n_rank * G; w += n_thr) {
            const unsigned int *flag = local + xchg_flag_word(set, w / G, w % G);
            bool seen = false;
            for (unsigned int spin = 0; spin < (1u << 26); ++spin) {   // the timer bounds the wait, the count bounds the loop
                unsigned int v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                if (v == e) { seen = true; break; }
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (now - t0 > limit) break;
                __nanosleep(100);
            }
            if (!seen) ok = 0;
        }
        ok = team_and(ok);
        if (ok) {
            // source = rank: rank p's block of kv head gg sits G blocks after rank p - 1's
            const float *slots = reinterpret_cast<const float *>(local + xchg_slot_word(set, 0, n_rank, xs->slot_words));
#pragma unroll 1
            for (int c = t; c < G * kRows * 8; c += n_thr) {
                const int gg = c / (kRows * 8), r = (c >> 3) & (kRows - 1);
                if (r < R) {
                    merge_row_chunk_ool(slots + static_cast<size_t>(gg) * kDecodePartialFloats, G, n_rank - 1,
                                        xd.out + static_cast<size_t>(gg) * R * kD, 2, r, (c & 7) * 16);
                }
            }
        } else if (t == 0) {
            atomicExch(&xs->hdr->status, static_cast<int>(CGLM_ERR_TIMEOUT));
        }
    }
    if (t == 0) *reinterpret_cast<volatile unsigned int *>(local) = e;   // the step is over for this rank, merged or not
}

// Called by a team of n_thr threads (the four consumer warps at the end of a span, or the helper warp in the
// middle of one) after CTA `b` stored its part of item da->ip.  t: index inside the team.  cta_flag: shared-memory
// word through which a multi-warp team hears its leader's verdict; null for a team of one warp.
__device__ __noinline__ void deliver_part(const DeliverArgs *da, long long b, int t, int n_thr, int *cta_flag) {
    const ItemPos ip = da->ip;
    const ItemOut sq = da->io;
    const MergeCtx mc = da->mc;
    AttnShape sh{};
    sh.G = da->G;
    sh.R = da->R;
    // synchronises the team (ordering its memory operations), lets the leader count this part and hands the
    // result to every member: did this team deliver the last part?
    auto lead = [&](int *ctr, int expected) -> int {
        if (cta_flag) {
            named_bar_sync(1, n_thr);
            if (t == 0) *cta_flag = count_part(ctr, expected);
            named_bar_sync(1, n_thr);
            return *cta_flag;
        }
        __syncwarp();
        int v = 0;
        if (t == 0) v = count_part(ctr, expected);
        return __shfl_sync(0xffffffffu, v, 0);
    };
    const long long b0 = da->is.b0, b1 = da->is.b1;   // CTAs b0..b1 hold parts of the item
    const int n_parts = static_cast<int>(b1 - b0 + 1);
    const int item = ip.seq * sh.G + ip.g;
    // Slot of the first source at each level: the CTA (group) in which the item begins holds it in its second slot
    // unless the item begins exactly where the CTA's span (the group's first span) does.
    const int first_cta_slot = da->is.first_slot;
    const long long g0 = b0 / kMergeFan, g1 = b1 / kMergeFan;
    const int first_grp_slot = group_slot(g0, b0);
    const bool out_f16 = (sq.flags & CGLM_SEQ_OUT_F16) != 0;
    float *final_dst = (sq.flags & CGLM_SEQ_PARTIAL) ? sq.partial + static_cast<long long>(ip.g) * sh.R * (kD + 2)
                       : out_f16 ? reinterpret_cast<float *>(reinterpret_cast<__half *>(sq.out) + static_cast<long long>(ip.g) * sh.R * kD)
                                 : sq.out + static_cast<long long>(ip.g) * sh.R * kD;
    int final_kind = (sq.flags & CGLM_SEQ_PARTIAL) ? 1 : (out_f16 ? 3 : 2);
    if (da->xs) {   // fused split-KV step: the item's block of this rank's exchange slot, in the partial layout
        final_dst = sq.partial + static_cast<long long>(ip.g) * kDecodePartialFloats;
        final_kind = 0;
    }
    // one merge loop for the three uses below (the arguments vary, the code does not)
    auto merge = [&](const float *base, long long k_first, int first_slot, long long k0, long long k1, float *dst, int kind) {
#pragma unroll 1
        for (int chunk = t; chunk < kRows * 8; chunk += n_thr) {
            const int r = chunk >> 3;
            if (r < sh.R) merge_row_chunk(base, 2, k_first, first_slot, k0, k1, dst, kind, r, (chunk & 7) * 16);
        }
    };
    const float *base = mc.partials;
    long long k_first = b0, k0 = b0, k1 = b1;
    int first_slot = first_cta_slot;
    if (n_parts <= kMergeFan) {
        if (!lead(mc.counters + item, n_parts)) return;
    } else {
        const long long grp = b / kMergeFan;
        const long long gb0 = max(b0, grp * kMergeFan), gb1 = min(b1, grp * kMergeFan + kMergeFan - 1);
        if (!lead(mc.gcounters + grp * 2 + group_slot(grp, b0), static_cast<int>(gb1 - gb0 + 1))) return;
        __threadfence();
        merge(mc.partials, b0, first_cta_slot, gb0, gb1,
              mc.gpartials + (grp * 2 + group_slot(grp, b0)) * kDecodePartialFloats, 0);
        __threadfence();   // every member publishes its piece of the group partial before the leader counts the group
        if (!lead(mc.counters + item, static_cast<int>(g1 - g0 + 1))) return;
        base = mc.gpartials; k_first = g0; first_slot = first_grp_slot; k0 = g0; k1 = g1;
    }
    __threadfence();
    merge(base, k_first, first_slot, k0, k1, final_dst, final_kind);
    if (da->xs) xchg_finish(da->xs, ip.g, t, n_thr, cta_flag);
}

// Tiles [pos, pos_end) of the line into L2 only (no shared memory, no barrier): issued by the producer of a launch
// whose caches are settled while the previous kernel of the stream is still draining.
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap *map, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap *map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}

// kDynPast: sequences may carry CGLM_SEQ_N_PAST_DEVICE.  Their position is read from device memory once the previous
// kernel of the stream has completed, the tile prefix is rebuilt from it, and nothing runs ahead of the dependency
// wait (the spans are not known before).  A second instantiation, so that the common case pays nothing for it.
// kXchg: fused split-KV step.  The launch holds one sequence (this rank's slice of the KV length, CGLM_SEQ_PARTIAL
// semantics); its partial rows are written into the local exchange buffer and published to every rank by the CTA
// that completes them (xchg_finish).  A third instantiation: the other two carry none of it.
template <bool kDynPast, bool kXchg>
__global__ void __launch_bounds__(kThreads, 2)
decode_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
              const __grid_constant__ typename std::conditional<kDynPast, DecodeTableDyn, DecodeTable>::type tab, AttnShape sh,
              uint16_t *__restrict__ k_base,
              uint16_t *__restrict__ v_base, WsHeader *hdr, int *counters, int *gcounters, float *partials,
              float *gpartials, const float2 *__restrict__ rope_tab, int rope_tab_len,
              const __grid_constant__ XchgDev xchg) {
    extern __shared__ uint8_t smem_raw[];
    DecodeSmem &sm = *reinterpret_cast<DecodeSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = sh.G, R = sh.R;

    if (tid == 0) {
        sm.abort_flag = 0;
        // read here, before the dependency wait: a first read of this parameter line after the wait cost every launch
        // 1.6 us (measured on the one-long-sequence workload)
        sm.gated = (tab.gate[0] != nullptr || tab.gate[1] != nullptr) ? 1 : 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], kConsumerWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.qfull[b], 1);
            mbar_init(&sm.qempty[b], kConsumerWarps);
        }
        mbar_init(&sm.hstart, 1);
        mbar_init(&sm.pdone[0], kConsumerWarps);
        mbar_init(&sm.pdone[1], kConsumerWarps);
        mbar_init(&sm.isready, 1);
        fence_mbar_init();
        if (kXchg) {
            sm.xs.xd = xchg;
            sm.xs.hdr = hdr;
            sm.xs.slot_words = sh.G * kDecodePartialFloats;
            sm.xs.H = sh.H; sm.xs.G = sh.G; sm.xs.R = sh.R;
        }
    }
    // The sequence descriptors and the prefix sums of their tile counts arrive as kernel parameters: no upload
    // precedes the launch.  The prefix sums are searched by every role, so they are copied to shared memory once
    // (dependent reads of parameter space miss the small constant cache one after another).
    const int n_seq = tab.n_seq;
    // Settled caches (every sequence carries CGLM_SEQ_CACHE_SETTLED): no kernel that can still be running writes the
    // cache rows this launch reads, so the producer streams tiles without waiting for the previous kernel of the
    // stream; tab.settled - 1 further tiles per CTA are pulled into L2 behind the ring.
    const bool settled = !kDynPast && tab.settled != 0;
    const int trigger = tab.trigger;
    if constexpr (kDynPast) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (trigger == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        static_assert(kDecodeMaxSeqPerLaunch <= 4 * 32, "the tile prefix is scanned by one warp, four sequences per lane");
        for (int i = tid; i < n_seq; i += kThreads) {
            int np = tab.n_past_of[i];
            const int fl = tab.flags_of[i];
            if (fl & CGLM_SEQ_N_PAST_DEVICE) {
                np = *reinterpret_cast<const volatile int *>(tab.n_past_dev_of[i]);
                const int np_max = sh.M - sh.V - 1;   // the appended token must fit the cache
                if (np < 0 || np > np_max) {
                    np = np < 0 ? 0 : np_max;
                    atomicExch(&hdr->status, static_cast<int>(CGLM_ERR_INVALID_ARG));
                }
            }
            sm.npast[i] = np;
            sm.slot[i] = tab.slot_of[i];
            const int L = sh.V + np + ((fl & CGLM_SEQ_NO_APPEND) ? 0 : 1);
            sm.prefix[i + 1] = (L + kTile - 1) / kTile;
        }
        __syncthreads();
        if (warp == 0) {   // inclusive scan of the tile counts: four per lane, then across the lanes
            int v[4], run = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int e = 4 * lane + j;
                run += e < n_seq ? sm.prefix[e + 1] : 0;
                v[j] = run;
            }
            int before = run;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, before, d);
                if (lane >= d) before += o;
            }
            before -= run;   // exclusive
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int e = 4 * lane + j;
                if (e < n_seq) sm.prefix[e + 1] = before + v[j];
            }
            if (lane == 0) sm.prefix[0] = 0;
        }
    } else {
        for (int i = tid; i <= n_seq; i += kThreads) {
            sm.prefix[i] = tab.prefix[i];
            if (i < n_seq) sm.slot[i] = tab.seqs[i].slot;
        }
    }
    __syncthreads();
    const long long total = static_cast<long long>(sm.prefix[n_seq]) * G;
    // never more spans than tiles (the grid of a launch with device-side positions is sized from upper bounds): an
    // empty span between two parts of an item would be counted as a part that never arrives
    const long long nb = min(static_cast<long long>(gridDim.x), total);
    const bool idle = blockIdx.x >= nb;
    // An item start is charged a sixth of the average span, at most tab.charge tiles (measured with a charge of 3 on spans
    // of 36 tiles: spans with an item start inside still ended 3.8 us after the others although they had 2.7 tiles less; 6
    // evens them out, and 32 sequences with spans of 18 tiles do better with 3), and only when the spans are long against
    // it (no span may come out empty).
    const int charge = nb > 0 ? static_cast<int>(min(static_cast<long long>(tab.charge), total / nb / 6)) : 0;
    const Geo geo{sm.prefix, total, nb, n_seq, G,
                  (charge > 0 && (total + static_cast<long long>(n_seq) * G * charge) / nb >= 4LL * charge) ? charge : 0};
    const long long span_lo = idle ? 0 : geo.span_start(blockIdx.x);
    const long long span_hi = idle ? 0 : geo.span_start(blockIdx.x + 1);
    // Launched with programmatic stream serialization: everything that reads only kernel parameters (barrier
    // set-up, the tables above, the first segment's descriptor, the tensor maps) runs while the previous kernel of
    // the stream is still draining.  A read of parameter space at a computed index costs about a microsecond when
    // it misses, so none is left on the path between the wait below and the first tile.
    if (span_lo < span_hi) {
        if (warp == kHelperWarp) {
            const ItemPos ip = locate(sm.prefix, n_seq, G, span_lo);
            load_seq_desc(sm.sq, tab.seqs[ip.seq], lane);
        } else if (warp == kProducerWarp && lane == 0) {
            tma_prefetch_desc(&k_map);
            tma_prefetch_desc(&v_map);
        }
    }
    // From here on this grid touches global memory, so it waits until the previous kernel has completed and its
    // writes are visible.  Stream order is preserved.
    // (The helper warp of a CTA with work waits inside its loop, after a dry pass over its first segment.)
    if (!kDynPast && (warp != kHelperWarp || span_lo >= span_hi) && !(settled && warp == kProducerWarp && span_lo < span_hi)) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (trigger == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    if (span_lo >= span_hi) {
        return;
    }

    if (warp == kProducerWarp) {
        // ================================ producer warp ================================================
        if (lane == 0) {
            long long pos = span_lo;
            unsigned int n = 0;
            bool ahead = settled;   // this thread has not waited for the previous kernel yet
            while (pos < span_hi && !sm.abort_flag) {
                const ItemPos ip = locate(sm.prefix, n_seq, G, pos);
                const int row = sm.slot[ip.seq] * G + ip.g;
                const long long seg_end = min(span_hi, ip.item_begin + ip.n_tiles);
                for (int t = ip.tile; pos < seg_end; ++t, ++pos, ++n) {
                    const int st = n % kStages;
                    if (n == 1 && !settled) {
                        // The first tile goes out at once; the rest of the ring's initial burst waits until the helper
                        // warp has issued the first segment's few small loads, so that they do not queue behind it.
                        mbar_wait_bounded(&sm.hstart, 0, &sm.abort_flag);
                    }
                    if (ahead && n == kStages) {
                        // The ring is full and nothing can be consumed before the previous kernel has completed (the
                        // consumers need q): pull the next tiles of the span into L2 meanwhile, then wait like every
                        // other thread, so that the bounded waits below only count time this grid could make progress.
                        const long long pf_end = min(span_hi, pos + (tab.settled - 1));
                        for (long long pp = pos; pp < pf_end; ++pp) {
                            const ItemPos pi = locate(sm.prefix, n_seq, G, pp);
                            const int prow = sm.slot[pi.seq] * G + pi.g;
                            tma_prefetch_l2_3d(&k_map, 0, pi.tile * kTile, prow);
                            tma_prefetch_l2_3d(&k_map, 64, pi.tile * kTile, prow);
                            tma_prefetch_l2_2d(&v_map, pi.tile * kTile, prow * kD);
                        }
                        asm volatile("griddepcontrol.wait;" ::: "memory");
                        ahead = false;
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
            if (trigger == 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        }
    } else if (warp == kHelperWarp) {
        // ================================ helper warp ==================================================
        const MergeCtx mc{geo, counters, gcounters, partials, gpartials};
        long long pos = span_lo;
        unsigned int sidx = 0;
        int prev_slot = 0;   // partial slot of the previous segment: 0 for the CTA's first segment, else 1
        bool prev_partial = false;
        ItemPos prev_ip{};
        ItemSpans prev_is{};
        ItemOut prev_sq{};
        while (pos < span_hi && !sm.abort_flag) {
            const ItemPos ip = locate(sm.prefix, n_seq, G, pos);
            if (sidx > 0) load_seq_desc(sm.sq, tab.seqs[ip.seq], lane);   // the first one was fetched before the wait
            SeqDev sq = sm.sq;
            __syncwarp();
            if (kDynPast) {
                sq.n_past = sm.npast[ip.seq];
                sq.kv_before = sh.V + sq.n_past;   // CGLM_SEQ_USE_KV_LOCAL is not combined with a device-side position
            }
            const long long item_end = ip.item_begin + ip.n_tiles;
            const long long seg_end = min(span_hi, item_end);
            const bool has_last_tile = seg_end == item_end;
            const bool appender = has_last_tile && !(sq.flags & CGLM_SEQ_NO_APPEND);
            const int b = sidx & 1;
            mbar_wait_bounded(&sm.qempty[b], ((sidx >> 1) & 1u) ^ 1u, &sm.abort_flag);
            // First segment: a dry pass while the previous kernel of the stream may still be running, then the wait
            // that every thread makes before it touches global memory, then the real pass over warm code.
            const int n_pass = (sidx == 0 && !kDynPast) ? 2 : 1;
#pragma unroll 1
            for (int pass = 0; pass < n_pass; ++pass) {
                const bool dry = pass + 1 < n_pass;
                if (sidx == 0 && !dry && !kDynPast) {
                    asm volatile("griddepcontrol.wait;" ::: "memory");
                }
                if (sidx == 0 && !dry && sm.gated) {
                    // host-buffer call: the activations are in place / the output buffer is free once the copy engines have
                    // written these words (see DecodeTable::gate)
                    if (lane == 0) {
                        for (int gi = 0; gi < 2; ++gi) {
                            const unsigned int *gp = tab.gate[gi];
                            if (!gp) continue;
                            bool seen = false;
                            for (unsigned int spin = 0; spin < kSpinLimit && !sm.abort_flag; ++spin) {
                                unsigned int v;
                                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(gp) : "memory");
                                if (v == tab.gate_value[gi]) { seen = true; break; }
                                __nanosleep(200);
                            }
                            if (!seen) sm.abort_flag = 1;
                        }
                    }
                    __syncwarp();
                }
                if (kXchg && !dry) {
                    // this step's number, and where this rank's rows go inside the local exchange buffer
                    if (sidx == 0) {
                        unsigned int ep = 0;
                        if (lane == 0) {
                            ep = *reinterpret_cast<volatile unsigned int *>(sm.xs.xd.peer[sm.xs.xd.rank]) + 1u;
                            sm.xs.epoch = ep;
                        }
                        __syncwarp();
                    }
                    sq.partial = reinterpret_cast<float *>(sm.xs.xd.peer[sm.xs.xd.rank] +
                                                           xchg_slot_word(static_cast<int>(sm.xs.epoch & 1u), sm.xs.xd.rank,
                                                                          sm.xs.xd.n_rank, sm.xs.slot_words));
                }
                prepare_segment(sm.qb[b], sh, sq, ip.g, sq.slot * G + ip.g, has_last_tile, appender, lane, k_base, v_base,
                                rope_tab, rope_tab_len, (sidx == 0 && !dry) ? &sm.hstart : nullptr, dry);
            }
            if (lane == 0) {
                QBuf &qo = sm.qb[b];
                qo.seq = ip.seq; qo.g = ip.g; qo.tile = ip.tile; qo.n_tiles = ip.n_tiles; qo.item_begin = ip.item_begin;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.qfull[b]);
            // The span's last segment is delivered by the consumer warps themselves; which CTAs hold parts of its item (a few
            // 64-bit divisions and searches of the tile prefix) is worked out here, by the warp that has nothing else to do,
            // and not by the consumers between two segments: there it stood between the fold of one item and the first
            // tile of the next for 4.5 us (measured), which was most of what an item start inside a span cost.
            if (seg_end == span_hi && !(pos == ip.item_begin && has_last_tile)) {
                if (lane == 0) {
                    sm.last_is = item_spans(geo, ip);
                    mbar_arrive(&sm.isready);
                }
                __syncwarp();
            }
            if (prev_partial) {   // the consumers are still on the previous segment, or just left it
                mbar_wait_bounded(&sm.pdone[prev_slot], 0, &sm.abort_flag);   // each used once: a CTA has <= 2 partials
                {
                    DeliverArgs &da = sm.dargs[kConsumerWarps];
                    if (lane == 0) { da.ip = prev_ip; da.is = prev_is; da.io = prev_sq; da.mc = mc; da.G = G; da.R = R; da.xs = kXchg ? &sm.xs : nullptr; }
                    __syncwarp();
                    deliver_part(&da, blockIdx.x, lane, 32, nullptr);
                    __syncwarp();
                }
            }
            // the span's final segment is finished by the consumer warps themselves
            prev_partial = !(pos == ip.item_begin && has_last_tile) && seg_end < span_hi;
            prev_slot = sidx == 0 ? 0 : 1;
            prev_ip = ip;
            if (prev_partial) prev_is = item_spans(geo, ip);   // while the consumers stream the segment
            prev_sq = ItemOut{sq.out, sq.partial, sq.flags};
            pos = seg_end;
            ++sidx;
        }
        if (prev_partial && !sm.abort_flag) {
            mbar_wait_bounded(&sm.pdone[prev_slot], 0, &sm.abort_flag);
            {
                    DeliverArgs &da = sm.dargs[kConsumerWarps];
                    if (lane == 0) { da.ip = prev_ip; da.is = prev_is; da.io = prev_sq; da.mc = mc; da.G = G; da.R = R; da.xs = kXchg ? &sm.xs : nullptr; }
                    __syncwarp();
                    deliver_part(&da, blockIdx.x, lane, 32, nullptr);
                    __syncwarp();
                }
        }
    } else {
        // ================================ consumer warps ===============================================
        const int quad_row = lane >> 2, c = lane & 3;
        long long pos = span_lo;
        unsigned int n = 0, sidx = 0;
        bool first_segment = true;
        while (pos < span_hi) {
            const QBuf &qb = sm.qb[sidx & 1];
            // what the helper warp prepared: where the segment lies, the sequence's scalars and the q tile (A fragments: 8
            // k-steps of 16 dims)
            const bool q_ok = mbar_wait_bounded(&sm.qfull[sidx & 1], (sidx >> 1) & 1u, &sm.abort_flag);
            ItemPos ip;
            if (q_ok) {
                ip.seq = qb.seq; ip.g = qb.g; ip.tile = qb.tile; ip.n_tiles = qb.n_tiles; ip.item_begin = qb.item_begin;
            } else {   // a wait ran out: the launch is abandoned, but every warp still walks its span to the end in step
                ip = locate(sm.prefix, n_seq, G, pos);
            }
            const int g = ip.g;
            const long long item_end = ip.item_begin + ip.n_tiles;
            const long long seg_end = min(span_hi, item_end);
            const bool has_last_tile = seg_end == item_end;
            const bool whole_item = pos == ip.item_begin && has_last_tile;
            const int last_tile = ip.n_tiles - 1;
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
                int n_valid = 16;
                if (t == last_tile) {
                    const int tok0 = t * kTile + 16 * warp;   // first token of this warp's slice
                    n_valid = min(16, L - tok0);
                    if (n_valid > 0) {
                        patch_last_tile(kb, vb, warp, lane, n_valid, appender ? kv_before - tok0 : -1, qb.newk, qb.newv);
                    }
                }
                if (n_valid > 0) {
                    float s[2][4];
                    qk_slice(kb, warp, lane, qa, s);
                    softmax_pv_slice(vb, warp, lane, n_valid, s, m_run, l_run, o);
                }
                __syncwarp();
                // the stage of the segment's last tile is kept: it becomes the fold space below
                if (lane == 0 && pos + 1 < seg_end) mbar_arrive(&sm.empty[st]);
            }
            // the q tile, newk and newv of this segment are no longer needed
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.qempty[sidx & 1]);
            // Every tile of the span has been consumed: from here on this CTA only folds and merges, so the next kernel
            // of the stream may take its place (it starts once every CTA of this grid has said so or has exited).
            if (trigger == 2 && seg_end == span_hi && warp == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

            // ---- fold the four warps' states -----------------------------------------------------------------
            // Each warp attended its own 16 tokens of every tile and holds (m, l, O[16][128]) for them.  The stage
            // of the last tile (32 KiB = four O's) is borrowed before it goes back to the producer: every warp
            // writes its O there, scaled to the common maximum; then warp w adds up dims [32w, 32w+32) of the four
            // copies in a fixed order and writes that slice of the result itself.  Two barriers, and the output
            // leaves through all 128 threads.
            float *fold = reinterpret_cast<float *>(sm.stage[(n - 1) % kStages]);
            float *stats = sm.xchg;   // [warp][m: 16 rows | l: 16 rows]
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
                l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
            }
            if (c == 0) {
                stats[warp * 32 + quad_row] = m_run[0];
                stats[warp * 32 + quad_row + 8] = m_run[1];
                stats[warp * 32 + 16 + quad_row] = l_run[0];
                stats[warp * 32 + 16 + quad_row + 8] = l_run[1];
            }
            named_bar_sync(1, kConsumerThreads);   // statistics visible; every warp has finished reading the tile
            {
                float a[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = quad_row + 8 * h;
                    const float m_star = fmaxf(fmaxf(stats[r], stats[32 + r]), fmaxf(stats[64 + r], stats[96 + r]));
                    a[h] = ex2_approx(m_run[h] - m_star);   // 0 for a warp that saw no attended token (m = -inf)
                }
                // float2 unit u of row r lives at unit u ^ 4(r & 3): conflict-free stores here, and 16-byte reads below
                float *mine = fold + warp * (kRows * kD);
                const int swz = 4 * (quad_row & 3);
#pragma unroll
                for (int nd = 0; nd < 16; ++nd) {
                    const int u = (4 * nd + c) ^ swz;
                    *reinterpret_cast<float2 *>(&mine[quad_row * kD + 2 * u]) = make_float2(o[nd][0] * a[0], o[nd][1] * a[0]);
                    *reinterpret_cast<float2 *>(&mine[(quad_row + 8) * kD + 2 * u]) = make_float2(o[nd][2] * a[1], o[nd][3] * a[1]);
                }
            }
            named_bar_sync(1, kConsumerThreads);
            {
                // lane -> row rr, and 16 of the warp's 32 dims as four float4 (q: index of a float4 inside the row)
                const int rr = lane >> 1, hf = lane & 1;
                const float m0 = stats[rr], m1 = stats[32 + rr], m2 = stats[64 + rr], m3 = stats[96 + rr];
                const float m_star = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                const float l_sum = ((stats[16 + rr] * ex2_approx(m0 - m_star) + stats[48 + rr] * ex2_approx(m1 - m_star)) +
                                     stats[80 + rr] * ex2_approx(m2 - m_star)) + stats[112 + rr] * ex2_approx(m3 - m_star);
                const bool want_partial = (flags & CGLM_SEQ_PARTIAL) != 0;
                const int head = g * R + rr;
                const float inv = 1.f / l_sum;
                // a part goes to this CTA's partial slot; a whole kv head of a fused split-KV step goes to its block of the
                // exchange slot in the same layout
                const bool as_partial = !whole_item || kXchg;
                float *scratch = (kXchg && whole_item) ? partial_ptr + static_cast<long long>(g) * kDecodePartialFloats
                                 : partials + (static_cast<long long>(blockIdx.x) * 2 + (first_segment ? 0 : 1)) * kDecodePartialFloats;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int q = 8 * warp + 4 * hf + (jj ^ hf);   // the two lanes of a row start on different banks
                    const float *src = fold + rr * kD + 4 * (q ^ (2 * (rr & 3)));
                    const float4 v0 = *reinterpret_cast<const float4 *>(src);
                    const float4 v1 = *reinterpret_cast<const float4 *>(src + kRows * kD);
                    const float4 v2 = *reinterpret_cast<const float4 *>(src + 2 * kRows * kD);
                    const float4 v3 = *reinterpret_cast<const float4 *>(src + 3 * kRows * kD);
                    float4 acc;
                    acc.x = ((v0.x + v1.x) + v2.x) + v3.x; acc.y = ((v0.y + v1.y) + v2.y) + v3.y;
                    acc.z = ((v0.z + v1.z) + v2.z) + v3.z; acc.w = ((v0.w + v1.w) + v2.w) + v3.w;
                    if (as_partial) {
                        __stcg(reinterpret_cast<float4 *>(scratch + rr * kD + 4 * q), acc);
                    } else if (rr < R) {
                        if (want_partial) {   // rows of kD + 2 floats: 8-byte aligned only
                            float *pp = partial_ptr + static_cast<long long>(head) * (kD + 2) + 4 * q;
                            *reinterpret_cast<float2 *>(pp) = make_float2(acc.x, acc.y);
                            *reinterpret_cast<float2 *>(pp + 2) = make_float2(acc.z, acc.w);
                        } else {
                            st_out4(out_ptr, static_cast<long long>(head) * kD + 4 * q, (flags & CGLM_SEQ_OUT_F16) != 0,
                                    acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
                        }
                    }
                }
                if (warp == 0 && hf == 0) {
                    if (as_partial) {
                        __stcg(&scratch[kRows * kD + rr], m_star);
                        __stcg(&scratch[kRows * kD + kRows + rr], l_sum);
                    } else if (want_partial && rr < R) {
                        float *pp = partial_ptr + static_cast<long long>(head) * (kD + 2);
                        pp[kD] = m_star * kLn2;
                        pp[kD + 1] = l_sum;
                    }
                }
            }
            // hand the stage back: generic-proxy writes above, TMA writes next
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&sm.empty[(n - 1) % kStages]);
                // more segments follow and this one left a partial: the helper warp counts and merges it
                if (!whole_item && seg_end < span_hi) mbar_arrive(&sm.pdone[first_segment ? 0 : 1]);
            }
            if (!whole_item && seg_end == span_hi) {
                // end of the span: nothing left to overlap with, all four warps complete the item if it is theirs to
                // complete.  The team barrier inside deliver_part also orders every warp's partial stores before the count.
                const MergeCtx mc{geo, counters, gcounters, partials, gpartials};
                DeliverArgs &da = sm.dargs[warp];   // every warp parks its own copy: no barrier needed before the call
                mbar_wait_bounded(&sm.isready, 0, &sm.abort_flag);   // long since there: the helper warp wrote it while the tiles streamed
                if (lane == 0) {
                    da.ip = ip; da.is = sm.last_is; da.io = ItemOut{out_ptr, partial_ptr, flags}; da.mc = mc; da.G = G; da.R = R;
                    da.xs = kXchg ? &sm.xs : nullptr;
                }
                __syncwarp();
                deliver_part(&da, blockIdx.x, tid, kConsumerThreads, &sm.last_flag);
            } else if (kXchg && whole_item) {
                // the whole kv head was this CTA's: its rows are in the local buffer, publish them
                xchg_finish(&sm.xs, g, tid, kConsumerThreads, &sm.last_flag);
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

int decode_max_ctas(int n_sm) { return 2 * n_sm; }   // bound used to size scratch; launch_decode picks the grid

cudaError_t launch_decode(const LaunchCtx &cx, const DecodeTableDyn &tab, bool n_past_on_device, const XchgDev *xchg) {
    // with device-side positions tab.prefix holds the tile counts of the host's upper bounds: good for sizing only
    const long long total_tiles = static_cast<long long>(tab.prefix[tab.n_seq]) * cx.shape.G;
    if (tab.n_seq == 0 || total_tiles == 0) {
        return cudaSuccess;
    }
    static PerDeviceOnce configured;
    const int smem_bytes = static_cast<int>(sizeof(DecodeSmem)) + 1024;
    if (configured.needed(cx.device)) {
        cudaError_t e = require_current_device(cx.device);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        configured.mark(cx.device);
    }
    // Grid: about 18 tiles (0.6 MiB of cache) per CTA, at least one CTA per SM and at most 1.75 per SM.  Measured on
    // B200: 64 sequences (9.3 k tiles) 61.8 us per launch with 259 CTAs, 63.3 with 228, 68.3 with 148, 62.7 with 296;
    // 32 sequences (4.7 k tiles) 39.9 us with 259 against 42.2 with 148; the MHA shape 34.9 us with 200 against 37.9
    // with 148; 16 and 8 sequences and the one long sequence do not care between 96 and 228.
    // A launch with fewer tiles than SMs (batch-1 decode of a short context) is all latency, and what costs is the number
    // of parts an item is delivered in: measured on one 512-token sequence (2 items of 9 tiles), 18 CTAs of one tile
    // 11.0 us per launch, 9 CTAs of two tiles (spans that straddle the items) 17.2 us, 6 CTAs of three tiles 9.6 us, 2
    // CTAs of nine tiles 11.4 us.  Such a launch is cut into at most four parts per item (one batch of the merge) of
    // about three tiles each; with items of equal length the spans then end where the items do.
    const long long lo_ctas = cx.n_sm, hi_ctas = 7LL * cx.n_sm / 4;
    long long want = total_tiles / 18;
    want = want < lo_ctas ? lo_ctas : (want > hi_ctas ? hi_ctas : want);
    if (static_cast<long long>(tab.n_seq) * cx.shape.G * 16 < lo_ctas) want = lo_ctas;   // a few very long items: every extra CTA is one more part per item
    if (total_tiles < lo_ctas) {
        const long long n_items = static_cast<long long>(tab.n_seq) * cx.shape.G;
        long long parts = (total_tiles / n_items + 2) / 3;
        parts = parts < 1 ? 1 : (parts > 4 ? 4 : parts);
        want = n_items * parts;
    }
    {   // CGLM_DECODE_GRID forces the number of CTAs (tuning knob, read once; clamped to what the scratch is sized for)
        static const int forced = [] { const char *e = std::getenv("CGLM_DECODE_GRID"); return e ? std::atoi(e) : 0; }();
        if (forced > 0) want = forced < 2 * cx.n_sm ? forced : 2 * cx.n_sm;
    }
    const int grid = static_cast<int>(total_tiles < want ? total_tiles : want);
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
    if (xchg && (n_past_on_device || tab.n_seq != 1)) return cudaErrorInvalidValue;
    static const XchgDev no_xchg = {};
    const XchgDev &xd = xchg ? *xchg : no_xchg;
    cudaError_t e;
    if (n_past_on_device) {   // the only instantiation that takes the larger table
        e = cudaLaunchKernelEx(&cfg, decode_kernel<true, false>, *cx.k_map, *cx.v_map, tab, cx.shape, cx.k_base, cx.v_base, cx.hdr,
                               cx.counters, cx.gcounters, cx.partials, cx.gpartials, cx.rope_tab, cx.rope_tab_len, xd);
    } else {
        auto kernel = xchg ? decode_kernel<false, true> : decode_kernel<false, false>;
        e = cudaLaunchKernelEx(&cfg, kernel, *cx.k_map, *cx.v_map, static_cast<const DecodeTable &>(tab), cx.shape, cx.k_base,
                               cx.v_base, cx.hdr, cx.counters, cx.gcounters, cx.partials, cx.gpartials, cx.rope_tab, cx.rope_tab_len, xd);
    }
    g_launch_count += 1;
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace cglm
