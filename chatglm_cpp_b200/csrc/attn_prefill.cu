// Prefill attention on 5th-generation tensor cores (tcgen05 + TMEM) for head_dim 128 (sm_100a).
//
// Covers chatglm.cpp:655-717 for a prompt (n_past == 0, qlen = S tokens) in two launches:
//   prefill_prepare_kernel  RoPE on q and k (:655-656), f16 append of the K rows and V^T columns (:668-675),
//                           q * 1/sqrt(d) (:686) written as an f16 [head][token][d] tile source;
//   prefill_attn_kernel     one CTA per (128-token q tile, q head): flash-attention forward over the freshly
//                           written cache.  S = Q K^T (128x128x128) and O_tile = P V (128x128x128) are tcgen05.mma
//                           instructions issued by one thread of a control warp, operands staged in shared memory by
//                           TMA (K and V^T tiles, non-multicast, 128-byte swizzle, double buffered) or by the softmax
//                           threads (P, double buffered), accumulators in tensor memory (two S buffers and the
//                           running O), read back with tcgen05.ld: each of the 128 softmax threads owns one q row,
//                           so the online softmax needs no cross-thread reduction.  O stays in tensor memory across
//                           KV tiles (the MMA accumulates into it); a row's O is rescaled there only when its running
//                           maximum grows by more than 2^8, otherwise the old reference maximum is kept (exact: the
//                           same reference enters the numerator and the denominator).  The control thread runs
//                           ahead: S of tile j+1 and P V of tile j execute while the softmax threads work on tile j+1.
// Masks (chatglm.cpp:689-707): causal (token t visible to row s iff t <= n_virtual + s; tiles right of the
// diagonal are skipped) or the ChatGLM-6B v1 prefix mask (every row but the last is blocked from the last token).
// Tokens past the attended length never reach shared memory: the per-call tensor maps end at that length, so TMA
// fills them with zeros.
#include "common.cuh"

namespace cglm {

namespace {

constexpr int kD = 128;
constexpr int kQTile = 128;        // q rows per CTA = TMEM lanes
constexpr int kKvTile = 128;       // tokens per KV tile
constexpr int kSoftmaxThreads = 128;
constexpr int kLoadWarp = kSoftmaxThreads / 32;       // issues every TMA load
constexpr int kScoreWarp = kLoadWarp + 1;             // issues the S = Q K^T MMAs
constexpr int kPvWarp = kLoadWarp + 2;                // issues the O += P V MMAs
constexpr int kThreads = kSoftmaxThreads + 96;
constexpr int kHalfBytes = 128 * 128;          // one 128-row x 128-byte swizzled half tile (16 KiB)
constexpr int kTileBytes = 2 * kHalfBytes;     // a 128 x 128 f16 operand tile
constexpr int kTmemCols = 512;                 // S[2]: columns [0,256), O: columns [256,384)
constexpr float kRescaleThreshold = 8.f;       // log2 units a row's maximum may grow before O is rescaled
constexpr int kOutStride = 132;                // floats per row of the output staging tile
constexpr float kLog2e = 1.4426950408889634f;

// instruction descriptor of tcgen05.mma.kind::f16: D = f32, A = B = f16, both K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

struct __align__(1024) PrefillSmem {
    uint8_t q[kTileBytes];            // A of QK^T: [2 d-halves][128 rows][64 d]
    uint8_t k[2][kTileBytes];         // B of QK^T: [2 d-halves][128 tokens][64 d], double buffered
    uint8_t v[2][kTileBytes];         // B of PV:   [2 token-halves][128 d][64 tokens], double buffered
    uint8_t p[2][kTileBytes];         // A of PV:   [2 token-halves][128 rows][64 tokens], double buffered
    uint64_t q_full;
    uint64_t k_full[2];               // TMA -> control: K tile landed
    uint64_t v_full[2];               // TMA -> control: V^T tile landed
    uint64_t s_done[2];               // tensor core -> softmax: S buffer written
    uint64_t p_ready[2];              // softmax -> control: P buffer written, S buffer read
    uint64_t o_done[2];               // tensor core -> softmax, control: P V(j) accumulated; K/V^T[b] and P[b] have been read
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(PrefillSmem) + 1024 <= 232448, "one prefill CTA must fit the shared memory of an SM");
static_assert(kTileBytes * 4 >= 128 * kOutStride * 4, "the K/V^T buffers hold the output staging tile");

// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    return static_cast<uint64_t>((saddr & 0x3ffffu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// packed f32x2 arithmetic and the three-input maximum of sm_100: half the instructions of the scalar forms
__device__ __forceinline__ void fma2(float &d0, float &d1, float a0, float a1, float b, float c) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float &d0, float &d1, float a0, float a1) {   // (d0, d1) += (a0, a1)
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%0, %1};\n\tmov.b64 rb, {%2, %3};\n\tadd.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// 32 consecutive f32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- launch 1: RoPE, append, f16 q ---------------------------------------------------------------------------
// Grid: (16-token blocks, roles).  Roles along y: pairs of q heads, then one CTA per k head, then one CTA per v head.
//   q / k CTAs  rotate their heads for the block's tokens with cos/sin from the arena's angle table (or, for
//               caller-supplied position ids, from a table rope_table_kernel filled just before);
//   v CTAs      transpose [16 tokens][128 dims] through shared memory so that the V^T cache rows are written as
//               contiguous runs of tokens instead of one 2-byte store per (token, dim).
// q_half: f16 [H][s_pad][D]; rows >= S are never read for an output.  Rope modes: the two GLM modes or none.
static int rope_n_pairs_host(int rope_type) { return rope_type == CGLM_ROPE_DISABLED ? 0 : 1; }
constexpr int kPrepTokens = 16;   // tokens per CTA: one batch of loads per thread (64 measured 2.4 us slower per call)
constexpr int kPrepThreads = 256;

// table: f32 [stream][token][32 ladder steps][cos, sin]
__global__ void __launch_bounds__(256)
rope_table_kernel(AttnShape sh, SeqDev sq, float2 *__restrict__ table) {
    const int S = sq.qlen;
    const int n_streams = sh.rope_type == CGLM_ROPE_CHATGLM ? 2 : 1;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_streams * S * 32) return;
    const int li = i & 31, t = (i >> 5) % S, st = (i >> 5) / S;
    int pos, block;
    derive_positions(sq, sh.rope_type, t, pos, block);
    float c, s;
    rope_cos_sin(st ? block : pos, li, sh.theta_scale, c, s);
    table[i] = make_float2(c, s);
}

__global__ void __launch_bounds__(kPrepThreads)
prefill_prepare_kernel(AttnShape sh, SeqDev sq, uint16_t *__restrict__ k_base, uint16_t *__restrict__ v_base,
                       __half *__restrict__ q_half, int s_pad, const float2 *__restrict__ table, int table_by_position) {
    // Launched as a programmatic dependent itself (its launch latency hides behind the previous kernel of the
    // stream): nothing is read or written before that kernel has completed.  The attention kernel that follows is a
    // programmatic dependent of this grid: let its CTAs take their places (shared memory, tensor memory, barriers)
    // while this grid runs; it waits for this grid before its first load.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ __half tile_mem[kD][kPrepTokens + 2];       // v CTAs: [dim][token] transpose tile
    const int S = sq.qlen, H = sh.H, G = sh.G, M = sh.M;
    const bool in_f16 = (sq.flags & CGLM_SEQ_QKV_F16) != 0;
    const int t_begin = blockIdx.x * kPrepTokens;
    const int n_tok = min(kPrepTokens, S - t_begin);
    const int n_qpair = (H + 1) / 2;
    const int role = blockIdx.y;
    const int tid = threadIdx.x;

    if (role >= n_qpair + G) {
        // ---- v head g: transpose through shared memory ---------------------------------------------------------
        const int g = role - n_qpair - G;
        __half(*tile)[kPrepTokens + 2] = tile_mem;
        for (int t0 = tid >> 7; t0 < n_tok; t0 += 16) {   // 2 tokens per sweep, 8 sweeps of loads in flight
            const int d = tid & 127;
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int t = t0 + 2 * u;
                x[u] = t < n_tok ? ld_act(sq.v, (t_begin + t) * sq.kv_tok_stride + g * sq.kv_head_stride + d, in_f16) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int t = t0 + 2 * u;
                if (t < n_tok) tile[d][t] = __float2half_rn(x[u]);
            }
        }
        __syncthreads();
        uint16_t *vrow0 = v_base + static_cast<long long>(sq.slot * G + g) * kD * M + sq.kv_before + t_begin;
        for (int idx = tid; idx < kD * kPrepTokens; idx += kPrepThreads) {
            const int d = idx / kPrepTokens, t = idx % kPrepTokens;
            if (t < n_tok) vrow0[static_cast<long long>(d) * M + t] = __half_as_ushort(tile[d][t]);
        }
        return;
    }

    const int n_pairs = rope_n_pairs(sh.rope_type, kD);   // 0, 32 (CHATGLM2) or 64 (CHATGLM)

    const bool is_q = role < n_qpair;
    const int head0 = is_q ? 2 * role : role - n_qpair;
    const int n_heads = is_q ? min(2, H - head0) : 1;
    // p (the pair inside the head) is the same for every item of a thread: 256 threads cover 4 (token, head) rows
    // of 64 pairs per sweep.  Loads of kBatch sweeps are issued together so that their latencies overlap.
    const int p = tid & 63;
    int i0, i1, cs_stream = 0, cs_ladder = 0;
    const bool rotated = p < n_pairs;
    if (rotated) {
        const RopePair rp = rope_pair(sh.rope_type, kD, p);
        i0 = rp.i0; i1 = rp.i1; cs_stream = rp.stream; cs_ladder = rp.ladder;
    } else {
        const int first_free = sh.rope_type == CGLM_ROPE_CHATGLM2 ? kD / 2 : 0;
        i0 = first_free + 2 * (p - n_pairs); i1 = i0 + 1;
    }
    constexpr int kBatch = 8;
    const bool v1 = sh.rope_type == CGLM_ROPE_CHATGLM;
    const int v1_lim = sq.n_ctx - 2;
    // table_by_position: the arena's table, row = position (or block position) of the token; otherwise the table
    // rope_table_kernel wrote for this call, row = (stream, token)
    const float2 *tab = table_by_position ? table + cs_ladder : table + (static_cast<long long>(cs_stream) * S + t_begin) * 32 + cs_ladder;
    for (int hi = 0; hi < n_heads; ++hi) {
        const int hh = head0 + hi;
        const float *src_base = is_q ? sq.q : sq.k;
        const long long head_off = is_q ? hh * sq.q_head_stride : hh * sq.kv_head_stride;
        const long long tok_stride = is_q ? sq.q_tok_stride : sq.kv_tok_stride;
        for (int t0 = tid >> 6; t0 < n_tok; t0 += 4 * kBatch) {
            float x0[kBatch], x1[kBatch];
            float2 cs[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int t = t0 + 4 * u;
                x0[u] = x1[u] = 0.f;
                cs[u] = make_float2(1.f, 0.f);
                if (t < n_tok) {
                    const long long src = head_off + (t_begin + t) * tok_stride;
                    x0[u] = ld_act(src_base, src + i0, in_f16);
                    x1[u] = ld_act(src_base, src + i1, in_f16);
                    if (rotated) {
                        // derived ids (chatglm.cpp:1142-1153, 1319-1327 with n_past = 0), as selects: a branch here
                        // would split the batch of loads into one round trip per token
                        const int s_tok = t_begin + t;
                        const int by_pos = v1 ? (cs_stream ? max(s_tok - v1_lim, 0) : min(s_tok, v1_lim)) : s_tok;
                        const int row = table_by_position ? by_pos : t;
                        cs[u] = __ldg(tab + row * 32);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int t = t0 + 4 * u;
                if (t >= n_tok) continue;
                const int s = t_begin + t;
                float y0 = x0[u], y1 = x1[u];
                if (rotated) rope_rotate(x0[u], x1[u], cs[u].x, cs[u].y, y0, y1);
                if (is_q) {
                    __half *dst = q_half + (static_cast<long long>(hh) * s_pad + s) * kD;
                    if (i1 == i0 + 1) {   // adjacent pair: one 4-byte store
                        *reinterpret_cast<__half2 *>(dst + i0) =
                            __halves2half2(__float2half_rn(__fmul_rn(y0, sh.scale)), __float2half_rn(__fmul_rn(y1, sh.scale)));
                    } else {
                        dst[i0] = __float2half_rn(__fmul_rn(y0, sh.scale));
                        dst[i1] = __float2half_rn(__fmul_rn(y1, sh.scale));
                    }
                    if (sq.q_roped) {
                        float *qr = sq.q_roped + (static_cast<long long>(s) * H + hh) * kD;
                        qr[i0] = y0; qr[i1] = y1;
                    }
                } else {
                    uint16_t *krow = k_base + (static_cast<long long>(sq.slot * G + hh) * M + sq.kv_before + s) * kD;
                    if (i1 == i0 + 1) {
                        *reinterpret_cast<__half2 *>(krow + i0) = __halves2half2(__float2half_rn(y0), __float2half_rn(y1));
                    } else {
                        krow[i0] = __half_as_ushort(__float2half_rn(y0));
                        krow[i1] = __half_as_ushort(__float2half_rn(y1));
                    }
                    if (sq.k_roped) {
                        float *kr = sq.k_roped + (static_cast<long long>(s) * G + hh) * kD;
                        kr[i0] = y0; kr[i1] = y1;
                    }
                }
            }
        }
    }
}

// ---- launch 2: attention ----------------------------------------------------------------------------------------
// q_map: f16 {D, s_pad, H}, box 64 x 128.  k_map: f16 {D, L, slots*G}, box 64 x 128.  v_map: f16 {L, slots*G*D},
// box 64 x 128.  L = n_virtual + S is the attended length of the last row.
//
// Buffer hand-offs for KV tile j (b = j & 1; every barrier is used once per two tiles, parity (j >> 1) & 1):
//   k_full[b]   TMA            -> control   K[b] landed      (K[b] is reloaded as soon as S(j) has completed)
//   v_full[b]   TMA            -> control   V^T[b] landed    (V^T[b] is reloaded once P V(j) has completed)
//   s_done[b]   tensor core    -> both      S[b] = Q K^T(j) written; K[b] has been read
//   p_ready[b]  softmax (x4)   -> control   P[b] written (and S[b] read): P V(j) may be issued, S[b] may be reused
//   o_done[b]   tensor core    -> both      O += P V(j) done; K/V^T[b] and P[b] have been read
__global__ void __launch_bounds__(kThreads, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, AttnShape sh, int S, int kv_row0, float *__restrict__ out,
                    int out_f16, WsHeader *hdr) {
    extern __shared__ uint8_t smem_raw[];
    PrefillSmem &sm = *reinterpret_cast<PrefillSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // A CTA takes q tile (n_q - 1 - x) and then q tile x of one head: under the causal mask the first sees the most
    // KV tiles and the second the fewest, so every CTA of the grid has the same amount of work.
    const int h = blockIdx.y;
    const int n_q = (S + kQTile - 1) / kQTile;
    const int V = sh.V, L = V + S;
    const int kv_row = kv_row0 + h / sh.R;
    const bool causal = sh.mask_type == CGLM_MASK_CAUSAL;
    const int q_tiles[2] = {n_q - 1 - static_cast<int>(blockIdx.x), static_cast<int>(blockIdx.x)};
    const int n_pass = q_tiles[0] == q_tiles[1] ? 1 : 2;
    auto kv_tiles_of = [&](int q_tile) {
        const int last_visible = causal ? min(L, V + q_tile * kQTile + kQTile) : L;   // one past the last visible token
        return (last_visible + kKvTile - 1) / kKvTile;
    };

    if (tid == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.q_full, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.k_full[b], 1);
            mbar_init(&sm.v_full[b], 1);
            mbar_init(&sm.s_done[b], 1);
            mbar_init(&sm.p_ready[b], kSoftmaxThreads / 32);
            mbar_init(&sm.o_done[b], 1);
        }
        fence_mbar_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    // Launched as a programmatic dependent of the prepare kernel: everything above overlapped its tail; its q, K and
    // V^T are read from here on.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // j: running tile count of the CTA (buffer j & 1, barrier parity (j >> 1) & 1); jl: KV tile index inside a pass.
    // Loads, score MMAs and P V MMAs are issued by three different warps, each a plain loop over the tiles that
    // waits only for what its own step needs: the next score tile is computed while the softmax warps work on the
    // current one, P V(j) follows as soon as they are done, and no step queues behind another step's barrier.
    if (warp == kLoadWarp) {
        // ================================ load warp: TMA ===================================================
        if (lane == 0) {
            tma_prefetch_desc(&q_map);
            tma_prefetch_desc(&k_map);
            tma_prefetch_desc(&v_map);
        }
        int jt0 = 0;
        for (int pass = 0; pass < n_pass; ++pass) {
            const int s0 = q_tiles[pass] * kQTile;
            const int n_kv = kv_tiles_of(q_tiles[pass]);
            if (lane == 0) {
                mbar_arrive_expect_tx(&sm.q_full, kTileBytes);
                tma_load_3d(sm.q, &q_map, 0, s0, h, &sm.q_full);
                tma_load_3d(sm.q + kHalfBytes, &q_map, 64, s0, h, &sm.q_full);
                for (int jl = 0; jl < n_kv; ++jl) {
                    const int j = jt0 + jl, b = j & 1;
                    // K[b] was read by S(j-2), V^T[b] by P V(j-2); at the start of a pass both buffers are free
                    if (jl >= 2) mbar_wait_bounded(&sm.s_done[b], ((j - 2) >> 1) & 1u, &sm.abort_flag);
                    mbar_arrive_expect_tx(&sm.k_full[b], kTileBytes);
                    tma_load_3d(sm.k[b], &k_map, 0, jl * kKvTile, kv_row, &sm.k_full[b]);
                    tma_load_3d(sm.k[b] + kHalfBytes, &k_map, 64, jl * kKvTile, kv_row, &sm.k_full[b]);
                    if (jl >= 2) mbar_wait_bounded(&sm.o_done[b], ((j - 2) >> 1) & 1u, &sm.abort_flag);
                    mbar_arrive_expect_tx(&sm.v_full[b], kTileBytes);
                    tma_load_2d(sm.v[b], &v_map, jl * kKvTile, kv_row * kD, &sm.v_full[b]);
                    tma_load_2d(sm.v[b] + kHalfBytes, &v_map, jl * kKvTile + 64, kv_row * kD, &sm.v_full[b]);
                }
            }
            jt0 += n_kv;
            __syncwarp();
            if (pass + 1 < n_pass) {
                // the next pass reloads Q, K, V^T: every MMA of this pass must have read them, and the softmax
                // warps must be done with the output staging tile that overlays the K/V^T buffers
                named_bar_sync(2, kThreads);
            }
        }
    } else if (warp == kScoreWarp) {
        // ================================ score warp: one thread issues S(j) = Q K(j)^T ======================
        int jt0 = 0;
        for (int pass = 0; pass < n_pass; ++pass) {
            const int n_kv = kv_tiles_of(q_tiles[pass]);
            if (lane == 0) {
                mbar_wait_bounded(&sm.q_full, pass & 1u, &sm.abort_flag);
                for (int jl = 0; jl < n_kv; ++jl) {
                    const int j = jt0 + jl, b = j & 1;
                    mbar_wait_bounded(&sm.k_full[b], (j >> 1) & 1u, &sm.abort_flag);
                    // S[b] was last read by the softmax of tile j-2
                    if (jl >= 2) mbar_wait_bounded(&sm.p_ready[b], ((j - 2) >> 1) & 1u, &sm.abort_flag);
                    tc_fence_after();
#pragma unroll
                    for (int kh = 0; kh < 2; ++kh) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            umma_f16(tmem + 128 * b, smem_desc(smem_u32(sm.q) + kh * kHalfBytes + ks * 32),
                                     smem_desc(smem_u32(sm.k[b]) + kh * kHalfBytes + ks * 32), (kh | ks) != 0);
                        }
                    }
                    umma_commit(&sm.s_done[b]);
                }
            }
            jt0 += n_kv;
            __syncwarp();
            if (pass + 1 < n_pass) {
                named_bar_sync(2, kThreads);
            }
        }
    } else if (warp == kPvWarp) {
        // ================================ PV warp: one thread issues O (+)= P(j) V(j) =========================
        int jt0 = 0;
        for (int pass = 0; pass < n_pass; ++pass) {
            const int n_kv = kv_tiles_of(q_tiles[pass]);
            if (lane == 0) {
                for (int jl = 0; jl < n_kv; ++jl) {
                    const int j = jt0 + jl, b = j & 1;
                    // any rescale of O for the tile precedes p_ready
                    mbar_wait_bounded(&sm.v_full[b], (j >> 1) & 1u, &sm.abort_flag);
                    mbar_wait_bounded(&sm.p_ready[b], (j >> 1) & 1u, &sm.abort_flag);
                    tc_fence_after();
#pragma unroll
                    for (int th = 0; th < 2; ++th) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            umma_f16(tmem + 256, smem_desc(smem_u32(sm.p[b]) + th * kHalfBytes + ks * 32),
                                     smem_desc(smem_u32(sm.v[b]) + th * kHalfBytes + ks * 32), (jl | th | ks) != 0);
                        }
                    }
                    umma_commit(&sm.o_done[b]);
                }
            }
            jt0 += n_kv;
            __syncwarp();
            if (pass + 1 < n_pass) {
                named_bar_sync(2, kThreads);
            }
        }
    } else {
        // ================================ softmax warps: one q row per thread =================================
        const uint32_t lane_base = static_cast<uint32_t>(32 * warp) << 16;   // this warp's quarter of the TMEM lanes
        const uint32_t to = tmem + 256 + lane_base;
        int jt0 = 0;
      for (int pass = 0; pass < n_pass; ++pass) {
        const int s0 = q_tiles[pass] * kQTile;
        const int n_kv = kv_tiles_of(q_tiles[pass]);
        const int s_row = s0 + tid;             // this thread's q row (may lie past S in the last q tile)
        float m_ref = -INFINITY, l_run = 0.f;   // reference maximum (log2 domain) and row sum relative to it
        // the last token a row may attend (inclusive)
        const int row_last = causal ? min(L - 1, V + s_row) : (s_row < S - 1 ? L - 2 : L - 1);

        for (int jl = 0; jl < n_kv; ++jl) {
            const int j = jt0 + jl;
            const int b = j & 1;
            mbar_wait_bounded(&sm.s_done[b], (j >> 1) & 1u, &sm.abort_flag);
            tc_fence_after();
            const uint32_t ts = tmem + 128 * b + lane_base;
            const int t0 = jl * kKvTile;
            // the whole score row of this tile: 4 loads in flight, one wait
            float sv[kKvTile];
            {
                uint32_t *r = reinterpret_cast<uint32_t *>(sv);
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
                        "%14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(r[32 * ch + 0]), "=r"(r[32 * ch + 1]), "=r"(r[32 * ch + 2]), "=r"(r[32 * ch + 3]),
                          "=r"(r[32 * ch + 4]), "=r"(r[32 * ch + 5]), "=r"(r[32 * ch + 6]), "=r"(r[32 * ch + 7]),
                          "=r"(r[32 * ch + 8]), "=r"(r[32 * ch + 9]), "=r"(r[32 * ch + 10]), "=r"(r[32 * ch + 11]),
                          "=r"(r[32 * ch + 12]), "=r"(r[32 * ch + 13]), "=r"(r[32 * ch + 14]), "=r"(r[32 * ch + 15]),
                          "=r"(r[32 * ch + 16]), "=r"(r[32 * ch + 17]), "=r"(r[32 * ch + 18]), "=r"(r[32 * ch + 19]),
                          "=r"(r[32 * ch + 20]), "=r"(r[32 * ch + 21]), "=r"(r[32 * ch + 22]), "=r"(r[32 * ch + 23]),
                          "=r"(r[32 * ch + 24]), "=r"(r[32 * ch + 25]), "=r"(r[32 * ch + 26]), "=r"(r[32 * ch + 27]),
                          "=r"(r[32 * ch + 28]), "=r"(r[32 * ch + 29]), "=r"(r[32 * ch + 30]), "=r"(r[32 * ch + 31])
                        : "r"(ts + ch * 32)
                        : "memory");
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            }
            // raw scores stay in sv; the log2(e) factor is folded into the exponent's FMA below.  Four independent
            // chains each for the maximum and the sum: a 128-long dependent chain would cost more than the math.
            if (t0 + kKvTile - 1 > row_last) {   // the diagonal tile (or the v1 mask's last column): blank hidden tokens
#pragma unroll
                for (int i = 0; i < kKvTile; ++i) {
                    sv[i] = t0 + i <= row_last ? sv[i] : -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < kKvTile; i += 8) {
                mx4[0] = max3(mx4[0], sv[i], sv[i + 1]); mx4[1] = max3(mx4[1], sv[i + 2], sv[i + 3]);
                mx4[2] = max3(mx4[2], sv[i + 4], sv[i + 5]); mx4[3] = max3(mx4[3], sv[i + 6], sv[i + 7]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * kLog2e;
            // keep the old reference unless the maximum outgrew it by more than the threshold
            const bool grow = mx > m_ref + kRescaleThreshold;   // also true for the first visible tile (m_ref = -inf)
            const float m_new = grow ? mx : m_ref;
            const float alpha = grow ? ex2_approx(m_ref - m_new) : 1.f;   // 0 when m_ref was -inf
            if (jl > 0 && __any_sync(0xffffffffu, grow)) {
                // rescale this warp's rows of O in tensor memory; P V(j-1) must have landed first
                mbar_wait_bounded(&sm.o_done[(j - 1) & 1], ((j - 1) >> 1) & 1u, &sm.abort_flag);
                tc_fence_after();
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    float ov[32];
                    tmem_ld32(to + ch * 32, ov);
                    asm volatile(
                        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
                        "%14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                        ::"r"(to + ch * 32), "f"(ov[0] * alpha), "f"(ov[1] * alpha), "f"(ov[2] * alpha), "f"(ov[3] * alpha),
                          "f"(ov[4] * alpha), "f"(ov[5] * alpha), "f"(ov[6] * alpha), "f"(ov[7] * alpha), "f"(ov[8] * alpha),
                          "f"(ov[9] * alpha), "f"(ov[10] * alpha), "f"(ov[11] * alpha), "f"(ov[12] * alpha),
                          "f"(ov[13] * alpha), "f"(ov[14] * alpha), "f"(ov[15] * alpha), "f"(ov[16] * alpha),
                          "f"(ov[17] * alpha), "f"(ov[18] * alpha), "f"(ov[19] * alpha), "f"(ov[20] * alpha),
                          "f"(ov[21] * alpha), "f"(ov[22] * alpha), "f"(ov[23] * alpha), "f"(ov[24] * alpha),
                          "f"(ov[25] * alpha), "f"(ov[26] * alpha), "f"(ov[27] * alpha), "f"(ov[28] * alpha),
                          "f"(ov[29] * alpha), "f"(ov[30] * alpha), "f"(ov[31] * alpha)
                        : "memory");
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            const float m_base = m_new == -INFINITY ? 0.f : m_new;   // a row that has seen nothing yet: every p is 0
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            // P[b] was last read by P V(j-2), issued by another thread than S(j): wait for it explicitly
            if (jl >= 2) mbar_wait_bounded(&sm.o_done[b], ((j - 2) >> 1) & 1u, &sm.abort_flag);
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float e0, e1;
                    fma2(e0, e1, sv[ch * 32 + i], sv[ch * 32 + i + 1], kLog2e, -m_base);   // masked scores are -inf: p = 0
                    const float p0 = ex2_approx(e0), p1 = ex2_approx(e1);
                    add2(sum4[2 * ((i >> 1) & 1)], sum4[2 * ((i >> 1) & 1) + 1], p0, p1);
                    packed[i >> 1] = pack_half2(p0, p1);
                }
                // tokens [32ch, 32ch+32) of the tile: half = ch / 2, 16-byte chunks (ch % 2) * 4 .. +3 of the 128-byte row
                const uint32_t rowaddr = smem_u32(sm.p[b]) + (ch >> 1) * kHalfBytes + tid * 128;
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    const int chunk = (ch & 1) * 4 + c4;
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + ((chunk ^ (tid & 7)) << 4)),
                                 "r"(packed[4 * c4]), "r"(packed[4 * c4 + 1]), "r"(packed[4 * c4 + 2]),
                                 "r"(packed[4 * c4 + 3])
                                 : "memory");
                }
            }
            l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            m_ref = m_new;
            fence_proxy_async();      // P was written with plain stores, the tensor core reads it through the async proxy
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_ready[b]);
        }
        // all of O has been accumulated once the last P V has landed
        mbar_wait_bounded(&sm.o_done[(jt0 + n_kv - 1) & 1], ((jt0 + n_kv - 1) >> 1) & 1u, &sm.abort_flag);
        tc_fence_after();

        // ---- output: context_layer[s][h*D + d] (chatglm.cpp:712-717), staged through shared memory so that the
        //      global stores of a warp cover whole rows.  All MMAs have completed: the K/V^T buffers are free. ------
        named_bar_sync(1, kSoftmaxThreads);
        float *stage = reinterpret_cast<float *>(sm.k[0]);
        const float inv = 1.f / l_run;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            float ov[32];
            tmem_ld32(to + ch * 32, ov);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                *reinterpret_cast<float4 *>(&stage[tid * kOutStride + ch * 32 + 4 * i]) =
                    make_float4(ov[4 * i] * inv, ov[4 * i + 1] * inv, ov[4 * i + 2] * inv, ov[4 * i + 3] * inv);
            }
        }
        named_bar_sync(1, kSoftmaxThreads);
        for (int r = warp; r < kQTile; r += kSoftmaxThreads / 32) {
            if (s0 + r < S) {
                const float4 val = *reinterpret_cast<const float4 *>(&stage[r * kOutStride + 4 * lane]);
                const long long o = (static_cast<long long>(s0 + r) * sh.H + h) * kD + 4 * lane;
                if (out_f16) {
                    *reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(out) + o) = make_uint2(pack_half2(val.x, val.y), pack_half2(val.z, val.w));
                } else {
                    *reinterpret_cast<float4 *>(out + o) = val;
                }
            }
        }
        jt0 += n_kv;
        if (pass + 1 < n_pass) {
            tc_fence_before();
            named_bar_sync(2, kThreads);   // pairs with the control warp: Q, K, V^T and the staging tile may be reused
            tc_fence_after();
        }
      }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
    if (sm.abort_flag && tid == 0) {
        atomicExch(&hdr->status, static_cast<int>(CGLM_ERR_TIMEOUT));
    }
}

}  // namespace

// staging of one prefill call: f16 q [H][s_pad][D], then the cos/sin table f32 [2][S][32][2]
static size_t prefill_q_bytes(int H, int S) {
    const int s_pad = (S + kQTile - 1) / kQTile * kQTile;
    return (static_cast<size_t>(H) * s_pad * kD * sizeof(__half) + 255) / 256 * 256;
}
size_t prefill_q_half_bytes(int H, int S) { return prefill_q_bytes(H, S) + static_cast<size_t>(2) * S * 32 * sizeof(float2); }

cudaError_t launch_prefill(const LaunchCtx &cx, const SeqDev &sq, const CUtensorMap &q_map, const CUtensorMap &k_map,
                           const CUtensorMap &v_map, __half *q_half) {
    const int S = sq.qlen;
    const int s_pad = (S + kQTile - 1) / kQTile * kQTile;
    static PerDeviceOnce configured;
    const int smem_bytes = static_cast<int>(sizeof(PrefillSmem)) + 1024;
    if (configured.needed(cx.device)) {
        cudaError_t e = require_current_device(cx.device);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(prefill_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        configured.mark(cx.device);
    }
    // Angles: positions derived from the token index lie inside the arena's table (one row per cache position);
    // explicit position ids may not, so a call that brings them gets a table of its own first.
    const float2 *table = cx.rope_tab;
    int table_by_position = 1;
    int launched = 2;
    if (rope_n_pairs_host(cx.shape.rope_type) > 0 && (sq.position_ids || !cx.rope_tab || S > cx.rope_tab_len)) {
        float2 *own = reinterpret_cast<float2 *>(reinterpret_cast<uint8_t *>(q_half) + prefill_q_bytes(cx.shape.H, S));
        const int n_entries = (cx.shape.rope_type == CGLM_ROPE_CHATGLM ? 2 : 1) * S * 32;
        rope_table_kernel<<<(n_entries + 255) / 256, 256, 0, cx.stream>>>(cx.shape, sq, own);
        table = own;
        table_by_position = 0;
        ++launched;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see griddepcontrol.wait in both kernels
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t pcfg = {};
    pcfg.gridDim = dim3((S + kPrepTokens - 1) / kPrepTokens, (cx.shape.H + 1) / 2 + 2 * cx.shape.G);
    pcfg.blockDim = dim3(kPrepThreads);
    pcfg.stream = cx.stream;
    pcfg.attrs = attr;
    pcfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&pcfg, prefill_prepare_kernel, cx.shape, sq, cx.k_base, cx.v_base, q_half, s_pad, table,
                                       table_by_position);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((s_pad / kQTile + 1) / 2, cx.shape.H);   // each CTA takes q tiles (n_q - 1 - x) and x
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = cx.stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, prefill_attn_kernel, q_map, k_map, v_map, cx.shape, S, sq.slot * cx.shape.G, sq.out,
                           (sq.flags & CGLM_SEQ_OUT_F16) ? 1 : 0, cx.hdr);
    g_launch_count += launched;
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace cglm
