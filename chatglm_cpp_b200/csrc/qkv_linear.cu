// query_key_value Linear with the front half of the attention path in its epilogue, for decode-sized batches (sm_100a).
//
// Covers chatglm.cpp:629 (query_key_value.forward = ggml_mul_mat(weight, x) + bias, Linear::forward chatglm.cpp:418-426)
// together with what the attention path does to its result before any score is computed: RoPE on q and k
// (chatglm.cpp:655-656, GLM-2/3/4 half-rotary mode) and the f16 append of the K row and the V^T column at n_past
// (chatglm.cpp:668-675).  The fused qkv activation never reaches memory; what leaves the kernel is the roped q (f32,
// for the decode kernel, which then runs with CGLM_SEQ_Q_ROPED | CGLM_SEQ_NO_APPEND) and the two cache updates.
//
// One token per sequence, up to 128 sequences per launch.  The GEMM is C[token][feature] = x[token][:] . W[feature][:]
// with f16 operands and f32 accumulation on the 5th-generation tensor cores: the (zero-padded) 128 tokens are the M
// rows of tcgen05.mma, a CTA owns 32 output features (N = 32), so 4608 features of a GLM-4 layer are 144 CTAs, one per
// SM, each streaming its 32 x K slice of the weight exactly once.  Operands are staged by TMA (128-byte swizzle, K-major,
// 64 k per stage), the accumulator lives in 32 columns of tensor memory, and the epilogue reads it back with
// tcgen05.ld: thread t holds the 32 features of token t, so a rotary pair (2i, 2i+1) sits in one thread.
// A stage holds only as many x rows as there are tokens (rounded up to 8; the MMA still reads 128 rows, the rest is
// whatever the shared memory holds and lands in accumulator rows nobody reads) and `kb` consecutive 64-k blocks: both
// operands are described to TMA as 3-D tensors {64 k, rows, k blocks}, so ONE box brings kb blocks, which land as kb
// consecutive K-major tiles.  kb is as large as leaves two stages in the ring (8 blocks up to 64 tokens, 4 for 128).
// Measured (B200, 4608 x 4096 f16 weight, every call another layer's weight, the step replayed as a graph): with one
// 64-k block per box the kernel took 29 us per launch for 8, 64 and 128 tokens alike, one stage every 0.4 us
// whatever the ring depth (6 or 32 stages), the token count or the order in which the CTAs walk k, while the four
// MMAs of a stage cost 0.03 us each: the number of TMA operations was the limiter, not the bytes in flight.  With kb
// blocks per box: 17.3 / 18.2 / 23.1 us for 8 / 64 / 128 tokens (2.1 TB/s of weight stream at 64 tokens).  The first
// round of the ring is filled with weights before the dependency wait; x follows after it.
//
// The same kernel with a plain epilogue (kPlain) is Linear::forward itself, y = x . W^T + bias written as f32 or f16
// [token][feature]: the dense projection behind the attention path (chatglm.cpp:719, fed by the f16 context the
// attention kernels store with CGLM_SEQ_OUT_F16) and the query_key_value projection of prompts and of shapes the fused
// epilogue does not cover.  More than 128 tokens are a second grid dimension: every 128-token tile of a feature slice
// streams that slice of the weight again, from L2 after the first.
//
// Two kernels live here.  qkv_linear_kernel (tokens on the M side of the MMA, 32 features per CTA) takes any
// out-features that are a multiple of 32 and the fused epilogue for 33 .. 128 sequences; linear_fm_kernel (features on
// the M side, 128 per CTA, k split over the CTAs of a tile; further down) takes out-features that are a multiple of 128:
// the plain Linear at every size and the fused epilogue up to 32 sequences.
#include "common.cuh"

namespace cglm {

namespace {

constexpr int kTok = 128;            // M of the MMA: tokens, zero padded
constexpr int kFeat = 32;            // N of the MMA: output features per CTA
constexpr int kKStep = 64;           // k per stage: one 128-byte swizzled row of f16
constexpr int kMaxStages = 32;
constexpr int kXBytes = kTok * 128;  // what the MMA reads from an x tile: [128 tokens][64 k]
constexpr int kWBytes = kFeat * 128; // W tile [32 features][64 k]
// One CTA per SM with all of its shared memory (two per SM with half each, so that consecutive launches overlap, was
// measured: 17.0 / 20.1 / 30.0 us for 8 / 64 / 128 tokens against 17.7 / 18.7 / 23.8 us: box size matters more).
constexpr int kSmemPerCta = 232448;
// bytes the MMA reads past the end of the ring's last x tile that the W tiles behind it do not already cover
constexpr int read_over_slack(int x_rows, int kb) {
    return (kTok - x_rows) * 128 > kb * kWBytes ? (kTok - x_rows) * 128 - kb * kWBytes : 0;
}
constexpr int ring_stages(int x_rows, int kb) {
    return (kSmemPerCta - 2048 - read_over_slack(x_rows, kb)) / (kb * (x_rows * 128 + kWBytes));
}
constexpr int kThreads = 6 * 32;     // 4 epilogue warps (TMEM lanes 0..127), TMA warp, MMA warp
constexpr int kTmaWarp = 4, kMmaWarp = 5;
// instruction descriptor of tcgen05.mma.kind::f16: D = f32, A = B = f16, both K-major, N = 32, M = 128
constexpr uint32_t kIdesc = (1u << 4) | ((static_cast<uint32_t>(kFeat) >> 3) << 17) | ((128u >> 4) << 24);

struct __align__(1024) QkvSmem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full;
    uint32_t tmem_base;
    int abort_flag;
    // 1024-byte aligned: n_stages stages of (kb x tiles of x_rows rows | kb W tiles), then read_over_slack(): the MMA
    // reads 128 rows from every x tile, whatever x_rows is
    __align__(1024) uint8_t ring[1];
};

__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {   // K-major operand, 128-byte swizzle, 8-row groups 1024 B apart
    return static_cast<uint64_t>((saddr & 0x3ffffu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_f16_idesc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// What the kernel knows about its tokens (kernel parameter): cache slot and position of every sequence.
struct QkvTable {
    int n_tok;
    int slot[kTok];
    int n_past[kTok];
};

// Where the plain epilogue stores: out f32 or f16 [n_tok][n_feat].
struct PlainOut {
    void *out;
    int n_tok, n_feat, f16;
};

template <bool kPlain>
__global__ void __launch_bounds__(kThreads, 1)
qkv_linear_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                  const __grid_constant__ QkvTable tab, AttnShape sh, int K, int x_rows, int kb, int n_stages, const float *__restrict__ bias,
                  float *__restrict__ q_out, uint16_t *__restrict__ k_base, uint16_t *__restrict__ v_base,
                  const float2 *__restrict__ rope_tab, int rope_tab_len, WsHeader *hdr, PlainOut po) {
    extern __shared__ uint8_t smem_raw[];
    QkvSmem &sm = *reinterpret_cast<QkvSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int f0 = blockIdx.x * kFeat;        // first output feature of this CTA
    const int tok0 = kPlain ? static_cast<int>(blockIdx.y) * kTok : 0;   // first token of this CTA's tile
    const int n_k = K / (kKStep * kb);                       // stages of kb 64-k blocks each
    const int x_tile = x_rows * 128, x_bytes = kb * x_tile;   // kb x tiles, then kb W tiles
    const int stage_bytes = x_bytes + kb * kWBytes;
    const int k_first = static_cast<int>(blockIdx.x) % n_k;

    if (tid == 0) {
        sm.abort_flag = 0;
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        mbar_init(&sm.acc_full, 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(32) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    // x is the previous kernel's output (the layer's input norm) and the caches and q_out may still be read by it: only
    // the weights are touched before it has completed (the first round of the ring is filled with them ahead of the wait)

    if (warp == kTmaWarp) {
        if (lane == 0) {
            tma_prefetch_desc(&x_map);
            tma_prefetch_desc(&w_map);
            // CTA b walks k from its own starting column and wraps, so that the 4608 weight rows are not all read at the
            // same offset inside their 8 KiB at the same time
            const int pre = n_stages < n_k ? n_stages : n_k;
            for (int i = 0; i < pre; ++i) {
                mbar_arrive_expect_tx(&sm.full[i], stage_bytes);
                tma_load_3d(sm.ring + i * stage_bytes + x_bytes, &w_map, 0, f0, ((i + k_first) % n_k) * kb, &sm.full[i]);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            // rows of x past n_tok are outside the tensor map and arrive as zeros: the box is x_rows tokens
            for (int i = 0; i < pre; ++i) tma_load_3d(sm.ring + i * stage_bytes, &x_map, 0, tok0, ((i + k_first) % n_k) * kb, &sm.full[i]);
            for (int i = pre, st = 0, round = 1; i < n_k; ++i) {
                if (!mbar_wait_bounded(&sm.empty[st], (round - 1) & 1u, &sm.abort_flag)) break;
                uint8_t *stage = sm.ring + st * stage_bytes;
                mbar_arrive_expect_tx(&sm.full[st], stage_bytes);
                const int kk = (i + k_first) % n_k;
                tma_load_3d(stage, &x_map, 0, tok0, kk * kb, &sm.full[st]);
                tma_load_3d(stage + x_bytes, &w_map, 0, f0, kk * kb, &sm.full[st]);
                if (++st == n_stages) { st = 0; ++round; }
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            for (int i = 0, st = 0, round = 0; i < n_k; ++i) {
                if (!mbar_wait_bounded(&sm.full[st], round & 1u, &sm.abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t xs = smem_u32(sm.ring + st * stage_bytes), wsm = xs + x_bytes;
#pragma unroll 1
                for (int b = 0; b < kb; ++b) {
#pragma unroll
                    for (int ks = 0; ks < kKStep / 16; ++ks) {
                        umma_f16(tmem, smem_desc(xs + b * x_tile + ks * 32), smem_desc(wsm + b * kWBytes + ks * 32), (i | b | ks) != 0);
                    }
                }
                umma_commit(&sm.empty[st]);   // the stage may be refilled once these MMAs have read it
                if (++st == n_stages) { st = 0; ++round; }
            }
            umma_commit(&sm.acc_full);
        }
    } else {
        // ================================ epilogue: thread t = token t ==============================================
        const int tok = tid;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // before this thread writes q_out and the caches
        const bool ok = mbar_wait_bounded(&sm.acc_full, 0, &sm.abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float acc[kFeat];
        {
            uint32_t r[kFeat];
            const uint32_t taddr = tmem + (static_cast<uint32_t>(32 * warp) << 16);
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
            for (int i = 0; i < kFeat; ++i) acc[i] = __uint_as_float(r[i]);
        }
        if constexpr (kPlain) {
            const int row = tok0 + tok;
            if (ok && row < po.n_tok) {
                if (bias) {
#pragma unroll
                    for (int i = 0; i < kFeat; ++i) acc[i] = __fadd_rn(acc[i], __ldg(bias + f0 + i));
                }
                const long long at = static_cast<long long>(row) * po.n_feat + f0;
                if (po.f16) {
                    uint4 *dst = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(po.out) + at);
#pragma unroll
                    for (int i = 0; i < kFeat / 8; ++i) {
                        dst[i] = make_uint4(pack_half2(acc[8 * i], acc[8 * i + 1]), pack_half2(acc[8 * i + 2], acc[8 * i + 3]),
                                            pack_half2(acc[8 * i + 4], acc[8 * i + 5]), pack_half2(acc[8 * i + 6], acc[8 * i + 7]));
                    }
                } else {
                    float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(po.out) + at);
#pragma unroll
                    for (int i = 0; i < kFeat / 4; ++i) dst[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
                }
            }
        } else if (ok && tok < tab.n_tok) {
            const int H = sh.H, G = sh.G, D = sh.D;
            if (bias) {
#pragma unroll
                for (int i = 0; i < kFeat; ++i) acc[i] = __fadd_rn(acc[i], __ldg(bias + f0 + i));
            }
            // which part of the fused row these 32 features are (blocked layout, chatglm.cpp:646-652): a multiple of 32
            // never straddles a head (head_dim 128)
            const int q_feats = H * D, k_feats = G * D;
            const int kind = f0 < q_feats ? 0 : (f0 < q_feats + k_feats ? 1 : 2);
            const int rel = kind == 0 ? f0 : (kind == 1 ? f0 - q_feats : f0 - q_feats - k_feats);
            const int head = rel / D, d0 = rel % D;
            const int pos = tab.n_past[tok];
            if (kind != 2 && sh.rope_type == CGLM_ROPE_CHATGLM2 && d0 < D / 2) {
                // pairs (2i, 2i+1) of the first half of the head, ladder step i = (d0 + 2j) / 2 at this token's position
#pragma unroll
                for (int j = 0; j < kFeat / 2; ++j) {
                    const int li = d0 / 2 + j;
                    float c, s;
                    if (pos < rope_tab_len) {
                        const float2 cs = __ldg(rope_tab + static_cast<long long>(pos) * 32 + li);
                        c = cs.x; s = cs.y;
                    } else {
                        rope_cos_sin(pos, li, sh.theta_scale, c, s);
                    }
                    float y0, y1;
                    rope_rotate(acc[2 * j], acc[2 * j + 1], c, s, y0, y1);
                    acc[2 * j] = y0; acc[2 * j + 1] = y1;
                }
            }
            const long long row = static_cast<long long>(tab.slot[tok]) * G + head;   // cache row of (slot, kv head)
            const int cache_pos = sh.V + pos;
            if (kind == 0) {          // roped q, f32 [token][H * D]
                float4 *dst = reinterpret_cast<float4 *>(q_out + static_cast<long long>(tok) * q_feats + f0);
#pragma unroll
                for (int i = 0; i < kFeat / 4; ++i) dst[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
            } else if (kind == 1) {   // k_cache[row][cache_pos][d0 .. d0 + 32)
                uint4 *dst = reinterpret_cast<uint4 *>(k_base + (row * sh.M + cache_pos) * D + d0);
#pragma unroll
                for (int i = 0; i < kFeat / 8; ++i) {
                    dst[i] = make_uint4(pack_half2(acc[8 * i], acc[8 * i + 1]), pack_half2(acc[8 * i + 2], acc[8 * i + 3]),
                                        pack_half2(acc[8 * i + 4], acc[8 * i + 5]), pack_half2(acc[8 * i + 6], acc[8 * i + 7]));
                }
            } else {                  // v_cache[row][d0 + i][cache_pos]
                uint16_t *col = v_base + (row * D + d0) * sh.M + cache_pos;
#pragma unroll
                for (int i = 0; i < kFeat; ++i) col[static_cast<long long>(i) * sh.M] = __half_as_ushort(__float2half_rn(acc[i]));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32) : "memory");
    }
    if (sm.abort_flag && tid == 0) atomicExch(&hdr->status, static_cast<int>(CGLM_ERR_TIMEOUT));
}


// =====================================================================================================================
// The same Linear with the output features on the M side of the MMA (linear_fm_kernel).
//
// With the tokens on the M side every MMA reads a 128-row x operand from shared memory whether 8 or 128 tokens are real,
// and every CTA pulls all of x through L2 (512 KB for 64 tokens, twice its slice of the weight).  Here a CTA owns 128
// output features (the M rows; one head of a head_dim-128 model) and the tokens are the N columns (16 .. 128), so an
// MMA reads 4 KB of weight and 32 bytes per token.  128 features per CTA are only n_feat / 128 tiles (36 for a GLM-4
// query_key_value), too few CTAs to pull the weight from HBM, so the k range is split over `ksplit` CTAs per tile
// (36 x 4 = 144 CTAs): each writes its partial sums [token][128 features] to scratch in the workspace, the last one to
// arrive at the tile's counter adds the partials in split order (the same bits whatever the arrival order) and runs the
// epilogue.  Without a split (prompts: tiles x token tiles fill the GPU) the sums pass through shared memory instead.
// No CTA waits for another: the counter decides who finishes the tile.
constexpr int kFmFeat = 128;                 // M of the MMA: output features per CTA
constexpr int kFmWBytes = kFmFeat * 128;     // W tile of one 64-k block: [128 features][64 k] f16
constexpr int kFmMaxStages = 8;
constexpr int kFmBatch = 6;                  // (token, 4 features) items a thread has in flight in the finishing pass

struct __align__(1024) FmSmem {
    uint64_t full[kFmMaxStages];
    uint64_t empty[kFmMaxStages];
    uint64_t acc_full;
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
    // 1024-byte aligned: n_stages stages of (kb x tiles of n_box token rows | kb W tiles); after the last MMA the sums
    // [token][128] of an unsplit tile
    __align__(1024) uint8_t ring[1];
};

struct FmArgs {
    int K, n_tok, n_feat;
    int n_box;            // tokens per tile, a multiple of 16: rows of the x box and N of the MMA
    int kb, n_stages;     // 64-k blocks per TMA box, ring depth
    int blocks_per_cta;   // 64-k blocks one CTA sums over: K / 64 / ksplit
    int ksplit;
    int tmem_cols;        // power of two >= max(n_box, 32)
    const float *bias;
    float *scratch;       // ksplit > 1: partial sums [tile][split][n_box][128]
    int *tile_counters;   // ksplit > 1: arrivals per (token tile, feature tile), self-resetting
    WsHeader *hdr;
    void *out;            // plain epilogue: f32 or f16 [n_tok][n_feat]
    int out_f16;
    float *q_out;         // query_key_value epilogue
    uint16_t *k_base, *v_base;
    const float2 *rope_tab;
    int rope_tab_len;
};

template <bool kPlain>
__device__ __forceinline__ void fm_finish_item(const FmArgs &a, const QkvTable &tab, const AttnShape &sh, int f0, int tok, int q, float4 v) {
    const int f = f0 + 4 * q;
    if (a.bias) {
        const float4 b = __ldg(reinterpret_cast<const float4 *>(a.bias + f));
        v.x = __fadd_rn(v.x, b.x); v.y = __fadd_rn(v.y, b.y); v.z = __fadd_rn(v.z, b.z); v.w = __fadd_rn(v.w, b.w);
    }
    if constexpr (kPlain) {
        const long long at = static_cast<long long>(tok) * a.n_feat + f;
        if (a.out_f16) {
            *reinterpret_cast<uint2 *>(static_cast<uint16_t *>(a.out) + at) = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
        } else {
            *reinterpret_cast<float4 *>(static_cast<float *>(a.out) + at) = v;
        }
    } else {
        // a tile of 128 features is one head (head_dim 128) of the blocked layout (chatglm.cpp:646-652)
        const int H = sh.H, G = sh.G, D = sh.D;
        const int q_feats = H * D, k_feats = G * D;
        const int kind = f0 < q_feats ? 0 : (f0 < q_feats + k_feats ? 1 : 2);
        const int head = (kind == 0 ? f0 : (kind == 1 ? f0 - q_feats : f0 - q_feats - k_feats)) / D;
        const int d0 = 4 * q;
        const int pos = tab.n_past[tok];
        if (kind != 2 && sh.rope_type == CGLM_ROPE_CHATGLM2 && d0 < D / 2) {
            // pairs (d0, d0 + 1) and (d0 + 2, d0 + 3): ladder steps 2q and 2q + 1 at this token's position
            float c0, s0, c1, s1;
            if (pos < a.rope_tab_len) {
                const float4 cs = __ldg(reinterpret_cast<const float4 *>(a.rope_tab + static_cast<long long>(pos) * 32 + 2 * q));
                c0 = cs.x; s0 = cs.y; c1 = cs.z; s1 = cs.w;
            } else {
                rope_cos_sin(pos, 2 * q, sh.theta_scale, c0, s0);
                rope_cos_sin(pos, 2 * q + 1, sh.theta_scale, c1, s1);
            }
            float y0, y1;
            rope_rotate(v.x, v.y, c0, s0, y0, y1);
            v.x = y0; v.y = y1;
            rope_rotate(v.z, v.w, c1, s1, y0, y1);
            v.z = y0; v.w = y1;
        }
        const long long row = static_cast<long long>(tab.slot[tok]) * G + head;   // cache row of (slot, kv head)
        const int cache_pos = sh.V + pos;
        if (kind == 0) {          // roped q, f32 [token][H * D]
            *reinterpret_cast<float4 *>(a.q_out + static_cast<long long>(tok) * q_feats + f) = v;
        } else if (kind == 1) {   // k_cache[row][cache_pos][d0 .. d0 + 4)
            *reinterpret_cast<uint2 *>(a.k_base + (row * sh.M + cache_pos) * D + d0) = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
        } else {                  // v_cache[row][d0 + i][cache_pos]
            uint16_t *col = a.v_base + (row * D + d0) * sh.M + cache_pos;
            col[0] = __half_as_ushort(__float2half_rn(v.x));
            col[sh.M] = __half_as_ushort(__float2half_rn(v.y));
            col[2LL * sh.M] = __half_as_ushort(__float2half_rn(v.z));
            col[3LL * sh.M] = __half_as_ushort(__float2half_rn(v.w));
        }
    }
}

// Finishing pass of one tile by all threads of the CTA: item = (token, 4 consecutive features).  Every load of a batch of
// items (all splits) is issued before the first sum, so that a thread waits for L2 once per batch, not once per split;
// the splits are added in order, whoever arrived last.
template <bool kPlain, int kSplit>
__device__ __forceinline__ void fm_finish_tile(const FmArgs &a, const QkvTable &tab, const AttnShape &sh, const float *part0,
                                               size_t split_stride, int n_items, int f0, int tok0, int tid) {
    for (int base = tid; base < n_items; base += kThreads * kFmBatch) {
        float4 v[kFmBatch][kSplit];
#pragma unroll
        for (int u = 0; u < kFmBatch; ++u) {
            const int idx = base + u * kThreads;
#pragma unroll
            for (int s = 0; s < kSplit; ++s) {
                v[u][s] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (idx < n_items) {
                    const float4 *src = reinterpret_cast<const float4 *>(part0 + s * split_stride) + idx;
                    v[u][s] = kSplit > 1 ? __ldcg(src) : *src;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kFmBatch; ++u) {
            const int idx = base + u * kThreads;
            float4 t = v[u][0];
#pragma unroll
            for (int s = 1; s < kSplit; ++s) {
                t.x = __fadd_rn(t.x, v[u][s].x); t.y = __fadd_rn(t.y, v[u][s].y);
                t.z = __fadd_rn(t.z, v[u][s].z); t.w = __fadd_rn(t.w, v[u][s].w);
            }
            if (idx < n_items) fm_finish_item<kPlain>(a, tab, sh, f0, tok0 + (idx >> 5), idx & 31, t);
        }
    }
}

template <bool kPlain>
__global__ void __launch_bounds__(kThreads, 1)
linear_fm_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                 const __grid_constant__ QkvTable tab, const __grid_constant__ FmArgs a, AttnShape sh) {
    extern __shared__ uint8_t smem_raw[];
    FmSmem &sm = *reinterpret_cast<FmSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, split = blockIdx.y, ttile = blockIdx.z;
    const int f0 = tile * kFmFeat;
    const int tok0 = ttile * 128;                                   // token tiles are 128 wide when there are several
    const int n_real = a.n_tok - tok0 < a.n_box ? a.n_tok - tok0 : a.n_box;   // tokens of this tile that exist
    const int kb = a.kb, n_stages = a.n_stages;
    const int n_k = a.blocks_per_cta / kb;                          // ring stages this CTA fills in all
    const int k_base = split * a.blocks_per_cta;                    // first 64-k block of this CTA
    const int x_tile = a.n_box * 128, x_bytes = kb * x_tile;
    const int stage_bytes = x_bytes + kb * kFmWBytes;

    if (tid == 0) {
        sm.abort_flag = 0;
        sm.is_last = 1;
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        mbar_init(&sm.acc_full, 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    // x, the scratch and the outputs may still be in use by the previous kernel: only the weights are touched before it
    // has completed (the first round of the ring is filled with them ahead of the wait)

    if (warp == kTmaWarp) {
        if (lane == 0) {
            tma_prefetch_desc(&x_map);
            tma_prefetch_desc(&w_map);
            const int pre = n_stages < n_k ? n_stages : n_k;
            for (int i = 0; i < pre; ++i) {
                mbar_arrive_expect_tx(&sm.full[i], stage_bytes);
                tma_load_3d(sm.ring + i * stage_bytes + x_bytes, &w_map, 0, f0, k_base + i * kb, &sm.full[i]);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            // token rows past n_tok are outside the tensor map and arrive as zeros
            for (int i = 0; i < pre; ++i) tma_load_3d(sm.ring + i * stage_bytes, &x_map, 0, tok0, k_base + i * kb, &sm.full[i]);
            for (int i = pre, st = 0, round = 1; i < n_k; ++i) {
                if (!mbar_wait_bounded(&sm.empty[st], (round - 1) & 1u, &sm.abort_flag)) break;
                uint8_t *stage = sm.ring + st * stage_bytes;
                mbar_arrive_expect_tx(&sm.full[st], stage_bytes);
                tma_load_3d(stage, &x_map, 0, tok0, k_base + i * kb, &sm.full[st]);
                tma_load_3d(stage + x_bytes, &w_map, 0, f0, k_base + i * kb, &sm.full[st]);
                if (++st == n_stages) { st = 0; ++round; }
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            // D = f32, A = B = f16, both K-major, N = n_box, M = 128
            const uint32_t idesc = (1u << 4) | ((static_cast<uint32_t>(a.n_box) >> 3) << 17) | ((128u >> 4) << 24);
            for (int i = 0, st = 0, round = 0; i < n_k; ++i) {
                if (!mbar_wait_bounded(&sm.full[st], round & 1u, &sm.abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t xs = smem_u32(sm.ring + st * stage_bytes), wsm = xs + x_bytes;
#pragma unroll 1
                for (int b = 0; b < kb; ++b) {
#pragma unroll
                    for (int ks = 0; ks < kKStep / 16; ++ks) {
                        umma_f16_idesc(tmem, smem_desc(wsm + b * kFmWBytes + ks * 32), smem_desc(xs + b * x_tile + ks * 32), idesc, (i | b | ks) != 0);
                    }
                }
                umma_commit(&sm.empty[st]);   // the stage may be refilled once these MMAs have read it
                if (++st == n_stages) { st = 0; ++round; }
            }
            umma_commit(&sm.acc_full);
        }
    } else {
        // ===== warps 0..3: TMEM lane t = feature f0 + t, column j = token j; hand the sums on as [token][128] ==========
        asm volatile("griddepcontrol.wait;" ::: "memory");   // before this thread writes the scratch
        mbar_wait_bounded(&sm.acc_full, 0, &sm.abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float *dump = a.ksplit > 1
                          ? a.scratch + (static_cast<size_t>(ttile * gridDim.x + tile) * a.ksplit + split) * a.n_box * kFmFeat
                          : reinterpret_cast<float *>(sm.ring);
        const uint32_t taddr = tmem + (static_cast<uint32_t>(32 * warp) << 16);
        for (int c = 0; c < n_real; c += 16) {   // the same trip count in every thread
            uint32_t r[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
                "tcgen05.wait::ld.sync.aligned;"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                  "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr + static_cast<uint32_t>(c))
                : "memory");
#pragma unroll
            for (int j = 0; j < 16; ++j) dump[(c + j) * kFmFeat + tid] = __uint_as_float(r[j]);   // rows < n_box: inside the block
        }
        if (a.ksplit > 1) __threadfence();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (a.ksplit > 1) {
        if (tid == 0) {
            int *counter = a.tile_counters + ttile * gridDim.x + tile;
            const int last = atomicAdd(counter, 1) == a.ksplit - 1;
            if (last) *counter = 0;   // for the next launch; nobody else touches it any more
            sm.is_last = last;
        }
        __syncthreads();
    }
    if (sm.is_last && !sm.abort_flag) {
        if (a.ksplit > 1) __threadfence();
        // ===== all six warps: sum the splits in order, bias, epilogue; item = (token, 4 consecutive features) ===========
        const int n_items = n_real * (kFmFeat / 4);
        const size_t split_stride = static_cast<size_t>(a.n_box) * kFmFeat;
        const float *part0 = a.ksplit > 1 ? a.scratch + static_cast<size_t>(ttile * gridDim.x + tile) * a.ksplit * split_stride
                                          : reinterpret_cast<const float *>(sm.ring);
        switch (a.ksplit) {
        case 4: fm_finish_tile<kPlain, 4>(a, tab, sh, part0, split_stride, n_items, f0, tok0, tid); break;
        case 2: fm_finish_tile<kPlain, 2>(a, tab, sh, part0, split_stride, n_items, f0, tok0, tid); break;
        default: fm_finish_tile<kPlain, 1>(a, tab, sh, part0, split_stride, n_items, f0, tok0, tid); break;
        }
    }
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(a.tmem_cols) : "memory");
    }
    if (sm.abort_flag && tid == 0) atomicExch(&a.hdr->status, static_cast<int>(CGLM_ERR_TIMEOUT));
}
}  // namespace

int qkv_linear_x_rows(int n_tok) { return n_tok <= 8 ? 8 : (n_tok + 7) / 8 * 8; }
// 64-k blocks per TMA box: as many as leave two stages in the ring (measured: large boxes matter more than depth;
// 29 us per launch with one block per box and 32 stages, 18-20 us with 8 or 4 blocks per box)
int qkv_linear_k_blocks(int n_tok, int K) {
    const int x_rows = qkv_linear_x_rows(n_tok);
    for (int kb = 8; kb > 1; kb >>= 1) {
        if ((K / kKStep) % kb == 0 && ring_stages(x_rows, kb) >= 2) return kb;
    }
    return 1;
}

namespace {

cudaError_t configure_once(int device) {
    static PerDeviceOnce configured;
    if (!configured.needed(device)) return cudaSuccess;
    cudaError_t e = require_current_device(device);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(qkv_linear_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPerCta);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(qkv_linear_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPerCta);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_fm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPerCta);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(linear_fm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPerCta);
    if (e == cudaSuccess) configured.mark(device);
    return e;
}

}  // namespace

// x_map: f16 {64, n_tok, K/64}, box {64, qkv_linear_x_rows(n_tok), kb}; w_map: f16 {64, n_feat, K/64}, box {64, 32, kb};
// both 128-byte swizzled.
cudaError_t launch_qkv_linear(const LaunchCtx &cx, const CUtensorMap &x_map, const CUtensorMap &w_map, const int *slots,
                              const int *n_past, int n_tok, int K, int n_feat, int kb, const float *bias, float *q_out) {
    const int x_rows = qkv_linear_x_rows(n_tok), stage_bytes = kb * (x_rows * 128 + kWBytes);
    int n_stages = ring_stages(x_rows, kb);
    if (n_stages < 1) return cudaErrorInvalidValue;
    n_stages = n_stages > kMaxStages ? kMaxStages : n_stages;
    const int smem_bytes = 2048 + n_stages * stage_bytes + read_over_slack(x_rows, kb);
    static_assert(offsetof(QkvSmem, ring) == 1024, "header, then the ring");
    cudaError_t e = configure_once(cx.device);
    if (e != cudaSuccess) return e;
    static thread_local QkvTable tab;
    tab.n_tok = n_tok;
    for (int i = 0; i < n_tok; ++i) { tab.slot[i] = slots[i]; tab.n_past[i] = n_past[i]; }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_feat / kFeat);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = cx.stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, qkv_linear_kernel<false>, x_map, w_map, tab, cx.shape, K, x_rows, kb, n_stages, bias, q_out, cx.k_base,
                           cx.v_base, cx.rope_tab, cx.rope_tab_len, cx.hdr, PlainOut{});
    g_launch_count += 1;
    return e != cudaSuccess ? e : cudaGetLastError();
}

// Plain Linear: out f32 / f16 [n_tok][n_feat] = x . W^T + bias.  x_map: f16 {64, n_tok, K/64} with box
// {64, qkv_linear_x_rows(min(n_tok, 128)), kb}; w_map as above.  n_feat a multiple of 32, K of 64 * kb.
cudaError_t launch_linear_plain(int device, cudaStream_t stream, WsHeader *hdr, const CUtensorMap &x_map, const CUtensorMap &w_map,
                                int n_tok, int K, int n_feat, int kb, const float *bias, void *out, bool out_f16) {
    const int x_rows = qkv_linear_x_rows(n_tok < kTok ? n_tok : kTok), stage_bytes = kb * (x_rows * 128 + kWBytes);
    int n_stages = ring_stages(x_rows, kb);
    if (n_stages < 1) return cudaErrorInvalidValue;
    n_stages = n_stages > kMaxStages ? kMaxStages : n_stages;
    const int smem_bytes = 2048 + n_stages * stage_bytes + read_over_slack(x_rows, kb);
    cudaError_t e = configure_once(device);
    if (e != cudaSuccess) return e;
    static thread_local QkvTable tab;   // the plain epilogue reads none of it
    tab.n_tok = 0;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_feat / kFeat, (n_tok + kTok - 1) / kTok);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PlainOut po;
    po.out = out; po.n_tok = n_tok; po.n_feat = n_feat; po.f16 = out_f16 ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, qkv_linear_kernel<true>, x_map, w_map, tab, AttnShape{}, K, x_rows, kb, n_stages, bias,
                           static_cast<float *>(nullptr), static_cast<uint16_t *>(nullptr), static_cast<uint16_t *>(nullptr),
                           static_cast<const float2 *>(nullptr), 0, hdr, po);
    g_launch_count += 1;
    return e != cudaSuccess ? e : cudaGetLastError();
}

// ---- features on the M side: plan and launch -------------------------------------------------------------------------
bool linear_fm_plan(int n_tok, int K, int n_feat, int n_sm, size_t scratch_bytes, LinearFmPlan *p) {
    if (n_tok <= 0 || K % kKStep != 0 || n_feat % kFmFeat != 0) return false;
    const int tiles = n_feat / kFmFeat, ttiles = (n_tok + 127) / 128;
    p->n_box = n_tok > 128 ? 128 : (n_tok + 15) / 16 * 16;
    p->tiles = tiles;
    p->token_tiles = ttiles;
    // split k while the CTAs of all tiles still run at once; a split tile needs a counter in the workspace header and
    // scratch for its partial sums
    p->ksplit = 1;
    for (int sp = 4; sp >= 2; sp >>= 1) {
        const long long ctas = static_cast<long long>(tiles) * ttiles * sp;
        if (ctas <= n_sm && (K / kKStep) % sp == 0 && tiles * ttiles <= kLinearFmMaxSplitTiles &&
            static_cast<size_t>(ctas) * p->n_box * kFmFeat * sizeof(float) <= scratch_bytes) {
            p->ksplit = sp;
            break;
        }
    }
    p->blocks_per_cta = K / kKStep / p->ksplit;
    const int ring = kSmemPerCta - 2048;
    p->kb = 1;
    for (int kb = 4; kb > 1; kb >>= 1) {
        if (p->blocks_per_cta % kb == 0 && ring / (kb * (p->n_box * 128 + kFmWBytes)) >= 2) {
            p->kb = kb;
            break;
        }
    }
    const int stage_bytes = p->kb * (p->n_box * 128 + kFmWBytes);
    int n_stages = ring / stage_bytes;
    if (n_stages > kFmMaxStages) n_stages = kFmMaxStages;
    if (n_stages > p->blocks_per_cta / p->kb) n_stages = p->blocks_per_cta / p->kb;
    if (n_stages < 1) return false;
    p->n_stages = n_stages;
    p->tmem_cols = p->n_box <= 32 ? 32 : (p->n_box <= 64 ? 64 : 128);
    // an unsplit tile hands its sums [n_box][128] f32 through the ring
    if (p->ksplit == 1 && n_stages * stage_bytes < p->n_box * kFmFeat * static_cast<int>(sizeof(float))) return false;
    return true;
}

// x_map: f16 {64, n_tok, K/64}, box {64, plan.n_box, plan.kb}; w_map: f16 {64, n_feat, K/64}, box {64, 128, plan.kb}; both
// 128-byte swizzled.  slots / n_past non-null: query_key_value epilogue (q_out, caches of cx); null: plain (out).
cudaError_t launch_linear_fm(const LaunchCtx &cx, const LinearFmPlan &plan, const CUtensorMap &x_map, const CUtensorMap &w_map,
                             const int *slots, const int *n_past, int n_tok, int K, int n_feat, const float *bias, float *q_out,
                             void *out, bool out_f16, float *scratch) {
    cudaError_t e = configure_once(cx.device);
    if (e != cudaSuccess) return e;
    static_assert(offsetof(FmSmem, ring) == 1024, "header, then the ring");
    static thread_local QkvTable tab;
    tab.n_tok = slots ? n_tok : 0;
    if (slots) {
        for (int i = 0; i < n_tok; ++i) { tab.slot[i] = slots[i]; tab.n_past[i] = n_past[i]; }
    }
    FmArgs a;
    a.K = K; a.n_tok = n_tok; a.n_feat = n_feat;
    a.n_box = plan.n_box; a.kb = plan.kb; a.n_stages = plan.n_stages; a.blocks_per_cta = plan.blocks_per_cta;
    a.ksplit = plan.ksplit; a.tmem_cols = plan.tmem_cols;
    a.bias = bias;
    a.scratch = scratch;
    a.tile_counters = cx.hdr->reserved;
    a.hdr = cx.hdr;
    a.out = out; a.out_f16 = out_f16 ? 1 : 0;
    a.q_out = q_out; a.k_base = cx.k_base; a.v_base = cx.v_base; a.rope_tab = cx.rope_tab; a.rope_tab_len = cx.rope_tab_len;
    const int smem_bytes = 2048 + plan.n_stages * plan.kb * (plan.n_box * 128 + kFmWBytes);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.tiles, plan.ksplit, plan.token_tiles);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = cx.stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (slots) {
        e = cudaLaunchKernelEx(&cfg, linear_fm_kernel<false>, x_map, w_map, tab, a, cx.shape);
    } else {
        e = cudaLaunchKernelEx(&cfg, linear_fm_kernel<true>, x_map, w_map, tab, a, AttnShape{});
    }
    g_launch_count += 1;
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace cglm
