// Prefill attention on 5th-generation tensor cores (tcgen05 + TMEM) for head_dim 128 (sm_100a).
//
// Covers chatglm.cpp:655-717 for a prompt (n_past == 0, qlen = S tokens) in two launches:
//   prefill_prepare_kernel  RoPE on q and k (:655-656), f16 append of the K rows and V^T columns (:668-675),
//                           q * 1/sqrt(d) (:686) written as an f16 [head][token][d] tile source;
//   prefill_attn_kernel     one CTA per (128-token q tile, q head): flash-attention forward over the freshly
//                           written cache.  S = Q K^T (128x128x128) and O_tile = P V (128x128x128) are tcgen05.mma
//                           instructions issued by one thread, operands staged in shared memory by TMA (K and V^T
//                           tiles, non-multicast, 128-byte swizzle, double buffered) or by the softmax threads (P),
//                           accumulators in tensor memory, read back with tcgen05.ld: each of the 128 threads owns
//                           one q row, so the online softmax needs no cross-thread reduction.
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
constexpr int kThreads = 128;
constexpr int kHalfBytes = 128 * 128;          // one 128-row x 128-byte swizzled half tile (16 KiB)
constexpr int kTileBytes = 2 * kHalfBytes;     // a 128 x 128 f16 operand tile
constexpr int kTmemCols = 256;                 // S: columns [0,128), O_tile: columns [128,256)
constexpr float kLog2e = 1.4426950408889634f;

// instruction descriptor of tcgen05.mma.kind::f16: D = f32, A = B = f16, both K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

struct __align__(1024) PrefillSmem {
    uint8_t q[kTileBytes];            // A of QK^T: [2 d-halves][128 rows][64 d]
    uint8_t k[2][kTileBytes];         // B of QK^T: [2 d-halves][128 tokens][64 d], double buffered
    uint8_t v[2][kTileBytes];         // B of PV:   [2 token-halves][128 d][64 tokens], double buffered
    uint8_t p[kTileBytes];            // A of PV:   [2 token-halves][128 rows][64 tokens]
    uint64_t q_full;
    uint64_t kv_full[2];
    uint64_t s_done;
    uint64_t o_done;
    uint32_t tmem_base;
    int abort_flag;
};

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
// One CTA per token.  q_half: f16 [H][s_pad][D], rows >= S are never read for an output.
__global__ void __launch_bounds__(128)
prefill_prepare_kernel(AttnShape sh, SeqDev sq, uint16_t *__restrict__ k_base, uint16_t *__restrict__ v_base,
                       __half *__restrict__ q_half, int s_pad) {
    __shared__ float cs[2][64][2];
    const int s = blockIdx.x;
    const int D = kD, H = sh.H, G = sh.G, M = sh.M;
    const int n_pairs = rope_n_pairs(sh.rope_type, D);
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
    for (int idx = threadIdx.x; idx < (H + G) * (D / 2); idx += blockDim.x) {
        const int head = idx / (D / 2), p = idx % (D / 2);
        const bool is_q = head < H;
        const int hh = is_q ? head : head - H;
        const float *src = is_q ? sq.q + s * sq.q_tok_stride + hh * sq.q_head_stride
                                : sq.k + s * sq.kv_tok_stride + hh * sq.kv_head_stride;
        int i0, i1;
        float y0, y1;
        if (p < n_pairs) {
            const RopePair rp = rope_pair(sh.rope_type, D, p);
            i0 = rp.i0; i1 = rp.i1;
            rope_rotate(src[i0], src[i1], cs[rp.stream][rp.ladder][0], cs[rp.stream][rp.ladder][1], y0, y1);
        } else {
            const int first_free = sh.rope_type == CGLM_ROPE_CHATGLM2 ? D / 2 : 0;
            i0 = first_free + 2 * (p - n_pairs); i1 = i0 + 1;
            y0 = src[i0]; y1 = src[i1];
        }
        if (is_q) {
            __half *dst = q_half + (static_cast<long long>(hh) * s_pad + s) * D;
            dst[i0] = __float2half_rn(__fmul_rn(y0, sh.scale));
            dst[i1] = __float2half_rn(__fmul_rn(y1, sh.scale));
            if (sq.q_roped) {
                float *qr = sq.q_roped + (static_cast<long long>(s) * H + hh) * D;
                qr[i0] = y0; qr[i1] = y1;
            }
        } else {
            uint16_t *krow = k_base + (static_cast<long long>(sq.slot * G + hh) * M + cache_pos) * D;
            krow[i0] = __half_as_ushort(__float2half_rn(y0));
            krow[i1] = __half_as_ushort(__float2half_rn(y1));
            if (sq.k_roped) {
                float *kr = sq.k_roped + (static_cast<long long>(s) * G + hh) * D;
                kr[i0] = y0; kr[i1] = y1;
            }
        }
    }
    for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
        const int g = idx / D, d = idx % D;
        const float x = sq.v[s * sq.kv_tok_stride + g * sq.kv_head_stride + d];
        v_base[(static_cast<long long>(sq.slot * G + g) * D + d) * M + cache_pos] = __half_as_ushort(__float2half_rn(x));
    }
}

// ---- launch 2: attention ----------------------------------------------------------------------------------------
// q_map: f16 {D, s_pad, H}, box 64 x 128.  k_map: f16 {D, L, slots*G}, box 64 x 128.  v_map: f16 {L, slots*G*D},
// box 64 x 128.  L = n_virtual + S is the attended length of the last row.
__global__ void __launch_bounds__(kThreads, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, AttnShape sh, int S, int kv_row0, float *__restrict__ out,
                    WsHeader *hdr) {
    extern __shared__ uint8_t smem_raw[];
    PrefillSmem &sm = *reinterpret_cast<PrefillSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5;
    const int q_tile = blockIdx.x, h = blockIdx.y;
    const int s0 = q_tile * kQTile;
    const int V = sh.V, L = V + S;
    const int kv_row = kv_row0 + h / sh.R;
    const bool causal = sh.mask_type == CGLM_MASK_CAUSAL;
    // KV tiles this q tile can see at all
    const int last_visible = causal ? min(L, V + s0 + kQTile) : L;   // one past the last visible token
    const int n_kv = (last_visible + kKvTile - 1) / kKvTile;

    if (tid == 0) {
        sm.abort_flag = 0;
        mbar_init(&sm.q_full, 1);
        mbar_init(&sm.kv_full[0], 1);
        mbar_init(&sm.kv_full[1], 1);
        mbar_init(&sm.s_done, 1);
        mbar_init(&sm.o_done, 1);
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
    const uint32_t tmem_s = tmem, tmem_o = tmem + 128;
    const uint32_t lane_base = static_cast<uint32_t>(32 * warp) << 16;   // this warp's quarter of the TMEM lanes

    auto load_kv = [&](int j) {   // thread 0 only
        const int b = j & 1;
        mbar_arrive_expect_tx(&sm.kv_full[b], 2 * kTileBytes);
        tma_load_3d(sm.k[b], &k_map, 0, j * kKvTile, kv_row, &sm.kv_full[b]);
        tma_load_3d(sm.k[b] + kHalfBytes, &k_map, 64, j * kKvTile, kv_row, &sm.kv_full[b]);
        tma_load_2d(sm.v[b], &v_map, j * kKvTile, kv_row * kD, &sm.kv_full[b]);
        tma_load_2d(sm.v[b] + kHalfBytes, &v_map, j * kKvTile + 64, kv_row * kD, &sm.kv_full[b]);
    };
    if (tid == 0) {
        tma_prefetch_desc(&q_map);
        tma_prefetch_desc(&k_map);
        tma_prefetch_desc(&v_map);
        mbar_arrive_expect_tx(&sm.q_full, kTileBytes);
        tma_load_3d(sm.q, &q_map, 0, s0, h, &sm.q_full);
        tma_load_3d(sm.q + kHalfBytes, &q_map, 64, s0, h, &sm.q_full);
        load_kv(0);
    }

    const int s_row = s0 + tid;             // this thread's q row (may lie past S in the last q tile)
    float o_acc[kD];
#pragma unroll
    for (int i = 0; i < kD; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    // the last token a row may attend (inclusive)
    const int row_last = causal ? min(L - 1, V + s_row) : (s_row < S - 1 ? L - 2 : L - 1);

    mbar_wait_bounded(&sm.q_full, 0, &sm.abort_flag);
    for (int j = 0; j < n_kv; ++j) {
        const int b = j & 1;
        if (tid == 0 && j + 1 < n_kv) {
            load_kv(j + 1);   // buffer (j+1)&1 was released by the o_done wait of tile j-1
        }
        mbar_wait_bounded(&sm.kv_full[b], (j >> 1) & 1u, &sm.abort_flag);
        tc_fence_after();
        // ---- S = Q K^T --------------------------------------------------------------------------------------
        if (tid == 0) {
#pragma unroll
            for (int kh = 0; kh < 2; ++kh) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    umma_f16(tmem_s, smem_desc(smem_u32(sm.q) + kh * kHalfBytes + ks * 32),
                             smem_desc(smem_u32(sm.k[b]) + kh * kHalfBytes + ks * 32), (kh | ks) != 0);
                }
            }
            umma_commit(&sm.s_done);
        }
        mbar_wait_bounded(&sm.s_done, j & 1u, &sm.abort_flag);
        tc_fence_after();
        // ---- online softmax of this thread's row, P -> shared memory ----------------------------------------
        const int t0 = j * kKvTile;
        float mx = -INFINITY;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            float sv[32];
            tmem_ld32(tmem_s + lane_base + ch * 32, sv);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int t = t0 + ch * 32 + i;
                mx = fmaxf(mx, t <= row_last ? sv[i] : -INFINITY);
            }
        }
        const float m_new = fmaxf(m_run, mx * kLog2e);
        // a row that sees nothing in this tile (only rows past S, or a fully masked tile) keeps m = -inf: use 0 as base
        const float m_base = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = ex2_approx(m_run - m_base);
        float row_sum = 0.f;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            float sv[32];
            tmem_ld32(tmem_s + lane_base + ch * 32, sv);
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const int t = t0 + ch * 32 + i;
                const float p0 = t <= row_last ? ex2_approx(sv[i] * kLog2e - m_base) : 0.f;
                const float p1 = t + 1 <= row_last ? ex2_approx(sv[i + 1] * kLog2e - m_base) : 0.f;
                row_sum += p0 + p1;
                packed[i >> 1] = pack_half2(p0, p1);
            }
            // tokens [32ch, 32ch+32) of the tile: half = ch / 2, 16-byte chunks (ch % 2) * 4 .. +3 of the 128-byte row
            const uint32_t rowaddr = smem_u32(sm.p) + (ch >> 1) * kHalfBytes + tid * 128;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const int chunk = (ch & 1) * 4 + c4;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + ((chunk ^ (tid & 7)) << 4)),
                             "r"(packed[4 * c4]), "r"(packed[4 * c4 + 1]), "r"(packed[4 * c4 + 2]), "r"(packed[4 * c4 + 3])
                             : "memory");
            }
        }
        l_run = l_run * alpha + row_sum;
        m_run = m_new;
        fence_proxy_async();      // P was written with plain stores, the tensor core reads it through the async proxy
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        // ---- O_tile = P V -----------------------------------------------------------------------------------
        if (tid == 0) {
#pragma unroll
            for (int th = 0; th < 2; ++th) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    umma_f16(tmem_o, smem_desc(smem_u32(sm.p) + th * kHalfBytes + ks * 32),
                             smem_desc(smem_u32(sm.v[b]) + th * kHalfBytes + ks * 32), (th | ks) != 0);
                }
            }
            umma_commit(&sm.o_done);
        }
        mbar_wait_bounded(&sm.o_done, j & 1u, &sm.abort_flag);
        tc_fence_after();
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            float ov[32];
            tmem_ld32(tmem_o + lane_base + ch * 32, ov);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                o_acc[ch * 32 + i] = o_acc[ch * 32 + i] * alpha + ov[i];
            }
        }
        tc_fence_before();
        __syncthreads();   // every thread is done with S, O_tile, P and the K/V buffer before they are reused
        tc_fence_after();
    }
    // ---- output: context_layer[s][h*D + d] (chatglm.cpp:712-717) ---------------------------------------------------
    if (s_row < S) {
        const float inv = 1.f / l_run;
        float4 *op = reinterpret_cast<float4 *>(out + (static_cast<long long>(s_row) * sh.H + h) * kD);
#pragma unroll
        for (int i = 0; i < kD / 4; ++i) {
            op[i] = make_float4(o_acc[4 * i] * inv, o_acc[4 * i + 1] * inv, o_acc[4 * i + 2] * inv, o_acc[4 * i + 3] * inv);
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

size_t prefill_q_half_bytes(int H, int S) {
    const int s_pad = (S + kQTile - 1) / kQTile * kQTile;
    return static_cast<size_t>(H) * s_pad * kD * sizeof(__half);
}

cudaError_t launch_prefill(const LaunchCtx &cx, const SeqDev &sq, const CUtensorMap &q_map, const CUtensorMap &k_map,
                           const CUtensorMap &v_map, __half *q_half) {
    const int S = sq.qlen;
    const int s_pad = (S + kQTile - 1) / kQTile * kQTile;
    static bool configured = false;
    const int smem_bytes = static_cast<int>(sizeof(PrefillSmem)) + 1024;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    prefill_prepare_kernel<<<S, 128, 0, cx.stream>>>(cx.shape, sq, cx.k_base, cx.v_base, q_half, s_pad);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    dim3 grid(s_pad / kQTile, cx.shape.H);
    prefill_attn_kernel<<<grid, kThreads, smem_bytes, cx.stream>>>(q_map, k_map, v_map, cx.shape, S, sq.slot * cx.shape.G,
                                                                  sq.out, cx.hdr);
    g_launch_count += 2;
    return cudaGetLastError();
}

}  // namespace cglm
