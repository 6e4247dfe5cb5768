// Shared device-side declarations of the attention KV-cache kernels (sm_100a).
#pragma once

#include <atomic>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cglm_attn.h"

namespace cglm {

// ---- workspace layout -------------------------------------------------------------------------------
// [0, 256)            control block (WsHeader)
// [256, ...)          item counters (int per (sequence, kv head)), partial slots, device copies of the
//                     sequence descriptors, roped/scaled q staging for the generic and prefill paths
struct WsHeader {
    unsigned int magic;   // kWsMagic once cglm_attn_workspace_init ran
    int status;           // sticky device-side status (0 or CGLM_ERR_*)
    int xchg_items;       // split-KV step: kv heads of this rank whose partial rows have been published (self-resetting)
    int reserved[61];
};
static_assert(sizeof(WsHeader) == 256, "control block is 256 bytes");
constexpr unsigned int kWsMagic = 0x5a5a5a5au;  // one byte repeated, so that a memset can write it

// Device-side copy of one cglm_attn_seq with everything resolved that the kernels would otherwise
// re-derive: cache row of the first kv head, attended length, rope positions.
struct SeqDev {
    const float *q, *k, *v;
    long long q_tok_stride, q_head_stride, kv_tok_stride, kv_head_stride;
    const int *position_ids;
    float *out;
    float *q_roped;
    float *k_roped;
    float *partial;
    int slot;
    int qlen;
    int n_past;
    int n_ctx;
    int kv_before;   // cached tokens attended besides the ones appended now (n_virtual + n_past, or kv_local)
    int flags;
    union {
        struct {
            int tok_begin;   // generic path: first row of this sequence in the staging buffers
            int pad;
        };
        const int *n_past_dev;   // fused decode with CGLM_SEQ_N_PAST_DEVICE: where the kernel reads n_past
    };
};
static_assert(sizeof(SeqDev) == 128, "descriptors travel as 32 words");

struct AttnShape {
    int H, G, D, R;       // heads, kv heads, head dim, H / G
    int M, V;             // cache capacity in tokens, virtual tokens
    int rope_type;
    int mask_type;
    float theta_scale;    // powf(base, -2 / n_dims) computed on the host with the C library's powf
    float scale;          // 1 / sqrtf(D)
};

// ---- bounded waiting --------------------------------------------------------------------------------
// Every device-side wait in this library gives up after kSpinLimit polls, records CGLM_ERR_TIMEOUT in the
// workspace status word and lets the kernel run to its end with invalid results instead of hanging.
constexpr unsigned int kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Returns false when the wait ran out (or an earlier wait of this CTA did): the caller carries on
// without touching the barrier again.  *abort_flag lives in shared memory.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    if (*abort_flag) {
        return false;
    }
    for (unsigned int i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((i & 1023u) == 1023u && *abort_flag) {
            return false;
        }
    }
    *abort_flag = 1;
    return false;
}

// ---- TMA (non-multicast tiled loads from this GPU's memory) -----------------------------------------
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int c0, int c1, int c2,
                                            uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- warp-level tensor-core pieces for the decode kernel ---------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void named_bar_sync(int id, int n_threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n_threads) : "memory");
}

// ---- activations: f32, or f16 with CGLM_SEQ_QKV_F16 / CGLM_SEQ_OUT_F16 (element indices either way) -----------------
__device__ __forceinline__ float ld_act(const float *base, long long e, bool f16) {
    return f16 ? __half2float(__ldg(reinterpret_cast<const __half *>(base) + e)) : __ldg(base + e);
}
__device__ __forceinline__ void st_out(float *base, long long e, bool f16, float x) {
    if (f16) reinterpret_cast<__half *>(base)[e] = __float2half_rn(x); else base[e] = x;
}

// ---- RoPE pieces shared by every kernel --------------------------------------------------------------
// Angle i of a position: theta_0 = pos, theta_{j+1} = theta_j * theta_scale, each product rounded to f32
// (the iterated ladder of ggml's rope cache).  cos/sin are taken in double and rounded once, which
// reproduces a correctly rounded f32 cosf/sinf in all but near-tie cases.
__device__ __forceinline__ void rope_cos_sin(int pos, int i, float theta_scale, float &c, float &s) {
    float theta = static_cast<float>(pos);
    for (int j = 0; j < i; ++j) {
        theta = __fmul_rn(theta, theta_scale);
    }
    double sd, cd;
    sincos(static_cast<double>(theta), &sd, &cd);
    c = static_cast<float>(cd);
    s = static_cast<float>(sd);
}
// The rotation keeps four products and two sums separately rounded (no FMA contraction), like the
// host oracle built with -ffp-contract=off.
__device__ __forceinline__ void rope_rotate(float x0, float x1, float c, float s, float &y0, float &y1) {
    y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    y1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

// Index bookkeeping of one rope mode: how many rotated pairs a head has, which two elements pair i
// touches, and which (position stream, ladder index) drives it.
struct RopePair {
    int i0, i1;     // element indices inside the head
    int stream;     // 0: position id, 1: block position id (CGLM_ROPE_CHATGLM only)
    int ladder;     // index into the angle ladder
};
__device__ __forceinline__ int rope_n_pairs(int rope_type, int D) {
    switch (rope_type) {
    case CGLM_ROPE_GPTJ:
    case CGLM_ROPE_NEOX:
    case CGLM_ROPE_CHATGLM: return D / 2;
    case CGLM_ROPE_CHATGLM2: return D / 4;
    default: return 0;
    }
}
// n_dims handed to ggml's rope for each mode: D for the basic modes, D/2 for both GLM modes.
__host__ __device__ __forceinline__ int rope_n_dims(int rope_type, int D) {
    return (rope_type == CGLM_ROPE_GPTJ || rope_type == CGLM_ROPE_NEOX) ? D : D / 2;
}
__device__ __forceinline__ RopePair rope_pair(int rope_type, int D, int p) {
    RopePair r;
    switch (rope_type) {
    case CGLM_ROPE_GPTJ:      // adjacent pairs over the whole head
    case CGLM_ROPE_CHATGLM2:  // adjacent pairs over the first half
        r.i0 = 2 * p; r.i1 = 2 * p + 1; r.stream = 0; r.ladder = p; break;
    case CGLM_ROPE_NEOX:      // (p, p + D/2)
        r.i0 = p; r.i1 = p + D / 2; r.stream = 0; r.ladder = p; break;
    default: {                // CGLM_ROPE_CHATGLM: halves of D/2, pairs (i, i + D/4) inside each
        const int q = D / 4, half = p / q, i = p % q;
        r.i0 = half * (D / 2) + i; r.i1 = r.i0 + q; r.stream = half; r.ladder = i; break;
    }
    }
    return r;
}
// Position ids of token s of a sequence when the caller passed none (chatglm.cpp:1142-1153, 1319-1327).
__device__ __forceinline__ void derive_positions(const SeqDev &sq, int rope_type, int s, int &pos, int &block) {
    const int p = sq.n_past + s;
    if (sq.position_ids) {
        pos = sq.position_ids[s];
        block = rope_type == CGLM_ROPE_CHATGLM ? sq.position_ids[sq.qlen + s] : 0;
    } else if (rope_type == CGLM_ROPE_CHATGLM) {
        pos = min(p, sq.n_ctx - 2);
        block = max(p - (sq.n_ctx - 2), 0);
    } else {
        pos = p;
        block = 0;
    }
}

// ---- split-KV exchange buffer (one per rank, in that rank's memory, mapped into every peer) ----------------------
// words: [0] step counter (the last step this rank combined), [1, 32) unused,
//        then 2 sets (alternating by step) of kXchgMaxRanks * kXchgMaxKvHeads arrival words [rank][kv head],
//        then 2 sets of n_rank partial slots of n_head * (head_dim + 2) floats (acc | m | l per q head).
constexpr int kXchgMaxRanks = 16;
constexpr int kXchgMaxKvHeads = 32;
constexpr int kXchgHeaderWords = 32;
__host__ __device__ inline size_t xchg_flag_word(int set, int rank, int g) {
    return kXchgHeaderWords + (static_cast<size_t>(set) * kXchgMaxRanks + rank) * kXchgMaxKvHeads + g;
}
__host__ __device__ inline size_t xchg_slot_word(int set, int rank, int n_rank, int slot_words) {
    return kXchgHeaderWords + 2 * kXchgMaxRanks * kXchgMaxKvHeads + (static_cast<size_t>(set) * n_rank + rank) * slot_words;
}
// What a fused split-KV step knows about the exchange (kernel parameter of the decode kernel's exchange instantiation).
struct XchgDev {
    unsigned int *peer[kXchgMaxRanks];   // every rank's buffer as mapped on this GPU; peer[rank] is the local one
    float *out;                          // combined context f32 [n_head * head_dim] (ranks that combine)
    int n_rank, rank;
    int combine;                         // 0: publish only (gather to the ranks that combine)
    unsigned int timeout_us;             // bound of the wait for the peers' arrival words
};

// ---- launchers implemented in the kernel translation units ------------------------------------------
struct LaunchCtx {
    AttnShape shape;
    uint16_t *k_base;            // arena K slabs: f16 [n_slots*G][M][D]
    uint16_t *v_base;            // arena V slabs: f16 [n_slots*G*D][M]
    WsHeader *hdr;
    int *counters;               // one per (sequence, kv head) of the decode list, zero between launches
    int *gcounters;              // two per group of 16 decode CTAs (long items merged in two levels)
    float *partials;             // decode split partials: 2 slots per CTA
    float *gpartials;            // decode group partials: 2 slots per group of 16 CTAs
    float *q_stage;              // generic path: roped, scaled q f32 [tokens][H][D]
    const CUtensorMap *k_map;    // host copies of the arena's tensor maps (passed by value to kernels)
    const CUtensorMap *v_map;
    const float2 *rope_tab;      // arena's angle table: [rope_tab_len positions][32 ladder steps] (cos, sin); may be null
    int rope_tab_len;
    cudaStream_t stream;
    int n_sm;
    int device;                  // ordinal of the arena's device, which must be the current one
};

// Per-function attributes (the opt-in to more than 48 KiB of dynamic shared memory) are per device: a process that
// drives several GPUs sets them once on each.  Returns true when `device` still needs its set-up; the caller then
// sets the attributes with that device current and calls device_setup_done.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
    std::atomic<bool> done[kMaxDevices];
    bool needed(int device) const { return device < 0 || device >= kMaxDevices || !done[device].load(std::memory_order_acquire); }
    void mark(int device) { if (device >= 0 && device < kMaxDevices) done[device].store(true, std::memory_order_release); }
};
// cudaErrorInvalidDevice unless `device` is the calling thread's current device
inline cudaError_t require_current_device(int device) {
    int cur = -1;
    cudaError_t e = cudaGetDevice(&cur);
    if (e != cudaSuccess) return e;
    return cur == device ? cudaSuccess : cudaErrorInvalidDevice;
}

// generic path (any head_dim <= 256, any cache capacity, prefill and decode, every rope and mask mode);
// seqs_dev[i].tok_begin indexes q_stage, total_tokens = sum of qlen
cudaError_t launch_generic(const LaunchCtx &cx, const SeqDev *seqs_dev, int n_seq, int total_tokens);
// fused rope + append + split-KV decode (head_dim 128, <= 16 q heads per kv head, capacity % 8 == 0)
constexpr int kDecodeTile = 64;   // tokens per TMA tile of the decode kernel
constexpr int kDecodeMaxSeqPerLaunch = 128;
// Everything the decode kernel needs to know about its sequences, passed by value as a kernel parameter so
// that no upload or load stands between the launch and its first memory request.
struct DecodeTable {
    int n_seq;
    int settled;   // 0, or 1 + tiles per CTA to pull into L2 ahead of the ring: every sequence carries CGLM_SEQ_CACHE_SETTLED
    int trigger;   // when a CTA releases the next kernel of the stream: 0 at its start, 1 last tile requested, 2 last tile consumed
    int charge;    // tiles a CTA's span is shortened by for every item start inside it (cost-balanced cut of the line)
    int prefix[kDecodeMaxSeqPerLaunch + 2];   // prefix[i] = 64-token tiles of sequences [0, i), per kv head
    SeqDev seqs[kDecodeMaxSeqPerLaunch];
    // Gates (host-buffer calls): device words that copy engines write, gate[i] null or a word that must hold
    // gate_value[i] before the launch reads its activations (0) / writes its outputs (1).  Every CTA's helper warp polls
    // them, with a bound, after the dependency wait; the stream itself carries no wait between two launches, so
    // consecutive launches keep their programmatic overlap.
    const unsigned int *gate[2];
    unsigned int gate_value[2];
};
// The table of a launch with device-side positions: what every CTA reads of EVERY sequence after the dependency wait,
// once more as arrays (decode_table_finish fills them): thread i reading seqs[i].flags touches one 128-byte descriptor
// per lane, and parameter space serves a warp one address at a time.  Only that instantiation takes the larger table
// (2.5 KiB more kernel parameters cost the other launches 0.4 us each, measured).
struct DecodeTableDyn : DecodeTable {
    int slot_of[kDecodeMaxSeqPerLaunch];
    int flags_of[kDecodeMaxSeqPerLaunch];
    int n_past_of[kDecodeMaxSeqPerLaunch];
    const int *n_past_dev_of[kDecodeMaxSeqPerLaunch];
};
inline void decode_table_finish(DecodeTableDyn &t) {
    for (int i = 0; i < t.n_seq; ++i) {
        t.slot_of[i] = t.seqs[i].slot;
        t.flags_of[i] = t.seqs[i].flags;
        t.n_past_of[i] = t.seqs[i].n_past;
        t.n_past_dev_of[i] = (t.seqs[i].flags & CGLM_SEQ_N_PAST_DEVICE) ? t.seqs[i].n_past_dev : nullptr;
    }
}
// xchg != null: the single sequence of tab is one rank's slice of a split-KV step (CGLM_SEQ_PARTIAL semantics); the
// kernel publishes its (acc, m, l) rows into every rank's exchange buffer and, on ranks that combine, merges them.
// n_past_on_device: tab must have been through decode_table_finish
cudaError_t launch_decode(const LaunchCtx &cx, const DecodeTableDyn &tab, bool n_past_on_device = false,
                          const XchgDev *xchg = nullptr);
// The decode kernel reads q/k/v head rows four elements at a time (sixteen bytes of f32, eight of f16) and writes the
// optional roped copies sixteen bytes at a time.
inline bool decode_rows_aligned(const float *q, const float *k, const float *v, long long q_head_stride,
                                long long kv_head_stride, const float *q_roped, const float *k_roped, bool qkv_f16 = false) {
    const uintptr_t in_bits = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v);
    const uintptr_t out_bits = reinterpret_cast<uintptr_t>(q_roped) | reinterpret_cast<uintptr_t>(k_roped);
    return (in_bits & (qkv_f16 ? 7 : 15)) == 0 && (out_bits & 15) == 0 && q_head_stride % 4 == 0 && kv_head_stride % 4 == 0;
}
// tcgen05 prefill (head_dim 128, n_past == 0, qlen >= 128): per-call tensor maps over the f16 q staging buffer
// [H][s_pad][D] and over the slot's caches cut at the attended length
size_t prefill_q_half_bytes(int H, int S);
cudaError_t launch_prefill(const LaunchCtx &cx, const SeqDev &sq, const CUtensorMap &q_map, const CUtensorMap &k_map,
                           const CUtensorMap &v_map, __half *q_half);
constexpr int kPrefillMinTokens = 128;
// fused query_key_value Linear + RoPE + append for one-token sequences (tcgen05): x_map f16 {64, n_tok, K/64} box
// {64, qkv_linear_x_rows(n_tok), kb}, w_map f16 {64, n_feat, K/64} box {64, 32, kb}, both 128-byte swizzled;
// kb (64-k blocks per box) <= qkv_linear_k_blocks(n_tok, K)
int qkv_linear_x_rows(int n_tok);
int qkv_linear_k_blocks(int n_tok, int K);
cudaError_t launch_qkv_linear(const LaunchCtx &cx, const CUtensorMap &x_map, const CUtensorMap &w_map, const int *slots,
                              const int *n_past, int n_tok, int K, int n_feat, int kb, const float *bias, float *q_out);
// the same GEMM with a plain epilogue: out f32 / f16 [n_tok][n_feat] = x . W^T + bias, any number of tokens (x box rows
// = qkv_linear_x_rows(min(n_tok, 128)), kb <= qkv_linear_k_blocks(min(n_tok, 128), K))
cudaError_t launch_linear_plain(int device, cudaStream_t stream, WsHeader *hdr, const CUtensorMap &x_map, const CUtensorMap &w_map,
                                int n_tok, int K, int n_feat, int kb, const float *bias, void *out, bool out_f16);
// The Linear with the output features on the M side of the MMA (n_feat a multiple of 128): k split over several CTAs per
// 128-feature tile, partial sums through `scratch` (kLinearScratchBytes at most), counters in WsHeader::reserved.
constexpr int kLinearFmMaxSplitTiles = 60;
constexpr size_t kLinearScratchBytes = static_cast<size_t>(148) * 128 * 128 * sizeof(float);   // 148 CTAs x [128 tokens][128 features]
struct LinearFmPlan {
    int n_box, tiles, token_tiles, ksplit, blocks_per_cta, kb, n_stages, tmem_cols;
};
bool linear_fm_plan(int n_tok, int K, int n_feat, int n_sm, size_t scratch_bytes, LinearFmPlan *plan);
cudaError_t launch_linear_fm(const LaunchCtx &cx, const LinearFmPlan &plan, const CUtensorMap &x_map, const CUtensorMap &w_map,
                             const int *slots, const int *n_past, int n_tok, int K, int n_feat, const float *bias, float *q_out,
                             void *out, bool out_f16, float *scratch);
int decode_max_ctas(int n_sm);
constexpr int kDecodeMergeFan = 16;   // CTAs per group of the two-level merge
constexpr int kDecodePartialFloats = 16 * 128 + 32;   // acc[16][128] | m[16] | l[16]

extern std::atomic<unsigned long long> g_launch_count;   // bumped from any host thread

}  // namespace cglm
