// C ABI of the attention KV-cache path: argument checking, the KV arena, workspace layout, dispatch of each
// sequence to the kernel that covers its shape.  Declarations and their reference counterparts are in
// include/cglm_attn.h.
#include <cmath>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"

using namespace cglm;

// the ctypes mirror of these structs (chatglm_cpp_b200/_lib.py) is checked against the same numbers
static_assert(sizeof(cglm_attn_desc) == 32, "cglm_attn_desc layout");
static_assert(sizeof(cglm_attn_seq) == 128 && offsetof(cglm_attn_seq, position_ids) == 72 &&
                  offsetof(cglm_attn_seq, partial) == 112,
              "cglm_attn_seq layout");

struct cglm_kv_arena {
    cglm_attn_desc desc;        // as the kernels see it: max_len is the PITCH of a cache row in tokens
    cglm_attn_desc user_desc;   // as the caller gave it: max_len is the capacity the calls are checked against
    int n_slots;
    int device;
    int n_sm;
    uint8_t *base;        // one allocation: K slabs, then V slabs; null when the caches are caller-owned (adopted)
    uint16_t *k_base;
    uint16_t *v_base;
    float2 *rope_tab;     // GLM rope modes at head_dim 128: (cos, sin) of ladder step i at position p, [max_len][32]
    int rope_tab_len;
    size_t k_slot_elems;  // G*M*D
    bool has_tmaps;
    CUtensorMap k_map, v_map;
    // pinned ring through which sequence descriptors travel to the device without a host sync
    SeqDev *ring;
    int ring_slots;
    int ring_cap;         // descriptors per slot
    int ring_next;
    cudaEvent_t *ring_events;
    // host-buffer calls: copies run on two streams of the arena's own so that they overlap the kernels of
    // neighbouring calls; the last kHostCalls calls are remembered to order the reuse of staging buffers
    static constexpr int kHostCalls = 8;
    struct HostCall {
        const void *dev_in;
        const void *dev_out;
        cudaEvent_t h2d, kernel, d2h;
        unsigned int seq;   // this call's number: what its two gate words hold once its copies have completed
        bool used;
    };
    // gate words of the host-buffer calls: device words [2 * record + {0: input staged, 1: output copied back}] and
    // the pinned host words they are copied from (the copy streams write them right behind the data)
    unsigned int *gate_dev;
    unsigned int *gate_host;
    unsigned int host_seq;
    cudaStream_t copy_in, copy_out;
    HostCall host_calls[kHostCalls];
    int host_next;
    bool host_ready;
    // calls served straight from mapped host memory (no staging): the last such call's kernel, for cglm_attn_host_drain
    std::mutex mu;
};

namespace {

thread_local char g_err[256] = "";

int fail_cuda(cudaError_t e, const char *what) {
    std::snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
    return CGLM_ERR_CUDA;
}
#define CGLM_CUDA(call)                                  \
    do {                                                 \
        cudaError_t e__ = (call);                        \
        if (e__ != cudaSuccess) return fail_cuda(e__, #call); \
    } while (0)

bool desc_ok(const cglm_attn_desc *d) {
    if (!d) return false;
    if (d->n_head <= 0 || d->n_kv_head <= 0 || d->n_head % d->n_kv_head) return false;
    if (d->head_dim <= 0 || d->head_dim % 2 || d->max_len <= 0 || d->n_virtual < 0 || d->n_virtual > d->max_len)
        return false;
    switch (d->rope_type) {
    case CGLM_ROPE_GPTJ: case CGLM_ROPE_NEOX: case CGLM_ROPE_DISABLED: break;
    case CGLM_ROPE_CHATGLM: case CGLM_ROPE_CHATGLM2:
        if (d->head_dim % 4) return false;
        break;
    default: return false;
    }
    return d->mask_type == CGLM_MASK_CAUSAL || d->mask_type == CGLM_MASK_CHATGLM;
}

AttnShape make_shape(const cglm_attn_desc &d) {
    AttnShape s;
    s.H = d.n_head; s.G = d.n_kv_head; s.D = d.head_dim; s.R = d.n_head / d.n_kv_head;
    s.M = d.max_len; s.V = d.n_virtual; s.rope_type = d.rope_type; s.mask_type = d.mask_type;
    // apply_rotary_emb_glm passes no base, i.e. ggml's default 10000 (chatglm.cpp:563-564)
    const float base = d.rope_type == CGLM_ROPE_CHATGLM ? 10000.f : d.rope_theta;
    s.theta_scale = powf(base, -2.0f / static_cast<float>(rope_n_dims(d.rope_type, d.head_dim)));
    s.scale = 1.f / std::sqrt(static_cast<float>(d.head_dim));
    return s;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Tiles per CTA that a settled decode launch pulls into L2 behind its shared-memory ring while the previous kernel
// drains.  CGLM_DECODE_L2_AHEAD overrides the default (tuning knob, read once).
int decode_l2_ahead() {
    static const int v = [] {
        const char *e = std::getenv("CGLM_DECODE_L2_AHEAD");
        const int x = e ? std::atoi(e) : 4;
        return x < 0 ? 0 : (x > 64 ? 64 : x);
    }();
    return v;
}
// Tiles by which a decode CTA's span is shortened for every item start inside it (see Geo in attn_decode.cu).
// CGLM_DECODE_CHARGE overrides the default (tuning knob, read once).
int decode_charge() {
    static const int v = [] {
        const char *e = std::getenv("CGLM_DECODE_CHARGE");
        const int x = e ? std::atoi(e) : 6;
        return x < 0 ? 0 : (x > 12 ? 12 : x);
    }();
    return v;
}
// When a decode CTA releases the next kernel of the stream (see DecodeTable::trigger): late (2) in general, because a
// kernel that is released early only sits on the SMs until its dependency wait returns; right after its own wait (0)
// when the launch runs on settled caches and is long (at least 8192 tiles over all kv heads), because the next launch
// of such a chain streams its cache tiles before its wait.  Measured per 40-layer step, settled caches, released early
// against late: 64 sequences x U[1024, 8191] 2.392 / 2.424 ms, 64 x 8191 3.758 / 3.834 ms; shorter launches lose
// (32 sequences 1.632 / 1.571 ms, 8 sequences 1.412 / 1.330 ms).  CGLM_DECODE_TRIGGER overrides (tuning knob, read once).
constexpr long long kEarlyReleaseMinTiles = 8192;
int decode_trigger(bool settled, long long total_tiles) {
    static const int forced = [] {
        const char *e = std::getenv("CGLM_DECODE_TRIGGER");
        const int x = e ? std::atoi(e) : -1;
        return x < 0 || x > 2 ? -1 : x;
    }();
    return forced >= 0 ? forced : (settled && total_tiles >= kEarlyReleaseMinTiles ? 0 : 2);
}

// ---- workspace layout (fixed regions first, so that self-resetting counters stay where they are) ------
struct WsLayout {
    size_t counters, gcounters, partials, gpartials, seqs, q_stage, total;
};
WsLayout ws_layout(const cglm_attn_desc &d, int n_sm, int n_seq, long long n_tokens, size_t prefill_bytes = 0) {
    WsLayout w;
    size_t off = sizeof(WsHeader);
    // scratch of the Linear kernels (partial sums of k-split tiles), at a fixed offset so that cglm_linear_forward finds
    // it in any workspace without knowing the attention configuration
    off = align_up(off + kLinearScratchBytes, 256);
    w.counters = off;
    off = align_up(off + sizeof(int) * kDecodeMaxSeqPerLaunch * static_cast<size_t>(d.n_kv_head), 256);
    const size_t n_groups = (decode_max_ctas(n_sm) + kDecodeMergeFan - 1) / kDecodeMergeFan;
    w.gcounters = off;
    off = align_up(off + sizeof(int) * 2 * n_groups, 256);
    w.partials = off;
    off = align_up(off + sizeof(float) * kDecodePartialFloats * 2 * static_cast<size_t>(decode_max_ctas(n_sm)), 256);
    w.gpartials = off;
    off = align_up(off + sizeof(float) * kDecodePartialFloats * 2 * n_groups, 256);
    w.seqs = off;
    off = align_up(off + sizeof(SeqDev) * static_cast<size_t>(n_seq), 256);
    off = align_up(off, 1024);
    w.q_stage = off;
    // roped, scaled q of the generic path (f32) or of one tcgen05 prefill (f16); used one launch at a time
    size_t stage = sizeof(float) * static_cast<size_t>(n_tokens) * d.n_head * d.head_dim;
    if (prefill_bytes > stage) stage = prefill_bytes;
    off = align_up(off + stage, 1024);
    w.total = off;
    return w;
}

int device_sm_count(int *n_sm, int *major) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        fail_cuda(e, "cudaGetDevice");
        return CGLM_ERR_NO_DEVICE;
    }
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) {
        fail_cuda(e, "cudaGetDeviceProperties");
        return CGLM_ERR_NO_DEVICE;
    }
    *n_sm = prop.multiProcessorCount;
    *major = prop.major;
    return CGLM_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    }
    return fn;
}

// K: f16 [n_slots*G][M][D=128] as a 3-D tensor, box 64 dims x 64 tokens; V^T: f16 [n_slots*G*D][M] as a
// 2-D tensor, box 64 tokens x 128 dims.  Both 128-byte swizzled; tokens past M read as zero.
bool build_tensor_maps(cglm_kv_arena *a) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    const cglm_attn_desc &d = a->desc;
    const cuuint64_t rows = static_cast<cuuint64_t>(a->n_slots) * d.n_kv_head;
    {
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(d.head_dim), static_cast<cuuint64_t>(d.max_len), rows};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(d.head_dim) * 2,
                                 static_cast<cuuint64_t>(d.head_dim) * 2 * d.max_len};
        cuuint32_t box[3] = {64, kDecodeTile, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        if (enc(&a->k_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, a->k_base, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    {
        cuuint64_t dims[2] = {static_cast<cuuint64_t>(d.max_len), rows * d.head_dim};
        cuuint64_t strides[1] = {static_cast<cuuint64_t>(d.max_len) * 2};
        cuuint32_t box[2] = {kDecodeTile, 128};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&a->v_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a->v_base, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    return true;
}

// Per-call maps of the tcgen05 prefill: q staging f16 [H][s_pad][128]; the slot's K rows and V^T rows cut at the
// attended length L, so that tokens past it read as zero whatever the cache holds there.
bool build_prefill_maps(const cglm_kv_arena *a, void *q_half, int s_pad, int L, CUtensorMap *q_map, CUtensorMap *k_map,
                        CUtensorMap *v_map) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    const cglm_attn_desc &d = a->desc;
    const cuuint64_t rows = static_cast<cuuint64_t>(a->n_slots) * d.n_kv_head;
    const cuuint32_t estr3[3] = {1, 1, 1}, estr2[2] = {1, 1};
    {
        cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(s_pad), static_cast<cuuint64_t>(d.n_head)};
        cuuint64_t strides[2] = {256, static_cast<cuuint64_t>(s_pad) * 256};
        cuuint32_t box[3] = {64, 128, 1};
        if (enc(q_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, q_half, dims, strides, box, estr3, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    {
        cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(L), rows};
        cuuint64_t strides[2] = {256, static_cast<cuuint64_t>(d.max_len) * 256};
        cuuint32_t box[3] = {64, 128, 1};
        if (enc(k_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, a->k_base, dims, strides, box, estr3, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    {
        cuuint64_t dims[2] = {static_cast<cuuint64_t>(L), rows * 128};
        cuuint64_t strides[1] = {static_cast<cuuint64_t>(d.max_len) * 2};
        cuuint32_t box[2] = {64, 128};
        if (enc(v_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a->v_base, dims, strides, box, estr2, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    return true;
}

bool fast_decode_shape(const cglm_kv_arena *a) {
    const cglm_attn_desc &d = a->desc;
    return a->has_tmaps && d.head_dim == 128 && d.n_head / d.n_kv_head <= 16 && d.max_len % 8 == 0 &&
           (d.rope_type == CGLM_ROPE_CHATGLM2 || d.rope_type == CGLM_ROPE_CHATGLM || d.rope_type == CGLM_ROPE_DISABLED);
}

// Angle table of an arena: entry [p][i] = (cos, sin) of ladder step i at position p, the same values the kernels
// would compute on the fly (rope_cos_sin).  The decode kernel reads 256 bytes of it per segment instead of
// evaluating a double-precision sincos between its start and its first tile.
__global__ void rope_arena_table_kernel(float theta_scale, int n_pos, float2 *__restrict__ table) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= static_cast<long long>(n_pos) * 32) return;
    float c, s;
    rope_cos_sin(static_cast<int>(i >> 5), static_cast<int>(i & 31), theta_scale, c, s);
    table[i] = make_float2(c, s);
}

__global__ void combine_kernel(const float *__restrict__ partials, int n_part, int H, int D, float *__restrict__ out) {
    const int h = blockIdx.x;
    float m_star = -INFINITY;
    for (int p = 0; p < n_part; ++p) {
        m_star = fmaxf(m_star, partials[(static_cast<long long>(p) * H + h) * (D + 2) + D]);
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f, den = 0.f;
        for (int p = 0; p < n_part; ++p) {
            const float *pp = partials + (static_cast<long long>(p) * H + h) * (D + 2);
            const float m = pp[D];
            const float w = m == -INFINITY ? 0.f : __expf(m - m_star);
            acc += w * pp[d];
            den += w * pp[D + 1];
        }
        out[static_cast<long long>(h) * D + d] = acc / den;
    }
}

// activation cast in front of an f16 Linear (ggml converts the f32 activation row the same way before it multiplies by
// an f16 matrix): round to nearest even, grid-stride over groups of 4
__global__ void f32_to_f16_kernel(const float *__restrict__ src, __half *__restrict__ dst, size_t n) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x * 4;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) & 15) | (reinterpret_cast<uintptr_t>(dst) & 7)) == 0;
    for (size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
        if (vec && i + 4 <= n) {
            const float4 v = *reinterpret_cast<const float4 *>(src + i);
            *reinterpret_cast<uint2 *>(dst + i) = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
        } else {
            for (size_t j = i; j < n && j < i + 4; ++j) dst[j] = __float2half_rn(src[j]);
        }
    }
}

__global__ void seq_advance_kernel(int *__restrict__ n_past, int n, int delta) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) n_past[i] += delta;
}

__global__ void load_prefix_kernel(const uint16_t *__restrict__ past_kv, uint16_t *__restrict__ k_slot,
                                   uint16_t *__restrict__ v_slot, int G, int V, int D, int M) {
    const long long n = static_cast<long long>(G) * V * D;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int d = static_cast<int>(i % D);
        const int t = static_cast<int>((i / D) % V);
        const int g = static_cast<int>(i / (static_cast<long long>(D) * V));
        k_slot[(static_cast<long long>(g) * M + t) * D + d] = past_kv[i];
        v_slot[(static_cast<long long>(g) * D + d) * M + t] = past_kv[n + i];
    }
}

LaunchCtx make_launch_ctx(const cglm_kv_arena *a, uint8_t *ws, const WsLayout &lay, cudaStream_t st) {
    LaunchCtx cx;
    cx.shape = make_shape(a->desc);
    cx.k_base = a->k_base;
    cx.v_base = a->v_base;
    cx.hdr = reinterpret_cast<WsHeader *>(ws);
    cx.counters = reinterpret_cast<int *>(ws + lay.counters);
    cx.gcounters = reinterpret_cast<int *>(ws + lay.gcounters);
    cx.partials = reinterpret_cast<float *>(ws + lay.partials);
    cx.gpartials = reinterpret_cast<float *>(ws + lay.gpartials);
    cx.q_stage = reinterpret_cast<float *>(ws + lay.q_stage);
    cx.k_map = &a->k_map;
    cx.v_map = &a->v_map;
    cx.rope_tab = a->rope_tab;
    cx.rope_tab_len = a->rope_tab_len;
    cx.stream = st;
    cx.n_sm = a->n_sm;
    cx.device = a->device;
    return cx;
}

int ring_reserve(cglm_kv_arena *a, int n_seq, SeqDev **slot, cudaEvent_t *ev) {
    if (n_seq > a->ring_cap) {
        // grow: wait for every copy in flight, then reallocate
        for (int i = 0; i < a->ring_slots; ++i) {
            CGLM_CUDA(cudaEventSynchronize(a->ring_events[i]));
        }
        if (a->ring) CGLM_CUDA(cudaFreeHost(a->ring));
        a->ring = nullptr;
        int cap = a->ring_cap ? a->ring_cap : 64;
        while (cap < n_seq) cap *= 2;
        CGLM_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&a->ring), sizeof(SeqDev) * cap * a->ring_slots,
                                cudaHostAllocDefault));
        a->ring_cap = cap;
    }
    const int i = a->ring_next;
    a->ring_next = (i + 1) % a->ring_slots;
    CGLM_CUDA(cudaEventSynchronize(a->ring_events[i]));   // the copy that last used this slot has run
    *slot = a->ring + static_cast<size_t>(i) * a->ring_cap;
    *ev = a->ring_events[i];
    return CGLM_OK;
}

}  // namespace

// read-only views of an arena for the other translation units of the library
namespace cglm {
const CUtensorMap *arena_k_map(const cglm_kv_arena *a) { return &a->k_map; }
const CUtensorMap *arena_v_map(const cglm_kv_arena *a) { return &a->v_map; }
bool arena_fast_decode(const cglm_kv_arena *a) { return fast_decode_shape(a); }
int arena_device(const cglm_kv_arena *a) { return a->device; }
int arena_sm_count(const cglm_kv_arena *a) { return a->n_sm; }
AttnShape arena_shape(const cglm_kv_arena *a) { return make_shape(a->desc); }
const float2 *arena_rope_tab(const cglm_kv_arena *a, int *len) { *len = a->rope_tab_len; return a->rope_tab; }
void set_last_error(const char *text) { std::snprintf(g_err, sizeof(g_err), "%s", text); }
}  // namespace cglm

extern "C" {

size_t cglm_kv_slot_bytes(const cglm_attn_desc *desc) {
    if (!desc_ok(desc)) return 0;
    return static_cast<size_t>(4) * desc->n_kv_head * desc->max_len * desc->head_dim;
}

int cglm_kv_arena_create(const cglm_attn_desc *desc, int n_slots, cglm_kv_arena **out) {
    if (!desc_ok(desc) || n_slots <= 0 || !out) return CGLM_ERR_INVALID_ARG;
    if (desc->head_dim > 256) return CGLM_ERR_UNSUPPORTED;
    int n_sm = 0, major = 0;
    int rc = device_sm_count(&n_sm, &major);
    if (rc != CGLM_OK) return rc;
    if (major < 10) {
        std::snprintf(g_err, sizeof(g_err), "compute capability %d.x device: this library carries sm_100a code only", major);
        return CGLM_ERR_NO_DEVICE;
    }
    cglm_kv_arena *a = new (std::nothrow) cglm_kv_arena();
    if (!a) return CGLM_ERR_INVALID_ARG;
    a->desc = *desc;
    a->user_desc = *desc;
    // A row of V^T is `pitch` tokens long and TMA wants row pitches in multiples of 16 bytes: caches of the library's
    // own are laid out with the capacity rounded up to a multiple of 8 tokens (a P-Tuning prefix makes max_length +
    // num_virtual_tokens odd-sized), so such models keep the fused kernels.  Calls are still checked against max_len.
    if (desc->head_dim == 128) a->desc.max_len = (desc->max_len + 7) / 8 * 8;
    desc = &a->desc;
    a->n_slots = n_slots;
    a->n_sm = n_sm;
    cudaGetDevice(&a->device);
    a->k_slot_elems = static_cast<size_t>(desc->n_kv_head) * desc->max_len * desc->head_dim;
    const size_t k_bytes = align_up(a->k_slot_elems * 2 * n_slots, 1024);
    const size_t v_bytes = align_up(a->k_slot_elems * 2 * n_slots, 1024);
    const bool glm_rope = desc->rope_type == CGLM_ROPE_CHATGLM2 || desc->rope_type == CGLM_ROPE_CHATGLM;
    a->rope_tab_len = desc->head_dim == 128 && glm_rope ? desc->max_len : 0;
    const size_t tab_bytes = static_cast<size_t>(a->rope_tab_len) * 32 * sizeof(float2);
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&a->base), k_bytes + v_bytes + tab_bytes);
    if (e != cudaSuccess) {
        delete a;
        return fail_cuda(e, "cudaMalloc(kv arena)");
    }
    a->k_base = reinterpret_cast<uint16_t *>(a->base);
    a->v_base = reinterpret_cast<uint16_t *>(a->base + k_bytes);
    e = cudaMemset(a->base, 0, k_bytes + v_bytes);
    if (e != cudaSuccess) {
        cudaFree(a->base);
        delete a;
        return fail_cuda(e, "cudaMemset(kv arena)");
    }
    a->rope_tab = nullptr;
    if (a->rope_tab_len > 0) {
        a->rope_tab = reinterpret_cast<float2 *>(a->base + k_bytes + v_bytes);
        const long long n = static_cast<long long>(a->rope_tab_len) * 32;
        rope_arena_table_kernel<<<static_cast<unsigned>((n + 255) / 256), 256>>>(make_shape(*desc).theta_scale, a->rope_tab_len,
                                                                               a->rope_tab);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        if (e != cudaSuccess) {
            cudaFree(a->base);
            delete a;
            return fail_cuda(e, "rope table");
        }
    }
    a->has_tmaps = desc->head_dim == 128 && desc->max_len % 8 == 0 && build_tensor_maps(a);
    a->ring = nullptr;
    a->ring_slots = 64;
    a->ring_cap = 0;
    a->ring_next = 0;
    a->ring_events = new cudaEvent_t[a->ring_slots];
    for (int i = 0; i < a->ring_slots; ++i) {
        cudaEventCreateWithFlags(&a->ring_events[i], cudaEventDisableTiming);
    }
    a->host_ready = false;
    a->host_next = 0;
    *out = a;
    return CGLM_OK;
}

size_t cglm_kv_angle_table_bytes(const cglm_attn_desc *desc) {
    if (!desc_ok(desc)) return 0;
    const bool glm_rope = desc->rope_type == CGLM_ROPE_CHATGLM2 || desc->rope_type == CGLM_ROPE_CHATGLM;
    return desc->head_dim == 128 && glm_rope ? static_cast<size_t>(desc->max_len) * 32 * sizeof(float2) : 0;
}

int cglm_kv_arena_adopt(const cglm_attn_desc *desc, int n_slots, void *k_base, void *v_base, void *angle_table,
                        cglm_kv_arena **out) {
    if (!desc_ok(desc) || n_slots <= 0 || !out || !k_base || !v_base) return CGLM_ERR_INVALID_ARG;
    if (desc->head_dim > 256) return CGLM_ERR_UNSUPPORTED;
    // TMA wants 16-byte aligned bases; ask for the 128 bytes a swizzled row spans
    if ((reinterpret_cast<uintptr_t>(k_base) | reinterpret_cast<uintptr_t>(v_base) | reinterpret_cast<uintptr_t>(angle_table)) & 127)
        return CGLM_ERR_INVALID_ARG;
    int n_sm = 0, major = 0;
    int rc = device_sm_count(&n_sm, &major);
    if (rc != CGLM_OK) return rc;
    if (major < 10) {
        std::snprintf(g_err, sizeof(g_err), "compute capability %d.x device: this library carries sm_100a code only", major);
        return CGLM_ERR_NO_DEVICE;
    }
    cudaPointerAttributes at;
    for (void *p : {k_base, v_base}) {   // device memory of the current device, not a host pointer
        int dev = -1;
        cudaGetDevice(&dev);
        if (cudaPointerGetAttributes(&at, p) != cudaSuccess || at.type != cudaMemoryTypeDevice || at.device != dev) {
            cudaGetLastError();
            std::snprintf(g_err, sizeof(g_err), "adopted caches must be device memory of the current device");
            return CGLM_ERR_INVALID_ARG;
        }
    }
    cglm_kv_arena *a = new (std::nothrow) cglm_kv_arena();
    if (!a) return CGLM_ERR_INVALID_ARG;
    a->desc = *desc;
    a->user_desc = *desc;   // caller-owned caches keep the caller's pitch
    a->n_slots = n_slots;
    a->n_sm = n_sm;
    cudaGetDevice(&a->device);
    a->k_slot_elems = static_cast<size_t>(desc->n_kv_head) * desc->max_len * desc->head_dim;
    a->base = nullptr;
    a->k_base = static_cast<uint16_t *>(k_base);
    a->v_base = static_cast<uint16_t *>(v_base);
    a->rope_tab = nullptr;
    a->rope_tab_len = 0;
    if (angle_table && cglm_kv_angle_table_bytes(desc) > 0) {
        a->rope_tab = static_cast<float2 *>(angle_table);
        a->rope_tab_len = desc->max_len;
        const long long n = static_cast<long long>(a->rope_tab_len) * 32;
        rope_arena_table_kernel<<<static_cast<unsigned>((n + 255) / 256), 256>>>(make_shape(*desc).theta_scale, a->rope_tab_len,
                                                                               a->rope_tab);
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        if (e != cudaSuccess) {
            delete a;
            return fail_cuda(e, "rope table");
        }
    }
    a->has_tmaps = desc->head_dim == 128 && desc->max_len % 8 == 0 && build_tensor_maps(a);
    a->ring = nullptr;
    a->ring_slots = 64;
    a->ring_cap = 0;
    a->ring_next = 0;
    a->ring_events = new cudaEvent_t[a->ring_slots];
    for (int i = 0; i < a->ring_slots; ++i) {
        cudaEventCreateWithFlags(&a->ring_events[i], cudaEventDisableTiming);
    }
    a->host_ready = false;
    a->host_next = 0;
    *out = a;
    return CGLM_OK;
}

int cglm_kv_arena_destroy(cglm_kv_arena *a) {
    if (!a) return CGLM_ERR_INVALID_ARG;
    cudaDeviceSynchronize();
    if (a->host_ready) {
        for (auto &c : a->host_calls) {
            cudaEventDestroy(c.h2d); cudaEventDestroy(c.kernel); cudaEventDestroy(c.d2h);
        }
        cudaStreamDestroy(a->copy_in);
        cudaStreamDestroy(a->copy_out);
        cudaFree(a->gate_dev);
        cudaFreeHost(a->gate_host);
    }
    for (int i = 0; i < a->ring_slots; ++i) cudaEventDestroy(a->ring_events[i]);
    delete[] a->ring_events;
    if (a->ring) cudaFreeHost(a->ring);
    if (a->base) cudaFree(a->base);   // adopted caches stay with their owner
    delete a;
    return CGLM_OK;
}

void *cglm_kv_arena_k_cache(const cglm_kv_arena *a, int slot) {
    if (!a || slot < 0 || slot >= a->n_slots) return nullptr;
    return a->k_base + a->k_slot_elems * slot;
}
void *cglm_kv_arena_v_cache(const cglm_kv_arena *a, int slot) {
    if (!a || slot < 0 || slot >= a->n_slots) return nullptr;
    return a->v_base + a->k_slot_elems * slot;
}
int cglm_kv_arena_n_slots(const cglm_kv_arena *a) { return a ? a->n_slots : 0; }
const cglm_attn_desc *cglm_kv_arena_desc(const cglm_kv_arena *a) { return a ? &a->user_desc : nullptr; }
int cglm_kv_arena_pitch(const cglm_kv_arena *a) { return a ? a->desc.max_len : 0; }

int cglm_kv_slot_copy(cglm_kv_arena *a, int slot, void *k_host, void *v_host, int to_device, void *cuda_stream) {
    if (!a || slot < 0 || slot >= a->n_slots) return CGLM_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const size_t bytes = a->k_slot_elems * 2;
    void *kd = cglm_kv_arena_k_cache(a, slot), *vd = cglm_kv_arena_v_cache(a, slot);
    if (k_host) {
        CGLM_CUDA(to_device ? cudaMemcpyAsync(kd, k_host, bytes, cudaMemcpyHostToDevice, st)
                            : cudaMemcpyAsync(k_host, kd, bytes, cudaMemcpyDeviceToHost, st));
    }
    if (v_host) {
        CGLM_CUDA(to_device ? cudaMemcpyAsync(vd, v_host, bytes, cudaMemcpyHostToDevice, st)
                            : cudaMemcpyAsync(v_host, vd, bytes, cudaMemcpyDeviceToHost, st));
    }
    return CGLM_OK;
}

size_t cglm_attn_workspace_bytes(const cglm_attn_desc *desc, int n_seq, int max_qlen) {
    if (!desc_ok(desc) || n_seq <= 0 || max_qlen <= 0) return 0;
    int n_sm = 148, major = 0;
    device_sm_count(&n_sm, &major);   // falls back to a B200's SM count when no device is visible
    // a prompt of >= 128 tokens at head_dim 128 may take the tensor-core prefill, whose staging is sized differently
    const size_t prefill = desc->head_dim == 128 && max_qlen >= kPrefillMinTokens ? prefill_q_half_bytes(desc->n_head, max_qlen) : 0;
    return ws_layout(*desc, n_sm, n_seq, static_cast<long long>(n_seq) * max_qlen, prefill).total;
}

int cglm_attn_workspace_init(void *workspace, size_t workspace_bytes, void *cuda_stream) {
    if (!workspace || workspace_bytes < sizeof(WsHeader)) return CGLM_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    CGLM_CUDA(cudaMemsetAsync(workspace, 0, workspace_bytes, st));
    CGLM_CUDA(cudaMemsetAsync(workspace, static_cast<int>(kWsMagic & 0xffu), sizeof(unsigned int), st));   // the magic is one byte, four times
    return CGLM_OK;
}

int cglm_attn_workspace_status(void *workspace, void *cuda_stream) {
    if (!workspace) return CGLM_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    WsHeader h;
    CGLM_CUDA(cudaMemcpyAsync(&h, workspace, sizeof(int) * 2, cudaMemcpyDeviceToHost, st));
    CGLM_CUDA(cudaStreamSynchronize(st));
    if (h.magic != kWsMagic) return CGLM_ERR_WORKSPACE;
    if (h.status != 0) {
        const int zero = 0;
        CGLM_CUDA(cudaMemcpyAsync(&static_cast<WsHeader *>(workspace)->status, &zero, sizeof(int),
                                  cudaMemcpyHostToDevice, st));
        CGLM_CUDA(cudaStreamSynchronize(st));
    }
    return h.status;
}

namespace {
// What a host-buffer call waits for before its kernels may read the staged activations / write the staged outputs:
// device words written by the copy streams for the fused decode kernel (polled inside the kernel, see
// DecodeTable::gate), and the matching events for every other kernel (waited for on the stream).
struct HostGates {
    const unsigned int *word[2];
    unsigned int value[2];
    cudaEvent_t event[2];   // null: nothing to wait for
};
int forward_impl(cglm_kv_arena *a, const cglm_attn_seq *seqs, int n_seq, void *workspace, size_t workspace_bytes,
                 void *cuda_stream, const HostGates *gates);
}  // namespace

int cglm_attn_forward(cglm_kv_arena *a, const cglm_attn_seq *seqs, int n_seq, void *workspace,
                      size_t workspace_bytes, void *cuda_stream) {
    return forward_impl(a, seqs, n_seq, workspace, workspace_bytes, cuda_stream, nullptr);
}

namespace {
int forward_impl(cglm_kv_arena *a, const cglm_attn_seq *seqs, int n_seq, void *workspace, size_t workspace_bytes,
                 void *cuda_stream, const HostGates *gates) {
    if (!a || !seqs || n_seq <= 0) return CGLM_ERR_INVALID_ARG;
    if (!workspace) return CGLM_ERR_WORKSPACE;
    const cglm_attn_desc &d = a->desc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const bool fast_ok = fast_decode_shape(a);

    // ---- validate and classify ---------------------------------------------------------------------------
    long long gen_tokens = 0, decode_tiles = 0;
    int n_fast = 0, n_prefill = 0;
    size_t prefill_bytes = 0;
    // 0: generic path, 1: fused decode, 2: tcgen05 prefill (per thread and reused: no allocation per call once it has grown)
    static thread_local std::vector<unsigned char> is_fast;
    is_fast.assign(static_cast<size_t>(n_seq), 0);
    const bool prefill_ok = a->has_tmaps && d.head_dim == 128 && d.max_len % 8 == 0 &&
                            (d.rope_type == CGLM_ROPE_CHATGLM2 || d.rope_type == CGLM_ROPE_CHATGLM ||
                             d.rope_type == CGLM_ROPE_DISABLED);
    for (int i = 0; i < n_seq; ++i) {
        const cglm_attn_seq &s = seqs[i];
        if (!s.q || !s.k || !s.v || s.qlen <= 0 || s.n_past < 0 || s.slot < 0 || s.slot >= a->n_slots)
            return CGLM_ERR_INVALID_ARG;
        // qlen > 1 with n_past != 0 (a prompt fed in chunks) is served like the reference serves it: no mask at all
        // (chatglm.cpp:689 masks only at n_past == 0), on the generic path
        const bool partial = (s.flags & CGLM_SEQ_PARTIAL) != 0;
        if (partial ? !s.partial : !s.out) return CGLM_ERR_INVALID_ARG;
        // vector stores: out rows are written four elements at a time (16 bytes of f32, 8 of f16), partial rows 8 bytes
        // at a time; activations are at least element-aligned
        const bool qkv_f16 = (s.flags & CGLM_SEQ_QKV_F16) != 0, out_f16 = (s.flags & CGLM_SEQ_OUT_F16) != 0;
        const uintptr_t in_mask = qkv_f16 ? 1 : 3;
        if ((reinterpret_cast<uintptr_t>(s.out) & (out_f16 ? 7 : 15)) || (reinterpret_cast<uintptr_t>(s.partial) & 7) ||
            (reinterpret_cast<uintptr_t>(s.q) & in_mask) || (reinterpret_cast<uintptr_t>(s.k) & in_mask) ||
            (reinterpret_cast<uintptr_t>(s.v) & in_mask))
            return CGLM_ERR_INVALID_ARG;
        if ((s.flags & CGLM_SEQ_NO_APPEND) && ((!partial && !(s.flags & CGLM_SEQ_Q_ROPED)) || s.qlen != 1)) return CGLM_ERR_INVALID_ARG;
        if ((s.flags & CGLM_SEQ_Q_ROPED) && s.qlen != 1) return CGLM_ERR_INVALID_ARG;
        if ((s.flags & CGLM_SEQ_USE_KV_LOCAL) && (s.kv_local < 0 || s.qlen != 1)) return CGLM_ERR_INVALID_ARG;
        const bool dyn_past = (s.flags & CGLM_SEQ_N_PAST_DEVICE) != 0;
        if (dyn_past && (!s.n_past_dev || (reinterpret_cast<uintptr_t>(s.n_past_dev) & 3) || s.qlen != 1 ||
                         (s.flags & CGLM_SEQ_USE_KV_LOCAL)))
            return CGLM_ERR_INVALID_ARG;
        const int kv_before = (s.flags & CGLM_SEQ_USE_KV_LOCAL) ? s.kv_local : d.n_virtual + s.n_past;
        const int appended = (s.flags & CGLM_SEQ_NO_APPEND) ? 0 : s.qlen;
        if (static_cast<long long>(kv_before) + appended > a->user_desc.max_len) return CGLM_ERR_INVALID_ARG;
        if (d.rope_type == CGLM_ROPE_CHATGLM && !s.position_ids && s.n_ctx < 2) return CGLM_ERR_INVALID_ARG;
        const int L = kv_before + appended;
        is_fast[i] = fast_ok && s.qlen == 1 && L >= 1 &&
                     decode_rows_aligned(s.q, s.k, s.v, s.q_head_stride, s.kv_head_stride, s.q_roped, s.k_roped, qkv_f16);
        if (dyn_past && !is_fast[i]) {
            std::snprintf(g_err, sizeof(g_err), "CGLM_SEQ_N_PAST_DEVICE needs a shape and alignment the fused decode kernel takes");
            return CGLM_ERR_UNSUPPORTED;
        }
        if (is_fast[i]) {
            ++n_fast;
            decode_tiles += static_cast<long long>((L + kDecodeTile - 1) / kDecodeTile) * d.n_kv_head;
        } else if (prefill_ok && s.qlen >= kPrefillMinTokens && s.n_past == 0 && (s.flags & ~(CGLM_SEQ_CACHE_SETTLED | CGLM_SEQ_QKV_F16 | CGLM_SEQ_OUT_F16)) == 0) {
            is_fast[i] = 2;
            ++n_prefill;
            const size_t need = prefill_q_half_bytes(d.n_head, s.qlen);
            if (need > prefill_bytes) prefill_bytes = need;
        } else {
            gen_tokens += s.qlen;
        }
    }
    const WsLayout lay = ws_layout(d, a->n_sm, n_seq, gen_tokens, prefill_bytes);
    if (workspace_bytes < lay.total) return CGLM_ERR_WORKSPACE;

    // ---- descriptors ---------------------------------------------------------------------------------------
    auto to_dev = [&](const cglm_attn_seq &s, SeqDev &o) {
        o.q = s.q; o.k = s.k; o.v = s.v;
        o.q_tok_stride = s.q_tok_stride; o.q_head_stride = s.q_head_stride;
        o.kv_tok_stride = s.kv_tok_stride; o.kv_head_stride = s.kv_head_stride;
        o.position_ids = s.position_ids;
        o.out = s.out; o.q_roped = s.q_roped; o.k_roped = s.k_roped; o.partial = s.partial;
        o.slot = s.slot; o.qlen = s.qlen; o.n_past = s.n_past; o.n_ctx = s.n_ctx;
        o.kv_before = (s.flags & CGLM_SEQ_USE_KV_LOCAL) ? s.kv_local : d.n_virtual + s.n_past;
        o.flags = s.flags;
        o.tok_begin = 0;
        o.pad = 0;
        if (s.flags & CGLM_SEQ_N_PAST_DEVICE) o.n_past_dev = s.n_past_dev;   // shares the words of tok_begin / pad
    };
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    LaunchCtx cx = make_launch_ctx(a, ws, lay, st);
    // a host-buffer call served by anything but fused decode launches alone waits on the stream
    const bool gate_in_kernel = gates && n_fast == n_seq;
    if (gates && !gate_in_kernel) {
        for (int gi = 0; gi < 2; ++gi) {
            if (gates->event[gi]) CGLM_CUDA(cudaStreamWaitEvent(st, gates->event[gi], 0));
        }
    }

    // fused decode: descriptors and tile prefix travel as kernel parameters, kDecodeMaxSeqPerLaunch per launch
    if (n_fast > 0) {
        static thread_local DecodeTableDyn tab;
        int filled = 0;
        bool dyn = false, settled = true;
        tab.prefix[0] = 0;
        for (int i = 0; i <= n_seq; ++i) {
            if (i < n_seq && is_fast[i] == 1) {
                SeqDev &o = tab.seqs[filled];
                to_dev(seqs[i], o);
                dyn = dyn || (o.flags & CGLM_SEQ_N_PAST_DEVICE);
                settled = settled && (o.flags & CGLM_SEQ_CACHE_SETTLED);
                const int L = o.kv_before + ((o.flags & CGLM_SEQ_NO_APPEND) ? 0 : 1);
                tab.prefix[filled + 1] = tab.prefix[filled] + (L + kDecodeTile - 1) / kDecodeTile;
                ++filled;
            }
            if (filled == kDecodeMaxSeqPerLaunch || (i == n_seq && filled > 0)) {
                tab.n_seq = filled;
                tab.settled = settled && !dyn ? 1 + decode_l2_ahead() : 0;
                tab.trigger = decode_trigger(tab.settled != 0, static_cast<long long>(tab.prefix[filled]) * d.n_kv_head);
                tab.charge = decode_charge();
                for (int gi = 0; gi < 2; ++gi) {
                    tab.gate[gi] = gate_in_kernel && gates->event[gi] ? gates->word[gi] : nullptr;
                    tab.gate_value[gi] = gate_in_kernel ? gates->value[gi] : 0;
                }
                if (dyn) decode_table_finish(tab);
                CGLM_CUDA(launch_decode(cx, tab, dyn));
                filled = 0;
                dyn = false;
                settled = true;
            }
        }
    }
    // generic path: descriptors are uploaded through the pinned ring
    // tcgen05 prefill: one pair of launches per prompt, tensor maps encoded for this call
    for (int i = 0; i < n_seq && n_prefill > 0; ++i) {
        if (is_fast[i] != 2) continue;
        SeqDev sq;
        to_dev(seqs[i], sq);
        const int s_pad = (sq.qlen + 127) / 128 * 128;
        CUtensorMap q_map, k_map, v_map;
        __half *q_half = reinterpret_cast<__half *>(ws + lay.q_stage);
        if (!build_prefill_maps(a, q_half, s_pad, d.n_virtual + sq.qlen, &q_map, &k_map, &v_map)) {
            std::snprintf(g_err, sizeof(g_err), "cuTensorMapEncodeTiled failed for a prefill call");
            return CGLM_ERR_CUDA;
        }
        CGLM_CUDA(launch_prefill(cx, sq, q_map, k_map, v_map, q_half));
    }
    const int n_gen = n_seq - n_fast - n_prefill;
    if (n_gen > 0) {
        std::lock_guard<std::mutex> lock(a->mu);
        SeqDev *host = nullptr;
        cudaEvent_t ev;
        int rc = ring_reserve(a, n_gen, &host, &ev);
        if (rc != CGLM_OK) return rc;
        int gi = 0, tok = 0;
        for (int i = 0; i < n_seq; ++i) {
            if (is_fast[i]) continue;   // fused decode and tcgen05 prefill sequences were launched above
            SeqDev &o = host[gi++];
            to_dev(seqs[i], o);
            o.tok_begin = tok;
            tok += seqs[i].qlen;
        }
        SeqDev *seqs_dev = reinterpret_cast<SeqDev *>(ws + lay.seqs);
        CGLM_CUDA(cudaMemcpyAsync(seqs_dev, host, sizeof(SeqDev) * n_gen, cudaMemcpyHostToDevice, st));
        CGLM_CUDA(cudaEventRecord(ev, st));
        CGLM_CUDA(launch_generic(cx, seqs_dev, n_gen, static_cast<int>(gen_tokens)));
    }
    (void)decode_tiles;
    return CGLM_OK;
}
}  // namespace

int cglm_attn_forward_host(cglm_kv_arena *a, const cglm_attn_seq *seqs, int n_seq, int layout,
                           const void *qkv_host, void *out_host, void *dev_qkv, void *dev_out, void *workspace,
                           size_t workspace_bytes, void *cuda_stream) {
    if (!a || !seqs || n_seq <= 0 || !qkv_host || !out_host || !dev_qkv || !dev_out) return CGLM_ERR_INVALID_ARG;
    if (layout & ~(CGLM_HOST_INTERLEAVED_QKV | CGLM_HOST_F16)) return CGLM_ERR_INVALID_ARG;
    const cglm_attn_desc &d = a->desc;
    const bool interleaved_qkv = (layout & CGLM_HOST_INTERLEAVED_QKV) != 0, act_f16 = (layout & CGLM_HOST_F16) != 0;
    const size_t esz = act_f16 ? 2 : 4;
    if (interleaved_qkv && d.n_head != d.n_kv_head) return CGLM_ERR_INVALID_ARG;   // chatglm.cpp:637
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const long long H = d.n_head, G = d.n_kv_head, D = d.head_dim;
    const long long row = (H + 2 * G) * D, orow = H * D;
    for (int i = 0; i < n_seq; ++i) {
        if (seqs[i].qlen <= 0) return CGLM_ERR_INVALID_ARG;
    }
    long long n_tok = 0;
    static thread_local std::vector<cglm_attn_seq> dev_seqs;   // reused: no allocation per call once it has grown
    dev_seqs.assign(seqs, seqs + n_seq);
    // descriptors over a packed [tokens][row] activation at in_base and a packed [tokens][orow] output at out_base
    auto point_at = [&](const void *in_base, void *out_base) {
        n_tok = 0;
        for (int i = 0; i < n_seq; ++i) {
            cglm_attn_seq &s = dev_seqs[i];
            const char *base = static_cast<const char *>(in_base) + n_tok * row * esz;
            auto at = [&](long long elems) { return reinterpret_cast<const float *>(base + elems * esz); };
            s.q = at(0);
            if (interleaved_qkv) {   // chatglm.cpp:638-644
                s.k = at(D); s.v = at(2 * D);
                s.q_head_stride = s.kv_head_stride = 3 * D;
            } else {                 // chatglm.cpp:646-652
                s.k = at(H * D); s.v = at((H + G) * D);
                s.q_head_stride = s.kv_head_stride = D;
            }
            s.q_tok_stride = s.kv_tok_stride = row;
            s.out = reinterpret_cast<float *>(static_cast<char *>(out_base) + n_tok * orow * esz);
            s.position_ids = nullptr; s.q_roped = nullptr; s.k_roped = nullptr; s.partial = nullptr;
            s.n_past_dev = nullptr;
            s.flags = (seqs[i].flags & CGLM_SEQ_CACHE_SETTLED) | (act_f16 ? (CGLM_SEQ_QKV_F16 | CGLM_SEQ_OUT_F16) : 0);
            s.kv_local = 0;
            n_tok += seqs[i].qlen;
        }
    };
    // Pinned host buffers are not read by the kernels directly, although the device could map them: with the copies
    // gated by device words (below) the staged pipeline is faster at every size.  Measured per decode step through
    // host buffers: one sequence, 28 calls, 0.99 ms staged against 1.11 ms direct; 8 sequences of 9 KiB, 40 calls,
    // 1.45 against 3.45 ms (every thread block that holds a part of a sequence repeats the small reads across the bus).
    point_at(dev_qkv, dev_out);
    // ---- pipeline: H2D on copy_in, kernel on the caller's stream, D2H on copy_out ---------------------------------
    std::unique_lock<std::mutex> lock(a->mu);
    if (!a->host_ready) {
        CGLM_CUDA(cudaStreamCreateWithFlags(&a->copy_in, cudaStreamNonBlocking));
        CGLM_CUDA(cudaStreamCreateWithFlags(&a->copy_out, cudaStreamNonBlocking));
        for (auto &c : a->host_calls) {
            CGLM_CUDA(cudaEventCreateWithFlags(&c.h2d, cudaEventDisableTiming));
            CGLM_CUDA(cudaEventCreateWithFlags(&c.kernel, cudaEventDisableTiming));
            CGLM_CUDA(cudaEventCreateWithFlags(&c.d2h, cudaEventDisableTiming));
            c.used = false;
            c.dev_in = c.dev_out = nullptr;
        }
        CGLM_CUDA(cudaMalloc(reinterpret_cast<void **>(&a->gate_dev), 2 * cglm_kv_arena::kHostCalls * sizeof(unsigned int)));
        CGLM_CUDA(cudaMemset(a->gate_dev, 0, 2 * cglm_kv_arena::kHostCalls * sizeof(unsigned int)));
        CGLM_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&a->gate_host), 2 * cglm_kv_arena::kHostCalls * sizeof(unsigned int),
                                cudaHostAllocDefault));
        CGLM_CUDA(cudaDeviceSynchronize());
        a->host_seq = 0;
        a->host_ready = true;
    }
    cglm_kv_arena::HostCall &me = a->host_calls[a->host_next];
    if (me.used) CGLM_CUDA(cudaEventSynchronize(me.d2h));   // the call that used this record eight calls ago
    // the staging buffers may still be in use by earlier calls: the input buffer by a kernel, the output buffer by a
    // device-to-host copy.  The most recent user of each is the one to wait for (earlier users precede it in order).
    const cglm_kv_arena::HostCall *last_in = nullptr, *last_out = nullptr;
    for (int back = 1; back < cglm_kv_arena::kHostCalls; ++back) {
        const cglm_kv_arena::HostCall &c =
            a->host_calls[(a->host_next - back + cglm_kv_arena::kHostCalls) % cglm_kv_arena::kHostCalls];
        if (!c.used) continue;
        if (!last_in && c.dev_in == dev_qkv) last_in = &c;
        if (!last_out && c.dev_out == dev_out) last_out = &c;
    }
    const int rec = a->host_next;
    a->host_next = (a->host_next + 1) % cglm_kv_arena::kHostCalls;
    me.seq = ++a->host_seq;
    if (me.seq == 0) me.seq = ++a->host_seq;   // 0 is what a fresh gate word holds
    lock.unlock();
    // A stream wait between two launches would end their programmatic overlap (the stream takes up the wait only once
    // the earlier launch has completed): decode launches instead poll two device words that the copy streams write
    // right behind the data, and the stream carries only event records.  Other kernels wait on the stream as before.
    a->gate_host[2 * rec] = a->gate_host[2 * rec + 1] = me.seq;
    if (last_in) CGLM_CUDA(cudaStreamWaitEvent(a->copy_in, last_in->kernel, 0));
    CGLM_CUDA(cudaMemcpyAsync(dev_qkv, qkv_host, esz * n_tok * row, cudaMemcpyHostToDevice, a->copy_in));
    CGLM_CUDA(cudaMemcpyAsync(a->gate_dev + 2 * rec, a->gate_host + 2 * rec, sizeof(unsigned int), cudaMemcpyHostToDevice, a->copy_in));
    CGLM_CUDA(cudaEventRecord(me.h2d, a->copy_in));
    HostGates gates;
    gates.word[0] = a->gate_dev + 2 * rec;
    gates.value[0] = me.seq;
    gates.event[0] = me.h2d;
    const int last_out_rec = last_out ? static_cast<int>(last_out - a->host_calls) : 0;
    gates.word[1] = last_out ? a->gate_dev + 2 * last_out_rec + 1 : nullptr;
    gates.value[1] = last_out ? last_out->seq : 0;
    gates.event[1] = last_out ? last_out->d2h : nullptr;
    const int rc = forward_impl(a, dev_seqs.data(), n_seq, workspace, workspace_bytes, cuda_stream, &gates);
    if (rc != CGLM_OK) return rc;
    CGLM_CUDA(cudaEventRecord(me.kernel, st));
    CGLM_CUDA(cudaStreamWaitEvent(a->copy_out, me.kernel, 0));
    CGLM_CUDA(cudaMemcpyAsync(out_host, dev_out, esz * n_tok * orow, cudaMemcpyDeviceToHost, a->copy_out));
    CGLM_CUDA(cudaMemcpyAsync(a->gate_dev + 2 * rec + 1, a->gate_host + 2 * rec + 1, sizeof(unsigned int), cudaMemcpyHostToDevice, a->copy_out));
    CGLM_CUDA(cudaEventRecord(me.d2h, a->copy_out));
    me.dev_in = dev_qkv;
    me.dev_out = dev_out;
    me.used = true;
    return CGLM_OK;
}

int cglm_attn_host_drain(cglm_kv_arena *a, void *cuda_stream) {
    if (!a) return CGLM_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    std::lock_guard<std::mutex> lock(a->mu);
    if (!a->host_ready) return CGLM_OK;
    for (auto &c : a->host_calls) {
        if (c.used) CGLM_CUDA(cudaStreamWaitEvent(st, c.d2h, 0));
    }
    return CGLM_OK;
}

int cglm_attn_splitkv_combine(const float *partials, int n_part, int n_head, int head_dim, float *out,
                              void *cuda_stream) {
    if (!partials || !out || n_part <= 0 || n_head <= 0 || head_dim <= 0) return CGLM_ERR_INVALID_ARG;
    combine_kernel<<<n_head, 128, 0, static_cast<cudaStream_t>(cuda_stream)>>>(partials, n_part, n_head, head_dim, out);
    g_launch_count += 1;
    CGLM_CUDA(cudaGetLastError());
    return CGLM_OK;
}

size_t cglm_attn_splitkv_xchg_bytes(int n_rank, int n_head, int head_dim) {
    if (n_rank <= 0 || n_rank > kXchgMaxRanks || n_head <= 0 || head_dim <= 0 || (head_dim & 1)) return 0;
    // a rank's slot holds one block in the layout of a decode partial per kv head; sized for as many kv heads as heads
    const int g_max = n_head < kXchgMaxKvHeads ? n_head : kXchgMaxKvHeads;
    return sizeof(unsigned int) * xchg_slot_word(2, 0, n_rank, g_max * kDecodePartialFloats);
}

int cglm_xchg_alloc(size_t bytes, void **ptr) {
    if (!ptr || bytes == 0) return CGLM_ERR_INVALID_ARG;
    CGLM_CUDA(cudaMalloc(ptr, bytes));
    CGLM_CUDA(cudaMemset(*ptr, 0, bytes));
    CGLM_CUDA(cudaDeviceSynchronize());
    return CGLM_OK;
}

int cglm_xchg_free(void *ptr) {
    if (!ptr) return CGLM_ERR_INVALID_ARG;
    CGLM_CUDA(cudaFree(ptr));
    return CGLM_OK;
}

int cglm_xchg_read(const void *ptr, void *host, size_t bytes) {
    if (!ptr || !host || bytes == 0) return CGLM_ERR_INVALID_ARG;
    CGLM_CUDA(cudaDeviceSynchronize());
    CGLM_CUDA(cudaMemcpy(host, ptr, bytes, cudaMemcpyDeviceToHost));
    return CGLM_OK;
}

int cglm_xchg_export(void *ptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
    if (!ptr || !handle) return CGLM_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    CGLM_CUDA(cudaIpcGetMemHandle(&h, ptr));
    std::memcpy(handle, &h, sizeof(h));
    return CGLM_OK;
}

int cglm_xchg_import(const unsigned char handle[64], int owner_device, void **ptr) {
    if (!handle || !ptr) return CGLM_ERR_INVALID_ARG;
    int dev = -1, can = 0;
    CGLM_CUDA(cudaGetDevice(&dev));
    if (owner_device != dev) {
        CGLM_CUDA(cudaDeviceCanAccessPeer(&can, dev, owner_device));
        if (!can) return CGLM_ERR_UNSUPPORTED;
    }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    // opened with the importing device current: the mapping belongs to this device's context
    CGLM_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    // the mapping must work for plain accesses from this device before a kernel is pointed at it: the runtime
    // reports a broken mapping as an error code here, a kernel would fault
    unsigned int probe = 0xffffffffu;
    CGLM_CUDA(cudaMemcpy(&probe, *ptr, sizeof(probe), cudaMemcpyDeviceToHost));
    void *scratch = nullptr;
    CGLM_CUDA(cudaMalloc(&scratch, 256));
    cudaError_t e = cudaMemcpy(scratch, *ptr, 256, cudaMemcpyDeviceToDevice);
    cudaFree(scratch);
    CGLM_CUDA(e);
    return CGLM_OK;
}

int cglm_attn_splitkv_step(cglm_kv_arena *a, const cglm_attn_seq *seq, void *const *xchg, int n_rank, int rank, float *out,
                           int combine, unsigned int timeout_us, void *workspace, size_t workspace_bytes, void *cuda_stream) {
    if (!a || !seq || !xchg || n_rank <= 0 || n_rank > kXchgMaxRanks || rank < 0 || rank >= n_rank) return CGLM_ERR_INVALID_ARG;
    if (combine && (!out || (reinterpret_cast<uintptr_t>(out) & 15))) return CGLM_ERR_INVALID_ARG;
    if (!workspace) return CGLM_ERR_WORKSPACE;
    const cglm_attn_desc &d = a->desc;
    if (!fast_decode_shape(a) || d.n_kv_head > kXchgMaxKvHeads) {
        std::snprintf(g_err, sizeof(g_err), "the fused split-KV step needs head_dim 128, <= 16 q heads per kv head, <= %d kv heads and a capacity that is a multiple of 8",
                      kXchgMaxKvHeads);
        return CGLM_ERR_UNSUPPORTED;
    }
    const cglm_attn_seq &s = *seq;
    if (!s.q || !s.k || !s.v || s.qlen != 1 || s.n_past < 0 || s.slot < 0 || s.slot >= a->n_slots) return CGLM_ERR_INVALID_ARG;
    if (s.flags & ~(CGLM_SEQ_NO_APPEND | CGLM_SEQ_USE_KV_LOCAL | CGLM_SEQ_PARTIAL | CGLM_SEQ_CACHE_SETTLED)) return CGLM_ERR_INVALID_ARG;
    if ((s.flags & CGLM_SEQ_USE_KV_LOCAL) && s.kv_local < 0) return CGLM_ERR_INVALID_ARG;
    const int kv_before = (s.flags & CGLM_SEQ_USE_KV_LOCAL) ? s.kv_local : d.n_virtual + s.n_past;
    const int appended = (s.flags & CGLM_SEQ_NO_APPEND) ? 0 : 1;
    if (static_cast<long long>(kv_before) + appended > a->user_desc.max_len) return CGLM_ERR_INVALID_ARG;
    if (kv_before + appended < 1) {
        std::snprintf(g_err, sizeof(g_err), "a rank of a fused split-KV step must hold at least one attended position");
        return CGLM_ERR_UNSUPPORTED;
    }
    if (d.rope_type == CGLM_ROPE_CHATGLM && !s.position_ids && s.n_ctx < 2) return CGLM_ERR_INVALID_ARG;
    if (!decode_rows_aligned(s.q, s.k, s.v, s.q_head_stride, s.kv_head_stride, s.q_roped, s.k_roped)) {
        std::snprintf(g_err, sizeof(g_err), "q, k, v rows must be 16-byte aligned (pointers and head strides)");
        return CGLM_ERR_UNSUPPORTED;
    }
    const WsLayout lay = ws_layout(d, a->n_sm, 1, 0, 0);
    if (workspace_bytes < lay.total) return CGLM_ERR_WORKSPACE;
    XchgDev xd = {};
    for (int r = 0; r < n_rank; ++r) {
        if (!xchg[r] || (reinterpret_cast<uintptr_t>(xchg[r]) & 15)) return CGLM_ERR_INVALID_ARG;
        xd.peer[r] = static_cast<unsigned int *>(xchg[r]);
    }
    xd.out = out;
    xd.n_rank = n_rank;
    xd.rank = rank;
    xd.combine = combine != 0;
    xd.timeout_us = timeout_us ? timeout_us : 20000u;
    LaunchCtx cx = make_launch_ctx(a, static_cast<uint8_t *>(workspace), lay, static_cast<cudaStream_t>(cuda_stream));
    static thread_local DecodeTableDyn tab;
    SeqDev &o = tab.seqs[0];
    o = SeqDev{};
    o.q = s.q; o.k = s.k; o.v = s.v;
    o.q_tok_stride = s.q_tok_stride; o.q_head_stride = s.q_head_stride;
    o.kv_tok_stride = s.kv_tok_stride; o.kv_head_stride = s.kv_head_stride;
    o.position_ids = s.position_ids;
    o.out = nullptr; o.q_roped = s.q_roped; o.k_roped = s.k_roped;
    o.partial = nullptr;   // the kernel points it into the local exchange buffer once it knows the step number
    o.slot = s.slot; o.qlen = 1; o.n_past = s.n_past; o.n_ctx = s.n_ctx;
    o.kv_before = kv_before;
    o.flags = s.flags | CGLM_SEQ_PARTIAL;
    tab.n_seq = 1;
    tab.settled = (s.flags & CGLM_SEQ_CACHE_SETTLED) ? 1 + decode_l2_ahead() : 0;
    tab.charge = decode_charge();
    tab.gate[0] = tab.gate[1] = nullptr;
    tab.prefix[0] = 0;
    tab.prefix[1] = (kv_before + appended + kDecodeTile - 1) / kDecodeTile;
    tab.trigger = decode_trigger(tab.settled != 0, static_cast<long long>(tab.prefix[1]) * d.n_kv_head);
    CGLM_CUDA(launch_decode(cx, tab, false, &xd));
    return CGLM_OK;
}

namespace {

// Both GEMM operands as 3-D tensors {64 k of a block, rows, k blocks}: one box brings `kb` consecutive 64-k blocks of its
// rows, which land in shared memory as kb consecutive K-major tiles (fewer, larger TMA operations per byte).
bool encode_linear_maps(EncodeTiledFn enc, const void *x_f16, int n_tok, const void *weight_f16, int n_feat, int K, int x_rows,
                        int w_rows, int kb, CUtensorMap *x_map, CUtensorMap *w_map) {
    const cuuint32_t estr[3] = {1, 1, 1};
    cuuint64_t xdims[3] = {64, static_cast<cuuint64_t>(n_tok), static_cast<cuuint64_t>(K / 64)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(K) * 2, 128};
    cuuint32_t xbox[3] = {64, static_cast<cuuint32_t>(x_rows), static_cast<cuuint32_t>(kb)};
    cuuint64_t wdims[3] = {64, static_cast<cuuint64_t>(n_feat), static_cast<cuuint64_t>(K / 64)};
    cuuint32_t wbox[3] = {64, static_cast<cuuint32_t>(w_rows), static_cast<cuuint32_t>(kb)};
    return enc(x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(x_f16), xdims, strides, xbox, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS &&
           enc(w_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(weight_f16), wdims, strides, wbox, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The kernel with the features on the M side when the shape and the workspace allow it (out-features a multiple of 128,
// a workspace that holds the Linear scratch).  CGLM_LINEAR_TOKENS_ON_M=1 keeps the other kernel (tuning knob, read once).
// Returns CGLM_OK when launched, 1 when the other kernel has to take the call.
int try_linear_fm(int device, int n_sm, cudaStream_t st, const LaunchCtx *qkv_cx, void *workspace, size_t workspace_bytes,
                  const void *x_f16, int n_tok, int K, const void *weight_f16, int n_feat, const float *bias, const int *slots,
                  const int *n_past, float *q_out, void *out, bool out_f16) {
    static const bool tokens_on_m = [] { const char *e = std::getenv("CGLM_LINEAR_TOKENS_ON_M"); return e && std::atoi(e) != 0; }();
    if (tokens_on_m || workspace_bytes < sizeof(WsHeader) + kLinearScratchBytes) return 1;
    if (reinterpret_cast<uintptr_t>(bias) & 15) return 1;   // this kernel reads the bias four features at a time
    LinearFmPlan plan;
    if (!linear_fm_plan(n_tok, K, n_feat, n_sm, kLinearScratchBytes, &plan)) return 1;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return CGLM_ERR_CUDA;
    CUtensorMap x_map, w_map;
    if (!encode_linear_maps(enc, x_f16, n_tok, weight_f16, n_feat, K, plan.n_box, 128, plan.kb, &x_map, &w_map)) return 1;
    LaunchCtx cx;
    if (qkv_cx) {
        cx = *qkv_cx;
    } else {
        cx = LaunchCtx{};
        cx.hdr = static_cast<WsHeader *>(workspace);
        cx.stream = st;
        cx.n_sm = n_sm;
        cx.device = device;
    }
    float *scratch = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + sizeof(WsHeader));
    CGLM_CUDA(launch_linear_fm(cx, plan, x_map, w_map, slots, n_past, n_tok, K, n_feat, bias, q_out, out, out_f16, scratch));
    return CGLM_OK;
}

}  // namespace

size_t cglm_linear_workspace_bytes(void) { return sizeof(WsHeader) + kLinearScratchBytes; }

int cglm_linear_kernel_plan(int n_tok, int in_features, int out_features, int n_sm, int plan[8]) {
    if (!plan || n_sm <= 0) return 0;
    LinearFmPlan p;
    if (!linear_fm_plan(n_tok, in_features, out_features, n_sm, kLinearScratchBytes, &p)) return 0;
    plan[0] = p.n_box; plan[1] = p.tiles; plan[2] = p.token_tiles; plan[3] = p.ksplit;
    plan[4] = p.blocks_per_cta; plan[5] = p.kb; plan[6] = p.n_stages; plan[7] = p.tmem_cols;
    return 1;
}

int cglm_qkv_linear_forward(cglm_kv_arena *a, const cglm_attn_seq *seqs, int n_seq, const void *x_f16, int hidden,
                            const void *weight_f16, const float *bias, float *q_roped, void *workspace, size_t workspace_bytes,
                            void *cuda_stream) {
    if (!a || !seqs || n_seq <= 0 || !x_f16 || !weight_f16 || !q_roped || hidden <= 0) return CGLM_ERR_INVALID_ARG;
    if (!workspace || workspace_bytes < sizeof(WsHeader)) return CGLM_ERR_WORKSPACE;
    const cglm_attn_desc &d = a->desc;
    if (!a->has_tmaps || d.head_dim != 128 || (d.rope_type != CGLM_ROPE_CHATGLM2 && d.rope_type != CGLM_ROPE_DISABLED) ||
        hidden % 64 != 0 || n_seq > 128) {
        std::snprintf(g_err, sizeof(g_err), "the fused qkv Linear needs head_dim 128, the GLM-2/3/4 rope mode (or none), hidden %% 64 == 0 and at most 128 sequences");
        return CGLM_ERR_UNSUPPORTED;
    }
    if ((reinterpret_cast<uintptr_t>(x_f16) | reinterpret_cast<uintptr_t>(weight_f16) | reinterpret_cast<uintptr_t>(q_roped)) & 15)
        return CGLM_ERR_INVALID_ARG;
    int slots[128], n_past[128];
    for (int i = 0; i < n_seq; ++i) {
        const cglm_attn_seq &s = seqs[i];
        if (s.qlen != 1 || s.n_past < 0 || s.slot < 0 || s.slot >= a->n_slots) return CGLM_ERR_INVALID_ARG;
        if (static_cast<long long>(d.n_virtual) + s.n_past + 1 > a->user_desc.max_len) return CGLM_ERR_INVALID_ARG;
        slots[i] = s.slot;
        n_past[i] = s.n_past;
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return CGLM_ERR_CUDA;
    const int n_feat = (d.n_head + 2 * d.n_kv_head) * d.head_dim;
    // Up to 32 sequences the kernel with the features on the M side is faster (8 sequences: 11.7 against 17.3 us).  Beyond,
    // the last thread block to arrive at a V head's tile scatters that head's whole V^T update (2-byte stores, one 32-byte
    // sector each: 8192 per tile at 64 sequences) while the other kernel spreads it over 8 thread blocks (64 sequences:
    // 24.2 against 18.2 us).
    if (n_seq <= 32) {
        const WsLayout lay = ws_layout(d, a->n_sm, 1, 0, 0);
        LaunchCtx cx = make_launch_ctx(a, static_cast<uint8_t *>(workspace), lay, static_cast<cudaStream_t>(cuda_stream));
        const int rc = try_linear_fm(a->device, a->n_sm, static_cast<cudaStream_t>(cuda_stream), &cx, workspace, workspace_bytes, x_f16,
                                     n_seq, hidden, weight_f16, n_feat, bias, slots, n_past, q_roped, nullptr, false);
        if (rc <= 0) return rc;
    }
    CUtensorMap x_map, w_map;
    // Both operands as 3-D tensors {64 k of a block, rows, k blocks}: one box brings `kb` consecutive 64-k blocks of its
    // rows, which land in shared memory as kb consecutive K-major tiles (fewer, larger TMA operations per byte).
    int kb = qkv_linear_k_blocks(n_seq, hidden);
    {   // CGLM_QKV_K_BLOCKS overrides the choice (tuning knob, read once; a value that does not divide hidden / 64 or leaves
        // fewer than two stages is ignored)
        static const int forced = [] { const char *e = std::getenv("CGLM_QKV_K_BLOCKS"); return e ? std::atoi(e) : 0; }();
        if (forced >= 1 && forced <= 16 && (hidden / 64) % forced == 0 &&
            forced * (qkv_linear_x_rows(n_seq) * 128 + 4096) <= 200 * 1024) kb = forced;
    }
    const int x_rows = qkv_linear_x_rows(n_seq);
    for (;; kb = 1) {
        const cuuint32_t estr[3] = {1, 1, 1};
        cuuint64_t xdims[3] = {64, static_cast<cuuint64_t>(n_seq), static_cast<cuuint64_t>(hidden / 64)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(hidden) * 2, 128};
        cuuint32_t xbox[3] = {64, static_cast<cuuint32_t>(x_rows), static_cast<cuuint32_t>(kb)};
        cuuint64_t wdims[3] = {64, static_cast<cuuint64_t>(n_feat), static_cast<cuuint64_t>(hidden / 64)};
        cuuint32_t wbox[3] = {64, 32, static_cast<cuuint32_t>(kb)};
        if (enc(&x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(x_f16), xdims, strides, xbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS &&
            enc(&w_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(weight_f16), wdims, strides, wbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
            break;
        }
        if (kb == 1) {
            std::snprintf(g_err, sizeof(g_err), "cuTensorMapEncodeTiled failed for the qkv Linear");
            return CGLM_ERR_CUDA;
        }
    }
    const WsLayout lay = ws_layout(d, a->n_sm, 1, 0, 0);
    LaunchCtx cx = make_launch_ctx(a, static_cast<uint8_t *>(workspace), lay, static_cast<cudaStream_t>(cuda_stream));
    CGLM_CUDA(launch_qkv_linear(cx, x_map, w_map, slots, n_past, n_seq, hidden, n_feat, kb, bias, q_roped));
    return CGLM_OK;
}

int cglm_linear_forward(const void *x_f16, int n_tok, int in_features, const void *weight_f16, int out_features,
                        const float *bias, void *out, int out_is_f16, void *workspace, size_t workspace_bytes, void *cuda_stream) {
    if (!x_f16 || !weight_f16 || !out || n_tok <= 0 || in_features <= 0 || out_features <= 0) return CGLM_ERR_INVALID_ARG;
    if (!workspace || workspace_bytes < sizeof(WsHeader)) return CGLM_ERR_WORKSPACE;
    if (in_features % 64 != 0 || out_features % 32 != 0) {
        std::snprintf(g_err, sizeof(g_err), "the Linear kernel needs in_features %% 64 == 0 and out_features %% 32 == 0");
        return CGLM_ERR_UNSUPPORTED;
    }
    if ((reinterpret_cast<uintptr_t>(x_f16) | reinterpret_cast<uintptr_t>(weight_f16) | reinterpret_cast<uintptr_t>(out)) & 15)
        return CGLM_ERR_INVALID_ARG;
    int device = -1;
    CGLM_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return CGLM_ERR_NO_DEVICE;
    {   // tcgen05: compute capability 10.x only (checked once per device)
        static std::atomic<int> major_of[kMaxDevices];
        int major = major_of[device].load(std::memory_order_relaxed);
        if (major == 0) {
            CGLM_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
            major_of[device].store(major, std::memory_order_relaxed);
        }
        if (major != 10) return CGLM_ERR_NO_DEVICE;
    }
    {
        static std::atomic<int> sm_of[kMaxDevices];
        int n_sm = sm_of[device].load(std::memory_order_relaxed);
        if (n_sm == 0) {
            CGLM_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device));
            sm_of[device].store(n_sm, std::memory_order_relaxed);
        }
        const int rc = try_linear_fm(device, n_sm, static_cast<cudaStream_t>(cuda_stream), nullptr, workspace, workspace_bytes, x_f16,
                                     n_tok, in_features, weight_f16, out_features, bias, nullptr, nullptr, nullptr, out, out_is_f16 != 0);
        if (rc <= 0) return rc;
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return CGLM_ERR_CUDA;
    const int tile_tok = n_tok < 128 ? n_tok : 128;
    const int x_rows = qkv_linear_x_rows(tile_tok);
    CUtensorMap x_map, w_map;
    for (int kb = qkv_linear_k_blocks(tile_tok, in_features);; kb = 1) {
        const cuuint32_t estr[3] = {1, 1, 1};
        cuuint64_t xdims[3] = {64, static_cast<cuuint64_t>(n_tok), static_cast<cuuint64_t>(in_features / 64)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(in_features) * 2, 128};
        cuuint32_t xbox[3] = {64, static_cast<cuuint32_t>(x_rows), static_cast<cuuint32_t>(kb)};
        cuuint64_t wdims[3] = {64, static_cast<cuuint64_t>(out_features), static_cast<cuuint64_t>(in_features / 64)};
        cuuint32_t wbox[3] = {64, 32, static_cast<cuuint32_t>(kb)};
        if (enc(&x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(x_f16), xdims, strides, xbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS &&
            enc(&w_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(weight_f16), wdims, strides, wbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
            CGLM_CUDA(launch_linear_plain(device, static_cast<cudaStream_t>(cuda_stream), static_cast<WsHeader *>(workspace), x_map,
                                          w_map, n_tok, in_features, out_features, kb, bias, out, out_is_f16 != 0));
            return CGLM_OK;
        }
        if (kb == 1) break;
    }
    std::snprintf(g_err, sizeof(g_err), "cuTensorMapEncodeTiled failed for the Linear");
    return CGLM_ERR_CUDA;
}

int cglm_convert_f32_to_f16(const float *src, void *dst_f16, size_t n, void *cuda_stream) {
    if (!src || !dst_f16) return CGLM_ERR_INVALID_ARG;
    if (n == 0) return CGLM_OK;
    const size_t blocks = (n + 1023) / 1024;
    f32_to_f16_kernel<<<static_cast<unsigned>(blocks < 4096 ? blocks : 4096), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        src, static_cast<__half *>(dst_f16), n);
    g_launch_count += 1;
    CGLM_CUDA(cudaGetLastError());
    return CGLM_OK;
}

int cglm_seq_advance(int *n_past_dev, int n, int delta, void *cuda_stream) {
    if (!n_past_dev || n <= 0) return CGLM_ERR_INVALID_ARG;
    seq_advance_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(cuda_stream)>>>(n_past_dev, n, delta);
    g_launch_count += 1;
    CGLM_CUDA(cudaGetLastError());
    return CGLM_OK;
}

int cglm_kv_load_prefix(cglm_kv_arena *a, int slot, const void *past_kv, void *cuda_stream) {
    if (!a || !past_kv || slot < 0 || slot >= a->n_slots) return CGLM_ERR_INVALID_ARG;
    const cglm_attn_desc &d = a->desc;
    if (d.n_virtual == 0) return CGLM_OK;
    const long long n = static_cast<long long>(d.n_kv_head) * d.n_virtual * d.head_dim;
    const int blocks = static_cast<int>((n + 255) / 256 < 1024 ? (n + 255) / 256 : 1024);
    load_prefix_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<const uint16_t *>(past_kv), static_cast<uint16_t *>(cglm_kv_arena_k_cache(a, slot)),
        static_cast<uint16_t *>(cglm_kv_arena_v_cache(a, slot)), d.n_kv_head, d.n_virtual, d.head_dim, d.max_len);
    g_launch_count += 1;
    CGLM_CUDA(cudaGetLastError());
    return CGLM_OK;
}

const char *cglm_status_string(int status) {
    switch (status) {
    case CGLM_OK: return "ok";
    case CGLM_ERR_INVALID_ARG: return "invalid argument";
    case CGLM_ERR_CUDA: return "CUDA call failed";
    case CGLM_ERR_WORKSPACE: return "workspace missing, too small or not initialised";
    case CGLM_ERR_UNSUPPORTED: return "shape not supported";
    case CGLM_ERR_TIMEOUT: return "device-side wait timed out";
    case CGLM_ERR_NO_DEVICE: return "no usable CUDA device (sm_100a required)";
    default: return "unknown status";
    }
}

const char *cglm_last_error_string(void) { return g_err; }

unsigned long long cglm_launch_count(void) { return g_launch_count.load(); }

}  // extern "C"
