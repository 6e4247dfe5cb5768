// cglm_attn_decode_static: the fused decode step for hosts that cannot give the library any scratch memory.
//
// cglm_attn_forward needs a caller-allocated workspace for the partial results of sequences that are split
// across thread blocks.  Some hosts cannot provide one at call time: an inference server whose own allocator
// has already claimed the whole GPU, a plugin sandbox that forbids the plugin to call cudaMalloc, a control loop
// that must not touch the allocator once it is running.  For them this entry point keeps that scratch in a
// fixed array inside the library image.  Every GPU that loads the library carries the array (about 5 MiB) until
// the process exits, whether or not the entry point is ever called.
#include <cstdio>
#include <mutex>

#include "common.cuh"

using namespace cglm;

struct cglm_kv_arena;   // defined in cglm_attn_api.cu; only passed through here

// accessors implemented next to the arena's definition
namespace cglm {
const CUtensorMap *arena_k_map(const cglm_kv_arena *a);
const CUtensorMap *arena_v_map(const cglm_kv_arena *a);
bool arena_fast_decode(const cglm_kv_arena *a);
int arena_device(const cglm_kv_arena *a);
int arena_sm_count(const cglm_kv_arena *a);
AttnShape arena_shape(const cglm_kv_arena *a);
const float2 *arena_rope_tab(const cglm_kv_arena *a, int *len);
void set_last_error(const char *text);   // what cglm_last_error_string returns on this thread
}  // namespace cglm

namespace {

// Limits of the static scratch: what one call may ask for.
constexpr int kStaticMaxSeq = kDecodeMaxSeqPerLaunch;   // sequences per call (128)
constexpr int kStaticMaxKvHeads = 32;                    // kv heads per sequence
constexpr int kStaticMaxCtas = 2 * 148;                  // thread blocks of the decode launch: two per SM of a B200
constexpr size_t kStaticCountersOff = sizeof(WsHeader);
constexpr size_t kStaticCountersBytes = sizeof(int) * kStaticMaxSeq * kStaticMaxKvHeads;
constexpr size_t kStaticGroups = (kStaticMaxCtas + kDecodeMergeFan - 1) / kDecodeMergeFan;
constexpr size_t kStaticGCountersOff = kStaticCountersOff + kStaticCountersBytes;
constexpr size_t kStaticPartialsOff = kStaticGCountersOff + 256;   // 2 * 19 group counters fit in 256 bytes
constexpr size_t kStaticPartialsBytes = sizeof(float) * kDecodePartialFloats * 2 * kStaticMaxCtas;
constexpr size_t kStaticGPartialsOff = kStaticPartialsOff + kStaticPartialsBytes;
constexpr size_t kStaticScratchBytes = kStaticGPartialsOff + sizeof(float) * kDecodePartialFloats * 2 * kStaticGroups;   // 5 258 496 bytes
static_assert(sizeof(int) * 2 * kStaticGroups <= 256, "group counters fit their region");
static_assert(kStaticCountersOff % 256 == 0 && kStaticPartialsOff % 256 == 0, "regions stay 256-byte aligned");

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

unsigned char *g_scratch_ptr[kMaxDevices] = {};   // device address of the array, per device ordinal
std::mutex g_setup_mu;

// One-time set-up per device, with that device current: resolve the array's device address.
int scratch_for_current_device(unsigned char **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        { char msg__[200]; std::snprintf(msg__, sizeof(msg__), "cudaGetDevice: %s", cudaGetErrorString(e)); set_last_error(msg__); }
        return CGLM_ERR_NO_DEVICE;
    }
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (!g_scratch_ptr[dev]) {
        unsigned char *p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_scratch);
        if (e != cudaSuccess || !p) {
            { char msg__[200]; std::snprintf(msg__, sizeof(msg__), "cudaGetSymbolAddress(static scratch): %s",
                          cudaGetErrorString(e)); set_last_error(msg__); }
            return CGLM_ERR_CUDA;
        }
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return CGLM_OK;
}

}  // namespace

extern "C" int cglm_attn_decode_static(cglm_kv_arena *arena, const cglm_attn_seq *seqs, int n_seq, int wait_and_check,
                                       void *cuda_stream) {
    if (!arena || !seqs || n_seq <= 0) return CGLM_ERR_INVALID_ARG;
    if (!arena_fast_decode(arena)) return CGLM_ERR_UNSUPPORTED;   // head_dim 128, <=16 q heads per kv head, capacity % 8 == 0
    const AttnShape shape = arena_shape(arena);
    if (n_seq > kStaticMaxSeq || shape.G > kStaticMaxKvHeads || decode_max_ctas(arena_sm_count(arena)) > kStaticMaxCtas) {
        { char msg__[200]; std::snprintf(msg__, sizeof(msg__),
                      "static scratch covers at most %d sequences, %d kv heads and %d thread blocks per call", kStaticMaxSeq,
                      kStaticMaxKvHeads, kStaticMaxCtas); set_last_error(msg__); }
        return CGLM_ERR_WORKSPACE;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != arena_device(arena)) return CGLM_ERR_INVALID_ARG;
    unsigned char *scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc != CGLM_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);

    const int n_slots = cglm_kv_arena_n_slots(arena);
    static thread_local DecodeTableDyn tab;
    tab.n_seq = n_seq;
    tab.settled = 0;
    tab.trigger = 2;
    tab.charge = 6;
    tab.gate[0] = tab.gate[1] = nullptr;
    tab.prefix[0] = 0;
    for (int i = 0; i < n_seq; ++i) {
        const cglm_attn_seq &s = seqs[i];
        if (!s.q || !s.k || !s.v || !s.out || s.qlen != 1 || s.n_past < 0 || s.flags != 0) return CGLM_ERR_INVALID_ARG;
        // the slot selects where the helper warp appends and which rows TMA reads: never outside the arena
        if (s.slot < 0 || s.slot >= n_slots) return CGLM_ERR_INVALID_ARG;
        if ((reinterpret_cast<uintptr_t>(s.out) & 15) || (reinterpret_cast<uintptr_t>(s.q) & 3) ||
            (reinterpret_cast<uintptr_t>(s.k) & 3) || (reinterpret_cast<uintptr_t>(s.v) & 3))
            return CGLM_ERR_INVALID_ARG;
        if (!decode_rows_aligned(s.q, s.k, s.v, s.q_head_stride, s.kv_head_stride, s.q_roped, s.k_roped)) {
            set_last_error("q, k, v rows must be 16-byte aligned (pointers and head strides)");
            return CGLM_ERR_UNSUPPORTED;
        }
        // against the capacity the caller asked for (shape.M is the row pitch, which an arena may have rounded up)
        if (static_cast<long long>(shape.V) + s.n_past + 1 > cglm_kv_arena_desc(arena)->max_len) return CGLM_ERR_INVALID_ARG;
        if (shape.rope_type == CGLM_ROPE_CHATGLM && !s.position_ids && s.n_ctx < 2) return CGLM_ERR_INVALID_ARG;
        SeqDev &o = tab.seqs[i];
        o.q = s.q; o.k = s.k; o.v = s.v;
        o.q_tok_stride = s.q_tok_stride; o.q_head_stride = s.q_head_stride;
        o.kv_tok_stride = s.kv_tok_stride; o.kv_head_stride = s.kv_head_stride;
        o.position_ids = s.position_ids;
        o.out = s.out; o.q_roped = s.q_roped; o.k_roped = s.k_roped; o.partial = nullptr;
        o.slot = s.slot; o.qlen = 1; o.n_past = s.n_past; o.n_ctx = s.n_ctx;
        o.kv_before = shape.V + s.n_past;
        o.flags = 0; o.tok_begin = 0; o.pad = 0;
        tab.prefix[i + 1] = tab.prefix[i] + (o.kv_before + 1 + kDecodeTile - 1) / kDecodeTile;
    }
    // The array keeps whatever the last call left.  The status word and the per-item completion counters must
    // start at zero (a call that ran into a timeout can leave counters behind); the partial slots need no
    // clearing, every slot that is read was written by the same launch.
    cudaError_t e = cudaMemsetAsync(scratch, 0, kStaticPartialsOff, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(scratch, static_cast<int>(kWsMagic & 0xffu), sizeof(unsigned int), st);   // header magic
    if (e != cudaSuccess) {
        { char msg__[200]; std::snprintf(msg__, sizeof(msg__), "cudaMemsetAsync: %s", cudaGetErrorString(e)); set_last_error(msg__); }
        return CGLM_ERR_CUDA;
    }
    LaunchCtx cx;
    cx.shape = shape;
    cx.k_base = static_cast<uint16_t *>(cglm_kv_arena_k_cache(arena, 0));
    cx.v_base = static_cast<uint16_t *>(cglm_kv_arena_v_cache(arena, 0));
    cx.hdr = reinterpret_cast<WsHeader *>(scratch);
    cx.counters = reinterpret_cast<int *>(scratch + kStaticCountersOff);
    cx.gcounters = reinterpret_cast<int *>(scratch + kStaticGCountersOff);
    cx.partials = reinterpret_cast<float *>(scratch + kStaticPartialsOff);
    cx.gpartials = reinterpret_cast<float *>(scratch + kStaticGPartialsOff);
    cx.q_stage = nullptr;
    cx.k_map = arena_k_map(arena);
    cx.v_map = arena_v_map(arena);
    cx.rope_tab = arena_rope_tab(arena, &cx.rope_tab_len);
    cx.stream = st;
    cx.n_sm = arena_sm_count(arena);
    cx.device = dev;
    e = launch_decode(cx, tab);
    if (e != cudaSuccess) {
        { char msg__[200]; std::snprintf(msg__, sizeof(msg__), "decode launch: %s", cudaGetErrorString(e)); set_last_error(msg__); }
        return CGLM_ERR_CUDA;
    }
    if (wait_and_check) {
        int status = 0;
        e = cudaMemcpyAsync(&status, &cx.hdr->status, sizeof(int), cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) {
            { char msg__[200]; std::snprintf(msg__, sizeof(msg__), "status read: %s", cudaGetErrorString(e)); set_last_error(msg__); }
            return CGLM_ERR_CUDA;
        }
        return status;
    }
    return CGLM_OK;
}
