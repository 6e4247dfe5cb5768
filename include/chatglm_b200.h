// chatglm_b200.h -- C++ host side of the B200 attention KV-cache path.
//
// Mirrors the module surface of li-plus/chatglm.cpp (chatglm.h) for the one path this library owns, so that
// BasicBlock::forward / GLMBlock::forward (chatglm.h:488-503, chatglm.cpp:1070-1087) can call it in place of
// the ggml graph that BasicAttention::forward builds:
//   - chatglm::RopeType, chatglm::AttentionMaskType        same enumerators and values (chatglm.h:93-104)
//   - chatglm::ModelContext                                 owner of the kv buffer, a scratch workspace and a stream
//                                                           (ctx_kv / buf_kv / backend of chatglm.h:331-348)
//   - chatglm::Tensor                                       ne[]/nb[] shaped device tensor (ggml_tensor stand-in; ggml
//                                                           itself is not a dependency)
//   - chatglm::BasicAttention                               same constructor arguments, public members and forward
//                                                           argument list (chatglm.h:440-472)
//   - CHATGLM_CHECK / CHATGLM_THROW                         std::runtime_error("file:line message") (chatglm.h:16-29)
// Everything below executes through the C ABI of cglm_attn.h; there is no CPU path.
#pragma once

#include <cstdint>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "cglm_attn.h"

namespace chatglm {

// ---- error handling (chatglm.h:16-35) ------------------------------------------------------------------
class LogMessageFatal {
  public:
    LogMessageFatal(const char *file, int line) { oss_ << file << ':' << line << ' '; }
    [[noreturn]] ~LogMessageFatal() noexcept(false) { throw std::runtime_error(oss_.str()); }
    std::ostringstream &stream() { return oss_; }

  private:
    std::ostringstream oss_;
};

#define CHATGLM_THROW ::chatglm::LogMessageFatal(__FILE__, __LINE__).stream()
#define CHATGLM_CHECK(cond) \
    if (!(cond)) CHATGLM_THROW << "check failed (" #cond ") "
// a non-zero status of the C ABI becomes the same exception a failed CHATGLM_CHECK_CUDA raises
#define CHATGLM_CHECK_CGLM(call)                                                                              \
    do {                                                                                                      \
        int status__ = (call);                                                                                \
        CHATGLM_CHECK(status__ == CGLM_OK) << "cglm error: " << cglm_status_string(status__) << ' '          \
                                           << cglm_last_error_string();                                       \
    } while (false)

// ---- enums (chatglm.h:93-104) --------------------------------------------------------------------------
enum class RopeType {
    GPTJ = 0,
    NEOX = 2,
    CHATGLM = 4,
    CHATGLM2 = 8,
    DISABLED = 10000,
};

enum class AttentionMaskType {
    CAUSAL,
    CHATGLM,
};

// ---- tensors -------------------------------------------------------------------------------------------
// Device tensor with ggml's conventions: ne[0] is the innermost extent, nb[] are byte strides.
enum TensorType { TYPE_F32 = 0, TYPE_F16 = 1, TYPE_I32 = 26 };   // numeric values of ggml_type

struct Tensor {
    TensorType type = TYPE_F32;
    int64_t ne[4] = {1, 1, 1, 1};
    size_t nb[4] = {0, 0, 0, 0};
    void *data = nullptr;   // device memory
    bool owned = false;
};

size_t element_size(TensorType type);
size_t nbytes(const Tensor *t);

// ---- context (chatglm.h:331-348) -------------------------------------------------------------------------
// Owns the kv arena of every BasicAttention created against it, a scratch workspace, per-step activation
// buffers and the CUDA stream all work is enqueued on.  Like the reference's ModelContext it is used by one
// host thread at a time.
class ModelContext {
  public:
    explicit ModelContext(void *cuda_stream = nullptr);
    ~ModelContext();
    ModelContext(const ModelContext &) = delete;
    ModelContext &operator=(const ModelContext &) = delete;

    // Allocates the kv buffer for every BasicAttention registered so far, as build_layers does with
    // ggml_backend_alloc_ctx_tensors(ctx_kv) after constructing the layers (chatglm.h:627-628).
    void alloc_kv();
    bool kv_allocated() const { return arena_ != nullptr; }

    // per-step device tensors (the reference's ctx_b scratch context); freed by reset_scratch()
    Tensor *new_tensor_1d(TensorType type, int64_t ne0);
    Tensor *new_tensor_2d(TensorType type, int64_t ne0, int64_t ne1);
    void reset_scratch();

    // ggml_backend_tensor_set / ggml_backend_tensor_get
    void tensor_set(Tensor *t, const void *host, size_t offset, size_t size);
    void tensor_get(const Tensor *t, void *host, size_t offset, size_t size);
    void synchronize();

    void *stream() const { return stream_; }
    cglm_kv_arena *arena() const { return arena_; }

  private:
    friend class BasicAttention;
    // creates the (still unallocated) cache tensors of one attention module and returns its arena slot
    int register_attention(const cglm_attn_desc &desc, Tensor **k_cache, Tensor **v_cache);
    void ensure_workspace(int n_seq, int max_qlen);

    void *stream_;
    cglm_kv_arena *arena_ = nullptr;
    cglm_attn_desc desc_{};
    bool have_desc_ = false;
    std::vector<std::unique_ptr<Tensor>> kv_tensors_;
    std::vector<std::unique_ptr<Tensor>> scratch_;
    void *workspace_ = nullptr;
    size_t workspace_bytes_ = 0;
};

// ---- graph inputs (chatglm.cpp:1123-1154, 1315-1327) ---------------------------------------------------------
// position ids of ChatGLM2/3/4: n_past .. n_past+qlen-1
std::vector<int> make_position_ids_glm2(int qlen, int n_past);
// position ids of ChatGLM-6B v1: [min(p, n_ctx-2)] ++ [max(p-(n_ctx-2), 0)], p = n_past+i
std::vector<int> make_position_ids_glm(int qlen, int n_past, int n_ctx);

// ---- the attention module (chatglm.h:440-472) ---------------------------------------------------------------
class BasicAttention {
  public:
    BasicAttention() = default;
    // Same arguments as the reference.  use_qkv_bias / use_dense_bias configure the two Linears, which stay
    // with the caller; they are accepted and ignored here.  The caches exist once mctx->alloc_kv() ran.
    BasicAttention(ModelContext *mctx, int hidden_size, int num_attention_heads, int num_key_value_heads,
                   int max_length, bool use_qkv_bias, bool use_dense_bias, bool interleaved_qkv, RopeType rope_type,
                   float rope_theta, AttentionMaskType attn_mask_type, int num_virtual_tokens);

    // Everything BasicAttention::forward does between query_key_value.forward (chatglm.cpp:629) and dense.forward
    // (chatglm.cpp:719).
    //   qkv            f32 [qlen, (#h + 2 * #kvh) * d]: ne = {(#h + 2#kvh) * d, qlen}
    //   attention_mask accepted for signature parity; the v1 mask it would carry (chatglm.cpp:1126-1140) is applied
    //                  from attn_mask_type, so the tensor may be null
    //   position_ids   i32 [qlen] (or [2 * qlen] for RopeType::CHATGLM) on the device; null derives them from
    //                  n_past (and n_ctx, see set_n_ctx)
    // Returns context_layer f32 [qlen, hidden] allocated from mctx's scratch.  Enqueued on mctx's stream.
    Tensor *forward(ModelContext *mctx, Tensor *qkv, Tensor *attention_mask, Tensor *position_ids, int n_past) const;

    // prompt length of the running generation; only RopeType::CHATGLM with null position_ids reads it
    void set_n_ctx(int n_ctx) { n_ctx_ = n_ctx; }

    // P-Tuning v2 prefix of this layer (BasicModel::load_prefix_cache, chatglm.h:580-615):
    // past_kv f16 [2, #kvh, v, d] on the device.
    void load_prefix_cache(ModelContext *mctx, const Tensor *past_kv) const;

  public:
    int num_attention_heads = 0;
    int num_key_value_heads = 0;
    bool interleaved_qkv = false;
    RopeType rope_type = RopeType::DISABLED;
    float rope_theta = 10000.f;
    AttentionMaskType attn_mask_type = AttentionMaskType::CAUSAL;
    int num_virtual_tokens = 0;
    Tensor *k_cache = nullptr;   // [#kvh, s, d]
    Tensor *v_cache = nullptr;   // [#kvh, d, s]

  private:
    int slot_ = -1;
    int head_size_ = 0;
    int n_ctx_ = 0;
};

}  // namespace chatglm
