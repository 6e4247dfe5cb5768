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
//   - chatglm::Linear                                       same constructor arguments, members and forward
//                                                           (chatglm.h:362-377), f16 weights
//   - chatglm::BasicAttention                               same constructor arguments, public members and forward
//                                                           (chatglm.h:440-472); attend() is the part between its
//                                                           two Linears for callers that keep them
//   - CHATGLM_CHECK / CHATGLM_THROW                         std::runtime_error("file:line message") (chatglm.h:16-29)
// Everything below executes through the C ABI of cglm_attn.h; there is no CPU path.
#pragma once

#include <cstdint>
#include <cstring>
#include <map>
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

    // parameter tensors (the reference's ctx_w): device memory, zero-filled, alive as long as the context
    Tensor *new_weight_1d(TensorType type, int64_t ne0);
    Tensor *new_weight_2d(TensorType type, int64_t ne0, int64_t ne1);

    // per-step device tensors (the reference's ctx_b scratch context), carved out of a pool; reset_scratch() takes them
    // all back (after synchronising the stream) and keeps the pool
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
    friend class DecodeStep;
    friend class Linear;
    // creates the (still unallocated) cache tensors of one attention module and returns its arena slot
    int register_attention(const cglm_attn_desc &desc, Tensor **k_cache, Tensor **v_cache);
    void ensure_workspace(int n_seq, int max_qlen);
    void ensure_status_workspace();   // at least the status word, for kernels that need nothing else

    void *stream_;
    cglm_kv_arena *arena_ = nullptr;
    cglm_attn_desc desc_{};
    bool have_desc_ = false;
    std::vector<std::unique_ptr<Tensor>> kv_tensors_;
    struct ScratchChunk {
        void *base;
        size_t size, used;
    };
    void *scratch_alloc(size_t bytes);
    std::vector<std::unique_ptr<Tensor>> scratch_;
    std::vector<ScratchChunk> pool_;
    std::vector<std::unique_ptr<Tensor>> weights_;
    void *workspace_ = nullptr;
    size_t workspace_bytes_ = 0;
};

// ---- graph inputs (chatglm.cpp:1123-1154, 1315-1327) ---------------------------------------------------------
// position ids of ChatGLM2/3/4: n_past .. n_past+qlen-1
std::vector<int> make_position_ids_glm2(int qlen, int n_past);
// position ids of ChatGLM-6B v1: [min(p, n_ctx-2)] ++ [max(p-(n_ctx-2), 0)], p = n_past+i
std::vector<int> make_position_ids_glm(int qlen, int n_past, int n_ctx);

// ---- Linear (chatglm.h:362-377, chatglm.cpp:418-426) --------------------------------------------------------------
// weight f16 [out_features, in_features] (ne = {in, out}) and bias f32 [out_features], both on the device and zero
// until loaded (mctx->tensor_set).  forward is a tcgen05 GEMM with f32 accumulation (cglm_linear_forward);
// in_features must be a multiple of 64 and out_features of 32.
class Linear {
  public:
    Linear() = default;
    Linear(ModelContext *mctx, int in_features, int out_features, bool use_bias = true);

    int in_features() const { return weight ? static_cast<int>(weight->ne[0]) : 0; }
    int out_features() const { return weight ? static_cast<int>(weight->ne[1]) : 0; }

    // input f32 or f16 [seqlen, in_features] on the device (an f32 input is rounded to f16 first, as ggml does in
    // front of an f16 matrix); returns [seqlen, out_features] from mctx's scratch, f32 like the reference's, or f16
    // when the consumer takes half precision.  Enqueued on mctx's stream.
    Tensor *forward(ModelContext *mctx, Tensor *input, TensorType out_type = TYPE_F32) const;

  public:
    Tensor *weight = nullptr;   // [out_features, in_features]
    Tensor *bias = nullptr;     // [out_features]
};

// ---- the attention module (chatglm.h:440-472) ---------------------------------------------------------------
class ModelFile;   // further down: the model container's reader

class BasicAttention {
  public:
    BasicAttention() = default;
    // Same arguments as the reference.  The caches exist once mctx->alloc_kv() ran; the two Linears' parameters are
    // allocated (zero) right away.
    BasicAttention(ModelContext *mctx, int hidden_size, int num_attention_heads, int num_key_value_heads,
                   int max_length, bool use_qkv_bias, bool use_dense_bias, bool interleaved_qkv, RopeType rope_type,
                   float rope_theta, AttentionMaskType attn_mask_type, int num_virtual_tokens);

    // The reference's call (chatglm.h:457-458, chatglm.cpp:625-722): query_key_value, RoPE, cache append, attention,
    // dense.
    //   hidden_states  f32 or f16 [qlen, hidden] on the device
    //   attention_mask, position_ids, n_past as for attend()
    // Returns attn_output f32 [qlen, hidden] from mctx's scratch.  One decode token of a GLM-2/3/4 shaped module
    // (head size 128, blocked qkv, no explicit position ids) takes three launches: the query_key_value GEMM with bias,
    // RoPE and append in its epilogue, the decode kernel, the dense GEMM; the activations between them are roped q
    // (f32) and the f16 context.  Everything else runs query_key_value as a plain GEMM with an f16 result, the
    // attention kernels on f16 input and output, and dense.  Intermediate tensors come from mctx's scratch pool
    // (call reset_scratch() between steps, as the reference drops its graph context); the launches are issued one by
    // one, so a token loop is better served by a DecodeStep (with_linears), which replays them as one graph.
    Tensor *forward(ModelContext *mctx, Tensor *hidden_states, Tensor *attention_mask, Tensor *position_ids,
                    int n_past) const;

    // Everything forward does between query_key_value.forward (chatglm.cpp:629) and dense.forward (chatglm.cpp:719),
    // for callers that keep the two Linears.
    //   qkv            f32 or f16 [qlen, (#h + 2 * #kvh) * d]: ne = {(#h + 2#kvh) * d, qlen}
    //   attention_mask accepted for signature parity; the v1 mask it would carry (chatglm.cpp:1126-1140) is applied
    //                  from attn_mask_type, so the tensor may be null
    //   position_ids   i32 [qlen] (or [2 * qlen] for RopeType::CHATGLM) on the device; null derives them from
    //                  n_past (and n_ctx, see set_n_ctx)
    // Returns context_layer [qlen, hidden] (f32, or f16 on request) allocated from mctx's scratch.  Enqueued on mctx's
    // stream.
    Tensor *attend(ModelContext *mctx, Tensor *qkv, Tensor *attention_mask, Tensor *position_ids, int n_past,
                   TensorType out_type = TYPE_F32) const;

    // prompt length of the running generation; only RopeType::CHATGLM with null position_ids reads it
    void set_n_ctx(int n_ctx) { n_ctx_ = n_ctx; }

    // Parameters of the two Linears from a model file, as load_state_dict does (chatglm.cpp:1250-1313): f16 weights,
    // f32 biases; a bias the file does not hold (GLM-2/3/4 have no dense bias) is left as it is.  Synchronous.
    void load_weights(ModelContext *mctx, const ModelFile &file, int layer) const;

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
    Linear query_key_value;
    Linear dense;
    Tensor *k_cache = nullptr;   // [#kvh, s, d]
    Tensor *v_cache = nullptr;   // [#kvh, d, s]

  private:
    friend class DecodeStep;
    int slot_ = -1;
    int head_size_ = 0;
    int n_ctx_ = 0;
};

// ---- the step loop (chatglm.cpp:726-755 forward_graph_compute, :886-925 generate) ------------------------------------
// The reference rebuilds its ggml graph for every generated token.  A DecodeStep records the attention calls of ONE
// decode step of a model (one call per layer, one sequence) in a CUDA graph whose kernels read the position from a
// device word (CGLM_SEQ_N_PAST_DEVICE); run() replays that graph and advances the word, so nothing is rebuilt, uploaded
// or re-validated per token.  The input and output tensors of every layer have fixed addresses: the caller's other
// kernels (the two Linears, norms, MLP) write qkv(l) and read context(l).  A caller that wants its own kernels inside
// the same graph records the layers itself with record(l) / record_advance() on a capturing stream instead of run().
class DecodeStep {
  public:
    // layers: the model's attention modules in order (all built against mctx, fused-decode shapes: head_dim 128, at
    // most 16 q heads per kv head, cache capacity a multiple of 8); mctx->alloc_kv() must have run.
    // with_linears: the step also runs every layer's two Linears (three launches per layer: query_key_value GEMM with an
    // f16 result, the decode kernel, dense GEMM), i.e. the whole of BasicAttention::forward per layer in the replayed
    // graph; the caller writes hidden(l) and reads attn_output(l).  The layers' Linear parameters must be loaded, with
    // in-features a multiple of 64 and out-features of 32.
    DecodeStep(ModelContext *mctx, const std::vector<const BasicAttention *> &layers, bool with_linears = false);
    ~DecodeStep();
    DecodeStep(const DecodeStep &) = delete;
    DecodeStep &operator=(const DecodeStep &) = delete;

    Tensor *qkv(int layer) const { return qkv_.at(layer).get(); }           // f32 [1, (#h + 2 #kvh) * d], device (f16 with_linears)
    Tensor *context(int layer) const { return context_.at(layer).get(); }   // f32 [1, #h * d], device (f16 with_linears)
    // with_linears only: the layer's input (f16 [1, hidden], e.g. what the caller's input norm writes) and its result
    // (f32 [1, hidden], chatglm.cpp:719-721)
    Tensor *hidden(int layer) const { return hidden_.at(layer).get(); }
    Tensor *attn_output(int layer) const { return attn_output_.at(layer).get(); }
    // position of the next token; also the value ChatGLM-6B v1 derives its 2-D ids from together with n_ctx
    void set_n_past(int n_past);
    int n_past() const { return n_past_; }
    // enqueue one layer's call / the position advance on `stream` (nullptr: the step's own stream)
    void record(int layer, void *stream = nullptr);
    void record_advance(void *stream = nullptr);
    // all layers, then n_past += 1.  The first call runs eagerly, the second captures the graph, and from then on
    // every call is one graph launch; ordered after what the context's stream holds, and the context's stream is
    // ordered after it
    void run();
    int graph_launches() const { return replays_; }
    // device-side status of the step's kernels since the last query (synchronises the step's stream)
    int status() { return cglm_attn_workspace_status(workspace_, stream_); }

  private:
    ModelContext *mctx_;
    std::vector<const BasicAttention *> layers_;
    bool with_linears_ = false;
    std::vector<std::unique_ptr<Tensor>> qkv_, context_, hidden_, attn_output_;
    std::vector<cglm_attn_seq> seqs_;
    int *n_past_dev_ = nullptr;
    int n_past_ = 0;
    void *workspace_ = nullptr;
    size_t workspace_bytes_ = 0;
    void *stream_ = nullptr;      // cudaStream_t: the step's own (capturable) stream
    void *graph_exec_ = nullptr;  // cudaGraphExec_t
    void *ev_in_ = nullptr, *ev_out_ = nullptr;
    int steps_ = 0, replays_ = 0;
};

// ---- model file (chatglm.h:40-86, 107-203; chatglm.cpp:295-391, 1754-1848) ---------------------------------------
// The container the reference's converter writes: header, config record, tokenizer blob, tensors.  Host code only.
enum class ModelType { CHATGLM = 1, CHATGLM2 = 2, CHATGLM3 = 3, CHATGLM4 = 4 };
enum class ActivationType { GELU, SILU };

// The three config records as they sit in the file (all members 4 bytes wide; dtype is a ggml_type value).
struct ConfigRecordV1 {
    int dtype, vocab_size, hidden_size, num_attention_heads, num_hidden_layers, intermediate_size;
    int max_length;                                        // sequence generation
    int bos_token_id, eos_token_id, pad_token_id, sep_token_id;   // tokenizer
};
struct ConfigRecordV1GQA : public ConfigRecordV1 {
    int num_key_value_heads;
};
struct ConfigRecordV2 {
    int dtype, vocab_size, hidden_size, num_attention_heads, num_key_value_heads, num_hidden_layers, intermediate_size;
    float norm_eps;
    int num_virtual_tokens;
    float rope_theta;
    int max_length, eos_token_id, pad_token_id;
};
static_assert(sizeof(ConfigRecordV1) == 44 && sizeof(ConfigRecordV1GQA) == 48 && sizeof(ConfigRecordV2) == 52,
              "config records are packed 4-byte fields");

class ModelConfig {
  public:
    ModelConfig() = default;
    ModelConfig(ModelType model_type, int dtype, int vocab_size, int hidden_size, int num_attention_heads,
                int num_key_value_heads, int num_hidden_layers, int intermediate_size, float norm_eps, float rope_theta,
                int num_virtual_tokens, int max_length, int bos_token_id, int eos_token_id, int pad_token_id,
                int sep_token_id);
    ModelConfig(ModelType model_type, const ConfigRecordV1 &rec, float norm_eps, float rope_theta, int num_virtual_tokens);
    ModelConfig(ModelType model_type, const ConfigRecordV1GQA &rec, float norm_eps, float rope_theta, int num_virtual_tokens);
    ModelConfig(ModelType model_type, const ConfigRecordV2 &rec);

    // what every BasicAttention of this model is constructed with (chatglm.h:443-455)
    cglm_attn_desc attn_desc() const;

    ModelType model_type = ModelType::CHATGLM2;
    int dtype = 0;
    int vocab_size = 0, hidden_size = 0, num_attention_heads = 0, num_key_value_heads = 0, num_hidden_layers = 0;
    int intermediate_size = 0;
    float norm_eps = 0.f;
    ActivationType hidden_act = ActivationType::SILU;
    bool use_qkv_bias = false, use_dense_bias = false, interleaved_qkv = false, tie_word_embeddings = false;
    RopeType rope_type = RopeType::CHATGLM2;
    float rope_theta = 10000.f;
    AttentionMaskType attn_mask_type = AttentionMaskType::CAUSAL;
    int num_virtual_tokens = 0;
    int max_length = 0;
    int bos_token_id = -1, eos_token_id = -1, pad_token_id = -1, sep_token_id = -1;
};

// read-only mapping of a file
class MappedFile {
  public:
    explicit MappedFile(const std::string &path);
    ~MappedFile();
    MappedFile(const MappedFile &) = delete;
    MappedFile &operator=(const MappedFile &) = delete;

    char *data = nullptr;
    size_t size = 0;
};

// a tensor of the state dict: a view into the mapped file
struct HostTensor {
    int ndim = 0;
    int64_t ne[4] = {1, 1, 1, 1};   // ne[0] innermost
    int dtype = 0;                  // ggml_type
    const void *data = nullptr;
    size_t nbytes = 0;
    size_t offset = 0;              // of data from the start of the file (a multiple of 16)
};

struct StateDict {
    std::vector<std::string> names;           // file order
    std::map<std::string, HostTensor> kv;
};

// elements and bytes per block of a ggml type the converter emits; false for any other type
bool ggml_type_block(int dtype, int *block_elems, int *block_bytes);

// cursor over the mapped bytes; every read is checked against the end of the file
class ModelLoader {
  public:
    ModelLoader(const char *data, size_t size) : data(data), size(size), ptr(data) {}

    int64_t tell() const { return ptr - data; }
    void seek(int64_t offset, int whence);

    template <typename T>
    T read_basic() {
        need(sizeof(T));
        T obj;
        std::memcpy(&obj, ptr, sizeof(T));
        ptr += sizeof(T);
        return obj;
    }
    std::string read_string(size_t length);
    // name, ndim, shape, dtype, data at the next 16-byte boundary, until the end of the file
    StateDict read_state_dict();

    const char *const data;
    const size_t size;
    const char *ptr;

  private:
    void need(size_t n) const;
};

// What the Pipeline constructor learns from a file before it builds the model: config (max_length optionally
// lowered, never raised), the tokenizer blob, the state dict.
class ModelFile {
  public:
    explicit ModelFile(const std::string &path, int max_length = 0);
    ModelFile(const void *data, size_t size, int max_length = 0);   // caller-owned memory

    // "query_key_value.weight" (0), "query_key_value.bias" (1), "dense.weight" (2), "dense.bias" (3) of a layer
    std::string attn_weight_name(int layer, int which) const;

    ModelConfig config;
    int version = 0;
    const char *tokenizer_data = nullptr;
    size_t tokenizer_size = 0;
    StateDict state_dict;

  private:
    void parse(const char *data, size_t size, int max_length);
    std::unique_ptr<MappedFile> mapped_;
};

}  // namespace chatglm
