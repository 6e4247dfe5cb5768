// Host side of the B200 attention KV-cache path: the chatglm:: module surface of include/chatglm_b200.h over the
// C ABI of include/cglm_attn.h.  Host code only; compiled by nvcc for the CUDA runtime declarations.
#include "../../include/chatglm_b200.h"

#include <algorithm>
#include <cuda_runtime.h>

namespace chatglm {

#define CHATGLM_CHECK_CUDA(call)                                                                   \
    do {                                                                                           \
        cudaError_t error__ = (call);                                                              \
        CHATGLM_CHECK(error__ == cudaSuccess) << "CUDA error: " << cudaGetErrorString(error__);    \
    } while (false)

size_t element_size(TensorType type) {
    switch (type) {
    case TYPE_F32: return 4;
    case TYPE_F16: return 2;
    case TYPE_I32: return 4;
    }
    CHATGLM_THROW << "unknown tensor type " << static_cast<int>(type);
    return 0;   // not reached
}

size_t nbytes(const Tensor *t) { return static_cast<size_t>(t->ne[0] * t->ne[1] * t->ne[2] * t->ne[3]) * element_size(t->type); }

static void set_contiguous(Tensor *t, TensorType type, int64_t ne0, int64_t ne1, int64_t ne2) {
    t->type = type;
    t->ne[0] = ne0; t->ne[1] = ne1; t->ne[2] = ne2; t->ne[3] = 1;
    t->nb[0] = element_size(type);
    t->nb[1] = t->nb[0] * ne0;
    t->nb[2] = t->nb[1] * ne1;
    t->nb[3] = t->nb[2] * ne2;
}

ModelContext::ModelContext(void *cuda_stream) : stream_(cuda_stream) {}

ModelContext::~ModelContext() {
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));
    reset_scratch();
    for (auto &c : pool_) cudaFree(c.base);
    for (auto &t : weights_) {
        if (t->owned && t->data) cudaFree(t->data);
    }
    if (workspace_) cudaFree(workspace_);
    if (arena_) cglm_kv_arena_destroy(arena_);
}

int ModelContext::register_attention(const cglm_attn_desc &desc, Tensor **k_cache, Tensor **v_cache) {
    CHATGLM_CHECK(!arena_) << "kv buffer already allocated: construct every BasicAttention before alloc_kv()";
    if (have_desc_) {
        CHATGLM_CHECK(desc.n_head == desc_.n_head && desc.n_kv_head == desc_.n_kv_head && desc.head_dim == desc_.head_dim &&
                      desc.max_len == desc_.max_len && desc.n_virtual == desc_.n_virtual &&
                      desc.rope_type == desc_.rope_type && desc.rope_theta == desc_.rope_theta &&
                      desc.mask_type == desc_.mask_type)
            << "all attention modules of one context share one configuration";
    } else {
        desc_ = desc;
        have_desc_ = true;
    }
    const int slot = static_cast<int>(kv_tensors_.size() / 2);
    auto k = std::make_unique<Tensor>(), v = std::make_unique<Tensor>();
    // chatglm.h:452-455: k_cache ne = [d, max_length + v, #kvh], v_cache ne = [max_length + v, d, #kvh], both F16
    set_contiguous(k.get(), TYPE_F16, desc.head_dim, desc.max_len, desc.n_kv_head);
    set_contiguous(v.get(), TYPE_F16, desc.max_len, desc.head_dim, desc.n_kv_head);
    *k_cache = k.get();
    *v_cache = v.get();
    kv_tensors_.push_back(std::move(k));
    kv_tensors_.push_back(std::move(v));
    return slot;
}

void ModelContext::alloc_kv() {
    CHATGLM_CHECK(!arena_) << "kv buffer already allocated";
    CHATGLM_CHECK(have_desc_ && !kv_tensors_.empty()) << "no attention module registered";
    const int n_slots = static_cast<int>(kv_tensors_.size() / 2);
    CHATGLM_CHECK_CGLM(cglm_kv_arena_create(&desc_, n_slots, &arena_));
    // the library lays a cache row out with a pitch that may exceed max_length + v (rounded up to 8 tokens at
    // head_dim 128): the tensors keep the reference's extents and carry the pitch in their byte strides
    const int64_t pitch = cglm_kv_arena_pitch(arena_);
    for (int s = 0; s < n_slots; ++s) {
        Tensor *k = kv_tensors_[2 * s].get(), *v = kv_tensors_[2 * s + 1].get();
        k->data = cglm_kv_arena_k_cache(arena_, s);
        v->data = cglm_kv_arena_v_cache(arena_, s);
        k->nb[2] = k->nb[1] * pitch;
        k->nb[3] = k->nb[2] * k->ne[2];
        v->nb[1] = v->nb[0] * pitch;
        v->nb[2] = v->nb[1] * v->ne[1];
        v->nb[3] = v->nb[2] * v->ne[2];
    }
}

void ModelContext::ensure_workspace(int n_seq, int max_qlen) {
    const size_t need = cglm_attn_workspace_bytes(&desc_, n_seq, max_qlen);
    CHATGLM_CHECK(need > 0) << "invalid attention configuration";
    if (need > workspace_bytes_) {
        if (workspace_) {
            CHATGLM_CHECK_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)));
            CHATGLM_CHECK_CUDA(cudaFree(workspace_));
            workspace_ = nullptr;
        }
        CHATGLM_CHECK_CUDA(cudaMalloc(&workspace_, need));
        workspace_bytes_ = need;
        CHATGLM_CHECK_CGLM(cglm_attn_workspace_init(workspace_, workspace_bytes_, stream_));
    }
}

void ModelContext::ensure_status_workspace() {
    if (workspace_) return;
    const size_t bytes = cglm_linear_workspace_bytes();
    CHATGLM_CHECK_CUDA(cudaMalloc(&workspace_, bytes));
    workspace_bytes_ = bytes;
    CHATGLM_CHECK_CGLM(cglm_attn_workspace_init(workspace_, workspace_bytes_, stream_));
}

Tensor *ModelContext::new_weight_2d(TensorType type, int64_t ne0, int64_t ne1) {
    auto t = std::make_unique<Tensor>();
    set_contiguous(t.get(), type, ne0, ne1, 1);
    const size_t bytes = std::max<size_t>(nbytes(t.get()), 16);
    CHATGLM_CHECK_CUDA(cudaMalloc(&t->data, bytes));
    CHATGLM_CHECK_CUDA(cudaMemsetAsync(t->data, 0, bytes, static_cast<cudaStream_t>(stream_)));
    t->owned = true;
    weights_.push_back(std::move(t));
    return weights_.back().get();
}

Tensor *ModelContext::new_weight_1d(TensorType type, int64_t ne0) { return new_weight_2d(type, ne0, 1); }

// Per-step tensors come out of a pool that is carved front to back and rewound by reset_scratch (the reference's ctx_b
// is the same kind of arena): no device allocation per tensor once the pool has grown to a step's needs.
void *ModelContext::scratch_alloc(size_t bytes) {
    const size_t need = (std::max<size_t>(bytes, 16) + 255) / 256 * 256;
    if (pool_.empty() || pool_.back().used + need > pool_.back().size) {
        ScratchChunk c;
        c.size = std::max<size_t>(need, static_cast<size_t>(32) << 20);
        c.used = 0;
        c.base = nullptr;
        CHATGLM_CHECK_CUDA(cudaMalloc(&c.base, c.size));
        pool_.push_back(c);   // earlier chunks stay where they are: tensors already handed out keep their addresses
    }
    ScratchChunk &c = pool_.back();
    void *p = static_cast<char *>(c.base) + c.used;
    c.used += need;
    return p;
}

Tensor *ModelContext::new_tensor_2d(TensorType type, int64_t ne0, int64_t ne1) {
    auto t = std::make_unique<Tensor>();
    set_contiguous(t.get(), type, ne0, ne1, 1);
    t->data = scratch_alloc(nbytes(t.get()));
    t->owned = false;   // the pool's
    scratch_.push_back(std::move(t));
    return scratch_.back().get();
}

Tensor *ModelContext::new_tensor_1d(TensorType type, int64_t ne0) { return new_tensor_2d(type, ne0, 1); }

void ModelContext::reset_scratch() {
    if (!scratch_.empty()) {
        cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));   // kernels that still read the tensors
    }
    scratch_.clear();
    if (pool_.size() > 1) {
        // the step needed more than one chunk: one chunk of the whole size from now on
        size_t total = 0;
        for (auto &c : pool_) {
            total += c.size;
            cudaFree(c.base);
        }
        pool_.clear();
        ScratchChunk c;
        c.size = total;
        c.used = 0;
        c.base = nullptr;
        if (cudaMalloc(&c.base, c.size) == cudaSuccess) pool_.push_back(c);   // on failure the next tensor allocates afresh
        else cudaGetLastError();
    }
    for (auto &c : pool_) c.used = 0;
}

// A cache tensor of an arena whose row pitch exceeds its extent is not contiguous: such a tensor is copied whole
// (offset 0, all of it) as a 2-D copy of its contiguous runs.  Returns false for a contiguous tensor.
static bool pitched_runs(const Tensor *t, size_t *width, size_t *height, size_t *pitch) {
    size_t run = element_size(t->type);
    for (int i = 0; i < 4; ++i) {
        if (static_cast<size_t>(t->nb[i]) != run) {
            *width = run;
            *pitch = static_cast<size_t>(t->nb[i]);
            *height = 1;
            for (int j = i; j < 4; ++j) *height *= static_cast<size_t>(t->ne[j]);
            return true;
        }
        run *= static_cast<size_t>(t->ne[i]);
    }
    return false;
}

void ModelContext::tensor_set(Tensor *t, const void *host, size_t offset, size_t size) {
    CHATGLM_CHECK(offset + size <= nbytes(t)) << "tensor_set out of range";
    size_t w, h, pitch;
    if (pitched_runs(t, &w, &h, &pitch)) {
        CHATGLM_CHECK(offset == 0 && size == nbytes(t)) << "a pitched tensor is copied whole";
        CHATGLM_CHECK_CUDA(cudaMemcpy2DAsync(t->data, pitch, host, w, w, h, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream_)));
        return;
    }
    CHATGLM_CHECK_CUDA(cudaMemcpyAsync(static_cast<char *>(t->data) + offset, host, size, cudaMemcpyHostToDevice,
                                       static_cast<cudaStream_t>(stream_)));
}

void ModelContext::tensor_get(const Tensor *t, void *host, size_t offset, size_t size) {
    CHATGLM_CHECK(offset + size <= nbytes(t)) << "tensor_get out of range";
    size_t w, h, pitch;
    if (pitched_runs(t, &w, &h, &pitch)) {
        CHATGLM_CHECK(offset == 0 && size == nbytes(t)) << "a pitched tensor is copied whole";
        CHATGLM_CHECK_CUDA(cudaMemcpy2DAsync(host, w, t->data, pitch, w, h, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream_)));
    } else {
        CHATGLM_CHECK_CUDA(cudaMemcpyAsync(host, static_cast<const char *>(t->data) + offset, size, cudaMemcpyDeviceToHost,
                                           static_cast<cudaStream_t>(stream_)));
    }
    CHATGLM_CHECK_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)));
}

void ModelContext::synchronize() {
    CHATGLM_CHECK_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)));
    if (workspace_) {
        CHATGLM_CHECK_CGLM(cglm_attn_workspace_status(workspace_, stream_));
    }
}

std::vector<int> make_position_ids_glm2(int qlen, int n_past) {
    std::vector<int> ids(qlen);
    for (int i = 0; i < qlen; i++) ids[i] = n_past + i;
    return ids;
}

std::vector<int> make_position_ids_glm(int qlen, int n_past, int n_ctx) {
    std::vector<int> ids(2 * qlen);
    for (int i = 0; i < qlen; i++) {
        const int p = n_past + i;
        ids[i] = std::min(p, n_ctx - 2);
        ids[qlen + i] = std::max(p - (n_ctx - 2), 0);
    }
    return ids;
}

// ---- Linear -------------------------------------------------------------------------------------------------------
Linear::Linear(ModelContext *mctx, int in_features, int out_features, bool use_bias) {
    CHATGLM_CHECK(mctx != nullptr) << "null context";
    CHATGLM_CHECK(in_features > 0 && out_features > 0) << "invalid Linear shape";
    weight = mctx->new_weight_2d(TYPE_F16, in_features, out_features);
    bias = use_bias ? mctx->new_weight_1d(TYPE_F32, out_features) : nullptr;
}

// f16 view of an activation: the tensor itself, or its rounded copy in mctx's scratch
static Tensor *as_f16(ModelContext *mctx, Tensor *t) {
    if (t->type == TYPE_F16) return t;
    CHATGLM_CHECK(t->type == TYPE_F32) << "activations are f32 or f16";
    CHATGLM_CHECK(t->nb[1] == t->nb[0] * static_cast<size_t>(t->ne[0])) << "activation rows must be contiguous";
    Tensor *h = mctx->new_tensor_2d(TYPE_F16, t->ne[0], t->ne[1]);
    CHATGLM_CHECK_CGLM(cglm_convert_f32_to_f16(static_cast<const float *>(t->data), h->data,
                                               static_cast<size_t>(t->ne[0] * t->ne[1]), mctx->stream()));
    return h;
}

Tensor *Linear::forward(ModelContext *mctx, Tensor *input, TensorType out_type) const {
    CHATGLM_CHECK(mctx != nullptr && weight != nullptr) << "Linear without parameters";
    CHATGLM_CHECK(input && input->data && input->ne[0] == weight->ne[0])
        << "input row is " << (input ? input->ne[0] : 0) << ", expected " << weight->ne[0];
    CHATGLM_CHECK(out_type == TYPE_F32 || out_type == TYPE_F16) << "output is f32 or f16";
    CHATGLM_CHECK(weight->type == TYPE_F16) << "weights are f16";
    Tensor *x = as_f16(mctx, input);
    CHATGLM_CHECK(x->nb[1] == 2 * static_cast<size_t>(x->ne[0])) << "activation rows must be contiguous";
    const int n_tok = static_cast<int>(x->ne[1]);
    Tensor *output = mctx->new_tensor_2d(out_type, weight->ne[1], n_tok);   // [seqlen, out_features]
    mctx->ensure_status_workspace();
    CHATGLM_CHECK_CGLM(cglm_linear_forward(x->data, n_tok, in_features(), weight->data, out_features(),
                                           bias ? static_cast<const float *>(bias->data) : nullptr, output->data,
                                           out_type == TYPE_F16, mctx->workspace_, mctx->workspace_bytes_, mctx->stream_));
    return output;
}

// ---- BasicAttention -------------------------------------------------------------------------------------------------
BasicAttention::BasicAttention(ModelContext *mctx, int hidden_size, int num_attention_heads, int num_key_value_heads,
                               int max_length, bool use_qkv_bias, bool use_dense_bias, bool interleaved_qkv,
                               RopeType rope_type, float rope_theta, AttentionMaskType attn_mask_type,
                               int num_virtual_tokens)
    : num_attention_heads(num_attention_heads), num_key_value_heads(num_key_value_heads),
      interleaved_qkv(interleaved_qkv), rope_type(rope_type), rope_theta(rope_theta), attn_mask_type(attn_mask_type),
      num_virtual_tokens(num_virtual_tokens) {
    CHATGLM_CHECK(mctx != nullptr) << "null context";
    CHATGLM_CHECK(num_attention_heads > 0 && hidden_size % num_attention_heads == 0) << "invalid head count";
    head_size_ = hidden_size / num_attention_heads;
    query_key_value = Linear(mctx, hidden_size, hidden_size + 2 * head_size_ * num_key_value_heads, use_qkv_bias);
    dense = Linear(mctx, hidden_size, hidden_size, use_dense_bias);
    cglm_attn_desc desc;
    desc.n_head = num_attention_heads;
    desc.n_kv_head = num_key_value_heads;
    desc.head_dim = head_size_;
    desc.max_len = max_length + num_virtual_tokens;
    desc.n_virtual = num_virtual_tokens;
    desc.rope_type = static_cast<int>(rope_type);
    desc.rope_theta = rope_theta;
    desc.mask_type = attn_mask_type == AttentionMaskType::CAUSAL ? CGLM_MASK_CAUSAL : CGLM_MASK_CHATGLM;
    slot_ = mctx->register_attention(desc, &k_cache, &v_cache);
}

Tensor *BasicAttention::attend(ModelContext *mctx, Tensor *qkv, Tensor * /*attention_mask*/, Tensor *position_ids,
                               int n_past, TensorType out_type) const {
    CHATGLM_CHECK(mctx && mctx->kv_allocated()) << "kv buffer not allocated";
    CHATGLM_CHECK(qkv && (qkv->type == TYPE_F32 || qkv->type == TYPE_F16) && qkv->data) << "qkv must be an f32 or f16 device tensor";
    CHATGLM_CHECK(out_type == TYPE_F32 || out_type == TYPE_F16) << "context_layer is f32 or f16";
    const int64_t hidden_size = static_cast<int64_t>(num_attention_heads) * head_size_;
    const int64_t qkv_width = hidden_size + 2LL * head_size_ * num_key_value_heads;
    CHATGLM_CHECK(qkv->ne[0] == qkv_width) << "qkv row is " << qkv->ne[0] << ", expected " << qkv_width;
    const int qlen = static_cast<int>(qkv->ne[1]);
    const int num_shared_q_heads = num_attention_heads / num_key_value_heads;

    cglm_attn_seq seq{};
    // pointers are typed float in the descriptor; with CGLM_SEQ_QKV_F16 they address f16 values, strides in elements
    const size_t esz = element_size(qkv->type);
    const char *base = static_cast<const char *>(qkv->data);
    auto at = [&](long long elems) { return reinterpret_cast<const float *>(base + elems * static_cast<long long>(esz)); };
    const long long row = static_cast<long long>(qkv->nb[1] / esz);
    if (interleaved_qkv) {   // chatglm.cpp:636-644
        CHATGLM_CHECK(num_shared_q_heads == 1) << "interleaved qkv is not supported for GQA";
        seq.q = at(0); seq.k = at(head_size_); seq.v = at(2 * head_size_);
        seq.q_head_stride = seq.kv_head_stride = 3 * head_size_;
    } else {                 // chatglm.cpp:646-652
        seq.q = at(0); seq.k = at(hidden_size); seq.v = at(hidden_size + static_cast<long long>(head_size_) * num_key_value_heads);
        seq.q_head_stride = seq.kv_head_stride = head_size_;
    }
    seq.q_tok_stride = seq.kv_tok_stride = row;
    seq.slot = slot_;
    seq.qlen = qlen;
    seq.n_past = n_past;
    seq.n_ctx = n_ctx_;
    seq.flags = (qkv->type == TYPE_F16 ? CGLM_SEQ_QKV_F16 : 0) | (out_type == TYPE_F16 ? CGLM_SEQ_OUT_F16 : 0);
    if (position_ids) {
        const int64_t want = rope_type == RopeType::CHATGLM ? 2 * qlen : qlen;
        CHATGLM_CHECK(position_ids->type == TYPE_I32 && position_ids->ne[0] == want)
            << "invalid position ids size " << position_ids->ne[0];
        seq.position_ids = static_cast<const int *>(position_ids->data);
    }
    Tensor *context_layer = mctx->new_tensor_2d(out_type, hidden_size, qlen);   // [s, #h * d]
    seq.out = static_cast<float *>(context_layer->data);
    mctx->ensure_workspace(1, qlen);
    CHATGLM_CHECK_CGLM(cglm_attn_forward(mctx->arena_, &seq, 1, mctx->workspace_, mctx->workspace_bytes_, mctx->stream_));
    return context_layer;
}

Tensor *BasicAttention::forward(ModelContext *mctx, Tensor *hidden_states, Tensor *attention_mask, Tensor *position_ids,
                                int n_past) const {
    CHATGLM_CHECK(mctx && mctx->kv_allocated()) << "kv buffer not allocated";
    CHATGLM_CHECK(hidden_states && hidden_states->data) << "null hidden_states";
    const int64_t hidden_size = static_cast<int64_t>(num_attention_heads) * head_size_;
    CHATGLM_CHECK(hidden_states->ne[0] == hidden_size) << "hidden_states row is " << hidden_states->ne[0] << ", expected " << hidden_size;
    const int qlen = static_cast<int>(hidden_states->ne[1]);
    Tensor *context_layer = nullptr;
    // one decode token of a GLM-2/3/4 shaped module: bias, RoPE and the cache append ride in the GEMM's epilogue
    const bool fused = qlen == 1 && !position_ids && !interleaved_qkv && head_size_ == 128 && hidden_size % 64 == 0 &&
                       (rope_type == RopeType::CHATGLM2 || rope_type == RopeType::DISABLED) &&
                       query_key_value.weight && query_key_value.weight->type == TYPE_F16;
    if (fused) {
        Tensor *x = as_f16(mctx, hidden_states);
        Tensor *q_roped = mctx->new_tensor_2d(TYPE_F32, hidden_size, 1);
        cglm_attn_seq seq{};
        seq.slot = slot_;
        seq.qlen = 1;
        seq.n_past = n_past;
        mctx->ensure_workspace(1, 1);
        const int rc = cglm_qkv_linear_forward(
            mctx->arena_, &seq, 1, x->data, static_cast<int>(hidden_size), query_key_value.weight->data,
            query_key_value.bias ? static_cast<const float *>(query_key_value.bias->data) : nullptr,
            static_cast<float *>(q_roped->data), mctx->workspace_, mctx->workspace_bytes_, mctx->stream_);
        if (rc != CGLM_ERR_UNSUPPORTED) {   // an arena without the fused decode layout takes the general route below
            CHATGLM_CHECK_CGLM(rc);
            context_layer = mctx->new_tensor_2d(TYPE_F16, hidden_size, 1);
            seq.q = seq.k = seq.v = static_cast<const float *>(q_roped->data);   // k and v are not read
            seq.q_head_stride = seq.kv_head_stride = head_size_;
            seq.q_tok_stride = seq.kv_tok_stride = hidden_size;
            seq.kv_local = num_virtual_tokens + n_past + 1;
            seq.flags = CGLM_SEQ_Q_ROPED | CGLM_SEQ_NO_APPEND | CGLM_SEQ_USE_KV_LOCAL | CGLM_SEQ_OUT_F16;
            seq.out = static_cast<float *>(context_layer->data);
            CHATGLM_CHECK_CGLM(cglm_attn_forward(mctx->arena_, &seq, 1, mctx->workspace_, mctx->workspace_bytes_, mctx->stream_));
        }
    }
    if (!context_layer) {
        Tensor *qkv = query_key_value.forward(mctx, hidden_states, TYPE_F16);                     // chatglm.cpp:629
        context_layer = attend(mctx, qkv, attention_mask, position_ids, n_past, TYPE_F16);         // chatglm.cpp:631-717
    }
    return dense.forward(mctx, context_layer, TYPE_F32);                                          // chatglm.cpp:719
}

void BasicAttention::load_weights(ModelContext *mctx, const ModelFile &file, int layer) const {
    CHATGLM_CHECK(mctx != nullptr) << "null context";
    Tensor *dst[4] = {query_key_value.weight, query_key_value.bias, dense.weight, dense.bias};
    for (int which = 0; which < 4; which++) {
        if (!dst[which]) continue;
        auto it = file.state_dict.kv.find(file.attn_weight_name(layer, which));
        if (it == file.state_dict.kv.end()) {
            CHATGLM_CHECK(which == 1 || which == 3) << "the model file has no " << file.attn_weight_name(layer, which);
            continue;
        }
        const HostTensor &t = it->second;
        const bool is_weight = which == 0 || which == 2;
        CHATGLM_CHECK(t.dtype == (is_weight ? static_cast<int>(TYPE_F16) : static_cast<int>(TYPE_F32)))
            << file.attn_weight_name(layer, which) << ": the Linear kernels take f16 weights and f32 biases";
        CHATGLM_CHECK(t.nbytes == nbytes(dst[which]) && t.ne[0] == dst[which]->ne[0] && t.ne[1] == dst[which]->ne[1])
            << file.attn_weight_name(layer, which) << ": shape does not match the module";
        mctx->tensor_set(dst[which], t.data, 0, t.nbytes);
    }
    mctx->synchronize();   // the copies read the file's mapping
}

void BasicAttention::load_prefix_cache(ModelContext *mctx, const Tensor *past_kv) const {
    CHATGLM_CHECK(mctx && mctx->kv_allocated()) << "kv buffer not allocated";
    CHATGLM_CHECK(past_kv && past_kv->type == TYPE_F16 && past_kv->data) << "prefix must be an f16 device tensor";
    CHATGLM_CHECK_CGLM(cglm_kv_load_prefix(mctx->arena_, slot_, past_kv->data, mctx->stream_));
}

// ---- DecodeStep ----------------------------------------------------------------------------------------------------
DecodeStep::DecodeStep(ModelContext *mctx, const std::vector<const BasicAttention *> &layers, bool with_linears)
    : mctx_(mctx), layers_(layers), with_linears_(with_linears) {
    CHATGLM_CHECK(mctx && mctx->kv_allocated()) << "kv buffer not allocated";
    CHATGLM_CHECK(!layers.empty()) << "no layers";
    cudaStream_t st;
    CHATGLM_CHECK_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    stream_ = st;
    // a workspace of its own: the captured graph holds its address, the context's may move when a longer prompt comes
    workspace_bytes_ = cglm_attn_workspace_bytes(&mctx->desc_, 1, 1);
    CHATGLM_CHECK(workspace_bytes_ > 0) << "invalid attention configuration";
    CHATGLM_CHECK_CUDA(cudaMalloc(&workspace_, workspace_bytes_));
    CHATGLM_CHECK_CGLM(cglm_attn_workspace_init(workspace_, workspace_bytes_, stream_));
    cudaEvent_t e0, e1;
    CHATGLM_CHECK_CUDA(cudaEventCreateWithFlags(&e0, cudaEventDisableTiming));
    CHATGLM_CHECK_CUDA(cudaEventCreateWithFlags(&e1, cudaEventDisableTiming));
    ev_in_ = e0;
    ev_out_ = e1;
    CHATGLM_CHECK_CUDA(cudaMalloc(reinterpret_cast<void **>(&n_past_dev_), sizeof(int)));
    CHATGLM_CHECK_CUDA(cudaMemset(n_past_dev_, 0, sizeof(int)));
    const cglm_attn_desc &d = mctx->desc_;
    const int64_t hidden = static_cast<int64_t>(d.n_head) * d.head_dim;
    const int64_t width = hidden + 2LL * d.head_dim * d.n_kv_head;
    for (const BasicAttention *attn : layers_) {
        CHATGLM_CHECK(attn && attn->slot_ >= 0) << "layer was not built against a context";
        // between the Linears the activations are f16 when the step runs the Linears itself, f32 when the caller does
        const TensorType act = with_linears_ ? TYPE_F16 : TYPE_F32;
        auto in = std::make_unique<Tensor>(), out = std::make_unique<Tensor>();
        set_contiguous(in.get(), act, width, 1, 1);
        set_contiguous(out.get(), act, hidden, 1, 1);
        CHATGLM_CHECK_CUDA(cudaMalloc(&in->data, std::max<size_t>(nbytes(in.get()), 16)));
        CHATGLM_CHECK_CUDA(cudaMalloc(&out->data, std::max<size_t>(nbytes(out.get()), 16)));
        in->owned = out->owned = true;
        if (with_linears_) {
            CHATGLM_CHECK(attn->query_key_value.weight && attn->dense.weight) << "layer has no Linear parameters";
            auto x = std::make_unique<Tensor>(), y = std::make_unique<Tensor>();
            set_contiguous(x.get(), TYPE_F16, hidden, 1, 1);
            set_contiguous(y.get(), TYPE_F32, hidden, 1, 1);
            CHATGLM_CHECK_CUDA(cudaMalloc(&x->data, std::max<size_t>(nbytes(x.get()), 16)));
            CHATGLM_CHECK_CUDA(cudaMalloc(&y->data, std::max<size_t>(nbytes(y.get()), 16)));
            CHATGLM_CHECK_CUDA(cudaMemset(x->data, 0, nbytes(x.get())));
            x->owned = y->owned = true;
            hidden_.push_back(std::move(x));
            attn_output_.push_back(std::move(y));
        }
        cglm_attn_seq seq{};
        // typed float in the descriptor; with CGLM_SEQ_QKV_F16 the same pointers address f16 values, strides in elements
        const size_t esz = element_size(act);
        const char *bytes = static_cast<const char *>(in->data);
        auto at = [&](long long elems) { return reinterpret_cast<const float *>(bytes + elems * static_cast<long long>(esz)); };
        if (attn->interleaved_qkv) {   // chatglm.cpp:636-644
            seq.q = at(0); seq.k = at(d.head_dim); seq.v = at(2 * d.head_dim);
            seq.q_head_stride = seq.kv_head_stride = 3 * d.head_dim;
        } else {                       // chatglm.cpp:646-652
            seq.q = at(0); seq.k = at(hidden); seq.v = at(hidden + static_cast<long long>(d.head_dim) * d.n_kv_head);
            seq.q_head_stride = seq.kv_head_stride = d.head_dim;
        }
        seq.q_tok_stride = seq.kv_tok_stride = width;
        seq.slot = attn->slot_;
        seq.qlen = 1;
        seq.n_past = d.max_len - d.n_virtual - 1;   // upper bound: sizes the launch, the kernel reads the device word
        seq.n_ctx = attn->n_ctx_;
        seq.out = static_cast<float *>(out->data);
        seq.flags = CGLM_SEQ_N_PAST_DEVICE | (with_linears_ ? (CGLM_SEQ_QKV_F16 | CGLM_SEQ_OUT_F16) : 0);
        seq.n_past_dev = n_past_dev_;
        seqs_.push_back(seq);
        qkv_.push_back(std::move(in));
        context_.push_back(std::move(out));
    }
}

DecodeStep::~DecodeStep() {
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));
    if (graph_exec_) cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph_exec_));
    for (auto &t : qkv_) cudaFree(t->data);
    for (auto &t : context_) cudaFree(t->data);
    for (auto &t : hidden_) cudaFree(t->data);
    for (auto &t : attn_output_) cudaFree(t->data);
    cudaFree(n_past_dev_);
    cudaFree(workspace_);
    cudaEventDestroy(static_cast<cudaEvent_t>(ev_in_));
    cudaEventDestroy(static_cast<cudaEvent_t>(ev_out_));
    cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
}

void DecodeStep::set_n_past(int n_past) {
    CHATGLM_CHECK(n_past >= 0 && n_past < mctx_->desc_.max_len - mctx_->desc_.n_virtual) << "n_past " << n_past << " beyond the cache";
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    CHATGLM_CHECK_CUDA(cudaStreamSynchronize(st));
    CHATGLM_CHECK_CUDA(cudaMemcpyAsync(n_past_dev_, &n_past, sizeof(int), cudaMemcpyHostToDevice, st));
    CHATGLM_CHECK_CUDA(cudaStreamSynchronize(st));
    n_past_ = n_past;
}

void DecodeStep::record(int layer, void *stream) {
    CHATGLM_CHECK(layer >= 0 && layer < static_cast<int>(seqs_.size())) << "no such layer";
    void *st = stream ? stream : stream_;
    if (!with_linears_) {
        CHATGLM_CHECK_CGLM(cglm_attn_forward(mctx_->arena_, &seqs_[layer], 1, workspace_, workspace_bytes_, st));
        return;
    }
    // query_key_value as a plain GEMM with an f16 result (chatglm.cpp:629); RoPE and the cache append happen in the decode
    // kernel, which reads the position from the device word; dense (chatglm.cpp:719) on the f16 context
    const BasicAttention *attn = layers_[layer];
    const Linear &qkv_lin = attn->query_key_value, &dense_lin = attn->dense;
    CHATGLM_CHECK_CGLM(cglm_linear_forward(hidden_[layer]->data, 1, qkv_lin.in_features(), qkv_lin.weight->data, qkv_lin.out_features(),
                                           qkv_lin.bias ? static_cast<const float *>(qkv_lin.bias->data) : nullptr, qkv_[layer]->data, 1,
                                           workspace_, workspace_bytes_, st));
    CHATGLM_CHECK_CGLM(cglm_attn_forward(mctx_->arena_, &seqs_[layer], 1, workspace_, workspace_bytes_, st));
    CHATGLM_CHECK_CGLM(cglm_linear_forward(context_[layer]->data, 1, dense_lin.in_features(), dense_lin.weight->data,
                                           dense_lin.out_features(), dense_lin.bias ? static_cast<const float *>(dense_lin.bias->data) : nullptr,
                                           attn_output_[layer]->data, 0, workspace_, workspace_bytes_, st));
}

void DecodeStep::record_advance(void *stream) {
    CHATGLM_CHECK_CGLM(cglm_seq_advance(n_past_dev_, 1, 1, stream ? stream : stream_));
}

void DecodeStep::run() {
    CHATGLM_CHECK(n_past_ + 1 <= mctx_->desc_.max_len - mctx_->desc_.n_virtual) << "the cache is full";
    cudaStream_t st = static_cast<cudaStream_t>(stream_), outer = static_cast<cudaStream_t>(mctx_->stream_);
    CHATGLM_CHECK_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev_in_), outer));
    CHATGLM_CHECK_CUDA(cudaStreamWaitEvent(st, static_cast<cudaEvent_t>(ev_in_), 0));
    if (steps_ == 0) {
        // the first step runs eagerly: whatever the library sets up on a first launch happens outside a capture
        for (int l = 0; l < static_cast<int>(seqs_.size()); l++) record(l);
        record_advance();
    } else if (!graph_exec_) {
        cudaGraph_t graph = nullptr;
        CHATGLM_CHECK_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        try {
            for (int l = 0; l < static_cast<int>(seqs_.size()); l++) record(l);
            record_advance();
        } catch (...) {
            cudaStreamEndCapture(st, &graph);
            if (graph) cudaGraphDestroy(graph);
            throw;
        }
        CHATGLM_CHECK_CUDA(cudaStreamEndCapture(st, &graph));
        cudaGraphExec_t exec = nullptr;
        cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        CHATGLM_CHECK(e == cudaSuccess) << "CUDA error: " << cudaGetErrorString(e);
        graph_exec_ = exec;
    }
    if (steps_ > 0) {
        CHATGLM_CHECK_CUDA(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph_exec_), st));
        replays_ += 1;
    }
    CHATGLM_CHECK_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(ev_out_), st));
    CHATGLM_CHECK_CUDA(cudaStreamWaitEvent(outer, static_cast<cudaEvent_t>(ev_out_), 0));
    n_past_ += 1;
    steps_ += 1;
}

}  // namespace chatglm
