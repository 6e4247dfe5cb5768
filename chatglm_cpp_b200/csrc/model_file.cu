// Reader of the model container written by li-plus/chatglm.cpp's converter: the C ABI of include/cglm_model_file.h and
// the chatglm:: classes of include/chatglm_b200.h that mirror MappedFile, ModelLoader, ModelConfig and the header walk
// of the Pipeline constructor (chatglm.cpp:295-391, 1754-1848; chatglm.h:49-203).  Host code; the only device work is
// the upload of a P-Tuning prefix block in cglm_model_file_load_prefix.
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <map>
#include <memory>
#include <new>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/chatglm_b200.h"
#include "../../include/cglm_model_file.h"

namespace cglm {
void set_last_error(const char *text);   // cglm_attn_api.cu: what cglm_last_error_string returns on this thread
}

namespace chatglm {

// ---- ggml block formats the converter emits (chatglm_cpp/convert.py:54-130): elements and bytes per block ----------
bool ggml_type_block(int dtype, int *block_elems, int *block_bytes) {
    switch (dtype) {
    case CGLM_TYPE_F32: *block_elems = 1; *block_bytes = 4; return true;
    case CGLM_TYPE_F16: *block_elems = 1; *block_bytes = 2; return true;
    case CGLM_TYPE_Q4_0: *block_elems = 32; *block_bytes = 2 + 16; return true;           // f16 scale, 32 nibbles
    case CGLM_TYPE_Q4_1: *block_elems = 32; *block_bytes = 2 + 2 + 16; return true;       // f16 scale, f16 min, nibbles
    case CGLM_TYPE_Q5_0: *block_elems = 32; *block_bytes = 2 + 4 + 16; return true;       // f16 scale, 32 high bits, nibbles
    case CGLM_TYPE_Q5_1: *block_elems = 32; *block_bytes = 2 + 2 + 4 + 16; return true;
    case CGLM_TYPE_Q8_0: *block_elems = 32; *block_bytes = 2 + 32; return true;           // f16 scale, 32 int8
    default: return false;
    }
}

// ---- MappedFile (chatglm.cpp:295-327) --------------------------------------------------------------------------
MappedFile::MappedFile(const std::string &path) {
    const int fd = open(path.c_str(), O_RDONLY);
    CHATGLM_CHECK(fd >= 0) << "cannot open file " << path << ": " << std::strerror(errno);
    struct stat sb;
    if (fstat(fd, &sb) != 0) {
        const int err = errno;
        close(fd);
        CHATGLM_THROW << "cannot stat file " << path << ": " << std::strerror(err);
    }
    size = static_cast<size_t>(sb.st_size);
    void *p = size ? mmap(nullptr, size, PROT_READ, MAP_SHARED, fd, 0) : MAP_FAILED;
    const int err = errno;
    close(fd);
    CHATGLM_CHECK(p != MAP_FAILED) << "cannot mmap file " << path << ": " << (size ? std::strerror(err) : "empty file");
    data = static_cast<char *>(p);
}

MappedFile::~MappedFile() {
    if (data) munmap(data, size);
}

// ---- ModelLoader (chatglm.cpp:337-391) -----------------------------------------------------------------------------
void ModelLoader::seek(int64_t offset, int whence) {
    int64_t target;
    if (whence == SEEK_SET) target = offset;
    else if (whence == SEEK_CUR) target = tell() + offset;
    else if (whence == SEEK_END) target = static_cast<int64_t>(size) + offset;
    else CHATGLM_THROW << "invalid seek mode " << whence;
    CHATGLM_CHECK(target >= 0 && target <= static_cast<int64_t>(size)) << "seek to " << target << " leaves the file (" << size << " bytes)";
    ptr = data + target;
}

void ModelLoader::need(size_t n) const {
    CHATGLM_CHECK(n <= size - static_cast<size_t>(ptr - data)) << "model file is truncated: " << n << " bytes wanted at offset " << tell();
}

std::string ModelLoader::read_string(size_t length) {
    need(length);
    std::string s(ptr, ptr + length);
    ptr += length;
    return s;
}

StateDict ModelLoader::read_state_dict() {
    StateDict sd;
    // the state dict occupies the rest of the file
    while (tell() < static_cast<int64_t>(size)) {
        const int name_size = read_basic<int>();
        CHATGLM_CHECK(name_size > 0 && name_size <= 4096) << "invalid tensor name length " << name_size;
        const std::string name = read_string(static_cast<size_t>(name_size));
        const int ndim = read_basic<int>();
        CHATGLM_CHECK(0 < ndim && ndim <= 4) << "tensor " << name << ": invalid ndim " << ndim;
        HostTensor t;
        t.ndim = ndim;
        for (int i = ndim - 1; i >= 0; i--) {   // stored outermost first, ne[0] is the innermost extent
            t.ne[i] = read_basic<int>();
            CHATGLM_CHECK(t.ne[i] > 0) << "tensor " << name << ": invalid extent " << t.ne[i];
        }
        t.dtype = read_basic<int>();
        int be = 0, bb = 0;
        CHATGLM_CHECK(ggml_type_block(t.dtype, &be, &bb)) << "tensor " << name << ": unsupported ggml type " << t.dtype;
        CHATGLM_CHECK(t.ne[0] % be == 0) << "tensor " << name << ": row of " << t.ne[0] << " elements is not a multiple of the block size";
        // bytes, with every product checked against the file size so that nothing overflows
        unsigned long long rows = 1;
        for (int i = 1; i < 4; i++) {
            rows *= static_cast<unsigned long long>(t.ne[i]);
            CHATGLM_CHECK(rows <= size) << "tensor " << name << ": shape exceeds the file";
        }
        const unsigned long long row_bytes = static_cast<unsigned long long>(t.ne[0] / be) * bb;
        CHATGLM_CHECK(row_bytes <= size && rows * row_bytes <= size) << "tensor " << name << ": shape exceeds the file";
        t.nbytes = static_cast<size_t>(rows * row_bytes);
        constexpr int64_t MEM_ALIGNED = 16;
        const int64_t data_offset = (tell() + (MEM_ALIGNED - 1)) & ~(MEM_ALIGNED - 1);
        CHATGLM_CHECK(static_cast<unsigned long long>(data_offset) + t.nbytes <= size) << "tensor " << name << ": data leaves the file";
        t.offset = static_cast<size_t>(data_offset);
        t.data = data + data_offset;
        seek(data_offset + static_cast<int64_t>(t.nbytes), SEEK_SET);
        sd.names.push_back(name);
        sd.kv[name] = t;
    }
    return sd;
}

// ---- ModelConfig (chatglm.h:107-203) -----------------------------------------------------------------------------
ModelConfig::ModelConfig(ModelType model_type, int dtype, int vocab_size, int hidden_size, int num_attention_heads,
                         int num_key_value_heads, int num_hidden_layers, int intermediate_size, float norm_eps,
                         float rope_theta, int num_virtual_tokens, int max_length, int bos_token_id, int eos_token_id,
                         int pad_token_id, int sep_token_id)
    : model_type(model_type), dtype(dtype), vocab_size(vocab_size), hidden_size(hidden_size),
      num_attention_heads(num_attention_heads), num_key_value_heads(num_key_value_heads),
      num_hidden_layers(num_hidden_layers), intermediate_size(intermediate_size), norm_eps(norm_eps),
      rope_theta(rope_theta), num_virtual_tokens(num_virtual_tokens), max_length(max_length), bos_token_id(bos_token_id),
      eos_token_id(eos_token_id), pad_token_id(pad_token_id), sep_token_id(sep_token_id) {
    const bool v1 = model_type == ModelType::CHATGLM;   // chatglm.h:121-137: two families
    hidden_act = v1 ? ActivationType::GELU : ActivationType::SILU;
    use_qkv_bias = true;
    use_dense_bias = v1;
    interleaved_qkv = v1;
    tie_word_embeddings = v1;
    rope_type = v1 ? RopeType::CHATGLM : RopeType::CHATGLM2;
    attn_mask_type = v1 ? AttentionMaskType::CHATGLM : AttentionMaskType::CAUSAL;
}

ModelConfig::ModelConfig(ModelType model_type, const ConfigRecordV1 &rec, float norm_eps, float rope_theta, int num_virtual_tokens)
    : ModelConfig(model_type, rec.dtype, rec.vocab_size, rec.hidden_size, rec.num_attention_heads, rec.num_attention_heads,
                  rec.num_hidden_layers, rec.intermediate_size, norm_eps, rope_theta, num_virtual_tokens, rec.max_length,
                  rec.bos_token_id, rec.eos_token_id, rec.pad_token_id, rec.sep_token_id) {}

ModelConfig::ModelConfig(ModelType model_type, const ConfigRecordV1GQA &rec, float norm_eps, float rope_theta, int num_virtual_tokens)
    : ModelConfig(model_type, rec.dtype, rec.vocab_size, rec.hidden_size, rec.num_attention_heads, rec.num_key_value_heads,
                  rec.num_hidden_layers, rec.intermediate_size, norm_eps, rope_theta, num_virtual_tokens, rec.max_length,
                  rec.bos_token_id, rec.eos_token_id, rec.pad_token_id, rec.sep_token_id) {}

ModelConfig::ModelConfig(ModelType model_type, const ConfigRecordV2 &rec)
    : ModelConfig(model_type, rec.dtype, rec.vocab_size, rec.hidden_size, rec.num_attention_heads, rec.num_key_value_heads,
                  rec.num_hidden_layers, rec.intermediate_size, rec.norm_eps, rec.rope_theta, rec.num_virtual_tokens,
                  rec.max_length, -1, rec.eos_token_id, rec.pad_token_id, -1) {}

cglm_attn_desc ModelConfig::attn_desc() const {
    cglm_attn_desc d;
    d.n_head = num_attention_heads;
    d.n_kv_head = num_key_value_heads;
    d.head_dim = num_attention_heads > 0 ? hidden_size / num_attention_heads : 0;
    d.max_len = max_length + num_virtual_tokens;
    d.n_virtual = num_virtual_tokens;
    d.rope_type = static_cast<int>(rope_type);
    d.rope_theta = rope_theta;
    d.mask_type = attn_mask_type == AttentionMaskType::CAUSAL ? CGLM_MASK_CAUSAL : CGLM_MASK_CHATGLM;
    return d;
}

// ---- the header walk of the Pipeline constructor (chatglm.cpp:1754-1848) ---------------------------------------------
ModelFile::ModelFile(const std::string &path, int max_length) : mapped_(std::make_unique<MappedFile>(path)) {
    parse(mapped_->data, mapped_->size, max_length);
}

ModelFile::ModelFile(const void *data, size_t size, int max_length) {
    parse(static_cast<const char *>(data), size, max_length);
}

void ModelFile::parse(const char *data, size_t size, int max_length) {
    ModelLoader loader(data, size);
    const std::string magic = loader.read_string(4);
    CHATGLM_CHECK(magic == "ggml") << "model file is broken (bad magic)";
    const ModelType model_type = static_cast<ModelType>(loader.read_basic<int>());
    version = loader.read_basic<int>();
    switch (model_type) {
    case ModelType::CHATGLM:
        if (version == 1) config = ModelConfig(model_type, loader.read_basic<ConfigRecordV1>(), 1e-5f, 10000.f, 0);
        else if (version == 2) config = ModelConfig(model_type, loader.read_basic<ConfigRecordV2>());
        else CHATGLM_THROW << "only support version 1 or 2 for now but got " << version;
        break;
    case ModelType::CHATGLM2:
    case ModelType::CHATGLM3:
        if (version == 1) config = ModelConfig(model_type, loader.read_basic<ConfigRecordV1GQA>(), 1e-5f, 10000.f, 0);
        else if (version == 2) config = ModelConfig(model_type, loader.read_basic<ConfigRecordV2>());
        else CHATGLM_THROW << "only support version 1 or 2 for now but got " << version;
        break;
    case ModelType::CHATGLM4:
        CHATGLM_CHECK(version == 2) << "only support version 2 for now but got " << version;
        config = ModelConfig(model_type, loader.read_basic<ConfigRecordV2>());
        break;
    default: CHATGLM_THROW << "invalid model type " << static_cast<int>(model_type);
    }
    CHATGLM_CHECK(config.num_attention_heads > 0 && config.num_key_value_heads > 0 && config.hidden_size > 0 &&
                  config.hidden_size % config.num_attention_heads == 0 &&
                  config.num_attention_heads % config.num_key_value_heads == 0 && config.num_hidden_layers > 0 &&
                  config.max_length > 0 && config.num_virtual_tokens >= 0)
        << "model file is broken (invalid config record)";
    if (max_length > 0) {
        CHATGLM_CHECK(max_length <= config.max_length)
            << "Requested max_length (" << max_length << ") exceeds the max possible model sequence length ("
            << config.max_length << ")";
        config.max_length = max_length;
    }
    // tokenizer blob: sentencepiece model proto, or the tiktoken vocabulary text of ChatGLM4; skipped by its size
    const int blob_size = loader.read_basic<int>();
    CHATGLM_CHECK(blob_size >= 0) << "invalid tokenizer size " << blob_size;
    tokenizer_data = data + loader.tell();
    tokenizer_size = static_cast<size_t>(blob_size);
    loader.seek(blob_size, SEEK_CUR);
    state_dict = loader.read_state_dict();
}

std::string ModelFile::attn_weight_name(int layer, int which) const {
    static const char *const kWhich[4] = {"query_key_value.weight", "query_key_value.bias", "dense.weight", "dense.bias"};
    CHATGLM_CHECK(which >= 0 && which < 4 && layer >= 0 && layer < config.num_hidden_layers) << "no such attention weight";
    CHATGLM_CHECK(which != 3 || config.use_dense_bias) << "this model family has no dense bias";
    // chatglm_cpp/convert.py:268-283 (ChatGLM) and :343-355 (ChatGLM2/3/4)
    const std::string prefix = config.model_type == ModelType::CHATGLM
                                   ? "transformer.layers." + std::to_string(layer) + ".attention."
                                   : "transformer.encoder.layers." + std::to_string(layer) + ".self_attention.";
    return prefix + kWhich[which];
}

}  // namespace chatglm

// ---- C ABI ------------------------------------------------------------------------------------------------------------
struct cglm_model_file {
    std::unique_ptr<chatglm::ModelFile> mf;
};

namespace {

template <class Fn>
int guarded(Fn &&fn) {
    try {
        return fn();
    } catch (const std::exception &e) {
        cglm::set_last_error(e.what());
        return CGLM_ERR_INVALID_ARG;
    }
}

void fill_info(const std::string &name, const chatglm::HostTensor &t, cglm_tensor_info *out) {
    out->name = name.c_str();
    out->ndim = t.ndim;
    for (int i = 0; i < 4; i++) out->ne[i] = t.ne[i];
    out->dtype = t.dtype;
    out->data = t.data;
    out->nbytes = t.nbytes;
    out->offset = t.offset;
}

}  // namespace

extern "C" {

int cglm_model_file_open(const char *path, cglm_model_file **out) {
    if (!path || !out) return CGLM_ERR_INVALID_ARG;
    return guarded([&] {
        std::unique_ptr<cglm_model_file> f(new cglm_model_file());
        f->mf = std::make_unique<chatglm::ModelFile>(std::string(path), 0);
        *out = f.release();
        return static_cast<int>(CGLM_OK);
    });
}

int cglm_model_file_open_memory(const void *data, size_t size, cglm_model_file **out) {
    if (!data || !out) return CGLM_ERR_INVALID_ARG;
    return guarded([&] {
        std::unique_ptr<cglm_model_file> f(new cglm_model_file());
        f->mf = std::make_unique<chatglm::ModelFile>(data, size, 0);
        *out = f.release();
        return static_cast<int>(CGLM_OK);
    });
}

int cglm_model_file_close(cglm_model_file *f) {
    if (!f) return CGLM_ERR_INVALID_ARG;
    delete f;
    return CGLM_OK;
}

int cglm_model_file_config(const cglm_model_file *f, cglm_model_config *out) {
    if (!f || !out) return CGLM_ERR_INVALID_ARG;
    const chatglm::ModelConfig &c = f->mf->config;
    out->model_type = static_cast<int>(c.model_type);
    out->version = f->mf->version;
    out->dtype = c.dtype;
    out->vocab_size = c.vocab_size; out->hidden_size = c.hidden_size;
    out->num_attention_heads = c.num_attention_heads; out->num_key_value_heads = c.num_key_value_heads;
    out->num_hidden_layers = c.num_hidden_layers; out->intermediate_size = c.intermediate_size;
    out->norm_eps = c.norm_eps; out->num_virtual_tokens = c.num_virtual_tokens; out->rope_theta = c.rope_theta;
    out->max_length = c.max_length;
    out->bos_token_id = c.bos_token_id; out->eos_token_id = c.eos_token_id;
    out->pad_token_id = c.pad_token_id; out->sep_token_id = c.sep_token_id;
    out->hidden_act = static_cast<int>(c.hidden_act);
    out->use_qkv_bias = c.use_qkv_bias; out->use_dense_bias = c.use_dense_bias;
    out->interleaved_qkv = c.interleaved_qkv; out->tie_word_embeddings = c.tie_word_embeddings;
    out->rope_type = static_cast<int>(c.rope_type);
    out->attn_mask_type = c.attn_mask_type == chatglm::AttentionMaskType::CAUSAL ? CGLM_MASK_CAUSAL : CGLM_MASK_CHATGLM;
    return CGLM_OK;
}

int cglm_model_file_tokenizer(const cglm_model_file *f, const void **data, size_t *size) {
    if (!f || !data || !size) return CGLM_ERR_INVALID_ARG;
    *data = f->mf->tokenizer_data;
    *size = f->mf->tokenizer_size;
    return CGLM_OK;
}

int cglm_model_file_n_tensors(const cglm_model_file *f) { return f ? static_cast<int>(f->mf->state_dict.names.size()) : 0; }

int cglm_model_file_tensor(const cglm_model_file *f, int index, cglm_tensor_info *out) {
    if (!f || !out || index < 0 || index >= static_cast<int>(f->mf->state_dict.names.size())) return CGLM_ERR_INVALID_ARG;
    const std::string &name = f->mf->state_dict.names[index];
    fill_info(name, f->mf->state_dict.kv.at(name), out);
    return CGLM_OK;
}

int cglm_model_file_find(const cglm_model_file *f, const char *name, cglm_tensor_info *out) {
    if (!f || !name || !out) return CGLM_ERR_INVALID_ARG;
    auto it = f->mf->state_dict.kv.find(name);
    if (it == f->mf->state_dict.kv.end()) return CGLM_ERR_INVALID_ARG;
    fill_info(it->first, it->second, out);
    return CGLM_OK;
}

int cglm_model_file_attn_desc(const cglm_model_file *f, int max_length, cglm_attn_desc *out) {
    if (!f || !out) return CGLM_ERR_INVALID_ARG;
    chatglm::ModelConfig c = f->mf->config;
    if (max_length > 0) {
        if (max_length > c.max_length) {
            cglm::set_last_error("requested max_length exceeds the model's sequence length");
            return CGLM_ERR_INVALID_ARG;
        }
        c.max_length = max_length;
    }
    *out = c.attn_desc();
    return CGLM_OK;
}

int cglm_model_file_attn_weight_name(const cglm_model_file *f, int layer, int which, char *buf, size_t cap) {
    if (!f || !buf || cap == 0) return CGLM_ERR_INVALID_ARG;
    return guarded([&] {
        const std::string s = f->mf->attn_weight_name(layer, which);
        if (s.size() + 1 > cap) return static_cast<int>(CGLM_ERR_INVALID_ARG);
        std::memcpy(buf, s.c_str(), s.size() + 1);
        return static_cast<int>(CGLM_OK);
    });
}

int cglm_model_file_load_prefix(const cglm_model_file *f, cglm_kv_arena *arena, int layer, int slot, void *staging_dev,
                                void *cuda_stream) {
    if (!f || !arena || !staging_dev) return CGLM_ERR_INVALID_ARG;
    const cglm_attn_desc *d = cglm_kv_arena_desc(arena);
    auto it = f->mf->state_dict.kv.find("past_key_values");
    if (!d || it == f->mf->state_dict.kv.end()) return CGLM_ERR_INVALID_ARG;
    const chatglm::HostTensor &t = it->second;
    const chatglm::ModelConfig &c = f->mf->config;
    // [l * 2, #kvh, v, d] f16 (chatglm.h:581), i.e. ne = {d, v, #kvh, 2l}
    if (t.dtype != CGLM_TYPE_F16 || t.ndim != 4 || t.ne[0] != d->head_dim || t.ne[1] != d->n_virtual || t.ne[2] != d->n_kv_head ||
        t.ne[3] != 2LL * c.num_hidden_layers || layer < 0 || layer >= c.num_hidden_layers || d->n_virtual <= 0) {
        cglm::set_last_error("past_key_values does not match the arena (head_dim, virtual tokens, kv heads) or the layer is out of range");
        return CGLM_ERR_INVALID_ARG;
    }
    const size_t block = static_cast<size_t>(2) * d->n_kv_head * d->n_virtual * d->head_dim * 2;
    const char *src = static_cast<const char *>(t.data) + block * static_cast<size_t>(layer);
    cudaError_t e = cudaMemcpyAsync(staging_dev, src, block, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(cuda_stream));
    if (e != cudaSuccess) {
        cglm::set_last_error(cudaGetErrorString(e));
        return CGLM_ERR_CUDA;
    }
    return cglm_kv_load_prefix(arena, slot, staging_dev, cuda_stream);
}

int cglm_model_file_load_attn_weight(const cglm_model_file *f, int layer, int which, void *dst_dev, size_t dst_bytes,
                                     void *cuda_stream) {
    if (!f || !dst_dev || which < 0 || which > 3) return CGLM_ERR_INVALID_ARG;
    return guarded([&] {
        const chatglm::ModelConfig &c = f->mf->config;
        if (layer < 0 || layer >= c.num_hidden_layers) return static_cast<int>(CGLM_ERR_INVALID_ARG);
        auto it = f->mf->state_dict.kv.find(f->mf->attn_weight_name(layer, which));
        if (it == f->mf->state_dict.kv.end()) {
            cglm::set_last_error("the model file has no such tensor for this layer");
            return static_cast<int>(CGLM_ERR_INVALID_ARG);
        }
        const chatglm::HostTensor &t = it->second;
        const int64_t hidden = c.hidden_size, head = c.hidden_size / c.num_attention_heads;
        const int64_t qkv = hidden + 2 * head * c.num_key_value_heads;
        const bool is_weight = which == 0 || which == 2;
        const int64_t rows = which < 2 ? qkv : hidden;
        // weights: [out, in] = ne {in, out} in the file's matrix type; biases: f32 [out]
        const bool shape_ok = is_weight ? (t.ndim == 2 && t.ne[0] == hidden && t.ne[1] == rows) : (t.ndim == 1 && t.ne[0] == rows);
        if (!shape_ok) {
            cglm::set_last_error("tensor shape does not match the configuration record");
            return static_cast<int>(CGLM_ERR_INVALID_ARG);
        }
        if (t.dtype != (is_weight ? CGLM_TYPE_F16 : CGLM_TYPE_F32)) {
            cglm::set_last_error("the Linear kernels take f16 weights and f32 biases: convert the checkpoint with type f16");
            return static_cast<int>(CGLM_ERR_UNSUPPORTED);
        }
        if (dst_bytes != t.nbytes) return static_cast<int>(CGLM_ERR_INVALID_ARG);
        cudaError_t e = cudaMemcpyAsync(dst_dev, t.data, t.nbytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(cuda_stream));
        if (e != cudaSuccess) {
            cglm::set_last_error(cudaGetErrorString(e));
            return static_cast<int>(CGLM_ERR_CUDA);
        }
        return static_cast<int>(CGLM_OK);
    });
}

}  // extern "C"
