/*
 * cglm_model_file.h -- reader of the model container that li-plus/chatglm.cpp's converter writes
 * (chatglm_cpp/convert.py:133-209, 225-360) and its Pipeline constructor reads (chatglm.cpp:1754-1848,
 * ModelLoader chatglm.cpp:337-391, config records chatglm.h:49-86).
 *
 * Layout of a file, little endian, no padding except before tensor data:
 *   "ggml" | i32 model_type (1 ChatGLM, 2 ChatGLM2, 3 ChatGLM3, 4 ChatGLM4) | i32 version (1 or 2)
 *   config record: version 1 = ConfigRecordV1 (ChatGLM) or ConfigRecordV1GQA (ChatGLM2/3); version 2 = ConfigRecordV2
 *   i32 size | tokenizer blob (sentencepiece model proto, or the tiktoken vocabulary text for ChatGLM4)
 *   tensors until the end of the file, each:
 *     i32 name length | name | i32 ndim | i32 shape[ndim] (outermost first) | i32 ggml_type |
 *     zero padding to the next multiple of 16 | data
 * The reader is host code only: it maps the file, validates every length against the file size and hands out
 * views into the mapping.  It exists so that real checkpoints can drive the attention path: it yields the
 * cglm_attn_desc of the model, the qkv / dense weights either side of the path, and the P-Tuning v2 prefix
 * ("past_key_values", f16 [2 * layers][kv_heads][virtual_tokens][head_dim], chatglm_cpp/convert.py:212-222).
 * Every function returns CGLM_OK or a negative CGLM_ERR_* (cglm_attn.h); nothing throws or aborts.
 */
#ifndef CGLM_MODEL_FILE_H
#define CGLM_MODEL_FILE_H

#include <stddef.h>

#include "cglm_attn.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ggml_type values the converter emits (chatglm_cpp/convert.py:37-44) */
enum {
    CGLM_TYPE_F32 = 0, CGLM_TYPE_F16 = 1, CGLM_TYPE_Q4_0 = 2, CGLM_TYPE_Q4_1 = 3, CGLM_TYPE_Q5_0 = 6,
    CGLM_TYPE_Q5_1 = 7, CGLM_TYPE_Q8_0 = 8
};

/* ModelConfig (chatglm.h:107-203): the stored record plus what its constructor derives from the model type
 * (chatglm.h:121-137). */
typedef struct cglm_model_config {
    int model_type;          /* ModelType, chatglm.h:40-45 */
    int version;             /* config record version in the file */
    int dtype;               /* ggml_type of the 2-D weights */
    int vocab_size, hidden_size, num_attention_heads, num_key_value_heads, num_hidden_layers, intermediate_size;
    float norm_eps;
    int num_virtual_tokens;
    float rope_theta;
    int max_length;
    int bos_token_id, eos_token_id, pad_token_id, sep_token_id;   /* -1 where the record has none */
    /* derived */
    int hidden_act;          /* 0 GELU (ChatGLM), 1 SILU */
    int use_qkv_bias, use_dense_bias, interleaved_qkv, tie_word_embeddings;
    int rope_type;           /* CGLM_ROPE_CHATGLM or CGLM_ROPE_CHATGLM2 */
    int attn_mask_type;      /* CGLM_MASK_CHATGLM or CGLM_MASK_CAUSAL */
} cglm_model_config;

typedef struct cglm_tensor_info {
    const char *name;        /* NUL-terminated copy owned by the file object */
    int ndim;                /* 1..4 */
    long long ne[4];         /* ggml order: ne[0] is the innermost extent (the file stores the outermost first) */
    int dtype;               /* ggml_type */
    const void *data;        /* view into the mapping, 16-byte aligned relative to the start of the file */
    size_t nbytes;
    size_t offset;           /* of data from the start of the file */
} cglm_tensor_info;

typedef struct cglm_model_file cglm_model_file;

/* Maps the file read-only and parses it (MappedFile + Pipeline's header walk + ModelLoader::read_state_dict).
 * CGLM_ERR_INVALID_ARG: unreadable path, bad magic, unknown model type or version, a length that leaves the file. */
int cglm_model_file_open(const char *path, cglm_model_file **out);
/* The same over caller-owned memory, which must outlive the object. */
int cglm_model_file_open_memory(const void *data, size_t size, cglm_model_file **out);
int cglm_model_file_close(cglm_model_file *f);

int cglm_model_file_config(const cglm_model_file *f, cglm_model_config *out);
/* The tokenizer blob (not interpreted here). */
int cglm_model_file_tokenizer(const cglm_model_file *f, const void **data, size_t *size);
int cglm_model_file_n_tensors(const cglm_model_file *f);
int cglm_model_file_tensor(const cglm_model_file *f, int index, cglm_tensor_info *out);   /* in file order */
int cglm_model_file_find(const cglm_model_file *f, const char *name, cglm_tensor_info *out);
/* The model's attention descriptor.  max_length <= 0 keeps the file's; a larger value than the file's is refused
 * like Pipeline refuses it (chatglm.cpp:1755-1762).  desc->max_len = max_length + num_virtual_tokens. */
int cglm_model_file_attn_desc(const cglm_model_file *f, int max_length, cglm_attn_desc *out);
/* Names of a layer's attention weights as the converter wrote them for this model type
 * (chatglm_cpp/convert.py:268-283, 343-355): which = 0 query_key_value.weight, 1 query_key_value.bias,
 * 2 dense.weight, 3 dense.bias (ChatGLM only).  Writes at most cap bytes including the NUL. */
int cglm_model_file_attn_weight_name(const cglm_model_file *f, int layer, int which, char *buf, size_t cap);
/* P-Tuning v2 prefix of one layer into one arena slot (BasicModel::load_prefix_cache, chatglm.h:580-615): copies the
 * layer's f16 [2][kv_heads][virtual_tokens][head_dim] block from the mapping to staging_dev (device memory of at
 * least that many bytes, 16-byte aligned) and scatters it into cache positions [0, virtual_tokens) with
 * cglm_kv_load_prefix.  Asynchronous on cuda_stream; allocates nothing.  CGLM_ERR_INVALID_ARG when the file has no
 * "past_key_values" tensor or its shape does not match the arena. */
int cglm_model_file_load_prefix(const cglm_model_file *f, cglm_kv_arena *arena, int layer, int slot, void *staging_dev,
                                void *cuda_stream);

/* One parameter of a layer's attention module into device memory, as load_state_dict does for the module's Linears
 * (chatglm.cpp:1250-1313): which as for cglm_model_file_attn_weight_name.  Weights must be stored as f16 [out][in]
 * (what cglm_linear_forward and cglm_qkv_linear_forward take), biases as f32; any other type is
 * CGLM_ERR_UNSUPPORTED.  dst_bytes must be the tensor's size; a tensor the file does not hold (a bias the model family
 * does not have) or a shape that contradicts the configuration record is CGLM_ERR_INVALID_ARG.  The copy is enqueued on
 * cuda_stream from the mapping: keep the file open until it has completed. */
int cglm_model_file_load_attn_weight(const cglm_model_file *f, int layer, int which, void *dst_dev, size_t dst_bytes,
                                     void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* CGLM_MODEL_FILE_H */
