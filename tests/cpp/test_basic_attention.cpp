// Drives chatglm::BasicAttention (include/chatglm_b200.h) the way the reference's model test drives its modules
// (chatglm_test.cpp:288-362: prefill of a few tokens, then two decode steps) and checks every step against the
// CPU oracle: output within max-abs 2e-3, caches bit-exact.  Prints one line per case and "ALL OK" at the end.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "../../include/chatglm_b200.h"
#include "../../oracle/attn_oracle.h"

using namespace chatglm;

static int g_failures = 0;
#define EXPECT(cond, ...)                         \
    do {                                          \
        if (!(cond)) {                            \
            std::printf("FAIL %s:%d ", __FILE__, __LINE__); \
            std::printf(__VA_ARGS__);             \
            std::printf("\n");                    \
            ++g_failures;                         \
        }                                         \
    } while (0)

struct Case {
    const char *name;
    int hidden, n_head, n_kv_head, max_length, n_virtual;
    bool interleaved;
    RopeType rope;
    AttentionMaskType mask;
    int prompt;
    bool explicit_ids;
};

static void run_case(const Case &c) {
    const int H = c.n_head, G = c.n_kv_head, D = c.hidden / c.n_head, M = c.max_length + c.n_virtual;
    ModelContext mctx(nullptr);
    // two layers, as stored by value in the reference's blocks (chatglm.h:506-513): copies must stay valid
    std::vector<BasicAttention> layers;
    for (int l = 0; l < 2; l++) {
        layers.emplace_back(&mctx, c.hidden, H, G, c.max_length, true, false, c.interleaved, c.rope, 10000.f, c.mask,
                            c.n_virtual);
    }
    mctx.alloc_kv();
    BasicAttention &attn = layers[1];
    attn.set_n_ctx(c.prompt);
    EXPECT(attn.k_cache->ne[0] == D && attn.k_cache->ne[1] == M && attn.k_cache->ne[2] == G, "k_cache shape");
    EXPECT(attn.v_cache->ne[0] == M && attn.v_cache->ne[1] == D && attn.v_cache->ne[2] == G, "v_cache shape");

    oracle_cfg cfg = {H, G, D, M, c.n_virtual, static_cast<int>(c.rope), 10000.f,
                      c.mask == AttentionMaskType::CAUSAL ? ORACLE_MASK_CAUSAL : ORACLE_MASK_CHATGLM, oracle_numerics_f32()};
    std::vector<uint16_t> kc(static_cast<size_t>(G) * M * D, 0), vc(kc.size(), 0);
    std::mt19937 rng(1234);
    std::normal_distribution<float> dist(0.f, 1.f);
    const int width = c.hidden + 2 * D * G;
    int n_past = 0;
    float worst = 0.f;
    for (int qlen : {c.prompt, 1, 1}) {
        std::vector<float> qkv(static_cast<size_t>(qlen) * width);
        for (auto &x : qkv) x = dist(rng);
        Tensor *qkv_t = mctx.new_tensor_2d(TYPE_F32, width, qlen);
        mctx.tensor_set(qkv_t, qkv.data(), 0, qkv.size() * sizeof(float));
        std::vector<int> ids = c.rope == RopeType::CHATGLM ? make_position_ids_glm(qlen, n_past, c.prompt)
                                                           : make_position_ids_glm2(qlen, n_past);
        Tensor *ids_t = nullptr;
        if (c.explicit_ids) {
            ids_t = mctx.new_tensor_1d(TYPE_I32, static_cast<int64_t>(ids.size()));
            mctx.tensor_set(ids_t, ids.data(), 0, ids.size() * sizeof(int));
        }
        Tensor *ctx = attn.attend(&mctx, qkv_t, nullptr, ids_t, n_past);
        EXPECT(ctx->ne[0] == c.hidden && ctx->ne[1] == qlen, "context_layer shape");
        std::vector<float> got(static_cast<size_t>(qlen) * c.hidden);
        mctx.tensor_get(ctx, got.data(), 0, got.size() * sizeof(float));
        mctx.synchronize();

        std::vector<float> want(got.size()), mask;
        const float *q = qkv.data(), *k, *v;
        long hs;
        if (c.interleaved) { k = q + D; v = q + 2 * D; hs = 3 * D; } else { k = q + c.hidden; v = q + c.hidden + G * D; hs = D; }
        if (n_past == 0 && c.mask == AttentionMaskType::CHATGLM) {
            mask.resize(static_cast<size_t>(qlen) * (c.n_virtual + qlen));
            oracle_attention_mask_glm(qlen, c.n_virtual + qlen, mask.data());
        }
        int rc = oracle_attn_forward(&cfg, q, width, hs, k, v, width, hs, kc.data(), vc.data(), ids.data(),
                                     mask.empty() ? nullptr : mask.data(), qlen, n_past, want.data(), nullptr, nullptr);
        EXPECT(rc == 0, "oracle rejected the arguments");
        for (size_t i = 0; i < got.size(); i++) {
            EXPECT(std::isfinite(got[i]), "non-finite output");
            worst = std::fmax(worst, std::fabs(got[i] - want[i]));
        }
        n_past += qlen;
        mctx.reset_scratch();
    }
    EXPECT(worst <= 2e-3f, "%s: max abs error %g", c.name, worst);
    std::vector<uint16_t> gk(kc.size()), gv(vc.size());
    mctx.tensor_get(attn.k_cache, gk.data(), 0, gk.size() * 2);
    mctx.tensor_get(attn.v_cache, gv.data(), 0, gv.size() * 2);
    EXPECT(std::memcmp(gk.data(), kc.data(), kc.size() * 2) == 0, "%s: k_cache differs from the oracle's", c.name);
    EXPECT(std::memcmp(gv.data(), vc.data(), vc.size() * 2) == 0, "%s: v_cache differs from the oracle's", c.name);
    // the other layer's cache was never touched
    std::vector<uint16_t> other(kc.size(), 1);
    mctx.tensor_get(layers[0].k_cache, other.data(), 0, other.size() * 2);
    bool zero = true;
    for (uint16_t x : other) zero = zero && x == 0;
    EXPECT(zero, "%s: layer 0's k_cache was written", c.name);
    std::printf("case %-28s max abs err %.3g\n", c.name, worst);
}

static void run_error_cases() {
    ModelContext mctx(nullptr);
    BasicAttention attn(&mctx, 4096, 32, 2, 256, true, false, false, RopeType::CHATGLM2, 10000.f, AttentionMaskType::CAUSAL, 0);
    Tensor bogus;
    bool threw = false;
    try {
        attn.attend(&mctx, &bogus, nullptr, nullptr, 0);   // kv buffer not allocated yet
    } catch (const std::runtime_error &e) {
        threw = std::strstr(e.what(), "chatglm_b200.cu") != nullptr;   // "file:line message", like CHATGLM_CHECK
    }
    EXPECT(threw, "attend before alloc_kv must throw std::runtime_error with file:line");
    mctx.alloc_kv();
    Tensor *bad = mctx.new_tensor_2d(TYPE_F32, 100, 1);   // wrong row width
    threw = false;
    try {
        attn.attend(&mctx, bad, nullptr, nullptr, 0);
    } catch (const std::runtime_error &) {
        threw = true;
    }
    EXPECT(threw, "a qkv row of the wrong width must throw");
    Tensor *qkv = mctx.new_tensor_2d(TYPE_F32, 4096 + 2 * 128 * 2, 1);
    threw = false;
    try {
        attn.attend(&mctx, qkv, nullptr, nullptr, 256);   // n_past + qlen beyond max_length
    } catch (const std::runtime_error &e) {
        threw = std::strstr(e.what(), "invalid argument") != nullptr;
    }
    EXPECT(threw, "n_past beyond the cache must throw with the C status text");
    std::printf("case %-28s ok\n", "error behaviour");
}

// chatglm::DecodeStep: four layers of one sequence, six tokens; the first step is eager, the second captures, the
// rest are graph launches.  Every token's context of every layer against the oracle, caches bit-exact at the end.
static void run_decode_step_case() {
    const int hidden = 4096, H = 32, G = 2, D = 128, max_length = 512, n_layer = 4, start = 131, n_token = 6;
    ModelContext mctx(nullptr);
    std::vector<BasicAttention> layers;
    for (int l = 0; l < n_layer; l++) {
        layers.emplace_back(&mctx, hidden, H, G, max_length, true, false, false, RopeType::CHATGLM2, 10000.f,
                            AttentionMaskType::CAUSAL, 0);
    }
    mctx.alloc_kv();
    oracle_cfg cfg = {H, G, D, max_length, 0, static_cast<int>(RopeType::CHATGLM2), 10000.f, ORACLE_MASK_CAUSAL, oracle_numerics_f32()};
    std::mt19937 rng(77);
    std::normal_distribution<float> dist(0.f, 1.f);
    const size_t cache_elems = static_cast<size_t>(G) * max_length * D;
    std::vector<std::vector<uint16_t>> kc(n_layer, std::vector<uint16_t>(cache_elems, 0)), vc(n_layer, std::vector<uint16_t>(cache_elems, 0));
    // a prompt of `start` tokens through the ordinary call fills the caches on both sides
    const int width = hidden + 2 * D * G;
    for (int l = 0; l < n_layer; l++) {
        std::vector<float> qkv(static_cast<size_t>(start) * width), want(static_cast<size_t>(start) * hidden);
        for (auto &x : qkv) x = dist(rng);
        Tensor *t = mctx.new_tensor_2d(TYPE_F32, width, start);
        mctx.tensor_set(t, qkv.data(), 0, qkv.size() * sizeof(float));
        layers[l].attend(&mctx, t, nullptr, nullptr, 0);
        std::vector<int> ids = make_position_ids_glm2(start, 0);
        oracle_attn_forward(&cfg, qkv.data(), width, D, qkv.data() + hidden, qkv.data() + hidden + G * D, width, D, kc[l].data(),
                            vc[l].data(), ids.data(), nullptr, start, 0, want.data(), nullptr, nullptr);
    }
    mctx.synchronize();
    mctx.reset_scratch();
    std::vector<const BasicAttention *> ptrs;
    for (auto &a : layers) ptrs.push_back(&a);
    DecodeStep step(&mctx, ptrs);
    step.set_n_past(start);
    float worst = 0.f;
    for (int tok = 0; tok < n_token; tok++) {
        std::vector<std::vector<float>> qkv(n_layer, std::vector<float>(width));
        for (int l = 0; l < n_layer; l++) {
            for (auto &x : qkv[l]) x = dist(rng);
            mctx.tensor_set(step.qkv(l), qkv[l].data(), 0, width * sizeof(float));
        }
        step.run();
        for (int l = 0; l < n_layer; l++) {
            std::vector<float> got(hidden), want(hidden);
            mctx.tensor_get(step.context(l), got.data(), 0, hidden * sizeof(float));
            int id = start + tok;
            oracle_attn_forward(&cfg, qkv[l].data(), width, D, qkv[l].data() + hidden, qkv[l].data() + hidden + G * D, width, D,
                                kc[l].data(), vc[l].data(), &id, nullptr, 1, start + tok, want.data(), nullptr, nullptr);
            for (int i = 0; i < hidden; i++) worst = std::fmax(worst, std::fabs(got[i] - want[i]));
        }
    }
    mctx.synchronize();
    EXPECT(worst <= 2e-3f, "decode step: max abs error %g", worst);
    EXPECT(step.n_past() == start + n_token, "decode step: position %d", step.n_past());
    EXPECT(step.graph_launches() == n_token - 1, "decode step: %d graph launches for %d tokens", step.graph_launches(), n_token);
    for (int l = 0; l < n_layer; l++) {
        std::vector<uint16_t> gk(cache_elems), gv(cache_elems);
        mctx.tensor_get(layers[l].k_cache, gk.data(), 0, gk.size() * 2);
        mctx.tensor_get(layers[l].v_cache, gv.data(), 0, gv.size() * 2);
        EXPECT(std::memcmp(gk.data(), kc[l].data(), cache_elems * 2) == 0, "decode step: k_cache of layer %d differs", l);
        EXPECT(std::memcmp(gv.data(), vc[l].data(), cache_elems * 2) == 0, "decode step: v_cache of layer %d differs", l);
    }
    bool threw = false;
    try {
        step.set_n_past(max_length);
    } catch (const std::runtime_error &) {
        threw = true;
    }
    EXPECT(threw, "a position beyond the cache must throw");
    std::printf("case %-28s max abs err %.3g, %d graph launches\n", "decode step graph", worst, step.graph_launches());
}

// BasicAttention::forward as the reference calls it (chatglm.h:457-458): hidden_states in, attn_output out, the two
// Linears inside.  Checked against the oracle's Linear -> attention -> Linear with the same f16 roundings between the
// stages (f16 activations into both GEMMs, f16 cache rows).  The GEMMs sum in another order than the oracle, so an
// appended cache value may be the neighbouring f16 value and the output carries that: max abs 6e-3 on outputs of unit
// scale.
struct FullCase {
    const char *name;
    int hidden, n_head, n_kv_head, max_length;
    bool interleaved, qkv_bias, dense_bias;
    RopeType rope;
    AttentionMaskType mask;
    int prompt;
};

static void run_full_forward_case(const FullCase &c) {
    const int H = c.n_head, G = c.n_kv_head, D = c.hidden / c.n_head, M = c.max_length;
    const int width = c.hidden + 2 * D * G;
    ModelContext mctx(nullptr);
    BasicAttention attn(&mctx, c.hidden, H, G, c.max_length, c.qkv_bias, c.dense_bias, c.interleaved, c.rope, 10000.f, c.mask, 0);
    mctx.alloc_kv();
    attn.set_n_ctx(c.prompt);
    EXPECT(attn.query_key_value.in_features() == c.hidden && attn.query_key_value.out_features() == width, "qkv Linear shape");
    EXPECT(attn.dense.in_features() == c.hidden && attn.dense.out_features() == c.hidden, "dense Linear shape");
    EXPECT((attn.query_key_value.bias != nullptr) == c.qkv_bias && (attn.dense.bias != nullptr) == c.dense_bias, "bias presence");

    std::mt19937 rng(4321);
    std::normal_distribution<float> dist(0.f, 1.f);
    const float w_scale = 1.f / std::sqrt(static_cast<float>(c.hidden));
    std::vector<uint16_t> w_qkv(static_cast<size_t>(width) * c.hidden), w_dense(static_cast<size_t>(c.hidden) * c.hidden);
    for (auto &w : w_qkv) w = oracle_f32_to_f16(dist(rng) * w_scale);
    for (auto &w : w_dense) w = oracle_f32_to_f16(dist(rng) * w_scale);
    std::vector<float> b_qkv(width), b_dense(c.hidden);
    for (auto &b : b_qkv) b = dist(rng);
    for (auto &b : b_dense) b = dist(rng);
    mctx.tensor_set(attn.query_key_value.weight, w_qkv.data(), 0, w_qkv.size() * 2);
    mctx.tensor_set(attn.dense.weight, w_dense.data(), 0, w_dense.size() * 2);
    if (c.qkv_bias) mctx.tensor_set(attn.query_key_value.bias, b_qkv.data(), 0, b_qkv.size() * 4);
    if (c.dense_bias) mctx.tensor_set(attn.dense.bias, b_dense.data(), 0, b_dense.size() * 4);

    oracle_cfg cfg = {H, G, D, M, 0, static_cast<int>(c.rope), 10000.f,
                      c.mask == AttentionMaskType::CAUSAL ? ORACLE_MASK_CAUSAL : ORACLE_MASK_CHATGLM, oracle_numerics_f32()};
    std::vector<uint16_t> kc(static_cast<size_t>(G) * M * D, 0), vc(kc.size(), 0);
    int n_past = 0;
    float worst = 0.f;
    auto round_f16 = [](std::vector<float> &v) { for (auto &x : v) x = oracle_f16_to_f32(oracle_f32_to_f16(x)); };
    for (int qlen : {c.prompt, 1, 1}) {
        std::vector<float> x(static_cast<size_t>(qlen) * c.hidden);
        for (auto &e : x) e = dist(rng);
        Tensor *x_t = mctx.new_tensor_2d(TYPE_F32, c.hidden, qlen);
        mctx.tensor_set(x_t, x.data(), 0, x.size() * sizeof(float));
        Tensor *out_t = attn.forward(&mctx, x_t, nullptr, nullptr, n_past);
        EXPECT(out_t->type == TYPE_F32 && out_t->ne[0] == c.hidden && out_t->ne[1] == qlen, "attn_output shape");
        std::vector<float> got(static_cast<size_t>(qlen) * c.hidden);
        mctx.tensor_get(out_t, got.data(), 0, got.size() * sizeof(float));
        mctx.synchronize();

        std::vector<float> qkv(static_cast<size_t>(qlen) * width), ctx(static_cast<size_t>(qlen) * c.hidden), want(got.size()), mask;
        oracle_linear(x.data(), qlen, c.hidden, w_qkv.data(), 1, c.qkv_bias ? b_qkv.data() : nullptr, width, 1, qkv.data());
        round_f16(qkv);
        const float *q = qkv.data(), *k, *v;
        long hs;
        if (c.interleaved) { k = q + D; v = q + 2 * D; hs = 3 * D; } else { k = q + c.hidden; v = q + c.hidden + G * D; hs = D; }
        std::vector<int> ids = c.rope == RopeType::CHATGLM ? make_position_ids_glm(qlen, n_past, c.prompt) : make_position_ids_glm2(qlen, n_past);
        if (n_past == 0 && c.mask == AttentionMaskType::CHATGLM) {
            mask.resize(static_cast<size_t>(qlen) * qlen);
            oracle_attention_mask_glm(qlen, qlen, mask.data());
        }
        int rc = oracle_attn_forward(&cfg, q, width, hs, k, v, width, hs, kc.data(), vc.data(), ids.data(),
                                     mask.empty() ? nullptr : mask.data(), qlen, n_past, ctx.data(), nullptr, nullptr);
        EXPECT(rc == 0, "oracle rejected the arguments");
        oracle_linear(ctx.data(), qlen, c.hidden, w_dense.data(), 1, c.dense_bias ? b_dense.data() : nullptr, c.hidden, 1, want.data());
        for (size_t i = 0; i < got.size(); i++) {
            EXPECT(std::isfinite(got[i]), "non-finite output");
            worst = std::fmax(worst, std::fabs(got[i] - want[i]));
        }
        n_past += qlen;
        mctx.reset_scratch();
    }
    EXPECT(worst <= 6e-3f, "%s: max abs error %g", c.name, worst);
    // The same module inside a DecodeStep that runs the Linears itself: three more tokens, one eager step, one captured,
    // one replayed (the fused decode kernel reads the position from the device word; shapes it does not take have no step).
    float worst_step = 0.f;
    int replays = 0;
    if (D == 128) {
        DecodeStep step(&mctx, {&attn}, /*with_linears=*/true);
        step.set_n_past(n_past);
        for (int t = 0; t < 3; t++) {
            std::vector<float> x(c.hidden);
            for (auto &e : x) e = dist(rng);
            std::vector<uint16_t> x16(x.size());
            for (size_t i = 0; i < x.size(); i++) x16[i] = oracle_f32_to_f16(x[i]);
            mctx.tensor_set(step.hidden(0), x16.data(), 0, x16.size() * 2);
            step.run();
            std::vector<float> got(c.hidden);
            mctx.tensor_get(step.attn_output(0), got.data(), 0, got.size() * sizeof(float));
            mctx.synchronize();
            std::vector<float> qkv(width), ctx(c.hidden), want(c.hidden);
            oracle_linear(x.data(), 1, c.hidden, w_qkv.data(), 1, c.qkv_bias ? b_qkv.data() : nullptr, width, 1, qkv.data());
            round_f16(qkv);
            const float *q = qkv.data(), *k, *v;
            long hs;
            if (c.interleaved) { k = q + D; v = q + 2 * D; hs = 3 * D; } else { k = q + c.hidden; v = q + c.hidden + G * D; hs = D; }
            std::vector<int> ids = c.rope == RopeType::CHATGLM ? make_position_ids_glm(1, n_past, c.prompt) : make_position_ids_glm2(1, n_past);
            int rc = oracle_attn_forward(&cfg, q, width, hs, k, v, width, hs, kc.data(), vc.data(), ids.data(), nullptr, 1, n_past,
                                         ctx.data(), nullptr, nullptr);
            EXPECT(rc == 0, "oracle rejected the arguments");
            oracle_linear(ctx.data(), 1, c.hidden, w_dense.data(), 1, c.dense_bias ? b_dense.data() : nullptr, c.hidden, 1, want.data());
            for (size_t i = 0; i < got.size(); i++) {
                EXPECT(std::isfinite(got[i]), "non-finite output");
                worst_step = std::fmax(worst_step, std::fabs(got[i] - want[i]));
            }
            n_past += 1;
        }
        EXPECT(step.n_past() == n_past && step.status() == 0, "%s: step position / status", c.name);
        replays = step.graph_launches();
        EXPECT(replays == 2, "%s: %d graph launches", c.name, replays);
        EXPECT(worst_step <= 6e-3f, "%s: step graph with Linears, max abs error %g", c.name, worst_step);
    }
    // caches: the same f16 values up to a neighbouring one where the GEMM's sum fell on the other side of a tie
    std::vector<uint16_t> gk(kc.size()), gv(vc.size());
    mctx.tensor_get(attn.k_cache, gk.data(), 0, gk.size() * 2);
    mctx.tensor_get(attn.v_cache, gv.data(), 0, gv.size() * 2);
    float cache_worst = 0.f;
    size_t differing = 0;
    for (size_t i = 0; i < kc.size(); i++) {
        cache_worst = std::fmax(cache_worst, std::fabs(oracle_f16_to_f32(gk[i]) - oracle_f16_to_f32(kc[i])));
        cache_worst = std::fmax(cache_worst, std::fabs(oracle_f16_to_f32(gv[i]) - oracle_f16_to_f32(vc[i])));
        differing += (gk[i] != kc[i]) + (gv[i] != vc[i]);
    }
    EXPECT(cache_worst <= 8e-3f, "%s: cache value off by %g", c.name, cache_worst);
    EXPECT(differing <= static_cast<size_t>(0.04 * 2 * G * D * n_past) + 4, "%s: %zu cache values differ", c.name, differing);
    std::printf("case %-28s max abs err %.3g, step graph with Linears %.3g over %d replays (caches: %zu values on a neighbouring f16)\n",
                c.name, worst, worst_step, replays, differing);
}

// A model file (written by the test driver with the converter's layout): every layer's attention module is built from
// the configuration record, takes its Linear parameters and its P-Tuning prefix from the file, and runs forward on a
// short prompt; checked against the oracle fed the tensors of the same file.
static void run_model_file_case(const char *path) {
    ModelFile file(path);
    const ModelConfig &c = file.config;
    const int H = c.num_attention_heads, G = c.num_key_value_heads, D = c.hidden_size / H, V = c.num_virtual_tokens;
    const int M = c.max_length + V, width = c.hidden_size + 2 * D * G;
    ModelContext mctx(nullptr);
    std::vector<BasicAttention> layers;
    for (int l = 0; l < c.num_hidden_layers; l++) {
        layers.emplace_back(&mctx, c.hidden_size, H, G, c.max_length, c.use_qkv_bias, c.use_dense_bias, c.interleaved_qkv,
                            c.rope_type, c.rope_theta, c.attn_mask_type, V);
    }
    mctx.alloc_kv();
    const int layer = c.num_hidden_layers - 1;
    BasicAttention &attn = layers[layer];
    attn.load_weights(&mctx, file, layer);
    auto tensor = [&](int which) -> const HostTensor * {
        if (which == 3 && !c.use_dense_bias) return nullptr;
        auto it = file.state_dict.kv.find(file.attn_weight_name(layer, which));
        return it == file.state_dict.kv.end() ? nullptr : &it->second;
    };
    const HostTensor *wq = tensor(0), *bq = tensor(1), *wd = tensor(2), *bd = tensor(3);
    EXPECT(wq && wd, "the file holds both weights");
    oracle_cfg cfg = {H, G, D, M, V, static_cast<int>(c.rope_type), c.rope_theta,
                      c.attn_mask_type == AttentionMaskType::CAUSAL ? ORACLE_MASK_CAUSAL : ORACLE_MASK_CHATGLM, oracle_numerics_f32()};
    std::vector<uint16_t> kc(static_cast<size_t>(G) * M * D, 0), vc(kc.size(), 0);
    if (V > 0) {
        auto it = file.state_dict.kv.find("past_key_values");
        EXPECT(it != file.state_dict.kv.end(), "prefix tensor present");
        const size_t block = static_cast<size_t>(2) * G * V * D;
        const uint16_t *past = static_cast<const uint16_t *>(it->second.data) + block * layer;
        Tensor *dev = mctx.new_tensor_1d(TYPE_F16, static_cast<int64_t>(block));
        mctx.tensor_set(dev, past, 0, block * 2);
        attn.load_prefix_cache(&mctx, dev);
        oracle_load_prefix_cache(&cfg, past, kc.data(), vc.data());
    }
    std::mt19937 rng(99);
    std::normal_distribution<float> dist(0.f, 0.05f);   // the file's weights are N(0, 1): keep the sums of unit scale
    const int qlen = 3;
    std::vector<float> x(static_cast<size_t>(qlen) * c.hidden_size);
    for (auto &e : x) e = dist(rng);
    Tensor *x_t = mctx.new_tensor_2d(TYPE_F32, c.hidden_size, qlen);
    mctx.tensor_set(x_t, x.data(), 0, x.size() * sizeof(float));
    Tensor *out_t = attn.forward(&mctx, x_t, nullptr, nullptr, 0);
    std::vector<float> got(static_cast<size_t>(qlen) * c.hidden_size);
    mctx.tensor_get(out_t, got.data(), 0, got.size() * sizeof(float));
    mctx.synchronize();
    std::vector<float> qkv(static_cast<size_t>(qlen) * width), ctx(got.size()), want(got.size());
    oracle_linear(x.data(), qlen, c.hidden_size, wq->data, 1, bq ? static_cast<const float *>(bq->data) : nullptr, width, 1, qkv.data());
    for (auto &e : qkv) e = oracle_f16_to_f32(oracle_f32_to_f16(e));
    const float *q = qkv.data(), *k = q + c.hidden_size, *v = q + c.hidden_size + G * D;
    std::vector<int> ids = make_position_ids_glm2(qlen, 0);
    int rc = oracle_attn_forward(&cfg, q, width, D, k, v, width, D, kc.data(), vc.data(), ids.data(), nullptr, qlen, 0, ctx.data(),
                                 nullptr, nullptr);
    EXPECT(rc == 0, "oracle rejected the arguments");
    oracle_linear(ctx.data(), qlen, c.hidden_size, wd->data, 1, bd ? static_cast<const float *>(bd->data) : nullptr, c.hidden_size, 1,
                  want.data());
    float worst = 0.f, scale = 0.f;
    for (size_t i = 0; i < got.size(); i++) {
        worst = std::fmax(worst, std::fabs(got[i] - want[i]));
        scale = std::fmax(scale, std::fabs(want[i]));
    }
    EXPECT(worst <= 6e-3f * std::fmax(1.f, scale), "model file case: max abs error %g at scale %g", worst, scale);
    std::printf("case %-28s max abs err %.3g (output scale %.3g)\n", "forward from a model file", worst, scale);
}

int main(int argc, char **argv) {
    const Case cases[] = {
        {"glm3 gqa d128 blocked", 4096, 32, 2, 512, 0, false, RopeType::CHATGLM2, AttentionMaskType::CAUSAL, 5, false},
        {"glm3 gqa d128 long prompt", 4096, 32, 2, 512, 0, false, RopeType::CHATGLM2, AttentionMaskType::CAUSAL, 200, true},
        {"glm1 mha interleaved 2d-rope", 1024, 8, 8, 256, 0, true, RopeType::CHATGLM, AttentionMaskType::CHATGLM, 7, true},
        {"glm1 derived position ids", 1024, 8, 8, 256, 0, true, RopeType::CHATGLM, AttentionMaskType::CHATGLM, 7, false},
        {"glm3 p-tuning prefix d4", 32, 8, 2, 8, 5, false, RopeType::CHATGLM2, AttentionMaskType::CAUSAL, 3, false},
        // max_length + num_virtual_tokens = 133: the arena's rows have a pitch of 136 tokens, the tensors keep ne = 133
        {"glm3 p-tuning prefix d128 odd capacity", 1024, 8, 2, 128, 5, false, RopeType::CHATGLM2, AttentionMaskType::CAUSAL, 9, false},
    };
    try {
        for (const Case &c : cases) run_case(c);
        run_error_cases();
        run_decode_step_case();
        const FullCase full[] = {
            // fused decode route after a tensor-core prefill
            {"forward glm3 gqa d128", 4096, 32, 2, 512, false, true, false, RopeType::CHATGLM2, AttentionMaskType::CAUSAL, 130},
            // general route: interleaved qkv, 2-D rotary, both biases
            {"forward glm1 mha interleaved", 1024, 8, 8, 256, true, true, true, RopeType::CHATGLM, AttentionMaskType::CHATGLM, 7},
            // head size 64: generic attention kernels behind the same GEMMs
            {"forward d64 neox", 512, 8, 8, 128, false, false, true, RopeType::NEOX, AttentionMaskType::CAUSAL, 5},
        };
        for (const FullCase &c : full) run_full_forward_case(c);
        if (argc > 1) run_model_file_case(argv[1]);
    } catch (const std::exception &e) {
        std::printf("FAIL unexpected exception: %s\n", e.what());
        return 1;
    }
    if (g_failures) {
        std::printf("%d failure(s)\n", g_failures);
        return 1;
    }
    std::printf("ALL OK\n");
    return 0;
}
