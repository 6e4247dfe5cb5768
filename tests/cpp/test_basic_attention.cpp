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
        Tensor *ctx = attn.forward(&mctx, qkv_t, nullptr, ids_t, n_past);
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
        attn.forward(&mctx, &bogus, nullptr, nullptr, 0);   // kv buffer not allocated yet
    } catch (const std::runtime_error &e) {
        threw = std::strstr(e.what(), "chatglm_b200.cu") != nullptr;   // "file:line message", like CHATGLM_CHECK
    }
    EXPECT(threw, "forward before alloc_kv must throw std::runtime_error with file:line");
    mctx.alloc_kv();
    Tensor *bad = mctx.new_tensor_2d(TYPE_F32, 100, 1);   // wrong row width
    threw = false;
    try {
        attn.forward(&mctx, bad, nullptr, nullptr, 0);
    } catch (const std::runtime_error &) {
        threw = true;
    }
    EXPECT(threw, "a qkv row of the wrong width must throw");
    Tensor *qkv = mctx.new_tensor_2d(TYPE_F32, 4096 + 2 * 128 * 2, 1);
    threw = false;
    try {
        attn.forward(&mctx, qkv, nullptr, nullptr, 256);   // n_past + qlen beyond max_length
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
        layers[l].forward(&mctx, t, nullptr, nullptr, 0);
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

int main() {
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
