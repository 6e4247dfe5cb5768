// Host-only driver of chatglm::ModelFile for the sanitizer run: parses the file named on the command line and prints
// what it found.  Exit code 0: parsed; 3: refused with a CHATGLM_CHECK exception (the expected answer for a broken
// file); anything else (a sanitizer report, a signal) is a bug in the reader.
#include <cstdio>
#include <exception>

#include "../../include/chatglm_b200.h"

int main(int argc, char **argv) {
    if (argc < 2) {
        std::fprintf(stderr, "usage: %s model-file [max_length]\n", argv[0]);
        return 2;
    }
    try {
        chatglm::ModelFile mf(std::string(argv[1]), argc > 2 ? std::atoi(argv[2]) : 0);
        const chatglm::ModelConfig &c = mf.config;
        const cglm_attn_desc d = c.attn_desc();
        std::printf("model_type=%d version=%d layers=%d heads=%d kv_heads=%d head_dim=%d max_len=%d virtual=%d rope=%d mask=%d\n",
                    static_cast<int>(c.model_type), mf.version, c.num_hidden_layers, d.n_head, d.n_kv_head, d.head_dim,
                    d.max_len, d.n_virtual, d.rope_type, d.mask_type);
        unsigned long long sum = 0;   // touch every byte the table points at: an over-long view would trip the sanitizer
        for (const std::string &name : mf.state_dict.names) {
            const chatglm::HostTensor &t = mf.state_dict.kv.at(name);
            const unsigned char *p = static_cast<const unsigned char *>(t.data);
            for (size_t i = 0; i < t.nbytes; i++) sum += p[i];
        }
        for (size_t i = 0; i < mf.tokenizer_size; i++) sum += static_cast<unsigned char>(mf.tokenizer_data[i]);
        std::printf("tensors=%zu qkv0=%s checksum=%llu\n", mf.state_dict.names.size(), mf.attn_weight_name(0, 0).c_str(), sum);
        return 0;
    } catch (const std::exception &e) {
        std::printf("refused: %s\n", e.what());
        return 3;
    }
}
