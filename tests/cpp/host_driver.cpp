// Drives the C++ host mirror (include/shady_host.hpp) the way the reference's generate_tokens drives Model::forward
// (src/inference.rs:89-99): reset seq_len, then per token and per layer the three helpers of model.rs:723-725.
// Usage: host_driver <in.bin> <out.bin>
// in.bin : u32 nh, nkv, hd, T, layers; f32 theta, partial_rotary_factor; per layer 2*hd bf16 norm weights (q then k);
//          then per token, per layer: q_proj_full [nh][2][hd], k_proj [nkv][hd], v_proj [nkv][hd] as f32.
// out.bin: per token, per layer: attn_output [nh][hd] f32 after the gate.
#include <cstdio>
#include <vector>

#include "shady_host.hpp"

using namespace shady_thinker;

template <typename T> static void rd(FILE *f, T *dst, size_t n) {
    if (fread(dst, sizeof(T), n, f) != n) throw std::runtime_error("short read");
}

int main(int argc, char **argv) {
    if (argc != 3) return 2;
    try {
        FILE *in = fopen(argv[1], "rb"), *out = fopen(argv[2], "wb");
        if (!in || !out) throw std::runtime_error("cannot open files");
        uint32_t hdr[5];
        float fl[2];
        rd(in, hdr, 5);
        rd(in, fl, 2);
        ModelConfig cfg;
        cfg.num_attention_heads = hdr[0]; cfg.num_key_value_heads = hdr[1]; cfg.head_dim = hdr[2];
        const uint32_t T = hdr[3];
        cfg.num_hidden_layers = hdr[4]; cfg.rope_theta = fl[0]; cfg.partial_rotary_factor = fl[1];
        GpuContext gpu(0);
        Model model(gpu, cfg, T + 1);
        const size_t nh = hdr[0], nkv = hdr[1], hd = hdr[2];
        for (uint32_t l = 0; l < cfg.num_hidden_layers; ++l) {
            std::vector<uint16_t> w(2 * hd);
            rd(in, w.data(), w.size());
            model.init_qknorm_params(gpu, l, w.data(), w.data() + hd);
        }
        std::vector<float> q(nh * 2 * hd), k(nkv * hd), v(nkv * hd);
        model.seq_len = 0;                                   // inference.rs:89
        for (uint32_t t = 0; t < T; ++t) {
            for (uint32_t l = 0; l < cfg.num_hidden_layers; ++l) {
                rd(in, q.data(), q.size()); rd(in, k.data(), k.size()); rd(in, v.data(), v.size());
                gpu.write_buffer(model.state.q_out, 0, q.data(), q.size() * 4);
                gpu.write_buffer(model.state.k_out, 0, k.data(), k.size() * 4);
                gpu.write_buffer(model.state.v_out, 0, v.data(), v.size() * 4);
                model.fused_split_qknorm_kvstore(gpu, l);    // model.rs:723
                model.gqa_attention(gpu, l);                 // model.rs:724
                model.sigmoid_mul_gate(gpu);                 // model.rs:725
                const std::vector<uint8_t> o = gpu.read_buffer(model.state.attn_output, nh * hd * 4);
                fwrite(o.data(), 1, o.size(), out);
            }
            model.seq_len += 1;                              // model.rs:837
        }
        // error behaviour: the cache is full now; one more append must throw, not abort
        bool threw = false;
        model.seq_len = T + 1;
        try { model.fused_split_qknorm_kvstore(gpu, 0); } catch (const std::runtime_error &) { threw = true; }
        fclose(in); fclose(out);
        return threw ? 0 : 3;
    } catch (const std::exception &e) {
        fprintf(stderr, "host_driver: %s\n", e.what());
        return 1;
    }
}
