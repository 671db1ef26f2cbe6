// Times kishida/questwend's own, unmodified engine on the benchmark's workload.  Nothing of questwend_b200 is used
// here: the program calls the reference's public classes only (Model::load, Runtime::decode, Sampler;
// core/model.h:98-119, core/runtime.h:47-143, core/sampler.h:30-40) the way its command line does
// (cli/main.cpp:408-425), and ggml's GGUF writer (third_party/ggml/include/gguf.h) to put seeded random weights of
// the wanted sizes into the container that the reference reads.
//
//   qw_ref_bench --gguf FILE [--layers L --hidden D --heads H --kv-heads Hkv --head-dim hd --inter F --vocab V]
//                [--n-ctx 4096] [--prompt 1024] [--prefill 2048] [--sequences 8] [--steps K] [--warmup W] [--seed S] [--cpu]
//
// The reference holds one sequence (core/runtime.cpp:166), so a "batch" of N sequences is N sequences one after the
// other: each gets its prompt, W untimed and K timed single-token steps.  One JSON line on standard output:
//   decode_tok_s      tokens a second over all timed Runtime::decode({token}) calls (token and mask in, logits out:
//                     core/runtime.cpp:1798-1818)
//   e2e_tok_s         the same with the reference's host sampler, greedy, in the timed region (cli/main.cpp:417-424)
//   prefill_tok_s     one prompt of --prefill tokens through Runtime::decode (chunks of 512, core/runtime.cpp:3092-3113)
// Weights: bfloat16 N(0, 0.02) for matrices, float32 1 + U(-0.1, 0.1) for norms, from --seed.
#include "model.h"
#include "runtime.h"
#include "sampler.h"
#include "ggml.h"
#include "gguf.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

using namespace questwend;
using clk = std::chrono::steady_clock;

static double seconds(clk::time_point a, clk::time_point b) { return std::chrono::duration<double>(b - a).count(); }

struct Rng {                                   // splitmix64
    uint64_t s;
    uint64_t next() { uint64_t z = (s += 0x9E3779B97F4A7C15ull); z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
                      z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; return z ^ (z >> 31); }
    double uniform() { return (next() >> 11) * (1.0 / 9007199254740992.0); }
};

static uint16_t to_bf16(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

// N(0, 0.02) as bfloat16, drawn by several threads, each with a stream of its own
static void fill_normal_bf16(uint16_t* dst, size_t n, uint64_t seed) {
    const unsigned nt = std::max(1u, std::min(32u, std::thread::hardware_concurrency()));
    std::vector<std::thread> th;
    for (unsigned t = 0; t < nt; ++t)
        th.emplace_back([=] {
            Rng r{seed * 1000003ull + t};
            const size_t a = n * t / nt, b = n * (t + 1) / nt;
            for (size_t i = a; i < b; i += 2) {
                const double u1 = 1.0 - r.uniform(), u2 = r.uniform();
                const double m = 0.02 * std::sqrt(-2.0 * std::log(u1));
                dst[i] = to_bf16((float)(m * std::cos(6.283185307179586 * u2)));
                if (i + 1 < b) dst[i + 1] = to_bf16((float)(m * std::sin(6.283185307179586 * u2)));
            }
        });
    for (auto& x : th) x.join();
}

struct Sizes { int L = 36, D = 4096, H = 32, Hkv = 8, hd = 128, F = 12288, V = 151936, n_ctx = 4096; };

static bool write_gguf(const std::string& path, const Sizes& z, uint64_t seed) {
    struct T { std::string name; ggml_type type; std::vector<int64_t> ne; void* data; };
    std::vector<T> ts;
    std::vector<std::vector<uint16_t>> mats;
    std::vector<std::vector<float>> vecs;
    uint64_t k = seed;
    auto mat = [&](const std::string& name, int64_t rows, int64_t cols) {      // stored [rows, cols]: ne = {cols, rows}
        mats.emplace_back((size_t)rows * cols);
        fill_normal_bf16(mats.back().data(), mats.back().size(), ++k);
        ts.push_back({name, GGML_TYPE_BF16, {cols, rows}, mats.back().data()});
    };
    auto vec = [&](const std::string& name, int64_t n) {
        vecs.emplace_back((size_t)n);
        Rng r{++k};
        for (auto& v : vecs.back()) v = (float)(1.0 + 0.1 * (2.0 * r.uniform() - 1.0));
        ts.push_back({name, GGML_TYPE_F32, {n}, vecs.back().data()});
    };
    mat("token_embd.weight", z.V, z.D);
    for (int l = 0; l < z.L; ++l) {
        const std::string b = "blk." + std::to_string(l) + ".";
        vec(b + "attn_norm.weight", z.D);
        mat(b + "attn_q.weight", (int64_t)z.H * z.hd, z.D);
        mat(b + "attn_k.weight", (int64_t)z.Hkv * z.hd, z.D);
        mat(b + "attn_v.weight", (int64_t)z.Hkv * z.hd, z.D);
        vec(b + "attn_q_norm.weight", z.hd);
        vec(b + "attn_k_norm.weight", z.hd);
        mat(b + "attn_output.weight", z.D, (int64_t)z.H * z.hd);
        vec(b + "ffn_norm.weight", z.D);
        mat(b + "ffn_gate.weight", z.F, z.D);
        mat(b + "ffn_up.weight", z.F, z.D);
        mat(b + "ffn_down.weight", z.D, z.F);
    }
    vec("output_norm.weight", z.D);
    mat("output.weight", z.V, z.D);

    ggml_init_params ip{};
    ip.mem_size = ggml_tensor_overhead() * (ts.size() + 4);
    ip.no_alloc = true;
    ggml_context* ctx = ggml_init(ip);
    gguf_context* g = gguf_init_empty();
    gguf_set_val_str(g, "general.architecture", "qwen3");
    gguf_set_val_u32(g, "qwen3.block_count", z.L);
    gguf_set_val_u32(g, "qwen3.embedding_length", z.D);
    gguf_set_val_u32(g, "qwen3.feed_forward_length", z.F);
    gguf_set_val_u32(g, "qwen3.attention.head_count", z.H);
    gguf_set_val_u32(g, "qwen3.attention.head_count_kv", z.Hkv);
    gguf_set_val_u32(g, "qwen3.attention.key_length", z.hd);
    gguf_set_val_u32(g, "qwen3.context_length", z.n_ctx);
    gguf_set_val_f32(g, "qwen3.rope.freq_base", 1e6f);
    gguf_set_val_f32(g, "qwen3.attention.layer_norm_rms_epsilon", 1e-6f);
    for (auto& t : ts) {
        ggml_tensor* gt = ggml_new_tensor(ctx, t.type, (int)t.ne.size(), t.ne.data());
        ggml_set_name(gt, t.name.c_str());
        gguf_add_tensor(g, gt);
        gguf_set_tensor_data(g, t.name.c_str(), t.data);
    }
    const bool ok = gguf_write_to_file(g, path.c_str(), false);
    gguf_free(g);
    ggml_free(ctx);
    return ok;
}

int main(int argc, char** argv) {
    Sizes z;
    std::string gguf;
    int prompt = 1024, prefill = 2048, sequences = 8, steps = 20, warmup = 5;
    uint64_t seed = 0;
    bool cpu = false;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto val = [&]() -> const char* { if (i + 1 >= argc) { fprintf(stderr, "%s needs a value\n", a.c_str()); exit(2); } return argv[++i]; };
        if (a == "--gguf") gguf = val();
        else if (a == "--layers") z.L = atoi(val());
        else if (a == "--hidden") z.D = atoi(val());
        else if (a == "--heads") z.H = atoi(val());
        else if (a == "--kv-heads") z.Hkv = atoi(val());
        else if (a == "--head-dim") z.hd = atoi(val());
        else if (a == "--inter") z.F = atoi(val());
        else if (a == "--vocab") z.V = atoi(val());
        else if (a == "--n-ctx") z.n_ctx = atoi(val());
        else if (a == "--prompt") prompt = atoi(val());
        else if (a == "--prefill") prefill = atoi(val());
        else if (a == "--sequences") sequences = atoi(val());
        else if (a == "--steps") steps = atoi(val());
        else if (a == "--warmup") warmup = atoi(val());
        else if (a == "--seed") seed = strtoull(val(), nullptr, 10);
        else if (a == "--cpu") cpu = true;
        else { fprintf(stderr, "unknown option %s\n", a.c_str()); return 2; }
    }
    if (gguf.empty()) { fprintf(stderr, "--gguf FILE is required\n"); return 2; }
    if (prompt + warmup + steps + 1 > z.n_ctx || prefill > z.n_ctx) { fprintf(stderr, "the workload exceeds n_ctx %d\n", z.n_ctx); return 2; }

    try {
        auto t0 = clk::now();
        if (!write_gguf(gguf, z, seed)) { fprintf(stderr, "cannot write %s\n", gguf.c_str()); return 1; }
        auto t1 = clk::now();
        fprintf(stderr, "[ref_bench] wrote %s in %.1f s\n", gguf.c_str(), seconds(t0, t1));
        auto model = Model::load(gguf);
        RuntimeConfig rc;
        rc.n_ctx = z.n_ctx;
        rc.use_cuda = !cpu;
        Runtime rt(*model, rc);
        auto t2 = clk::now();
        fprintf(stderr, "[ref_bench] loaded in %.1f s\n", seconds(t1, t2));

        Rng r{seed + 77};
        auto random_ids = [&](int n) { std::vector<int32_t> v(n); for (auto& t : v) t = (int32_t)(r.next() % (uint64_t)z.V); return v; };

        // ---- prefill of one prompt: one untimed run, then the median of three
        std::vector<double> pf;
        for (int rep = 0; rep < 4 && prefill > 0; ++rep) {
            rt.reset();
            const auto ids = random_ids(prefill);
            auto a = clk::now();
            rt.decode(ids);
            auto b = clk::now();
            if (rep) pf.push_back(seconds(a, b));
        }
        std::sort(pf.begin(), pf.end());
        const double pf_s = pf.empty() ? 0.0 : pf[pf.size() / 2];

        // ---- decode: the sequences one after the other; first decode() alone, then with the host sampler
        SamplerConfig sc;
        sc.temperature = 0.f;                                  // the command line's default: greedy (cli/main.cpp:134)
        double t_decode = 0.0, t_e2e = 0.0;
        long n_decode = 0, n_e2e = 0;
        for (int mode = 0; mode < 2; ++mode)
            for (int s = 0; s < sequences; ++s) {
                rt.reset();
                Sampler smp(sc);
                const auto ids = random_ids(prompt);
                std::vector<float> logits = rt.decode(ids);
                smp.prime(ids);
                int32_t next = smp.sample(logits);
                for (int i = 0; i < warmup; ++i) { logits = rt.decode({next}); next = smp.sample(logits); smp.accept(next); }
                if (mode == 0) {
                    for (int i = 0; i < steps; ++i) {
                        auto a = clk::now();
                        const std::vector<float>& lg = rt.decode({next});
                        auto b = clk::now();
                        t_decode += seconds(a, b);
                        next = smp.sample(lg);
                        smp.accept(next);
                    }
                    n_decode += steps;
                } else {
                    auto a = clk::now();
                    for (int i = 0; i < steps; ++i) {
                        const std::vector<float>& lg = rt.decode({next});
                        next = smp.sample(lg);
                        smp.accept(next);
                    }
                    auto b = clk::now();
                    t_e2e += seconds(a, b);
                    n_e2e += steps;
                }
            }
        printf("{\"decode_tok_s\": %.3f, \"ms_per_token\": %.4f, \"e2e_tok_s\": %.3f, \"prefill_tok_s\": %.1f, \"prefill_ms\": %.3f, "
               "\"prefill_tokens\": %d, \"sequences\": %d, \"steps\": %d, \"warmup\": %d, \"prompt\": %d, \"layers\": %d, "
               "\"backend\": \"%s\", \"load_s\": %.1f, \"write_s\": %.1f}\n",
               n_decode / t_decode, 1e3 * t_decode / n_decode, n_e2e / t_e2e, pf_s > 0 ? prefill / pf_s : 0.0, pf_s * 1e3,
               prefill, sequences, steps, warmup, prompt, z.L, cpu ? "cpu" : "gpu", seconds(t1, t2), seconds(t0, t1));
    } catch (const std::exception& e) {
        fprintf(stderr, "[ref_bench] error: %s\n", e.what());
        return 1;
    }
    return 0;
}
