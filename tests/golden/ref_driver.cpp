// Runs kishida/questwend's own CPU code on a tiny Qwen3 model and writes its logits.
// Used once by make_golden.py; not part of the library.  It calls the reference's public
// classes only (Model::load, Runtime::decode, core/model.h:98-119, core/runtime.h:47-143)
// and ggml's GGUF writer (third_party/ggml/include/gguf.h) to put the weights into the
// container the reference reads.
//
//   ref_driver <dump.bin> <tmp.gguf> <out.bin>
//
// dump.bin:  int32 L D H Hkv hd F V tie n_tokens; float32 theta eps; int32 tokens[n_tokens];
//            then, n_tensors times: int32 name_len, name bytes (GGUF name), int32 n_dims,
//            int32 dims[n_dims] (row-major, outermost first), float32 data.
// out.bin:   float32 logits[n_tokens][V] from feeding the tokens one at a time, then
//            float32 logits[V] of the last position from feeding the whole prompt at once.
#include "model.h"
#include "runtime.h"
#include "ggml.h"
#include "gguf.h"

#include <cstdio>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

using namespace questwend;

template <typename T> static T rd(FILE* f) { T v; if (fread(&v, sizeof(T), 1, f) != 1) { fprintf(stderr, "short read\n"); exit(2); } return v; }

int main(int argc, char** argv) {
    if (argc != 4) { fprintf(stderr, "usage: ref_driver dump.bin tmp.gguf out.bin\n"); return 1; }
    FILE* f = fopen(argv[1], "rb");
    if (!f) { perror(argv[1]); return 1; }
    const int L = rd<int32_t>(f), D = rd<int32_t>(f), H = rd<int32_t>(f), Hkv = rd<int32_t>(f), hd = rd<int32_t>(f);
    const int F = rd<int32_t>(f), V = rd<int32_t>(f), tie = rd<int32_t>(f), T = rd<int32_t>(f);
    const float theta = rd<float>(f), eps = rd<float>(f);
    (void)tie;
    std::vector<int32_t> toks(T);
    for (auto& t : toks) t = rd<int32_t>(f);
    std::map<std::string, std::vector<float>> data;
    std::map<std::string, std::vector<int64_t>> shape;      // ggml order: contiguous dimension first
    for (;;) {
        int32_t len;
        if (fread(&len, 4, 1, f) != 1) break;
        std::string name(len, 0);
        if (fread(&name[0], 1, len, f) != (size_t)len) return 2;
        const int nd = rd<int32_t>(f);
        std::vector<int64_t> dims(nd);
        size_t n = 1;
        for (int i = 0; i < nd; ++i) { dims[i] = rd<int32_t>(f); n *= dims[i]; }
        std::vector<float> v(n);
        if (fread(v.data(), 4, n, f) != n) return 2;
        shape[name] = std::vector<int64_t>(dims.rbegin(), dims.rend());
        data[name] = std::move(v);
    }
    fclose(f);

    {
        ggml_init_params ip{};
        ip.mem_size = ggml_tensor_overhead() * (data.size() + 4);
        ip.no_alloc = true;
        ggml_context* ctx = ggml_init(ip);
        gguf_context* g = gguf_init_empty();
        gguf_set_val_str(g, "general.architecture", "qwen3");
        gguf_set_val_u32(g, "qwen3.block_count", L);
        gguf_set_val_u32(g, "qwen3.embedding_length", D);
        gguf_set_val_u32(g, "qwen3.feed_forward_length", F);
        gguf_set_val_u32(g, "qwen3.attention.head_count", H);
        gguf_set_val_u32(g, "qwen3.attention.head_count_kv", Hkv);
        gguf_set_val_u32(g, "qwen3.attention.key_length", hd);
        gguf_set_val_u32(g, "qwen3.context_length", 256);
        gguf_set_val_f32(g, "qwen3.rope.freq_base", theta);
        gguf_set_val_f32(g, "qwen3.attention.layer_norm_rms_epsilon", eps);
        for (auto& kv : data) {
            ggml_tensor* t = ggml_new_tensor(ctx, GGML_TYPE_F32, (int)shape[kv.first].size(), shape[kv.first].data());
            ggml_set_name(t, kv.first.c_str());
            gguf_add_tensor(g, t);
            gguf_set_tensor_data(g, kv.first.c_str(), kv.second.data());
        }
        if (!gguf_write_to_file(g, argv[2], false)) { fprintf(stderr, "cannot write %s\n", argv[2]); return 1; }
        gguf_free(g);
        ggml_free(ctx);
    }

    auto model = Model::load(argv[2]);
    if ((int)model->hparams().n_vocab != V) { fprintf(stderr, "vocab mismatch\n"); return 1; }
    RuntimeConfig rc;
    rc.n_ctx = 256;
    rc.use_cuda = false;
    rc.n_threads = 1;
    Runtime rt(*model, rc);
    FILE* out = fopen(argv[3], "wb");
    if (!out) { perror(argv[3]); return 1; }
    for (int32_t t : toks) {
        std::vector<float> lg = rt.decode({t});
        fwrite(lg.data(), 4, lg.size(), out);
    }
    rt.reset();
    std::vector<float> whole = rt.decode(toks);
    fwrite(whole.data(), 4, whole.size(), out);
    fclose(out);
    return 0;
}
