// Driver around upstream's dense Qwen3 classes, for timing and for dumping logits.
//
// Upstream's main() (inference.cpp:29-209) builds the mixture-of-experts model, reads a prompt from the
// keyboard and decodes 601 tokens at batch 1.  This program does the same steps around the dense classes
// instead, with the batch size as an argument and token ids from a file or a counter:
//   load      Qwen3Config::from_pretrained / Qwen3::from_pretrained   (src/models/qwen3/qwen3.cpp:24-112)
//   caches    one KVCache per layer                                   (inference.cpp:77-96, src/kvcache.h:40-61)
//   engine    FlashAttnEngine + get_graph                             (inference.cpp:129-134)
//   a step    prepare_table per layer, Qwen3::forward, argmax         (inference.cpp:140-145)
//   next x    argmax's result as a [B,1] tensor, new position tensor  (inference.cpp:151-160)
// All arithmetic, the cache and the attention are upstream's, unmodified; nothing of this repository's
// library is linked.  Upstream never checks the cache's capacity (src/src-cuda/kvcache.cu:46-55) and leaves
// unmapped block-table entries at -1, so the tables are sized for the whole run and every page is mapped once
// before the first step (one prepare_table call over the full capacity): no index can leave its table.
// Upstream counts elements in `int` (src/tensor.h:294-299): a prompt whose [B,S,vocab] logits would pass 2^31
// elements is fed in equal chunks (--chunk), which upstream's bottom-right causal mask allows.
//
//   reference_runner MODEL_DIR [--batch B] [--prompt-len S] [--chunk C] [--steps K] [--warmup W]
//                    [--ids FILE] [--dump FILE] [--prefill-repeats R]
// --ids FILE   uint32 ids, B rows of S+W+K: the prompt, then the token fed at each decode step (teacher forcing);
//              without it prompts come from a counter and each step feeds the argmax of the one before.
// --dump FILE  append every step's logits as float32 [B,S_step,vocab].
// It prints one JSON line with device-timed (CUDA events on upstream's compute stream) and wall-clock step times.
#include <cuda_runtime.h>
#include "cuda-common.cuh"
#include "simple-ops.cuh"
#include "tensor.h"
#include "argmax.cuh"
#include "fattn.cuh"
#include "kvcache.h"
#include "profiler.h"
#include "qwen3.h"
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

_TIMING_RESULTS tmrs{};       // upstream's timing macros add into this global (src/profiler.h:43)

// Upstream allocates its activations anew in every forward pass and never checks an allocation
// (src/models/qwen3/qwen3.cpp:263-288, src/tensor.h:66-70); whether and when its stream-ordered frees give the
// memory back is the driver's business.  So before every pass this program checks that plenty is free and
// stops with a message otherwise, instead of letting a kernel write through a null pointer.
static double free_gb() {
    size_t f = 0, t = 0;
    cudaMemGetInfo(&f, &t);
    return (double)f / 1e9;
}
static void need_free(double gb, const char* where) {
    if (free_gb() < gb) {
        fprintf(stderr, "reference_runner: only %.1f GB free before %s (%.1f wanted): stopping\n", free_gb(), where, gb);
        exit(3);
    }
}

static std::vector<KVCache> make_caches(const Qwen3Config& c, int pages, int batch, int pages_per_seq, cudaDataType_t t) {
    std::vector<KVCache> caches;
    caches.reserve(c.num_hidden_layers);
    for (int i = 0; i < c.num_hidden_layers; ++i)
        caches.emplace_back(c.num_key_value_heads, c.head_dim, pages, batch, pages_per_seq, t);
    for (auto& kv : caches) kv.prepare_table(pages_per_seq * PAGE_SIZE);     // map every page up front
    return caches;
}

// Upper bound of what one forward pass over B x S tokens allocates (bf16): the activations of
// qwen3.cpp:263-288, four transposed copies per layer (qwen3.cpp:160-175), the logits, and as much again.
static double pass_gb(const Qwen3Config& c, int B, int S) {
    const double rows = (double)B * S, qd = (double)c.num_attention_heads * c.head_dim, kd = (double)c.num_key_value_heads * c.head_dim;
    const double once = rows * (3.0 * c.hidden_size + 2 * qd + 2 * kd + 2.0 * c.intermediate_size + c.vocab_size + 4.0 * c.head_dim);
    const double per_layer = rows * (2 * qd + 2 * kd + c.hidden_size);
    return 2.0 * 2.0 * (once + c.num_hidden_layers * per_layer) / 1e9 + 2.0;
}

static void dump_logits(FILE* f, const Tensor& logits) {
    size_t n = (size_t)logits.num_elements();
    std::vector<__nv_bfloat16> h(n);
    cudaStreamSynchronize(get_compute_stream());
    cudaMemcpy(h.data(), logits.data(), n * sizeof(__nv_bfloat16), cudaMemcpyDeviceToHost);
    std::vector<float> out(n);
    for (size_t i = 0; i < n; ++i) out[i] = __bfloat162float(h[i]);
    fwrite(out.data(), sizeof(float), n, f);
}

int main(int argc, char** argv) {
    if (argc < 2) { fprintf(stderr, "usage: reference_runner MODEL_DIR [options]\n"); return 2; }
    std::string dir = argv[1], ids_path, dump_path;
    int B = 1, S = 16, C = 0, K = 8, W = 0, R = 0;
    for (int i = 2; i + 1 < argc; i += 2) {
        std::string a = argv[i]; const char* v = argv[i + 1];
        if (a == "--batch") B = atoi(v); else if (a == "--prompt-len") S = atoi(v); else if (a == "--chunk") C = atoi(v);
        else if (a == "--steps") K = atoi(v); else if (a == "--warmup") W = atoi(v); else if (a == "--ids") ids_path = v;
        else if (a == "--dump") dump_path = v; else if (a == "--prefill-repeats") R = atoi(v);
        else { fprintf(stderr, "unknown option %s\n", a.c_str()); return 2; }
    }
    if (C <= 0) C = S;
    if (S % C) { fprintf(stderr, "--chunk must divide --prompt-len\n"); return 2; }

    Qwen3Config config = Qwen3Config::from_pretrained(dir);
    if ((long long)B * C * config.vocab_size >= (1LL << 31)) {
        fprintf(stderr, "[B,chunk,vocab] logits would pass 2^31 elements (upstream counts in int): use a smaller --chunk\n");
        return 2;
    }
    std::unique_ptr<Qwen3> model = Qwen3::from_pretrained(config);
    const cudaDataType_t T = model->lm_head.dtype();
    const int total = S + W + K;
    const int pages_per_seq = (total + PAGE_SIZE - 1) / PAGE_SIZE + 1;
    const int pages = B * pages_per_seq;

    std::vector<uint32_t> ids((size_t)B * total);
    if (!ids_path.empty()) {
        FILE* f = fopen(ids_path.c_str(), "rb");
        if (!f || fread(ids.data(), 4, ids.size(), f) != ids.size()) { fprintf(stderr, "cannot read %s\n", ids_path.c_str()); return 2; }
        fclose(f);
    } else {
        uint64_t s = 0x9E3779B97F4A7C15ull;
        for (auto& t : ids) { s = s * 6364136223846793005ull + 1442695040888963407ull; t = (uint32_t)((s >> 33) % (uint64_t)config.vocab_size); }
    }
    FILE* dump = dump_path.empty() ? nullptr : fopen(dump_path.c_str(), "wb");
    FlashAttnEngine engine(B, config.num_attention_heads, config.num_key_value_heads, config.head_dim, pages, pages_per_seq);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);

    // ---- whole prompts, timed alone (fresh caches each repeat; the first repeat is a warm-up) ----
    std::vector<float> prefill_ms;
    for (int r = 0; r < R; ++r) {
        std::vector<KVCache> caches = make_caches(config, pages, B, pages_per_seq, T);
        engine.get_graph(S, T);
        Tensor x({B, S}, CUDA_R_32U, 0);
        std::vector<uint32_t> xs((size_t)B * S);
        for (int b = 0; b < B; ++b) std::copy_n(&ids[(size_t)b * total], S, &xs[(size_t)b * S]);
        x.set_data<uint32_t>(xs, 4 * xs.size());
        Tensor pos({B, S}, CUDA_R_32U);
        arrange(pos, 0, 1);
        cudaStreamSynchronize(get_compute_stream());
        need_free(pass_gb(config, B, S), "a whole-prompt pass");
        cudaEventRecord(e0, get_compute_stream());
        for (auto& kv : caches) kv.prepare_table(S);
        Tensor logits = model->forward(x, pos, caches, engine);
        auto ret = argmax(logits, x);
        cudaEventRecord(e1, get_compute_stream());
        cudaEventSynchronize(e1);
        float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
        prefill_ms.push_back(ms);
    }

    // ---- prompts (in chunks), then one token per sequence and step ----
    std::vector<KVCache> caches = make_caches(config, pages, B, pages_per_seq, T);
    engine.get_graph(C, T);
    std::vector<uint32_t> last(B);
    for (int c0 = 0; c0 < S; c0 += C) {
        Tensor x({B, C}, CUDA_R_32U, 0);
        std::vector<uint32_t> xs((size_t)B * C);
        for (int b = 0; b < B; ++b) std::copy_n(&ids[(size_t)b * total + c0], C, &xs[(size_t)b * C]);
        x.set_data<uint32_t>(xs, 4 * xs.size());
        Tensor pos({B, C}, CUDA_R_32U);
        arrange(pos, c0, 1);
        need_free(pass_gb(config, B, C), "a prompt chunk");
        for (auto& kv : caches) kv.prepare_table(C);
        Tensor logits = model->forward(x, pos, caches, engine);
        if (dump) dump_logits(dump, logits);
        auto ret = argmax(logits, x);
        for (int b = 0; b < B; ++b) last[b] = ret[(size_t)b * C + C - 1];
        // upstream frees its per-pass buffers with cudaFreeAsync on its load stream and never synchronises that
        // stream, so the driver gives nothing back; between prompt chunks (argmax has just drained the compute
        // stream, and the decode loop below is left as upstream runs it) this wait lets the frees take effect
        cudaStreamSynchronize(get_load_offload_stream());
    }
    const double free_after_prompt = free_gb();
    Tensor x({B, 1}, CUDA_R_32U, 0);
    engine.get_graph(1, T);
    float dev_ms = 0;
    double wall_ms = 0;
    auto t0 = std::chrono::high_resolution_clock::now();
    for (int j = 0; j < W + K; ++j) {
        if (j == W) {
            cudaStreamSynchronize(get_compute_stream());
            t0 = std::chrono::high_resolution_clock::now();
            cudaEventRecord(e0, get_compute_stream());
        }
        if (!ids_path.empty()) for (int b = 0; b < B; ++b) last[b] = ids[(size_t)b * total + S + j];
        if (j == 0 || !ids_path.empty()) x.set_data<uint32_t>(last, 4 * (size_t)B);   // later steps: argmax wrote x in place
        Tensor pos({B, 1}, CUDA_R_32U, 0);
        std::vector<uint32_t> p(B, (uint32_t)(S + j));
        pos.set_data<uint32_t>(p, 4 * (size_t)B);
        if (j % 16 == 0) need_free(pass_gb(config, B, 1), "a decode step");
        for (auto& kv : caches) kv.prepare_table(1);
        Tensor logits = model->forward(x, pos, caches, engine);
        if (dump) dump_logits(dump, logits);
        auto ret = argmax(logits, x);
        for (int b = 0; b < B; ++b) last[b] = ret[b];
    }
    if (K > 0) {
        cudaEventRecord(e1, get_compute_stream());
        cudaEventSynchronize(e1);
        cudaEventElapsedTime(&dev_ms, e0, e1);
        wall_ms = std::chrono::duration<double, std::milli>(std::chrono::high_resolution_clock::now() - t0).count();
    }
    if (dump) fclose(dump);
    const double free_at_end = free_gb();
    cudaError_t err = cudaDeviceSynchronize();
    printf("{\"batch\": %d, \"prompt_len\": %d, \"chunk\": %d, \"steps\": %d, \"warmup\": %d, \"layers\": %d, "
           "\"decode_ms_per_step\": %.6f, \"decode_wall_ms_per_step\": %.6f, \"h2d_bytes_per_step\": %lld, "
           "\"d2h_bytes_per_step\": %d, \"last_token\": %u, \"cuda_error\": \"%s\", \"free_gb_after_prompt\": %.2f, "
           "\"free_gb_at_end\": %.2f, \"prefill_ms\": [",
           B, S, C, K, W, config.num_hidden_layers, K ? dev_ms / K : 0.0, K ? wall_ms / K : 0.0,
           (long long)config.num_hidden_layers * B * pages_per_seq * 4 + 4LL * B, 4 * B, last[0], cudaGetErrorString(err), free_after_prompt, free_at_end);
    for (size_t i = 0; i < prefill_ms.size(); ++i) printf("%s%.4f", i ? ", " : "", prefill_ms[i]);
    printf("]}\n");
    return err == cudaSuccess ? 0 : 1;
}
