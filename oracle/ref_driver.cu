// TEST INFRASTRUCTURE — a thin driver around the UNMODIFIED reference inference sources.
//
// It is compiled together with the reference's own files (see oracle/Makefile; the sources
// are used where they lie, nothing is copied) into oracle/_ref/ref_driver and calls the
// reference's public functions exactly as its main() does (inference/src/main.cpp:97-197):
// cublasCreate + TF32 math mode, qwen_load, expert_alloc + checkpoint_load, qwen_forward,
// qwen_reset. It replaces only the tokenizer/text part of main() with token-id files so
// that seeded prompts can be fed and raw logits / hidden states written out.
//
// usage: ref_driver --model DIR [--expert BIN --expert-scale F] --max-seq N
//                   --tokens FILE.i32 --prompt-len P --new N --out PREFIX
//                   [--teacher] [--all-logits] [--hidden] [--time REPS] [--seqs K]
// FILE.i32 holds P prompt ids, then (with --teacher) N ids to feed instead of the greedy pick; with
// --seqs K it holds K such records back to back and the sequences run one after the other with
// qwen_reset in between (the reference has no batching), their outputs concatenated.
// writes PREFIX.logits.f32  [K][(P or 1) + N, V] rows: prompt rows (all or last), then one per decode step
//        PREFIX.tokens.i32  [K][1 + N]           greedy pick after the prompt and after every step
//        PREFIX.hidden.bf16 [L, P, H]            residual stream after each layer for the first prompt
//        PREFIX.time.json                       decode timing of the reference's own loop
#include "backend/cuda_ops.h"
#include "backend/memory.h"
#include "model/qwen.h"
#include "model/expert.h"
#include "io/checkpoint.h"
#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

static const char* flag(int argc, char** argv, const char* f, const char* def = "") {
    for (int i = 1; i < argc - 1; ++i)
        if (!strcmp(argv[i], f)) return argv[i + 1];
    return def;
}
static bool sw(int argc, char** argv, const char* f) {
    for (int i = 1; i < argc; ++i)
        if (!strcmp(argv[i], f)) return true;
    return false;
}
static int greedy(const float* lg, int V) {  // inference/src/main.cpp:45-51
    int best = 0;
    for (int i = 1; i < V; ++i)
        if (lg[i] > lg[best]) best = i;
    return best;
}
static void dump(const std::string& path, const void* p, size_t bytes) {
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) { perror(path.c_str()); exit(1); }
    fwrite(p, 1, bytes, f);
    fclose(f);
}

int main(int argc, char** argv) {
    std::string dir = flag(argc, argv, "--model"), ex = flag(argc, argv, "--expert");
    std::string tokf = flag(argc, argv, "--tokens"), out = flag(argc, argv, "--out");
    float scale = atof(flag(argc, argv, "--expert-scale", "0.1"));
    int max_seq = atoi(flag(argc, argv, "--max-seq", "2048"));
    int P = atoi(flag(argc, argv, "--prompt-len", "0"));
    int N = atoi(flag(argc, argv, "--new", "0"));
    int reps = atoi(flag(argc, argv, "--time", "0"));
    int nseq = atoi(flag(argc, argv, "--seqs", "1"));
    bool teacher = sw(argc, argv, "--teacher"), all = sw(argc, argv, "--all-logits"), hid = sw(argc, argv, "--hidden");
    if (dir.empty() || tokf.empty() || out.empty() || P <= 0) {
        fprintf(stderr, "ref_driver: --model --tokens --prompt-len --out are required\n");
        return 2;
    }
    std::vector<int32_t> toks;
    {
        FILE* f = fopen(tokf.c_str(), "rb");
        if (!f) { perror(tokf.c_str()); return 2; }
        fseek(f, 0, SEEK_END);
        long n = ftell(f) / 4;
        fseek(f, 0, SEEK_SET);
        toks.resize(n);
        if (fread(toks.data(), 4, n, f) != (size_t)n) return 2;
        fclose(f);
    }
    const int rec = P + (teacher ? N : 0);
    if (nseq < 1 || (int)toks.size() < nseq * rec) { fprintf(stderr, "token file too short\n"); return 2; }

    cublasHandle_t cublas;
    CUBLAS_CHECK(cublasCreate(&cublas));
    CUBLAS_CHECK(cublasSetMathMode(cublas, CUBLAS_TF32_TENSOR_OP_MATH));

    model::QwenModel mdl;
    model::qwen_load(mdl, dir, max_seq);
    model::ExpertModel expert;
    bool has_expert = !ex.empty();
    if (has_expert) {
        model::expert_alloc(expert, mdl.cfg.num_layers, mdl.cfg.hidden_size, mdl.cfg.intermediate_size, max_seq);
        io::checkpoint_load(ex, expert);
        expert.output_scale = scale;
    }
    const model::ExpertModel* ep = has_expert ? &expert : nullptr;
    int V = mdl.cfg.vocab_size, H = mdl.cfg.hidden_size, L = mdl.cfg.num_layers;

    int32_t* d_tokens = (int32_t*)backend::device_alloc((size_t)max_seq * 4);
    float* d_logits = (float*)backend::device_alloc((size_t)P * V * 4);
    std::vector<float> row(V);

    if (hid) {
        // qwen_forward loops l < cfg.num_layers and leaves the residual stream in h_work
        // (inference/src/model/qwen.cu:310, include/model/qwen.h:72): run the prompt with the
        // layer count cut to k = 1..L and read h_work each time.
        std::vector<uint16_t> hbuf((size_t)L * P * H);
        backend::host_to_device(d_tokens, toks.data(), (size_t)P * 4);
        for (int k = 1; k <= L; ++k) {
            mdl.cfg.num_layers = k;
            model::qwen_reset(mdl);
            model::qwen_forward(mdl, cublas, d_tokens, P, ep, d_logits);
            backend::device_to_host(&hbuf[(size_t)(k - 1) * P * H], mdl.h_work, (size_t)P * H * 2);
        }
        mdl.cfg.num_layers = L;
        dump(out + ".hidden.bf16", hbuf.data(), hbuf.size() * 2);
    }

    // prompt + decode, as main.cpp:159-197 (no EOS break, no text), one sequence after the other
    std::vector<float> logits;
    std::vector<int32_t> picks;
    int next = 0;
    for (int q = 0; q < nseq; ++q) {
        const int32_t* tk = toks.data() + (size_t)q * rec;
        model::qwen_reset(mdl);
        backend::host_to_device(d_tokens, tk, (size_t)P * 4);
        model::qwen_forward(mdl, cublas, d_tokens, P, ep, d_logits);
        if (all) {
            const size_t at = logits.size();
            logits.resize(at + (size_t)P * V);
            backend::device_to_host(&logits[at], d_logits, (size_t)P * V * 4);
            memcpy(row.data(), &logits[at + (size_t)(P - 1) * V], (size_t)V * 4);
        } else {
            backend::device_to_host(row.data(), d_logits + (size_t)(P - 1) * V, (size_t)V * 4);
            logits.insert(logits.end(), row.begin(), row.end());
        }
        next = greedy(row.data(), V);
        picks.push_back(next);
        for (int s = 0; s < N; ++s) {
            int32_t one = teacher ? tk[P + s] : next;
            backend::host_to_device(d_tokens, &one, 4);
            model::qwen_forward(mdl, cublas, d_tokens, 1, ep, d_logits);
            backend::device_to_host(row.data(), d_logits, (size_t)V * 4);
            logits.insert(logits.end(), row.begin(), row.end());
            next = greedy(row.data(), V);
            picks.push_back(next);
        }
    }
    dump(out + ".logits.f32", logits.data(), logits.size() * 4);
    dump(out + ".tokens.i32", picks.data(), picks.size() * 4);

    if (reps > 0) {
        // time the reference's own decode loop: H2D token, forward, D2H logits, host argmax
        double best_ms = 1e30, sum_ms = 0, prefill_ms = 0;
        for (int r = 0; r < reps; ++r) {
            model::qwen_reset(mdl);
            backend::host_to_device(d_tokens, toks.data(), (size_t)P * 4);
            cudaDeviceSynchronize();
            auto p0 = std::chrono::steady_clock::now();
            model::qwen_forward(mdl, cublas, d_tokens, P, ep, d_logits);
            backend::device_to_host(row.data(), d_logits + (size_t)(P - 1) * V, (size_t)V * 4);
            auto p1 = std::chrono::steady_clock::now();
            prefill_ms = std::chrono::duration<double, std::milli>(p1 - p0).count();
            next = greedy(row.data(), V);
            auto t0 = std::chrono::steady_clock::now();
            for (int s = 0; s < N; ++s) {
                int32_t one = next;
                backend::host_to_device(d_tokens, &one, 4);
                model::qwen_forward(mdl, cublas, d_tokens, 1, ep, d_logits);
                backend::device_to_host(row.data(), d_logits, (size_t)V * 4);
                next = greedy(row.data(), V);
            }
            auto t1 = std::chrono::steady_clock::now();
            double ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
            best_ms = ms < best_ms ? ms : best_ms;
            sum_ms += ms;
        }
        FILE* f = fopen((out + ".time.json").c_str(), "w");
        fprintf(f, "{\"prompt_len\": %d, \"new_tokens\": %d, \"reps\": %d, \"decode_ms_best\": %.4f, "
                   "\"decode_ms_mean\": %.4f, \"prefill_ms_last\": %.4f, \"expert\": %s}\n",
                P, N, reps, best_ms, sum_ms / reps, prefill_ms, has_expert ? "true" : "false");
        fclose(f);
    }

    backend::device_free(d_tokens);
    backend::device_free(d_logits);
    if (has_expert) model::expert_free(expert);
    model::qwen_free(mdl);
    cublasDestroy(cublas);
    return 0;
}
