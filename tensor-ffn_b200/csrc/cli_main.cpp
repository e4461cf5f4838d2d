// tensor-ffn-inference — the reference's command line (inference/src/main.cpp) on top of the
// C ABI of include/tffn.h. Same flags, defaults, stdout protocol and exit codes; a leading
// "inference" word is accepted so that `tensor-ffn inference --model ...` from the
// reference's README works too. Extra flags (not in the reference): --prompt-ids <file> (raw
// int32 ids instead of --prompt), --ignore-eos, --device <N>, --host-sampling (with --temperature: sample
// on the host from downloaded logits as the reference does, instead of on the device), --bpe (tokenise the
// prompt and print the output with the byte-level BPE that tokenizer.json specifies, instead of the
// reference's encoder, which drops spaces and newlines).
// The usage text, the flag scanning, the ChatML sequence, the stdout protocol and the host sampler
// are the reference's own (inference/src/main.cpp:17-63, 127-144, 157-198), reproduced on purpose:
// they ARE the command-line contract. What differs is what runs underneath: the six calls into the
// reference's model code are replaced by calls into the C ABI.
#include "../../include/tffn.h"
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

static void usage() {
    fprintf(stderr,
            "tensor-ffn-inference\n"
            "\n"
            "  --model        <dir>   HuggingFace model directory  (required)\n"
            "  --prompt       <str>   Input prompt                  (required)\n"
            "  --chat                 Enable ChatML formatting      (optional)\n"
            "  --expert       <path>  Expert .bin file              (optional)\n"
            "  --expert-scale <F>     Expert delta scale            (default 0.1)\n"
            "  --max-tokens   <N>     Tokens to generate            (default 128)\n"
            "  --temperature  <F>     Sampling temperature          (default 0 = greedy)\n"
            "  --max-seq      <N>     KV cache capacity             (default 2048)\n"
            "\n");
    exit(1);
}

// value = the argument after the flag; like the reference, the last argument is never taken
// as a flag name (inference/src/main.cpp:33-37)
static std::string get_flag(int argc, char** argv, const char* flag, const char* def = "") {
    for (int i = 1; i < argc - 1; ++i)
        if (strcmp(argv[i], flag) == 0) return argv[i + 1];
    return def;
}
static int get_flag_i(int argc, char** argv, const char* f, int d) {
    auto v = get_flag(argc, argv, f);
    return v.empty() ? d : atoi(v.c_str());
}
static float get_flag_f(int argc, char** argv, const char* f, float d) {
    auto v = get_flag(argc, argv, f);
    return v.empty() ? d : (float)atof(v.c_str());
}
static bool has_switch(int argc, char** argv, const char* f) {
    for (int i = 1; i < argc; ++i)
        if (strcmp(argv[i], f) == 0) return true;
    return false;
}

// temperature sampling exactly as inference/src/main.cpp:52-63 (double softmax, inverse CDF)
static int sample_temperature(const float* logits, int V, float temperature, std::mt19937& rng) {
    float maxv = logits[0];
    for (int i = 1; i < V; ++i) maxv = std::max(maxv, logits[i]);
    std::vector<double> probs(V);
    double sum = 0.0;
    for (int i = 0; i < V; ++i) {
        probs[i] = std::exp((logits[i] - maxv) / temperature);
        sum += probs[i];
    }
    std::uniform_real_distribution<double> dist(0.0, sum);
    double r = dist(rng), acc = 0.0;
    for (int i = 0; i < V; ++i) {
        acc += probs[i];
        if (acc >= r) return i;
    }
    return V - 1;
}

#define CHECK(call)                                          \
    do {                                                     \
        int rc_ = (call);                                    \
        if (rc_ < 0) {                                       \
            fprintf(stderr, "%s\n", tffn_last_error());      \
            return 1;                                        \
        }                                                    \
    } while (0)

int main(int argc, char** argv) {
    if (argc < 2) usage();
    std::string model_dir = get_flag(argc, argv, "--model");
    std::string prompt = get_flag(argc, argv, "--prompt");
    std::string expert_path = get_flag(argc, argv, "--expert");
    std::string ids_path = get_flag(argc, argv, "--prompt-ids");
    float expert_scale = get_flag_f(argc, argv, "--expert-scale", 0.1f);
    int max_new_tokens = get_flag_i(argc, argv, "--max-tokens", 128);
    float temperature = get_flag_f(argc, argv, "--temperature", 0.f);
    int max_seq = get_flag_i(argc, argv, "--max-seq", 2048);
    int device = get_flag_i(argc, argv, "--device", 0);
    bool use_chat = has_switch(argc, argv, "--chat");
    bool ignore_eos = has_switch(argc, argv, "--ignore-eos");
    bool bpe = has_switch(argc, argv, "--bpe");

    if (model_dir.empty() || (prompt.empty() && ids_path.empty())) {
        fprintf(stderr, "--model and --prompt are required\n");
        usage();
    }

    tffn_tokenizer* tok = nullptr;
    CHECK(tffn_tokenizer_load(model_dir.c_str(), &tok));
    tffn_model* mdl = nullptr;
    CHECK(tffn_model_load(model_dir.c_str(), device, 0, 1, &mdl));
    tffn_config cfg;
    CHECK(tffn_model_config(mdl, &cfg));
    printf("Model loaded: %d layers, hidden=%d, vocab=%d\n", cfg.num_layers, cfg.hidden_size, cfg.vocab_size);

    tffn_expert* expert = nullptr;
    if (!expert_path.empty()) {
        CHECK(tffn_expert_load(mdl, expert_path.c_str(), expert_scale, &expert));
        printf("Expert loaded from %s  (scale=%.4f)\n", expert_path.c_str(), expert_scale);
    } else {
        printf("No expert — running base model only.\n");
    }

    std::vector<uint32_t> prompt_ids;
    auto push_text = [&](const std::string& text) {
        auto enc = bpe ? tffn_tokenizer_encode_bpe : tffn_tokenizer_encode;
        int n = enc(tok, text.c_str(), nullptr, 0);
        if (n <= 0) return;
        size_t o = prompt_ids.size();
        prompt_ids.resize(o + n);
        enc(tok, text.c_str(), prompt_ids.data() + o, n);
    };
    auto push_special = [&](const char* name) {
        uint32_t id = 0;
        tffn_tokenizer_token_id(tok, name, &id);
        prompt_ids.push_back(id);
    };
    if (!ids_path.empty()) {
        FILE* f = fopen(ids_path.c_str(), "rb");
        if (!f) { fprintf(stderr, "Cannot open %s\n", ids_path.c_str()); return 1; }
        int32_t v;
        while (fread(&v, 4, 1, f) == 1) prompt_ids.push_back((uint32_t)v);
        fclose(f);
        if (prompt.empty()) prompt = "<" + ids_path + ">";
    } else if (use_chat) {
        // ChatML template of inference/src/main.cpp:127-144
        push_special("<|im_start|>");
        push_text("system\nYou are a helpful coding assistant.");
        push_special("<|im_end|>");
        push_text("\n");
        push_special("<|im_start|>");
        push_text("user\n" + prompt);
        push_special("<|im_end|>");
        push_text("\n");
        push_special("<|im_start|>");
        push_text("assistant\n");
    } else {
        push_text(prompt);
    }
    if (prompt_ids.empty()) { fprintf(stderr, "Prompt encoded to zero tokens.\n"); return 1; }
    int prompt_len = (int)prompt_ids.size();
    if (prompt_len > max_seq - 1) {
        fprintf(stderr, "Prompt too long (%d tokens, max %d).\n", prompt_len, max_seq - 1);
        return 1;
    }
    printf("\nPrompt (%d tokens): %s\n", prompt_len, prompt.c_str());

    tffn_session* sess = nullptr;
    CHECK(tffn_session_create(mdl, expert, 1, max_seq, nullptr, &sess));
    uint32_t eos = 151645;
    tffn_tokenizer_special(tok, &eos, nullptr, nullptr);

    std::vector<int32_t> h_tokens(prompt_ids.begin(), prompt_ids.end());
    const int V = cfg.vocab_size;
    // Temperature sampling runs on the device with the reference's arithmetic and its mt19937(42) stream
    // (tffn_session_set_sampling); --host-sampling keeps the reference's host loop over a downloaded
    // logits row instead (608 KB per token), for cross-checks.
    const bool host_sampling = temperature > 0.f && has_switch(argc, argv, "--host-sampling");
    if (temperature > 0.f && !host_sampling) CHECK(tffn_session_set_sampling(sess, temperature, 42));
    std::vector<float> h_logits(host_sampling ? V : 0);
    printf("\nGenerating:\n");
    fflush(stdout);

    int32_t next = 0;
    CHECK(tffn_prefill(sess, h_tokens.data(), &prompt_len, 1, &next, host_sampling ? h_logits.data() : nullptr));
    std::mt19937 rng(42);
    if (host_sampling) next = sample_temperature(h_logits.data(), V, temperature, rng);

    for (int step = 0; step < max_new_tokens; ++step) {
        if (!ignore_eos && next == (int32_t)eos) break;
        if (tffn_session_seq_len(sess, 0) >= max_seq) {
            fprintf(stderr, "\nKV cache overflow — increase --max-seq\n");
            break;
        }
        char text[512];
        uint32_t id = (uint32_t)next;
        (bpe ? tffn_tokenizer_decode_bpe : tffn_tokenizer_decode)(tok, &id, 1, text, sizeof text);
        printf("%s", text);
        fflush(stdout);
        int32_t fed = next;
        CHECK(tffn_decode_step(sess, &fed, 1, &next, host_sampling ? h_logits.data() : nullptr));
        if (host_sampling) next = sample_temperature(h_logits.data(), V, temperature, rng);
    }
    printf("\n");

    tffn_session_free(sess);
    tffn_expert_free(expert);
    tffn_model_free(mdl);
    tffn_tokenizer_free(tok);
    return 0;
}
