// Drives the unmodified reference engine (xissleah/Citlali-LLM-Engine) through its own public
// class citlali::model::QwenModel (include/citlali/model/qwen_model.h:38-42: load, forward_token)
// for two purposes:
//
//   logits  every token of every given sequence is fed at its position with compute_logits=true
//           and the model's logits buffer is written out: [tokens, vocab] little-endian float32.
//           The buffer is a private member (qwen_model.h:76); this translation unit alone reads
//           the header with `private` spelled `public`.  Nothing of the reference is edited and
//           the library it links is the stock build.
//   decode  the reference's generation loop for one sequence (src/runtime/session.cpp:69-92):
//           the prompt token by token without logits, then greedy tokens fed back one by one;
//           the last `steps` of them are timed on the host clock around forward_token, which
//           itself synchronises the device before it reads the logits (qwen_model.cpp:448-450).
//           --start-position P begins at position P instead of 0 (to time steps near the end of a long
//           context without the minutes its token-by-token prompt loop takes).
//
// Token ids come from files and go to files: the reference's tokenizer is not involved.
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#define private public
#include "citlali/model/qwen_model.h"
#undef private
#include "citlali/io/gguf_reader.h"

namespace {

std::vector<std::vector<int32_t>> read_sequences(const std::string& path) {
    std::ifstream in(path);
    if (!in) throw std::runtime_error("cannot open " + path);
    std::vector<std::vector<int32_t>> out;
    std::string line;
    while (std::getline(in, line)) {
        std::istringstream fields(line);
        std::vector<int32_t> ids;
        long long v;
        while (fields >> v) ids.push_back(static_cast<int32_t>(v));
        if (!ids.empty()) out.push_back(ids);
    }
    return out;
}

const char* option(int argc, char** argv, const char* name, const char* fallback) {
    for (int i = 2; i + 1 < argc; ++i) {
        if (std::strcmp(argv[i], name) == 0) return argv[i + 1];
    }
    return fallback;
}

int run_logits(int argc, char** argv) {
    const std::string model_path = option(argc, argv, "--model", "");
    const std::string tokens_path = option(argc, argv, "--tokens", "");
    const std::string out_path = option(argc, argv, "--out", "");
    const uint32_t ctx = static_cast<uint32_t>(std::atoi(option(argc, argv, "--ctx", "256")));
    citlali::io::GgufFile gguf;
    gguf.load(model_path);
    citlali::model::QwenModel model;
    model.load(gguf, ctx);
    const size_t vocab = model.config().vocab_size;
    std::vector<float> row(vocab);
    std::ofstream out(out_path, std::ios::binary);
    if (!out) throw std::runtime_error("cannot write " + out_path);
    size_t rows = 0;
    for (const auto& ids : read_sequences(tokens_path)) {
        // a new sequence starts at position 0: keys and values of the sequence before are overwritten
        // position by position before they are read again (attention reads positions <= p only)
        for (size_t p = 0; p < ids.size(); ++p) {
            model.forward_token(ids[p], static_cast<uint32_t>(p), true);
            model.logits_->copy_to_host(row.data(), vocab * sizeof(float));
            out.write(reinterpret_cast<const char*>(row.data()), static_cast<std::streamsize>(vocab * sizeof(float)));
            ++rows;
        }
    }
    std::printf("{\"rows\": %zu, \"vocab\": %zu}\n", rows, vocab);
    return 0;
}

int run_decode(int argc, char** argv) {
    const std::string model_path = option(argc, argv, "--model", "");
    const uint32_t ctx = static_cast<uint32_t>(std::atoi(option(argc, argv, "--ctx", "4096")));
    const int prompt = std::atoi(option(argc, argv, "--prompt-tokens", "16"));
    const int start = std::atoi(option(argc, argv, "--start-position", "0"));
    const int warmup = std::atoi(option(argc, argv, "--warmup", "3"));
    const int steps = std::atoi(option(argc, argv, "--steps", "20"));
    uint64_t state = static_cast<uint64_t>(std::atoll(option(argc, argv, "--seed", "1")));
    const auto t_load = std::chrono::steady_clock::now();
    citlali::io::GgufFile gguf;
    gguf.load(model_path);
    citlali::model::QwenModel model;
    model.load(gguf, ctx);
    const double load_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_load).count();
    const uint32_t vocab = model.config().vocab_size;
    if (static_cast<uint32_t>(start + prompt + warmup + steps) > model.max_context()) {
        throw std::runtime_error("start + prompt + warmup + steps exceed the context");
    }
    // forward_token takes the position as an argument (qwen_model.h:42).  Starting above 0 leaves the
    // cache below `start` as cudaMalloc returned it: the kernels' work depends on the position alone
    // (no value decides a branch or a trip count), so a step costs what it costs after a real prompt.
    uint32_t position = static_cast<uint32_t>(start);
    int32_t next = 0;
    const auto t_prompt = std::chrono::steady_clock::now();
    for (int i = 0; i < prompt; ++i) {
        state = state * 6364136223846793005ull + 1442695040888963407ull;       // ids uniform over the vocabulary
        const int32_t id = static_cast<int32_t>((state >> 33) % vocab);
        next = model.forward_token(id, position++, i == prompt - 1);
    }
    model.synchronize();
    const double prompt_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_prompt).count();
    for (int i = 0; i < warmup; ++i) next = model.forward_token(next, position++);
    model.synchronize();
    const uint32_t first_timed = position;
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < steps; ++i) next = model.forward_token(next, position++);
    model.synchronize();
    const double seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    std::printf("{\"steps\": %d, \"warmup\": %d, \"prompt_tokens\": %d, \"start_position\": %d, \"first_timed_position\": %u, "
                "\"last_timed_position\": %u, \"seconds\": %.6f, \"ms_per_step\": %.4f, \"tokens_per_second\": %.3f, "
                "\"prompt_seconds\": %.3f, \"load_seconds\": %.1f, \"last_token\": %d}\n",
                steps, warmup, prompt, start, first_timed, position - 1, seconds, 1e3 * seconds / steps, steps / seconds,
                prompt_s, load_s, next);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        if (argc >= 2 && std::strcmp(argv[1], "logits") == 0) return run_logits(argc, argv);
        if (argc >= 2 && std::strcmp(argv[1], "decode") == 0) return run_decode(argc, argv);
        std::fprintf(stderr, "usage: reference_harness logits --model M.gguf --ctx N --tokens ids.txt --out logits.f32\n"
                             "       reference_harness decode --model M.gguf --ctx N [--start-position S] --prompt-tokens P --warmup W --steps K\n");
        return 2;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
}
