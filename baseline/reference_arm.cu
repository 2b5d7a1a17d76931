// A main() for the UNMODIFIED taejuk/mini-llm sources (copied to baseline/_ref): it is compiled
// together with the reference's own src/kernels/*.cu and src/model/*.cu and drives nothing but
// the reference's public model API, GPT2Model::get().prefill / decode and the logits hooks
// prefill_logits_for_test / decode_logits_for_test (include/model/gpt2_model.cuh:84-109), the
// way its own benches do (benchmarks/gpt2/bench_batch_vs_single_wall.cu:52-176: requests with
// sequential block ids per layer, prefill, then decode steps with the scheduler's bookkeeping).
// No file of this engine is compiled or loaded here.
//
//   reference_arm decode  PROMPTS.txt STEPS WARMUP   time STEPS decode steps after WARMUP untimed ones
//   reference_arm prefill PROMPTS.txt ITERS WARMUP   time prefill of all prompts as one batch
//   reference_arm logits  PROMPTS.txt OUT_DIR        last-token logits of the prefill and of one decode step
//
// PROMPTS.txt: one request per line, token ids separated by blanks (the reference's wire format,
// src/runtime/server.cpp:271-306).  Limits of the reference are checked here before anything runs:
// at most MAX_BATCH_NUM requests, MAX_SEQ positions, DEFAULT_TOTAL_KV_BLOCKS blocks
// (include/constants.h:16-26).  Each mode prints one JSON line.
#include "constants.h"
#include "model/gpt2_model.cuh"
#include "runtime/request.h"
#include "runtime/response.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

namespace C = mini_llm::constants;
namespace Rt = mini_llm::runtime;
namespace Model = mini_llm::model;

namespace {

void check(cudaError_t err, const char* what) {
    if (err != cudaSuccess) {
        std::fprintf(stderr, "reference_arm: %s failed: %s\n", what, cudaGetErrorString(err));
        std::exit(1);
    }
}

std::vector<std::vector<int>> read_prompts(const char* path) {
    std::ifstream in(path);
    if (!in) {
        std::fprintf(stderr, "reference_arm: cannot open %s\n", path);
        std::exit(1);
    }
    std::vector<std::vector<int>> prompts;
    std::string line;
    while (std::getline(in, line)) {
        std::istringstream ss(line);
        std::vector<int> ids;
        long v;
        while (ss >> v) {
            if (v < 0 || v >= C::GPT2_VOCAB_SIZE) {
                std::fprintf(stderr, "reference_arm: token id %ld outside the vocabulary\n", v);
                std::exit(1);
            }
            ids.push_back(static_cast<int>(v));
        }
        if (!ids.empty()) prompts.push_back(std::move(ids));
    }
    if (prompts.empty() || static_cast<int>(prompts.size()) > C::MAX_BATCH_NUM) {
        std::fprintf(stderr, "reference_arm: %zu requests; the reference takes 1..%d\n", prompts.size(), C::MAX_BATCH_NUM);
        std::exit(1);
    }
    return prompts;
}

// Requests with block ids handed out in order, layer by layer, as the reference's benches do.
std::vector<std::unique_ptr<Rt::Request>> make_requests(const std::vector<std::vector<int>>& prompts, int new_tokens,
                                                        int id_base) {
    std::vector<std::unique_ptr<Rt::Request>> reqs;
    int next_block = 0;
    for (size_t i = 0; i < prompts.size(); ++i) {
        int total = static_cast<int>(prompts[i].size()) + new_tokens;
        if (total > C::MAX_SEQ) {
            std::fprintf(stderr, "reference_arm: request %zu needs %d positions, the reference has %d\n", i, total, C::MAX_SEQ);
            std::exit(1);
        }
        auto req = std::make_unique<Rt::Request>(id_base + static_cast<int>(i), prompts[i], new_tokens);
        int blocks = (total + C::DEFAULT_KV_BLOCK_SIZE - 1) / C::DEFAULT_KV_BLOCK_SIZE;
        for (int layer = 0; layer < C::GPT2_N_LAYERS; ++layer) {
            auto& kv = req->layer_kv[layer];
            kv.reset();
            for (int b = 0; b < blocks; ++b) kv.append_block(next_block++);
        }
        reqs.push_back(std::move(req));
    }
    if (next_block > C::DEFAULT_TOTAL_KV_BLOCKS) {
        std::fprintf(stderr, "reference_arm: %d KV blocks needed, the reference's pool has %d\n", next_block,
                     C::DEFAULT_TOTAL_KV_BLOCKS);
        std::exit(1);
    }
    return reqs;
}

// What the reference's scheduler does after a model call (src/runtime/scheduler.cpp:170-174, 237-239).
void after_prefill(std::vector<std::unique_ptr<Rt::Request>>& reqs, const std::vector<Rt::Response>& out) {
    for (size_t i = 0; i < reqs.size(); ++i) {
        for (auto& kv : reqs[i]->layer_kv) kv.set_num_tokens(reqs[i]->prompts_len);
        reqs[i]->tokens.push_back(i < out.size() ? out[i].token : 0);
    }
}

void after_decode(std::vector<std::unique_ptr<Rt::Request>>& reqs, const std::vector<Rt::Response>& out) {
    for (size_t i = 0; i < reqs.size(); ++i) {
        for (auto& kv : reqs[i]->layer_kv) kv.increment_tokens(1);
        reqs[i]->tokens.push_back(i < out.size() ? out[i].token : 0);
    }
}

double now_ms() {
    using Clock = std::chrono::steady_clock;
    return std::chrono::duration<double, std::milli>(Clock::now().time_since_epoch()).count();
}

// The warm-up is a generation by other requests of the same shape (their blocks are handed out again afterwards),
// so the timed steps start right after the timed requests' prompts are in: contexts prompt_len .. prompt_len+STEPS.
int run_decode(const char* path, int steps, int warmup) {
    auto prompts = read_prompts(path);
    auto& model = Model::GPT2Model::get();
    {
        auto warm = make_requests(prompts, warmup + 1, 1000);
        after_prefill(warm, model.prefill(warm));
        for (int i = 0; i < warmup; ++i) after_decode(warm, model.decode(warm));
    }
    auto reqs = make_requests(prompts, steps + 1, 2000);
    after_prefill(reqs, model.prefill(reqs));
    cudaEvent_t e0, e1;
    check(cudaEventCreate(&e0), "cudaEventCreate");
    check(cudaEventCreate(&e1), "cudaEventCreate");
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize(before)");
    int ctx0 = static_cast<int>(reqs[0]->tokens.size()) - 1;     // tokens in the cache before the first timed step
    double t0 = now_ms();
    check(cudaEventRecord(e0), "cudaEventRecord");
    for (int i = 0; i < steps; ++i) after_decode(reqs, model.decode(reqs));
    check(cudaEventRecord(e1), "cudaEventRecord");
    check(cudaEventSynchronize(e1), "cudaEventSynchronize");
    double wall = now_ms() - t0;
    float ms = 0.f;
    check(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
    check(cudaGetLastError(), "the reference's kernels");
    std::printf("{\"mode\": \"decode\", \"batch\": %zu, \"steps\": %d, \"warmup\": %d, \"first_context\": %d, "
                "\"device_ms_per_step\": %.6f, \"wall_ms_per_step\": %.6f, \"last_tokens\": [",
                reqs.size(), steps, warmup, ctx0, ms / steps, wall / steps);
    for (size_t i = 0; i < reqs.size(); ++i) std::printf("%s%d", i ? ", " : "", reqs[i]->tokens.back());
    std::printf("]}\n");
    return 0;
}

int run_prefill(const char* path, int iters, int warmup) {
    auto prompts = read_prompts(path);
    auto& model = Model::GPT2Model::get();
    size_t flush_bytes = size_t(256) << 20;                        // larger than the L2: every iteration starts cold
    void* flush = nullptr;
    check(cudaMalloc(&flush, flush_bytes), "cudaMalloc(flush)");
    cudaEvent_t e0, e1;
    check(cudaEventCreate(&e0), "cudaEventCreate");
    check(cudaEventCreate(&e1), "cudaEventCreate");
    std::vector<float> times;
    int tokens = 0;
    for (auto& p : prompts) tokens += static_cast<int>(p.size());
    for (int it = 0; it < warmup + iters; ++it) {
        auto reqs = make_requests(prompts, 0, 2000 + it * 100);
        check(cudaMemset(flush, it, flush_bytes), "cudaMemset(flush)");
        check(cudaDeviceSynchronize(), "cudaDeviceSynchronize(before)");
        check(cudaEventRecord(e0), "cudaEventRecord");
        (void)model.prefill(reqs);
        check(cudaEventRecord(e1), "cudaEventRecord");
        check(cudaEventSynchronize(e1), "cudaEventSynchronize");
        float ms = 0.f;
        check(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
        if (it >= warmup) times.push_back(ms);
    }
    check(cudaGetLastError(), "the reference's kernels");
    std::sort(times.begin(), times.end());
    std::printf("{\"mode\": \"prefill\", \"batch\": %zu, \"tokens\": %d, \"iters\": %d, \"warmup\": %d, \"median_ms\": %.6f}\n",
                prompts.size(), tokens, iters, warmup, times[times.size() / 2]);
    return 0;
}

void write_f32(const std::string& path, const std::vector<float>& v) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f || std::fwrite(v.data(), sizeof(float), v.size(), f) != v.size()) {
        std::fprintf(stderr, "reference_arm: cannot write %s\n", path.c_str());
        std::exit(1);
    }
    std::fclose(f);
}

// prefill.f32 [B, V]: logits at each prompt's last token; decode.f32 [B, V]: logits of the step that is fed the
// reference's own argmax of those; tokens.txt: that argmax and the next one, per request.
int run_logits(const char* path, const char* out_dir) {
    auto prompts = read_prompts(path);
    auto& model = Model::GPT2Model::get();
    auto reqs = make_requests(prompts, 2, 3000);
    std::vector<float> pre = model.prefill_logits_for_test(reqs);
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize(prefill)");
    std::vector<int> first(reqs.size());
    for (size_t i = 0; i < reqs.size(); ++i) {
        const float* row = pre.data() + i * static_cast<size_t>(C::GPT2_VOCAB_SIZE);
        int best = 0;
        for (int v = 1; v < C::GPT2_VOCAB_SIZE; ++v) if (row[v] > row[best]) best = v;
        first[i] = best;
        for (auto& kv : reqs[i]->layer_kv) kv.set_num_tokens(reqs[i]->prompts_len);
        reqs[i]->tokens.push_back(best);
    }
    std::vector<float> dec = model.decode_logits_for_test(reqs);
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize(decode)");
    check(cudaGetLastError(), "the reference's kernels");
    std::string dir(out_dir);
    write_f32(dir + "/prefill.f32", pre);
    write_f32(dir + "/decode.f32", dec);
    std::ofstream tk(dir + "/tokens.txt");
    for (size_t i = 0; i < reqs.size(); ++i) tk << first[i] << "\n";
    std::printf("{\"mode\": \"logits\", \"batch\": %zu, \"vocab\": %d}\n", reqs.size(), C::GPT2_VOCAB_SIZE);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc >= 5 && std::string(argv[1]) == "decode") {
        int steps = std::atoi(argv[3]), warmup = std::atoi(argv[4]);
        if (steps > 0 && warmup >= 0) return run_decode(argv[2], steps, warmup);
    } else if (argc >= 5 && std::string(argv[1]) == "prefill") {
        int iters = std::atoi(argv[3]), warmup = std::atoi(argv[4]);
        if (iters > 0 && warmup >= 0) return run_prefill(argv[2], iters, warmup);
    } else if (argc >= 4 && std::string(argv[1]) == "logits") {
        return run_logits(argv[2], argv[3]);
    }
    std::fprintf(stderr, "usage: reference_arm decode|prefill PROMPTS.txt N WARMUP | logits PROMPTS.txt OUT_DIR\n");
    return 2;
}
