// Benchmark driver for the reference engine (BusyaPrime/from-scratch-inference-engine-), built by
// baseline/build_reference.py against the reference's own, unmodified sources.  It follows the
// reference's harness (benchmarks/harness/bench_cuda.cpp:43-93: synthetic token ids, a warm-up
// forward, wall-clock timing around calls that end in a device synchronisation) but drives the
// batched path: CudaEngine::step -> CudaModel::forward_batch_argmax (src/cuda/engine.cu:39-119,
// src/cuda/model.cu:573-625), which is how the reference decodes several requests at once.
//
//   ref_bench MODEL_DIR BATCH CONTEXT STEPS WARMUP PREFILL_TOKENS
//
// BATCH requests with prompts of CONTEXT - (STEPS + WARMUP) tokens are prefilled in the engine's
// first step; WARMUP untimed decode steps follow, then STEPS timed ones, whose contexts end at
// CONTEXT.  Every step of the reference engine copies token ids to the device and reads the
// chosen tokens back after a device synchronisation, so its wall time is both the device time
// and the end-to-end time.  One prompt of PREFILL_TOKENS tokens is then timed through
// CudaModel::forward_with_cache, as bench_cuda does for its time to first token.
// Prints one JSON object on the last line of standard output.
//
// The checkpoint is mapped into memory and handed to the reference's own parser
// (SafeTensors::parse, then CudaModel::from_safetensors: both public): SafeTensors::load reads
// the file one character at a time, which takes minutes for 15 GB.
#include "engine/cuda/engine.hpp"
#include "engine/cuda/kv_cache.hpp"
#include "engine/cuda/model.hpp"
#include "engine/model_config.hpp"
#include "engine/safetensors.hpp"

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <fcntl.h>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

namespace {

using Clock = std::chrono::steady_clock;

double seconds_since(Clock::time_point start) {
    return std::chrono::duration<double>(Clock::now() - start).count();
}

std::string read_text(const std::string& path) {
    std::ifstream f(path);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::stringstream s;
    s << f.rdbuf();
    return s.str();
}

// Uniform token ids from a fixed linear congruential sequence.
std::vector<int64_t> token_ids(int64_t n, int64_t vocab, uint64_t seed) {
    std::vector<int64_t> ids(static_cast<std::size_t>(n));
    uint64_t state = seed * 6364136223846793005ULL + 1442695040888963407ULL;
    for (auto& id : ids) {
        state = state * 6364136223846793005ULL + 1442695040888963407ULL;
        id = static_cast<int64_t>((state >> 33) % static_cast<uint64_t>(vocab));
    }
    return ids;
}

engine::cuda::CudaModel load_model(const std::string& dir) {
    engine::ModelConfig config = engine::ModelConfig::from_json(read_text(dir + "/config.json"));
    const std::string path = dir + "/model.safetensors";
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) throw std::runtime_error("cannot open " + path);
    struct stat st {};
    if (::fstat(fd, &st) != 0) throw std::runtime_error("cannot stat " + path);
    void* data = ::mmap(nullptr, static_cast<std::size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    if (data == MAP_FAILED) throw std::runtime_error("cannot map " + path);
    engine::cuda::CudaModel model = engine::cuda::CudaModel::from_safetensors(
        std::move(config),
        engine::SafeTensors::parse(static_cast<const uint8_t*>(data), static_cast<std::size_t>(st.st_size)));
    ::munmap(data, static_cast<std::size_t>(st.st_size));
    ::close(fd);
    return model;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc < 7) {
        std::fprintf(stderr, "usage: ref_bench MODEL_DIR BATCH CONTEXT STEPS WARMUP PREFILL_TOKENS\n");
        return 2;
    }
    try {
        const std::string dir = argv[1];
        const int64_t batch = std::atoll(argv[2]), context = std::atoll(argv[3]);
        const int64_t steps = std::atoll(argv[4]), warmup = std::atoll(argv[5]);
        const int64_t prefill_tokens = std::atoll(argv[6]);
        if (batch <= 0 || steps <= 0 || warmup < 0 || context <= steps + warmup) {
            std::fprintf(stderr, "ref_bench: need batch, steps > 0 and context > steps + warmup\n");
            return 2;
        }
        Clock::time_point t0 = Clock::now();
        const engine::cuda::CudaModel model = load_model(dir);
        const engine::ModelConfig& c = model.config();
        const double load_s = seconds_since(t0);
        std::fprintf(stderr, "ref_bench: model loaded in %.1f s\n", load_s);
        const int64_t kv_dim = c.num_key_value_heads * c.head_dim;
        {   // libraries initialise and kernels load outside the measurement (bench_cuda.cpp:57-62)
            engine::cuda::GpuKVCache warm(c.num_hidden_layers, kv_dim, 8);
            (void)model.forward_with_cache({0, 1}, warm);
        }

        double decode_s = 0.0, fill_s = 0.0;
        int64_t produced = 0;
        if (steps > 0) {
            engine::cuda::CudaEngine eng(model, 0, batch);
            engine::SamplingParams greedy;
            greedy.temperature = 0.0;
            const int64_t prompt_len = context - (steps + warmup);
            std::vector<int64_t> ids;
            for (int64_t r = 0; r < batch; ++r) {
                engine::Request request;
                request.prompt = token_ids(prompt_len, c.vocab_size, static_cast<uint64_t>(r) + 1);
                request.params = greedy;
                request.max_tokens = steps + warmup + 1;
                ids.push_back(eng.add_request(std::move(request)));
            }
            t0 = Clock::now();
            eng.step();                                   // prefill of all requests
            fill_s = seconds_since(t0);
            std::fprintf(stderr, "ref_bench: %lld prompts of %lld tokens prefilled in %.1f s\n",
                         static_cast<long long>(batch), static_cast<long long>(prompt_len), fill_s);
            for (int64_t i = 0; i < warmup; ++i) eng.step();
            t0 = Clock::now();
            for (int64_t i = 0; i < steps; ++i) eng.step();
            decode_s = seconds_since(t0);
            for (const int64_t id : ids) produced += static_cast<int64_t>(eng.output(id).size());
            if (produced != batch * (steps + warmup + 1))
                throw std::runtime_error("the engine did not produce one token per request and step");
        }

        double prefill_s = 0.0;
        if (prefill_tokens > 0) {
            engine::cuda::GpuKVCache cache(c.num_hidden_layers, kv_dim, prefill_tokens + 1);
            const std::vector<int64_t> prompt = token_ids(prefill_tokens, c.vocab_size, 99);
            t0 = Clock::now();
            (void)model.forward_with_cache(prompt, cache);
            prefill_s = seconds_since(t0);
        }
        std::printf("{\"batch\": %lld, \"context\": %lld, \"steps\": %lld, \"warmup\": %lld, "
                    "\"ms_per_step\": %.6f, \"decode_tokens_per_s\": %.6f, \"load_s\": %.3f, "
                    "\"fill_s\": %.3f, \"prefill_tokens\": %lld, \"prefill_ms\": %.3f, "
                    "\"layers\": %lld, \"hidden\": %lld, \"vocab\": %lld}\n",
                    static_cast<long long>(batch), static_cast<long long>(context),
                    static_cast<long long>(steps), static_cast<long long>(warmup),
                    decode_s * 1000.0 / static_cast<double>(steps),
                    static_cast<double>(batch * steps) / decode_s, load_s, fill_s,
                    static_cast<long long>(prefill_tokens), prefill_s * 1000.0,
                    static_cast<long long>(c.num_hidden_layers), static_cast<long long>(c.hidden_size),
                    static_cast<long long>(c.vocab_size));
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ref_bench: %s\n", e.what());
        return 1;
    }
}
