// Driver for tests/golden/make_golden.py: runs the reference's own CPU model
// (BusyaPrime/from-scratch-inference-engine-, src/model/model.cpp) on a model folder and
// writes what the plain implementation of the tests is compared with.
//   ref_dump MODEL_DIR OUT_PREFIX id id id ...
// writes OUT_PREFIX.forward.f32   logits [S, V] of Model::forward(ids)
//        OUT_PREFIX.chunked.f32   logits [S, V] of forward_paged: first S-3 tokens in one
//                                 call, then one token per call (block size 4)
//        OUT_PREFIX.greedy.txt    8 greedy tokens of Engine::generate (block 4, 64 blocks)
#include "engine/engine.hpp"
#include "engine/model.hpp"
#include "engine/paged_kv_cache.hpp"

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

static void dump(const std::string& path, const engine::Tensor& t) {
    FILE* f = std::fopen(path.c_str(), "wb");
    std::fwrite(t.data(), sizeof(float), static_cast<size_t>(t.numel()), f);
    std::fclose(f);
}

int main(int argc, char** argv) {
    if (argc < 4) return 2;
    const std::string dir = argv[1], prefix = argv[2];
    std::vector<int64_t> ids;
    for (int i = 3; i < argc; ++i) ids.push_back(std::atoll(argv[i]));
    const engine::Model model = engine::Model::from_pretrained(dir);
    const engine::ModelConfig& c = model.config();

    dump(prefix + ".forward.f32", model.forward(ids));

    {
        const int64_t vocab = c.vocab_size;
        const int64_t s = static_cast<int64_t>(ids.size());
        engine::PagedKVCache cache(c.num_hidden_layers, c.num_key_value_heads * c.head_dim, 4, 64);
        engine::Tensor all({s, vocab});
        const int64_t head = s - 3;
        std::vector<int64_t> first(ids.begin(), ids.begin() + head);
        engine::Tensor a = model.forward_paged(first, cache);
        for (int64_t i = 0; i < a.numel(); ++i) all.data()[i] = a.data()[i];
        for (int64_t t = head; t < s; ++t) {
            engine::Tensor b = model.forward_paged({ids[static_cast<size_t>(t)]}, cache);
            for (int64_t i = 0; i < vocab; ++i) all.data()[t * vocab + i] = b.data()[i];
        }
        dump(prefix + ".chunked.f32", all);
    }
    {
        engine::Engine eng(model, 4, 64, 0);
        engine::SamplingParams greedy;
        greedy.temperature = 0.0;
        const std::vector<int64_t> out = eng.generate(ids, greedy, 8);
        FILE* f = std::fopen((prefix + ".greedy.txt").c_str(), "w");
        for (const int64_t t : out) std::fprintf(f, "%lld\n", static_cast<long long>(t));
        std::fclose(f);
    }
    return 0;
}
