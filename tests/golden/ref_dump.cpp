// Driver for tests/golden/make_golden.py: runs the reference's own CPU model and engine
// (BusyaPrime/from-scratch-inference-engine-, src/model/model.cpp, src/engine/engine.cpp) on a
// model folder and writes what the plain implementation and the engine are compared with.
//   ref_dump MODEL_DIR SCENARIO.json OUT_PREFIX
// The scenario names token ids, a block size, the steps of a mixed batch, prompts for
// concurrent greedy generation and the two prompts of the preemption case.  Written:
//   OUT_PREFIX.forward.f32  logits [S, V] of Model::forward(ids)
//   OUT_PREFIX.chunked.f32  logits [S, V] of forward_paged: the first S-3 tokens in one call,
//                           then one token per call
//   OUT_PREFIX.batch.f32    last-row logits of every item of every step of the mixed batch
//                           through Model::forward_batch over one BlockManager, in order
//                           (the scheme of tests/cpp/test_continuous_batch.cpp:50-82, with a
//                           prompt portion that starts behind cached tokens among the items)
//   OUT_PREFIX.engine.json  tokens of the prompts generated concurrently by one Engine, and
//                           the preemption case of tests/cpp/test_engine.cpp:103-128: two
//                           requests in a pool of two blocks, their outputs, the outputs of
//                           each alone, and Engine::preemptions()
#include "engine/block_manager.hpp"
#include "engine/engine.hpp"
#include "engine/model.hpp"
#include "engine/paged_kv_cache.hpp"

#include <nlohmann/json.hpp>

#include <cstdio>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

using json = nlohmann::json;
using Ids = std::vector<int64_t>;

static void dump(const std::string& path, const std::vector<float>& values) {
    FILE* f = std::fopen(path.c_str(), "wb");
    std::fwrite(values.data(), sizeof(float), values.size(), f);
    std::fclose(f);
}

static std::vector<float> flat(const engine::Tensor& t) {
    return std::vector<float>(t.data(), t.data() + t.numel());
}

int main(int argc, char** argv) {
    if (argc != 4) return 2;
    const std::string dir = argv[1], prefix = argv[3];
    std::ifstream in(argv[2]);
    std::stringstream text;
    text << in.rdbuf();
    const json scenario = json::parse(text.str());
    const Ids ids = scenario.at("ids").get<Ids>();
    const int64_t block = scenario.at("block_size").get<int64_t>();

    const engine::Model model = engine::Model::from_pretrained(dir);
    const engine::ModelConfig& c = model.config();
    const int64_t vocab = c.vocab_size;
    const int64_t kv_dim = c.num_key_value_heads * c.head_dim;

    dump(prefix + ".forward.f32", flat(model.forward(ids)));

    {
        const int64_t s = static_cast<int64_t>(ids.size());
        engine::PagedKVCache cache(c.num_hidden_layers, kv_dim, block, 64);
        std::vector<float> all(static_cast<size_t>(s * vocab));
        const int64_t head = s - 3;
        const engine::Tensor a = model.forward_paged(Ids(ids.begin(), ids.begin() + head), cache);
        for (int64_t i = 0; i < a.numel(); ++i) all[static_cast<size_t>(i)] = a.data()[i];
        for (int64_t t = head; t < s; ++t) {
            const engine::Tensor b = model.forward_paged({ids[static_cast<size_t>(t)]}, cache);
            for (int64_t i = 0; i < vocab; ++i) all[static_cast<size_t>(t * vocab + i)] = b.data()[i];
        }
        dump(prefix + ".chunked.f32", all);
    }
    {
        engine::BlockManager manager(c.num_hidden_layers, kv_dim, block, 256);
        std::map<std::string, engine::SequenceBlocks> blocks;
        std::vector<float> rows;
        for (const json& step : scenario.at("batch_steps")) {
            std::vector<engine::BatchItem> items;
            for (const json& item : step)
                items.push_back({&blocks[item.at("request").get<std::string>()],
                                 item.at("tokens").get<Ids>()});
            const std::vector<float> last = flat(model.forward_batch(manager, items));
            rows.insert(rows.end(), last.begin(), last.end());
        }
        dump(prefix + ".batch.f32", rows);
    }
    json out;
    engine::SamplingParams greedy;
    greedy.temperature = 0.0;
    {
        engine::Engine eng(model, block, 256, 0);
        std::vector<int64_t> handles;
        const int64_t n = scenario.at("greedy_tokens").get<int64_t>();
        for (const json& prompt : scenario.at("greedy_prompts"))
            handles.push_back(eng.add_request({prompt.get<Ids>(), greedy, n, -1}));
        while (eng.has_work()) eng.step();
        out["greedy"] = json::array();
        for (const int64_t h : handles) out["greedy"].push_back(eng.output(h));
    }
    {
        const json& p = scenario.at("preempt");
        const Ids pa = p.at("a").get<Ids>(), pb = p.at("b").get<Ids>();
        const int64_t n = p.at("tokens").get<int64_t>();
        const int64_t pool_blocks = p.at("num_blocks").get<int64_t>();
        engine::Engine alone_a(model, block, 64, 9), alone_b(model, block, 64, 9);
        out["preempt"]["alone_a"] = alone_a.generate(pa, greedy, n);
        out["preempt"]["alone_b"] = alone_b.generate(pb, greedy, n);
        engine::Engine eng(model, block, pool_blocks, 9);
        const int64_t id_a = eng.add_request({pa, greedy, n, -1});
        const int64_t id_b = eng.add_request({pb, greedy, n, -1});
        int guard = 0;
        while (eng.has_work() && guard++ < 2000) eng.step();
        out["preempt"]["a"] = eng.output(id_a);
        out["preempt"]["b"] = eng.output(id_b);
        out["preempt"]["preemptions"] = eng.preemptions();
    }
    std::ofstream(prefix + ".engine.json") << out.dump(1) << "\n";
    return 0;
}
