// Test tooling, not part of the engine: runs EmersonDowell/AIR's own CPU reference
// executor (src/reference/reference_executor.cpp) on a tiny model given as raw files,
// token by token, and writes the float32 logits of every position.
//
// It is compiled by tests/golden/make_golden.py against AIR's unmodified sources
// (their folder is given on the compiler's command line); nothing of AIR is kept here.
//
//   air_driver MANIFEST DATA OUT TOKEN [TOKEN ...]
//
// MANIFEST (text): a first line "layers hidden ffn heads kv_heads context vocab theta eps",
// then one line per tensor: "name rank dim0 [dim1] byte_offset byte_size" with AIR's own
// tensor names and its {in, out} order of dimensions.  DATA: the float32 bytes.
#include "air/reference.hpp"
#include "air/storage.hpp"

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

int main(int argc, char** argv) {
    if (argc < 5) {
        std::cerr << "usage: air_driver MANIFEST DATA OUT TOKEN...\n";
        return 2;
    }
    std::ifstream manifest(argv[1]);
    air::ModelConfig config;
    config.architecture = "qwen2";
    manifest >> config.layer_count >> config.embedding_size >> config.feed_forward_size >>
        config.attention_head_count >> config.kv_head_count >> config.context_length >>
        config.vocabulary_size >> config.rope_frequency_base >> config.rms_norm_epsilon;
    config.rope_dimension_count = config.embedding_size / config.attention_head_count;

    std::vector<air::TensorDescriptor> tensors;
    std::string line;
    std::getline(manifest, line);
    while (std::getline(manifest, line)) {
        if (line.empty()) continue;
        std::istringstream in(line);
        air::TensorDescriptor t;
        std::size_t rank = 0;
        in >> t.name >> rank;
        t.shape.dimensions.resize(rank);
        for (auto& d : t.shape.dimensions) in >> d;
        in >> t.byte_offset >> t.byte_size;
        t.type = air::DataType::f32;
        t.byte_size_exact = true;
        tensors.push_back(std::move(t));
    }

    air::TokenizerDefinition tokenizer;
    tokenizer.model = "gpt2";
    tokenizer.pre_tokenizer = "gpt2";
    for (std::uint64_t i = 0; i < config.vocabulary_size; ++i) {
        tokenizer.vocabulary.push_back("t" + std::to_string(i));
    }

    auto storage = air::ModelStorage::map_read_only(argv[2]);
    if (!storage) {
        std::cerr << storage.status().message() << "\n";
        return 3;
    }
    auto model = std::make_shared<air::ModelDefinition>(
        air::ModelFingerprint{"golden", config.architecture, "tiny"}, config, std::move(tokenizer),
        std::move(tensors), std::move(storage).value());
    auto executor = air::ReferenceExecutor::create(model);
    if (!executor) {
        std::cerr << executor.status().message() << "\n";
        return 6;
    }
    air::ReferenceKvCache cache(config.layer_count, config.kv_head_count,
                                config.embedding_size / config.attention_head_count,
                                config.context_length);
    std::FILE* out = std::fopen(argv[3], "wb");
    if (!out) return 3;
    for (int i = 4; i < argc; ++i) {
        auto logits = executor.value()->step(static_cast<air::TokenId>(std::atoi(argv[i])), cache);
        if (!logits) {
            std::cerr << logits.status().message() << "\n";
            return 7;
        }
        std::fwrite(logits.value().data(), sizeof(float), logits.value().size(), out);
    }
    std::fclose(out);
    return 0;
}
