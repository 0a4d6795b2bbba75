// Driver of the reference arm of bench.py.  It is this repository's code; everything it
// drives is EmersonDowell/AIR's own, unmodified: its model definition, its CUDA executor
// (src/cuda/cuda_backend.cu: CudaExecutor::create, prefill, prefill_discard, step,
// step_greedy_batch) and its paged cache.  Nothing of air_b200 is linked or called.
//
//   air_cuda_driver check MANIFEST DATA OUT TOKEN...
//       A tiny float32 model given as raw files (the format of tests/golden/air_driver.cpp).
//       Writes float32 logits [tokens, vocab] of CudaExecutor::step token by token, then one
//       more row: the logits of CudaExecutor::prefill of the whole sequence (its last place),
//       then prints the tokens that step_greedy_batch gives for two copies of the sequence.
//   air_cuda_driver bench key=value ...
//       A model of the given sizes with random weights (matrices bfloat16, vectors float32) in
//       a scratch file, AIR's stock code path on it: one prefill of `prefill` tokens, then
//       `batch` sequences of `context` tokens decoded together for `warmup` + `steps` steps.
//       fill=prefill computes every sequence's context (minutes at 28 layers: AIR's products are
//       scalar kernels); fill=fork (the default) computes one and makes the others with AIR's own
//       CudaKvCache::fork, which shares the prefix's pages between them.
//       Prints one JSON object with the times.
//
// AIR's executor calls block until their result is on the host, so steps are timed with the
// host's clock around the call (the device is idle before each call).
#include "air/cuda.hpp"
#include "air/storage.hpp"

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <memory>
#include <random>
#include <sstream>
#include <string>
#include <vector>

#include <unistd.h>

namespace {

air::TokenizerDefinition dummy_tokenizer(std::uint64_t vocab) {
    air::TokenizerDefinition tokenizer;
    tokenizer.model = "gpt2";
    tokenizer.pre_tokenizer = "gpt2";
    tokenizer.vocabulary.reserve(vocab);
    for (std::uint64_t i = 0; i < vocab; ++i) tokenizer.vocabulary.push_back("t" + std::to_string(i));
    return tokenizer;
}

double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int fail(const air::Status& status, int code) {
    std::cerr << status.message() << "\n";
    return code;
}

int run_check(int argc, char** argv) {
    if (argc < 6) return 2;
    std::ifstream manifest(argv[2]);
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
    auto storage = air::ModelStorage::map_read_only(argv[3]);
    if (!storage) return fail(storage.status(), 3);
    auto model = std::make_shared<air::ModelDefinition>(
        air::ModelFingerprint{"golden", config.architecture, "tiny"}, config,
        dummy_tokenizer(config.vocabulary_size), std::move(tensors), std::move(storage).value());
    auto executor = air::CudaExecutor::create(model, 0);
    if (!executor) return fail(executor.status(), 6);
    std::vector<air::TokenId> tokens;
    for (int i = 5; i < argc; ++i) tokens.push_back(std::atoi(argv[i]));
    std::FILE* out = std::fopen(argv[4], "wb");
    if (!out) return 3;
    {
        auto cache = executor.value()->create_kv_cache(16U);
        if (!cache) return fail(cache.status(), 6);
        for (const auto token : tokens) {
            auto logits = executor.value()->step(token, *cache.value());
            if (!logits) return fail(logits.status(), 7);
            std::fwrite(logits.value().data(), sizeof(float), logits.value().size(), out);
        }
    }
    {
        auto cache = executor.value()->create_kv_cache(16U);
        if (!cache) return fail(cache.status(), 6);
        auto logits = executor.value()->prefill(tokens, *cache.value());
        if (!logits) return fail(logits.status(), 7);
        std::fwrite(logits.value().data(), sizeof(float), logits.value().size(), out);
    }
    std::fclose(out);
    {
        // two sequences decoded together, greedy: both must give the argmax of the last row
        auto a = executor.value()->create_kv_cache(16U);
        auto b = executor.value()->create_kv_cache(16U);
        if (!a || !b) return 6;
        std::span<const air::TokenId> head(tokens.data(), tokens.size() - 1U);
        auto s = executor.value()->prefill_discard(head, *a.value());
        if (!s) return fail(s, 7);
        s = executor.value()->prefill_discard(head, *b.value());
        if (!s) return fail(s, 7);
        std::vector<air::TokenId> last{tokens.back(), tokens.back()};
        std::vector<air::CudaKvCache*> caches{a.value().get(), b.value().get()};
        auto chosen = executor.value()->step_greedy_batch(last, caches);
        if (!chosen) return fail(chosen.status(), 7);
        std::cout << "greedy_batch " << chosen.value()[0] << " " << chosen.value()[1] << "\n";
    }
    return 0;
}

// bfloat16 bit pattern of a float, round to nearest even
std::uint16_t bf16_bits(float x) {
    std::uint32_t u;
    std::memcpy(&u, &x, 4);
    u += 0x7FFFU + ((u >> 16) & 1U);
    return static_cast<std::uint16_t>(u >> 16);
}

struct Writer {
    std::FILE* file;
    std::uint64_t offset{0};
    std::vector<air::TensorDescriptor> tensors;
    std::vector<std::uint16_t> table;    // 65,536 draws of N(0, 0.02) as bfloat16
    std::uint64_t state{0x9E3779B97F4A7C15ULL};

    std::uint64_t next() {
        state ^= state << 13;
        state ^= state >> 7;
        state ^= state << 17;
        return state;
    }
    void pad() {
        static const char zeros[256] = {};
        const auto rest = (256U - offset % 256U) % 256U;
        std::fwrite(zeros, 1, rest, file);
        offset += rest;
    }
    // {in, out}: AIR's order of dimensions; rows of `in` elements, `out` of them
    void matrix(const std::string& name, std::uint64_t in, std::uint64_t out) {
        pad();
        air::TensorDescriptor t;
        t.name = name;
        t.type = air::DataType::bf16;
        t.shape.dimensions = {in, out};
        t.byte_offset = offset;
        t.byte_size = in * out * 2U;
        t.byte_size_exact = true;
        std::vector<std::uint16_t> buffer(1U << 20);
        std::uint64_t left = in * out;
        while (left) {
            const auto n = std::min<std::uint64_t>(left, buffer.size());
            for (std::uint64_t i = 0; i < n; i += 4) {
                const auto r = next();
                buffer[i] = table[r & 0xFFFF];
                buffer[i + 1] = table[(r >> 16) & 0xFFFF];
                buffer[i + 2] = table[(r >> 32) & 0xFFFF];
                buffer[i + 3] = table[(r >> 48) & 0xFFFF];
            }
            std::fwrite(buffer.data(), 2, n, file);
            left -= n;
        }
        offset += t.byte_size;
        tensors.push_back(std::move(t));
    }
    void vector(const std::string& name, std::uint64_t n, float mean) {
        pad();
        air::TensorDescriptor t;
        t.name = name;
        t.type = air::DataType::f32;
        t.shape.dimensions = {n};
        t.byte_offset = offset;
        t.byte_size = n * 4U;
        t.byte_size_exact = true;
        std::vector<float> values(n);
        for (auto& v : values) {
            const std::uint32_t bits = static_cast<std::uint32_t>(table[next() & 0xFFFF]) << 16;
            float f;
            std::memcpy(&f, &bits, 4);
            v = mean + f;
        }
        std::fwrite(values.data(), 4, n, file);
        offset += t.byte_size;
        tensors.push_back(std::move(t));
    }
};

int run_bench(int argc, char** argv) {
    std::map<std::string, std::string> arg;
    for (int i = 2; i < argc; ++i) {
        const std::string s = argv[i];
        const auto eq = s.find('=');
        if (eq == std::string::npos) return 2;
        arg[s.substr(0, eq)] = s.substr(eq + 1);
    }
    const auto num = [&](const char* key, double fallback) {
        const auto it = arg.find(key);
        return it == arg.end() ? fallback : std::atof(it->second.c_str());
    };
    air::ModelConfig config;
    config.architecture = "qwen2";
    config.layer_count = static_cast<std::uint32_t>(num("layers", 2));
    config.embedding_size = static_cast<std::uint32_t>(num("hidden", 256));
    config.feed_forward_size = static_cast<std::uint32_t>(num("ffn", 512));
    config.attention_head_count = static_cast<std::uint32_t>(num("heads", 2));
    config.kv_head_count = static_cast<std::uint32_t>(num("kv_heads", 1));
    config.context_length = static_cast<std::uint32_t>(num("max_positions", 32768));
    config.vocabulary_size = static_cast<std::uint64_t>(num("vocab", 1024));
    config.rope_frequency_base = num("theta", 1e6);
    config.rms_norm_epsilon = num("eps", 1e-6);
    config.rope_dimension_count = config.embedding_size / config.attention_head_count;
    const auto batch = static_cast<std::size_t>(num("batch", 8));
    const auto context = static_cast<std::size_t>(num("context", 8192));
    const auto prefill_tokens = static_cast<std::size_t>(num("prefill", 2048));
    const auto steps = static_cast<std::size_t>(num("steps", 8));
    const auto warmup = static_cast<std::size_t>(num("warmup", 3));
    const auto page_tokens = static_cast<std::uint32_t>(num("page_tokens", 16));
    const bool fork_fill = !arg.count("fill") || arg["fill"] == "fork";
    const std::string tmp = arg.count("tmp") ? arg["tmp"] : "/tmp";
    const std::string path = tmp + "/air_reference_weights_" + std::to_string(getpid()) + ".bin";

    const double t_write = now_ms();
    Writer w{std::fopen(path.c_str(), "wb")};
    if (!w.file) {
        std::cerr << "cannot write " << path << "\n";
        return 3;
    }
    {
        std::mt19937_64 rng(static_cast<std::uint64_t>(num("seed", 0)));
        std::normal_distribution<float> normal(0.0F, 0.02F);
        w.table.resize(65536);
        for (auto& v : w.table) v = bf16_bits(normal(rng));
    }
    const std::uint64_t E = config.embedding_size, I = config.feed_forward_size, V = config.vocabulary_size;
    const std::uint64_t d = E / config.attention_head_count, KV = config.kv_head_count * d;
    w.matrix("token_embd.weight", E, V);
    w.vector("output_norm.weight", E, 1.0F);
    w.matrix("output.weight", E, V);
    for (std::uint32_t l = 0; l < config.layer_count; ++l) {
        const std::string p = "blk." + std::to_string(l) + ".";
        w.vector(p + "attn_norm.weight", E, 1.0F);
        w.matrix(p + "attn_q.weight", E, E);
        w.matrix(p + "attn_k.weight", E, KV);
        w.matrix(p + "attn_v.weight", E, KV);
        w.vector(p + "attn_q.bias", E, 0.0F);
        w.vector(p + "attn_k.bias", KV, 0.0F);
        w.vector(p + "attn_v.bias", KV, 0.0F);
        w.matrix(p + "attn_output.weight", E, E);
        w.vector(p + "ffn_norm.weight", E, 1.0F);
        w.matrix(p + "ffn_gate.weight", E, I);
        w.matrix(p + "ffn_up.weight", E, I);
        w.matrix(p + "ffn_down.weight", I, E);
    }
    std::fclose(w.file);
    const double write_ms = now_ms() - t_write;

    auto storage = air::ModelStorage::map_read_only(path);
    if (!storage) {
        std::remove(path.c_str());
        return fail(storage.status(), 3);
    }
    const double t_load = now_ms();
    auto model = std::make_shared<air::ModelDefinition>(
        air::ModelFingerprint{"bench", config.architecture, "random"}, config,
        dummy_tokenizer(config.vocabulary_size), std::move(w.tensors), std::move(storage).value());
    auto executor = air::CudaExecutor::create(model, 0);
    std::remove(path.c_str());      // the mapping keeps the bytes until the model is gone
    if (!executor) return fail(executor.status(), 6);
    auto& ex = *executor.value();
    const double load_ms = now_ms() - t_load;

    std::mt19937_64 rng(7);
    const auto draw = [&](std::size_t n) {
        std::vector<air::TokenId> t(n);
        for (auto& x : t) x = static_cast<air::TokenId>(rng() % config.vocabulary_size);
        return t;
    };

    // prefill of one request, whole, greedy output (the stock call of the serving path)
    double prefill_ms = -1.0;
    if (prefill_tokens) {
        const auto prompt = draw(prefill_tokens);
        for (int round = 0; round < 2; ++round) {
            auto cache = ex.create_kv_cache(page_tokens);
            if (!cache) return fail(cache.status(), 6);
            const double t0 = now_ms();
            auto token = ex.prefill_greedy(prompt, *cache.value());
            if (!token) return fail(token.status(), 7);
            const double ms = now_ms() - t0;
            prefill_ms = round == 0 ? ms : std::min(prefill_ms, ms);
        }
    }

    // `batch` sequences of `context` tokens each, then decoded together
    double decode_ms = -1.0, fill_ms = 0.0;
    if (batch && steps) {
        std::vector<std::unique_ptr<air::CudaKvCache>> caches;
        std::vector<air::CudaKvCache*> pointers;
        const std::size_t start = context - (steps + warmup + 2U);
        const double t_fill = now_ms();
        for (std::size_t b = 0; b < batch; ++b) {
            if (b > 0 && fork_fill) {
                auto copy = caches.front()->fork(start);
                if (!copy) return fail(copy.status(), 6);
                caches.push_back(std::move(copy).value());
            } else {
                auto cache = ex.create_kv_cache(page_tokens);
                if (!cache) return fail(cache.status(), 6);
                const auto prompt = draw(start);
                auto s = ex.prefill_discard(prompt, *cache.value());
                if (!s) return fail(s, 7);
                caches.push_back(std::move(cache).value());
            }
            pointers.push_back(caches.back().get());
        }
        fill_ms = now_ms() - t_fill;
        std::vector<air::TokenId> tokens = draw(batch);
        for (std::size_t i = 0; i < warmup; ++i) {
            auto next = ex.step_greedy_batch(tokens, pointers);
            if (!next) return fail(next.status(), 7);
            tokens = next.value();
        }
        const double t0 = now_ms();
        for (std::size_t i = 0; i < steps; ++i) {
            auto next = ex.step_greedy_batch(tokens, pointers);
            if (!next) return fail(next.status(), 7);
            tokens = next.value();
        }
        decode_ms = (now_ms() - t0) / static_cast<double>(steps);
    }
    const auto stats = ex.stats();
    std::printf("{\"prefill_ms\": %.4f, \"prefill_tokens\": %zu, \"decode_ms_per_step\": %.4f, \"batch\": %zu, "
                "\"context\": %zu, \"steps\": %zu, \"warmup\": %zu, \"fill\": \"%s\", \"fill_ms\": %.1f, \"write_ms\": %.1f, "
                "\"load_ms\": %.1f, \"resident_model_bytes\": %llu, \"kv_pool_allocated_bytes\": %llu, "
                "\"specialized_matmul_calls\": %llu, \"decode_batch_calls\": %llu}\n",
                prefill_ms, prefill_tokens, decode_ms, batch, context, steps, warmup,
                fork_fill ? "fork" : "prefill", fill_ms, write_ms, load_ms,
                static_cast<unsigned long long>(stats.resident_model_bytes),
                static_cast<unsigned long long>(stats.kv_pool_allocated_bytes),
                static_cast<unsigned long long>(stats.specialized_matmul_calls),
                static_cast<unsigned long long>(stats.decode_batch_calls));
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc >= 2 && std::string(argv[1]) == "check") return run_check(argc, argv);
    if (argc >= 2 && std::string(argv[1]) == "bench") return run_bench(argc, argv);
    std::cerr << "usage: air_cuda_driver check MANIFEST DATA OUT TOKEN... | bench key=value ...\n";
    return 2;
}
