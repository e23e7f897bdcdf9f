// Timing harness for the UNMODIFIED reference library (namespace quant) on BASELINE config 1: a GPT-2-small-sized decoder
// (12 layers, d_model 768, 12 heads, d_ff 3072, GELU, vocab 50257, context 1024; fp32, seeded random init), batch 1,
// 32 prompt tokens drawn uniformly from the vocabulary, 64 greedy tokens through quant::Generator::generate_tokens.
// The reference has no LayerNorm / learned-position model, so its own Llama-style block (RMSNorm + RoPE) of the same
// dimensions stands in; the arithmetic per token is the same to within the norm and position terms.
// Built by baseline/build_reference.sh against the reference's own static libraries; prints one JSON line.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>

#include "quant/generator.h"
#include "quant/model.h"
#include "quant/sampler.h"
#include "quant/tokenizer.h"

namespace {
struct NoTokenizer : quant::Tokenizer {
  std::vector<int> encode(const std::string&) override { return {}; }
  std::string decode(const std::vector<int>&) override { return ""; }
  int vocab_size() const override { return 50257; }
  int bos_id() const override { return 0; }
  int eos_id() const override { return -1; }   // never produced: all 64 tokens are generated
};
}  // namespace

int main(int argc, char** argv) {
  const int layers = argc > 1 ? std::atoi(argv[1]) : 12;
  const int new_tokens = argc > 2 ? std::atoi(argv[2]) : 64;
  quant::TransformerConfig cfg;
  cfg.vocab_size = 50257; cfg.hidden_size = 768; cfg.num_layers = layers; cfg.num_heads = 12; cfg.head_dim = 64;
  cfg.ffn_hidden_size = 3072; cfg.max_seq_len = 1024; cfg.activation = quant::Activation::GELU;
  quant::DenseModel model(cfg);
  model.init_weights(1);
  NoTokenizer tok;
  quant::Generator gen(&model, &tok);
  std::mt19937 rng(0);
  std::vector<int> prompt(32);
  for (auto& t : prompt) t = int(rng() % 50257);
  quant::SamplerConfig sc;
  sc.temperature = 0.0f; sc.top_k = 1; sc.top_p = 1.0f; sc.max_tokens = new_tokens;
  const auto t0 = std::chrono::steady_clock::now();
  const std::vector<int> out = gen.generate_tokens(prompt, sc);
  const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  const int made = int(out.size()) - int(prompt.size());
  std::printf("{\"impl\": \"reference\", \"metric\": \"generated_tokens_per_s\", \"value\": %.4f, \"unit\": \"tokens/s\", "
              "\"seconds\": %.3f, \"prompt_tokens\": 32, \"new_tokens\": %d, \"layers\": %d, \"dtype\": \"fp32\", \"device\": \"cpu\"}\n",
              made / s, s, made, layers);
  return made > 0 ? 0 : 1;
}
