// Test program for the drop-in seam: the reference's UNMODIFIED inference engine, sampler, tokenizer and checkpoint
// reader (compiled from where they lie in the reference tree by `make -C oracle engine`) driven through
// IModelBackend, once with the reference's own ModelBackend and once with B200ModelBackend (the adapter over
// librwkv7_b200.so).  Test infrastructure only; nothing here is linked into the product library.
//
//   engine_seam <ref|b200> <model.pth> <vocab.txt> <wkv32: 0|1> <max_tokens> <prompt> [<prompt> ...]
//
// Prints one line per prompt: "out <index> <hex of the generated text>", after "ok <backend>".
#include <cstdio>
#include <cstdlib>
#include <exception>
#include <memory>
#include <string>
#include <vector>

#include "b200_model_backend.hpp"
#include "rwkv_inference_engine.hpp"
#include "rwkv_server_backend.hpp"
#include "rwkv_tokenizer.hpp"

int main(int argc, char** argv) {
  if (argc < 7) {
    std::fprintf(stderr, "usage: engine_seam <ref|b200> <model.pth> <vocab.txt> <wkv32> <max_tokens> <prompt>...\n");
    return 2;
  }
  try {
    const std::string which = argv[1], path = argv[2], vocab = argv[3];
    const bool wkv32 = std::atoi(argv[4]) != 0;
    auto tokenizer = std::make_shared<rwkv7_server::TrieTokenizer>();
    if (tokenizer->load(vocab) != rwkv7_server::kTokenizerSuccess) {
      std::fprintf(stderr, "cannot load vocabulary %s\n", vocab.c_str());
      return 3;
    }
    std::shared_ptr<rwkv7_server::IModelBackend> backend;
    if (which == "ref") backend = std::make_shared<rwkv7_server::ModelBackend>(path, wkv32, false);
    else backend = std::make_shared<rwkv7_server::B200ModelBackend>(path, wkv32, false, 0);
    rwkv7_server::InferenceEngine engine(backend, tokenizer, backend->model_name(), 128);
    rwkv7_server::GenerateOptions opt;
    opt.max_tokens = std::atoi(argv[5]);
    opt.top_p = 0.0;            // the sampler's greedy case
    opt.alpha_presence = 0.0;   // no penalties: the choice depends on the logits alone
    opt.alpha_frequency = 0.0;
    opt.stop_tokens = {0};
    std::vector<std::string> prompts;
    for (int i = 6; i < argc; ++i) prompts.emplace_back(argv[i]);
    const auto outs = engine.batch_generate(prompts, opt);
    std::printf("ok %s vocab %d\n", which.c_str(), backend->vocab_size());
    for (size_t i = 0; i < outs.size(); ++i) {
      std::printf("out %zu ", i);
      for (unsigned char c : outs[i]) std::printf("%02x", c);
      std::printf("\n");
    }
    // the batch-1 stateful entry point as well (the state cache's path): prefill + decode on a caller-held state
    auto st = backend->create_state(1);
    opt.max_tokens = 4;
    const auto one = engine.batch_generate_state({prompts[0]}, st, opt);
    std::printf("state ");
    for (unsigned char c : one[0]) std::printf("%02x", c);
    std::printf("\n");
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "engine_seam: %s\n", e.what());
    return 1;
  }
}
