// Exercises sneppx.hpp from a plain C++ program; tests/test_cpp_api_cpu.py compiles and runs it.
#include <cstdio>
#include <iostream>

#include "sneppx.hpp"

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  const std::string dir = argv[1];
  std::cout << "version " << sneppx::version() << "\n";

  sneppx::Checkpoint ck;
  ck.tensors.push_back(sneppx::Tensor::from({1.f, 2.f, 3.f, 4.f, 5.f, 6.f}, {2, 3}));
  sneppx::Tensor idx({4}, sneppx::DType::i64);
  for (int i = 0; i < 4; ++i) idx.data<int64_t>()[i] = 10 * i;
  ck.tensors.push_back(idx);
  ck.metadata_json = "{\"names\": [\"w\", \"idx\"], \"step\": 7}";
  ck.save(dir + "/from_cpp.sneppx");
  sneppx::Checkpoint back = sneppx::Checkpoint::load(dir + "/from_cpp.sneppx");
  if (back.tensors.size() != 2 || back.tensors[0].shape != std::vector<uint64_t>{2, 3} || back.tensors[0].data<float>()[5] != 6.f ||
      back.tensors[1].dtype != sneppx::DType::i64 || back.tensors[1].data<int64_t>()[3] != 30 || back.metadata_json != ck.metadata_json)
    return 3;
  try { sneppx::Checkpoint::load(dir + "/missing.sneppx"); return 4; } catch (const std::runtime_error&) {}

  sneppx::Tokenizer tok;
  std::string corpus;
  for (int i = 0; i < 50; ++i) corpus += "the quick brown fox jumps over the lazy dog. ";
  tok.train(corpus, 300);
  const std::string text = "the lazy fox";
  std::vector<int> ids = tok.encode(text);
  if (tok.decode(ids) != text || ids.size() >= text.size() || tok.vocab_size() <= 256) return 5;
  tok.save(dir + "/tok.bin");
  sneppx::Tokenizer tok2;
  tok2.load(dir + "/tok.bin");
  if (tok2.encode(text) != ids) return 6;

  if (sneppx::model_config("llama3-8b").find("4096") == std::string::npos) return 7;
  try { sneppx::model_config("no-such-model"); return 8; } catch (const std::runtime_error&) {}
  std::cout << "sha256 " << sneppx::sha256_hex("abc") << "\n";

  uint8_t seed[64], m[32];
  for (int i = 0; i < 64; ++i) seed[i] = (uint8_t)i;
  for (int i = 0; i < 32; ++i) m[i] = (uint8_t)(200 + i);
  sneppx::MlKem768 key = sneppx::MlKem768::generate(seed);
  auto [ct, ss] = sneppx::MlKem768::encapsulate(key.ek, m);
  if (key.decapsulate(ct) != ss) return 9;
  ct[3] ^= 1;
  if (key.decapsulate(ct) == ss) return 10;
  std::cout << "CPP_API_OK\n";
  return 0;
}
