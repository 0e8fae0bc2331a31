// A C++ program on the host runtime library: train a byte-pair tokenizer on a small corpus, encode a sentence, store
// the ids and an embedding table in a `.sneppx` checkpoint, read the file back, look up a model preset and agree on a
// key with ML-KEM-768.
//
// Build (from the repository root, after `python __graft_entry__.py` has built the libraries):
//   g++ -std=c++17 -O2 -I sneppx_alg_b200/csrc/host/include examples/cpp/host_runtime_demo.cpp
//       -L sneppx_alg_b200/lib -lsneppx_host -Wl,-rpath,$PWD/sneppx_alg_b200/lib -o host_runtime_demo    (one command line)
//   ./host_runtime_demo /tmp
#include <cstdio>
#include <string>

#include "sneppx.hpp"

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : ".";
  std::printf("host library %s\n", sneppx::version().c_str());

  std::string corpus;
  for (int i = 0; i < 40; ++i) corpus += "the quick brown fox jumps over the lazy dog. the dog sleeps; the fox runs. ";
  sneppx::Tokenizer tok;
  tok.train(corpus, 300);
  const std::string sentence = "the lazy fox sleeps over the quick dog.";
  const std::vector<int> ids = tok.encode(sentence);
  std::printf("vocabulary %d; %zu bytes -> %zu tokens; round trip %s\n", tok.vocab_size(), sentence.size(), ids.size(),
              tok.decode(ids) == sentence ? "exact" : "DIFFERS");
  if (tok.decode(ids) != sentence || ids.size() >= sentence.size()) return 1;
  tok.save(dir + "/demo.tok");

  // an embedding table with one recognisable row per token id, and the encoded sentence
  const uint64_t vocab = (uint64_t)tok.vocab_size(), dim = 8;
  sneppx::Tensor table({vocab, dim});
  for (uint64_t r = 0; r < vocab; ++r)
    for (uint64_t c = 0; c < dim; ++c) table.data<float>()[r * dim + c] = (float)r + 0.125f * (float)c;
  sneppx::Tensor encoded({(uint64_t)ids.size()}, sneppx::DType::i32);
  for (size_t i = 0; i < ids.size(); ++i) encoded.data<int32_t>()[i] = ids[i];
  sneppx::Checkpoint ck;
  ck.tensors = {table, encoded};
  ck.metadata_json = "{\"names\": [\"embedding\", \"sentence\"], \"tokenizer\": \"demo.tok\"}";
  ck.save(dir + "/demo.sneppx");

  const sneppx::Checkpoint back = sneppx::Checkpoint::load(dir + "/demo.sneppx");
  const int32_t first = back.tensors[1].data<int32_t>()[0];
  const float* row = back.tensors[0].data<float>() + (uint64_t)first * dim;
  std::printf("checkpoint: %zu tensors, metadata %s; embedding row of the first token starts %.3f %.3f\n", back.tensors.size(),
              back.metadata_json.c_str(), row[0], row[1]);
  if (back.tensors.size() != 2 || row[0] != (float)first || row[1] != (float)first + 0.125f) return 2;

  sneppx::Tokenizer again;
  again.load(dir + "/demo.tok");
  if (again.encode(sentence) != ids) return 3;

  const std::string preset = sneppx::model_config("llama3-8b");
  std::printf("llama3-8b preset: %.72s...\n", preset.c_str());
  std::printf("sha256(corpus) = %s\n", sneppx::sha256_hex(corpus).c_str());

  uint8_t seed[64], m[32];
  for (int i = 0; i < 64; ++i) seed[i] = (uint8_t)(i * 7 + 1);
  for (int i = 0; i < 32; ++i) m[i] = (uint8_t)(255 - i);
  const sneppx::MlKem768 receiver = sneppx::MlKem768::generate(seed);
  const auto sent = sneppx::MlKem768::encapsulate(receiver.ek, m);           // {ciphertext, sender's shared secret}
  const bool agree = receiver.decapsulate(sent.first) == sent.second;
  std::printf("ML-KEM-768: %zu-byte ciphertext, shared secrets %s\n", sent.first.size(), agree ? "agree" : "DIFFER");
  if (!agree) return 4;
  std::printf("HOST_RUNTIME_DEMO_OK\n");
  return 0;
}
