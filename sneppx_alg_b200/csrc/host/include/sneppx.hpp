// sneppx.hpp: header-only C++17 interface to the host runtime library (libsneppx_host.so).
//
// The reference ships a second-language binding crate whose tensor / model / train types are placeholders
// (lib/rust/src/{lib,tensor,model,train}.rs). This header is that layer for C++ programs, over the library's C ABI:
// host tensors, `.sneppx` checkpoint files, the byte-level BPE tokenizer, the model preset factory, hashing and the
// post-quantum key exchange. Link with -lsneppx_host. Everything throws std::runtime_error on failure.
#pragma once

#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

extern "C" {
const char* sx_host_version();
int sx_ckpt_write(const char* path, int n, const uint64_t* shapes, const uint32_t* ndims, const uint32_t* dtypes,
                  const void* const* data, const uint64_t* nbytes, const char* metadata_json, const uint64_t* strides);
void* sx_ckpt_open(const char* path);
int sx_ckpt_num_tensors(void* h);
int sx_ckpt_tensor_info(void* h, int i, uint64_t* shape8, uint32_t* ndim, uint32_t* dtype, uint64_t* nbytes);
int sx_ckpt_read_tensor(void* h, int i, void* dst);
const char* sx_ckpt_metadata(void* h);
void sx_ckpt_close(void* h);
void* sx_tok_create();
void sx_tok_destroy(void* h);
int sx_tok_vocab_size(void* h);
int sx_tok_train(void* h, const uint8_t* text, long long n, int vocab_size);
long long sx_tok_encode(void* h, const uint8_t* text, long long n, int* out, long long cap);
long long sx_tok_decode(void* h, const int* ids, long long n, uint8_t* out, long long cap);
int sx_tok_save(void* h, const char* path);
int sx_tok_load(void* h, const char* path);
int sx_factory_config_from_name(const char* name, char* out, int cap);
void sx_sha256(const uint8_t* p, size_t n, uint8_t* out32);
int sx_mlkem_sizes(int k, int* ek, int* dk, int* ct);
int sx_mlkem_keygen(int k, const uint8_t* d, const uint8_t* z, uint8_t* ek, uint8_t* dk);
int sx_mlkem_encaps(int k, const uint8_t* ek, const uint8_t* m, uint8_t* ct, uint8_t* ss);
int sx_mlkem_decaps(int k, const uint8_t* dk, const uint8_t* ct, uint8_t* ss);
}

namespace sneppx {

inline std::string version() { return sx_host_version(); }

enum class DType : uint32_t { f32 = 0, f64 = 1, f16 = 2, bf16 = 3, i32 = 4, i64 = 5 };
inline size_t element_size(DType t) {
  switch (t) {
    case DType::f32: case DType::i32: return 4;
    case DType::f64: case DType::i64: return 8;
    default: return 2;
  }
}

// Host tensor: contiguous, row-major, owns its bytes.
struct Tensor {
  std::vector<uint64_t> shape;
  DType dtype = DType::f32;
  std::vector<uint8_t> bytes;

  Tensor() = default;
  Tensor(std::vector<uint64_t> shape_, DType dtype_ = DType::f32) : shape(std::move(shape_)), dtype(dtype_) {
    if (shape.size() > 8) throw std::runtime_error("at most 8 dimensions");
    bytes.assign(numel() * element_size(dtype), 0);
  }
  static Tensor from(const std::vector<float>& values, std::vector<uint64_t> shape_) {
    Tensor t(std::move(shape_), DType::f32);
    if (values.size() != t.numel()) throw std::runtime_error("value count does not match the shape");
    memcpy(t.bytes.data(), values.data(), t.bytes.size());
    return t;
  }
  uint64_t numel() const { uint64_t n = 1; for (uint64_t d : shape) n *= d; return n; }
  template <class T> T* data() { return reinterpret_cast<T*>(bytes.data()); }
  template <class T> const T* data() const { return reinterpret_cast<const T*>(bytes.data()); }
};

// `.sneppx` checkpoint container: tensors in file order (names travel in the metadata JSON under "names").
struct Checkpoint {
  std::vector<Tensor> tensors;
  std::string metadata_json = "{}";

  void save(const std::string& path) const {
    const int n = (int)tensors.size();
    std::vector<uint64_t> shapes((size_t)n * 8, 0), nbytes((size_t)n);
    std::vector<uint32_t> ndims((size_t)n), dtypes((size_t)n);
    std::vector<const void*> data((size_t)n);
    for (int i = 0; i < n; ++i) {
      const Tensor& t = tensors[(size_t)i];
      for (size_t d = 0; d < t.shape.size(); ++d) shapes[(size_t)i * 8 + d] = t.shape[d];
      ndims[(size_t)i] = (uint32_t)t.shape.size(); dtypes[(size_t)i] = (uint32_t)t.dtype;
      data[(size_t)i] = t.bytes.data(); nbytes[(size_t)i] = t.bytes.size();
    }
    if (sx_ckpt_write(path.c_str(), n, shapes.data(), ndims.data(), dtypes.data(), data.data(), nbytes.data(), metadata_json.c_str(), nullptr) != 0)
      throw std::runtime_error("cannot write " + path);
  }
  static Checkpoint load(const std::string& path) {
    void* h = sx_ckpt_open(path.c_str());
    if (!h) throw std::runtime_error("cannot open " + path + " as a checkpoint");
    Checkpoint c;
    try {
      c.metadata_json = sx_ckpt_metadata(h);
      for (int i = 0, n = sx_ckpt_num_tensors(h); i < n; ++i) {
        uint64_t shape[8], nbytes; uint32_t nd, dt;
        if (sx_ckpt_tensor_info(h, i, shape, &nd, &dt, &nbytes) != 0 || nd > 8) throw std::runtime_error("bad tensor record");
        Tensor t;
        t.shape.assign(shape, shape + nd); t.dtype = (DType)dt; t.bytes.resize(nbytes);
        if (sx_ckpt_read_tensor(h, i, t.bytes.data()) != 0) throw std::runtime_error("cannot read tensor data");
        c.tensors.push_back(std::move(t));
      }
    } catch (...) { sx_ckpt_close(h); throw; }
    sx_ckpt_close(h);
    return c;
  }
};

class Tokenizer {
 public:
  Tokenizer() : h_(sx_tok_create()) {}
  ~Tokenizer() { sx_tok_destroy(h_); }
  Tokenizer(const Tokenizer&) = delete;
  Tokenizer& operator=(const Tokenizer&) = delete;
  int vocab_size() const { return sx_tok_vocab_size(h_); }
  void train(const std::string& text, int vocab) {
    if (sx_tok_train(h_, (const uint8_t*)text.data(), (long long)text.size(), vocab) < 0) throw std::runtime_error("tokenizer training failed");
  }
  std::vector<int> encode(const std::string& text) const {
    std::vector<int> ids(text.size() + 1);
    const long long n = sx_tok_encode(h_, (const uint8_t*)text.data(), (long long)text.size(), ids.data(), (long long)ids.size());
    if (n < 0) throw std::runtime_error("encode failed");
    ids.resize((size_t)n);
    return ids;
  }
  std::string decode(const std::vector<int>& ids) const {
    std::string out(ids.size() * 64 + 16, '\0');
    const long long n = sx_tok_decode(h_, ids.data(), (long long)ids.size(), (uint8_t*)&out[0], (long long)out.size());
    if (n < 0) throw std::runtime_error("decode failed");
    out.resize((size_t)n);
    return out;
  }
  void save(const std::string& path) const { if (sx_tok_save(h_, path.c_str()) != 0) throw std::runtime_error("cannot save tokenizer"); }
  void load(const std::string& path) { if (sx_tok_load(h_, path.c_str()) != 0) throw std::runtime_error("cannot load tokenizer"); }
 private:
  void* h_;
};

// JSON text of a model preset ("llama3-8b", "mistral-7b", "deepseek-v2-lite", ...).
inline std::string model_config(const std::string& name) {
  std::string out(8192, '\0');
  const int n = sx_factory_config_from_name(name.c_str(), &out[0], (int)out.size());
  if (n < 0) throw std::runtime_error("unknown model preset " + name);
  out.resize((size_t)n);
  return out;
}

inline std::string sha256_hex(const std::string& data) {
  uint8_t d[32];
  sx_sha256((const uint8_t*)data.data(), data.size(), d);
  static const char* hex = "0123456789abcdef";
  std::string s;
  for (uint8_t b : d) { s += hex[b >> 4]; s += hex[b & 15]; }
  return s;
}

// ML-KEM-768 key exchange (FIPS 203).
struct MlKem768 {
  std::vector<uint8_t> ek, dk;
  static MlKem768 generate(const uint8_t seed64[64]) {
    int a, b, c; sx_mlkem_sizes(3, &a, &b, &c);
    MlKem768 k; k.ek.resize((size_t)a); k.dk.resize((size_t)b);
    sx_mlkem_keygen(3, seed64, seed64 + 32, k.ek.data(), k.dk.data());
    return k;
  }
  static std::pair<std::vector<uint8_t>, std::vector<uint8_t>> encapsulate(const std::vector<uint8_t>& ek, const uint8_t m32[32]) {
    int a, b, c; sx_mlkem_sizes(3, &a, &b, &c);
    if ((int)ek.size() != a) throw std::runtime_error("encapsulation key has the wrong length");
    std::vector<uint8_t> ct((size_t)c), ss(32);
    if (sx_mlkem_encaps(3, ek.data(), m32, ct.data(), ss.data()) != 0) throw std::runtime_error("invalid encapsulation key");
    return {ct, ss};
  }
  std::vector<uint8_t> decapsulate(const std::vector<uint8_t>& ct) const {
    int a, b, c; sx_mlkem_sizes(3, &a, &b, &c);
    if ((int)ct.size() != c) throw std::runtime_error("ciphertext has the wrong length");
    std::vector<uint8_t> ss(32);
    sx_mlkem_decaps(3, dk.data(), ct.data(), ss.data());
    return ss;
  }
};

}  // namespace sneppx
