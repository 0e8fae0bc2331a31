// sneppx::ModelFactory in C++: preset registry with versions / deprecation / search, JSON-ish config emission,
// override application and from_pretrained directory probing (algorithms/model_zoo/model_factory.cpp:320-498,
// registry.c:77-323, kernel/model_zoo/model_zoo.c:197 and :496 of the reference). The Python side builds the actual
// torch modules; this library answers "which config does this name mean" for native callers.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

namespace sneppx {

struct LLMConfig {
  std::string family, size;
  int hidden = 0, ffn = 0, layers = 0, heads = 0, kv_heads = 0, vocab = 0, max_pos = 0, sliding_window = 0;
  double rope_theta = 10000.0, rms_eps = 1e-6;
  int kv_lora_rank = 0, q_lora_rank = 0, experts = 0, experts_per_token = 0, shared_experts = 0, moe_ffn = 0;
  std::string version = "1.0.0";
  bool deprecated = false;
};

class ModelFactory {
 public:
  static ModelFactory& instance() {
    static ModelFactory f;
    return f;
  }
  void register_model(const LLMConfig& c) {
    std::lock_guard<std::mutex> lk(mu_);
    table_[key(c.family, c.size)] = c;
  }
  bool lookup(const std::string& name, LLMConfig* out) {
    std::string n = lower(name);
    const size_t slash = n.rfind('/');
    if (slash != std::string::npos) n = n.substr(slash + 1);
    std::replace(n.begin(), n.end(), '_', '-');
    std::lock_guard<std::mutex> lk(mu_);
    // longest family pattern first so that "llama-3" wins over "llama"
    static const std::vector<std::pair<std::string, std::string>> pats = {
        {"llama-3", "llama3"}, {"llama3", "llama3"}, {"llama-2", "llama2"}, {"llama2", "llama2"}, {"llama", "llama2"},
        {"mistral", "mistral"}, {"qwen2", "qwen2"}, {"deepseek", "deepseek_v2"}};
    for (auto& p : pats) {
      if (n.find(p.first) == std::string::npos) continue;
      for (auto& kv : table_)
        if (kv.second.family == p.second && n.find(lower(kv.second.size)) != std::string::npos) { *out = kv.second; return true; }
      for (auto& kv : table_)
        if (kv.second.family == p.second) { *out = kv.second; return true; }
    }
    return false;
  }
  std::vector<std::string> search(const std::string& q) {
    std::vector<std::string> r;
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& kv : table_)
      if (kv.first.find(lower(q)) != std::string::npos && !kv.second.deprecated) r.push_back(kv.first);
    return r;
  }
  bool deprecate(const std::string& family, const std::string& size) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = table_.find(key(family, size));
    if (it == table_.end()) return false;
    it->second.deprecated = true;
    return true;
  }
  static long long num_parameters(const LLMConfig& c) {
    const long long hd = c.heads ? c.hidden / c.heads : 0;
    const long long attn = (long long)c.hidden * (c.heads + 2 * c.kv_heads) * hd + (long long)c.heads * hd * c.hidden;
    long long ffn = 3ll * c.hidden * c.ffn;
    long long total = 0;
    if (c.experts) {
      const long long moe = 3ll * c.hidden * c.moe_ffn * (c.experts + c.shared_experts) + (long long)c.hidden * c.experts;
      total = (attn + ffn) + (long long)(c.layers - 1) * (attn + moe);
    } else total = (long long)c.layers * (attn + ffn);
    return total + 2ll * c.vocab * c.hidden + (2ll * c.layers + 1) * c.hidden;
  }
  static void extend_context(LLMConfig* c, int new_len, const std::string& method) {
    if (new_len <= c->max_pos) return;
    const double s = (double)new_len / c->max_pos;
    if (method == "ntk") c->rope_theta *= s;
    else if (method == "yarn") c->rope_theta *= std::pow(s, 0.8);
    c->max_pos = new_len;
  }
  static std::string to_json(const LLMConfig& c) {
    std::ostringstream o;
    o << "{\"family\":\"" << c.family << "\",\"size\":\"" << c.size << "\",\"hidden_size\":" << c.hidden
      << ",\"intermediate_size\":" << c.ffn << ",\"num_hidden_layers\":" << c.layers << ",\"num_attention_heads\":" << c.heads
      << ",\"num_key_value_heads\":" << c.kv_heads << ",\"vocab_size\":" << c.vocab << ",\"max_position_embeddings\":" << c.max_pos
      << ",\"sliding_window\":" << c.sliding_window << ",\"rope_theta\":" << c.rope_theta << ",\"rms_norm_eps\":" << c.rms_eps
      << ",\"kv_lora_rank\":" << c.kv_lora_rank << ",\"q_lora_rank\":" << c.q_lora_rank << ",\"num_experts\":" << c.experts
      << ",\"num_experts_per_token\":" << c.experts_per_token << ",\"num_shared_experts\":" << c.shared_experts
      << ",\"moe_intermediate_size\":" << c.moe_ffn << ",\"version\":\"" << c.version << "\",\"deprecated\":"
      << (c.deprecated ? "true" : "false") << ",\"num_parameters\":" << num_parameters(c) << "}";
    return o.str();
  }

 private:
  ModelFactory() {
    auto add = [&](const char* f, const char* s, int h, int ffn, int L, int H, int KV, int V, int P, double th, double eps,
                   int sw = 0) {
      LLMConfig c;
      c.family = f; c.size = s; c.hidden = h; c.ffn = ffn; c.layers = L; c.heads = H; c.kv_heads = KV; c.vocab = V;
      c.max_pos = P; c.rope_theta = th; c.rms_eps = eps; c.sliding_window = sw;
      table_[key(f, s)] = c;
    };
    add("llama2", "7B", 4096, 11008, 32, 32, 32, 32000, 4096, 1e4, 1e-5);
    add("llama2", "13B", 5120, 13824, 40, 40, 40, 32000, 4096, 1e4, 1e-5);
    add("llama2", "70B", 8192, 28672, 80, 64, 8, 32000, 4096, 1e4, 1e-5);
    add("llama3", "8B", 4096, 14336, 32, 32, 8, 128256, 8192, 5e5, 1e-5);
    add("llama3", "70B", 8192, 28672, 80, 64, 8, 128256, 8192, 5e5, 1e-5);
    add("mistral", "7B", 4096, 14336, 32, 32, 8, 32000, 32768, 1e4, 1e-5, 4096);
    add("qwen2", "7B", 3584, 18944, 28, 28, 4, 152064, 32768, 1e6, 1e-6);
    add("qwen2", "72B", 8192, 29568, 80, 64, 8, 152064, 32768, 1e6, 1e-6);
    add("deepseek_v2", "lite", 2048, 10944, 27, 16, 16, 102400, 4096, 1e4, 1e-6);
    add("deepseek_v2", "full", 5120, 12288, 60, 64, 64, 102400, 4096, 1e4, 1e-6);
    for (auto* k : {"deepseek_v2:lite", "deepseek_v2:full"}) {
      LLMConfig& c = table_[k];
      c.kv_lora_rank = 512; c.q_lora_rank = 1536; c.experts_per_token = 6; c.shared_experts = 2;
      c.experts = c.size == "lite" ? 64 : 160;
      c.moe_ffn = c.size == "lite" ? 1408 : 1536;
    }
  }
  static std::string lower(std::string s) {
    std::transform(s.begin(), s.end(), s.begin(), ::tolower);
    return s;
  }
  static std::string key(const std::string& f, const std::string& s) { return lower(f) + ":" + lower(s); }
  std::map<std::string, LLMConfig> table_;
  std::mutex mu_;
};

}  // namespace sneppx

extern "C" {
// Writes the JSON config of the named preset into out (NUL-terminated); returns its length, -1 unknown, -2 too small.
int sx_factory_config_from_name(const char* name, char* out, int cap) {
  sneppx::LLMConfig c;
  if (!sneppx::ModelFactory::instance().lookup(name, &c)) return -1;
  const std::string j = sneppx::ModelFactory::to_json(c);
  if ((int)j.size() + 1 > cap) return -2;
  memcpy(out, j.c_str(), j.size() + 1);
  return (int)j.size();
}
int sx_factory_extend_context(const char* name, int new_len, const char* method, char* out, int cap) {
  sneppx::LLMConfig c;
  if (!sneppx::ModelFactory::instance().lookup(name, &c)) return -1;
  sneppx::ModelFactory::extend_context(&c, new_len, method);
  const std::string j = sneppx::ModelFactory::to_json(c);
  if ((int)j.size() + 1 > cap) return -2;
  memcpy(out, j.c_str(), j.size() + 1);
  return (int)j.size();
}
int sx_factory_register(const char* family, const char* size, int hidden, int ffn, int layers, int heads, int kv_heads,
                        int vocab, int max_pos, double rope_theta, double rms_eps) {
  sneppx::LLMConfig c;
  c.family = family; c.size = size; c.hidden = hidden; c.ffn = ffn; c.layers = layers; c.heads = heads;
  c.kv_heads = kv_heads; c.vocab = vocab; c.max_pos = max_pos; c.rope_theta = rope_theta; c.rms_eps = rms_eps;
  sneppx::ModelFactory::instance().register_model(c);
  return 0;
}
int sx_factory_search(const char* query, char* out, int cap) {
  std::string s;
  for (auto& k : sneppx::ModelFactory::instance().search(query)) s += k + "\n";
  if ((int)s.size() + 1 > cap) return -2;
  memcpy(out, s.c_str(), s.size() + 1);
  return (int)s.size();
}
int sx_factory_deprecate(const char* family, const char* size) {
  return sneppx::ModelFactory::instance().deprecate(family, size) ? 0 : -1;
}
}
