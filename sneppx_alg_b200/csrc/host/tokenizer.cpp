// Byte-level BPE tokenizer: train / encode / decode / save / load (the reference's C tokenizer,
// kernel/tokenizer/tokenizer.c: SNEPPX_tokenizer_train_bpe and friends). Ids 0..255 are bytes, merges follow.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace {
struct Tok {
  std::vector<std::pair<int, int>> merges;              // merge i creates id 256 + i
  std::map<std::pair<int, int>, int> rank;
  void rebuild() {
    rank.clear();
    for (size_t i = 0; i < merges.size(); ++i) rank[merges[i]] = (int)i;
  }
};
void apply_merge(std::vector<int>& ids, std::pair<int, int> pr, int nid) {
  size_t w = 0;
  for (size_t i = 0; i < ids.size();) {
    if (i + 1 < ids.size() && ids[i] == pr.first && ids[i + 1] == pr.second) { ids[w++] = nid; i += 2; }
    else ids[w++] = ids[i++];
  }
  ids.resize(w);
}
}  // namespace

extern "C" {
void* sx_tok_create() { return new Tok(); }
void sx_tok_destroy(void* h) { delete static_cast<Tok*>(h); }
int sx_tok_vocab_size(void* h) { return 256 + (int)static_cast<Tok*>(h)->merges.size(); }

int sx_tok_train(void* h, const uint8_t* text, long long n, int vocab_size) {
  Tok* t = static_cast<Tok*>(h);
  t->merges.clear();
  std::vector<int> ids(text, text + n);
  while (256 + (int)t->merges.size() < vocab_size) {
    std::map<std::pair<int, int>, long long> cnt;
    for (size_t i = 0; i + 1 < ids.size(); ++i) cnt[{ids[i], ids[i + 1]}]++;
    std::pair<int, int> best{-1, -1};
    long long bc = 1;
    for (auto& kv : cnt)
      if (kv.second > bc) { bc = kv.second; best = kv.first; }
    if (best.first < 0) break;
    apply_merge(ids, best, 256 + (int)t->merges.size());
    t->merges.push_back(best);
  }
  t->rebuild();
  return (int)t->merges.size();
}

// returns number of ids written (<= cap) or the required size as a negative number
long long sx_tok_encode(void* h, const uint8_t* text, long long n, int* out, long long cap) {
  Tok* t = static_cast<Tok*>(h);
  std::vector<int> ids(text, text + n);
  for (;;) {
    int best_rank = 1 << 30;
    std::pair<int, int> best{-1, -1};
    for (size_t i = 0; i + 1 < ids.size(); ++i) {
      auto it = t->rank.find({ids[i], ids[i + 1]});
      if (it != t->rank.end() && it->second < best_rank) { best_rank = it->second; best = it->first; }
    }
    if (best.first < 0) break;
    apply_merge(ids, best, 256 + best_rank);
  }
  if ((long long)ids.size() > cap) return -(long long)ids.size();
  memcpy(out, ids.data(), ids.size() * sizeof(int));
  return (long long)ids.size();
}

long long sx_tok_decode(void* h, const int* ids, long long n, uint8_t* out, long long cap) {
  Tok* t = static_cast<Tok*>(h);
  std::string s;
  std::vector<int> stack;
  for (long long i = 0; i < n; ++i) {
    stack.push_back(ids[i]);
    while (!stack.empty()) {
      int id = stack.back();
      stack.pop_back();
      if (id < 256) s.push_back((char)id);
      else if (id - 256 < (int)t->merges.size()) {
        stack.push_back(t->merges[id - 256].second);
        stack.push_back(t->merges[id - 256].first);
      }
    }
  }
  if ((long long)s.size() > cap) return -(long long)s.size();
  memcpy(out, s.data(), s.size());
  return (long long)s.size();
}

int sx_tok_save(void* h, const char* path) {
  Tok* t = static_cast<Tok*>(h);
  FILE* f = fopen(path, "w");
  if (!f) return -1;
  fprintf(f, "sneppx-bpe 1 %zu\n", t->merges.size());
  for (auto& m : t->merges) fprintf(f, "%d %d\n", m.first, m.second);
  fclose(f);
  return 0;
}
int sx_tok_load(void* h, const char* path) {
  Tok* t = static_cast<Tok*>(h);
  FILE* f = fopen(path, "r");
  if (!f) return -1;
  size_t n = 0;
  int ver = 0;
  if (fscanf(f, "sneppx-bpe %d %zu", &ver, &n) != 2 || n > (1u << 22)) { fclose(f); return -2; }
  std::vector<std::pair<int, int>> merges(n);
  for (size_t i = 0; i < n; ++i) {
    // merge i creates token 256 + i out of two tokens that already exist
    if (fscanf(f, "%d %d", &merges[i].first, &merges[i].second) != 2 || merges[i].first < 0 || merges[i].second < 0 ||
        merges[i].first >= 256 + (int)i || merges[i].second >= 256 + (int)i) { fclose(f); return -3; }
  }
  fclose(f);
  t->merges.swap(merges);
  t->rebuild();
  return 0;
}
}
