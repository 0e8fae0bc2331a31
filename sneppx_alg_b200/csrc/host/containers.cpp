// Small containers of the host runtime with a C interface: an open-addressing hash table (64-bit keys, robin-hood
// probing, tombstone-free backward-shift deletion), a binary-heap priority queue (smallest priority first, FIFO among
// equal priorities), a red-black tree (ordered 64-bit keys with min / max / successor / predecessor / in-order walk)
// and bounded string helpers. Values are opaque 64-bit words (pointers or integers).
// Same roles as the reference's lib/internal/{hashtable,pqueue,rbtree,strutil}.c; written from the textbook algorithms.
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace {

// ---------------------------------------------------------------- hash table
uint64_t mix(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ull;
  return x ^ (x >> 33);
}
struct Slot {
  uint64_t key, value;
  uint32_t dist;   // probe distance + 1; 0 = empty
};
struct HashTable {
  std::vector<Slot> slots;
  size_t count = 0;
};
void ht_rehash(HashTable* h, size_t cap);
long long ht_find(const HashTable* h, uint64_t key);
int ht_put(HashTable* h, uint64_t key, uint64_t value) {
  const long long at = ht_find(h, key);
  if (at >= 0) {
    h->slots[(size_t)at].value = value;
    return 1;
  }
  if ((h->count + 1) * 10 > h->slots.size() * 7) ht_rehash(h, h->slots.size() * 2);
  const size_t mask = h->slots.size() - 1;
  size_t i = mix(key) & mask;
  Slot cur{key, value, 1};
  while (true) {
    Slot& s = h->slots[i];
    if (s.dist == 0) {
      s = cur;
      h->count++;
      return 0;
    }
    if (s.dist < cur.dist) std::swap(s, cur);   // robin hood: the entry closer to its home gives way
    cur.dist++;
    i = (i + 1) & mask;
  }
}
void ht_rehash(HashTable* h, size_t cap) {
  size_t n = 8;
  while (n < cap) n <<= 1;
  std::vector<Slot> old;
  old.swap(h->slots);
  h->slots.assign(n, Slot{0, 0, 0});
  h->count = 0;
  for (auto& s : old)
    if (s.dist) ht_put(h, s.key, s.value);
}
long long ht_find(const HashTable* h, uint64_t key) {
  const size_t mask = h->slots.size() - 1;
  size_t i = mix(key) & mask;
  uint32_t d = 1;
  while (true) {
    const Slot& s = h->slots[i];
    if (s.dist == 0 || s.dist < d) return -1;
    if (s.key == key) return (long long)i;
    ++d;
    i = (i + 1) & mask;
  }
}

// ---------------------------------------------------------------- priority queue
struct PqItem {
  uint64_t priority, seq, value;
};
struct PQueue {
  std::vector<PqItem> heap;
  uint64_t seq = 0;
};
bool pq_less(const PqItem& a, const PqItem& b) { return a.priority != b.priority ? a.priority < b.priority : a.seq < b.seq; }
void pq_down(PQueue* q, size_t i) {
  const size_t n = q->heap.size();
  while (true) {
    size_t l = 2 * i + 1, r = l + 1, m = i;
    if (l < n && pq_less(q->heap[l], q->heap[m])) m = l;
    if (r < n && pq_less(q->heap[r], q->heap[m])) m = r;
    if (m == i) return;
    std::swap(q->heap[i], q->heap[m]);
    i = m;
  }
}

// ---------------------------------------------------------------- red-black tree
struct Node {
  uint64_t key, value;
  Node *l, *r, *p;
  bool red;
};
struct RBTree {
  Node* root = nullptr;
  size_t count = 0;
};
void rot_left(RBTree* t, Node* x) {
  Node* y = x->r;
  x->r = y->l;
  if (y->l) y->l->p = x;
  y->p = x->p;
  if (!x->p) t->root = y;
  else if (x == x->p->l) x->p->l = y;
  else x->p->r = y;
  y->l = x;
  x->p = y;
}
void rot_right(RBTree* t, Node* x) {
  Node* y = x->l;
  x->l = y->r;
  if (y->r) y->r->p = x;
  y->p = x->p;
  if (!x->p) t->root = y;
  else if (x == x->p->r) x->p->r = y;
  else x->p->l = y;
  y->r = x;
  x->p = y;
}
Node* rb_find(const RBTree* t, uint64_t k) {
  Node* n = t->root;
  while (n && n->key != k) n = k < n->key ? n->l : n->r;
  return n;
}
Node* rb_min(Node* n) {
  while (n && n->l) n = n->l;
  return n;
}
Node* rb_max(Node* n) {
  while (n && n->r) n = n->r;
  return n;
}
bool is_red(Node* n) { return n && n->red; }
void insert_fix(RBTree* t, Node* z) {
  while (z->p && z->p->red) {
    Node* g = z->p->p;
    if (z->p == g->l) {
      Node* u = g->r;
      if (is_red(u)) {
        z->p->red = false; u->red = false; g->red = true; z = g;
      } else {
        if (z == z->p->r) { z = z->p; rot_left(t, z); }
        z->p->red = false; g->red = true; rot_right(t, g);
      }
    } else {
      Node* u = g->l;
      if (is_red(u)) {
        z->p->red = false; u->red = false; g->red = true; z = g;
      } else {
        if (z == z->p->l) { z = z->p; rot_right(t, z); }
        z->p->red = false; g->red = true; rot_left(t, g);
      }
    }
  }
  t->root->red = false;
}
void transplant(RBTree* t, Node* u, Node* v) {
  if (!u->p) t->root = v;
  else if (u == u->p->l) u->p->l = v;
  else u->p->r = v;
  if (v) v->p = u->p;
}
void delete_fix(RBTree* t, Node* x, Node* xp) {
  while (x != t->root && !is_red(x)) {
    if (x == xp->l) {
      Node* w = xp->r;
      if (is_red(w)) { w->red = false; xp->red = true; rot_left(t, xp); w = xp->r; }
      if (!is_red(w->l) && !is_red(w->r)) { w->red = true; x = xp; xp = x->p; }
      else {
        if (!is_red(w->r)) { if (w->l) w->l->red = false; w->red = true; rot_right(t, w); w = xp->r; }
        w->red = xp->red; xp->red = false; if (w->r) w->r->red = false; rot_left(t, xp); x = t->root; break;
      }
    } else {
      Node* w = xp->l;
      if (is_red(w)) { w->red = false; xp->red = true; rot_right(t, xp); w = xp->l; }
      if (!is_red(w->l) && !is_red(w->r)) { w->red = true; x = xp; xp = x->p; }
      else {
        if (!is_red(w->l)) { if (w->r) w->r->red = false; w->red = true; rot_left(t, w); w = xp->l; }
        w->red = xp->red; xp->red = false; if (w->l) w->l->red = false; rot_right(t, xp); x = t->root; break;
      }
    }
  }
  if (x) x->red = false;
}
void rb_free(Node* n) {
  if (!n) return;
  rb_free(n->l);
  rb_free(n->r);
  delete n;
}
// black height, or -1 when a red-black rule is broken (tests)
int rb_check(Node* n, uint64_t lo, uint64_t hi, bool has_lo, bool has_hi) {
  if (!n) return 1;
  if ((has_lo && n->key <= lo) || (has_hi && n->key >= hi)) return -1;
  if (n->red && (is_red(n->l) || is_red(n->r))) return -1;
  const int a = rb_check(n->l, lo, n->key, has_lo, true), b = rb_check(n->r, n->key, hi, true, has_hi);
  if (a < 0 || b < 0 || a != b) return -1;
  return a + (n->red ? 0 : 1);
}

}  // namespace

extern "C" {

// ---- hash table
void* sx_ht_create(size_t cap) {
  HashTable* h = new HashTable();
  ht_rehash(h, cap < 8 ? 8 : cap);
  return h;
}
void sx_ht_destroy(void* h) { delete static_cast<HashTable*>(h); }
// 0 inserted, 1 replaced an existing value
int sx_ht_insert(void* h, unsigned long long key, unsigned long long value) { return ht_put(static_cast<HashTable*>(h), key, value); }
int sx_ht_lookup(void* h, unsigned long long key, unsigned long long* value) {
  HashTable* t = static_cast<HashTable*>(h);
  const long long i = ht_find(t, key);
  if (i < 0) return 0;
  if (value) *value = t->slots[(size_t)i].value;
  return 1;
}
int sx_ht_delete(void* h, unsigned long long key) {
  HashTable* t = static_cast<HashTable*>(h);
  long long i = ht_find(t, key);
  if (i < 0) return 0;
  const size_t mask = t->slots.size() - 1;
  size_t cur = (size_t)i;
  while (true) {   // backward shift: pull the following entries one slot closer to their home
    const size_t nxt = (cur + 1) & mask;
    if (t->slots[nxt].dist <= 1) break;
    t->slots[cur] = t->slots[nxt];
    t->slots[cur].dist--;
    cur = nxt;
  }
  t->slots[cur] = Slot{0, 0, 0};
  t->count--;
  return 1;
}
size_t sx_ht_size(void* h) { return static_cast<HashTable*>(h)->count; }
size_t sx_ht_capacity(void* h) { return static_cast<HashTable*>(h)->slots.size(); }
void sx_ht_clear(void* h) {
  HashTable* t = static_cast<HashTable*>(h);
  t->slots.assign(t->slots.size(), Slot{0, 0, 0});
  t->count = 0;
}
int sx_ht_resize(void* h, size_t cap) {
  HashTable* t = static_cast<HashTable*>(h);
  if (cap * 7 < t->count * 10) return -1;
  ht_rehash(t, cap);
  return 0;
}
void sx_ht_foreach(void* h, void (*fn)(unsigned long long, unsigned long long, void*), void* ctx) {
  for (auto& s : static_cast<HashTable*>(h)->slots)
    if (s.dist) fn(s.key, s.value, ctx);
}
// longest probe sequence in the table (a quality measure of the hashing)
int sx_ht_max_probe(void* h) {
  uint32_t m = 0;
  for (auto& s : static_cast<HashTable*>(h)->slots) m = s.dist > m ? s.dist : m;
  return (int)m;
}

// ---- priority queue
void* sx_pq_create(size_t cap) {
  PQueue* q = new PQueue();
  q->heap.reserve(cap);
  return q;
}
void sx_pq_destroy(void* q) { delete static_cast<PQueue*>(q); }
int sx_pq_push(void* qh, unsigned long long priority, unsigned long long value) {
  PQueue* q = static_cast<PQueue*>(qh);
  q->heap.push_back({priority, q->seq++, value});
  size_t i = q->heap.size() - 1;
  while (i > 0) {
    const size_t p = (i - 1) / 2;
    if (!pq_less(q->heap[i], q->heap[p])) break;
    std::swap(q->heap[i], q->heap[p]);
    i = p;
  }
  return 0;
}
int sx_pq_peek(void* qh, unsigned long long* priority, unsigned long long* value) {
  PQueue* q = static_cast<PQueue*>(qh);
  if (q->heap.empty()) return 0;
  if (priority) *priority = q->heap[0].priority;
  if (value) *value = q->heap[0].value;
  return 1;
}
int sx_pq_pop(void* qh, unsigned long long* priority, unsigned long long* value) {
  PQueue* q = static_cast<PQueue*>(qh);
  if (!sx_pq_peek(qh, priority, value)) return 0;
  q->heap[0] = q->heap.back();
  q->heap.pop_back();
  if (!q->heap.empty()) pq_down(q, 0);
  return 1;
}
size_t sx_pq_size(void* q) { return static_cast<PQueue*>(q)->heap.size(); }
int sx_pq_is_empty(void* q) { return static_cast<PQueue*>(q)->heap.empty() ? 1 : 0; }
void sx_pq_clear(void* q) { static_cast<PQueue*>(q)->heap.clear(); }

// ---- red-black tree
void* sx_rbtree_create(void) { return new RBTree(); }
void sx_rbtree_destroy(void* t) {
  rb_free(static_cast<RBTree*>(t)->root);
  delete static_cast<RBTree*>(t);
}
// 0 inserted, 1 replaced
int sx_rbtree_insert(void* th, unsigned long long key, unsigned long long value) {
  RBTree* t = static_cast<RBTree*>(th);
  Node *y = nullptr, *x = t->root;
  while (x) {
    y = x;
    if (key == x->key) {
      x->value = value;
      return 1;
    }
    x = key < x->key ? x->l : x->r;
  }
  Node* z = new Node{key, value, nullptr, nullptr, y, true};
  if (!y) t->root = z;
  else if (key < y->key) y->l = z;
  else y->r = z;
  t->count++;
  insert_fix(t, z);
  return 0;
}
int sx_rbtree_search(void* t, unsigned long long key, unsigned long long* value) {
  Node* n = rb_find(static_cast<RBTree*>(t), key);
  if (!n) return 0;
  if (value) *value = n->value;
  return 1;
}
int sx_rbtree_delete(void* th, unsigned long long key) {
  RBTree* t = static_cast<RBTree*>(th);
  Node* z = rb_find(t, key);
  if (!z) return 0;
  Node *y = z, *x, *xp;
  bool y_red = y->red;
  if (!z->l) {
    x = z->r; xp = z->p; transplant(t, z, z->r);
  } else if (!z->r) {
    x = z->l; xp = z->p; transplant(t, z, z->l);
  } else {
    y = rb_min(z->r);
    y_red = y->red;
    x = y->r;
    if (y->p == z) xp = y;
    else {
      xp = y->p;
      transplant(t, y, y->r);
      y->r = z->r;
      y->r->p = y;
    }
    transplant(t, z, y);
    y->l = z->l;
    y->l->p = y;
    y->red = z->red;
  }
  delete z;
  t->count--;
  if (!y_red && t->root) delete_fix(t, x, xp);
  return 1;
}
size_t sx_rbtree_size(void* t) { return static_cast<RBTree*>(t)->count; }
int sx_rbtree_min(void* t, unsigned long long* key) {
  Node* n = rb_min(static_cast<RBTree*>(t)->root);
  if (!n) return 0;
  *key = n->key;
  return 1;
}
int sx_rbtree_max(void* t, unsigned long long* key) {
  Node* n = rb_max(static_cast<RBTree*>(t)->root);
  if (!n) return 0;
  *key = n->key;
  return 1;
}
// smallest key greater than `key` (the key itself need not be present)
int sx_rbtree_successor(void* t, unsigned long long key, unsigned long long* out) {
  Node *n = static_cast<RBTree*>(t)->root, *best = nullptr;
  while (n) {
    if (n->key > key) { best = n; n = n->l; }
    else n = n->r;
  }
  if (!best) return 0;
  *out = best->key;
  return 1;
}
int sx_rbtree_predecessor(void* t, unsigned long long key, unsigned long long* out) {
  Node *n = static_cast<RBTree*>(t)->root, *best = nullptr;
  while (n) {
    if (n->key < key) { best = n; n = n->r; }
    else n = n->l;
  }
  if (!best) return 0;
  *out = best->key;
  return 1;
}
void sx_rbtree_foreach(void* t, void (*fn)(unsigned long long, unsigned long long, void*), void* ctx) {
  std::vector<Node*> st;
  Node* n = static_cast<RBTree*>(t)->root;
  while (n || !st.empty()) {
    while (n) { st.push_back(n); n = n->l; }
    n = st.back();
    st.pop_back();
    fn(n->key, n->value, ctx);
    n = n->r;
  }
}
// black height (>= 1) when every red-black and ordering rule holds, else -1
int sx_rbtree_validate(void* t) {
  RBTree* tr = static_cast<RBTree*>(t);
  if (is_red(tr->root)) return -1;
  return rb_check(tr->root, 0, 0, false, false);
}

// ---- strings
size_t sx_strlcpy(char* dst, const char* src, size_t cap) {
  const size_t n = std::strlen(src);
  if (cap) {
    const size_t c = n < cap - 1 ? n : cap - 1;
    std::memcpy(dst, src, c);
    dst[c] = 0;
  }
  return n;
}
size_t sx_strlcat(char* dst, const char* src, size_t cap) {
  size_t d = 0;
  while (d < cap && dst[d]) ++d;
  if (d == cap) return cap + std::strlen(src);
  return d + sx_strlcpy(dst + d, src, cap - d);
}
void* sx_strbuf_create(size_t cap) {
  std::string* s = new std::string();
  s->reserve(cap);
  return s;
}
void sx_strbuf_destroy(void* s) { delete static_cast<std::string*>(s); }
int sx_strbuf_append_n(void* s, const char* src, size_t n) {
  static_cast<std::string*>(s)->append(src, n);
  return 0;
}
int sx_strbuf_append(void* s, const char* src) { return sx_strbuf_append_n(s, src, std::strlen(src)); }
int sx_strbuf_format(void* s, const char* fmt, ...) {
  va_list ap, ap2;
  va_start(ap, fmt);
  va_copy(ap2, ap);
  const int n = std::vsnprintf(nullptr, 0, fmt, ap);
  va_end(ap);
  if (n < 0) {
    va_end(ap2);
    return -1;
  }
  std::string tmp((size_t)n + 1, '\0');
  std::vsnprintf(&tmp[0], tmp.size(), fmt, ap2);
  va_end(ap2);
  static_cast<std::string*>(s)->append(tmp.c_str(), (size_t)n);
  return n;
}
void sx_strbuf_clear(void* s) { static_cast<std::string*>(s)->clear(); }
size_t sx_strbuf_length(void* s) { return static_cast<std::string*>(s)->size(); }
const char* sx_strbuf_cstr(void* s) { return static_cast<std::string*>(s)->c_str(); }
// Writes the tokens NUL-separated into out (cap bytes); returns the number of tokens found (empty tokens included),
// or -1 when out is too small.
long long sx_strsplit(const char* str, char delim, char* out, size_t cap, size_t max_tokens) {
  size_t off = 0;
  long long n = 0;
  const char* p = str;
  while (true) {
    const char* e = std::strchr(p, delim);
    const bool last = !e || (max_tokens && (size_t)n + 1 == max_tokens);
    const size_t len = last ? std::strlen(p) : (size_t)(e - p);
    if (off + len + 1 > cap) return -1;
    std::memcpy(out + off, p, len);
    out[off + len] = 0;
    off += len + 1;
    ++n;
    if (last) break;
    p = e + 1;
  }
  return n;
}
// Joins `count` NUL-terminated tokens; returns the length needed (without the terminator).
size_t sx_strjoin(const char* const* tokens, size_t count, char delim, char* out, size_t cap) {
  size_t need = 0;
  for (size_t i = 0; i < count; ++i) need += std::strlen(tokens[i]) + (i + 1 < count ? 1 : 0);
  if (out && cap > need) {
    size_t off = 0;
    for (size_t i = 0; i < count; ++i) {
      const size_t l = std::strlen(tokens[i]);
      std::memcpy(out + off, tokens[i], l);
      off += l;
      if (i + 1 < count) out[off++] = delim;
    }
    out[off] = 0;
  }
  return need;
}

}  // extern "C"
