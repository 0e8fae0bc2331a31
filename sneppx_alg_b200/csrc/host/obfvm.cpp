// S2 code obfuscation for native logic: a small register IR with control-flow graphs, a control-flow flattening
// pass, a bytecode compiler whose opcode encoding is private to each compiled program, the virtual machine that
// runs it, sealed string tables and debugger detection.
//
//   IR            blocks of register instructions (16 x int64 registers), each ending in jmp / conditional jump /
//                 ret; written as text: "entry: movi r0 5 ; cmpi r0 3 ; jg big small" (labels, ';' or newlines)
//   flattening    every block gets a random 31-bit state id; terminators no longer jump to their successors but
//                 store the successor's id in r15 (conditional ones pick between two ids with a select) and jump to
//                 a dispatcher that compares r15 against every id: the static graph becomes a star
//   bytecode      8 bytes per instruction; the opcode byte is permuted by a per-program table and masked with a
//                 byte derived from the instruction's position and the program key, so equal instructions encode
//                 differently and the table cannot be read off one sample
//   VM            validates register indices and jump targets before running, counts steps (limit), returns the
//                 value given to ret and the values passed to out
//   strings       sealed with ChaCha20 under (key, string id); opened into a caller buffer that is wiped on request
//   debugger      TracerPid in /proc/self/status, LD_PRELOAD set, and a timing probe around a fixed busy loop
// Behavioural counterparts: security/obfuscation/cfg_flatten.cpp:30-140 (state ids + dispatcher),
// security/obfuscation/vm.cpp:38-519 (encrypted handler table, compile_to_bytecode, validate, execute),
// security/obfuscation/string_encrypt.cpp, security/obfuscation/debug_detect.cpp.
#include <unistd.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <random>
#include <sstream>
#include <string>
#include <vector>

extern "C" void sx_chacha20(const uint8_t* key32, uint32_t counter, const uint8_t* nonce12, const uint8_t* in, uint8_t* out,
                            size_t n);

namespace {

enum OpCode : uint8_t { MOVI, MOV, ADD, SUB, MUL, XOR, AND, OR, ADDI, CMP, CMPI, JMP, JZ, JNZ, JG, JLE, RET, OUT, SEL, NOPC, N_OPS };
const char* NAMES[N_OPS] = {"movi", "mov", "add", "sub", "mul", "xor", "and", "or", "addi", "cmp",
                            "cmpi", "jmp", "jz", "jnz", "jg", "jle", "ret", "out", "sel", "nop"};

struct Inst {
  uint8_t op;
  uint8_t d = 0, s = 0;
  int64_t imm = 0;
  int target = -1, target2 = -1;   // block indices (jumps); target2: fall-through successor of a conditional jump
};
struct Block {
  std::string label;
  std::vector<Inst> body;           // the last one is the terminator
};
struct Cfg {
  std::vector<Block> blocks;
  bool flattened = false;
  std::string error;
};

bool is_cond(uint8_t op) { return op == JZ || op == JNZ || op == JG || op == JLE; }
bool is_term(uint8_t op) { return op == JMP || is_cond(op) || op == RET; }

bool parse_reg(const std::string& t, uint8_t& r) {
  if (t.size() < 2 || t[0] != 'r') return false;
  char* end;
  const long v = std::strtol(t.c_str() + 1, &end, 10);
  if (*end || v < 0 || v > 15) return false;
  r = (uint8_t)v;
  return true;
}

Cfg* parse(const char* text) {
  Cfg* g = new Cfg();
  std::string src(text);
  for (char& c : src)
    if (c == ';') c = '\n';
  std::istringstream in(src);
  std::string line;
  struct Pending { int block, inst; std::string a, b; };
  std::vector<Pending> fix;
  std::map<std::string, int> labels;
  auto fail = [&](const std::string& m) {
    g->error = m;
    return g;
  };
  while (std::getline(in, line)) {
    std::istringstream ls(line);
    std::vector<std::string> tok;
    std::string t;
    while (ls >> t) tok.push_back(t);
    if (tok.empty() || tok[0][0] == '#') continue;
    if (tok[0].back() == ':') {
      const std::string name = tok[0].substr(0, tok[0].size() - 1);
      if (labels.count(name)) return fail("duplicate label " + name);
      labels[name] = (int)g->blocks.size();
      g->blocks.push_back(Block{name, {}});
      tok.erase(tok.begin());
      if (tok.empty()) continue;
    }
    if (g->blocks.empty()) {
      labels["entry"] = 0;
      g->blocks.push_back(Block{"entry", {}});
    }
    int op = -1;
    for (int i = 0; i < N_OPS; ++i)
      if (tok[0] == NAMES[i]) op = i;
    if (op < 0 || op == SEL) return fail("unknown instruction " + tok[0]);
    Inst ins;
    ins.op = (uint8_t)op;
    auto need = [&](size_t n) { return tok.size() == n + 1; };
    switch (op) {
      case MOVI: case ADDI: case CMPI:
        if (!need(2) || !parse_reg(tok[1], ins.d)) return fail("bad operands: " + line);
        ins.imm = std::strtoll(tok[2].c_str(), nullptr, 0);
        break;
      case MOV: case ADD: case SUB: case MUL: case XOR: case AND: case OR: case CMP:
        if (!need(2) || !parse_reg(tok[1], ins.d) || !parse_reg(tok[2], ins.s)) return fail("bad operands: " + line);
        break;
      case RET: case OUT:
        if (!need(1) || !parse_reg(tok[1], ins.s)) return fail("bad operands: " + line);
        break;
      case JMP:
        if (!need(1)) return fail("bad operands: " + line);
        fix.push_back({(int)g->blocks.size() - 1, (int)g->blocks.back().body.size(), tok[1], ""});
        break;
      case JZ: case JNZ: case JG: case JLE:
        if (!need(2)) return fail("conditional jumps name both successors: " + line);
        fix.push_back({(int)g->blocks.size() - 1, (int)g->blocks.back().body.size(), tok[1], tok[2]});
        break;
      default:
        break;
    }
    if (ins.d == 15 || (ins.s == 15 && op != RET && op != OUT && op != CMP && op != MOV))
      if (op != NOPC && !is_term(ins.op)) return fail("r15 is reserved for the dispatcher: " + line);
    Block& b = g->blocks.back();
    if (!b.body.empty() && is_term(b.body.back().op)) return fail("instruction after a terminator in block " + b.label);
    b.body.push_back(ins);
  }
  for (auto& f : fix) {
    if (!labels.count(f.a) || (!f.b.empty() && !labels.count(f.b))) return fail("unknown label " + (labels.count(f.a) ? f.b : f.a));
    g->blocks[f.block].body[f.inst].target = labels[f.a];
    if (!f.b.empty()) g->blocks[f.block].body[f.inst].target2 = labels[f.b];
  }
  for (auto& b : g->blocks)
    if (b.body.empty() || !is_term(b.body.back().op)) return fail("block " + b.label + " does not end in jmp / conditional jump / ret");
  return g;
}

// Reference interpreter over the IR (what the bytecode must reproduce).
int run_ir(const Cfg& g, const int64_t* in, int n_in, int64_t* out, int out_cap, int* n_out, int64_t* ret, long long step_limit) {
  int64_t r[16] = {0};
  for (int i = 0; i < n_in && i < 8; ++i) r[i] = in[i];
  int64_t flag = 0;
  int blk = 0;
  long long steps = 0;
  *n_out = 0;
  while (true) {
    for (const Inst& x : g.blocks[blk].body) {
      if (++steps > step_limit) return -2;
      switch (x.op) {
        case MOVI: r[x.d] = x.imm; break;
        case MOV: r[x.d] = r[x.s]; break;
        case ADD: r[x.d] += r[x.s]; break;
        case SUB: r[x.d] -= r[x.s]; break;
        case MUL: r[x.d] *= r[x.s]; break;
        case XOR: r[x.d] ^= r[x.s]; break;
        case AND: r[x.d] &= r[x.s]; break;
        case OR: r[x.d] |= r[x.s]; break;
        case ADDI: r[x.d] += x.imm; break;
        case CMP: flag = r[x.d] - r[x.s]; break;
        case CMPI: flag = r[x.d] - x.imm; break;
        case SEL: r[x.d] = ((x.s == JZ && flag == 0) || (x.s == JNZ && flag != 0) || (x.s == JG && flag > 0) || (x.s == JLE && flag <= 0))
                               ? (x.imm >> 32) : (x.imm & 0xffffffff); break;
        case OUT: if (*n_out < out_cap) out[(*n_out)++] = r[x.s]; break;
        case RET: *ret = r[x.s]; return 0;
        case JMP: blk = x.target; break;
        case JZ: blk = flag == 0 ? x.target : x.target2; break;
        case JNZ: blk = flag != 0 ? x.target : x.target2; break;
        case JG: blk = flag > 0 ? x.target : x.target2; break;
        case JLE: blk = flag <= 0 ? x.target : x.target2; break;
        default: break;
      }
    }
  }
}

void flatten(Cfg& g, uint64_t seed) {
  if (g.flattened || g.blocks.empty()) return;
  std::mt19937_64 rng(seed);
  const int n = (int)g.blocks.size();
  std::vector<int64_t> id(n);
  for (int i = 0; i < n; ++i) {
    bool fresh;
    do {
      id[i] = (int64_t)(rng() & 0x7fffffff) | 1;
      fresh = true;
      for (int j = 0; j < i; ++j) fresh = fresh && id[j] != id[i];
    } while (!fresh);
  }
  // block order is shuffled as well: position says nothing about the original order
  std::vector<int> order(n);
  for (int i = 0; i < n; ++i) order[i] = i;
  for (int i = n - 1; i > 0; --i) std::swap(order[i], order[rng() % (i + 1)]);
  std::vector<int> newpos(n);
  for (int i = 0; i < n; ++i) newpos[order[i]] = i + 2;       // 0: prologue, 1: dispatcher
  std::vector<Block> out;
  Block pro{"__enter", {}};
  pro.body.push_back(Inst{MOVI, 15, 0, id[0]});
  pro.body.push_back(Inst{JMP, 0, 0, 0, 1});
  out.push_back(pro);
  out.push_back(Block{"__dispatch", {}});
  for (int k = 0; k < n; ++k) {
    Block b = g.blocks[order[k]];
    Inst term = b.body.back();
    b.body.pop_back();
    if (term.op == JMP) {
      b.body.push_back(Inst{MOVI, 15, 0, id[term.target]});
      b.body.push_back(Inst{JMP, 0, 0, 0, 1});
    } else if (is_cond(term.op)) {
      Inst sel{SEL, 15, term.op, (int64_t)(((uint64_t)id[term.target] << 32) | (uint64_t)id[term.target2])};
      b.body.push_back(sel);
      b.body.push_back(Inst{JMP, 0, 0, 0, 1});
    } else {
      b.body.push_back(term);
    }
    out.push_back(b);
  }
  // dispatcher: a chain of compare-and-branch blocks, one per state, in shuffled order
  Block& disp = out[1];
  std::vector<int> probe(n);
  for (int i = 0; i < n; ++i) probe[i] = i;
  for (int i = n - 1; i > 0; --i) std::swap(probe[i], probe[rng() % (i + 1)]);
  // dispatcher block k compares against one id; its miss edge goes to the next dispatcher block (appended after the
  // real blocks); the last miss edge loops to a trap block that returns -1 (unreachable for valid states)
  const int first_extra = (int)out.size();
  for (int k = 0; k < n; ++k) {
    Block* cur = k == 0 ? &disp : nullptr;
    Block extra{"__d" + std::to_string(k), {}};
    if (!cur) cur = &extra;
    const int o = probe[k];
    cur->body.push_back(Inst{CMPI, 15, 0, id[o]});
    Inst j{JZ, 0, 0, 0, newpos[o], -1};          // the miss edge is filled in below
    cur->body.push_back(j);
    if (k > 0) out.push_back(extra);
  }
  Block trap{"__trap", {}};
  trap.body.push_back(Inst{MOVI, 14, 0, -1});
  trap.body.push_back(Inst{RET, 0, 14, 0});
  out.push_back(trap);
  // fix the miss edges: dispatcher k (k >= 1) lives at first_extra + k - 1, the trap at first_extra + n - 1
  for (int k = 0; k < n; ++k) {
    Block& b = k == 0 ? out[1] : out[first_extra + k - 1];
    b.body.back().target2 = (k + 1 < n) ? first_extra + k : first_extra + n - 1;
  }
  g.blocks = out;
  g.flattened = true;
}

// ---------------------------------------------------------------- bytecode
struct Program {
  std::vector<uint8_t> code;      // 8 bytes per instruction + conditional jumps carry a second word
  uint8_t perm[N_OPS], inv[256];
  uint8_t key[8];
};

uint8_t pos_mask(const uint8_t key[8], uint32_t ip) {
  uint32_t x = ip * 2654435761u;
  x ^= x >> 15;
  return (uint8_t)(x ^ key[ip & 7] ^ (x >> 8));
}

Program* compile(const Cfg& g, uint64_t seed) {
  Program* p = new Program();
  std::mt19937_64 rng(seed ^ 0x9e3779b97f4a7c15ull);
  uint8_t all[256];
  for (int i = 0; i < 256; ++i) all[i] = (uint8_t)i;
  for (int i = 255; i > 0; --i) std::swap(all[i], all[rng() % (i + 1)]);
  std::memset(p->inv, 0xff, sizeof p->inv);
  for (int i = 0; i < N_OPS; ++i) {
    p->perm[i] = all[i];
    p->inv[all[i]] = (uint8_t)i;
  }
  for (auto& k : p->key) k = (uint8_t)rng();
  // layout: block start offsets (in instruction words)
  std::vector<uint32_t> start(g.blocks.size());
  uint32_t ip = 0;
  for (size_t b = 0; b < g.blocks.size(); ++b) {
    start[b] = ip;
    for (const Inst& x : g.blocks[b].body) ip += (is_cond(x.op) || x.op == SEL) ? 2 : 1;
  }
  p->code.resize((size_t)ip * 8);
  ip = 0;
  auto emit = [&](uint8_t op, uint8_t d, uint8_t s, uint32_t lo, uint16_t hi16) {
    uint8_t* w = p->code.data() + (size_t)ip * 8;
    w[0] = p->perm[op] ^ pos_mask(p->key, ip);
    w[1] = d ^ p->key[(ip + 1) & 7];
    w[2] = s ^ p->key[(ip + 2) & 7];
    w[3] = (uint8_t)(hi16 & 0xff);
    std::memcpy(w + 4, &lo, 4);
    ++ip;
  };
  auto emit_raw64 = [&](uint64_t v) {
    v ^= 0xA5A5A5A5A5A5A5A5ull * (uint64_t)(p->key[ip & 7] | 1);
    std::memcpy(p->code.data() + (size_t)ip * 8, &v, 8);
    ++ip;
  };
  for (const Block& b : g.blocks)
    for (const Inst& x : b.body) {
      if (x.op == JMP) emit(JMP, 0, 0, start[x.target], 0);
      else if (is_cond(x.op)) {
        emit(x.op, 0, 0, start[x.target], 0);
        emit_raw64(start[x.target2]);
      } else if (x.op == SEL) {
        emit(SEL, x.d, x.s, 0, 0);
        emit_raw64((uint64_t)x.imm);
      } else {
        // 32-bit immediates inline; MOVI with a wider value is split by the parser's range (kept to int32 here)
        emit(x.op, x.d, x.s, (uint32_t)(int32_t)x.imm, 0);
      }
    }
  return p;
}

struct Decoded {
  uint8_t op, d, s;
  int32_t imm;
};
bool decode(const Program& p, uint32_t ip, Decoded& o) {
  const uint8_t* w = p.code.data() + (size_t)ip * 8;
  const uint8_t raw = w[0] ^ pos_mask(p.key, ip);
  if (p.inv[raw] == 0xff) return false;
  o.op = p.inv[raw];
  o.d = w[1] ^ p.key[(ip + 1) & 7];
  o.s = w[2] ^ p.key[(ip + 2) & 7];
  std::memcpy(&o.imm, w + 4, 4);
  return true;
}
uint64_t raw64(const Program& p, uint32_t ip) {
  uint64_t v;
  std::memcpy(&v, p.code.data() + (size_t)ip * 8, 8);
  return v ^ (0xA5A5A5A5A5A5A5A5ull * (uint64_t)(p.key[ip & 7] | 1));
}

// 0 ok; -1 undecodable opcode, -3 register out of range, -4 jump target out of range, -5 truncated
int validate(const Program& p) {
  const uint32_t n = (uint32_t)(p.code.size() / 8);
  for (uint32_t ip = 0; ip < n; ++ip) {
    Decoded x;
    if (!decode(p, ip, x)) return -1;
    if (x.op != SEL && (x.d > 15 || x.s > 15)) return -3;
    if (x.op == SEL && x.d > 15) return -3;
    if (x.op == JMP && (uint32_t)x.imm >= n) return -4;
    if (is_cond(x.op)) {
      if (ip + 1 >= n) return -5;
      if ((uint32_t)x.imm >= n || raw64(p, ip + 1) >= n) return -4;
      ++ip;
    } else if (x.op == SEL) {
      if (ip + 1 >= n) return -5;
      ++ip;
    }
  }
  return 0;
}

int execute(const Program& p, const int64_t* in, int n_in, int64_t* out, int out_cap, int* n_out, int64_t* ret,
            long long step_limit) {
  const int v = validate(p);
  if (v) return v;
  const uint32_t n = (uint32_t)(p.code.size() / 8);
  int64_t r[16] = {0};
  for (int i = 0; i < n_in && i < 8; ++i) r[i] = in[i];
  int64_t flag = 0;
  uint32_t ip = 0;
  long long steps = 0;
  *n_out = 0;
  while (ip < n) {
    if (++steps > step_limit) return -2;
    Decoded x;
    decode(p, ip, x);
    switch (x.op) {
      case MOVI: r[x.d] = x.imm; ++ip; break;
      case MOV: r[x.d] = r[x.s]; ++ip; break;
      case ADD: r[x.d] += r[x.s]; ++ip; break;
      case SUB: r[x.d] -= r[x.s]; ++ip; break;
      case MUL: r[x.d] *= r[x.s]; ++ip; break;
      case XOR: r[x.d] ^= r[x.s]; ++ip; break;
      case AND: r[x.d] &= r[x.s]; ++ip; break;
      case OR: r[x.d] |= r[x.s]; ++ip; break;
      case ADDI: r[x.d] += x.imm; ++ip; break;
      case CMP: flag = r[x.d] - r[x.s]; ++ip; break;
      case CMPI: flag = r[x.d] - x.imm; ++ip; break;
      case OUT: if (*n_out < out_cap) out[(*n_out)++] = r[x.s]; ++ip; break;
      case RET: *ret = r[x.s]; return 0;
      case JMP: ip = (uint32_t)x.imm; break;
      case JZ: ip = flag == 0 ? (uint32_t)x.imm : (uint32_t)raw64(p, ip + 1); break;
      case JNZ: ip = flag != 0 ? (uint32_t)x.imm : (uint32_t)raw64(p, ip + 1); break;
      case JG: ip = flag > 0 ? (uint32_t)x.imm : (uint32_t)raw64(p, ip + 1); break;
      case JLE: ip = flag <= 0 ? (uint32_t)x.imm : (uint32_t)raw64(p, ip + 1); break;
      case SEL: {
        const uint64_t both = raw64(p, ip + 1);
        const bool take = (x.s == JZ && flag == 0) || (x.s == JNZ && flag != 0) || (x.s == JG && flag > 0) || (x.s == JLE && flag <= 0);
        r[x.d] = take ? (int64_t)(both >> 32) : (int64_t)(both & 0xffffffff);
        ip += 2;
        break;
      }
      default: ++ip; break;
    }
  }
  return -6;   // ran off the end without ret
}

}  // namespace

extern "C" {

void* sx_obf_parse(const char* text) { return parse(text); }
void sx_obf_cfg_free(void* g) { delete static_cast<Cfg*>(g); }
// empty string when the program parsed
const char* sx_obf_cfg_error(void* g) { return static_cast<Cfg*>(g)->error.c_str(); }
int sx_obf_cfg_blocks(void* g) { return (int)static_cast<Cfg*>(g)->blocks.size(); }
// number of distinct successor blocks of block i (what a static reader of the graph sees)
int sx_obf_cfg_successors(void* g, int i, int* out, int cap) {
  Cfg* c = static_cast<Cfg*>(g);
  if (i < 0 || (size_t)i >= c->blocks.size()) return -1;
  const Inst& t = c->blocks[(size_t)i].body.back();
  int n = 0;
  if (t.target >= 0 && n < cap) out[n++] = t.target;
  if (t.target2 >= 0 && t.target2 != t.target && n < cap) out[n++] = t.target2;
  return n;
}
void sx_obf_flatten(void* g, unsigned long long seed) {
  Cfg* c = static_cast<Cfg*>(g);
  if (c->error.empty()) flatten(*c, seed);
}
int sx_obf_run_ir(void* g, const long long* in, int n_in, long long* out, int out_cap, int* n_out, long long* ret,
                  long long step_limit) {
  Cfg* c = static_cast<Cfg*>(g);
  if (!c->error.empty()) return -7;
  return run_ir(*c, (const int64_t*)in, n_in, (int64_t*)out, out_cap, n_out, (int64_t*)ret, step_limit);
}
void* sx_obf_compile(void* g, unsigned long long seed) {
  Cfg* c = static_cast<Cfg*>(g);
  if (!c->error.empty()) return nullptr;
  for (auto& b : c->blocks)
    for (auto& x : b.body)
      if (x.op != SEL && (x.imm > INT32_MAX || x.imm < INT32_MIN)) return nullptr;   // immediates are 32 bit in bytecode
  return compile(*c, seed);
}
void sx_obf_program_free(void* p) { delete static_cast<Program*>(p); }
long long sx_obf_program_size(void* p) { return (long long)static_cast<Program*>(p)->code.size(); }
// copies the encoded bytes (for inspection / storage)
void sx_obf_program_bytes(void* p, unsigned char* out) {
  Program* pr = static_cast<Program*>(p);
  std::memcpy(out, pr->code.data(), pr->code.size());
}
// overwrite one encoded byte (tamper tests)
void sx_obf_program_poke(void* p, long long offset, unsigned char v) {
  Program* pr = static_cast<Program*>(p);
  if (offset >= 0 && (size_t)offset < pr->code.size()) pr->code[(size_t)offset] = v;
}
int sx_obf_validate(void* p) { return validate(*static_cast<Program*>(p)); }
int sx_obf_execute(void* p, const long long* in, int n_in, long long* out, int out_cap, int* n_out, long long* ret,
                   long long step_limit) {
  return execute(*static_cast<Program*>(p), (const int64_t*)in, n_in, (int64_t*)out, out_cap, n_out, (int64_t*)ret, step_limit);
}

// ---- sealed strings: out = ChaCha20(key, nonce = string id) xor in (the same call seals and opens)
void sx_obf_string_xform(const unsigned char* key32, unsigned long long id, const unsigned char* in, unsigned char* out, size_t n) {
  uint8_t nonce[12] = {0};
  std::memcpy(nonce, &id, 8);
  nonce[8] = 's';
  nonce[9] = 'x';
  sx_chacha20(key32, 1, nonce, in, out, n);
}
void sx_obf_wipe(void* p, size_t n) {
  volatile unsigned char* v = static_cast<volatile unsigned char*>(p);
  for (size_t i = 0; i < n; ++i) v[i] = 0;
}

// ---- debugger detection. bit 0: a tracer is attached (TracerPid != 0); bit 1: LD_PRELOAD is set; bit 2: the timing probe
// ran more than `slow_factor` times slower than its own best of three (single-stepping / heavy instrumentation).
int sx_obf_debugger_signals(double slow_factor) {
  int bits = 0;
  if (FILE* f = std::fopen("/proc/self/status", "r")) {
    char line[256];
    while (std::fgets(line, sizeof line, f))
      if (std::strncmp(line, "TracerPid:", 10) == 0 && std::atoi(line + 10) != 0) bits |= 1;
    std::fclose(f);
  }
  const char* pre = std::getenv("LD_PRELOAD");
  if (pre && *pre) bits |= 2;
  double best = 1e30, worst = 0;
  for (int rep = 0; rep < 3; ++rep) {
    const auto t0 = std::chrono::steady_clock::now();
    volatile uint64_t acc = 1;
    for (int i = 0; i < 200000; ++i) acc = acc * 6364136223846793005ull + 1442695040888963407ull;
    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    best = dt < best ? dt : best;
    worst = dt > worst ? dt : worst;
  }
  if (slow_factor > 0 && worst > best * slow_factor) bits |= 4;
  return bits;
}

}  // extern "C"
