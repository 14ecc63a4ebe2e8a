// Grammar-constrained decoding on the host: GBNF parser, lazily built DFA over Unicode code points,
// token trie over raw token bytes, and per-state valid-token masks.
//
// A grammar is a set of rules; each rule is a list of alternatives; each alternative a sequence of
// character classes and rule references (groups and repetitions are lowered to synthetic rules).
// A parse state is a set of stacks of "return positions"; state sets are canonicalised and numbered,
// and transitions (state, code point) -> state are memoised, so walking the whole vocabulary trie for
// a mask costs one table look-up per trie node.  Masks are cached per state.  Tokens may split a
// UTF-8 sequence: the request state carries the pending bytes, and a token that ends inside a sequence
// is allowed when some stack can accept a non-ASCII character next.
//
// Bounds: rules <= 4096, elements <= 65536, DFA states <= 200000, stack depth <= 256.
// Counterpart in the reference: crates/sllm-core/src/grammar.rs (GBNF + JSON subsets -> bounded e-NFA,
// token trie over raw token bytes, partial UTF-8 state, limits :17-34).
#include "host_api.h"

#include <algorithm>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

constexpr int kMaxRules = 4096;
constexpr int kMaxElems = 65536;
constexpr int kMaxStates = 200000;
constexpr int kMaxDepth = 256;
constexpr int kMaskCache = 512;

struct Elem {
  bool is_ref = false;
  int rule = -1;                                   // for refs
  bool negated = false;
  std::vector<std::pair<uint32_t, uint32_t>> ranges;  // for char classes
  bool matches(uint32_t cp) const {
    bool in = false;
    for (auto& r : ranges)
      if (cp >= r.first && cp <= r.second) { in = true; break; }
    return in != negated;
  }
  bool may_match_non_ascii() const {
    if (negated) return true;
    for (auto& r : ranges)
      if (r.second >= 0x80) return true;
    return false;
  }
};
using Alt = std::vector<Elem>;
struct Rule { std::vector<Alt> alts; };

struct Pos { int rule, alt, idx; bool operator<(const Pos& o) const { return std::tie(rule, alt, idx) < std::tie(o.rule, o.alt, o.idx); }
             bool operator==(const Pos& o) const { return rule == o.rule && alt == o.alt && idx == o.idx; } };
using Stack = std::vector<Pos>;   // back() = next element to match; empty = grammar complete

struct TrieNode { int child[256]; int token = -1; std::vector<int> more_tokens; TrieNode() { std::fill(child, child + 256, -1); } };

struct Grammar {
  std::vector<Rule> rules;
  std::map<std::string, int> names;
  int root = 0;
  int total_elems = 0;
  // DFA
  std::vector<std::vector<Stack>> states;
  std::map<std::vector<Stack>, int> state_ids;
  std::vector<std::unordered_map<uint32_t, int>> trans;
  // vocabulary
  std::vector<TrieNode> trie;
  int n_tokens = 0;
  std::vector<std::string> tok_bytes;
  std::unordered_map<int, std::vector<uint8_t>> mask_cache;
  std::vector<int> mask_cache_order;
  std::mutex mu;
  std::string error;
};

struct ReqState { int dfa = 0; std::string pending; bool dead = false; };

std::mutex g_mu;
std::unordered_map<int, std::shared_ptr<Grammar>> g_grammars;
std::unordered_map<int, std::pair<int, ReqState>> g_states;   // handle -> (grammar handle, state)
int g_next = 1;

// ---------------------------------------------------------------- GBNF parser
struct Parser {
  Grammar& g;
  const std::string& s;
  size_t i = 0;
  int synth = 0;
  explicit Parser(Grammar& gr, const std::string& src) : g(gr), s(src) {}

  bool fail(const std::string& m) { if (g.error.empty()) g.error = m + " at offset " + std::to_string(i); return false; }
  void ws(bool newlines) {
    while (i < s.size()) {
      char c = s[i];
      if (c == '#') { while (i < s.size() && s[i] != '\n') ++i; }
      else if (c == ' ' || c == '\t' || c == '\r' || (newlines && c == '\n')) ++i;
      else break;
    }
  }
  int rule_id(const std::string& name) {
    auto it = g.names.find(name);
    if (it != g.names.end()) return it->second;
    int id = static_cast<int>(g.rules.size());
    g.rules.emplace_back();
    g.names[name] = id;
    return id;
  }
  static bool name_char(char c) { return isalnum(static_cast<unsigned char>(c)) || c == '-' || c == '_'; }
  bool parse_name(std::string* out) {
    size_t b = i;
    while (i < s.size() && name_char(s[i])) ++i;
    if (i == b) return fail("expected a rule name");
    *out = s.substr(b, i - b);
    return true;
  }
  bool parse_cp(uint32_t* cp) {   // one (possibly escaped) code point
    if (i >= s.size()) return fail("unexpected end");
    unsigned char c = s[i];
    if (c == '\\') {
      if (i + 1 >= s.size()) return fail("dangling escape");
      char e = s[i + 1];
      i += 2;
      auto hex = [&](int n, uint32_t* v) {
        *v = 0;
        for (int k = 0; k < n; ++k) {
          if (i >= s.size() || !isxdigit(static_cast<unsigned char>(s[i]))) return false;
          char h = s[i++];
          *v = *v * 16 + (isdigit(static_cast<unsigned char>(h)) ? h - '0' : (tolower(h) - 'a' + 10));
        }
        return true;
      };
      switch (e) {
        case 'n': *cp = '\n'; return true;
        case 'r': *cp = '\r'; return true;
        case 't': *cp = '\t'; return true;
        case 'x': return hex(2, cp) || fail("bad \\x escape");
        case 'u': return hex(4, cp) || fail("bad \\u escape");
        case 'U': return hex(8, cp) || fail("bad \\U escape");
        default: *cp = static_cast<unsigned char>(e); return true;
      }
    }
    int n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 0;
    if (n == 0 || i + n > s.size()) return fail("invalid UTF-8 in grammar");
    uint32_t v = n == 1 ? c : c & (0xFF >> (n + 1));
    for (int k = 1; k < n; ++k) v = (v << 6) | (static_cast<unsigned char>(s[i + k]) & 0x3F);
    i += n;
    *cp = v;
    return true;
  }
  int new_synth_rule() {
    int id = static_cast<int>(g.rules.size());
    g.rules.emplace_back();
    g.names["%synth" + std::to_string(synth++)] = id;
    return id;
  }
  // wraps the last item (elements [start, end) of alt) according to a repetition operator
  bool apply_repeat(Alt& alt, size_t start, int lo, int hi) {
    Alt item(alt.begin() + start, alt.end());
    alt.resize(start);
    if (lo < 0 || (hi >= 0 && hi < lo) || lo > 64 || hi > 64) return fail("repetition bounds out of range");
    int sub = new_synth_rule();
    g.rules[sub].alts.push_back(item);
    Elem ref; ref.is_ref = true; ref.rule = sub;
    for (int k = 0; k < lo; ++k) alt.push_back(ref);
    if (hi < 0) {                       // item*  ==  star ::= item star |
      int star = new_synth_rule();
      Alt a; a.push_back(ref); Elem self; self.is_ref = true; self.rule = star; a.push_back(self);
      g.rules[star].alts.push_back(a);
      g.rules[star].alts.push_back(Alt());
      alt.push_back(self);
    } else {
      int prev = -1;                    // nested optionals: opt_k ::= item opt_{k+1} |
      for (int k = 0; k < hi - lo; ++k) {
        int opt = new_synth_rule();
        Alt a; a.push_back(ref);
        if (prev >= 0) { Elem p; p.is_ref = true; p.rule = prev; a.push_back(p); }
        g.rules[opt].alts.push_back(a);
        g.rules[opt].alts.push_back(Alt());
        prev = opt;
      }
      if (prev >= 0) { Elem p; p.is_ref = true; p.rule = prev; alt.push_back(p); }
    }
    return true;
  }
  bool parse_alternates(int rule, bool nested) {
    for (;;) {
      Alt alt;
      if (!parse_sequence(alt, nested)) return false;
      g.rules[rule].alts.push_back(alt);
      ws(nested);
      if (i < s.size() && s[i] == '|') { ++i; ws(true); continue; }
      return true;
    }
  }
  bool parse_sequence(Alt& alt, bool nested) {
    for (;;) {
      ws(nested);
      if (i >= s.size()) return true;
      char c = s[i];
      size_t start = alt.size();
      if (c == '"') {
        ++i;
        while (i < s.size() && s[i] != '"') {
          uint32_t cp;
          if (!parse_cp(&cp)) return false;
          Elem e; e.ranges.push_back({cp, cp}); alt.push_back(e);
        }
        if (i >= s.size()) return fail("unterminated string");
        ++i;
      } else if (c == '[') {
        ++i;
        Elem e;
        if (i < s.size() && s[i] == '^') { e.negated = true; ++i; }
        while (i < s.size() && s[i] != ']') {
          uint32_t a, b;
          if (!parse_cp(&a)) return false;
          b = a;
          if (i + 1 < s.size() && s[i] == '-' && s[i + 1] != ']') { ++i; if (!parse_cp(&b)) return false; }
          if (b < a) return fail("inverted range");
          e.ranges.push_back({a, b});
        }
        if (i >= s.size()) return fail("unterminated character class");
        ++i;
        alt.push_back(e);
      } else if (c == '.') {
        ++i;
        Elem e; e.negated = true; alt.push_back(e);   // any code point
      } else if (c == '(') {
        ++i;
        int sub = new_synth_rule();
        ws(true);
        if (!parse_alternates(sub, true)) return false;
        ws(true);
        if (i >= s.size() || s[i] != ')') return fail("expected )");
        ++i;
        Elem e; e.is_ref = true; e.rule = sub; alt.push_back(e);
      } else if (name_char(c)) {
        size_t save = i;
        std::string name;
        if (!parse_name(&name)) return false;
        size_t after = i;
        ws(false);
        if (i + 2 < s.size() && s.compare(i, 3, "::=") == 0) { i = save; return true; }  // next rule starts
        i = after;
        Elem e; e.is_ref = true; e.rule = rule_id(name); alt.push_back(e);
      } else {
        return true;   // ')' '|' newline-terminated etc. handled by the caller
      }
      // repetition suffixes
      if (i < s.size()) {
        char r = s[i];
        if (r == '*') { ++i; if (!apply_repeat(alt, start, 0, -1)) return false; }
        else if (r == '+') { ++i; if (!apply_repeat(alt, start, 1, -1)) return false; }
        else if (r == '?') { ++i; if (!apply_repeat(alt, start, 0, 1)) return false; }
        else if (r == '{') {
          ++i;
          int lo = 0, hi = -1; bool have_lo = false;
          while (i < s.size() && isdigit(static_cast<unsigned char>(s[i]))) { lo = lo * 10 + (s[i++] - '0'); have_lo = true; if (lo > 1000) return fail("repetition too large"); }
          if (!have_lo) return fail("expected a number in {}");
          if (i < s.size() && s[i] == ',') {
            ++i;
            if (i < s.size() && isdigit(static_cast<unsigned char>(s[i]))) { hi = 0; while (i < s.size() && isdigit(static_cast<unsigned char>(s[i]))) { hi = hi * 10 + (s[i++] - '0'); if (hi > 1000) return fail("repetition too large"); } }
          } else hi = lo;
          if (i >= s.size() || s[i] != '}') return fail("expected }");
          ++i;
          if (!apply_repeat(alt, start, lo, hi)) return false;
        }
      }
      if (static_cast<int>(g.rules.size()) > kMaxRules) return fail("too many rules");
    }
  }
  bool parse() {
    ws(true);
    while (i < s.size()) {
      std::string name;
      if (!parse_name(&name)) return false;
      ws(false);
      if (i + 2 >= s.size() || s.compare(i, 3, "::=") != 0) return fail("expected ::=");
      i += 3;
      ws(true);
      int id = rule_id(name);
      if (!g.rules[id].alts.empty()) return fail("rule defined twice: " + name);
      if (!parse_alternates(id, false)) return false;
      ws(true);
    }
    for (auto& kv : g.names)
      if (g.rules[kv.second].alts.empty()) return fail("undefined rule: " + kv.first);
    int total = 0;
    for (auto& r : g.rules) for (auto& a : r.alts) total += static_cast<int>(a.size()) + 1;
    g.total_elems = total;
    if (total > kMaxElems) return fail("grammar too large");
    return true;
  }
};

// ---------------------------------------------------------------- automaton
// Expand rule references on top of `st` until every resulting stack has a character class on top
// (or is empty).  `seen` guards against left recursion.
void advance(const Grammar& g, Stack st, std::vector<Stack>& out, int depth) {
  if (depth > kMaxDepth || st.size() > static_cast<size_t>(kMaxDepth)) return;
  if (st.empty()) { if (std::find(out.begin(), out.end(), st) == out.end()) out.push_back(st); return; }
  Pos p = st.back();
  const Alt& alt = g.rules[p.rule].alts[p.alt];
  if (p.idx >= static_cast<int>(alt.size())) {     // alternative finished: return to the caller
    st.pop_back();
    advance(g, st, out, depth + 1);
    return;
  }
  const Elem& e = alt[p.idx];
  if (!e.is_ref) { if (std::find(out.begin(), out.end(), st) == out.end()) out.push_back(st); return; }
  // replace the reference by "continue after it", then push each alternative of the callee
  st.back().idx += 1;
  for (size_t a = 0; a < g.rules[e.rule].alts.size(); ++a) {
    Stack s2 = st;
    s2.push_back(Pos{e.rule, static_cast<int>(a), 0});
    advance(g, s2, out, depth + 1);
  }
}

int intern_state(Grammar& g, std::vector<Stack>& stacks) {
  std::sort(stacks.begin(), stacks.end());
  stacks.erase(std::unique(stacks.begin(), stacks.end()), stacks.end());
  auto it = g.state_ids.find(stacks);
  if (it != g.state_ids.end()) return it->second;
  if (static_cast<int>(g.states.size()) >= kMaxStates) return -1;
  int id = static_cast<int>(g.states.size());
  g.states.push_back(stacks);
  g.trans.emplace_back();
  g.state_ids[stacks] = id;
  return id;
}

// -1: dead (no stack accepts cp); -2: state limit
int step(Grammar& g, int state, uint32_t cp) {
  auto& cache = g.trans[state];
  auto it = cache.find(cp);
  if (it != cache.end()) return it->second;
  std::vector<Stack> next;
  const std::vector<Stack> cur = g.states[state];   // copy: g.states may grow
  for (const Stack& st : cur) {
    if (st.empty()) continue;
    Pos p = st.back();
    const Elem& e = g.rules[p.rule].alts[p.alt][p.idx];
    if (!e.matches(cp)) continue;
    Stack s2 = st;
    s2.back().idx += 1;
    advance(g, s2, next, 0);
  }
  int id = next.empty() ? -1 : intern_state(g, next);
  if (id == -1 && !next.empty()) id = -2;
  g.trans[state][cp] = id;
  return id;
}

bool state_complete(const Grammar& g, int state) {
  for (const Stack& st : g.states[state]) if (st.empty()) return true;
  return false;
}
bool state_accepts_non_ascii(const Grammar& g, int state) {
  for (const Stack& st : g.states[state]) {
    if (st.empty()) continue;
    Pos p = st.back();
    if (g.rules[p.rule].alts[p.alt][p.idx].may_match_non_ascii()) return true;
  }
  return false;
}

// Feed bytes; returns the new DFA state or -1 (dead).  `pending` holds an incomplete UTF-8 tail.
int feed(Grammar& g, int state, std::string& pending, const unsigned char* b, size_t n) {
  for (size_t k = 0; k < n; ++k) {
    pending.push_back(static_cast<char>(b[k]));
    unsigned char c0 = pending[0];
    int need = c0 < 0x80 ? 1 : (c0 >> 5) == 6 ? 2 : (c0 >> 4) == 14 ? 3 : (c0 >> 3) == 30 ? 4 : 0;
    if (need == 0) return -1;
    if (pending.size() > 1 && (static_cast<unsigned char>(pending.back()) & 0xC0) != 0x80) return -1;
    if (static_cast<int>(pending.size()) < need) continue;
    uint32_t cp = need == 1 ? c0 : c0 & (0xFF >> (need + 1));
    for (int q = 1; q < need; ++q) cp = (cp << 6) | (static_cast<unsigned char>(pending[q]) & 0x3F);
    pending.clear();
    state = step(g, state, cp);
    if (state < 0) return -1;
  }
  return state;
}

void trie_walk(Grammar& g, int node, int state, std::string& pending, std::vector<uint8_t>& mask) {
  const TrieNode& tn = g.trie[node];
  if (tn.token >= 0 && node != 0) {
    const bool ok = pending.empty() || state_accepts_non_ascii(g, state);
    if (ok) {
      mask[tn.token] = 1;
      for (int t : tn.more_tokens) mask[t] = 1;
    }
  }
  for (int c = 0; c < 256; ++c) {
    const int ch = g.trie[node].child[c];
    if (ch < 0) continue;
    std::string p2 = pending;
    unsigned char byte = static_cast<unsigned char>(c);
    const int s2 = feed(g, state, p2, &byte, 1);
    if (s2 < 0) continue;
    trie_walk(g, ch, s2, p2, mask);
  }
}

std::shared_ptr<Grammar> find_grammar(int h) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_grammars.find(h);
  return it == g_grammars.end() ? nullptr : it->second;
}

}  // namespace

SLLM_HOST_EXPORT int sllm_grammar_create(const char* gbnf, const char* root, char* err, int err_cap) {
  if (!gbnf) return -SLLM_HOST_INVALID;
  auto g = std::make_shared<Grammar>();
  std::string src(gbnf);
  if (src.size() > (1u << 20)) return -SLLM_HOST_LIMIT;
  Parser p(*g, src);
  auto it_ok = p.parse();
  std::string root_name = root && root[0] ? root : "root";
  if (it_ok && !g->names.count(root_name)) { g->error = "missing root rule: " + root_name; it_ok = false; }
  if (!it_ok) {
    if (err && err_cap > 0) { strncpy(err, g->error.c_str(), err_cap - 1); err[err_cap - 1] = 0; }
    return -SLLM_HOST_PARSE_ERROR;
  }
  g->root = g->names[root_name];
  std::vector<Stack> init;
  for (size_t a = 0; a < g->rules[g->root].alts.size(); ++a) advance(*g, Stack{Pos{g->root, static_cast<int>(a), 0}}, init, 0);
  if (init.empty()) {
    if (err && err_cap > 0) strncpy(err, "grammar accepts nothing (left recursion?)", err_cap - 1);
    return -SLLM_HOST_PARSE_ERROR;
  }
  intern_state(*g, init);
  std::lock_guard<std::mutex> l(g_mu);
  int h = g_next++;
  g_grammars[h] = g;
  return h;
}

SLLM_HOST_EXPORT int sllm_grammar_destroy(int h) {
  std::lock_guard<std::mutex> l(g_mu);
  for (auto it = g_states.begin(); it != g_states.end();) it = it->second.first == h ? g_states.erase(it) : std::next(it);
  return g_grammars.erase(h) ? SLLM_HOST_OK : SLLM_HOST_NOT_FOUND;
}

// Token bytes: blob + offsets[n_tokens + 1].  Empty tokens (specials) are never allowed by a mask.
SLLM_HOST_EXPORT int sllm_grammar_set_vocab(int h, int n_tokens, const unsigned char* blob, const unsigned int* offsets) {
  auto g = find_grammar(h);
  if (!g || n_tokens <= 0 || !blob || !offsets) return SLLM_HOST_INVALID;
  std::lock_guard<std::mutex> l(g->mu);
  g->trie.clear();
  g->trie.emplace_back();
  g->n_tokens = n_tokens;
  g->mask_cache.clear();
  g->mask_cache_order.clear();
  for (int t = 0; t < n_tokens; ++t) {
    const unsigned int b = offsets[t], e = offsets[t + 1];
    if (e <= b) continue;
    if (e - b > 128) return SLLM_HOST_LIMIT;
    int node = 0;
    for (unsigned int k = b; k < e; ++k) {
      int c = blob[k];
      if (g->trie[node].child[c] < 0) {
        g->trie[node].child[c] = static_cast<int>(g->trie.size());
        g->trie.emplace_back();
      }
      node = g->trie[node].child[c];
    }
    if (g->trie[node].token < 0) g->trie[node].token = t; else g->trie[node].more_tokens.push_back(t);
  }
  g->tok_bytes.assign(n_tokens, std::string());
  for (int t = 0; t < n_tokens; ++t) g->tok_bytes[t].assign(reinterpret_cast<const char*>(blob) + offsets[t], offsets[t + 1] - offsets[t]);
  return SLLM_HOST_OK;
}

SLLM_HOST_EXPORT int sllm_grammar_state_new(int h) {
  auto g = find_grammar(h);
  if (!g) return -SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> l(g_mu);
  int s = g_next++;
  g_states[s] = {h, ReqState()};
  return s;
}

SLLM_HOST_EXPORT int sllm_grammar_state_clone(int s) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_states.find(s);
  if (it == g_states.end()) return -SLLM_HOST_NOT_FOUND;
  int n = g_next++;
  g_states[n] = it->second;
  return n;
}

SLLM_HOST_EXPORT int sllm_grammar_state_free(int s) {
  std::lock_guard<std::mutex> l(g_mu);
  return g_states.erase(s) ? SLLM_HOST_OK : SLLM_HOST_NOT_FOUND;
}

static bool get_state(int s, int* gh, ReqState* st) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_states.find(s);
  if (it == g_states.end()) return false;
  *gh = it->second.first;
  *st = it->second.second;
  return true;
}
static void put_state(int s, const ReqState& st) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_states.find(s);
  if (it != g_states.end()) it->second.second = st;
}

// out_mask[n_tokens] = 1 for tokens the grammar allows next.  Returns the number of allowed tokens.
SLLM_HOST_EXPORT int sllm_grammar_mask(int s, unsigned char* out_mask, int n) {
  int gh; ReqState st;
  if (!get_state(s, &gh, &st) || !out_mask) return -SLLM_HOST_NOT_FOUND;
  auto g = find_grammar(gh);
  if (!g || n != g->n_tokens) return -SLLM_HOST_INVALID;
  std::lock_guard<std::mutex> l(g->mu);
  if (st.dead) { memset(out_mask, 0, n); return 0; }
  const bool cacheable = st.pending.empty();
  if (cacheable) {
    auto it = g->mask_cache.find(st.dfa);
    if (it != g->mask_cache.end()) {
      memcpy(out_mask, it->second.data(), n);
      int c = 0; for (int i = 0; i < n; ++i) c += out_mask[i];
      return c;
    }
  }
  std::vector<uint8_t> mask(n, 0);
  std::string pending = st.pending;
  trie_walk(*g, 0, st.dfa, pending, mask);
  memcpy(out_mask, mask.data(), n);
  if (cacheable) {
    if (static_cast<int>(g->mask_cache_order.size()) >= kMaskCache) {
      g->mask_cache.erase(g->mask_cache_order.front());
      g->mask_cache_order.erase(g->mask_cache_order.begin());
    }
    g->mask_cache[st.dfa] = mask;
    g->mask_cache_order.push_back(st.dfa);
  }
  int c = 0; for (int i = 0; i < n; ++i) c += mask[i];
  return c;
}

// Advance by one token.  0 = accepted, SLLM_HOST_INVALID = the grammar rejects it (state becomes dead).
SLLM_HOST_EXPORT int sllm_grammar_accept(int s, int token) {
  int gh; ReqState st;
  if (!get_state(s, &gh, &st)) return SLLM_HOST_NOT_FOUND;
  auto g = find_grammar(gh);
  if (!g || token < 0 || token >= g->n_tokens) return SLLM_HOST_INVALID;
  std::lock_guard<std::mutex> l(g->mu);
  const std::string& b = g->tok_bytes[token];
  int rc = SLLM_HOST_OK;
  if (st.dead || b.empty()) { st.dead = true; rc = SLLM_HOST_INVALID; }
  else {
    int ns = feed(*g, st.dfa, st.pending, reinterpret_cast<const unsigned char*>(b.data()), b.size());
    if (ns < 0) { st.dead = true; rc = SLLM_HOST_INVALID; } else st.dfa = ns;
  }
  put_state(s, st);
  return rc;
}

// Feed raw text (assistant prefill) instead of a token.
SLLM_HOST_EXPORT int sllm_grammar_accept_bytes(int s, const unsigned char* bytes, int n) {
  int gh; ReqState st;
  if (!get_state(s, &gh, &st)) return SLLM_HOST_NOT_FOUND;
  auto g = find_grammar(gh);
  if (!g || n < 0) return SLLM_HOST_INVALID;
  std::lock_guard<std::mutex> l(g->mu);
  int rc = SLLM_HOST_OK;
  int ns = st.dead ? -1 : feed(*g, st.dfa, st.pending, bytes, n);
  if (ns < 0) { st.dead = true; rc = SLLM_HOST_INVALID; } else st.dfa = ns;
  put_state(s, st);
  return rc;
}

// 1 when the text so far is a complete sentence of the grammar (end-of-sequence may be allowed).
SLLM_HOST_EXPORT int sllm_grammar_is_complete(int s) {
  int gh; ReqState st;
  if (!get_state(s, &gh, &st)) return -SLLM_HOST_NOT_FOUND;
  auto g = find_grammar(gh);
  if (!g) return -SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> l(g->mu);
  return (!st.dead && st.pending.empty() && state_complete(*g, st.dfa)) ? 1 : 0;
}

SLLM_HOST_EXPORT int sllm_grammar_stats(int h, long long* out3) {
  auto g = find_grammar(h);
  if (!g || !out3) return SLLM_HOST_NOT_FOUND;
  std::lock_guard<std::mutex> l(g->mu);
  out3[0] = static_cast<long long>(g->rules.size());
  out3[1] = static_cast<long long>(g->states.size());
  out3[2] = static_cast<long long>(g->trie.size());
  return SLLM_HOST_OK;
}
