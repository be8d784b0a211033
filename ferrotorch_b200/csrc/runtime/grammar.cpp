// Native token-mask computation for JSON-schema constrained decoding (`ferrotorch_b200.grammar.JsonSchemaProcessor`).
//
// Every decoding step asks, for each vocabulary entry, whether the text generated so far followed by that entry is still a prefix of a
// document that matches the schema. The prefix matcher below is the same recursive matcher as `grammar.JsonGrammar` (same outcomes:
// invalid, text ended inside a valid value, number complete but extendable, value ended at a position); this file runs it over the whole
// vocabulary, spread over threads, on UTF-8 bytes (every character the grammar looks at is ASCII; bytes >= 0x80 only occur inside strings,
// where they pass).
//
// Capability parity: ferrotorch-grammar/src/json_schema.rs:53-125 (Schema, JsonGrammar), lib.rs:58-85 (TokenMask, JsonSchemaProcessor).
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstring>
#include <string>
#include <string_view>
#include <thread>
#include <vector>

#define FT_API extern "C" __attribute__((visibility("default")))

namespace {

enum Kind : int32_t { K_OBJECT = 0, K_ARRAY = 1, K_STRING = 2, K_NUMBER = 3, K_INTEGER = 4, K_BOOLEAN = 5, K_NULL = 6, K_ENUM = 7, K_ANY = 8, K_NULLABLE = 9 };

struct Edge { std::string lit; int32_t child; bool required; };
struct Node { int32_t kind; std::vector<Edge> edges; };      // object: properties in schema order; array: one edge (items); enum: literals

struct Grammar {
  std::vector<Node> nodes;                                    // node 0 is the root
  std::string vocab;                                          // all entries back to back
  std::vector<int64_t> voff;
  std::vector<uint8_t> plain;                                 // per entry: no quote, no backslash, no control byte (stays inside a string body)
};

// Where the innermost matcher ran out of text on the last PARTIAL outcome of this thread: inside the body of a string (not right after a
// backslash) or anywhere else. A text that ends inside a string body stays valid under any continuation made of plain characters, which lets
// the mask skip the re-parse for most of the vocabulary while a string is being generated.
thread_local bool g_ended_in_string_body = false;

// Outcome of matching a value that starts at a position of the text.
enum Tag : int { INVALID = 0, PARTIAL = 1, OPEN = 2, POS = 3 };   // PARTIAL: text ended inside a still-valid value; OPEN: a number that is complete
struct R { Tag tag; int64_t pos; };                               // at the end of the text but could take more digits; POS: value ended at pos

using sv = std::string_view;
constexpr int MAX_DEPTH = 256;

inline bool digit(char c) { return c >= '0' && c <= '9'; }

R lit(sv l, sv t, int64_t i) {
  g_ended_in_string_body = false;
  const int64_t n = (int64_t)t.size() - i, m = (int64_t)l.size();
  if (n >= m) return t.compare((size_t)i, (size_t)m, l) == 0 ? R{POS, i + m} : R{INVALID, 0};
  return l.compare(0, (size_t)n, t.substr((size_t)i)) == 0 ? R{PARTIAL, 0} : R{INVALID, 0};
}

R string_(sv t, int64_t i) {
  const int64_t n = (int64_t)t.size();
  g_ended_in_string_body = false;
  if (i >= n) return {PARTIAL, 0};
  if (t[i] != '"') return {INVALID, 0};
  i++;
  while (i < n) {
    const unsigned char c = (unsigned char)t[i];
    if (c == '"') return {POS, i + 1};
    if (c == '\\') {
      if (i + 1 >= n) return {PARTIAL, 0};
      if (!std::strchr("\"\\/bfnrtu", t[i + 1]) || t[i + 1] == '\0') return {INVALID, 0};
      i += 2;
      continue;
    }
    if (c < 0x20) return {INVALID, 0};
    i++;
  }
  g_ended_in_string_body = true;
  return {PARTIAL, 0};
}

R number_(sv t, int64_t i, bool integer) {
  g_ended_in_string_body = false;
  const int64_t n = (int64_t)t.size();
  int64_t j = i;
  if (j >= n) return {PARTIAL, 0};
  if (t[j] == '-') {
    j++;
    if (j >= n) return {PARTIAL, 0};
  }
  if (!digit(t[j])) return {INVALID, 0};
  if (t[j] == '0') j++;
  else while (j < n && digit(t[j])) j++;
  if (j >= n) return {OPEN, j};
  if (!integer && t[j] == '.') {
    j++;
    if (j >= n) return {PARTIAL, 0};
    if (!digit(t[j])) return {INVALID, 0};
    while (j < n && digit(t[j])) j++;
    if (j >= n) return {OPEN, j};
  }
  if (!integer && (t[j] == 'e' || t[j] == 'E')) {
    j++;
    if (j < n && (t[j] == '+' || t[j] == '-')) j++;
    if (j >= n) return {PARTIAL, 0};
    if (!digit(t[j])) return {INVALID, 0};
    while (j < n && digit(t[j])) j++;
    if (j >= n) return {OPEN, j};
  }
  return {POS, j};
}

inline int64_t sep(sv t, int64_t i) { return (i < (int64_t)t.size() && t[i] == ' ') ? i + 1 : i; }

R value(const Grammar& g, int32_t node, sv t, int64_t i, int depth);

// kind < 0: a schema node; otherwise one of the built-in alternatives of "any" (array of any, object without properties)
R value_any(const Grammar& g, sv t, int64_t i, int depth);

R array_(const Grammar& g, int32_t items, sv t, int64_t i, int depth) {      // items < 0: any
  const int64_t n = (int64_t)t.size();
  if (t[i] != '[') return {INVALID, 0};
  i++;
  if (i >= n) { g_ended_in_string_body = false; return {PARTIAL, 0}; }
  if (t[i] == ']') return {POS, i + 1};
  for (;;) {
    const R r = items >= 0 ? value(g, items, t, i, depth + 1) : value_any(g, t, i, depth + 1);
    if (r.tag == INVALID || r.tag == PARTIAL) return r;
    g_ended_in_string_body = false;                       // the element is complete: whatever follows is structure
    if (r.tag == OPEN) return {PARTIAL, 0};
    i = r.pos;
    if (i >= n) return {PARTIAL, 0};
    if (t[i] == ']') return {POS, i + 1};
    if (t[i] != ',') return {INVALID, 0};
    i = sep(t, i + 1);
    if (i >= n) return {PARTIAL, 0};
  }
}

R object_(const Grammar& g, const Node* s, sv t, int64_t i, int depth) {      // s null: no properties
  const int64_t n = (int64_t)t.size();
  g_ended_in_string_body = false;
  if (t[i] != '{') return {INVALID, 0};
  i++;
  if (!s || s->edges.empty()) {
    if (i >= n) return {PARTIAL, 0};
    return t[i] == '}' ? R{POS, i + 1} : R{INVALID, 0};
  }
  const auto& props = s->edges;
  bool first = true;
  for (size_t idx = 0; idx < props.size(); idx++) {
    if (i >= n) return {PARTIAL, 0};
    bool optional_rest = true;
    for (size_t k = idx; k < props.size(); k++) optional_rest = optional_rest && !props[k].required;
    if (t[i] == '}' && optional_rest) return (first || t[i - 1] != ',') ? R{POS, i + 1} : R{INVALID, 0};
    if (!first) {
      if (t[i] != ',') return {INVALID, 0};
      i = sep(t, i + 1);
      if (i >= n) return {PARTIAL, 0};
    }
    R r = lit(props[idx].lit, t, i);
    if (r.tag == INVALID) {
      if (props[idx].required) return {INVALID, 0};
      bool continue_ok = false;                   // an optional property may be skipped if a later key can start here
      for (size_t k = idx + 1; k < props.size() && !continue_ok; k++) continue_ok = lit(props[k].lit, t, i).tag != INVALID;
      if (!continue_ok) return {INVALID, 0};
      first = true;                               // the separator before the skipped key is already consumed
      continue;
    }
    if (r.tag == PARTIAL) return r;
    i = r.pos;
    if (i >= n) return {PARTIAL, 0};
    if (t[i] != ':') return {INVALID, 0};
    i = sep(t, i + 1);
    r = value(g, props[idx].child, t, i, depth + 1);
    if (r.tag == INVALID || r.tag == PARTIAL) return r;
    g_ended_in_string_body = false;                       // the property value is complete
    if (r.tag == OPEN) return {PARTIAL, 0};
    i = r.pos;
    first = false;
  }
  if (i >= n) return {PARTIAL, 0};
  return t[i] == '}' ? R{POS, i + 1} : R{INVALID, 0};
}

R boolean_(sv t, int64_t i) {
  const R a = lit("true", t, i);
  return a.tag != INVALID ? a : lit("false", t, i);
}

R value_any(const Grammar& g, sv t, int64_t i, int depth) {
  if (depth > MAX_DEPTH) return {INVALID, 0};
  if (i >= (int64_t)t.size()) { g_ended_in_string_body = false; return {PARTIAL, 0}; }
  R r = string_(t, i);
  if (r.tag != INVALID) return r;
  r = number_(t, i, false);
  if (r.tag != INVALID) return r;
  r = boolean_(t, i);
  if (r.tag != INVALID) return r;
  r = lit("null", t, i);
  if (r.tag != INVALID) return r;
  r = array_(g, -1, t, i, depth);
  if (r.tag != INVALID) return r;
  return object_(g, nullptr, t, i, depth);
}

R value(const Grammar& g, int32_t node, sv t, int64_t i, int depth) {
  if (depth > MAX_DEPTH) return {INVALID, 0};
  if (i >= (int64_t)t.size()) { g_ended_in_string_body = false; return {PARTIAL, 0}; }
  const Node& s = g.nodes[(size_t)node];
  switch (s.kind) {
    case K_STRING: return string_(t, i);
    case K_NUMBER: return number_(t, i, false);
    case K_INTEGER: return number_(t, i, true);
    case K_BOOLEAN: return boolean_(t, i);
    case K_NULL: return lit("null", t, i);
    case K_ENUM: {
      R res{INVALID, 0};
      for (const Edge& e : s.edges) {
        const R r = lit(e.lit, t, i);
        if (r.tag == POS) return r;
        if (r.tag == PARTIAL) res = r;
      }
      return res;
    }
    case K_ANY: return value_any(g, t, i, depth);
    case K_NULLABLE: {
      const R r = lit("null", t, i);
      if (r.tag != INVALID || s.edges.empty()) return r;
      return value(g, s.edges[0].child, t, i, depth + 1);
    }
    case K_ARRAY: return array_(g, s.edges.empty() ? -1 : s.edges[0].child, t, i, depth);
    case K_OBJECT: return object_(g, &s, t, i, depth);
  }
  return {INVALID, 0};
}

inline bool valid(const Grammar& g, sv t) {
  const R r = value(g, 0, t, 0, 0);
  return r.tag == PARTIAL || r.tag == OPEN || (r.tag == POS && r.pos == (int64_t)t.size());
}

inline bool complete(const Grammar& g, sv t) {
  const R r = value(g, 0, t, 0, 0);
  return (r.tag == OPEN || r.tag == POS) && r.pos == (int64_t)t.size();
}

}  // namespace

// Builds a grammar from a flattened schema and the vocabulary. Node k has kind[k] (0 object, 1 array, 2 string, 3 number, 4 integer,
// 5 boolean, 6 null, 7 enum, 8 any, 9 nullable: null or its one child) and the edges edge_first[k] .. edge_first[k+1]: for an object its properties in schema order (lit = the
// key as a JSON string literal), for an array or a nullable at most one (child = items / inner node), for an enum its values as JSON literals (child -1). Edge e
// has the literal lits[lit_off[e] .. lit_off[e+1]). Vocabulary entry v is vocab[voff[v] .. voff[v+1]) in UTF-8. Node 0 is the root.
FT_API void* ft_json_grammar_create(const int32_t* kind, const int32_t* edge_first, int64_t n_nodes, const uint8_t* lits, const int64_t* lit_off,
                                    const int32_t* edge_child, const uint8_t* edge_required, const uint8_t* vocab, const int64_t* voff, int64_t n_vocab) {
  Grammar* g = new Grammar();
  g->nodes.resize((size_t)n_nodes);
  for (int64_t k = 0; k < n_nodes; k++) {
    g->nodes[(size_t)k].kind = kind[k];
    for (int32_t e = edge_first[k]; e < edge_first[k + 1]; e++)
      g->nodes[(size_t)k].edges.push_back(Edge{std::string((const char*)lits + lit_off[e], (size_t)(lit_off[e + 1] - lit_off[e])), edge_child[e],
                                               edge_required[e] != 0});
  }
  g->vocab.assign((const char*)vocab, (size_t)voff[n_vocab]);
  g->voff.assign(voff, voff + n_vocab + 1);
  g->plain.resize((size_t)n_vocab);
  for (int64_t v = 0; v < n_vocab; v++) {
    bool ok = voff[v + 1] > voff[v];
    for (int64_t k = voff[v]; k < voff[v + 1] && ok; k++) {
      const unsigned char c = vocab[k];
      ok = c != '"' && c != '\\' && c >= 0x20;
    }
    g->plain[(size_t)v] = ok ? 1 : 0;
  }
  return g;
}

FT_API void ft_json_grammar_destroy(void* h) { delete static_cast<Grammar*>(h); }

// 1 if text (UTF-8, n bytes) can still be extended to a matching document (or is one), else 0; *is_complete = 1 if it is one already.
FT_API int ft_json_grammar_check(void* h, const uint8_t* text, int64_t n, int* is_complete) {
  const Grammar& g = *static_cast<const Grammar*>(h);
  const sv t((const char*)text, (size_t)n);
  if (is_complete) *is_complete = complete(g, t) ? 1 : 0;
  return valid(g, t) ? 1 : 0;
}

// allowed[v] = 1 if vocabulary entry v may follow text: the end-of-sequence entry (eos_id, -1 for none) exactly when text is a complete
// document; an empty entry never; any other entry when text + entry is still valid, except that after a complete document nothing but a
// longer number (root of kind number / integer) may follow. Returns the number of allowed entries.
FT_API int64_t ft_json_grammar_mask(void* h, const uint8_t* text, int64_t n, int64_t eos_id, uint8_t* allowed, int nthreads) {
  const Grammar& g = *static_cast<const Grammar*>(h);
  const sv t((const char*)text, (size_t)n);
  const int64_t V = (int64_t)g.voff.size() - 1;
  const bool done = complete(g, t);
  const bool closed = done && g.nodes[0].kind != K_NUMBER && g.nodes[0].kind != K_INTEGER;
  g_ended_in_string_body = false;
  const R whole = value(g, 0, t, 0, 0);
  const bool in_string = whole.tag == PARTIAL && g_ended_in_string_body;       // text ends inside a string body: plain entries need no re-parse
  nthreads = (int)std::max<int64_t>(1, std::min<int64_t>(std::min(nthreads, 64), V / 2048));
  if (closed) nthreads = 1;                               // nothing to parse: starting threads would cost more than the loop
  std::vector<int64_t> counts((size_t)nthreads, 0);
  auto work = [&](int k) {
    const int64_t lo = V * k / nthreads, hi = V * (k + 1) / nthreads;
    std::string buf(t);
    int64_t c = 0;
    int8_t first_ok[256];                                 // does text + this byte still parse? (-1: not asked yet) An entry whose first byte
    std::memset(first_ok, -1, sizeof(first_ok));          // already fails cannot be valid: the matcher never recovers from an invalid prefix
    for (int64_t v = lo; v < hi; v++) {
      bool ok;
      const int64_t len = g.voff[(size_t)v + 1] - g.voff[(size_t)v];
      if (v == eos_id) ok = done;
      else if (len == 0 || closed) ok = false;
      else if (in_string && g.plain[(size_t)v]) ok = true;
      else if (len > 1 && [&] {
                 const unsigned char b0 = (unsigned char)g.vocab[(size_t)g.voff[(size_t)v]];
                 if (first_ok[b0] < 0) {
                   buf.resize((size_t)n);
                   buf.push_back((char)b0);
                   first_ok[b0] = valid(g, buf) ? 1 : 0;
                 }
                 return first_ok[b0] == 0;
               }()) ok = false;
      else {
        buf.resize((size_t)n);
        buf.append(g.vocab.data() + g.voff[(size_t)v], (size_t)len);
        ok = valid(g, buf);
      }
      allowed[v] = ok ? 1 : 0;
      c += ok;
    }
    counts[(size_t)k] = c;
  };
  if (nthreads == 1) {
    work(0);
  } else {
    std::vector<std::thread> ts;
    for (int k = 0; k < nthreads; k++) ts.emplace_back(work, k);
    for (auto& th : ts) th.join();
  }
  int64_t total = 0;
  for (auto c : counts) total += c;
  return total;
}

// The masks of several texts over the same grammar and vocabulary: text k is texts[off[k] .. off[k+1]), its mask goes to allowed[k * V ..].
// The texts are spread over up to nthreads threads (each mask itself runs on one). counts [n_texts] (may be null) receives the number of
// allowed entries per text.
FT_API void ft_json_grammar_mask_batch(void* h, const uint8_t* texts, const int64_t* off, int64_t n_texts, int64_t eos_id, uint8_t* allowed, int64_t* counts,
                                       int nthreads) {
  const Grammar& g = *static_cast<const Grammar*>(h);
  const int64_t V = (int64_t)g.voff.size() - 1;
  nthreads = (int)std::max<int64_t>(1, std::min<int64_t>(std::min(nthreads, 64), n_texts));
  std::atomic<int64_t> next{0};
  auto work = [&] {
    for (;;) {
      const int64_t k = next.fetch_add(1);
      if (k >= n_texts) return;
      const int64_t c = ft_json_grammar_mask(h, texts + off[k], off[k + 1] - off[k], eos_id, allowed + k * V, 1);
      if (counts) counts[k] = c;
    }
  };
  if (nthreads == 1) { work(); return; }
  std::vector<std::thread> ts;
  for (int t = 0; t < nthreads; t++) ts.emplace_back(work);
  for (auto& th : ts) th.join();
}
