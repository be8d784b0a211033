// Native byte-pair-encoding merge engine behind `ferrotorch_b200.tokenize.Tokenizer`.
//
// The Python side splits the text into pieces (the pre-tokeniser's regular expression) and hands all pieces of one call, or of a whole
// batch of texts, over as one UTF-8 byte string with piece offsets. For every piece this file maps the bytes (byte-level models) or the
// code points (plain models) to their initial symbol ids and applies the merges in rank order: symbols in a doubly linked list, the
// candidate pairs in a min-heap keyed by (rank, position), stale heap entries recognised when popped. That is O(n log n) per piece against
// the O(n^2) rescan of the direct loop, and the pieces of a call are spread over threads.
//
// ft_bpe_encode_texts also does the splitting: the two pre-tokeniser patterns in general use (GPT-2 and Llama-3) are restated as hand-written
// matchers over code points with a class table (letter / number / white space per code point) that the Python side derives once from the
// same regular-expression engine it would otherwise run, so both routes cut a text at the same places; the texts of a batch are spread
// over threads.
//
// Capability parity: the reference wraps the HF `tokenizers` library (ferrotorch-tokenize/src/lib.rs:59-131); the merge order here is that
// library's: lowest rank first, leftmost occurrence on equal rank, one occurrence per step.
#include <algorithm>
#include <atomic>
#include <climits>
#include <cstdint>
#include <cstring>
#include <string>
#include <string_view>
#include <thread>
#include <unordered_map>
#include <vector>

#define FT_API extern "C" __attribute__((visibility("default")))

namespace {

struct Merge { int32_t rank, merged; };

// (left id << 32 | right id) -> rank and id of the concatenation: open addressing with linear probing, at most half full.
struct MergeTable {
  struct Slot { uint64_t key; Merge val; };
  std::vector<Slot> slots;
  int shift = 63;
  static constexpr uint64_t EMPTY = ~0ull;             // no pair of non-negative ids has this key
  void init(int64_t n) {
    int bits = 4;
    while ((1ll << bits) < 2 * n + 2) bits++;
    shift = 64 - bits;
    slots.assign((size_t)1 << bits, Slot{EMPTY, Merge{0, 0}});
  }
  size_t home(uint64_t k) const { return (size_t)((k * 0x9E3779B97F4A7C15ull) >> shift); }
  void insert(uint64_t k, Merge v) {                   // the first entry of a key stays
    for (size_t i = home(k);; i = (i + 1) & (slots.size() - 1)) {
      if (slots[i].key == k) return;
      if (slots[i].key == EMPTY) { slots[i] = Slot{k, v}; return; }
    }
  }
  const Merge* find(uint64_t k) const {
    for (size_t i = home(k);; i = (i + 1) & (slots.size() - 1)) {
      if (slots[i].key == k) return &slots[i].val;
      if (slots[i].key == EMPTY) return nullptr;
    }
  }
};

struct Bpe {
  MergeTable merges;
  int32_t byte_sym[256];                               // byte-level models: id of the one-character token that stands for each byte, -1 if none
  std::unordered_map<uint32_t, int32_t> char_sym;      // plain models: code point -> id of the one-character token
  bool byte_level = true;
  bool ignore_merges = false;                          // a piece that is a vocabulary entry as a whole is emitted without merging
  std::string whole_blob;                              // vocabulary entries as raw piece bytes (only filled when ignore_merges)
  std::unordered_map<std::string_view, int32_t> whole;
};

inline uint64_t key(int32_t a, int32_t b) { return ((uint64_t)(uint32_t)a << 32) | (uint32_t)b; }

// Decodes one UTF-8 code point starting at s[i] (i < n); returns its length, 0 on malformed input.
inline int utf8_next(const uint8_t* s, int64_t i, int64_t n, uint32_t& cp) {
  const uint8_t c = s[i];
  if (c < 0x80) { cp = c; return 1; }
  const int len = (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 0;
  if (len == 0 || i + len > n) return 0;
  cp = c & (0xFF >> (len + 1));
  for (int k = 1; k < len; k++) {
    if ((s[i + k] & 0xC0) != 0x80) return 0;
    cp = (cp << 6) | (s[i + k] & 0x3F);
  }
  return len;
}

// Encodes one piece into `out`; returns false if a byte or character of the piece has no one-character token (the caller falls back).
struct Cand {
  int32_t rank, pos, left, right;                      // pos: index of the left symbol; left/right: the ids the entry was made for
  bool operator>(const Cand& o) const { return rank != o.rank ? rank > o.rank : pos > o.pos; }
};

// Per-thread scratch of the encoder, reused from piece to piece.
struct Scratch {
  std::vector<int32_t> sym, prev, next;
  std::vector<Cand> heap;
  std::vector<uint32_t> cp;
  std::vector<int64_t> pos;
};

bool encode_piece(const Bpe& t, const uint8_t* s, int64_t n, std::vector<int32_t>& out, Scratch& w) {
  auto& sym = w.sym;
  auto& prev = w.prev;
  auto& next = w.next;
  auto& heap = w.heap;
  if (n == 0) return true;
  if (t.ignore_merges) {
    auto it = t.whole.find(std::string_view((const char*)s, (size_t)n));
    if (it != t.whole.end()) { out.push_back(it->second); return true; }
  }
  sym.clear();
  if (t.byte_level) {
    for (int64_t i = 0; i < n; i++) {
      const int32_t id = t.byte_sym[s[i]];
      if (id < 0) return false;
      sym.push_back(id);
    }
  } else {
    for (int64_t i = 0; i < n;) {
      uint32_t cp;
      const int len = utf8_next(s, i, n, cp);
      if (len == 0) return false;
      auto it = t.char_sym.find(cp);
      if (it == t.char_sym.end()) return false;
      sym.push_back(it->second);
      i += len;
    }
  }
  const int32_t m = (int32_t)sym.size();
  if (m == 1) { out.push_back(sym[0]); return true; }
  if (m == 2) {
    if (const Merge* mg = t.merges.find(key(sym[0], sym[1]))) out.push_back(mg->merged);
    else { out.push_back(sym[0]); out.push_back(sym[1]); }
    return true;
  }
  if (m <= 24) {
    // Short pieces (nearly all of them): pair ranks in a small array, rescanned for the leftmost minimum after every merge; cheaper than
    // the heap below until the piece gets long.
    int32_t id[24], rk[24];
    int32_t len = m;
    constexpr int32_t NONE = INT32_MAX;
    auto rank_of = [&](int32_t i) -> int32_t {
      const Merge* mg = t.merges.find(key(id[i], id[i + 1]));
      return mg ? mg->rank : NONE;
    };
    for (int32_t i = 0; i < m; i++) id[i] = sym[i];
    for (int32_t i = 0; i + 1 < m; i++) rk[i] = rank_of(i);
    for (;;) {
      int32_t best = NONE, bi = -1;
      for (int32_t i = 0; i + 1 < len; i++)
        if (rk[i] < best) { best = rk[i]; bi = i; }
      if (bi < 0) break;
      id[bi] = t.merges.find(key(id[bi], id[bi + 1]))->merged;
      for (int32_t i = bi + 1; i + 1 < len; i++) { id[i] = id[i + 1]; rk[i] = rk[i + 1]; }
      len--;
      if (bi > 0) rk[bi - 1] = rank_of(bi - 1);
      if (bi + 1 < len) rk[bi] = rank_of(bi);
    }
    out.insert(out.end(), id, id + len);
    return true;
  }
  prev.resize(m);
  next.resize(m);
  for (int32_t i = 0; i < m; i++) { prev[i] = i - 1; next[i] = i + 1 < m ? i + 1 : -1; }
  heap.clear();
  const std::greater<Cand> cmp;
  auto push = [&](int32_t i) {
    const int32_t j = next[i];
    if (j < 0) return;
    if (const Merge* mg = t.merges.find(key(sym[i], sym[j]))) {
      heap.push_back(Cand{mg->rank, i, sym[i], sym[j]});
      std::push_heap(heap.begin(), heap.end(), cmp);
    }
  };
  for (int32_t i = 0; i + 1 < m; i++) push(i);
  while (!heap.empty()) {
    std::pop_heap(heap.begin(), heap.end(), cmp);
    const Cand c = heap.back();
    heap.pop_back();
    const int32_t i = c.pos, j = sym[i] < 0 ? -1 : next[i];
    if (j < 0 || sym[i] != c.left || sym[j] != c.right) continue;          // one of the two symbols was merged away since the entry was pushed
    sym[i] = t.merges.find(key(c.left, c.right))->merged;
    sym[j] = -1;                                                           // unlinked
    next[i] = next[j];
    if (next[j] >= 0) prev[next[j]] = i;
    if (prev[i] >= 0) push(prev[i]);
    push(i);
  }
  for (int32_t i = 0; i >= 0; i = next[i]) out.push_back(sym[i]);
  return true;
}

// ---- pre-tokeniser ---------------------------------------------------------------------------------------------------
enum : uint8_t { CL = 1, CN = 2, CS = 4 };             // letter (\p{L}), number (\p{N}), white space (\s); 0 = everything else
std::vector<uint8_t> g_cls;                            // indexed by code point

inline uint8_t cls(uint32_t cp) { return cp < g_cls.size() ? g_cls[cp] : 0; }
inline bool is_nl(uint32_t c) { return c == '\r' || c == '\n'; }

// Length (in code points) of a contraction suffix 's 't 're 've 'm 'll 'd at cp[i], 0 if none. fold: ASCII letters of either case and
// U+017F (which the case-insensitive form of the pattern accepts for "s").
inline int contraction(const uint32_t* cp, int64_t i, int64_t m, bool fold) {
  if (cp[i] != '\'' || i + 1 >= m) return 0;
  auto low = [&](uint32_t c) -> uint32_t { return !fold ? c : (c >= 'A' && c <= 'Z') ? c + 32 : c == 0x17F ? 's' : c; };
  const uint32_t d = low(cp[i + 1]);
  if (d == 's' || d == 't' || d == 'm' || d == 'd') return 2;
  if (i + 2 < m) {
    const uint32_t e = low(cp[i + 2]);
    if ((d == 'r' && e == 'e') || (d == 'v' && e == 'e') || (d == 'l' && e == 'l')) return 3;
  }
  return 0;
}

// End of the white-space piece that starts at i (both patterns end with `\s+(?!\S)|\s+`): the whole run at the end of the text, the run
// without its last character when something follows it (that character then leads the next piece), a single character otherwise.
inline int64_t space_piece_end(const uint32_t* cp, int64_t i, int64_t m) {
  int64_t r = i;
  while (r < m && (cls(cp[r]) & CS)) r++;
  return r == m ? r : (r - i >= 2 ? r - 1 : i + 1);
}

// kind 0: 's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
inline int64_t next_piece_gpt2(const uint32_t* cp, int64_t i, int64_t m) {
  if (const int k = contraction(cp, i, m, false)) return i + k;
  int64_t j = i;
  if (cp[i] == ' ' && i + 1 < m && !(cls(cp[i + 1]) & CS)) j = i + 1;          // the optional space before a run
  const uint8_t c = cls(cp[j]);
  if (c & CS) return space_piece_end(cp, i, m);
  int64_t r = j + 1;
  if (c & CL) { while (r < m && (cls(cp[r]) & CL)) r++; }
  else if (c & CN) { while (r < m && (cls(cp[r]) & CN)) r++; }
  else { while (r < m && cls(cp[r]) == 0) r++; }
  return r;
}

// kind 1: (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
inline int64_t next_piece_llama3(const uint32_t* cp, int64_t i, int64_t m) {
  if (const int k = contraction(cp, i, m, true)) return i + k;
  const uint32_t ch = cp[i];
  const uint8_t c = cls(ch);
  if (c & CL) { int64_t r = i + 1; while (r < m && (cls(cp[r]) & CL)) r++; return r; }
  if (!(c & CN) && !is_nl(ch) && i + 1 < m && (cls(cp[i + 1]) & CL)) { int64_t r = i + 2; while (r < m && (cls(cp[r]) & CL)) r++; return r; }
  if (c & CN) { int64_t r = i + 1; while (r < m && r < i + 3 && (cls(cp[r]) & CN)) r++; return r; }
  int64_t j = -1;
  if (c == 0) j = i;
  else if (ch == ' ' && i + 1 < m && cls(cp[i + 1]) == 0) j = i + 1;
  if (j >= 0) {
    int64_t r = j + 1;
    while (r < m && cls(cp[r]) == 0) r++;
    while (r < m && is_nl(cp[r])) r++;
    return r;
  }
  int64_t r = i, last_nl = -1;                                                 // white space from here on
  while (r < m && (cls(cp[r]) & CS)) { if (is_nl(cp[r])) last_nl = r; r++; }
  if (last_nl >= 0) return last_nl + 1;
  return space_piece_end(cp, i, m);
}

// Splits text s[0..n) and encodes its pieces into out. False on malformed UTF-8 or a piece the engine cannot take.
bool encode_text(const Bpe& t, int kind, const uint8_t* s, int64_t n, std::vector<int32_t>& out, Scratch& w) {
  auto& cp = w.cp;
  auto& pos = w.pos;
  cp.clear();
  pos.clear();
  for (int64_t i = 0; i < n;) {
    uint32_t c;
    const int len = utf8_next(s, i, n, c);
    if (len == 0) return false;
    cp.push_back(c);
    pos.push_back(i);
    i += len;
  }
  pos.push_back(n);
  const int64_t m = (int64_t)cp.size();
  for (int64_t i = 0; i < m;) {
    const int64_t e = kind == 0 ? next_piece_gpt2(cp.data(), i, m) : next_piece_llama3(cp.data(), i, m);
    if (!encode_piece(t, s + pos[i], pos[e] - pos[i], out, w)) return false;
    i = e;
  }
  return true;
}

}  // namespace

// Installs the code-point class table used by ft_bpe_encode_texts: cls[c] = 1 letter | 2 number | 4 white space, for c < n.
FT_API void ft_tok_set_classes(const uint8_t* cls_table, int64_t n) { g_cls.assign(cls_table, cls_table + n); }

// Splits one text with the native matcher of pattern `kind` and writes the byte offset of the end of each piece to ends (capacity cap).
// Returns the number of pieces, -1 if cap is too small, -2 on malformed UTF-8, -1000000 without a class table.
FT_API int64_t ft_tok_split(int kind, const uint8_t* s, int64_t n, int64_t* ends, int64_t cap) {
  if (g_cls.empty() || kind < 0 || kind > 1) return -1000000;
  std::vector<uint32_t> cp;
  std::vector<int64_t> pos;
  for (int64_t i = 0; i < n;) {
    uint32_t c;
    const int len = utf8_next(s, i, n, c);
    if (len == 0) return -2;
    cp.push_back(c);
    pos.push_back(i);
    i += len;
  }
  pos.push_back(n);
  const int64_t m = (int64_t)cp.size();
  int64_t k = 0;
  for (int64_t i = 0; i < m;) {
    i = kind == 0 ? next_piece_gpt2(cp.data(), i, m) : next_piece_llama3(cp.data(), i, m);
    if (k >= cap) return -1;
    ends[k++] = pos[i];
  }
  return k;
}

// Builds a merge engine. left/right/merged [n_merges]: token ids of the two halves of merge r (r = its rank) and of their concatenation.
// byte_sym [256] (byte-level models) or char_cp/char_id [n_chars] (plain models; byte_sym null). whole_bytes/whole_off/whole_id
// [n_whole]: the vocabulary as raw piece bytes for models that emit a piece found in the vocabulary without merging (n_whole 0 otherwise).
// Returns an opaque handle for ft_bpe_encode / ft_bpe_destroy.
FT_API void* ft_bpe_create(const int32_t* left, const int32_t* right, const int32_t* merged, int64_t n_merges, const int32_t* byte_sym,
                           const uint32_t* char_cp, const int32_t* char_id, int64_t n_chars, const uint8_t* whole_bytes, const int64_t* whole_off,
                           const int32_t* whole_id, int64_t n_whole) {
  Bpe* t = new Bpe();
  t->merges.init(n_merges);
  for (int64_t r = 0; r < n_merges; r++) t->merges.insert(key(left[r], right[r]), Merge{(int32_t)r, merged[r]});   // first (lowest) rank wins
  t->byte_level = byte_sym != nullptr;
  if (byte_sym) std::memcpy(t->byte_sym, byte_sym, sizeof(t->byte_sym));
  for (int64_t i = 0; i < n_chars; i++) t->char_sym.emplace(char_cp[i], char_id[i]);
  if (n_whole > 0) {
    t->ignore_merges = true;
    t->whole_blob.assign((const char*)whole_bytes, (size_t)whole_off[n_whole]);
    t->whole.reserve((size_t)n_whole * 2);
    for (int64_t i = 0; i < n_whole; i++)
      t->whole.emplace(std::string_view(t->whole_blob.data() + whole_off[i], (size_t)(whole_off[i + 1] - whole_off[i])), whole_id[i]);
  }
  return t;
}

FT_API void ft_bpe_destroy(void* h) { delete static_cast<Bpe*>(h); }

// Encodes n_pieces pieces: piece p is bytes[off[p] .. off[p+1]). Writes the ids of all pieces, in order, to out (capacity out_cap; a piece
// never yields more ids than it has bytes, so off[n_pieces] is always enough) and the running id count after each piece to out_off
// [n_pieces + 1] (may be null). Returns the number of ids written, -1 if out_cap is too small, or -(2 + p) if piece p contains a byte or
// character without a one-character token (nothing useful is in out then).
FT_API int64_t ft_bpe_encode(void* h, const uint8_t* bytes, const int64_t* off, int64_t n_pieces, int32_t* out, int64_t out_cap, int64_t* out_off,
                             int nthreads) {
  const Bpe& t = *static_cast<const Bpe*>(h);
  if (n_pieces <= 0) { if (out_off) out_off[0] = 0; return 0; }
  const int64_t total_bytes = off[n_pieces] - off[0];
  nthreads = std::max(1, std::min<int>(nthreads, 64));
  if (total_bytes < (1 << 15)) nthreads = 1;
  nthreads = (int)std::min<int64_t>(nthreads, n_pieces);
  // contiguous ranges of pieces per thread, balanced by bytes
  std::vector<int64_t> lo(nthreads + 1, n_pieces);
  lo[0] = 0;
  for (int k = 1, p = 0; k < nthreads; k++) {
    const int64_t target = off[0] + total_bytes * k / nthreads;
    while (p < n_pieces && off[p] < target) p++;
    lo[k] = p;
  }
  std::vector<std::vector<int32_t>> ids(nthreads);
  std::vector<std::vector<int64_t>> counts(nthreads);
  std::atomic<int64_t> bad{-1};
  auto work = [&](int k) {
    Scratch w;
    auto& o = ids[k];
    o.reserve((size_t)(off[lo[k + 1]] - off[lo[k]]) / 3 + 16);
    counts[k].reserve((size_t)(lo[k + 1] - lo[k]));
    for (int64_t p = lo[k]; p < lo[k + 1]; p++) {
      if (!encode_piece(t, bytes + off[p], off[p + 1] - off[p], o, w)) {
        int64_t expect = -1;
        bad.compare_exchange_strong(expect, p);
        return;
      }
      counts[k].push_back((int64_t)o.size());
    }
  };
  if (nthreads == 1) {
    work(0);
  } else {
    std::vector<std::thread> ts;
    for (int k = 0; k < nthreads; k++) ts.emplace_back(work, k);
    for (auto& th : ts) th.join();
  }
  if (bad.load() >= 0) return -(2 + bad.load());
  int64_t total = 0;
  for (auto& v : ids) total += (int64_t)v.size();
  if (total > out_cap) return -1;
  int64_t base = 0;
  if (out_off) out_off[0] = 0;
  for (int k = 0; k < nthreads; k++) {
    if (!ids[k].empty()) std::memcpy(out + base, ids[k].data(), ids[k].size() * sizeof(int32_t));
    if (out_off)
      for (int64_t p = lo[k]; p < lo[k + 1]; p++) out_off[p + 1] = base + counts[k][p - lo[k]];
    base += (int64_t)ids[k].size();
  }
  return total;
}

// Splits and encodes n_texts texts: text k is bytes[off[k] .. off[k+1]), kind 0 = the GPT-2 pattern, 1 = the Llama-3 pattern. Output as in
// ft_bpe_encode with one entry of out_off per text. Returns the number of ids, -1 if out_cap is too small, -(2 + k) if text k is not
// valid UTF-8 or holds a byte or character without a one-character token, -1000000 if no class table has been installed.
FT_API int64_t ft_bpe_encode_texts(void* h, int kind, const uint8_t* bytes, const int64_t* off, int64_t n_texts, int32_t* out, int64_t out_cap,
                                   int64_t* out_off, int nthreads) {
  const Bpe& t = *static_cast<const Bpe*>(h);
  if (g_cls.empty() || kind < 0 || kind > 1) return -1000000;
  if (n_texts <= 0) { if (out_off) out_off[0] = 0; return 0; }
  const int64_t total_bytes = off[n_texts] - off[0];
  nthreads = std::max(1, std::min<int>(nthreads, 64));
  if (total_bytes < (1 << 15)) nthreads = 1;
  nthreads = (int)std::min<int64_t>(nthreads, n_texts);
  // Texts are handed out one at a time, longest first: a batch of uneven files keeps every thread busy to the end.
  std::vector<int64_t> order(n_texts);
  for (int64_t k = 0; k < n_texts; k++) order[k] = k;
  if (nthreads > 1) std::sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return off[a + 1] - off[a] > off[b + 1] - off[b]; });
  std::vector<std::vector<int32_t>> ids(n_texts);
  std::atomic<int64_t> cursor{0}, bad{-1};
  auto work = [&]() {
    Scratch w;
    for (;;) {
      const int64_t q = cursor.fetch_add(1);
      if (q >= n_texts || bad.load() >= 0) return;
      const int64_t k = order[q];
      ids[k].reserve((size_t)(off[k + 1] - off[k]) / 3 + 16);
      if (!encode_text(t, kind, bytes + off[k], off[k + 1] - off[k], ids[k], w)) {
        int64_t expect = -1;
        bad.compare_exchange_strong(expect, k);
        return;
      }
    }
  };
  if (nthreads == 1) {
    work();
  } else {
    std::vector<std::thread> ts;
    for (int k = 0; k < nthreads; k++) ts.emplace_back(work);
    for (auto& th : ts) th.join();
  }
  if (bad.load() >= 0) return -(2 + bad.load());
  int64_t total = 0;
  for (auto& v : ids) total += (int64_t)v.size();
  if (total > out_cap) return -1;
  int64_t base = 0;
  if (out_off) out_off[0] = 0;
  for (int64_t k = 0; k < n_texts; k++) {
    if (!ids[k].empty()) std::memcpy(out + base, ids[k].data(), ids[k].size() * sizeof(int32_t));
    base += (int64_t)ids[k].size();
    if (out_off) out_off[k + 1] = base;
  }
  return total;
}
