// Self-test of the host runtime, meant to be built with -fsanitize=thread or -fsanitize=address,undefined together with
// dist_runtime.cpp, loader.cpp and vision_ops.cpp: ranks are threads of this process, over the in-process fabric and over TCP on
// loopback. Exits 0 and prints "selftest ok" when every check passed; a sanitizer report makes the process exit non-zero.
//
// The reference has no sanitizer configuration (its ranks-as-threads pattern is ferrotorch-distributed/src/fsdp.rs:946-976 and
// tests/conformance_distributed.rs:615-680); this driver is that pattern under ThreadSanitizer / AddressSanitizer.
#include <atomic>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <string>
#include <thread>
#include <vector>

#include <unistd.h>

extern "C" {
int64_t ft_tcp_backend_create(int rank, int world, const char* host, int port, int full_mesh, int64_t connect_timeout_ms, int* err);
int64_t ft_sim_fabric_create(int world);
int64_t ft_sim_backend_create(int64_t fabric, int rank);
int64_t ft_sub_backend_create(int64_t parent, const int* members, int n);
void ft_backend_destroy(int64_t h);
int ft_backend_rank(int64_t h);
int ft_backend_world(int64_t h);
int ft_backend_send(int64_t h, const void* d, int64_t n, int dst);
int ft_backend_recv(int64_t h, void* d, int64_t n, int src, int64_t timeout_ms);
int ft_backend_barrier(int64_t h, int64_t timeout_ms);
int ft_backend_set_fault(int64_t h, int kind, int64_t param);
int ft_allreduce(int64_t h, void* data, int64_t n, int dtype, int op, int algo, int64_t timeout_ms);
int ft_broadcast(int64_t h, void* data, int64_t bytes, int root, int algo, int64_t timeout_ms);
int ft_all_gather(int64_t h, const void* mine, int64_t bytes, void* out, int64_t timeout_ms);
int ft_reduce_scatter(int64_t h, const void* full, int64_t chunk, void* out, int dtype, int op, int64_t timeout_ms);
int ft_all_to_all(int64_t h, const void* send, const int64_t* send_counts, void* recv, const int64_t* recv_counts, int64_t timeout_ms);
int ft_ddp_plan_buckets(const int64_t* numels, int n_params, int elem_bytes, int64_t cap_bytes, int* bucket_of);
int ft_gather_rows(const void* src, int64_t row_bytes, const int64_t* idx, int64_t n, int64_t n_rows_src, void* dst, int nthreads);
void ft_permutation(int64_t n, uint64_t seed, int64_t* out);
void ft_philox_uniform(uint64_t seed, uint64_t offset, int64_t n, float* out);
void ft_philox_normal(uint64_t seed, uint64_t offset, int64_t n, float* out);
int64_t ft_nms_sorted_f32(const float* boxes, int64_t n, float thr, uint8_t* keep);
void ft_tok_set_classes(const uint8_t* cls_table, int64_t n);
int64_t ft_tok_split(int kind, const uint8_t* s, int64_t n, int64_t* ends, int64_t cap);
void* ft_bpe_create(const int32_t* left, const int32_t* right, const int32_t* merged, int64_t n_merges, const int32_t* byte_sym, const uint32_t* char_cp,
                    const int32_t* char_id, int64_t n_chars, const uint8_t* whole_bytes, const int64_t* whole_off, const int32_t* whole_id, int64_t n_whole);
void ft_bpe_destroy(void* h);
int64_t ft_bpe_encode(void* h, const uint8_t* bytes, const int64_t* off, int64_t n_pieces, int32_t* out, int64_t out_cap, int64_t* out_off, int nthreads);
void* ft_json_grammar_create(const int32_t* kind, const int32_t* edge_first, int64_t n_nodes, const uint8_t* lits, const int64_t* lit_off,
                             const int32_t* edge_child, const uint8_t* edge_required, const uint8_t* vocab, const int64_t* voff, int64_t n_vocab);
void ft_json_grammar_destroy(void* h);
int ft_json_grammar_check(void* h, const uint8_t* text, int64_t n, int* is_complete);
int64_t ft_json_grammar_mask(void* h, const uint8_t* text, int64_t n, int64_t eos_id, uint8_t* allowed, int nthreads);
void ft_json_grammar_mask_batch(void* h, const uint8_t* texts, const int64_t* off, int64_t n_texts, int64_t eos_id, uint8_t* allowed, int64_t* counts, int nthreads);
int ft_la_cholesky(double* a, int64_t batch, int64_t n, int32_t* info);
int ft_la_lu(double* a, int64_t batch, int64_t m, int64_t n, int32_t* piv, int32_t* info);
int ft_la_lu_solve(const double* lu, const int32_t* piv, double* bmat, int64_t batch, int64_t n, int64_t k, int trans);
int ft_la_trsm(const double* t, double* bmat, int64_t batch, int64_t n, int64_t k, int upper, int trans, int unit);
int ft_la_qr(const double* a, double* q, double* r, int64_t batch, int64_t m, int64_t n, int complete);
int ft_la_eigh(const double* a, double* w, double* v, int64_t batch, int64_t n, int lower);
int ft_la_svd(const double* a, double* u, double* s, double* vt, int64_t batch, int64_t m, int64_t n);
int ft_la_eig(const double* a, double* w, double* v, int64_t batch, int64_t n);
int64_t ft_bpe_encode_texts(void* h, int kind, const uint8_t* bytes, const int64_t* off, int64_t n_texts, int32_t* out, int64_t out_cap, int64_t* out_off,
                            int nthreads);
}

static std::atomic<int> g_fail{0};
#define CHECK(cond)                                                                     \
  do {                                                                                  \
    if (!(cond)) {                                                                      \
      std::fprintf(stderr, "selftest: %s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
      g_fail++;                                                                         \
    }                                                                                   \
  } while (0)

constexpr int64_t TMO = 20000;
constexpr int E_TIMEOUT = 9;

// every rank runs `body(handle, rank)` on its own thread
static void run_ranks(const std::vector<int64_t>& handles, const std::function<void(int64_t, int)>& body) {
  std::vector<std::thread> th;
  for (size_t r = 0; r < handles.size(); r++) th.emplace_back([&, r] { body(handles[r], (int)r); });
  for (auto& t : th) t.join();
}

// neighbours_connected: ring / tree algorithms need links between non-zero ranks (the in-process fabric, full-mesh TCP)
static void collectives(const std::vector<int64_t>& hs, int world, bool neighbours_connected) {
  run_ranks(hs, [world, neighbours_connected](int64_t h, int r) {
    CHECK(ft_backend_rank(h) == r && ft_backend_world(h) == world);
    for (int algo = 0; algo < (neighbours_connected ? 2 : 1); algo++) {
      for (int64_t n : {1, 7, 1000, 40001, 600011}) {          // the last one takes the chunked star path (2.4 MB)
        std::vector<float> v((size_t)n);
        for (int64_t i = 0; i < n; i++) v[(size_t)i] = (float)(r + 1) + (float)(i % 13);
        CHECK(ft_allreduce(h, v.data(), n, 0, 0, algo, TMO) == 0);
        for (int64_t i = 0; i < n; i += 97) CHECK(std::fabs(v[(size_t)i] - (world * (world + 1) / 2.0f + world * (float)(i % 13))) < 1e-3f);
        std::vector<double> d((size_t)n, (double)(r + 1));
        CHECK(ft_allreduce(h, d.data(), n, 1, 1, algo, TMO) == 0);             // mean
        CHECK(std::fabs(d[0] - (world + 1) / 2.0) < 1e-12);
        std::vector<float> m((size_t)n, (float)r);
        CHECK(ft_allreduce(h, m.data(), n, 0, 2, algo, TMO) == 0);             // max
        CHECK(m[(size_t)n - 1] == (float)(world - 1));
      }
      for (int root = 0; root < (neighbours_connected ? world : 1); root++) {      // on the star only rank 0 reaches everybody
        std::vector<uint8_t> b(3001, (uint8_t)(r == root ? 42 + root : 0));
        CHECK(ft_broadcast(h, b.data(), (int64_t)b.size(), root, algo, TMO) == 0);
        CHECK(b[0] == 42 + root && b[3000] == 42 + root);
      }
    }
    std::vector<int32_t> mine(5, r), all((size_t)5 * world, -1);
    CHECK(ft_all_gather(h, mine.data(), 20, all.data(), TMO) == 0);
    for (int q = 0; q < world; q++) CHECK(all[(size_t)q * 5 + 4] == q);
    std::vector<float> full((size_t)world * 6), out(6);
    for (size_t i = 0; i < full.size(); i++) full[i] = (float)(r + 1) * (float)(i + 1);
    CHECK(ft_reduce_scatter(h, full.data(), 6, out.data(), 0, 0, TMO) == 0);
    for (int i = 0; i < 6; i++) CHECK(std::fabs(out[i] - (world * (world + 1) / 2.0f) * (float)(r * 6 + i + 1)) < 1e-3f);
    if (!neighbours_connected) { CHECK(ft_backend_barrier(h, TMO) == 0); return; }
    // uneven all-to-all: rank r sends (q + 1) bytes to rank q, so it receives (r + 1) bytes from everyone
    std::vector<int64_t> sc(world), rc(world);
    size_t stot = 0;
    for (int q = 0; q < world; q++) { sc[q] = q + 1; rc[q] = r + 1; stot += (size_t)q + 1; }
    std::vector<uint8_t> sb(stot, (uint8_t)(100 + r)), rb((size_t)(r + 1) * world, 0);
    CHECK(ft_all_to_all(h, sb.data(), sc.data(), rb.data(), rc.data(), TMO) == 0);
    for (int q = 0; q < world; q++) CHECK(rb[(size_t)q * (r + 1)] == (uint8_t)(100 + q));
    CHECK(ft_backend_barrier(h, TMO) == 0);
  });
}

static void test_simulated() {
  const int world = 4;
  const int64_t fab = ft_sim_fabric_create(world);
  CHECK(fab != 0);
  std::vector<int64_t> hs;
  for (int r = 0; r < world; r++) hs.push_back(ft_sim_backend_create(fab, r));
  collectives(hs, world, true);
  // sub-group {1, 3}: a two-rank view on the same fabric, used concurrently with a {0, 2} view
  const int a[2] = {1, 3}, b[2] = {0, 2};
  std::vector<int64_t> sub(world);
  sub[1] = ft_sub_backend_create(hs[1], a, 2);
  sub[3] = ft_sub_backend_create(hs[3], a, 2);
  sub[0] = ft_sub_backend_create(hs[0], b, 2);
  sub[2] = ft_sub_backend_create(hs[2], b, 2);
  run_ranks(sub, [](int64_t h, int r) {
    CHECK(h != 0 && ft_backend_world(h) == 2);
    float v = (float)r;
    CHECK(ft_allreduce(h, &v, 1, 0, 0, 0, TMO) == 0);
    CHECK(v == ((r % 2) ? 4.0f : 2.0f));
  });
  // a receive nobody answers runs into its timeout; a dropped message does too
  uint8_t byte = 0;
  CHECK(ft_backend_recv(hs[0], &byte, 1, 1, 50) == E_TIMEOUT);
  CHECK(ft_backend_set_fault(hs[2], 1, 0) == 0);                                 // drop the next send of rank 2
  CHECK(ft_backend_send(hs[2], &byte, 1, 3) == 0);
  CHECK(ft_backend_recv(hs[3], &byte, 1, 2, 50) == E_TIMEOUT);
  for (auto h : sub) ft_backend_destroy(h);
  for (auto h : hs) ft_backend_destroy(h);
  ft_backend_destroy(fab);
}

static void test_tcp(int full_mesh) {
  const int world = 3;
  const int port = 20000 + (int)(getpid() % 20000) + full_mesh;
  std::vector<int64_t> hs(world, 0);
  {
    std::vector<std::thread> th;
    for (int r = 0; r < world; r++)
      th.emplace_back([&, r] {
        int err = -1;
        hs[(size_t)r] = ft_tcp_backend_create(r, world, "127.0.0.1", port, full_mesh, TMO, &err);
        CHECK(err == 0 && hs[(size_t)r] != 0);
      });
    for (auto& t : th) t.join();
  }
  if (g_fail) return;
  collectives(hs, world, full_mesh != 0);
  for (auto h : hs) ft_backend_destroy(h);
}

static void test_loader_and_planner() {
  const int64_t numels[5] = {10, 3000000, 5, 7000000, 100};
  int bucket_of[5];
  const int nb = ft_ddp_plan_buckets(numels, 5, 4, 25 << 20, bucket_of);
  CHECK(nb == 3 && bucket_of[4] == 0 && bucket_of[3] == 1 && bucket_of[2] == 2 && bucket_of[1] == 2 && bucket_of[0] == 2);
  const int64_t rows = 30000, row_bytes = 52;          // 1.5 MB: large enough for the threaded path
  std::vector<uint8_t> src((size_t)(rows * row_bytes));
  for (size_t i = 0; i < src.size(); i++) src[i] = (uint8_t)(i / row_bytes);
  std::vector<int64_t> perm((size_t)rows);
  ft_permutation(rows, 9, perm.data());
  std::vector<uint8_t> seen((size_t)rows, 0);
  for (auto p : perm) { CHECK(p >= 0 && p < rows); seen[(size_t)p]++; }
  for (auto s : seen) CHECK(s == 1);
  std::vector<uint8_t> dst(src.size());
  CHECK(ft_gather_rows(src.data(), row_bytes, perm.data(), rows, rows, dst.data(), 4) == 0);
  for (int64_t i = 0; i < rows; i += 37) CHECK(dst[(size_t)(i * row_bytes)] == (uint8_t)perm[(size_t)i]);
  const int64_t bad[1] = {rows};
  CHECK(ft_gather_rows(src.data(), row_bytes, bad, 1, rows, dst.data(), 1) != 0);
  std::vector<float> u(1001), u2(1001), nrm(1001);
  ft_philox_uniform(3, 0, 1001, u.data());
  ft_philox_uniform(3, 0, 1001, u2.data());
  ft_philox_normal(3, 0, 1001, nrm.data());
  double mean = 0;
  for (size_t i = 0; i < u.size(); i++) { CHECK(u[i] == u2[i] && u[i] >= 0.f && u[i] < 1.f); mean += nrm[i]; }
  CHECK(std::fabs(mean / 1001.0) < 0.2);
  // boxes sorted by score: the second overlaps the first heavily, the third is apart
  const float boxes[12] = {0, 0, 10, 10, 1, 1, 10, 10, 20, 20, 30, 30};
  uint8_t keep[3] = {0, 0, 0};
  CHECK(ft_nms_sorted_f32(boxes, 3, 0.5f, keep) == 2);
  CHECK(keep[0] == 1 && keep[1] == 0 && keep[2] == 1);
}

// Byte-level vocabulary: ids 0..255 are the bytes, 256 = "ab", 257 = "abc", 258 = " a", 259 = " ab" (never reachable: rank order forms
// "ab" first). Single-threaded and threaded calls must agree, short pieces (array scan) and long ones (heap) too.
static void test_tokenizer() {
  std::vector<uint8_t> cls(128, 0);
  for (int c = 'a'; c <= 'z'; c++) cls[(size_t)c] = 1;
  for (int c = '0'; c <= '9'; c++) cls[(size_t)c] = 2;
  cls[' '] = cls['\n'] = cls['\t'] = cls['\r'] = 4;
  ft_tok_set_classes(cls.data(), (int64_t)cls.size());
  int32_t byte_sym[256];
  for (int i = 0; i < 256; i++) byte_sym[i] = i;
  const int32_t left[4] = {'a', 256, ' ', 258}, right[4] = {'b', 'c', 'a', 'b'}, merged[4] = {256, 257, 258, 259};
  void* h = ft_bpe_create(left, right, merged, 4, byte_sym, nullptr, nullptr, 0, nullptr, nullptr, nullptr, 0);
  CHECK(h != nullptr);
  const char* text = "abc ab  abcabc 12";
  int64_t ends[32];
  const int64_t np = ft_tok_split(0, (const uint8_t*)text, (int64_t)std::strlen(text), ends, 32);
  CHECK(np == 5 && ends[0] == 3 && ends[1] == 6 && ends[2] == 7 && ends[3] == 14 && ends[4] == 17);   // "abc" " ab" " " " abcabc" " 12"
  std::string big;
  for (int i = 0; i < 4000; i++) big += (i % 7 == 0) ? std::string(40, 'a') + "b " : "abc ab\n";
  std::vector<std::string> texts(9, big);
  texts.push_back(text);
  std::string blob;
  std::vector<int64_t> off{0};
  for (auto& t : texts) { blob += t; off.push_back((int64_t)blob.size()); }
  std::vector<int32_t> a(blob.size()), b(blob.size());
  std::vector<int64_t> ao(texts.size() + 1), bo(texts.size() + 1);
  const int64_t na = ft_bpe_encode_texts(h, 0, (const uint8_t*)blob.data(), off.data(), (int64_t)texts.size(), a.data(), (int64_t)a.size(), ao.data(), 1);
  const int64_t nb = ft_bpe_encode_texts(h, 0, (const uint8_t*)blob.data(), off.data(), (int64_t)texts.size(), b.data(), (int64_t)b.size(), bo.data(), 4);
  CHECK(na > 0 && na == nb && ao == bo && std::equal(a.begin(), a.begin() + na, b.begin()));
  const int64_t last = ao[texts.size() - 1];
  // "abc" | " ab" -> ' ' 256 ... : " a" (rank 2) loses to "ab" (rank 0)
  CHECK(a[(size_t)last] == 257 && a[(size_t)last + 1] == ' ' && a[(size_t)last + 2] == 256);
  const int64_t moff[2] = {0, 2};
  CHECK(ft_bpe_encode_texts(h, 0, (const uint8_t*)"\xff\xfe", moff, 1, a.data(), 2, nullptr, 1) == -2);   // malformed UTF-8 is refused
  const int64_t poff[3] = {0, 3, 43};
  const std::string pieces = "abc" + std::string(39, 'a') + "b";
  CHECK(ft_bpe_encode(h, (const uint8_t*)pieces.data(), poff, 2, a.data(), (int64_t)a.size(), ao.data(), 2) == 1 + 39 && ao[1] == 1);
  ft_bpe_destroy(h);
}

// Schema {"a": integer (required)} over a vocabulary large enough for the threaded walk; the masks of one and of several threads must agree.
static void test_grammar() {
  const int32_t kind[2] = {0, 4}, edge_first[3] = {0, 1, 1}, child[1] = {1};
  const uint8_t req[1] = {1};
  const std::string lits = "\"a\"";
  const int64_t lit_off[2] = {0, 3};
  std::vector<std::string> vocab = {"{", "}", "\"a\"", ":", "1", "12}", "x", "", "<eos>"};
  for (int i = 0; i < 9000; i++) vocab.push_back((i % 3 == 0 ? "1" : "q") + std::to_string(i));
  std::string blob;
  std::vector<int64_t> voff{0};
  for (auto& v : vocab) { blob += v; voff.push_back((int64_t)blob.size()); }
  void* h = ft_json_grammar_create(kind, edge_first, 2, (const uint8_t*)lits.data(), lit_off, child, req, (const uint8_t*)blob.data(), voff.data(), (int64_t)vocab.size());
  CHECK(h != nullptr);
  int done = -1;
  CHECK(ft_json_grammar_check(h, (const uint8_t*)"{\"a\":1", 6, &done) == 1 && done == 0);
  CHECK(ft_json_grammar_check(h, (const uint8_t*)"{\"a\":1}", 7, &done) == 1 && done == 1);
  CHECK(ft_json_grammar_check(h, (const uint8_t*)"{\"b", 3, &done) == 0);
  std::vector<uint8_t> m1(vocab.size()), m4(vocab.size());
  const int64_t c1 = ft_json_grammar_mask(h, (const uint8_t*)"{\"a\":", 5, 8, m1.data(), 1);
  const int64_t c4 = ft_json_grammar_mask(h, (const uint8_t*)"{\"a\":", 5, 8, m4.data(), 4);
  CHECK(c1 == c4 && m1 == m4 && c1 == 2 + 3000);          // "1", "12}" and every "1<digits>" entry
  CHECK(m1[4] == 1 && m1[5] == 1 && m1[6] == 0 && m1[7] == 0 && m1[8] == 0);
  CHECK(ft_json_grammar_mask(h, (const uint8_t*)"{\"a\":1}", 7, 8, m1.data(), 4) == 1 && m1[8] == 1);
  const std::vector<std::string> texts = {"", "{", "{\"a\"", "{\"a\":", "{\"a\":1", "{\"a\":12}"};
  std::string tb;
  std::vector<int64_t> toff{0};
  for (auto& t : texts) { tb += t; toff.push_back((int64_t)tb.size()); }
  std::vector<uint8_t> mb(texts.size() * vocab.size());
  std::vector<int64_t> cnt(texts.size());
  ft_json_grammar_mask_batch(h, (const uint8_t*)tb.data(), toff.data(), (int64_t)texts.size(), 8, mb.data(), cnt.data(), 4);
  for (size_t k = 0; k < texts.size(); k++) {              // every row equals the mask of that text computed on its own
    const int64_t c = ft_json_grammar_mask(h, (const uint8_t*)texts[k].data(), (int64_t)texts[k].size(), 8, m1.data(), 1);
    CHECK(c == cnt[k] && std::equal(m1.begin(), m1.end(), mb.begin() + (int64_t)(k * vocab.size())));
  }
  ft_json_grammar_destroy(h);
}

// A batch large enough for the threaded path: every factorisation must reproduce its input (A = L L^T, P A = L U and A x = b, A = Q R,
// A = V diag(w) V^T, A = U diag(s) V^T) on each matrix of the batch.
static void test_linalg() {
  const int64_t batch = 64, n = 24, m = 30;
  uint64_t seed = 7;
  auto rnd = [&]() { seed = seed * 6364136223846793005ull + 1442695040888963407ull; return (double)((seed >> 33) % 2001) / 1000.0 - 1.0; };
  std::vector<double> a((size_t)(batch * n * n)), spd(a.size()), rect((size_t)(batch * m * n));
  for (auto& x : a) x = rnd();
  for (auto& x : rect) x = rnd();
  for (int64_t b = 0; b < batch; b++)
    for (int64_t i = 0; i < n; i++)
      for (int64_t j = 0; j < n; j++) {
        double s = i == j ? (double)n : 0.0;
        for (int64_t k = 0; k < n; k++) s += a[(size_t)(b * n * n + i * n + k)] * a[(size_t)(b * n * n + j * n + k)];
        spd[(size_t)(b * n * n + i * n + j)] = s;
      }
  auto maxerr = [](const std::vector<double>& x, const std::vector<double>& y) { double e = 0; for (size_t i = 0; i < x.size(); i++) e = std::max(e, std::fabs(x[i] - y[i])); return e; };
  std::vector<int32_t> info((size_t)batch), piv((size_t)(batch * n));
  std::vector<double> l = spd, rec(spd.size());
  CHECK(ft_la_cholesky(l.data(), batch, n, info.data()) == 0);
  for (int64_t b = 0; b < batch; b++) {
    CHECK(info[(size_t)b] == 0);
    for (int64_t i = 0; i < n; i++)
      for (int64_t j = 0; j < n; j++) {
        double s = 0;
        for (int64_t k = 0; k < n; k++) s += l[(size_t)(b * n * n + i * n + k)] * l[(size_t)(b * n * n + j * n + k)];
        rec[(size_t)(b * n * n + i * n + j)] = s;
      }
  }
  CHECK(maxerr(rec, spd) < 1e-9);
  std::vector<double> lu = a, rhs((size_t)(batch * n * 2)), x;
  for (auto& v : rhs) v = rnd();
  x = rhs;
  CHECK(ft_la_lu(lu.data(), batch, n, n, piv.data(), info.data()) == 0);
  CHECK(ft_la_lu_solve(lu.data(), piv.data(), x.data(), batch, n, 2, 0) == 0);
  std::vector<double> ax(rhs.size(), 0.0);
  for (int64_t b = 0; b < batch; b++)
    for (int64_t i = 0; i < n; i++)
      for (int64_t c = 0; c < 2; c++)
        for (int64_t k = 0; k < n; k++) ax[(size_t)(b * n * 2 + i * 2 + c)] += a[(size_t)(b * n * n + i * n + k)] * x[(size_t)(b * n * 2 + k * 2 + c)];
  CHECK(maxerr(ax, rhs) < 1e-8);
  std::vector<double> t = l, y = rhs;                       // L z = rhs, then check L z
  CHECK(ft_la_trsm(t.data(), y.data(), batch, n, 2, 0, 0, 0) == 0);
  std::fill(ax.begin(), ax.end(), 0.0);
  for (int64_t b = 0; b < batch; b++)
    for (int64_t i = 0; i < n; i++)
      for (int64_t c = 0; c < 2; c++)
        for (int64_t k = 0; k <= i; k++) ax[(size_t)(b * n * 2 + i * 2 + c)] += l[(size_t)(b * n * n + i * n + k)] * y[(size_t)(b * n * 2 + k * 2 + c)];
  CHECK(maxerr(ax, rhs) < 1e-9);
  std::vector<double> q((size_t)(batch * m * n)), r((size_t)(batch * n * n)), qr(rect.size(), 0.0);
  CHECK(ft_la_qr(rect.data(), q.data(), r.data(), batch, m, n, 0) == 0);
  for (int64_t b = 0; b < batch; b++)
    for (int64_t i = 0; i < m; i++)
      for (int64_t j = 0; j < n; j++)
        for (int64_t k = 0; k < n; k++) qr[(size_t)(b * m * n + i * n + j)] += q[(size_t)(b * m * n + i * n + k)] * r[(size_t)(b * n * n + k * n + j)];
  CHECK(maxerr(qr, rect) < 1e-10);
  std::vector<double> w((size_t)(batch * n)), v((size_t)(batch * n * n));
  CHECK(ft_la_eigh(spd.data(), w.data(), v.data(), batch, n, 1) > 0);
  std::fill(rec.begin(), rec.end(), 0.0);
  for (int64_t b = 0; b < batch; b++)
    for (int64_t i = 0; i < n; i++)
      for (int64_t j = 0; j < n; j++)
        for (int64_t k = 0; k < n; k++) rec[(size_t)(b * n * n + i * n + j)] += v[(size_t)(b * n * n + i * n + k)] * w[(size_t)(b * n + k)] * v[(size_t)(b * n * n + j * n + k)];
  CHECK(maxerr(rec, spd) < 1e-8);
  std::vector<double> u((size_t)(batch * m * n)), sv((size_t)(batch * n)), vt((size_t)(batch * n * n)), usv(rect.size(), 0.0);
  CHECK(ft_la_svd(rect.data(), u.data(), sv.data(), vt.data(), batch, m, n) > 0);
  for (int64_t b = 0; b < batch; b++)
    for (int64_t i = 0; i < m; i++)
      for (int64_t j = 0; j < n; j++)
        for (int64_t k = 0; k < n; k++) usv[(size_t)(b * m * n + i * n + j)] += u[(size_t)(b * m * n + i * n + k)] * sv[(size_t)(b * n + k)] * vt[(size_t)(b * n * n + k * n + j)];
  CHECK(maxerr(usv, rect) < 1e-10);
  for (int64_t b = 0; b < batch; b++)
    for (int64_t k = 0; k + 1 < n; k++) CHECK(sv[(size_t)(b * n + k)] >= sv[(size_t)(b * n + k + 1)]);
  std::vector<double> ew((size_t)(batch * n * 2)), ev((size_t)(batch * n * n * 2));
  CHECK(ft_la_eig(a.data(), ew.data(), ev.data(), batch, n) == 1);
  double worst = 0.0;                                      // A v - lambda v, real and imaginary parts, for every pair of every matrix
  for (int64_t b = 0; b < batch; b++)
    for (int64_t k = 0; k < n; k++) {
      const double lr = ew[(size_t)((b * n + k) * 2)], li = ew[(size_t)((b * n + k) * 2 + 1)];
      for (int64_t i = 0; i < n; i++) {
        double sr = 0, si = 0;
        for (int64_t j = 0; j < n; j++) {
          sr += a[(size_t)(b * n * n + i * n + j)] * ev[(size_t)(((b * n + j) * n + k) * 2)];
          si += a[(size_t)(b * n * n + i * n + j)] * ev[(size_t)(((b * n + j) * n + k) * 2 + 1)];
        }
        const double vr = ev[(size_t)(((b * n + i) * n + k) * 2)], vi = ev[(size_t)(((b * n + i) * n + k) * 2 + 1)];
        worst = std::max(worst, std::max(std::fabs(sr - (lr * vr - li * vi)), std::fabs(si - (lr * vi + li * vr))));
      }
    }
  CHECK(worst < 1e-10);
}

int main() {
  test_loader_and_planner();
  test_tokenizer();
  test_grammar();
  test_linalg();
  test_simulated();
  test_tcp(0);
  test_tcp(1);
  if (g_fail) {
    std::fprintf(stderr, "selftest: %d check(s) failed\n", g_fail.load());
    return 1;
  }
  std::printf("selftest ok\n");
  return 0;
}
