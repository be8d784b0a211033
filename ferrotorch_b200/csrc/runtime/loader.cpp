// Native pieces of the data pipeline: multi-threaded row gather (the collate hot loop for in-memory datasets), a
// SplitMix64/Fisher-Yates permutation for samplers, and a Philox4x32-10 generator that matches the device kernels
// (same key/counter layout) so host-side and device-side random streams can be replayed from a checkpointed state.
//
// Capability parity: rayon worker collate (ferrotorch-data/src/dataloader.rs:905-1255), sampler shuffles
// (sampler.rs:95-188), Philox state (ferrotorch-gpu/src/rng.rs:75-520).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#define FT_API extern "C" __attribute__((visibility("default")))

// dst[i, :] = src[idx[i], :] for i < n, rows of row_bytes bytes, split over nthreads threads.
FT_API int ft_gather_rows(const void* src, int64_t row_bytes, const int64_t* idx, int64_t n, int64_t n_rows_src, void* dst, int nthreads) {
  if (row_bytes <= 0 || n < 0) return 12;
  for (int64_t i = 0; i < n; i++) if (idx[i] < 0 || idx[i] >= n_rows_src) return 12;
  nthreads = std::max(1, std::min<int>(nthreads, 64));
  if (n * row_bytes < (1 << 20) || nthreads == 1) {
    for (int64_t i = 0; i < n; i++) std::memcpy((uint8_t*)dst + i * row_bytes, (const uint8_t*)src + idx[i] * row_bytes, (size_t)row_bytes);
    return 0;
  }
  std::vector<std::thread> ts;
  const int64_t per = (n + nthreads - 1) / nthreads;
  for (int t = 0; t < nthreads; t++) {
    const int64_t lo = t * per, hi = std::min<int64_t>(n, lo + per);
    if (lo >= hi) break;
    ts.emplace_back([=] {
      for (int64_t i = lo; i < hi; i++) std::memcpy((uint8_t*)dst + i * row_bytes, (const uint8_t*)src + idx[i] * row_bytes, (size_t)row_bytes);
    });
  }
  for (auto& t : ts) t.join();
  return 0;
}

static inline uint64_t splitmix64(uint64_t& s) {
  uint64_t z = (s += 0x9e3779b97f4a7c15ull);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

// out[0..n) = a permutation of 0..n-1 determined by seed (Fisher-Yates driven by SplitMix64).
FT_API void ft_permutation(int64_t n, uint64_t seed, int64_t* out) {
  for (int64_t i = 0; i < n; i++) out[i] = i;
  uint64_t s = seed;
  for (int64_t i = n - 1; i > 0; i--) {
    const uint64_t j = splitmix64(s) % (uint64_t)(i + 1);
    std::swap(out[i], out[j]);
  }
}

// Philox4x32-10
static inline void philox_round(uint32_t c[4], const uint32_t k[2]) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
  const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k[0], n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k[1], n3 = (uint32_t)p0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
static inline void philox4x32_10(uint64_t seed, uint64_t offset, uint64_t subsequence, uint32_t out[4]) {
  uint32_t c[4] = {(uint32_t)offset, (uint32_t)(offset >> 32), (uint32_t)subsequence, (uint32_t)(subsequence >> 32)};
  uint32_t k[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  for (int r = 0; r < 10; r++) {
    philox_round(c, k);
    k[0] += 0x9E3779B9u;
    k[1] += 0xBB67AE85u;
  }
  for (int i = 0; i < 4; i++) out[i] = c[i];
}

// Eight consecutive counters at once with AVX2 (checked at run time): 32 uniforms per call, written in stream order.
#if defined(__x86_64__)
#include <immintrin.h>
__attribute__((target("avx2")))
static inline void mulhilo8(__m256i a, uint32_t m, __m256i& hi, __m256i& lo) {
  const __m256i mm = _mm256_set1_epi32((int)m);
  const __m256i even = _mm256_mul_epu32(a, mm), odd = _mm256_mul_epu32(_mm256_srli_epi64(a, 32), mm);
  hi = _mm256_blend_epi32(_mm256_srli_epi64(even, 32), odd, 0xAA);
  lo = _mm256_blend_epi32(even, _mm256_slli_epi64(odd, 32), 0xAA);
}
__attribute__((target("avx2")))
static void philox_uniform32_avx2(uint64_t seed, uint64_t offset, float* out) {
  alignas(32) uint32_t lo32[8], hi32[8];
  for (int l = 0; l < 8; l++) { const uint64_t o = offset + (uint64_t)l; lo32[l] = (uint32_t)o; hi32[l] = (uint32_t)(o >> 32); }
  __m256i c0 = _mm256_load_si256((const __m256i*)lo32), c1 = _mm256_load_si256((const __m256i*)hi32), c2 = _mm256_setzero_si256(), c3 = c2;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; r++) {
    __m256i h0, l0, h1, l1;
    mulhilo8(c0, 0xD2511F53u, h0, l0);
    mulhilo8(c2, 0xCD9E8D57u, h1, l1);
    const __m256i n0 = _mm256_xor_si256(_mm256_xor_si256(h1, c1), _mm256_set1_epi32((int)k0));
    const __m256i n2 = _mm256_xor_si256(_mm256_xor_si256(h0, c3), _mm256_set1_epi32((int)k1));
    c0 = n0; c1 = l1; c2 = n2; c3 = l0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  // words (c0..c3) x counters (8 lanes) -> stream order out[4 * lane + word]
  const __m256i t0 = _mm256_unpacklo_epi32(c0, c1), t1 = _mm256_unpackhi_epi32(c0, c1), t2 = _mm256_unpacklo_epi32(c2, c3), t3 = _mm256_unpackhi_epi32(c2, c3);
  const __m256i u0 = _mm256_unpacklo_epi64(t0, t2), u1 = _mm256_unpackhi_epi64(t0, t2), u2 = _mm256_unpacklo_epi64(t1, t3), u3 = _mm256_unpackhi_epi64(t1, t3);
  const __m256i v[4] = {_mm256_permute2x128_si256(u0, u1, 0x20), _mm256_permute2x128_si256(u2, u3, 0x20), _mm256_permute2x128_si256(u0, u1, 0x31),
                        _mm256_permute2x128_si256(u2, u3, 0x31)};
  const __m256 half = _mm256_set1_ps(0.5f), scale = _mm256_set1_ps(1.0f / 16777216.0f);
  for (int j = 0; j < 4; j++) {
    const __m256 f = _mm256_mul_ps(_mm256_add_ps(_mm256_cvtepi32_ps(_mm256_srli_epi32(v[j], 8)), half), scale);
    _mm256_storeu_ps(out + 8 * j, f);
  }
}
#endif
static bool have_avx2() {
#if defined(__x86_64__)
  static const bool v = __builtin_cpu_supports("avx2") && std::getenv("FT_NO_AVX2") == nullptr;      // FT_NO_AVX2: force the generic code (tests)
  return v;
#else
  return false;
#endif
}

// Element i of the stream uses counter (offset + i/4, subsequence 0) lane i%4: the layout the device kernels use.
FT_API void ft_philox_uniform(uint64_t seed, uint64_t offset, int64_t n, float* out) {
  int64_t i0 = 0;
#if defined(__x86_64__)
  if (have_avx2())
    for (; i0 + 32 <= n; i0 += 32) philox_uniform32_avx2(seed, offset + (uint64_t)(i0 / 4), out + i0);
#endif
  for (int64_t i = i0; i < n; i += 4) {
    uint32_t r[4];
    philox4x32_10(seed, offset + (uint64_t)(i / 4), 0, r);
    for (int e = 0; e < 4 && i + e < n; e++) out[i + e] = ((r[e] >> 8) + 0.5f) * (1.0f / 16777216.0f);   // (0,1)
  }
}
// Box-Muller on pairs of the uniform stream: z[2p] = r cos(2 pi u[2p+1]), z[2p+1] = r sin(2 pi u[2p+1]) with r = sqrt(-2 ln u[2p]). The logarithm
// and the sine / cosine are branch-free polynomials (Cephes coefficients, 1-2 ulp) written as plain arithmetic and selects, so that the pair
// loop vectorises; the same code runs for every element, whatever the block or thread split, so the values depend only on (seed, offset, index).
static inline __attribute__((always_inline)) float bm_log(float x) {                       // x in (0, 1)
  uint32_t b;
  std::memcpy(&b, &x, 4);
  int32_t e = (int32_t)((b >> 23) & 0xffu) - 126;
  uint32_t mb = (b & 0x807fffffu) | 0x3f000000u;
  float m;
  std::memcpy(&m, &mb, 4);
  const bool lo = m < 0.707106781186547524f;
  e -= lo ? 1 : 0;
  m = lo ? m + m - 1.0f : m - 1.0f;
  const float z = m * m;
  float p = 7.0376836292e-2f;
  p = p * m - 1.1514610310e-1f;
  p = p * m + 1.1676998740e-1f;
  p = p * m - 1.2420140846e-1f;
  p = p * m + 1.4249322787e-1f;
  p = p * m - 1.6668057665e-1f;
  p = p * m + 2.0000714765e-1f;
  p = p * m - 2.4999993993e-1f;
  p = p * m + 3.3333331174e-1f;
  const float fe = (float)e;
  float y = p * m * z;
  y += fe * -2.12194440e-4f;
  y -= 0.5f * z;
  return m + y + fe * 0.693359375f;
}
static inline __attribute__((always_inline)) void bm_sincos_2pi(float u, float& sn, float& cs) {      // u in (0, 1): angle 2 pi u
  const float t = u - 0.5f;                                            // sin(2 pi u) = -sin(2 pi t), cos(2 pi u) = -cos(2 pi t), t in (-1/2, 1/2)
  const float k = __builtin_nearbyintf(4.0f * t);                            // quadrant: -2 .. 2
  const float phi = 6.283185307179586f * (t - 0.25f * k);              // [-pi/4, pi/4]
  const float z = phi * phi;
  const float s0 = phi + phi * z * ((-1.9515295891e-4f * z + 8.3321608736e-3f) * z - 1.6666654611e-1f);
  const float c0 = 1.0f - 0.5f * z + z * z * ((2.443315711809948e-5f * z - 1.388731625493765e-3f) * z + 4.166664568298827e-2f);
  const int q = (int)k & 3;                                            // rotate by k quarter turns: (c, s) -> (c, s), (-s, c), (-c, -s), (s, -c)
  const bool sw = (q & 1) != 0;
  const float a = sw ? c0 : s0, b = sw ? s0 : c0;
  const float s1 = (q & 2) ? -a : a;
  const float c1 = ((q + 1) & 2) ? -b : b;
  sn = -s1;
  cs = -c1;
}
#define FT_BM_PAIRS_BODY                                        \
  for (int p = 0; p < pairs; p++) {                             \
    const float r = __builtin_sqrtf(-2.0f * bm_log(u[2 * p]));  \
    float sn, cs;                                               \
    bm_sincos_2pi(u[2 * p + 1], sn, cs);                        \
    z[2 * p] = r * cs;                                          \
    z[2 * p + 1] = r * sn;                                      \
  }
// the same loop compiled twice (no FMA contraction in either, so both give the same bits); the AVX2 build is picked at run time
static void bm_pairs_generic(const float* __restrict__ u, float* __restrict__ z, int pairs) { FT_BM_PAIRS_BODY }
#if defined(__x86_64__)
__attribute__((target("avx2"))) static void bm_pairs_avx2(const float* __restrict__ u, float* __restrict__ z, int pairs) { FT_BM_PAIRS_BODY }
#endif
static void bm_pairs(const float* u, float* z, int pairs) {
#if defined(__x86_64__)
  if (have_avx2()) { bm_pairs_avx2(u, z, pairs); return; }
#endif
  bm_pairs_generic(u, z, pairs);
}
FT_API void ft_philox_normal(uint64_t seed, uint64_t offset, int64_t n, float* out) {
  constexpr int BLK = 1024;                                  // uniforms per block (a multiple of 32)
  float u[BLK], z[BLK];
  for (int64_t i0 = 0; i0 < n; i0 += BLK) {
    const int64_t len = std::min<int64_t>(BLK, n - i0);
    const int64_t padded = (len + 3) / 4 * 4;
    ft_philox_uniform(seed, offset + (uint64_t)(i0 / 4), padded, u);
    bm_pairs(u, z, (int)(padded / 2));
    std::memcpy(out + i0, z, (size_t)len * sizeof(float));
  }
}

// Threaded fills of large host tensors: the range is cut at multiples of four elements, so the values do not depend on the thread count.
template <typename F>
static void philox_parallel(int64_t n, int nthreads, F body) {
  nthreads = std::max(1, std::min<int>(nthreads, 64));
  if (n < (1 << 16) || nthreads == 1) { body((int64_t)0, n); return; }
  const int64_t per = ((n + nthreads - 1) / nthreads + 3) / 4 * 4;
  std::vector<std::thread> ts;
  for (int t = 0; t < nthreads; t++) {
    const int64_t lo = t * per, hi = std::min<int64_t>(n, lo + per);
    if (lo >= hi) break;
    ts.emplace_back([=] { body(lo, hi); });
  }
  for (auto& t : ts) t.join();
}
FT_API void ft_philox_uniform_mt(uint64_t seed, uint64_t offset, int64_t n, float* out, int nthreads) {
  philox_parallel(n, nthreads, [=](int64_t lo, int64_t hi) { ft_philox_uniform(seed, offset + (uint64_t)(lo / 4), hi - lo, out + lo); });
}
FT_API void ft_philox_normal_mt(uint64_t seed, uint64_t offset, int64_t n, float* out, int nthreads) {
  philox_parallel(n, nthreads, [=](int64_t lo, int64_t hi) { ft_philox_normal(seed, offset + (uint64_t)(lo / 4), hi - lo, out + lo); });
}
