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
  static const bool v = __builtin_cpu_supports("avx2");
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
FT_API void ft_philox_normal(uint64_t seed, uint64_t offset, int64_t n, float* out) {
  for (int64_t i = 0; i < n; i += 4) {
    uint32_t r[4];
    philox4x32_10(seed, offset + (uint64_t)(i / 4), 0, r);
    float u[4];
    for (int e = 0; e < 4; e++) u[e] = ((r[e] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float r0 = std::sqrt(-2.0f * std::log(u[0])), r1 = std::sqrt(-2.0f * std::log(u[2]));
    const float z[4] = {r0 * std::cos(6.283185307179586f * u[1]), r0 * std::sin(6.283185307179586f * u[1]),
                        r1 * std::cos(6.283185307179586f * u[3]), r1 * std::sin(6.283185307179586f * u[3])};
    for (int e = 0; e < 4 && i + e < n; e++) out[i + e] = z[e];
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
