// Dense factorisations on the host for `ferrotorch_b200.core.linalg`: Cholesky, LU with partial pivoting (and the solves built on it),
// triangular solves, Householder QR, the symmetric eigenproblem by Householder tridiagonalisation + implicit QL iterations (cyclic Jacobi
// rotations as the fallback), the singular value decomposition by one-sided (Hestenes) Jacobi rotations and the general eigenproblem through
// the complex Schur form (Hessenberg reduction + shifted QR). Row-major f64 at the interface
// (the QR, QL and Jacobi loops work on transposed copies so that they run over contiguous memory), batched over a leading dimension with
// the matrices of a batch spread over threads.
// The Python side supplies f64 copies of f32 inputs and the derivative formulas.
//
// Capability parity: ferrotorch-core/src/linalg.rs:121-2170 (svd, solve, det, inv, qr, cholesky, eigh, lu, lstsq, ...), which calls the
// faer library for the same factorisations.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <complex>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define FT_API extern "C" __attribute__((visibility("default")))

namespace {

template <class F>
void for_batch(int64_t batch, int64_t work_per_item, F&& body) {
  int nt = (int)std::min<int64_t>(std::min<int64_t>(batch, (int64_t)std::thread::hardware_concurrency()), 16);
  if (nt <= 1 || batch * work_per_item < (1 << 18)) {
    for (int64_t b = 0; b < batch; b++) body(b);
    return;
  }
  std::atomic<int64_t> next{0};
  std::vector<std::thread> ts;
  for (int t = 0; t < nt; t++)
    ts.emplace_back([&] {
      for (;;) {
        const int64_t b = next.fetch_add(1);
        if (b >= batch) return;
        body(b);
      }
    });
  for (auto& th : ts) th.join();
}

}  // namespace

// a [batch, n, n]: on return the lower Cholesky factor L (A = L L^T; the strict upper part is zeroed). Only the lower triangle of the input
// is read. info[b] = 0, or k (1-based) when the leading minor of order k is not positive definite (the factor of that matrix is unfinished).
FT_API int ft_la_cholesky(double* a, int64_t batch, int64_t n, int32_t* info) {
  for_batch(batch, n * n * n / 3 + 1, [&](int64_t b) {
    double* A = a + b * n * n;
    info[b] = 0;
    for (int64_t j = 0; j < n && info[b] == 0; j++) {
      double d = A[j * n + j];
      for (int64_t k = 0; k < j; k++) d -= A[j * n + k] * A[j * n + k];
      if (!(d > 0.0)) { info[b] = (int32_t)(j + 1); break; }
      d = std::sqrt(d);
      A[j * n + j] = d;
      for (int64_t i = j + 1; i < n; i++) {
        double s = A[i * n + j];
        for (int64_t k = 0; k < j; k++) s -= A[i * n + k] * A[j * n + k];
        A[i * n + j] = s / d;
      }
    }
    for (int64_t i = 0; i < n; i++)
      for (int64_t j = i + 1; j < n; j++) A[i * n + j] = 0.0;
  });
  return 0;
}

// a [batch, m, n]: on return L (unit lower, below the diagonal) and U (on and above it) of P A = L U with partial pivoting.
// piv [batch, min(m, n)]: row k was exchanged with row piv[k] >= k. info[b] = 0, or k (1-based) for the first exactly zero pivot.
FT_API int ft_la_lu(double* a, int64_t batch, int64_t m, int64_t n, int32_t* piv, int32_t* info) {
  const int64_t r = std::min(m, n);
  for_batch(batch, m * n * r / 2 + 1, [&](int64_t b) {
    double* A = a + b * m * n;
    int32_t* P = piv + b * r;
    info[b] = 0;
    for (int64_t k = 0; k < r; k++) {
      int64_t p = k;
      double best = std::fabs(A[k * n + k]);
      for (int64_t i = k + 1; i < m; i++)
        if (std::fabs(A[i * n + k]) > best) { best = std::fabs(A[i * n + k]); p = i; }
      P[k] = (int32_t)p;
      if (p != k)
        for (int64_t j = 0; j < n; j++) std::swap(A[k * n + j], A[p * n + j]);
      const double d = A[k * n + k];
      if (d == 0.0) { if (info[b] == 0) info[b] = (int32_t)(k + 1); continue; }
      for (int64_t i = k + 1; i < m; i++) {
        const double f = A[i * n + k] / d;
        A[i * n + k] = f;
        if (f != 0.0)
          for (int64_t j = k + 1; j < n; j++) A[i * n + j] -= f * A[k * n + j];
      }
    }
  });
  return 0;
}

// Solves A X = B (trans = 0) or A^T X = B (trans = 1) from the factors of ft_la_lu of a square A. lu [batch, n, n], piv [batch, n],
// b [batch, n, k] in place.
FT_API int ft_la_lu_solve(const double* lu, const int32_t* piv, double* bmat, int64_t batch, int64_t n, int64_t k, int trans) {
  for_batch(batch, n * n * k + 1, [&](int64_t b) {
    const double* A = lu + b * n * n;
    const int32_t* P = piv + b * n;
    double* B = bmat + b * n * k;
    if (!trans) {
      for (int64_t i = 0; i < n; i++)
        if (P[i] != i)
          for (int64_t c = 0; c < k; c++) std::swap(B[i * k + c], B[(int64_t)P[i] * k + c]);
      for (int64_t i = 0; i < n; i++)                                   // L y = P b
        for (int64_t j = 0; j < i; j++) {
          const double f = A[i * n + j];
          if (f != 0.0)
            for (int64_t c = 0; c < k; c++) B[i * k + c] -= f * B[j * k + c];
        }
      for (int64_t i = n - 1; i >= 0; i--) {                            // U x = y
        for (int64_t j = i + 1; j < n; j++) {
          const double f = A[i * n + j];
          if (f != 0.0)
            for (int64_t c = 0; c < k; c++) B[i * k + c] -= f * B[j * k + c];
        }
        const double d = A[i * n + i];
        for (int64_t c = 0; c < k; c++) B[i * k + c] /= d;
      }
    } else {
      for (int64_t i = 0; i < n; i++) {                                 // U^T y = b
        for (int64_t j = 0; j < i; j++) {
          const double f = A[j * n + i];
          if (f != 0.0)
            for (int64_t c = 0; c < k; c++) B[i * k + c] -= f * B[j * k + c];
        }
        const double d = A[i * n + i];
        for (int64_t c = 0; c < k; c++) B[i * k + c] /= d;
      }
      for (int64_t i = n - 1; i >= 0; i--)                              // L^T z = y
        for (int64_t j = i + 1; j < n; j++) {
          const double f = A[j * n + i];
          if (f != 0.0)
            for (int64_t c = 0; c < k; c++) B[i * k + c] -= f * B[j * k + c];
        }
      for (int64_t i = n - 1; i >= 0; i--)                              // x = P^T z
        if (P[i] != i)
          for (int64_t c = 0; c < k; c++) std::swap(B[i * k + c], B[(int64_t)P[i] * k + c]);
    }
  });
  return 0;
}

// Solves op(T) X = B for a triangular T [batch, n, n] (upper or lower, op = identity or transpose, unit diagonal or not); b [batch, n, k]
// in place. Only the named triangle of T is read.
FT_API int ft_la_trsm(const double* t, double* bmat, int64_t batch, int64_t n, int64_t k, int upper, int trans, int unit) {
  for_batch(batch, n * n * k / 2 + 1, [&](int64_t b) {
    const double* T = t + b * n * n;
    double* B = bmat + b * n * k;
    auto at = [&](int64_t i, int64_t j) { return trans ? T[j * n + i] : T[i * n + j]; };
    const bool eff_upper = (upper != 0) != (trans != 0);
    if (eff_upper) {
      for (int64_t i = n - 1; i >= 0; i--) {
        for (int64_t j = i + 1; j < n; j++) {
          const double f = at(i, j);
          if (f != 0.0)
            for (int64_t c = 0; c < k; c++) B[i * k + c] -= f * B[j * k + c];
        }
        if (!unit) { const double d = at(i, i); for (int64_t c = 0; c < k; c++) B[i * k + c] /= d; }
      }
    } else {
      for (int64_t i = 0; i < n; i++) {
        for (int64_t j = 0; j < i; j++) {
          const double f = at(i, j);
          if (f != 0.0)
            for (int64_t c = 0; c < k; c++) B[i * k + c] -= f * B[j * k + c];
        }
        if (!unit) { const double d = at(i, i); for (int64_t c = 0; c < k; c++) B[i * k + c] /= d; }
      }
    }
  });
  return 0;
}

// Householder QR of a [batch, m, n]: q [batch, m, kq] with orthonormal columns and r [batch, kq, n] upper triangular, kq = min(m, n)
// (complete = 0) or m (complete = 1).
FT_API int ft_la_qr(const double* a, double* q, double* r, int64_t batch, int64_t m, int64_t n, int complete) {
  const int64_t kq = complete ? m : std::min(m, n), steps = std::min(m, n);
  for_batch(batch, m * n * std::min(m, n) * 2 + 1, [&](int64_t b) {
    // Rt[j] is column j of the working matrix, Qt[i] is row i of Q: every inner loop below runs over contiguous memory
    std::vector<double> Rt((size_t)(n * m)), Qt((size_t)(m * m), 0.0), v((size_t)m);
    for (int64_t i = 0; i < m; i++)
      for (int64_t j = 0; j < n; j++) Rt[(size_t)(j * m + i)] = a[b * m * n + i * n + j];
    for (int64_t i = 0; i < m; i++) Qt[(size_t)(i * m + i)] = 1.0;
    for (int64_t k = 0; k < steps; k++) {
      double* ck = &Rt[(size_t)(k * m)];
      double norm = 0.0;
      for (int64_t i = k; i < m; i++) norm += ck[i] * ck[i];
      norm = std::sqrt(norm);
      if (norm == 0.0) continue;
      const double alpha = ck[k] > 0 ? -norm : norm;
      double vnorm2 = 0.0;
      for (int64_t i = k; i < m; i++) {
        v[(size_t)i] = ck[i] - (i == k ? alpha : 0.0);
        vnorm2 += v[(size_t)i] * v[(size_t)i];
      }
      if (vnorm2 == 0.0) continue;
      for (int64_t j = k; j < n; j++) {                                 // R <- (I - 2 v v^T / v^T v) R, column by column
        double* cj = &Rt[(size_t)(j * m)];
        double sdot = 0.0;
        for (int64_t i = k; i < m; i++) sdot += v[(size_t)i] * cj[i];
        sdot = 2.0 * sdot / vnorm2;
        for (int64_t i = k; i < m; i++) cj[i] -= sdot * v[(size_t)i];
      }
      for (int64_t i = 0; i < m; i++) {                                 // Q <- Q (I - 2 v v^T / v^T v), row by row
        double* qi = &Qt[(size_t)(i * m)];
        double sdot = 0.0;
        for (int64_t j = k; j < m; j++) sdot += qi[j] * v[(size_t)j];
        sdot = 2.0 * sdot / vnorm2;
        for (int64_t j = k; j < m; j++) qi[j] -= sdot * v[(size_t)j];
      }
    }
    double* Qo = q + b * m * kq;
    double* Ro = r + b * kq * n;
    for (int64_t i = 0; i < m; i++)
      for (int64_t j = 0; j < kq; j++) Qo[i * kq + j] = Qt[(size_t)(i * m + j)];
    for (int64_t i = 0; i < kq; i++)
      for (int64_t j = 0; j < n; j++) Ro[i * n + j] = j >= i ? Rt[(size_t)(j * m + i)] : 0.0;
  });
  return 0;
}

namespace {

inline double hyp(double x, double y) { return std::hypot(x, y); }

// Householder reduction of the symmetric matrix A (row-major n x n, full storage) to tridiagonal form: on return A holds the orthogonal
// matrix of the reduction, d the diagonal and e the sub-diagonal (e[0] = 0).
void tridiagonalise(double* A, int64_t n, double* d, double* e) {
  for (int64_t i = n - 1; i >= 1; i--) {
    const int64_t l = i - 1;
    double h = 0.0, scale = 0.0;
    if (l > 0) {
      for (int64_t k = 0; k <= l; k++) scale += std::fabs(A[i * n + k]);
      if (scale == 0.0) {
        e[i] = A[i * n + l];
      } else {
        for (int64_t k = 0; k <= l; k++) { A[i * n + k] /= scale; h += A[i * n + k] * A[i * n + k]; }
        double f = A[i * n + l];
        double g = f >= 0.0 ? -std::sqrt(h) : std::sqrt(h);
        e[i] = scale * g;
        h -= f * g;
        A[i * n + l] = f - g;
        f = 0.0;
        for (int64_t j = 0; j <= l; j++) {
          A[j * n + i] = A[i * n + j] / h;
          g = 0.0;
          for (int64_t k = 0; k <= j; k++) g += A[j * n + k] * A[i * n + k];
          for (int64_t k = j + 1; k <= l; k++) g += A[k * n + j] * A[i * n + k];
          e[j] = g / h;
          f += e[j] * A[i * n + j];
        }
        const double hh = f / (h + h);
        for (int64_t j = 0; j <= l; j++) {
          f = A[i * n + j];
          e[j] = g = e[j] - hh * f;
          for (int64_t k = 0; k <= j; k++) A[j * n + k] -= f * e[k] + g * A[i * n + k];
        }
      }
    } else {
      e[i] = A[i * n + l];
    }
    d[i] = h;
  }
  d[0] = 0.0;
  e[0] = 0.0;
  for (int64_t i = 0; i < n; i++) {
    const int64_t l = i - 1;
    if (d[i] != 0.0) {
      for (int64_t j = 0; j <= l; j++) {
        double g = 0.0;
        for (int64_t k = 0; k <= l; k++) g += A[i * n + k] * A[k * n + j];
        for (int64_t k = 0; k <= l; k++) A[k * n + j] -= g * A[k * n + i];
      }
    }
    d[i] = A[i * n + i];
    A[i * n + i] = 1.0;
    for (int64_t j = 0; j <= l; j++) A[j * n + i] = A[i * n + j] = 0.0;
  }
}

// Implicit QL iterations on the tridiagonal matrix (d, e as left by tridiagonalise). Zt holds the accumulated transformation TRANSPOSED
// (row j = vector j), so every rotation touches two contiguous rows. False if an eigenvalue needs more than 80 iterations.
bool ql_implicit(double* d, double* e, int64_t n, double* Zt) {
  for (int64_t i = 1; i < n; i++) e[i - 1] = e[i];
  e[n - 1] = 0.0;
  for (int64_t l = 0; l < n; l++) {
    int iter = 0;
    int64_t m;
    do {
      for (m = l; m < n - 1; m++) {
        const double dd = std::fabs(d[m]) + std::fabs(d[m + 1]);
        if (std::fabs(e[m]) <= 2.3e-16 * dd) break;
      }
      if (m != l) {
        if (iter++ == 80) return false;
        double g = (d[l + 1] - d[l]) / (2.0 * e[l]);
        double r = hyp(g, 1.0);
        g = d[m] - d[l] + e[l] / (g + (g >= 0.0 ? std::fabs(r) : -std::fabs(r)));
        double s = 1.0, c = 1.0, p = 0.0;
        int64_t i;
        for (i = m - 1; i >= l; i--) {
          double f = s * e[i];
          const double bb = c * e[i];
          e[i + 1] = (r = hyp(f, g));
          if (r == 0.0) {
            d[i + 1] -= p;
            e[m] = 0.0;
            break;
          }
          s = f / r;
          c = g / r;
          g = d[i + 1] - p;
          r = (d[i] - g) * s + 2.0 * c * bb;
          d[i + 1] = g + (p = s * r);
          g = c * r - bb;
          double* z0 = Zt + i * n;
          double* z1 = Zt + (i + 1) * n;
          for (int64_t k = 0; k < n; k++) {
            f = z1[k];
            z1[k] = s * z0[k] + c * f;
            z0[k] = c * z0[k] - s * f;
          }
        }
        if (r == 0.0 && i >= l) continue;
        d[l] -= p;
        e[l] = g;
        e[m] = 0.0;
      }
    } while (m != l);
  }
  return true;
}

}  // namespace

// Symmetric eigenproblem: Householder tridiagonalisation and implicit QL iterations; a matrix on which those do not converge is redone by
// cyclic Jacobi rotations. a [batch, n, n] (one triangle is read: the lower one if `lower`); w [batch, n] ascending eigenvalues,
// v [batch, n, n] with the eigenvectors in its columns. Returns a positive number, or a negative one if some matrix did not converge.
FT_API int ft_la_eigh(const double* a, double* w, double* v, int64_t batch, int64_t n, int lower) {
  std::atomic<int> worst{0};
  for_batch(batch, n * n * n * 8 + 1, [&](int64_t b) {
    std::vector<double> A((size_t)(n * n));
    for (int64_t i = 0; i < n; i++)
      for (int64_t j = 0; j < n; j++) {
        const int64_t lo = std::max(i, j), hi = std::min(i, j);
        A[(size_t)(i * n + j)] = lower ? a[b * n * n + lo * n + hi] : a[b * n * n + hi * n + lo];
      }
    double* V = v + b * n * n;
    if (n >= 3) {
      std::vector<double> T(A), d((size_t)n), e((size_t)n), Zt((size_t)(n * n));
      tridiagonalise(T.data(), n, d.data(), e.data());
      for (int64_t i = 0; i < n; i++)
        for (int64_t j = 0; j < n; j++) Zt[(size_t)(j * n + i)] = T[(size_t)(i * n + j)];
      if (ql_implicit(d.data(), e.data(), n, Zt.data())) {
        std::vector<int64_t> ord((size_t)n);
        for (int64_t i = 0; i < n; i++) ord[(size_t)i] = i;
        std::sort(ord.begin(), ord.end(), [&](int64_t x, int64_t y) { return d[(size_t)x] < d[(size_t)y]; });
        for (int64_t j = 0; j < n; j++) {
          w[b * n + j] = d[(size_t)ord[(size_t)j]];
          const double* zj = &Zt[(size_t)(ord[(size_t)j] * n)];
          for (int64_t k = 0; k < n; k++) V[k * n + j] = zj[k];
        }
        int cur = worst.load();
        while (cur >= 0 && cur < 1 && !worst.compare_exchange_weak(cur, 1)) {}
        return;
      }
    }
    for (int64_t i = 0; i < n * n; i++) V[i] = 0.0;
    for (int64_t i = 0; i < n; i++) V[i * n + i] = 1.0;
    int sweep = 1;
    bool done = n < 2;
    for (; sweep < 60 && !done; sweep++) {
      double off = 0.0, diag = 0.0;
      for (int64_t i = 0; i < n; i++) {
        diag += A[(size_t)(i * n + i)] * A[(size_t)(i * n + i)];
        for (int64_t j = i + 1; j < n; j++) off += A[(size_t)(i * n + j)] * A[(size_t)(i * n + j)];
      }
      if (off <= 1e-32 * (diag + off) || off == 0.0) { done = true; break; }
      for (int64_t p = 0; p < n - 1; p++)
        for (int64_t q = p + 1; q < n; q++) {
          const double apq = A[(size_t)(p * n + q)];
          if (apq == 0.0) continue;
          const double app = A[(size_t)(p * n + p)], aqq = A[(size_t)(q * n + q)];
          const double theta = (aqq - app) / (2.0 * apq);
          const double t = (theta >= 0 ? 1.0 : -1.0) / (std::fabs(theta) + std::sqrt(theta * theta + 1.0));
          const double c = 1.0 / std::sqrt(t * t + 1.0), s = t * c;
          for (int64_t k = 0; k < n; k++) {                             // columns p, q
            const double akp = A[(size_t)(k * n + p)], akq = A[(size_t)(k * n + q)];
            A[(size_t)(k * n + p)] = c * akp - s * akq;
            A[(size_t)(k * n + q)] = s * akp + c * akq;
          }
          for (int64_t k = 0; k < n; k++) {                             // rows p, q
            const double apk = A[(size_t)(p * n + k)], aqk = A[(size_t)(q * n + k)];
            A[(size_t)(p * n + k)] = c * apk - s * aqk;
            A[(size_t)(q * n + k)] = s * apk + c * aqk;
          }
          for (int64_t k = 0; k < n; k++) {
            const double vkp = V[k * n + p], vkq = V[k * n + q];
            V[k * n + p] = c * vkp - s * vkq;
            V[k * n + q] = s * vkp + c * vkq;
          }
        }
    }
    std::vector<int64_t> order((size_t)n);
    for (int64_t i = 0; i < n; i++) order[(size_t)i] = i;
    std::sort(order.begin(), order.end(), [&](int64_t x, int64_t y) { return A[(size_t)(x * n + x)] < A[(size_t)(y * n + y)]; });
    std::vector<double> Vs(V, V + n * n);
    for (int64_t j = 0; j < n; j++) {
      const int64_t src = order[(size_t)j];
      w[b * n + j] = A[(size_t)(src * n + src)];
      for (int64_t k = 0; k < n; k++) V[k * n + j] = Vs[(size_t)(k * n + src)];
    }
    int cur = worst.load();
    const int mine = done ? sweep : -1;
    while ((mine < 0 ? cur >= 0 : (cur >= 0 && mine > cur)) && !worst.compare_exchange_weak(cur, mine)) {}
  });
  return worst.load();
}

// Singular value decomposition by one-sided Jacobi rotations. a [batch, m, n]; u [batch, m, k], s [batch, k] descending, vt [batch, k, n],
// k = min(m, n) (the reduced form). Returns the largest number of sweeps taken (negative: not converged).
FT_API int ft_la_svd(const double* a, double* u, double* s, double* vt, int64_t batch, int64_t m, int64_t n) {
  const int64_t k = std::min(m, n);
  std::atomic<int> worst{0};
  for_batch(batch, m * n * k * 8 + 1, [&](int64_t b) {
    // work on G = A (m >= n) or A^T (m < n): rows >= cols, columns are orthogonalised
    const bool tr = m < n;
    const int64_t rows = tr ? n : m, cols = tr ? m : n;
    // Gt[j] is column j of G, Wt[j] column j of W: the rotations and dot products below run over contiguous memory
    std::vector<double> Gt((size_t)(rows * cols)), Wt((size_t)(cols * cols), 0.0);
    for (int64_t i = 0; i < rows; i++)
      for (int64_t j = 0; j < cols; j++) Gt[(size_t)(j * rows + i)] = tr ? a[b * m * n + j * n + i] : a[b * m * n + i * n + j];
    for (int64_t i = 0; i < cols; i++) Wt[(size_t)(i * cols + i)] = 1.0;
    std::vector<double> nrm((size_t)cols);
    int sweep = 1;
    bool done = cols < 2;
    for (; sweep < 60 && !done; sweep++) {
      bool rotated = false;
      for (int64_t j = 0; j < cols; j++) {
        const double* gj = &Gt[(size_t)(j * rows)];
        double t = 0.0;
        for (int64_t i = 0; i < rows; i++) t += gj[i] * gj[i];
        nrm[(size_t)j] = t;
      }
      for (int64_t p = 0; p < cols - 1; p++)
        for (int64_t q = p + 1; q < cols; q++) {
          double* gp = &Gt[(size_t)(p * rows)];
          double* gq = &Gt[(size_t)(q * rows)];
          double gamma = 0.0;
          for (int64_t i = 0; i < rows; i++) gamma += gp[i] * gq[i];
          const double alpha = nrm[(size_t)p], beta = nrm[(size_t)q];
          if (gamma == 0.0 || std::fabs(gamma) <= 1e-15 * std::sqrt(alpha * beta)) continue;
          rotated = true;
          const double zeta = (beta - alpha) / (2.0 * gamma);
          const double t = (zeta >= 0 ? 1.0 : -1.0) / (std::fabs(zeta) + std::sqrt(1.0 + zeta * zeta));
          const double c = 1.0 / std::sqrt(1.0 + t * t), sn = c * t;
          for (int64_t i = 0; i < rows; i++) {
            const double x = gp[i], y = gq[i];
            gp[i] = c * x - sn * y;
            gq[i] = sn * x + c * y;
          }
          nrm[(size_t)p] = alpha - t * gamma;
          nrm[(size_t)q] = beta + t * gamma;
          double* wp = &Wt[(size_t)(p * cols)];
          double* wq = &Wt[(size_t)(q * cols)];
          for (int64_t i = 0; i < cols; i++) {
            const double x = wp[i], y = wq[i];
            wp[i] = c * x - sn * y;
            wq[i] = sn * x + c * y;
          }
        }
      if (!rotated) done = true;
    }
    auto G = [&](int64_t i, int64_t j) -> double& { return Gt[(size_t)(j * rows + i)]; };
    auto W = [&](int64_t i, int64_t j) -> double& { return Wt[(size_t)(j * cols + i)]; };
    std::vector<double> sv((size_t)cols);
    for (int64_t j = 0; j < cols; j++) {
      double nn = 0.0;
      for (int64_t i = 0; i < rows; i++) nn += G(i, j) * G(i, j);
      sv[(size_t)j] = std::sqrt(nn);
    }
    std::vector<int64_t> order((size_t)cols);
    for (int64_t i = 0; i < cols; i++) order[(size_t)i] = i;
    std::sort(order.begin(), order.end(), [&](int64_t x, int64_t y) { return sv[(size_t)x] > sv[(size_t)y]; });
    // left factor of G: normalised columns (a zero singular value gets a unit vector orthogonal to the others by Gram-Schmidt)
    std::vector<double> L((size_t)(rows * cols), 0.0);
    for (int64_t jj = 0; jj < cols; jj++) {
      const int64_t j = order[(size_t)jj];
      const double sj = sv[(size_t)j];
      s[b * k + jj] = sj;
      if (sj > 0.0) {
        for (int64_t i = 0; i < rows; i++) L[(size_t)(i * cols + jj)] = G(i, j) / sj;
      }
    }
    for (int64_t jj = 0; jj < cols; jj++) {
      if (s[b * k + jj] > 0.0) continue;
      for (int64_t e = 0; e < rows; e++) {                              // try unit vectors until one survives the projection
        std::vector<double> cand((size_t)rows, 0.0);
        cand[(size_t)e] = 1.0;
        for (int64_t c2 = 0; c2 < cols; c2++) {
          if (c2 == jj) continue;
          double dot = 0.0;
          for (int64_t i = 0; i < rows; i++) dot += cand[(size_t)i] * L[(size_t)(i * cols + c2)];
          for (int64_t i = 0; i < rows; i++) cand[(size_t)i] -= dot * L[(size_t)(i * cols + c2)];
        }
        double nn = 0.0;
        for (int64_t i = 0; i < rows; i++) nn += cand[(size_t)i] * cand[(size_t)i];
        if (nn > 1e-8) {
          nn = std::sqrt(nn);
          for (int64_t i = 0; i < rows; i++) L[(size_t)(i * cols + jj)] = cand[(size_t)i] / nn;
          break;
        }
      }
    }
    // G = L S W^T. Not transposed: A = U S V^T with U = L (m x k), V = W. Transposed: A^T = L S W^T so A = W S L^T: U = W, V = L.
    double* U = u + b * m * k;
    double* VT = vt + b * k * n;
    for (int64_t jj = 0; jj < cols; jj++) {
      const int64_t j = order[(size_t)jj];
      if (!tr) {
        for (int64_t i = 0; i < m; i++) U[i * k + jj] = L[(size_t)(i * cols + jj)];
        for (int64_t i = 0; i < n; i++) VT[jj * n + i] = W(i, j);
      } else {
        for (int64_t i = 0; i < m; i++) U[i * k + jj] = W(i, j);
        for (int64_t i = 0; i < n; i++) VT[jj * n + i] = L[(size_t)(i * cols + jj)];
      }
    }
    int cur = worst.load();
    const int mine = done ? sweep : -1;
    while ((mine < 0 ? cur >= 0 : (cur >= 0 && mine > cur)) && !worst.compare_exchange_weak(cur, mine)) {}
  });
  return worst.load();
}

// General (non-symmetric) eigenproblem in complex arithmetic: Householder reduction to Hessenberg form, shifted QR iterations with Givens
// rotations (Wilkinson shift, an exceptional shift every tenth iteration) down to the complex Schur form T = Q^H A Q, eigenvalues from the
// diagonal of T, eigenvectors by back-substitution on T and multiplication by Q, each scaled to unit length with its largest component
// real and positive. a [batch, n, n] real; w [batch, n, 2] (real, imaginary); v [batch, n, n, 2] with the eigenvectors in the columns.
// Returns 1, or -1 if the iterations of some matrix did not converge.
FT_API int ft_la_eig(const double* a, double* w, double* v, int64_t batch, int64_t n) {
  using cd = std::complex<double>;
  std::atomic<int> status{1};
  for_batch(batch, n * n * n * 30 + 1, [&](int64_t b) {
    std::vector<cd> H((size_t)(n * n)), Z((size_t)(n * n), cd(0.0)), u((size_t)n);
    double norm = 0.0;
    for (int64_t i = 0; i < n * n; i++) { H[(size_t)i] = a[b * n * n + i]; norm = std::max(norm, std::fabs(a[b * n * n + i])); }
    for (int64_t i = 0; i < n; i++) Z[(size_t)(i * n + i)] = 1.0;      // Z is kept transposed (row j = column j of the accumulated
    if (norm == 0.0) norm = 1.0;                                        // transformation), so a rotation of two columns touches two contiguous rows
    for (int64_t k = 0; k + 2 < n; k++) {                               // Hessenberg: zero column k below the sub-diagonal
      double xn = 0.0;
      for (int64_t i = k + 1; i < n; i++) xn += std::norm(H[(size_t)(i * n + k)]);
      xn = std::sqrt(xn);
      if (xn == 0.0) continue;
      const cd x0 = H[(size_t)((k + 1) * n + k)];
      const cd alpha = (std::abs(x0) == 0.0 ? cd(1.0) : x0 / std::abs(x0)) * (-xn);
      double un = 0.0;
      for (int64_t i = k + 1; i < n; i++) { u[(size_t)i] = H[(size_t)(i * n + k)] - (i == k + 1 ? alpha : cd(0.0)); un += std::norm(u[(size_t)i]); }
      if (un == 0.0) continue;
      for (int64_t j = 0; j < n; j++) {                                 // H <- (I - 2 u u^H / u^H u) H
        cd s = 0.0;
        for (int64_t i = k + 1; i < n; i++) s += std::conj(u[(size_t)i]) * H[(size_t)(i * n + j)];
        s *= 2.0 / un;
        for (int64_t i = k + 1; i < n; i++) H[(size_t)(i * n + j)] -= s * u[(size_t)i];
      }
      for (int64_t i = 0; i < n; i++) {                                 // H <- H (I - 2 u u^H / u^H u), and the same on Z
        cd s = 0.0, sz = 0.0;
        for (int64_t j = k + 1; j < n; j++) { s += H[(size_t)(i * n + j)] * u[(size_t)j]; sz += Z[(size_t)(j * n + i)] * u[(size_t)j]; }
        s *= 2.0 / un;
        sz *= 2.0 / un;
        for (int64_t j = k + 1; j < n; j++) { H[(size_t)(i * n + j)] -= s * std::conj(u[(size_t)j]); Z[(size_t)(j * n + i)] -= sz * std::conj(u[(size_t)j]); }
      }
    }
    std::vector<cd> gc((size_t)n), gs((size_t)n);
    int64_t hi = n - 1;
    int iter = 0;
    bool ok = true;
    while (hi > 0) {
      int64_t l = hi;
      while (l > 0) {
        double s = std::abs(H[(size_t)((l - 1) * n + l - 1)]) + std::abs(H[(size_t)(l * n + l)]);
        if (s == 0.0) s = norm;
        if (std::abs(H[(size_t)(l * n + l - 1)]) < 2.3e-16 * s) { H[(size_t)(l * n + l - 1)] = 0.0; break; }
        l--;
      }
      if (l == hi) { hi--; iter = 0; continue; }
      if (++iter > 300) { ok = false; break; }
      const cd pa = H[(size_t)((hi - 1) * n + hi - 1)], pb = H[(size_t)((hi - 1) * n + hi)], pc = H[(size_t)(hi * n + hi - 1)], pd = H[(size_t)(hi * n + hi)];
      const cd tr = pa + pd, disc = std::sqrt(tr * tr * 0.25 - (pa * pd - pb * pc));
      const cd m1 = tr * 0.5 + disc, m2 = tr * 0.5 - disc;
      cd mu = std::abs(m1 - pd) < std::abs(m2 - pd) ? m1 : m2;
      if (iter % 10 == 0) mu = pd + cd(std::abs(pc) + (hi >= 2 ? std::abs(H[(size_t)((hi - 1) * n + hi - 2)]) : 0.0), 0.0);
      for (int64_t k = l; k <= hi; k++) H[(size_t)(k * n + k)] -= mu;
      for (int64_t k = l; k < hi; k++) {                                // rotations from the left make the active block upper triangular
        const cd x = H[(size_t)(k * n + k)], y = H[(size_t)((k + 1) * n + k)];
        const double r = std::sqrt(std::norm(x) + std::norm(y));
        cd c = 1.0, s = 0.0;
        if (r != 0.0) { c = x / r; s = y / r; }
        gc[(size_t)k] = c;
        gs[(size_t)k] = s;
        for (int64_t j = k; j < n; j++) {
          const cd t0 = H[(size_t)(k * n + j)], t1 = H[(size_t)((k + 1) * n + j)];
          H[(size_t)(k * n + j)] = std::conj(c) * t0 + std::conj(s) * t1;
          H[(size_t)((k + 1) * n + j)] = -s * t0 + c * t1;
        }
      }
      for (int64_t k = l; k < hi; k++) {                                // the same rotations from the right restore the Hessenberg form
        const cd c = gc[(size_t)k], s = gs[(size_t)k];
        const int64_t top = std::min<int64_t>(k + 2, hi);
        for (int64_t i = 0; i <= top; i++) {
          const cd t0 = H[(size_t)(i * n + k)], t1 = H[(size_t)(i * n + k + 1)];
          H[(size_t)(i * n + k)] = t0 * c + t1 * s;
          H[(size_t)(i * n + k + 1)] = -t0 * std::conj(s) + t1 * std::conj(c);
        }
        cd* z0 = &Z[(size_t)(k * n)];
        cd* z1 = &Z[(size_t)((k + 1) * n)];
        for (int64_t i = 0; i < n; i++) {
          const cd t0 = z0[i], t1 = z1[i];
          z0[i] = t0 * c + t1 * s;
          z1[i] = -t0 * std::conj(s) + t1 * std::conj(c);
        }
      }
      for (int64_t k = l; k <= hi; k++) H[(size_t)(k * n + k)] += mu;
    }
    if (!ok) { status.store(-1); return; }
    std::vector<cd> y((size_t)n);
    for (int64_t k = 0; k < n; k++) {
      const cd lam = H[(size_t)(k * n + k)];
      w[(b * n + k) * 2] = lam.real();
      w[(b * n + k) * 2 + 1] = lam.imag();
      y[(size_t)k] = 1.0;
      for (int64_t i = k - 1; i >= 0; i--) {                            // (T - lambda I) y = 0 on the leading block
        cd s = 0.0;
        for (int64_t j = i + 1; j <= k; j++) s += H[(size_t)(i * n + j)] * y[(size_t)j];
        cd d = H[(size_t)(i * n + i)] - lam;
        if (std::abs(d) < 2.3e-16 * norm) d = 2.3e-16 * norm;
        y[(size_t)i] = -s / d;
      }
      double vn = 0.0, biggest = -1.0;
      cd phase = 1.0;
      for (int64_t i = 0; i < n; i++) {
        cd s = 0.0;
        for (int64_t j = 0; j <= k; j++) s += Z[(size_t)(j * n + i)] * y[(size_t)j];
        u[(size_t)i] = s;
        vn += std::norm(s);
        if (std::abs(s) > biggest) { biggest = std::abs(s); phase = s; }
      }
      vn = std::sqrt(vn);
      const cd scale = (vn == 0.0 || biggest <= 0.0) ? cd(1.0) : std::conj(phase) / (std::abs(phase) * vn);
      for (int64_t i = 0; i < n; i++) {
        const cd e = u[(size_t)i] * scale;
        v[((b * n + i) * n + k) * 2] = e.real();
        v[((b * n + i) * n + k) * 2 + 1] = e.imag();
      }
    }
  });
  return status.load();
}
