/* Plain-C restatement of one Lloyd iteration of the reference's CPU k-means path.
 *
 * TEST INFRASTRUCTURE, not product code: only tests, the smoke check and the
 * benchmark's CPU-baseline leg may load the library built from this file; the
 * shipped engine never does.
 *
 * The reference's n_gpus=0 path is scikit-learn's dense Lloyd solver
 * (src/interface_py/h2o4gpu/solvers/kmeans.py:738-750, 768-770).  Rules restated
 * (all arithmetic in double, input rows float or double):
 *   E-step   label = argmin_j (|c_j|^2 - 2 x.c_j), first minimum wins
 *            (same tie rule as src/gpu/kmeans/kmeans_labels.h:360-377);
 *   M-step   sums / counts; each empty cluster, lowest id first, takes the
 *            remaining row farthest from its assigned centre (ties: lowest
 *            row), which its donor cluster loses; a cluster still empty
 *            copies the largest cluster's row as it stands at that moment;
 *   output   transform = |xn + cn - 2 x.c| column-major n x k
 *            (src/gpu/kmeans/kmeans_labels.cu:115-244).
 * Pinned against oracle/lloyd.py (itself pinned against scikit-learn) by
 * tests/test_oracle.py.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define DEFINE_ALL(T, SUF)                                                                  \
  void oracle_assign_##SUF(const T* X, size_t n, int d, const double* C, int k,             \
                           int32_t* labels, double* best_sq) {                              \
    double* cn = (double*)malloc(sizeof(double) * (size_t)k);                               \
    for (int j = 0; j < k; ++j) {                                                           \
      double s = 0;                                                                         \
      for (int t = 0; t < d; ++t) s += C[(size_t)j * d + t] * C[(size_t)j * d + t];         \
      cn[j] = s;                                                                            \
    }                                                                                       \
    _Pragma("omp parallel for schedule(static)")                                            \
    for (size_t i = 0; i < n; ++i) {                                                        \
      const T* x = X + i * (size_t)d;                                                       \
      double bestv = INFINITY;                                                              \
      int bestj = 0;                                                                        \
      for (int j = 0; j < k; ++j) {                                                         \
        const double* c = C + (size_t)j * d;                                                \
        double dot = 0;                                                                     \
        for (int t = 0; t < d; ++t) dot += (double)x[t] * c[t];                             \
        double v = cn[j] - 2.0 * dot;                                                       \
        if (v < bestv) { bestv = v; bestj = j; }                                            \
      }                                                                                     \
      labels[i] = bestj;                                                                    \
      if (best_sq) {                                                                        \
        double xn = 0;                                                                      \
        for (int t = 0; t < d; ++t) xn += (double)x[t] * (double)x[t];                      \
        best_sq[i] = xn + bestv;                                                            \
      }                                                                                     \
    }                                                                                       \
    free(cn);                                                                               \
  }                                                                                         \
                                                                                            \
  void oracle_sums_counts_##SUF(const T* X, size_t n, int d, const int32_t* labels, int k,  \
                                double* sums, int64_t* counts) {                            \
    memset(sums, 0, sizeof(double) * (size_t)k * d);                                        \
    memset(counts, 0, sizeof(int64_t) * (size_t)k);                                         \
    for (size_t i = 0; i < n; ++i) {                                                        \
      int j = labels[i];                                                                    \
      counts[j] += 1;                                                                       \
      for (int t = 0; t < d; ++t) sums[(size_t)j * d + t] += (double)X[i * (size_t)d + t];  \
    }                                                                                       \
  }                                                                                         \
                                                                                            \
  /* returns the number of relocated clusters; moved_rows[e] = row given to the e-th */    \
  int oracle_relocate_##SUF(const T* X, size_t n, int d, const int32_t* labels,             \
                            const double* C_old, int k, double* sums, int64_t* counts,      \
                            int64_t* moved_rows) {                                          \
    int n_empty = 0;                                                                        \
    for (int j = 0; j < k; ++j) n_empty += (counts[j] == 0);                                \
    if (!n_empty) return 0;                                                                 \
    double* dist = (double*)malloc(sizeof(double) * n);                                     \
    double dmax = 0;                                                                        \
    for (size_t i = 0; i < n; ++i) {                                                        \
      const double* c = C_old + (size_t)labels[i] * d;                                      \
      double s = 0;                                                                         \
      for (int t = 0; t < d; ++t) {                                                         \
        double q = (double)X[i * (size_t)d + t] - c[t];                                     \
        s += q * q;                                                                         \
      }                                                                                     \
      dist[i] = s;                                                                          \
      if (s > dmax) dmax = s;                                                               \
    }                                                                                       \
    int e = 0;                                                                              \
    if (dmax > 0) {                                                                         \
      int* empties = (int*)malloc(sizeof(int) * (size_t)n_empty);                           \
      for (int j = 0, q = 0; j < k; ++j) if (counts[j] == 0) empties[q++] = j;              \
      for (; e < n_empty; ++e) {                                                            \
        size_t far = 0;                                                                     \
        double fv = -1;                                                                     \
        for (size_t i = 0; i < n; ++i) if (dist[i] > fv) { fv = dist[i]; far = i; }         \
        dist[far] = -2;                                                                     \
        int cid = empties[e], old = labels[far];                                            \
        for (int t = 0; t < d; ++t) {                                                       \
          double xv = (double)X[far * (size_t)d + t];                                       \
          sums[(size_t)old * d + t] -= xv;                                                  \
          sums[(size_t)cid * d + t] = xv;                                                   \
        }                                                                                   \
        counts[cid] = 1;                                                                    \
        counts[old] -= 1;                                                                   \
        if (moved_rows) moved_rows[e] = (int64_t)far;                                       \
      }                                                                                     \
      free(empties);                                                                        \
    }                                                                                       \
    free(dist);                                                                             \
    return e;                                                                               \
  }                                                                                         \
                                                                                            \
  void oracle_transform_##SUF(const T* X, size_t n, int d, const double* C, int k,          \
                              double* out_colmajor) {                                       \
    _Pragma("omp parallel for schedule(static)")                                            \
    for (size_t i = 0; i < n; ++i) {                                                        \
      const T* x = X + i * (size_t)d;                                                       \
      double xn = 0;                                                                        \
      for (int t = 0; t < d; ++t) xn += (double)x[t] * (double)x[t];                        \
      for (int j = 0; j < k; ++j) {                                                         \
        const double* c = C + (size_t)j * d;                                                \
        double dot = 0, cn = 0;                                                             \
        for (int t = 0; t < d; ++t) { dot += (double)x[t] * c[t]; cn += c[t] * c[t]; }      \
        out_colmajor[(size_t)j * n + i] = fabs(xn + cn - 2.0 * dot);                        \
      }                                                                                     \
    }                                                                                       \
  }                                                                                         \
                                                                                            \
  /* one whole iteration: C_old -> C_new, labels; returns relocations done */              \
  int oracle_step_##SUF(const T* X, size_t n, int d, const double* C_old, int k,            \
                        double* C_new, int32_t* labels, int64_t* counts) {                  \
    oracle_assign_##SUF(X, n, d, C_old, k, labels, NULL);                                   \
    oracle_sums_counts_##SUF(X, n, d, labels, k, C_new, counts);                            \
    int moved = oracle_relocate_##SUF(X, n, d, labels, C_old, k, C_new, counts, NULL);      \
    oracle_average(C_new, counts, k, d);                                                    \
    return moved;                                                                           \
  }

void oracle_average(double* sums, const int64_t* counts, int k, int d) {
  int big = 0;
  for (int j = 1; j < k; ++j) if (counts[j] > counts[big]) big = j;
  for (int j = 0; j < k; ++j) {
    if (counts[j] > 0) {
      double a = 1.0 / (double)counts[j];
      for (int t = 0; t < d; ++t) sums[(size_t)j * d + t] *= a;
    } else {
      for (int t = 0; t < d; ++t) sums[(size_t)j * d + t] = sums[(size_t)big * d + t];
    }
  }
}

DEFINE_ALL(float, f32)
DEFINE_ALL(double, f64)
