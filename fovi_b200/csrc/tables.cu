// Host-side construction of a KNN layer's tables with a reproducible rule for ties: the K nearest input points of
// every output point, and the tap of the filter's reference frame each neighbour is assigned to.
//
// The reference builds both with float32 library calls whose results depend on the BLAS underneath
// (fovi/arch/knn.py:101-152: cdist in its matrix-multiply form + topk; :599-647: arctan2/cos/sin, cdist, argmin).
// Rings of a foveated sensor are symmetric, so exact and near ties are the rule, and the reference's tables change
// with the machine.  Here every quantity is computed in double precision from the float32 coordinates with
// +, -, *, / and sqrt only (all correctly rounded, no fused multiply-add, fixed order), and ties go to the lower index:
// the same inputs give the same tables everywhere.  Runs on host threads; no device is needed.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <thread>
#include <vector>

#include "../../include/fovi_b200.h"

namespace {

// Squared distance in double, products and sums rounded separately.
inline double sqdist(const float* a, const float* b, int dim) {
  volatile double acc = 0.0;   // volatile: keeps the compiler from contracting the multiply and the add
  for (int d = 0; d < dim; ++d) {
    const double diff = (double)a[d] - (double)b[d];
    volatile double sq = diff * diff;
    acc = acc + sq;
  }
  return acc;
}

template <typename F>
void parallel_for(int n, F&& body) {
  const int hw = (int)std::thread::hardware_concurrency();
  const int threads = std::max(1, std::min(n, std::min(hw > 0 ? hw : 1, 64)));
  if (threads == 1) {
    for (int i = 0; i < n; ++i) body(i);
    return;
  }
  std::atomic<int> next(0);
  std::vector<std::thread> pool;
  pool.reserve(threads);
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&]() {
      for (int i = next.fetch_add(1); i < n; i = next.fetch_add(1)) body(i);
    });
  for (auto& th : pool) th.join();
}

// Nearest node of `side` equally spaced nodes on [-1,1] (node i = -1 + 2i/(side-1)); a tie goes to the lower node.
inline int nearest_node(double x, int side) {
  if (side <= 1) return 0;
  int best = 0;
  double bd = INFINITY;
  for (int i = 0; i < side; ++i) {
    const double node = -1.0 + 2.0 * (double)i / (double)(side - 1);
    const double d = std::fabs(x - node);
    if (d < bd) { bd = d; best = i; }
  }
  return best;
}

}  // namespace

extern "C" int fovi_knn_table_build(const float* pts, int n_pts, int dim, const float* targets, int n_out, int K, int32_t* idx_out,
                                    float* dist_out) {
  if (!pts || !targets || !idx_out || n_pts <= 0 || n_out < 0 || dim <= 0 || dim > 8 || K <= 0 || K > n_pts)
    return FOVI_ERR_INVALID_ARGUMENT;
  try {
    parallel_for(n_out, [&](int n) {
      std::vector<std::pair<double, int32_t>> key((size_t)n_pts);
      for (int m = 0; m < n_pts; ++m) key[m] = {sqdist(pts + (size_t)m * dim, targets + (size_t)n * dim, dim), (int32_t)m};
      // (distance, index) lexicographic: std::pair's operator<
      std::partial_sort(key.begin(), key.begin() + K, key.end());
      for (int k = 0; k < K; ++k) {
        idx_out[(size_t)k * n_out + n] = key[k].second;
        if (dist_out) dist_out[(size_t)k * n_out + n] = (float)std::sqrt(key[k].first);
      }
    });
  } catch (...) {
    return FOVI_ERR_INVALID_ARGUMENT;
  }
  return FOVI_OK;
}

extern "C" int fovi_tap_table_build(const int32_t* knn_idx, int K, int n_out, const float* pts, int n_pts, int dim, const float* pts_cart,
                                    const float* out_pts, const float* out_cart, int side, int sample_cortex, uint16_t* tap_out,
                                    float* nb_out) {
  if (!knn_idx || !pts || !tap_out || K <= 0 || n_out < 0 || n_pts <= 0 || dim <= 0 || dim > 8 || side <= 0 || side > 255)
    return FOVI_ERR_INVALID_ARGUMENT;
  if (sample_cortex && (!pts_cart || !out_pts || !out_cart)) return FOVI_ERR_INVALID_ARGUMENT;
  if (!sample_cortex && dim != 2) return FOVI_ERR_INVALID_ARGUMENT;
  for (size_t i = 0; i < (size_t)K * n_out; ++i)
    if (knn_idx[i] < 0 || knn_idx[i] >= n_pts) return FOVI_ERR_TABLE_RANGE;
  try {
    parallel_for(n_out, [&](int n) {
      std::vector<double> x((size_t)K), y((size_t)K);
      for (int k = 0; k < K; ++k) {
        const int m = knn_idx[(size_t)k * n_out + n];
        if (sample_cortex) {
          // polar frame: length = distance on the manifold, direction = direction in the visual field.
          // (r cos(atan2(dy,dx)), r sin(atan2(dy,dx))) = (r dx/h, r dy/h), h = |(dx,dy)|; atan2(0,0) = 0 gives (r, 0).
          const double r = std::sqrt(sqdist(pts + (size_t)m * dim, out_pts + (size_t)n * dim, dim));
          const double dx = (double)pts_cart[(size_t)m * 2] - (double)out_cart[(size_t)n * 2];
          const double dy = (double)pts_cart[(size_t)m * 2 + 1] - (double)out_cart[(size_t)n * 2 + 1];
          volatile double dx2 = dx * dx, dy2 = dy * dy;
          const double h = std::sqrt(dx2 + dy2);
          x[k] = h > 0.0 ? r * dx / h : r;
          y[k] = h > 0.0 ? r * dy / h : 0.0;
        } else {
          x[k] = (double)pts[(size_t)m * 2];
          y[k] = (double)pts[(size_t)m * 2 + 1];
        }
      }
      double xlo = x[0], xhi = x[0], ylo = y[0], yhi = y[0];
      for (int k = 1; k < K; ++k) {
        xlo = std::min(xlo, x[k]); xhi = std::max(xhi, x[k]);
        ylo = std::min(ylo, y[k]); yhi = std::max(yhi, y[k]);
      }
      for (int k = 0; k < K; ++k) {
        // the neighbourhood stretched to [-1,1]^2 (the 1e-6 guards a degenerate extent, as in the reference)
        const double xn = 2.0 * (x[k] - xlo) / (xhi - xlo + 1e-6) - 1.0;
        const double yn = 2.0 * (y[k] - ylo) / (yhi - ylo + 1e-6) - 1.0;
        tap_out[(size_t)n * K + k] = (uint16_t)(nearest_node(xn, side) * side + nearest_node(yn, side));   // x-major node order
        if (nb_out) {
          nb_out[((size_t)k * n_out + n) * 2] = (float)xn;
          nb_out[((size_t)k * n_out + n) * 2 + 1] = (float)yn;
        }
      }
    });
  } catch (...) {
    return FOVI_ERR_INVALID_ARGUMENT;
  }
  return FOVI_OK;
}
