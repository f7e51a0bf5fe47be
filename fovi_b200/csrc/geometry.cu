// Host-side sensor geometry: the foveated sample points of a sensor or layer (ring radii, angles per ring, cartesian /
// polar coordinates, the pad rings outside the field of view) and their coordinates on the cortical manifold.
//
// The reference computes these with a mix of float32 torch calls (linspace, exp, arange), float64 NumPy trigonometry
// and SciPy's trapezoid integral + linear interpolant (fovi/sensing/coords.py:204-370, 68-87;
// fovi/sensing/manifold.py:32-48, 139-170), so its last bits depend on the vector math libraries underneath.  Here
// every quantity follows the same formulas in the same order with the C library's correctly-rounded-or-nearly
// functions: float32 where the reference rounds to float32 (ring radii, spacings), double elsewhere.  The point
// COUNTS are integers derived from ratios that are not near integers for any shipped sensor and come out identical;
// coordinates agree with the reference's to a few units in the last float32 place (the float32 exp of the C library
// and of the reference's vector library can differ in the last bit of a ring radius).  No device is needed.
#include <cmath>
#include <cstdint>
#include <map>
#include <mutex>
#include <utility>
#include <vector>

#include "../../include/fovi_b200.h"

namespace {

constexpr double kManifoldK = 10.0;      // mm scale of the magnification function M(r) = k / (a + r)
constexpr double kMeshStep = 0.0001;     // degrees: integration mesh of the manifold's z
constexpr double kPi = 3.14159265358979323846;

// float32 linspace as torch computes it: a step in float32, values counted up from the start in the first half and down
// from the end in the second half.
std::vector<float> linspace_f32(float start, float end, int steps) {
  std::vector<float> v((size_t)steps);
  if (steps == 1) { v[0] = start; return v; }
  const float step = (end - start) / (float)(steps - 1);
  const int half = steps / 2;
  for (int i = 0; i < steps; ++i) v[(size_t)i] = i < half ? start + step * (float)i : end - step * (float)(steps - i - 1);
  return v;
}

// Ring radii in degrees (float32, res + 1 of them: one extra ring for the last spacing) and angles per ring.
void ring_layout(double fov, double a, int res, std::vector<float>& r, std::vector<int>& counts) {
  const double w_lo = std::log(a), w_hi = std::log(fov / 2 + a);
  const double dw = (w_hi - w_lo) / (res - 1);
  const std::vector<float> w = linspace_f32((float)w_lo, (float)(w_hi + dw), res + 1);
  r.resize((size_t)res + 1);
  const float af = (float)a;
  for (int i = 0; i <= res; ++i) r[(size_t)i] = std::exp(w[(size_t)i]) - af;
  counts.assign((size_t)res, 1);
  for (int i = 1; i < res; ++i) {
    // mean of the spacings to the neighbouring rings, circumference, all in float32; the ratio and its ceiling in double
    const float spacing = ((r[(size_t)i] - r[(size_t)i - 1]) + (r[(size_t)i + 1] - r[(size_t)i])) / 2.f;
    const float circumference = 2.f * (float)kPi * r[(size_t)i];
    counts[(size_t)i] = (int)std::ceil((double)circumference / (double)spacing);
  }
}

// z(r) of the cortical manifold on the integration mesh: cumulative trapezoid of sqrt(M^2 - rho'^2).
struct Manifold {
  std::vector<double> z;   // z at mesh point i = i * kMeshStep degrees
  double z_at(double r) const {
    const double t = r / kMeshStep;
    size_t i = (size_t)t;
    if (i + 1 >= z.size()) i = z.size() - 2;
    const double x0 = (double)i * kMeshStep, x1 = (double)(i + 1) * kMeshStep;
    const double slope = (z[i + 1] - z[i]) / (x1 - x0);
    return slope * (r - x0) + z[i];   // the linear interpolant's form: y0 + slope * (x - x0)
  }
};

const Manifold& manifold(double a, double fov) {
  static std::mutex mu;
  static std::map<std::pair<double, double>, Manifold> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_pair(a, fov);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  Manifold m;
  const size_t n = (size_t)std::ceil(2 * fov / kMeshStep);
  m.z.resize(n);
  double prev_x = 0, prev_f = 0, acc = 0;
  for (size_t i = 0; i < n; ++i) {
    const double x = (double)i * kMeshStep;
    const double mag = kManifoldK / (a + x);
    const double dmag = -kManifoldK * std::pow(a + x, -2.0);
    const double rad = x * (kPi / 180.0);
    const double drho = dmag * std::sin(rad) * (180 / kPi) + mag * std::cos(rad);
    const double f = std::sqrt(mag * mag - drho * drho);
    if (i > 0) acc += (x - prev_x) * (f + prev_f) / 2.0;
    m.z[i] = acc;
    prev_x = x; prev_f = f;
  }
  return cache.emplace(key, std::move(m)).first->second;
}

// Visual cartesian point in degrees -> cortical cartesian (double).
void cortical_point(const Manifold& man, double a, double x, double y, double* out) {
  const double r = std::sqrt(x * x + y * y);
  const double theta = std::atan2(y, x);
  const double rho = kManifoldK / (a + r) * std::sin(r * (kPi / 180.0)) * (180 / kPi);
  out[0] = rho * std::cos(theta); out[1] = rho * std::sin(theta); out[2] = man.z_at(r);
}

}  // namespace

extern "C" long long fovi_sensor_ring_layout(double fov, double cmf_a, int res, float* radius, int* counts) {
  if (res < 1 || !(fov > 0) || !(cmf_a > 0)) return -(long long)FOVI_ERR_INVALID_ARGUMENT;
  if (res == 1) {
    if (radius) radius[0] = 0.f;
    if (counts) counts[0] = 1;
    return 1;
  }
  std::vector<float> r;
  std::vector<int> c;
  ring_layout(fov, cmf_a, res, r, c);
  long long total = 0;
  const float half = (float)(fov / 2);
  for (int i = 0; i < res; ++i) {
    if (radius) radius[i] = r[(size_t)i] / half;
    if (counts) counts[i] = c[(size_t)i];
    total += c[(size_t)i];
  }
  return total;
}

extern "C" int fovi_sensor_points(double fov, double cmf_a, int res, double max_val, long long n_points, double* cartesian, double* polar,
                                  double* cortical) {
  if (res < 1 || !cartesian || !polar || !cortical) return FOVI_ERR_INVALID_ARGUMENT;
  if (res == 1) {
    if (n_points != 1) return FOVI_ERR_INVALID_ARGUMENT;
    cartesian[0] = cartesian[1] = polar[0] = polar[1] = cortical[0] = cortical[1] = cortical[2] = 0.0;
    return FOVI_OK;
  }
  std::vector<float> r;
  std::vector<int> c;
  ring_layout(fov, cmf_a, res, r, c);
  long long total = 0;
  for (int i = 0; i < res; ++i) total += c[(size_t)i];
  if (total != n_points) return FOVI_ERR_INVALID_ARGUMENT;
  const Manifold& man = manifold(cmf_a, fov);
  const float half = (float)(fov / 2);
  long long p = 0;
  for (int i = 0; i < res; ++i) {
    // normalised radius in float32 (divided, then scaled by max_val, as the reference does), widened to double for the points
    const double ring = (double)((r[(size_t)i] / half) * (float)max_val);
    const int cnt = c[(size_t)i];
    for (int j = 0; j < cnt; ++j, ++p) {
      const double angle = (double)j * (2 * kPi / (double)cnt);   // linspace(0, 2 pi, cnt, endpoint=False)
      const double x = ring * std::cos(angle), y = ring * std::sin(angle);
      cartesian[2 * p] = x; cartesian[2 * p + 1] = y;
      polar[2 * p] = ring; polar[2 * p + 1] = angle;
      cortical_point(man, cmf_a, x * (fov / 2), y * (fov / 2), cortical + 3 * p);
    }
  }
  return FOVI_OK;
}

extern "C" long long fovi_sensor_pad_points(double fov, double cmf_a, int res, double max_val, double padding_distance, long long capacity,
                                            float* cartesian_pad, float* cortical_pad) {
  if (res < 2) return -(long long)FOVI_ERR_INVALID_ARGUMENT;
  std::vector<float> r;
  std::vector<int> c;
  ring_layout(fov, cmf_a, res, r, c);
  const float half = (float)(fov / 2);
  const double last = (double)((r[(size_t)res - 1] / half) * (float)max_val), before = (double)((r[(size_t)res - 2] / half) * (float)max_val);
  const double gap = last - before, first = last + gap;
  if (!(gap > 0)) return -(long long)FOVI_ERR_INVALID_ARGUMENT;
  // arange(first, first + padding_distance, gap) and arange(0, 2 pi, gap): ceil((end - start) / step) values
  const long long n_rings = (long long)std::ceil(padding_distance / gap), n_ang = (long long)std::ceil(2 * kPi / gap);
  const long long total = n_rings * n_ang;
  if (!cartesian_pad && !cortical_pad) return total;
  if (capacity < total) return -(long long)FOVI_ERR_INVALID_ARGUMENT;
  const Manifold& man = manifold(cmf_a, fov);
  long long p = 0;
  for (long long i = 0; i < n_rings; ++i) {
    const double rr = first + (double)i * gap;
    for (long long j = 0; j < n_ang; ++j, ++p) {
      const double ang = (double)j * gap;
      const float x = (float)(rr * std::cos(ang)), y = (float)(rr * std::sin(ang));
      if (cartesian_pad) { cartesian_pad[2 * p] = x; cartesian_pad[2 * p + 1] = y; }
      if (cortical_pad) {
        // the reference maps the float32 pad points in float32 arithmetic; double here, rounded once at the end
        double q[3];
        cortical_point(man, cmf_a, (double)x * (fov / 2), (double)y * (fov / 2), q);
        cortical_pad[3 * p] = (float)q[0]; cortical_pad[3 * p + 1] = (float)q[1]; cortical_pad[3 * p + 2] = (float)q[2];
      }
    }
  }
  return total;
}
