// Sensor -> first KNNConv in one call, the sensor output handed over through L2.
//
// The two kernels stay separate (every sensor point feeds ~30 output points of the first layer: sampling inside the
// convolution's producer would redo each bilinear gather 30 times, and the union of the neighbourhoods of even four
// output points does not fit shared memory at 128 rows).  What is fused is the memory path: the sampler writes the
// convolution's input layout into a caller-provided intermediate (16 bytes per point pair and row: 33 MB for 1024
// image x fixation rows of a 4010-point sensor), and for the duration of the two launches that buffer is declared
// PERSISTING in L2 through the stream's access-policy window while the images the sampler streams through stay
// ordinary lines.  Without the window the sampler's 200 MB of image reads push most of the intermediate out to DRAM
// before the convolution reads it back; with it the intermediate is written and read in L2 only.  The convolution is
// launched with the same window set to the NORMAL property: a normal access to a persisting line returns it to
// ordinary replacement, so the lines are released by the very reads that consume them and nothing stays pinned after
// the call; the window itself is cleared before returning.  The L2 carve-out that persisting lines may occupy is a
// limit of this process's context (not a device setting), raised once per device to what the intermediate needs, at
// most the device's maximum.
#include <algorithm>
#include <mutex>
#include <string.h>

#include "knnconv_plan.cuh"

namespace {

// Bytes of L2 this device lets a context set aside for persisting lines and the largest access-policy window; the
// context limit is raised (never lowered) to `want`.  Returns the window size usable for `want` bytes, 0 if none.
size_t persisting_window(size_t want) {
  static std::mutex mu;
  static size_t limit_set[64] = {0};
  int dev = -1, max_persist = 0, max_window = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cudaDeviceGetAttribute(&max_persist, cudaDevAttrMaxPersistingL2CacheSize, dev) != cudaSuccess || max_persist <= 0) return 0;
  if (cudaDeviceGetAttribute(&max_window, cudaDevAttrMaxAccessPolicyWindowSize, dev) != cudaSuccess || max_window <= 0) return 0;
  const size_t bytes = std::min<size_t>(want, std::min<size_t>((size_t)max_persist, (size_t)max_window));
  std::lock_guard<std::mutex> lock(mu);
  if (limit_set[dev] < bytes) {
    if (cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, bytes) != cudaSuccess) { cudaGetLastError(); return 0; }
    limit_set[dev] = bytes;
  }
  return bytes;
}

// Access-policy window of the launches that follow on `st`: accesses inside [base, base + bytes) get `prop`.
void set_window(cudaStream_t st, void* base, size_t bytes, cudaAccessProperty prop) {
  cudaStreamAttrValue v;
  memset(&v, 0, sizeof(v));
  v.accessPolicyWindow.base_ptr = base;
  v.accessPolicyWindow.num_bytes = bytes;
  v.accessPolicyWindow.hitRatio = 1.0f;
  v.accessPolicyWindow.hitProp = prop;
  v.accessPolicyWindow.missProp = cudaAccessPropertyNormal;
  if (cudaStreamSetAttribute(st, cudaStreamAttributeAccessPolicyWindow, &v) != cudaSuccess) cudaGetLastError();
}

}  // namespace

extern "C" int64_t fovi_fused_intermediate_bytes(const fovi_knnconv_plan* conv, int rows) {
  if (!conv || rows < 0) return -1;
  if (conv->x_layout == FOVI_X_PAIRS) return (int64_t)((rows + 127) / 128) * conv->n_pairs * 2048;
  return (int64_t)rows * conv->n_in * conv->cin_packed * 2;
}

extern "C" int fovi_sample_knnconv_fused(const fovi_sampler_plan* sampler, fovi_knnconv_plan* conv, const void* img, int dtype,
                                         int B, int C, int H, int W, const int64_t* img_strides, const float* fix_rc,
                                         const float* fix_hw, int F, int mode, int pad, void* intermediate, const void* Wt,
                                         const float* bias, void* Y, int y_dtype, int relu, int row_order, void* stream) {
  if (!sampler || !conv || (row_order != 0 && row_order != 1)) return FOVI_ERR_INVALID_ARGUMENT;
  if (fovi_sampler_plan_num_points(sampler) != conv->n_in || C != conv->c_in) return FOVI_ERR_INVALID_ARGUMENT;
  if (B > 0 && !intermediate) return FOVI_ERR_INVALID_ARGUMENT;
  const bool pairs = conv->x_layout == FOVI_X_PAIRS;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t need = B > 0 ? (size_t)fovi_fused_intermediate_bytes(conv, B * F) : 0;
  const size_t window = need ? persisting_window(need) : 0;
  if (window) set_window(st, intermediate, window, cudaAccessPropertyPersisting);      // the sampler's writes stay in L2
  int rc = fovi_sample_forward(sampler, img, dtype, B, C, H, W, img_strides, fix_rc, fix_hw, F, mode, pad, intermediate, FOVI_BF16,
                               pairs ? (row_order ? FOVI_OUT_BF_PAIRS : FOVI_OUT_FB_PAIRS) : (row_order ? FOVI_OUT_BFNC : FOVI_OUT_FBNC), conv->cin_packed,
                               stream);
  if (window) set_window(st, intermediate, window, cudaAccessPropertyNormal);          // the convolution's reads release them
  if (rc == FOVI_OK) rc = fovi_knnconv_forward(conv, intermediate, Wt, bias, Y, y_dtype, B * F, relu, stream);
  if (window) set_window(st, nullptr, 0, cudaAccessPropertyNormal);                    // later launches on this stream: no window
  return rc;
}
