// Sensor -> first KNNConv in one call.  The sampler writes the KNNConv's input layout directly into a
// caller-provided intermediate buffer and the tensor-core kernel is enqueued right behind it on the same
// stream.  The intermediate is small (16 bytes per point pair and row: 33 MB for 1024 image x fixation rows
// of a 4010-point sensor) and stays resident in the 126 MB L2 between the two kernels (measured: the sampler
// writes 19 of 33 MB to DRAM at that size, nothing at a quarter of it), so the sensor output makes no HBM
// round trip; what a single fused kernel would add is only the removal of one launch.
#include "knnconv_plan.cuh"

extern "C" int64_t fovi_fused_intermediate_bytes(const fovi_knnconv_plan* conv, int rows) {
  if (!conv || rows < 0) return -1;
  if (conv->x_layout == FOVI_X_PAIRS) return (int64_t)((rows + 127) / 128) * conv->n_pairs * 2048;
  return (int64_t)rows * conv->n_in * conv->cin_packed * 2;
}

extern "C" int fovi_sample_knnconv_fused(const fovi_sampler_plan* sampler, fovi_knnconv_plan* conv, const void* img, int dtype,
                                         int B, int C, int H, int W, const int64_t* img_strides, const float* fix_rc,
                                         const float* fix_hw, int F, int mode, int pad, void* intermediate, const void* Wt,
                                         const float* bias, void* Y, int y_dtype, int relu, void* stream) {
  if (!sampler || !conv) return FOVI_ERR_INVALID_ARGUMENT;
  if (fovi_sampler_plan_num_points(sampler) != conv->n_in || C != conv->c_in) return FOVI_ERR_INVALID_ARGUMENT;
  if (B > 0 && !intermediate) return FOVI_ERR_INVALID_ARGUMENT;
  const bool pairs = conv->x_layout == FOVI_X_PAIRS;
  int rc = fovi_sample_forward(sampler, img, dtype, B, C, H, W, img_strides, fix_rc, fix_hw, F, mode, pad, intermediate, FOVI_BF16,
                               pairs ? FOVI_OUT_FB_PAIRS : FOVI_OUT_FBNC, conv->cin_packed, stream);
  if (rc) return rc;
  return fovi_knnconv_forward(conv, intermediate, Wt, bias, Y, y_dtype, B * F, relu, stream);
}
