// Depthwise KNN convolution: every input channel is filtered on its own,
//   out[b, c*g + j, n] = bias[c*g + j] + sum_k Xpad[b, c, idx[k,n]] * W[c, tap[n,k], j]        (g = c_out / c_in)
// (KNNDepthwiseConvLayer.forward, fovi/arch/knn.py:847-872, and the first half of KNNDepthwiseSeparableConvLayer.forward,
// :776-800).  There is no contraction over channels, so this is a gather with K multiply-adds per output element:
// bound by memory traffic, it runs on the ordinary cores.  Uses the compacted neighbour lists of a fovi_knnconv_plan.
#include <cuda_bf16.h>

#include "common.cuh"
#include "knnconv_plan.cuh"

namespace {

constexpr int BT = 8;   // batch rows per CTA: a filter value is loaded once and used for all of them

// One CTA: one output point, BT batch rows, all output channels (thread = output channel, looping when c_out > blockDim).
// X / Y are addressed through element strides, so both [B,C,N] and [B,N,C] work.  Wp: [V, c_out] float32.
template <typename TX, typename TY>
__global__ void __launch_bounds__(256) knn_depthwise_kernel(const TX* __restrict__ X, const float* __restrict__ Wp, const float* __restrict__ bias,
                                                            TY* __restrict__ Y, const int* __restrict__ nbr_idx,
                                                            const uint16_t* __restrict__ nbr_tap, const int* __restrict__ nbr_cnt, int kp,
                                                            int B, int c_out, int g, long long xsb, long long xsn, long long xsc, long long ysb,
                                                            long long ysn, long long ysc, int relu) {
  extern __shared__ int list_s[];                  // [kp] neighbour indices, then [kp] taps
  const int n = blockIdx.x;
  const int b0 = blockIdx.y * BT;
  const int cnt = nbr_cnt[n];
  int* idx_s = list_s;
  int* tap_s = list_s + kp;
  for (int k = threadIdx.x; k < cnt; k += blockDim.x) {
    idx_s[k] = nbr_idx[(long long)n * kp + k];
    tap_s[k] = nbr_tap[(long long)n * kp + k];
  }
  __syncthreads();
  const int bt = min(BT, B - b0);
  for (int co = threadIdx.x; co < c_out; co += blockDim.x) {
    const int c = co / g;
    float acc[BT];
#pragma unroll
    for (int r = 0; r < BT; ++r) acc[r] = 0.f;
    const TX* xc = X + (long long)b0 * xsb + (long long)c * xsc;
    for (int k = 0; k < cnt; ++k) {
      const float w = __ldg(Wp + (long long)tap_s[k] * c_out + co);
      const TX* xk = xc + (long long)idx_s[k] * xsn;
#pragma unroll
      for (int r = 0; r < BT; ++r)
        if (r < bt) acc[r] = fmaf(ld_as_float(xk + r * xsb), w, acc[r]);
    }
    const float bv = bias ? __ldg(bias + co) : 0.f;
#pragma unroll
    for (int r = 0; r < BT; ++r)
      if (r < bt) {
        const float v = acc[r] + bv;
        Y[(long long)(b0 + r) * ysb + (long long)n * ysn + (long long)co * ysc] = from_float<TY>(relu ? fmaxf(v, 0.f) : v);
      }
  }
}

// Gradients of the depthwise layer (autograd through fovi/arch/knn.py:847-872).  float32 atomics, so sums agree with the
// reference to rounding.  gX: every (row, output point, output channel) scatters gY * W onto the neighbours it read.
template <typename TG>
__global__ void __launch_bounds__(256) knn_depthwise_dx_kernel(const TG* __restrict__ gY, const float* __restrict__ Wp, float* __restrict__ gX,
                                                               const int* __restrict__ nbr_idx, const uint16_t* __restrict__ nbr_tap,
                                                               const int* __restrict__ nbr_cnt, int kp, int B, int c_out, int g, long long xsb,
                                                               long long xsn, long long xsc, long long ysb, long long ysn, long long ysc) {
  extern __shared__ int list_s[];
  const int n = blockIdx.x, b0 = blockIdx.y * BT;
  const int cnt = nbr_cnt[n];
  int* idx_s = list_s;
  int* tap_s = list_s + kp;
  for (int k = threadIdx.x; k < cnt; k += blockDim.x) { idx_s[k] = nbr_idx[(long long)n * kp + k]; tap_s[k] = nbr_tap[(long long)n * kp + k]; }
  __syncthreads();
  const int bt = min(BT, B - b0);
  for (int co = threadIdx.x; co < c_out; co += blockDim.x) {
    const int c = co / g;
    float gy[BT];
#pragma unroll
    for (int r = 0; r < BT; ++r) gy[r] = r < bt ? ld_as_float(gY + (long long)(b0 + r) * ysb + (long long)n * ysn + (long long)co * ysc) : 0.f;
    for (int k = 0; k < cnt; ++k) {
      const float w = __ldg(Wp + (long long)tap_s[k] * c_out + co);
      float* xk = gX + (long long)b0 * xsb + (long long)c * xsc + (long long)idx_s[k] * xsn;
#pragma unroll
      for (int r = 0; r < BT; ++r)
        if (r < bt) atomicAdd(xk + r * xsb, gy[r] * w);
    }
  }
}

// gW: for one output point and output channel, sum over the batch of X * gY per neighbour, added onto the neighbour's tap.
template <typename TX, typename TG>
__global__ void __launch_bounds__(256) knn_depthwise_dw_kernel(const TX* __restrict__ X, const TG* __restrict__ gY, float* __restrict__ gWp,
                                                               const int* __restrict__ nbr_idx, const uint16_t* __restrict__ nbr_tap,
                                                               const int* __restrict__ nbr_cnt, int kp, int B, int c_out, int g, long long xsb,
                                                               long long xsn, long long xsc, long long ysb, long long ysn, long long ysc) {
  const int n = blockIdx.x;
  const int cnt = nbr_cnt[n];
  for (int co = threadIdx.x; co < c_out; co += blockDim.x) {
    const int c = co / g;
    for (int k = 0; k < cnt; ++k) {
      const int j = nbr_idx[(long long)n * kp + k];
      float s = 0.f;
      for (int b = 0; b < B; ++b)
        s = fmaf(ld_as_float(X + (long long)b * xsb + (long long)c * xsc + (long long)j * xsn),
                 ld_as_float(gY + (long long)b * ysb + (long long)n * ysn + (long long)co * ysc), s);
      atomicAdd(gWp + (long long)nbr_tap[(long long)n * kp + k] * c_out + co, s);
    }
  }
}

}  // namespace

extern "C" int fovi_knn_depthwise_backward(const fovi_knnconv_plan* p, const void* X, int x_dtype, int x_layout, const float* Wp, const void* gY,
                                           int g_dtype, int y_layout, int B, float* gX, float* gWp, void* stream) {
  if (!p || !fovi::valid_dtype(x_dtype) || !fovi::valid_dtype(g_dtype) || B < 0) return FOVI_ERR_INVALID_ARGUMENT;
  if ((x_layout != FOVI_ACT_BCN && x_layout != FOVI_ACT_BNC) || (y_layout != FOVI_ACT_BCN && y_layout != FOVI_ACT_BNC))
    return FOVI_ERR_INVALID_ARGUMENT;
  if (p->c_in <= 0 || p->c_out % p->c_in) return FOVI_ERR_UNSUPPORTED;
  if (B == 0) return FOVI_OK;
  if (!gY || (gX && !Wp) || (gWp && !X)) return FOVI_ERR_INVALID_ARGUMENT;
  if ((B + BT - 1) / BT > 65535) return FOVI_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int g = p->c_out / p->c_in;
  const bool xb = x_layout == FOVI_ACT_BNC, yb = y_layout == FOVI_ACT_BNC;
  const long long xsb = (long long)p->c_in * p->n_in, xsn = xb ? p->c_in : 1, xsc = xb ? 1 : p->n_in;
  const long long ysb = (long long)p->c_out * p->n_out, ysn = yb ? p->c_out : 1, ysc = yb ? 1 : p->n_out;
  const int threads = std::min(256, (p->c_out + 31) / 32 * 32);
  if (gX) {
    const size_t smem = (size_t)p->kp * 2 * sizeof(int);
    dim3 grid(p->n_out, (B + BT - 1) / BT);
    if (g_dtype == FOVI_F32)
      knn_depthwise_dx_kernel<float><<<grid, threads, smem, st>>>((const float*)gY, Wp, gX, p->nbr_idx, p->nbr_tap, p->nbr_cnt, p->kp, B, p->c_out, g,
                                                                  xsb, xsn, xsc, ysb, ysn, ysc);
    else
      knn_depthwise_dx_kernel<__nv_bfloat16><<<grid, threads, smem, st>>>((const __nv_bfloat16*)gY, Wp, gX, p->nbr_idx, p->nbr_tap, p->nbr_cnt, p->kp, B,
                                                                          p->c_out, g, xsb, xsn, xsc, ysb, ysn, ysc);
    int rc = fovi::after_launch("knn_depthwise_dx_kernel");
    if (rc) return rc;
  }
  if (gWp) {
#define RUN(TX, TG) knn_depthwise_dw_kernel<TX, TG><<<p->n_out, threads, 0, st>>>((const TX*)X, (const TG*)gY, gWp, p->nbr_idx, p->nbr_tap, p->nbr_cnt, p->kp, \
                                                                                  B, p->c_out, g, xsb, xsn, xsc, ysb, ysn, ysc)
    if (x_dtype == FOVI_F32) { if (g_dtype == FOVI_F32) RUN(float, float); else RUN(float, __nv_bfloat16); }
    else { if (g_dtype == FOVI_F32) RUN(__nv_bfloat16, float); else RUN(__nv_bfloat16, __nv_bfloat16); }
#undef RUN
    return fovi::after_launch("knn_depthwise_dw_kernel");
  }
  return FOVI_OK;
}

extern "C" int fovi_knn_depthwise_forward(const fovi_knnconv_plan* p, const void* X, int x_dtype, int x_layout, const float* Wp,
                                          const float* bias, void* Y, int y_dtype, int y_layout, int B, int relu, void* stream) {
  if (!p || !fovi::valid_dtype(x_dtype) || !fovi::valid_dtype(y_dtype) || B < 0) return FOVI_ERR_INVALID_ARGUMENT;
  if ((x_layout != FOVI_ACT_BCN && x_layout != FOVI_ACT_BNC) || (y_layout != FOVI_ACT_BCN && y_layout != FOVI_ACT_BNC))
    return FOVI_ERR_INVALID_ARGUMENT;
  if (p->c_in <= 0 || p->c_out % p->c_in) return FOVI_ERR_UNSUPPORTED;
  if (B == 0) return FOVI_OK;
  if (!X || !Wp || !Y) return FOVI_ERR_INVALID_ARGUMENT;
  if ((B + BT - 1) / BT > 65535) return FOVI_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int g = p->c_out / p->c_in;
  const bool xb = x_layout == FOVI_ACT_BNC, yb = y_layout == FOVI_ACT_BNC;
  const long long xsb = (long long)p->c_in * p->n_in, xsn = xb ? p->c_in : 1, xsc = xb ? 1 : p->n_in;
  const long long ysb = (long long)p->c_out * p->n_out, ysn = yb ? p->c_out : 1, ysc = yb ? 1 : p->n_out;
  const int threads = std::min(256, (p->c_out + 31) / 32 * 32);
  const size_t smem = (size_t)p->kp * 2 * sizeof(int);
  dim3 grid(p->n_out, (B + BT - 1) / BT);
#define RUN(TX, TY)                                                                                                              \
  knn_depthwise_kernel<TX, TY><<<grid, threads, smem, st>>>((const TX*)X, Wp, bias, (TY*)Y, p->nbr_idx, p->nbr_tap, p->nbr_cnt, p->kp, B, \
                                                            p->c_out, g, xsb, xsn, xsc, ysb, ysn, ysc, relu)
  if (x_dtype == FOVI_F32) { if (y_dtype == FOVI_F32) RUN(float, float); else RUN(float, __nv_bfloat16); }
  else { if (y_dtype == FOVI_F32) RUN(__nv_bfloat16, float); else RUN(__nv_bfloat16, __nv_bfloat16); }
#undef RUN
  return fovi::after_launch("knn_depthwise_kernel");
}
