// Per-sample normalisation of KNN activations: the layer / group / channel / coordinate norms of the reference
// (fovi/arch/norm.py:14-101, thin wrappers over torch's LayerNorm and GroupNorm applied to [B, C, N]):
//   channel : statistics over the C channels of every (sample, point);            weight, bias [C]
//   coord   : statistics over the N points of every (sample, channel);            weight, bias [N]
//   layer   : statistics over all C x N values of a sample;                       weight, bias [C, N]
//   group   : statistics over the N points x (C / groups) channels of a group;    weight, bias [C]
//   y = (x - mean) / sqrt(var + eps) * weight + bias      (biased variance, float32 statistics, two passes)
// Two small kernels: one CTA per statistics group computes (mean, 1/std), an element-wise pass applies them with the
// affine parameters and an optional ReLU.  Both activation layouts ([B,C,N] and the kernels' channels-last [B,N,C]).
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

enum { NORM_CHANNEL = 0, NORM_COORD = 1, NORM_LAYER = 2, NORM_GROUP = 3 };

struct NormGeom {
  int B, C, N, mode, groups;      // groups: channel groups of NORM_GROUP
  long long sb, sn, sc;           // element strides of x and y (same layout)
  int bnc;                        // 1: channels-last (c fastest), 0: points fastest
};

__device__ __forceinline__ float block_sum(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
  return t;
}

// Element `e` of statistics group `g` -> offset in x.  cnt = elements per group.
__device__ __forceinline__ long long group_elem(const NormGeom& q, long long g, int e) {
  const int cpg = q.mode == NORM_GROUP ? q.C / q.groups : 0;
  int b, n, c;
  switch (q.mode) {
    case NORM_CHANNEL: b = (int)(g / q.N); n = (int)(g % q.N); c = e; break;
    case NORM_COORD:   b = (int)(g / q.C); c = (int)(g % q.C); n = e; break;
    case NORM_LAYER:   b = (int)g; if (q.bnc) { n = e / q.C; c = e % q.C; } else { c = e / q.N; n = e % q.N; } break;
    default: {
      b = (int)(g / q.groups); const int c0 = (int)(g % q.groups) * cpg;
      if (q.bnc) { n = e / cpg; c = c0 + e % cpg; } else { c = c0 + e / q.N; n = e % q.N; }
    }
  }
  return (long long)b * q.sb + (long long)n * q.sn + (long long)c * q.sc;
}

template <typename T>
__global__ void __launch_bounds__(256) knn_norm_stats_kernel(const T* __restrict__ x, float2* __restrict__ stats, const NormGeom q, int cnt, float eps) {
  __shared__ float red[8];
  const long long g = blockIdx.x;
  float s = 0.f;
  for (int e = threadIdx.x; e < cnt; e += blockDim.x) s += ld_as_float(x + group_elem(q, g, e));
  const float mean = block_sum(s, red) / (float)cnt;
  float v = 0.f;
  for (int e = threadIdx.x; e < cnt; e += blockDim.x) { const float d = ld_as_float(x + group_elem(q, g, e)) - mean; v += d * d; }
  const float var = block_sum(v, red) / (float)cnt;
  if (threadIdx.x == 0) stats[g] = make_float2(mean, rsqrtf(var + eps));
}

template <typename TX, typename TY>
__global__ void knn_norm_apply_kernel(const TX* __restrict__ x, TY* __restrict__ y, const float2* __restrict__ stats, const float* __restrict__ w,
                                      const float* __restrict__ bias, const NormGeom q, int relu) {
  const long long total = (long long)q.B * q.C * q.N;
  const int cpg = q.mode == NORM_GROUP ? q.C / q.groups : 1;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    int b, n, c;
    if (q.bnc) { c = (int)(i % q.C); n = (int)((i / q.C) % q.N); b = (int)(i / ((long long)q.C * q.N)); }
    else { n = (int)(i % q.N); c = (int)((i / q.N) % q.C); b = (int)(i / ((long long)q.C * q.N)); }
    long long g; int p;
    switch (q.mode) {
      case NORM_CHANNEL: g = (long long)b * q.N + n; p = c; break;
      case NORM_COORD:   g = (long long)b * q.C + c; p = n; break;
      case NORM_LAYER:   g = b; p = c * q.N + n; break;
      default:           g = (long long)b * q.groups + c / cpg; p = c;
    }
    const float2 st = __ldg(stats + g);
    float v = (ld_as_float(x + i) - st.x) * st.y;
    if (w) v = v * __ldg(w + p);
    if (bias) v = v + __ldg(bias + p);
    if (relu) v = fmaxf(v, 0.f);
    y[i] = from_float<TY>(v);
  }
}

}  // namespace

extern "C" int64_t fovi_knn_norm_stat_groups(int mode, int B, int C, int N, int groups) {
  switch (mode) {
    case NORM_CHANNEL: return (int64_t)B * N;
    case NORM_COORD: return (int64_t)B * C;
    case NORM_LAYER: return B;
    case NORM_GROUP: return (groups > 0 && C % groups == 0) ? (int64_t)B * groups : -1;
    default: return -1;
  }
}

extern "C" int fovi_knn_norm_forward(const void* x, int x_dtype, int layout, int B, int C, int N, int mode, int groups, const float* weight,
                                     const float* bias, float eps, int relu, float* stats, void* y, int y_dtype, void* stream) {
  if (!fovi::valid_dtype(x_dtype) || !fovi::valid_dtype(y_dtype) || B < 0 || C <= 0 || N <= 0) return FOVI_ERR_INVALID_ARGUMENT;
  if (layout != FOVI_ACT_BCN && layout != FOVI_ACT_BNC) return FOVI_ERR_INVALID_ARGUMENT;
  const int64_t ng = fovi_knn_norm_stat_groups(mode, B, C, N, groups);
  if (ng < 0) return FOVI_ERR_INVALID_ARGUMENT;
  if (B == 0) return FOVI_OK;
  if (!x || !y || !stats) return FOVI_ERR_INVALID_ARGUMENT;
  if (ng >= (1ll << 31) || (long long)C * N >= (1ll << 31)) return FOVI_ERR_UNSUPPORTED;
  NormGeom q;
  q.B = B; q.C = C; q.N = N; q.mode = mode; q.groups = groups; q.bnc = layout == FOVI_ACT_BNC ? 1 : 0;
  q.sb = (long long)C * N; q.sn = q.bnc ? C : 1; q.sc = q.bnc ? 1 : N;
  const int cnt = mode == NORM_CHANNEL ? C : mode == NORM_COORD ? N : mode == NORM_LAYER ? C * N : (C / groups) * N;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  float2* s2 = reinterpret_cast<float2*>(stats);
  if (x_dtype == FOVI_F32) knn_norm_stats_kernel<float><<<(int)ng, 256, 0, st>>>((const float*)x, s2, q, cnt, eps);
  else knn_norm_stats_kernel<__nv_bfloat16><<<(int)ng, 256, 0, st>>>((const __nv_bfloat16*)x, s2, q, cnt, eps);
  int rc = fovi::after_launch("knn_norm_stats_kernel");
  if (rc) return rc;
  const long long total = (long long)B * C * N;
  const int grid = (int)std::min<long long>((total + 255) / 256, (long long)fovi::sm_count() * 16);
#define RUN(TX, TY) knn_norm_apply_kernel<TX, TY><<<grid, 256, 0, st>>>((const TX*)x, (TY*)y, s2, weight, bias, q, relu)
  if (x_dtype == FOVI_F32) { if (y_dtype == FOVI_F32) RUN(float, float); else RUN(float, __nv_bfloat16); }
  else { if (y_dtype == FOVI_F32) RUN(__nv_bfloat16, float); else RUN(__nv_bfloat16, __nv_bfloat16); }
#undef RUN
  return fovi::after_launch("knn_norm_apply_kernel");
}
