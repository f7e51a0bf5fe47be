// KNN pooling: max / mean / sum over the K nearest input points of every output point, pad neighbours
// ignored (the reference pads with NaN and uses nan-aware reductions, fovi/arch/knn.py:345-371).
// A pure gather-reduce, bound by HBM/L2 bandwidth: one thread per output element walks its K neighbours.
// Threads are laid out along the contiguous dimension of the activations (channels for the channels-last
// layout, points for the reference's [B,C,N]), so every neighbour read of a warp is one or two cache lines
// (channels-last) or a short gather (points-last).  NaN inputs are skipped like pads, as nanmean/nansum do.
#include <cstdint>
#include <vector>

#include <cuda_bf16.h>

#include "common.cuh"

struct fovi_knnpool_plan {
  int n_in = 0, n_out = 0, K = 0;
  int* idx = nullptr;   // [n_out, K] neighbour indices, pad = n_in
  float* wgt = nullptr; // [n_out, K] neighbour weights of the 'gaussian' mode (null until set)
};

namespace {

// MODE 0 max, 1 mean, 2 sum, 3 weighted mean: sum_k x_k * w_k / (sum of the weights of the valid neighbours + 1e-8), the
// 'gaussian' pooling of the reference (fovi/arch/knn.py:372-394: weights of pad / NaN neighbours are dropped and the rest
// renormalised).
template <typename T, int MODE>
__global__ void knnpool_kernel(const T* __restrict__ X, T* __restrict__ Y, const int* __restrict__ idx, const float* __restrict__ wgt, int B,
                               int C, int n_in, int n_out, int K, int bnc) {
  const long long total = (long long)B * C * n_out;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    int b, c, n;
    if (bnc) { c = (int)(e % C); n = (int)((e / C) % n_out); b = (int)(e / ((long long)C * n_out)); }
    else { n = (int)(e % n_out); c = (int)((e / n_out) % C); b = (int)(e / ((long long)C * n_out)); }
    const int* nb = idx + (long long)n * K;
    float acc = MODE == 0 ? -INFINITY : 0.f, wsum = 0.f;
    int cnt = 0;
    for (int k = 0; k < K; ++k) {
      const int j = __ldg(nb + k);
      if (j >= n_in) continue;
      const float v = ld_as_float(bnc ? X + ((long long)b * n_in + j) * C + c : X + ((long long)b * C + c) * n_in + j);
      if (v != v) continue;   // NaN: ignored
      if (MODE == 0) acc = fmaxf(acc, v);
      else if (MODE == 3) { const float w = __ldg(wgt + (long long)n * K + k); acc = fmaf(v, w, acc); wsum += w; }
      else acc += v;
      ++cnt;
    }
    if (MODE == 1) acc = acc / (float)cnt;   // no valid neighbour: 0/0 = NaN, as nanmean
    if (MODE == 3) acc = acc / (wsum + 1e-8f);
    Y[e] = from_float<T>(acc);
  }
}

// Channels-last bf16 with C a multiple of 8: one thread per (row, output point, 8 channels), 16-byte loads, so a warp
// reads up to 512 contiguous bytes per neighbour.  Same arithmetic as the scalar kernel (float32 compare / add, NaN skipped).
template <int MODE>
__global__ void knnpool_bnc8_kernel(const __nv_bfloat16* __restrict__ X, __nv_bfloat16* __restrict__ Y, const int* __restrict__ idx, int B,
                                    int C, int n_in, int n_out, int K) {
  const int c8 = C >> 3;
  const long long total = (long long)B * n_out * c8;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int cg = (int)(e % c8);
    const long long r = e / c8;
    const int n = (int)(r % n_out);
    const long long b = r / n_out;
    const int* nb = idx + (long long)n * K;
    const uint4* xb = reinterpret_cast<const uint4*>(X + b * (long long)n_in * C) + cg;
    float acc[8];
    int cnt[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { acc[i] = MODE == 0 ? -INFINITY : 0.f; cnt[i] = 0; }
    for (int k = 0; k < K; ++k) {
      const int j = __ldg(nb + k);
      if (j >= n_in) continue;
      const uint4 q = __ldg(xb + (long long)j * c8);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);   // bf16 -> float32, exact
        if (lo == lo) { if (MODE == 0) acc[2 * i] = fmaxf(acc[2 * i], lo); else acc[2 * i] += lo; ++cnt[2 * i]; }
        if (hi == hi) { if (MODE == 0) acc[2 * i + 1] = fmaxf(acc[2 * i + 1], hi); else acc[2 * i + 1] += hi; ++cnt[2 * i + 1]; }
      }
    }
    __align__(16) __nv_bfloat16 out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __float2bfloat16_rn(MODE == 1 ? acc[i] / (float)cnt[i] : acc[i]);
    reinterpret_cast<uint4*>(Y)[e] = *reinterpret_cast<const uint4*>(out);
  }
}

// Gradient of the pooling with respect to its input, what autograd computes through the reference's gather and
// nan-aware reductions (fovi/arch/knn.py:345-394): every output element hands its upstream gradient back to the
// neighbours it read -- 'sum': all of it to each; 'avg': 1/count to each; 'gaussian': the renormalised weight w_k /
// (sum of valid weights + 1e-8) to each; 'max': all of it to the first neighbour (in list order) that holds the maximum.
// One thread per output element, float32 atomic adds into a zero-initialised dX (neighbourhoods overlap).
template <typename TX, typename TG, int MODE>
__global__ void knnpool_backward_kernel(const TX* __restrict__ X, const TG* __restrict__ G, float* __restrict__ dX, const int* __restrict__ idx,
                                        const float* __restrict__ wgt, int B, int C, int n_in, int n_out, int K, int bnc) {
  const long long total = (long long)B * C * n_out;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    int b, c, n;
    if (bnc) { c = (int)(e % C); n = (int)((e / C) % n_out); b = (int)(e / ((long long)C * n_out)); }
    else { n = (int)(e % n_out); c = (int)((e / n_out) % C); b = (int)(e / ((long long)C * n_out)); }
    const int* nb = idx + (long long)n * K;
    const float g = ld_as_float(G + e);
    auto at = [&](int j) { return bnc ? ((long long)b * n_in + j) * C + c : ((long long)b * C + c) * n_in + j; };
    // first pass: what the forward reduced over (valid = not a pad, not NaN)
    float best = -INFINITY, wsum = 0.f;
    int cnt = 0, arg = -1;
    for (int k = 0; k < K; ++k) {
      const int j = __ldg(nb + k);
      if (j >= n_in) continue;
      const float v = ld_as_float(X + at(j));
      if (v != v) continue;
      if (MODE == 0 && (arg < 0 || v > best)) { best = v; arg = j; }
      if (MODE == 3) wsum += __ldg(wgt + (long long)n * K + k);
      ++cnt;
    }
    if (cnt == 0) continue;
    if constexpr (MODE == 0) {
      atomicAdd(dX + at(arg), g);
    } else {
      for (int k = 0; k < K; ++k) {
        const int j = __ldg(nb + k);
        if (j >= n_in) continue;
        const float v = ld_as_float(X + at(j));
        if (v != v) continue;
        const float coeff = MODE == 1 ? 1.f / (float)cnt : MODE == 3 ? __ldg(wgt + (long long)n * K + k) / (wsum + 1e-8f) : 1.f;
        atomicAdd(dX + at(j), g * coeff);
      }
    }
  }
}

}  // namespace

extern "C" int fovi_knnpool_plan_create(const int32_t* knn_idx_pad, int n_in, int n_out, int K, fovi_knnpool_plan** out) {
  if (!knn_idx_pad || !out || n_in <= 0 || n_out <= 0 || K <= 0) return FOVI_ERR_INVALID_ARGUMENT;
  std::vector<int> t((size_t)n_out * K);
  for (int k = 0; k < K; ++k)
    for (int n = 0; n < n_out; ++n) {
      const int j = knn_idx_pad[(size_t)k * n_out + n];
      if (j < 0 || j > n_in) return FOVI_ERR_TABLE_RANGE;
      t[(size_t)n * K + k] = j;
    }
  auto* p = new fovi_knnpool_plan();
  p->n_in = n_in; p->n_out = n_out; p->K = K;
  cudaError_t e = cudaMalloc(&p->idx, sizeof(int) * t.size());
  if (e == cudaSuccess) e = cudaMemcpy(p->idx, t.data(), sizeof(int) * t.size(), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    if (p->idx) cudaFree(p->idx);
    delete p;
    return fovi::cuda_fail(e, "fovi_knnpool_plan_create");
  }
  *out = p;
  return FOVI_OK;
}

extern "C" void fovi_knnpool_plan_destroy(fovi_knnpool_plan* p) {
  if (!p) return;
  if (p->idx) cudaFree(p->idx);
  if (p->wgt) cudaFree(p->wgt);
  delete p;
}

extern "C" int fovi_knnpool_set_weights(fovi_knnpool_plan* p, const float* w_kn) {
  if (!p || !w_kn) return FOVI_ERR_INVALID_ARGUMENT;
  std::vector<float> t((size_t)p->n_out * p->K);
  for (int k = 0; k < p->K; ++k)
    for (int n = 0; n < p->n_out; ++n) t[(size_t)n * p->K + k] = w_kn[(size_t)k * p->n_out + n];
  if (!p->wgt) FOVI_CUDA(cudaMalloc(&p->wgt, sizeof(float) * t.size()));
  FOVI_CUDA(cudaMemcpy(p->wgt, t.data(), sizeof(float) * t.size(), cudaMemcpyHostToDevice));
  return FOVI_OK;
}

extern "C" int fovi_knnpool_forward(const fovi_knnpool_plan* p, const void* X, int dtype, int layout, int B, int C, int mode,
                                    void* Y, void* stream) {
  if (!p || !fovi::valid_dtype(dtype) || B < 0 || C <= 0 || mode < 0 || mode > 3) return FOVI_ERR_INVALID_ARGUMENT;
  if (mode == 3 && !p->wgt) return FOVI_ERR_INVALID_ARGUMENT;   // fovi_knnpool_set_weights first
  if (layout != FOVI_ACT_BCN && layout != FOVI_ACT_BNC) return FOVI_ERR_INVALID_ARGUMENT;
  if (B == 0) return FOVI_OK;
  if (!X || !Y) return FOVI_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long total = (long long)B * C * p->n_out;
  const int grid = (int)std::min<long long>((total + 255) / 256, (long long)fovi::sm_count() * 32);
  const int bnc = layout == FOVI_ACT_BNC;
  if (mode != 3 && bnc && dtype == FOVI_BF16 && C % 8 == 0 && (reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(Y)) % 16 == 0) {
    const long long tot8 = total / 8;
    const int g8 = (int)std::min<long long>((tot8 + 255) / 256, (long long)fovi::sm_count() * 32);
    const __nv_bfloat16* x = (const __nv_bfloat16*)X;
    __nv_bfloat16* y = (__nv_bfloat16*)Y;
    if (mode == 0) knnpool_bnc8_kernel<0><<<g8, 256, 0, st>>>(x, y, p->idx, B, C, p->n_in, p->n_out, p->K);
    else if (mode == 1) knnpool_bnc8_kernel<1><<<g8, 256, 0, st>>>(x, y, p->idx, B, C, p->n_in, p->n_out, p->K);
    else knnpool_bnc8_kernel<2><<<g8, 256, 0, st>>>(x, y, p->idx, B, C, p->n_in, p->n_out, p->K);
    return fovi::after_launch("knnpool_bnc8_kernel");
  }
#define RUN(T, M) knnpool_kernel<T, M><<<grid, 256, 0, st>>>((const T*)X, (T*)Y, p->idx, p->wgt, B, C, p->n_in, p->n_out, p->K, bnc)
  if (dtype == FOVI_F32) { if (mode == 0) RUN(float, 0); else if (mode == 1) RUN(float, 1); else if (mode == 2) RUN(float, 2); else RUN(float, 3); }
  else { if (mode == 0) RUN(__nv_bfloat16, 0); else if (mode == 1) RUN(__nv_bfloat16, 1); else if (mode == 2) RUN(__nv_bfloat16, 2); else RUN(__nv_bfloat16, 3); }
#undef RUN
  return fovi::after_launch("knnpool_kernel");
}

extern "C" int fovi_knnpool_backward(const fovi_knnpool_plan* p, const void* X, int x_dtype, const void* gY, int g_dtype, int layout, int B, int C,
                                     int mode, float* dX, void* stream) {
  if (!p || !fovi::valid_dtype(x_dtype) || !fovi::valid_dtype(g_dtype) || B < 0 || C <= 0 || mode < 0 || mode > 3) return FOVI_ERR_INVALID_ARGUMENT;
  if (mode == 3 && !p->wgt) return FOVI_ERR_INVALID_ARGUMENT;
  if (layout != FOVI_ACT_BCN && layout != FOVI_ACT_BNC) return FOVI_ERR_INVALID_ARGUMENT;
  if (B == 0) return FOVI_OK;
  if (!X || !gY || !dX) return FOVI_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  FOVI_CUDA(cudaMemsetAsync(dX, 0, sizeof(float) * (size_t)B * C * p->n_in, st));
  const long long total = (long long)B * C * p->n_out;
  const int grid = (int)std::min<long long>((total + 255) / 256, (long long)fovi::sm_count() * 32);
  const int bnc = layout == FOVI_ACT_BNC;
#define RUNB(TX, TG, M) knnpool_backward_kernel<TX, TG, M><<<grid, 256, 0, st>>>((const TX*)X, (const TG*)gY, dX, p->idx, p->wgt, B, C, p->n_in, \
                                                                                  p->n_out, p->K, bnc)
#define RUNM(TX, TG) do { if (mode == 0) RUNB(TX, TG, 0); else if (mode == 1) RUNB(TX, TG, 1); else if (mode == 2) RUNB(TX, TG, 2); else RUNB(TX, TG, 3); } while (0)
  if (x_dtype == FOVI_F32) { if (g_dtype == FOVI_F32) RUNM(float, float); else RUNM(float, __nv_bfloat16); }
  else { if (g_dtype == FOVI_F32) RUNM(__nv_bfloat16, float); else RUNM(__nv_bfloat16, __nv_bfloat16); }
#undef RUNM
#undef RUNB
  return fovi::after_launch("knnpool_backward_kernel");
}
