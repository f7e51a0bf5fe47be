// Sensor sampler for sm_100a: nearest / bilinear gather of image pixels at the foveated sample
// points, for every fixation of every image in one launch.
//
// One CTA owns one (image, fixation) pair.  Its threads walk the sensor's points in a
// spatially sorted order (Morton order of the fixed sensor grid, built once per plan), so the
// 32 points of a warp fall in a compact image patch and their taps share cache lines.  Results
// are staged in shared memory at the points' ORIGINAL indices and leave the CTA as one
// contiguous, 16-byte vectorised store, so global writes are fully coalesced whatever the
// visiting order was.
//
// Arithmetic: float32, one rounding per operation in the order of the reference
// (fovi/sensing/coords.py:624-640 followed by torch's CPU grid_sample with align_corners=False):
//   g  = ((2 * (x * (fw/2) + col*W)) / W) - 1          five separately rounded operations
//   ix = fma(g + 1, W/2, -0.5)
//   bilinear: weights are rounded products; the four taps are accumulated NW, NE, SW, SE with
//   fused multiply-adds.  The explicit __f*_rn intrinsics keep the compiler from contracting or
//   re-associating any of it, which is what makes float32 results bit-identical to the CPU
//   reference.
#include <algorithm>
#include <vector>

#include "common.cuh"

struct fovi_sampler_plan {
  int n_points = 0;
  int device = -1;
  float2* sorted_xy = nullptr;  // [N] grid (x, y) in visiting order
  int* sorted_idx = nullptr;    // [N] original index of each visited point
};

namespace {

struct SampleArgs {
  const void* img;
  void* out;
  const float2* sorted_xy;
  const int* sorted_idx;
  const float* fix_rc;
  const float* fix_hw;
  long long sb, sc, sy, sx;  // image element strides
  int B, C, H, W, F, N;
  int cp;        // channel stride of the points-major layouts (8 = 2 points x 4 channels in pair layout)
  int f_major;   // 1: output row = f*B + b, 0: b*F + f
  int pairs;     // 1: pair layout [ceil(rows/128)][ceil(N/2)][128 rows][2][4]
  int pow2;      // 1: W and H are powers of two, so x / W == x * (1 / W) exactly
};

template <typename TIn, int PAD>
__device__ __forceinline__ float tap(const TIn* plane, long long sy, long long sx, int x, int y, int W, int H) {
  bool ok = (x >= 0) & (x < W) & (y >= 0) & (y < H);
  return ok ? ld_as_float(plane + (long long)y * sy + (long long)x * sx) : 0.f;
}

// NC == false: out row is [C][N];  NC == true: out row is [N][cp] with channels >= C zeroed.
// STAGE: stage the whole output row in shared memory before one coalesced store.
template <typename TIn, typename TOut, int MODE, int PAD, bool NC, bool STAGE>
__global__ void __launch_bounds__(256, 3) fovi_sample_kernel(const SampleArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TOut* stage = reinterpret_cast<TOut*>(smem_raw);

  const int bf = blockIdx.x;  // b*F + f
  const int b = bf / a.F, f = bf - b * a.F;
  const long long row = a.f_major ? ((long long)f * a.B + b) : (long long)bf;
  const int row_elems = NC ? (a.pairs ? ((a.N + 1) / 2) * 8 : a.N * a.cp) : a.C * a.N;
  // pair layout: rows are tiled by 128; this row's 16-byte slot of pair p sits at ((tile*n_pairs + p)*128 + r)*8
  TOut* out_row = reinterpret_cast<TOut*>(a.out) +
                  (a.pairs ? ((row >> 7) * (long long)((a.N + 1) / 2) * 128 + (row & 127)) * 8 : row * row_elems);
  TOut* dst = STAGE ? stage : out_row;

  const float fr = __ldg(a.fix_rc + 2 * bf), fc = __ldg(a.fix_rc + 2 * bf + 1);
  const float fh = __ldg(a.fix_hw + 2 * bf), fw = __ldg(a.fix_hw + 2 * bf + 1);
  const float Wf = (float)a.W, Hf = (float)a.H;
  const float cx = __fmul_rn(fc, Wf), cy = __fmul_rn(fr, Hf);
  const float half_w = __fdiv_rn(fw, 2.f), half_h = __fdiv_rn(fh, 2.f);
  const float sxw = Wf * 0.5f, syh = Hf * 0.5f;  // exact
  const float inv_w = 1.f / Wf, inv_h = 1.f / Hf; // exact when a.pow2 (the only case they are used in)
  const TIn* img_b = reinterpret_cast<const TIn*>(a.img) + (long long)b * a.sb;
  const int pitch = a.pairs ? 4 : a.cp;  // per-point element pitch of the points-major layouts

  if (NC && STAGE) {  // zero the pad channels once
    for (int i = threadIdx.x; i < row_elems; i += blockDim.x) stage[i] = from_float<TOut>(0.f);
    __syncthreads();
  }

#pragma unroll 2
  for (int i = threadIdx.x; i < a.N; i += blockDim.x) {
    const float2 g = __ldg(a.sorted_xy + i);
    const int n = __ldg(a.sorted_idx + i);
    float gx = __fadd_rn(__fmul_rn(g.x, half_w), cx);
    float gy = __fadd_rn(__fmul_rn(g.y, half_h), cy);
    // division by a power of two is a multiplication by its exact reciprocal: same bits, far fewer instructions
    gx = __fsub_rn(a.pow2 ? __fmul_rn(__fmul_rn(2.f, gx), inv_w) : __fdiv_rn(__fmul_rn(2.f, gx), Wf), 1.f);
    gy = __fsub_rn(a.pow2 ? __fmul_rn(__fmul_rn(2.f, gy), inv_h) : __fdiv_rn(__fmul_rn(2.f, gy), Hf), 1.f);
    float ix = __fmaf_rn(__fadd_rn(gx, 1.f), sxw, -0.5f);
    float iy = __fmaf_rn(__fadd_rn(gy, 1.f), syh, -0.5f);
    if (PAD == FOVI_PAD_BORDER) {
      ix = fminf(fmaxf(ix, 0.f), Wf - 1.f);
      iy = fminf(fmaxf(iy, 0.f), Hf - 1.f);
    }
    if (MODE == FOVI_NEAREST) {
      const int x = (int)rintf(ix), y = (int)rintf(iy);
      for (int c = 0; c < a.C; ++c) {
        const float v = tap<TIn, PAD>(img_b + c * a.sc, a.sy, a.sx, x, y, a.W, a.H);
        dst[NC ? (n * pitch + c) : (c * a.N + n)] = from_float<TOut>(v);
      }
    } else {
      const float x0f = floorf(ix), y0f = floorf(iy);
      const float tx = __fsub_rn(ix, x0f), ty = __fsub_rn(iy, y0f);
      const float ux = __fsub_rn(1.f, tx), uy = __fsub_rn(1.f, ty);
      const float w_nw = __fmul_rn(uy, ux), w_ne = __fmul_rn(uy, tx);
      const float w_sw = __fmul_rn(ty, ux), w_se = __fmul_rn(ty, tx);
      const int x0 = (int)x0f, y0 = (int)y0f;
#pragma unroll 3
      for (int c = 0; c < a.C; ++c) {
        const TIn* plane = img_b + c * a.sc;
        const float v_nw = tap<TIn, PAD>(plane, a.sy, a.sx, x0, y0, a.W, a.H);
        const float v_ne = tap<TIn, PAD>(plane, a.sy, a.sx, x0 + 1, y0, a.W, a.H);
        const float v_sw = tap<TIn, PAD>(plane, a.sy, a.sx, x0, y0 + 1, a.W, a.H);
        const float v_se = tap<TIn, PAD>(plane, a.sy, a.sx, x0 + 1, y0 + 1, a.W, a.H);
        float acc = __fmul_rn(v_nw, w_nw);
        acc = __fmaf_rn(v_ne, w_ne, acc);
        acc = __fmaf_rn(v_sw, w_sw, acc);
        acc = __fmaf_rn(v_se, w_se, acc);
        dst[NC ? (n * pitch + c) : (c * a.N + n)] = from_float<TOut>(acc);
      }
    }
    if (NC && !STAGE) {
      for (int c = a.C; c < pitch; ++c) dst[n * pitch + c] = from_float<TOut>(0.f);
    }
  }

  if (STAGE && NC && a.pairs) {
    // pair layout: this row owns one 16-byte slot in each pair's 128-row block of its row tile
    __syncthreads();
    const long long rows = 128;
    const int4* s4 = reinterpret_cast<const int4*>(stage);
    int4* d4 = reinterpret_cast<int4*>(out_row);
    const int n_pairs = (a.N + 1) / 2;
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) d4[(long long)i * rows] = s4[i];
  } else if (STAGE) {
    __syncthreads();
    const size_t bytes = (size_t)row_elems * sizeof(TOut);
    const bool vec = ((reinterpret_cast<uintptr_t>(out_row) & 15) == 0) && (bytes % 16 == 0);
    if (vec) {
      const int4* s4 = reinterpret_cast<const int4*>(stage);
      int4* d4 = reinterpret_cast<int4*>(out_row);
      for (int i = threadIdx.x; i < (int)(bytes / 16); i += blockDim.x) d4[i] = s4[i];
    } else {
      for (int i = threadIdx.x; i < row_elems; i += blockDim.x) out_row[i] = stage[i];
    }
  }
}

template <typename TIn, typename TOut, int MODE, int PAD, bool NC>
int launch_sample(const SampleArgs& a, size_t stage_bytes, cudaStream_t st) {
  const int grid = a.B * a.F;
  if (stage_bytes <= 200 * 1024) {
    auto k = fovi_sample_kernel<TIn, TOut, MODE, PAD, NC, true>;
    if (stage_bytes > 48 * 1024) FOVI_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stage_bytes));
    k<<<grid, 256, stage_bytes, st>>>(a);
  } else {
    if (a.pairs) return FOVI_ERR_UNSUPPORTED;  // the pair layout is only written from the staged row
    fovi_sample_kernel<TIn, TOut, MODE, PAD, NC, false><<<grid, 256, 0, st>>>(a);
  }
  return fovi::after_launch("fovi_sample_kernel");
}

template <typename TIn, typename TOut, int MODE, int PAD>
int dispatch_layout(const SampleArgs& a, bool nc, cudaStream_t st) {
  const size_t stage_bytes = (size_t)(nc ? (a.pairs ? ((a.N + 1) / 2) * 8 : a.N * a.cp) : a.C * a.N) * sizeof(TOut);
  return nc ? launch_sample<TIn, TOut, MODE, PAD, true>(a, stage_bytes, st)
            : launch_sample<TIn, TOut, MODE, PAD, false>(a, stage_bytes, st);
}

template <typename TIn, typename TOut>
int dispatch_mode(const SampleArgs& a, int mode, int pad, bool nc, cudaStream_t st) {
  if (mode == FOVI_NEAREST)
    return pad == FOVI_PAD_ZEROS ? dispatch_layout<TIn, TOut, FOVI_NEAREST, FOVI_PAD_ZEROS>(a, nc, st)
                                 : dispatch_layout<TIn, TOut, FOVI_NEAREST, FOVI_PAD_BORDER>(a, nc, st);
  return pad == FOVI_PAD_ZEROS ? dispatch_layout<TIn, TOut, FOVI_BILINEAR, FOVI_PAD_ZEROS>(a, nc, st)
                               : dispatch_layout<TIn, TOut, FOVI_BILINEAR, FOVI_PAD_BORDER>(a, nc, st);
}

// Interleave the low 16 bits of x and y (Morton / Z-order key).
uint32_t morton16(uint32_t x, uint32_t y) {
  auto spread = [](uint32_t v) {
    v &= 0xFFFF;
    v = (v | (v << 8)) & 0x00FF00FF;
    v = (v | (v << 4)) & 0x0F0F0F0F;
    v = (v | (v << 2)) & 0x33333333;
    v = (v | (v << 1)) & 0x55555555;
    return v;
  };
  return spread(x) | (spread(y) << 1);
}

}  // namespace

extern "C" int fovi_sampler_plan_create(const float* grid_xy, int n_points, fovi_sampler_plan** out) {
  if (!grid_xy || !out || n_points <= 0) return FOVI_ERR_INVALID_ARGUMENT;
  std::vector<std::pair<uint32_t, int>> keys(n_points);
  for (int i = 0; i < n_points; ++i) {
    // Quantise [-1.5, 1.5] to 12 bits per axis; the fixation transform is a positive-scale
    // affine map, so spatial order on the sensor grid is spatial order in the image.
    auto q = [](float v) {
      float t = (std::min(std::max(v, -1.5f), 1.5f) + 1.5f) * (4095.f / 3.f);
      return (uint32_t)t;
    };
    keys[i] = {morton16(q(grid_xy[2 * i]), q(grid_xy[2 * i + 1])), i};
  }
  std::stable_sort(keys.begin(), keys.end());
  std::vector<float2> xy(n_points);
  std::vector<int> idx(n_points);
  for (int i = 0; i < n_points; ++i) {
    idx[i] = keys[i].second;
    xy[i] = make_float2(grid_xy[2 * idx[i]], grid_xy[2 * idx[i] + 1]);
  }
  auto* p = new fovi_sampler_plan();
  p->n_points = n_points;
  cudaError_t e = cudaGetDevice(&p->device);
  if (e == cudaSuccess) e = cudaMalloc(&p->sorted_xy, sizeof(float2) * n_points);
  if (e == cudaSuccess) e = cudaMalloc(&p->sorted_idx, sizeof(int) * n_points);
  if (e == cudaSuccess) e = cudaMemcpy(p->sorted_xy, xy.data(), sizeof(float2) * n_points, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(p->sorted_idx, idx.data(), sizeof(int) * n_points, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    fovi_sampler_plan_destroy(p);
    return fovi::cuda_fail(e, "fovi_sampler_plan_create");
  }
  *out = p;
  return FOVI_OK;
}

extern "C" void fovi_sampler_plan_destroy(fovi_sampler_plan* plan) {
  if (!plan) return;
  if (plan->sorted_xy) cudaFree(plan->sorted_xy);
  if (plan->sorted_idx) cudaFree(plan->sorted_idx);
  delete plan;
}

extern "C" int fovi_sampler_plan_num_points(const fovi_sampler_plan* plan) { return plan ? plan->n_points : -1; }

extern "C" int fovi_sample_forward(const fovi_sampler_plan* plan, const void* img, int dtype, int B, int C, int H, int W,
                                   const int64_t* img_strides, const float* fix_rc, const float* fix_hw, int F, int mode,
                                   int pad, void* out, int out_dtype, int layout, int out_channel_stride, void* stream) {
  if (!plan || !img_strides) return FOVI_ERR_INVALID_ARGUMENT;
  if (B > 0 && (!img || !fix_rc || !fix_hw || !out)) return FOVI_ERR_INVALID_ARGUMENT;
  if (B < 0 || C <= 0 || H <= 0 || W <= 0 || F <= 0) return FOVI_ERR_INVALID_ARGUMENT;
  if (!fovi::valid_dtype(dtype) || !fovi::valid_dtype(out_dtype)) return FOVI_ERR_INVALID_ARGUMENT;
  if (mode != FOVI_NEAREST && mode != FOVI_BILINEAR) return FOVI_ERR_INVALID_ARGUMENT;
  if (pad != FOVI_PAD_ZEROS && pad != FOVI_PAD_BORDER) return FOVI_ERR_INVALID_ARGUMENT;
  if (layout < FOVI_OUT_BFCN || layout > FOVI_OUT_BF_PAIRS) return FOVI_ERR_INVALID_ARGUMENT;
  const bool pairs = layout == FOVI_OUT_FB_PAIRS || layout == FOVI_OUT_BF_PAIRS;
  const bool nc = layout == FOVI_OUT_BFNC || layout == FOVI_OUT_FBNC || pairs;
  if (pairs && (C > 4 || out_dtype != FOVI_BF16)) return FOVI_ERR_UNSUPPORTED;
  if (pairs) out_channel_stride = 8;
  if (pairs && (reinterpret_cast<uintptr_t>(out) & 15)) return FOVI_ERR_ALIGNMENT;
  if (nc && out_channel_stride < C) return FOVI_ERR_INVALID_ARGUMENT;
  if ((long long)H * W >= (1ll << 31) || (long long)plan->n_points * (nc ? out_channel_stride : C) >= (1ll << 31))
    return FOVI_ERR_UNSUPPORTED;
  if (B == 0) return FOVI_OK;
  SampleArgs a;
  a.img = img; a.out = out; a.sorted_xy = plan->sorted_xy; a.sorted_idx = plan->sorted_idx;
  a.fix_rc = fix_rc; a.fix_hw = fix_hw;
  a.sb = img_strides[0]; a.sc = img_strides[1]; a.sy = img_strides[2]; a.sx = img_strides[3];
  a.B = B; a.C = C; a.H = H; a.W = W; a.F = F; a.N = plan->n_points;
  a.cp = nc ? out_channel_stride : C;
  a.f_major = (layout == FOVI_OUT_FBCN || layout == FOVI_OUT_FBNC || layout == FOVI_OUT_FB_PAIRS) ? 1 : 0;
  a.pairs = pairs ? 1 : 0;
  a.pow2 = ((W & (W - 1)) == 0 && (H & (H - 1)) == 0) ? 1 : 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == FOVI_F32 && out_dtype == FOVI_F32) return dispatch_mode<float, float>(a, mode, pad, nc, st);
  if (dtype == FOVI_F32 && out_dtype == FOVI_BF16) return dispatch_mode<float, __nv_bfloat16>(a, mode, pad, nc, st);
  if (dtype == FOVI_BF16 && out_dtype == FOVI_BF16) return dispatch_mode<__nv_bfloat16, __nv_bfloat16>(a, mode, pad, nc, st);
  return dispatch_mode<__nv_bfloat16, float>(a, mode, pad, nc, st);
}
