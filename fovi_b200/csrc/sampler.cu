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
#include <mutex>
#include <type_traits>
#include <stdlib.h>
#include <string.h>
#include <vector>

#include "common.cuh"

constexpr int MAX_TEX = 16;

// Texture objects over one image buffer (see the texture path below), remembered so that a buffer that comes back
// (a pre-allocated input, the slots of a copy pipeline) costs nothing to bind again.
struct TexBinding {
  const void* ptr = nullptr;
  int B = 0, C = 0, H = 0, W = 0, images_per_tex = 0, n_tex = 0;
  cudaTextureObject_t tex[MAX_TEX] = {};
};

struct fovi_sampler_plan {
  int n_points = 0;
  int device = -1;
  float2* sorted_xy = nullptr;  // [N] grid (x, y) in visiting order
  int* sorted_idx = nullptr;    // [N] original index of each visited point
  std::mutex tex_mutex;
  std::vector<TexBinding> tex_cache;   // most recently used last, at most 8
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
  int images_per_tex;                  // texture path: images covered by each texture object
  cudaTextureObject_t tex[MAX_TEX];    // texture path: the image planes as 2-D textures of height images*C*H
};

template <typename TIn, int PAD>
__device__ __forceinline__ float tap(const TIn* plane, long long sy, long long sx, int x, int y, int W, int H) {
  bool ok = (x >= 0) & (x < W) & (y >= 0) & (y < H);
  return ok ? ld_as_float(plane + (long long)y * sy + (long long)x * sx) : 0.f;
}

// NC == false: out row is [C][N];  NC == true: out row is [N][cp] with channels >= C zeroed.
// STAGE: stage the whole output row in shared memory before one coalesced store.
// TEX (float32 contiguous NCHW images, bilinear): the 2x2 footprint of a point in one channel plane is fetched with
// ONE texture gather (tex2Dgather returns the four raw texels a bilinear fetch would blend; the blend itself stays
// in the float32 code below, so results are unchanged bit for bit).  Twelve scattered 4-byte loads per point become
// three gathers on the texture path, which is built for exactly this 2-D footprint; the L1 data pipe that bounds the
// plain-load variant is relieved.  A texture covers the planes of `images_per_tex` images stacked along y, so rows
// outside [0,H) would fall into a neighbouring plane: they are masked here; columns outside [0,W) read 0 through the
// border address mode.
template <typename TIn, typename TOut, int MODE, int PAD, bool NC, bool STAGE, bool TEX = false>
__global__ void __launch_bounds__(256, 3) fovi_sample_kernel(const SampleArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TOut* stage = reinterpret_cast<TOut*>(smem_raw);
  // Programmatic dependent launch: once every CTA of this grid has started, a following kernel launched with the
  // programmatic-serialization attribute (the first KNNConv) may be scheduled onto SMs as they free up and run its
  // prologue; it still waits for this grid's completion before it reads the output.  A no-op otherwise.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

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
      const bool top = y0 >= 0 && y0 < a.H, bot = y0 + 1 >= 0 && y0 + 1 < a.H;
      const cudaTextureObject_t tex = TEX ? a.tex[b / a.images_per_tex] : 0;
      const int plane0 = TEX ? (b % a.images_per_tex) * a.C : 0;
#pragma unroll 3
      for (int c = 0; c < a.C; ++c) {
        float v_nw, v_ne, v_sw, v_se;
        if (TEX) {
          // footprint of (x, y) is texels floor(x-0.5), +1: aim at the middle of the range that selects x0 / y0
          const float4 q = tex2Dgather<float4>(tex, (float)x0 + 1.0f, (float)((plane0 + c) * a.H + y0) + 1.0f, 0);
          v_nw = top ? q.w : 0.f; v_ne = top ? q.z : 0.f; v_sw = bot ? q.x : 0.f; v_se = bot ? q.y : 0.f;
        } else {
          const TIn* plane = img_b + c * a.sc;
          v_nw = tap<TIn, PAD>(plane, a.sy, a.sx, x0, y0, a.W, a.H);
          v_ne = tap<TIn, PAD>(plane, a.sy, a.sx, x0 + 1, y0, a.W, a.H);
          v_sw = tap<TIn, PAD>(plane, a.sy, a.sx, x0, y0 + 1, a.W, a.H);
          v_se = tap<TIn, PAD>(plane, a.sy, a.sx, x0 + 1, y0 + 1, a.W, a.H);
        }
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
  if constexpr (std::is_same<TIn, float>::value && MODE == FOVI_BILINEAR) {
    if (a.images_per_tex > 0 && stage_bytes <= 200 * 1024) {
      auto k = fovi_sample_kernel<TIn, TOut, MODE, PAD, NC, true, true>;
      if (stage_bytes > 48 * 1024) FOVI_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stage_bytes));
      k<<<grid, 256, stage_bytes, st>>>(a);
      return fovi::after_launch("fovi_sample_kernel(tex)");
    }
  }
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

// Binds (or finds) texture objects over a contiguous float32 [B,C,H,W] buffer.  Returns false when the buffer does not
// qualify (alignment, size limits) — the caller then uses the plain-load kernel.
bool bind_textures(fovi_sampler_plan* plan, const void* img, int B, int C, int H, int W, SampleArgs& a) {
  static const bool disabled = getenv("FOVI_B200_NO_TEXTURE") != nullptr;
  if (disabled) return false;
  int dev = 0, max_h = 0, max_w = 0, pitch_align = 0, tex_align = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  cudaDeviceGetAttribute(&max_h, cudaDevAttrMaxTexture2DLinearHeight, dev);
  cudaDeviceGetAttribute(&max_w, cudaDevAttrMaxTexture2DLinearWidth, dev);
  cudaDeviceGetAttribute(&pitch_align, cudaDevAttrTexturePitchAlignment, dev);
  cudaDeviceGetAttribute(&tex_align, cudaDevAttrTextureAlignment, dev);
  if (pitch_align <= 0 || tex_align <= 0) return false;
  const size_t pitch = (size_t)W * 4, image_bytes = (size_t)C * H * pitch;
  const long long rows_per_image = (long long)C * H;
  if (W > max_w || rows_per_image > max_h || pitch % pitch_align || image_bytes % tex_align ||
      (reinterpret_cast<uintptr_t>(img) % tex_align) || rows_per_image * 1 >= (1 << 24))
    return false;
  const int per_tex = (int)std::min<long long>(B, std::min<long long>(max_h, (1 << 24) - 2) / rows_per_image);
  const int n_tex = (B + per_tex - 1) / per_tex;
  if (n_tex > MAX_TEX) return false;
  std::lock_guard<std::mutex> lock(plan->tex_mutex);
  for (size_t i = 0; i < plan->tex_cache.size(); ++i) {
    TexBinding& t = plan->tex_cache[i];
    if (t.ptr == img && t.B == B && t.C == C && t.H == H && t.W == W) {
      a.images_per_tex = t.images_per_tex;
      for (int k = 0; k < t.n_tex; ++k) a.tex[k] = t.tex[k];
      std::rotate(plan->tex_cache.begin() + i, plan->tex_cache.begin() + i + 1, plan->tex_cache.end());
      return true;
    }
  }
  TexBinding t;
  t.ptr = img; t.B = B; t.C = C; t.H = H; t.W = W; t.images_per_tex = per_tex; t.n_tex = n_tex;
  for (int k = 0; k < n_tex; ++k) {
    const int images = std::min(per_tex, B - k * per_tex);
    cudaResourceDesc rd;
    memset(&rd, 0, sizeof(rd));
    rd.resType = cudaResourceTypePitch2D;
    rd.res.pitch2D.devPtr = const_cast<char*>(static_cast<const char*>(img)) + (size_t)k * per_tex * image_bytes;
    rd.res.pitch2D.desc = cudaCreateChannelDesc<float>();
    rd.res.pitch2D.width = W;
    rd.res.pitch2D.height = (size_t)images * rows_per_image;
    rd.res.pitch2D.pitchInBytes = pitch;
    cudaTextureDesc td;
    memset(&td, 0, sizeof(td));
    td.addressMode[0] = td.addressMode[1] = cudaAddressModeBorder;
    td.filterMode = cudaFilterModePoint;
    td.readMode = cudaReadModeElementType;
    td.normalizedCoords = 0;
    if (cudaCreateTextureObject(&t.tex[k], &rd, &td, nullptr) != cudaSuccess) {
      cudaGetLastError();
      for (int j = 0; j < k; ++j) cudaDestroyTextureObject(t.tex[j]);
      return false;
    }
  }
  if (plan->tex_cache.size() >= 8) {
    for (int k = 0; k < plan->tex_cache.front().n_tex; ++k) cudaDestroyTextureObject(plan->tex_cache.front().tex[k]);
    plan->tex_cache.erase(plan->tex_cache.begin());
  }
  plan->tex_cache.push_back(t);
  a.images_per_tex = per_tex;
  for (int k = 0; k < n_tex; ++k) a.tex[k] = t.tex[k];
  return true;
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
  for (auto& t : plan->tex_cache)
    for (int k = 0; k < t.n_tex; ++k) cudaDestroyTextureObject(t.tex[k]);
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
  a.images_per_tex = 0;
  if (dtype == FOVI_F32 && mode == FOVI_BILINEAR && a.sx == 1 && a.sy == W && a.sc == (long long)H * W && a.sb == (long long)C * H * W)
    bind_textures(const_cast<fovi_sampler_plan*>(plan), img, B, C, H, W, a);   // leaves images_per_tex = 0 when not applicable
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == FOVI_F32 && out_dtype == FOVI_F32) return dispatch_mode<float, float>(a, mode, pad, nc, st);
  if (dtype == FOVI_F32 && out_dtype == FOVI_BF16) return dispatch_mode<float, __nv_bfloat16>(a, mode, pad, nc, st);
  if (dtype == FOVI_BF16 && out_dtype == FOVI_BF16) return dispatch_mode<__nv_bfloat16, __nv_bfloat16>(a, mode, pad, nc, st);
  return dispatch_mode<__nv_bfloat16, float>(a, mode, pad, nc, st);
}
