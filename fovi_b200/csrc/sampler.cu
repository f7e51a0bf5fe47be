// Sensor sampler for sm_100a: nearest / bilinear gather of image pixels at the foveated sample
// points, for every fixation of every image in one launch.
//
// Two kernels share one arithmetic core.
//
// fovi_sample_strip_kernel (the fast path: x-contiguous images whose rows are 16-byte aligned, C <= 4).
//   The image, not the output row, is what a CTA holds still.  One CTA owns a horizontal strip of R rows of one
//   image.  It hands the strip (R rows + the next row, all channel planes; for wide images only the columns the
//   fixations of this image can touch) to the TMA unit as one bulk copy per row (cp.async.bulk onto an mbarrier) --
//   whole lines, in address order, every byte of the image fetched from DRAM once -- and then serves ALL
//   fixations of that image from shared memory.  The plan keeps the sensor's points sorted by their grid y with a
//   rank table over y buckets.  The fixation transform is an affine map with positive scale, so the points of one
//   fixation whose 2x2 footprint starts in the strip's rows lie in ONE contiguous range of that order; the range is
//   read off the rank table from the analytically inverted transform (widened by two buckets, far more than float32
//   rounding can move a point) and every point in it is then tested with the exact float32 row it maps to.  Every
//   point therefore has exactly one owning strip, and an owned point's footprint always lies inside the rows the
//   strip loaded; points that fall outside the image above (below) belong to the first (last) strip and read
//   nothing.  The scattered 4-byte gathers that bound a one-row-per-CTA kernel (latency of L1/L2 misses at low
//   occupancy) become shared-memory reads; DRAM sees a plain stream.
//   Outputs go straight to global memory at the points' original indices (8 bytes per point in the pair layout).
//   The one wait (for the copies) is bounded: a strip that gives up sets the plan's status word, read back by
//   fovi_sampler_check, and leaves.
//
// fovi_sample_kernel (any strides, any channel count).  One CTA per (image, fixation) walks the points in Morton
//   order with plain loads and stages the output row in shared memory for one coalesced store.
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
#include <limits.h>
#include <type_traits>
#include <stdlib.h>
#include <string.h>
#include <vector>

#include "common.cuh"

#ifndef FOVI_STRIP_ROWS_MAX
#define FOVI_STRIP_ROWS_MAX 8       // rows a strip owns at most (it loads one more)
#endif
#ifndef FOVI_STRIP_SMEM_BUDGET
#define FOVI_STRIP_SMEM_BUDGET (27 * 1024)   // shared memory per CTA: eight CTAs per SM
#endif
#ifndef FOVI_STRIP_THREADS
#define FOVI_STRIP_THREADS 128
#endif
#ifndef FOVI_STRIP_MIN_CTAS
#define FOVI_STRIP_MIN_CTAS 8
#endif

struct fovi_sampler_plan {
  int n_points = 0;
  int device = -1;
  float2* sorted_xy = nullptr;  // [N] grid (x, y) in Morton order (general kernel)
  int* sorted_idx = nullptr;    // [N] original index of each visited point
  float2* grid_xy = nullptr;    // [N] grid (x, y) in the caller's order (gradient kernel)
  void* ys = nullptr;           // [N] {x, y, original index, 0} sorted by grid y (strip kernel); null: no such order
  float gx_min = 0, gx_max = 0, gy_min = 0, gy_max = 0;
  int* rank_lut = nullptr;      // [4097] rank table over gy buckets (see the strip kernel)
  float lut_scale = 0;
  int* status = nullptr;        // device word: set by a strip kernel whose wait for its copies gave up
};

namespace {

struct __align__(16) YPoint { float x, y; int n; int pad_; };   // one sensor point of the y-sorted order

struct SampleArgs {
  const void* img;
  void* out;
  const float2* sorted_xy;   // visiting order of the kernel that runs (Morton order, or y order for the strip kernel)
  const int* sorted_idx;
  const YPoint* ys;          // y order (null: the plan has none)
  const float* fix_rc;
  const float* fix_hw;
  long long sb, sc, sy, sx;  // image element strides
  int B, C, H, W, F, N;
  int cp;        // channel stride of the points-major layouts (8 = 2 points x 4 channels in pair layout)
  int f_major;   // 1: output row = f*B + b, 0: b*F + f
  int pairs;     // 1: pair layout [ceil(rows/128)][ceil(N/2)][128 rows][2][4]
  int pow2;      // 1: W and H are powers of two, so x / W == x * (1 / W) exactly
  // strip kernel only
  int R, n_strips, pitch;   // rows owned per strip, strips per image, shared-memory row pitch in elements
  int layout;               // LAY_PLANAR / LAY_NC / LAY_PAIRS
  int full_rows;            // 1: rows are short enough to be copied whole, without waiting for the fixations
  const int* rank_lut;      // [RANK_LUT_Q + 1] number of points whose gy falls in a bucket below q
  float lut_scale;          // buckets per unit of gy
  int* status;              // device word set when a strip gave up waiting for its copies
  float gx_min, gx_max, gy_min, gy_max;   // extent of the sensor grid
};

// Grid coordinate -> source pixel coordinate, the reference's operation order (see the file comment).
// Every step is a correctly rounded, monotone non-decreasing function of g when half >= 0.
__device__ __forceinline__ float grid_to_pixel(float g, float half, float centre, float dim, float inv_dim, float half_dim, int pow2) {
  float v = __fadd_rn(__fmul_rn(g, half), centre);
  // division by a power of two is a multiplication by its exact reciprocal: same bits, far fewer instructions
  v = __fsub_rn(pow2 ? __fmul_rn(__fmul_rn(2.f, v), inv_dim) : __fdiv_rn(__fmul_rn(2.f, v), dim), 1.f);
  return __fmaf_rn(__fadd_rn(v, 1.f), half_dim, -0.5f);
}

template <typename TIn, int PAD>
__device__ __forceinline__ float tap(const TIn* plane, long long sy, long long sx, int x, int y, int W, int H) {
  bool ok = (x >= 0) & (x < W) & (y >= 0) & (y < H);
  return ok ? ld_as_float(plane + (long long)y * sy + (long long)x * sx) : 0.f;
}

template <typename T> __device__ __forceinline__ float smem_as_float(const T* p);
template <> __device__ __forceinline__ float smem_as_float<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float smem_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float smem_as_float<unsigned char>(const unsigned char* p) { return (float)*p; }

// ------------------------------------------------------------------------------------------------------------
// Strip kernel.
// ------------------------------------------------------------------------------------------------------------
constexpr int STRIP_THREADS = FOVI_STRIP_THREADS;
constexpr int FCHUNK = 16;        // fixations served per pass over the strip
constexpr int RANK_LUT_Q = 4096;  // buckets of the plan's rank table over [gy_min, gy_max]
constexpr uint32_t STRIP_WAIT_LIMIT = 1u << 22;   // mbarrier polls before the kernel gives up on its copies
enum { LAY_PLANAR = 0, LAY_NC = 1, LAY_PAIRS = 2 };

struct __align__(16) FixInfo {
  float cx, cy, half_w, half_h;
  long long out_off;   // element offset of this (image, fixation) row in the output
  int lo, hi;          // range of y-sorted points that contains every point this strip owns
};

__device__ __forceinline__ uint32_t s_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void s_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void s_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool s_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Contiguous global -> shared bulk copy by the TMA unit (both addresses 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void s_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Row key of a point: the first image row its footprint reads (bilinear) or the row it reads (nearest).
template <int MODE, int PAD>
__device__ __forceinline__ int row_key(float iy, float Hf) {
  if (PAD == FOVI_PAD_BORDER) iy = fminf(fmaxf(iy, 0.f), Hf - 1.f);
  return MODE == FOVI_NEAREST ? (int)rintf(iy) : (int)floorf(iy);
}

// Shared-memory tile of a strip: per channel plane, (R+1) rows of `pitch` = W + EPV elements; the EPV elements after
// every row (and before the first row of the first plane) hold zeros.  Column -1 / -2 of a row is the tail of the row
// before it and columns W, W+1 its own tail, so a footprint that sticks out of the image to the left or right reads
// zeros without any test: the x index is only clamped to [-2, W].  Rows outside the image exist only for points of
// the first and the last strip; those strips run the YCHECK variant, which masks the rows instead.
//
// A sensor point is handled in three straight-line steps -- transform (with the exact ownership test: the candidate
// ranges are supersets), gather + blend from the tile, store -- and a thread carries PU points through each step
// together, so that their independent instruction chains interleave (the work per point is one long dependent
// chain; with the few warps that the tile's shared memory leaves room for, issue slots would otherwise stay empty).
// Points that turn out to be another strip's are computed from clamped, valid tile addresses and simply not stored.
// NCH: channel count known at compile time (3), or 0: read a.C.
struct PointState {
  float w_nw, w_ne, w_sw, w_se;   // bilinear weights (nearest: unused)
  int off_t, off_b;               // tile element offsets of the footprint's upper-left pixel and of the one below it
  int n;                          // original index of the point
  bool own, top, bot;             // this strip's point; rows of the footprint inside the image (YCHECK strips)
};

template <int MODE, int PAD, bool YCHECK>
__device__ __forceinline__ PointState strip_prepare(const SampleArgs& a, const float4 pt, const float4 k /* cx, cy, half_w, half_h */,
                                                    const int r0, const int nrows, const int klo, const int khi) {
  const float Wf = (float)a.W, Hf = (float)a.H;
  const float sxw = Wf * 0.5f, syh = Hf * 0.5f;   // exact
  const float inv_w = 1.f / Wf, inv_h = 1.f / Hf; // exact when a.pow2 (the only case they are used in)
  PointState p;
  p.n = __float_as_int(pt.z);
  float ix = grid_to_pixel(pt.x, k.z, k.x, Wf, inv_w, sxw, a.pow2);
  float iy = grid_to_pixel(pt.y, k.w, k.y, Hf, inv_h, syh, a.pow2);
  if (PAD == FOVI_PAD_BORDER) {
    ix = fminf(fmaxf(ix, 0.f), Wf - 1.f);
    iy = fminf(fmaxf(iy, 0.f), Hf - 1.f);
  }
  int x, y;
  if (MODE == FOVI_NEAREST) {
    x = (int)rintf(ix); y = (int)rintf(iy);
    p.w_nw = p.w_ne = p.w_sw = p.w_se = 0.f;
  } else {
    const float x0f = floorf(ix), y0f = floorf(iy);
    x = (int)x0f; y = (int)y0f;
    const float tx = __fsub_rn(ix, x0f), ty = __fsub_rn(iy, y0f);
    const float ux = __fsub_rn(1.f, tx), uy = __fsub_rn(1.f, ty);
    p.w_nw = __fmul_rn(uy, ux); p.w_ne = __fmul_rn(uy, tx);
    p.w_sw = __fmul_rn(ty, ux); p.w_se = __fmul_rn(ty, tx);
  }
  p.own = (y >= klo) & (y < khi);
  const int ry = y - r0;
  const int xc = min(max(x, -2), a.W);
  // rows are clamped into the tile: a no-op for the strip's own points (of a YCHECK strip: for their rows inside the image)
  const int last_row = YCHECK ? nrows - 1 : nrows - 2;
  p.off_t = min(max(ry, 0), last_row) * a.pitch + xc;
  p.off_b = YCHECK ? min(max(ry + 1, 0), last_row) * a.pitch + xc : p.off_t + a.pitch;
  p.top = (y >= 0) & (y < a.H);
  p.bot = (y + 1 >= 0) & (y + 1 < a.H);
  return p;
}

template <typename TIn, int MODE, int NCH, bool YCHECK>
__device__ __forceinline__ void strip_gather(const SampleArgs& a, const PointState& p, const TIn* __restrict__ tile, float (&v)[4]) {
  const int plane = (a.R + 1) * a.pitch;
  const int C = NCH ? NCH : a.C;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    v[c] = 0.f;
    if (c < C) {
      const TIn* pt_ = tile + c * plane + p.off_t;
      if (MODE == FOVI_NEAREST) {
        const float t = smem_as_float(pt_);
        v[c] = (YCHECK && !p.top) ? 0.f : t;
      } else {
        const TIn* pb_ = tile + c * plane + p.off_b;
        float v_nw = smem_as_float(pt_), v_ne = smem_as_float(pt_ + 1);
        float v_sw = smem_as_float(pb_), v_se = smem_as_float(pb_ + 1);
        if (YCHECK) {
          v_nw = p.top ? v_nw : 0.f; v_ne = p.top ? v_ne : 0.f;
          v_sw = p.bot ? v_sw : 0.f; v_se = p.bot ? v_se : 0.f;
        }
        float acc = __fmul_rn(v_nw, p.w_nw);
        acc = __fmaf_rn(v_ne, p.w_ne, acc);
        acc = __fmaf_rn(v_sw, p.w_sw, acc);
        acc = __fmaf_rn(v_se, p.w_se, acc);
        v[c] = acc;
      }
    }
  }
}

template <typename TOut, int NCH>
__device__ __forceinline__ void strip_store(const SampleArgs& a, const int n, const float (&v)[4], TOut* __restrict__ out) {
  const int C = NCH ? NCH : a.C;
  if (a.layout == LAY_PAIRS) {
    if constexpr (sizeof(TOut) == 2) {
      // 8 bytes per point: this row's 16-byte slot of pair n/2, half n&1
      __nv_bfloat162 h01 = __floats2bfloat162_rn(v[0], v[1]), h23 = __floats2bfloat162_rn(v[2], v[3]);
      uint2 w;
      w.x = *reinterpret_cast<uint32_t*>(&h01); w.y = *reinterpret_cast<uint32_t*>(&h23);
      uint2* d = reinterpret_cast<uint2*>(out + (long long)(n >> 1) * 1024 + (n & 1) * 4);
      *d = w;
      if ((a.N & 1) && n == a.N - 1) d[1] = make_uint2(0u, 0u);   // the odd last point's empty partner
    }
  } else if (a.layout == LAY_NC) {
    TOut* d = out + (long long)n * a.cp;
    if (sizeof(TOut) == 2 && a.cp == 4 && ((reinterpret_cast<uintptr_t>(a.out) & 7) == 0)) {
      __nv_bfloat162 h01 = __floats2bfloat162_rn(v[0], v[1]), h23 = __floats2bfloat162_rn(v[2], v[3]);
      uint2 w;
      w.x = *reinterpret_cast<uint32_t*>(&h01); w.y = *reinterpret_cast<uint32_t*>(&h23);
      *reinterpret_cast<uint2*>(d) = w;
    } else if (sizeof(TOut) == 4 && a.cp == 4 && ((reinterpret_cast<uintptr_t>(a.out) & 15) == 0)) {
      *reinterpret_cast<float4*>(d) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c < a.cp) d[c] = from_float<TOut>(v[c]);
      for (int c = 4; c < a.cp; ++c) d[c] = from_float<TOut>(0.f);
    }
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c)
      if (c < C) out[(long long)c * a.N + n] = from_float<TOut>(v[c]);
  }
}

// The candidate points of all fixations are flattened into one index range so that every thread has work.
#ifndef FOVI_STRIP_UNROLL
#define FOVI_STRIP_UNROLL 1
#endif
template <typename TIn, typename TOut, int MODE, int PAD, int NCH, bool YCHECK>
__device__ __forceinline__ void strip_points(const SampleArgs& a, const FixInfo* fi, const int* s_pre, const int nf, const TIn* tile,
                                             const int r0, const int nrows, const bool first, const bool last) {
  constexpr int PU = FOVI_STRIP_UNROLL;
  const int total = s_pre[nf];
  const int klo = first ? INT_MIN : r0, khi = last ? INT_MAX : r0 + a.R;
  int f = 0;
  for (int j0 = threadIdx.x; j0 < total; j0 += PU * STRIP_THREADS) {
    float4 pt[PU];
    int fu[PU];
#pragma unroll
    for (int u = 0; u < PU; ++u) {
      const int j = min(j0 + u * STRIP_THREADS, total - 1);   // past the end: the last point again, not stored
      while (j >= s_pre[f + 1]) ++f;
      fu[u] = f;
      pt[u] = __ldg(reinterpret_cast<const float4*>(a.ys + (fi[f].lo - s_pre[f] + j)));
    }
    PointState ps[PU];
#pragma unroll
    for (int u = 0; u < PU; ++u) {
      ps[u] = strip_prepare<MODE, PAD, YCHECK>(a, pt[u], *reinterpret_cast<const float4*>(fi + fu[u]), r0, nrows, klo, khi);
      ps[u].own = ps[u].own && (j0 + u * STRIP_THREADS < total);
    }
    float v[PU][4];
#pragma unroll
    for (int u = 0; u < PU; ++u) strip_gather<TIn, MODE, NCH, YCHECK>(a, ps[u], tile, v[u]);
#pragma unroll
    for (int u = 0; u < PU; ++u)
      if (ps[u].own) strip_store<TOut, NCH>(a, ps[u].n, v[u], reinterpret_cast<TOut*>(a.out) + fi[fu[u]].out_off);
  }
}

template <typename TIn, typename TOut, int MODE, int PAD>
__global__ void __launch_bounds__(STRIP_THREADS, FOVI_STRIP_MIN_CTAS) fovi_sample_strip_kernel(const SampleArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int EPV = 16 / (int)sizeof(TIn);      // elements per 16 bytes
  TIn* tile = reinterpret_cast<TIn*>(smem_raw) + EPV;   // [C][R+1][pitch], 16 bytes of zeros in front
  __shared__ FixInfo fi[FCHUNK];
  __shared__ int s_pre[FCHUNK + 1];
  __shared__ int s_need, s_col_lo, s_col_hi;
  __shared__ __align__(8) unsigned long long s_bar;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // see fovi_sample_kernel

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int s = blockIdx.x, b = blockIdx.y + blockIdx.z * 65535;   // strip, image
  if (b >= a.B) return;
  const int r0 = s * a.R;
  const int nrows = min(a.H - r0, a.R + 1);
  const bool first = s == 0, last = s == a.n_strips - 1;
  const float Wf = (float)a.W, Hf = (float)a.H;
  const float sxw = Wf * 0.5f, syh = Hf * 0.5f;
  const float inv_w = 1.f / Wf, inv_h = 1.f / Hf;
  const TIn* img_b = reinterpret_cast<const TIn*>(a.img) + (long long)b * a.sb;
  const int plane = (a.R + 1) * a.pitch;          // elements per channel plane in shared memory
  const int n_pairs = (a.N + 1) / 2;
  const uint32_t bar = s_addr(&s_bar);
  uint32_t bar_phase = 0;
  bool loaded = false, gave_up = false;

  // One warp hands the strip's rows to the TMA unit, one bulk copy per (channel, row), columns [col_lo, col_hi).
  auto issue_rows = [&](int col_lo, int col_hi) {
    const uint32_t row_bytes = (uint32_t)(col_hi - col_lo) * (uint32_t)sizeof(TIn);
    const int rows = a.C * nrows;
    if (lane == 0) s_mbar_expect_tx(bar, row_bytes * (uint32_t)rows);
    __syncwarp();
    for (int rid = lane; rid < rows; rid += 32) {
      const int c = rid / nrows, r = rid - c * nrows;
      s_bulk_load(s_addr(tile + c * plane + r * a.pitch + col_lo), img_b + c * a.sc + (long long)(r0 + r) * a.sy + col_lo, row_bytes, bar);
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      s_mbar_init(bar, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // Narrow images: whole rows, at once, before anything is known about the fixations (a strip none of them touches
    // is rare, and waiting for the fixations first would put a global-memory round trip in front of the copies).
    if (a.full_rows) { issue_rows(0, a.W); }
  }
  loaded = a.full_rows != 0;
  // the zero tails (see strip_point); the copies never touch them
  if (tid <= a.C * (a.R + 1)) {
    int4* z = tid == 0 ? reinterpret_cast<int4*>(smem_raw)
                       : reinterpret_cast<int4*>(tile + (tid - 1) * a.pitch + a.W);
    *z = make_int4(0, 0, 0, 0);
  }

  for (int f0 = 0; f0 < a.F; f0 += FCHUNK) {
    const int nf = min(FCHUNK, a.F - f0);
    if (f0 > 0 || !a.full_rows) {
      // (Not on the first pass over whole rows: warp 1 then computes the ranges while warp 0 is still handing rows to
      // the copy unit, and the barrier is only ever touched by warp 0.)
      if (tid == 0) { s_need = 0; s_col_lo = INT_MAX; s_col_hi = INT_MIN; }
      __syncthreads();   // also: the previous pass has finished reading the tile and the range table
    }

    // ---- per-fixation constants and candidate range, one thread per fixation.
    // The source row of a point is iy = gy * half_h + cy - 0.5 up to rounding, so the points whose row key lies in
    // [r0, r0 + R) have gy in [(r0 + 0.5 - cy) / half_h, (r0 + R + 0.5 - cy) / half_h); the plan's rank table turns
    // that interval, widened by two buckets on either side (far more than the rounding of the float32 transform can
    // move a point), into a range of the y-sorted order.  Every point of the range is tested exactly later on, so the
    // range only has to be a superset.
    const int ft = tid - (STRIP_THREADS > 32 ? 32 : 0);   // warp 1 when there is one: warp 0 is busy issuing the copies
    if (ft >= 0 && ft < nf) {
      const int f = f0 + ft, bf = b * a.F + f;
      const float fr = __ldg(a.fix_rc + 2 * bf), fc = __ldg(a.fix_rc + 2 * bf + 1);
      const float fh = __ldg(a.fix_hw + 2 * bf), fw = __ldg(a.fix_hw + 2 * bf + 1);
      FixInfo q;
      q.cx = __fmul_rn(fc, Wf); q.cy = __fmul_rn(fr, Hf);
      q.half_w = __fdiv_rn(fw, 2.f); q.half_h = __fdiv_rn(fh, 2.f);
      const long long row = a.f_major ? ((long long)f * a.B + b) : (long long)bf;
      q.out_off = a.layout == LAY_PAIRS ? ((row >> 7) * (long long)n_pairs * 128 + (row & 127)) * 8
                : a.layout == LAY_NC    ? row * (long long)a.N * a.cp
                                        : row * (long long)a.C * a.N;
      q.lo = 0; q.hi = a.N;
      // usable inverse: a positive scale that is neither tiny next to the image (the transform's rounding error, a few
      // 1e-8 * H pixels, must stay far below a bucket: 5e-4 grid units = 5e-4 * half_h pixels) nor huge, and a centre of
      // moderate size relative to it; anything else keeps the full range
      const bool invertible = (q.half_h * 1024.f >= Hf) && (q.half_h < 1e6f) && (fabsf(q.cy) <= 256.f * q.half_h);
      if (invertible && a.rank_lut) {
        const float off = MODE == FOVI_NEAREST ? 0.f : 0.5f;   // nearest: key = rint(iy) >= r  <=>  iy >= r - 0.5
        const float inv = 1.f / q.half_h;
        const float g_lo = ((float)r0 + off - q.cy) * inv, g_hi = ((float)(r0 + a.R) + off - q.cy) * inv;
        const float qlo = floorf((g_lo - a.gy_min) * a.lut_scale), qhi = floorf((g_hi - a.gy_min) * a.lut_scale);
        const int b_lo = (int)fminf(fmaxf(qlo - 2.f, 0.f), (float)RANK_LUT_Q);
        const int b_hi = (int)fminf(fmaxf(qhi + 3.f, 0.f), (float)RANK_LUT_Q);
        if (!first) q.lo = __ldg(a.rank_lut + b_lo);
        if (!last) q.hi = __ldg(a.rank_lut + b_hi);
      }
      if (!a.full_rows) {
        // wide images: which rows / columns of the image can this fixation touch at all?
        const float ya = grid_to_pixel(a.gy_min, q.half_h, q.cy, Hf, inv_h, syh, a.pow2);
        const float yb = grid_to_pixel(a.gy_max, q.half_h, q.cy, Hf, inv_h, syh, a.pow2);
        const float xa = grid_to_pixel(a.gx_min, q.half_w, q.cx, Wf, inv_w, sxw, a.pow2);
        const float xb = grid_to_pixel(a.gx_max, q.half_w, q.cx, Wf, inv_w, sxw, a.pow2);
        const bool sane = (ya == ya) && (yb == yb) && (xa == xa) && (xb == xb);
        int need = 1, c_lo = 0, c_hi = a.W - 1;
        if (sane) {
          const int ext = MODE == FOVI_BILINEAR ? 1 : 0;
          const int ky0 = row_key<MODE, PAD>(fminf(ya, yb), Hf), ky1 = row_key<MODE, PAD>(fmaxf(ya, yb), Hf) + ext;
          need = (ky1 >= r0) && (ky0 < r0 + nrows);
          float x0 = fminf(xa, xb), x1 = fmaxf(xa, xb);
          if (PAD == FOVI_PAD_BORDER) { x0 = fminf(fmaxf(x0, 0.f), Wf - 1.f); x1 = fminf(fmaxf(x1, 0.f), Wf - 1.f); }
          c_lo = MODE == FOVI_NEAREST ? (int)rintf(x0) : (int)floorf(x0);
          c_hi = (MODE == FOVI_NEAREST ? (int)rintf(x1) : (int)floorf(x1)) + ext;
          need = need && (c_hi >= 0) && (c_lo < a.W);
        }
        if (need) { atomicOr(&s_need, 1); atomicMin(&s_col_lo, c_lo); atomicMax(&s_col_hi, c_hi); }
      }
      fi[ft] = q;
    }
    __syncthreads();

    if (!a.full_rows) {
      loaded = s_need != 0;
      if (loaded && warp == 0) {
        const int col_lo = (max(s_col_lo, 0) / EPV) * EPV;
        const int col_hi = min(a.W, ((min(s_col_hi, a.W - 1) + EPV) / EPV) * EPV);   // exclusive; W is a multiple of EPV
        issue_rows(col_lo, col_hi);
      }
    }
    if (tid == 0) {
      int acc = 0;
      for (int f = 0; f < nf; ++f) { s_pre[f] = acc; acc += max(fi[f].hi - fi[f].lo, 0); }
      s_pre[nf] = acc;
    }
    if (loaded && (f0 == 0 || !a.full_rows)) {
      // one thread watches the barrier (bounded); the CTA barrier below passes what it saw on to the others
      if (tid == 0) {
        bool done = false;
        for (uint32_t it = 0; it < STRIP_WAIT_LIMIT && !done; ++it) done = s_mbar_try_wait(bar, bar_phase);
        if (!done) gave_up = true;
      }
      bar_phase ^= 1u;
    }
    gave_up = __syncthreads_or(gave_up ? 1 : 0) != 0;
    if (gave_up) {
      // The copies did not complete in time: record it for fovi_sampler_check, give copies still in flight a bounded
      // time to land (the barrier would complete then), and leave without touching the tile.
      if (tid == 0) {
        if (a.status) atomicExch(a.status, 1);
        for (uint32_t it = 0; it < (1u << 16); ++it)
          if (s_mbar_try_wait(bar, bar_phase ^ 1u)) break;
      }
      return;
    }

    const bool ycheck = first || last;
    if (a.C == 3) {
      if (ycheck) strip_points<TIn, TOut, MODE, PAD, 3, true>(a, fi, s_pre, nf, tile, r0, nrows, first, last);
      else strip_points<TIn, TOut, MODE, PAD, 3, false>(a, fi, s_pre, nf, tile, r0, nrows, first, last);
    } else {
      if (ycheck) strip_points<TIn, TOut, MODE, PAD, 0, true>(a, fi, s_pre, nf, tile, r0, nrows, first, last);
      else strip_points<TIn, TOut, MODE, PAD, 0, false>(a, fi, s_pre, nf, tile, r0, nrows, first, last);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// General kernel.
// NC == false: out row is [C][N];  NC == true: out row is [N][cp] with channels >= C zeroed.
// STAGE: stage the whole output row in shared memory before one coalesced store.
// ------------------------------------------------------------------------------------------------------------
template <typename TIn, typename TOut, int MODE, int PAD, bool NC, bool STAGE>
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
    float ix = grid_to_pixel(g.x, half_w, cx, Wf, inv_w, sxw, a.pow2);
    float iy = grid_to_pixel(g.y, half_h, cy, Hf, inv_h, syh, a.pow2);
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

// ------------------------------------------------------------------------------------------------------------
// Gradient with respect to the image (what autograd through F.grid_sample gives the reference, samplers.py:108): every
// output gradient is scattered onto the taps of its footprint with the forward's weights.  One thread per
// (image, fixation, point); float32 atomics into a zero-initialised (or accumulating) gradient image.
// ------------------------------------------------------------------------------------------------------------
template <typename TG, int MODE, int PAD>
__global__ void __launch_bounds__(256) fovi_sample_backward_kernel(const SampleArgs a, const TG* __restrict__ gout, float* __restrict__ gimg) {
  const long long total = (long long)a.B * a.F * a.N;
  const float Wf = (float)a.W, Hf = (float)a.H;
  const float sxw = Wf * 0.5f, syh = Hf * 0.5f, inv_w = 1.f / Wf, inv_h = 1.f / Hf;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(e % a.N);
    const int bf = (int)(e / a.N);
    const int b = bf / a.F, f = bf - b * a.F;
    const float fr = __ldg(a.fix_rc + 2 * bf), fc = __ldg(a.fix_rc + 2 * bf + 1);
    const float fh = __ldg(a.fix_hw + 2 * bf), fw = __ldg(a.fix_hw + 2 * bf + 1);
    const float2 g = __ldg(a.sorted_xy + n);      // here: the grid in its ORIGINAL order
    float ix = grid_to_pixel(g.x, __fdiv_rn(fw, 2.f), __fmul_rn(fc, Wf), Wf, inv_w, sxw, a.pow2);
    float iy = grid_to_pixel(g.y, __fdiv_rn(fh, 2.f), __fmul_rn(fr, Hf), Hf, inv_h, syh, a.pow2);
    if (PAD == FOVI_PAD_BORDER) {
      ix = fminf(fmaxf(ix, 0.f), Wf - 1.f);
      iy = fminf(fmaxf(iy, 0.f), Hf - 1.f);
    }
    const long long row = a.f_major ? ((long long)f * a.B + b) : (long long)bf;
    const TG* go = gout + row * (long long)a.C * a.N + n;
    float* gi = gimg + (long long)b * a.C * a.H * a.W;
    if (MODE == FOVI_NEAREST) {
      const int x = (int)rintf(ix), y = (int)rintf(iy);
      if (x < 0 || x >= a.W || y < 0 || y >= a.H) continue;
      for (int c = 0; c < a.C; ++c) atomicAdd(gi + ((long long)c * a.H + y) * a.W + x, ld_as_float(go + (long long)c * a.N));
    } else {
      const float x0f = floorf(ix), y0f = floorf(iy);
      const float tx = __fsub_rn(ix, x0f), ty = __fsub_rn(iy, y0f);
      const float ux = __fsub_rn(1.f, tx), uy = __fsub_rn(1.f, ty);
      const float w4[4] = {__fmul_rn(uy, ux), __fmul_rn(uy, tx), __fmul_rn(ty, ux), __fmul_rn(ty, tx)};
      const int x0 = (int)x0f, y0 = (int)y0f;
      for (int c = 0; c < a.C; ++c) {
        const float gv = ld_as_float(go + (long long)c * a.N);
        float* plane = gi + (long long)c * a.H * a.W;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int x = x0 + (t & 1), y = y0 + (t >> 1);
          if (x >= 0 && x < a.W && y >= 0 && y < a.H) atomicAdd(plane + (long long)y * a.W + x, gv * w4[t]);
        }
      }
    }
  }
}

// Does the strip kernel apply?  Fills R, n_strips, pitch.
template <typename TIn>
bool plan_strips(SampleArgs& a, bool nc) {
  constexpr int EPV = 16 / (int)sizeof(TIn);
  if (a.C > 4 || a.sx != 1 || !a.ys) return false;
  if (nc && !a.pairs && a.cp < a.C) return false;
  if ((a.W % EPV) || (a.sy % EPV) || (a.sc % EPV) || (a.sb % EPV) || (reinterpret_cast<uintptr_t>(a.img) & 15)) return false;
  a.pitch = a.W + EPV;   // one 16-byte piece of padding: vertically adjacent pixels fall in different banks
  const long long row_bytes = (long long)a.C * a.pitch * sizeof(TIn);
  const int rows_fit = (int)std::min<long long>((FOVI_STRIP_SMEM_BUDGET - 16) / row_bytes, 1 << 20);
  a.R = std::min(std::min(rows_fit - 1, FOVI_STRIP_ROWS_MAX), a.H);
  if (a.R < 4) return false;   // very wide rows: the extra row per strip would dominate
  a.n_strips = (a.H + a.R - 1) / a.R;
  a.full_rows = (size_t)a.W * sizeof(TIn) <= 4096 ? 1 : 0;
  return (long long)a.B * a.n_strips < (1ll << 31);
}

template <typename TIn, typename TOut, int MODE, int PAD, bool NC>
int launch_sample(SampleArgs a, size_t stage_bytes, cudaStream_t st) {
  if (plan_strips<TIn>(a, NC) && (!a.pairs || std::is_same<TOut, __nv_bfloat16>::value)) {
    const size_t smem = 16 + (size_t)a.C * (a.R + 1) * a.pitch * sizeof(TIn);
    const dim3 grid(a.n_strips, std::min(a.B, 65535), (a.B + 65534) / 65535);   // strips of one image are neighbours
    a.layout = a.pairs ? LAY_PAIRS : (NC ? LAY_NC : LAY_PLANAR);
    auto k = fovi_sample_strip_kernel<TIn, TOut, MODE, PAD>;
    FOVI_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k<<<grid, STRIP_THREADS, smem, st>>>(a);
    return fovi::after_launch("fovi_sample_strip_kernel");
  }
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
  std::vector<YPoint> ypts(n_points);
  std::vector<int> idx(n_points), yidx(n_points);
  for (int i = 0; i < n_points; ++i) {
    idx[i] = keys[i].second;
    xy[i] = make_float2(grid_xy[2 * idx[i]], grid_xy[2 * idx[i] + 1]);
  }
  // second order: by grid y (ties by x, then index), for the strip kernel's range search
  for (int i = 0; i < n_points; ++i) yidx[i] = i;
  std::stable_sort(yidx.begin(), yidx.end(), [&](int p, int q) {
    const float yp = grid_xy[2 * p + 1], yq = grid_xy[2 * q + 1];
    if (yp != yq) return yp < yq;
    return grid_xy[2 * p] < grid_xy[2 * q];
  });
  auto* p = new fovi_sampler_plan();
  p->n_points = n_points;
  p->gx_min = p->gx_max = grid_xy[0];
  p->gy_min = p->gy_max = grid_xy[1];
  bool finite = true;
  for (int i = 0; i < n_points; ++i) {
    const float x = grid_xy[2 * i], y = grid_xy[2 * i + 1];
    ypts[i] = YPoint{grid_xy[2 * yidx[i]], grid_xy[2 * yidx[i] + 1], yidx[i], 0};
    finite = finite && (x - x == 0.f) && (y - y == 0.f);
    p->gx_min = std::min(p->gx_min, x); p->gx_max = std::max(p->gx_max, x);
    p->gy_min = std::min(p->gy_min, y); p->gy_max = std::max(p->gy_max, y);
  }
  cudaError_t e = cudaGetDevice(&p->device);
  if (e == cudaSuccess) e = cudaMalloc(&p->sorted_xy, sizeof(float2) * n_points);
  if (e == cudaSuccess) e = cudaMalloc(&p->sorted_idx, sizeof(int) * n_points);
  if (e == cudaSuccess) e = cudaMemcpy(p->sorted_xy, xy.data(), sizeof(float2) * n_points, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(p->sorted_idx, idx.data(), sizeof(int) * n_points, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMalloc(&p->grid_xy, sizeof(float2) * n_points);
  if (e == cudaSuccess) e = cudaMemcpy(p->grid_xy, grid_xy, sizeof(float2) * n_points, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMalloc(&p->status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(p->status, 0, sizeof(int));
  if (e == cudaSuccess && finite) {
    // rank table: lut[q] = number of points whose bucket floor((gy - gy_min) * scale) is below q
    const float span = p->gy_max - p->gy_min;
    p->lut_scale = span > 0.f ? (float)RANK_LUT_Q / span : 0.f;
    std::vector<int> lut(RANK_LUT_Q + 1, 0);
    for (int i = 0; i < n_points; ++i) {
      const float t = floorf((grid_xy[2 * i + 1] - p->gy_min) * p->lut_scale);
      const int q = (int)std::min(std::max(t, 0.f), (float)(RANK_LUT_Q - 1));
      lut[q + 1] += 1;
    }
    for (int q = 0; q < RANK_LUT_Q; ++q) lut[q + 1] += lut[q];
    e = cudaMalloc(&p->rank_lut, sizeof(int) * lut.size());
    if (e == cudaSuccess) e = cudaMemcpy(p->rank_lut, lut.data(), sizeof(int) * lut.size(), cudaMemcpyHostToDevice);
  }
  if (e == cudaSuccess && finite) {   // a grid with NaN / Inf entries has no y order: the general kernel serves it
    e = cudaMalloc(&p->ys, sizeof(YPoint) * n_points);
    if (e == cudaSuccess) e = cudaMemcpy(p->ys, ypts.data(), sizeof(YPoint) * n_points, cudaMemcpyHostToDevice);
  }
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
  if (plan->ys) cudaFree(plan->ys);
  if (plan->grid_xy) cudaFree(plan->grid_xy);
  if (plan->rank_lut) cudaFree(plan->rank_lut);
  if (plan->status) cudaFree(plan->status);
  delete plan;
}

extern "C" int fovi_sampler_plan_num_points(const fovi_sampler_plan* plan) { return plan ? plan->n_points : -1; }

extern "C" int fovi_sample_forward(const fovi_sampler_plan* plan, const void* img, int dtype, int B, int C, int H, int W,
                                   const int64_t* img_strides, const float* fix_rc, const float* fix_hw, int F, int mode,
                                   int pad, void* out, int out_dtype, int layout, int out_channel_stride, void* stream) {
  if (!plan || !img_strides) return FOVI_ERR_INVALID_ARGUMENT;
  if (B > 0 && (!img || !fix_rc || !fix_hw || !out)) return FOVI_ERR_INVALID_ARGUMENT;
  if (B < 0 || C <= 0 || H <= 0 || W <= 0 || F <= 0) return FOVI_ERR_INVALID_ARGUMENT;
  if ((!fovi::valid_dtype(dtype) && dtype != FOVI_U8) || !fovi::valid_dtype(out_dtype)) return FOVI_ERR_INVALID_ARGUMENT;
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
  a.ys = static_cast<const YPoint*>(plan->ys);
  a.gx_min = plan->gx_min; a.gx_max = plan->gx_max; a.gy_min = plan->gy_min; a.gy_max = plan->gy_max;
  a.R = a.n_strips = a.pitch = a.layout = a.full_rows = 0;
  a.rank_lut = plan->rank_lut; a.lut_scale = plan->lut_scale; a.status = plan->status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == FOVI_U8 && out_dtype == FOVI_F32) return dispatch_mode<unsigned char, float>(a, mode, pad, nc, st);
  if (dtype == FOVI_U8) return dispatch_mode<unsigned char, __nv_bfloat16>(a, mode, pad, nc, st);
  if (dtype == FOVI_F32 && out_dtype == FOVI_F32) return dispatch_mode<float, float>(a, mode, pad, nc, st);
  if (dtype == FOVI_F32 && out_dtype == FOVI_BF16) return dispatch_mode<float, __nv_bfloat16>(a, mode, pad, nc, st);
  if (dtype == FOVI_BF16 && out_dtype == FOVI_BF16) return dispatch_mode<__nv_bfloat16, __nv_bfloat16>(a, mode, pad, nc, st);
  return dispatch_mode<__nv_bfloat16, float>(a, mode, pad, nc, st);
}


extern "C" int fovi_sampler_check(fovi_sampler_plan* plan, void* stream) {
  if (!plan) return FOVI_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int h = 0;
  FOVI_CUDA(cudaMemcpyAsync(&h, plan->status, sizeof(int), cudaMemcpyDeviceToHost, st));
  FOVI_CUDA(cudaStreamSynchronize(st));
  if (h != 0) {
    FOVI_CUDA(cudaMemsetAsync(plan->status, 0, sizeof(int), st));
    FOVI_CUDA(cudaStreamSynchronize(st));
    fovi::g_last_cuda_error = "sampler kernel gave up waiting for its image copies";
    return FOVI_ERR_DEVICE_TIMEOUT;
  }
  return FOVI_OK;
}

extern "C" int fovi_sample_backward(const fovi_sampler_plan* plan, const void* grad_out, int go_dtype, int layout, int B, int C, int H, int W,
                                    const float* fix_rc, const float* fix_hw, int F, int mode, int pad, float* grad_img, void* stream) {
  if (!plan || B < 0 || C <= 0 || H <= 0 || W <= 0 || F <= 0 || !fovi::valid_dtype(go_dtype)) return FOVI_ERR_INVALID_ARGUMENT;
  if (mode != FOVI_NEAREST && mode != FOVI_BILINEAR) return FOVI_ERR_INVALID_ARGUMENT;
  if (pad != FOVI_PAD_ZEROS && pad != FOVI_PAD_BORDER) return FOVI_ERR_INVALID_ARGUMENT;
  if (layout != FOVI_OUT_BFCN && layout != FOVI_OUT_FBCN) return FOVI_ERR_UNSUPPORTED;
  if (B == 0) return FOVI_OK;
  if (!grad_out || !fix_rc || !fix_hw || !grad_img || !plan->grid_xy) return FOVI_ERR_INVALID_ARGUMENT;
  SampleArgs a;
  memset(&a, 0, sizeof(a));
  a.sorted_xy = plan->grid_xy; a.fix_rc = fix_rc; a.fix_hw = fix_hw;
  a.B = B; a.C = C; a.H = H; a.W = W; a.F = F; a.N = plan->n_points;
  a.f_major = layout == FOVI_OUT_FBCN ? 1 : 0;
  a.pow2 = ((W & (W - 1)) == 0 && (H & (H - 1)) == 0) ? 1 : 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long total = (long long)B * F * plan->n_points;
  const int grid = (int)std::min<long long>((total + 255) / 256, (long long)fovi::sm_count() * 32);
#define RUN(TG, M, P) fovi_sample_backward_kernel<TG, M, P><<<grid, 256, 0, st>>>(a, (const TG*)grad_out, grad_img)
#define RUN_T(TG)                                                                                          \
  do {                                                                                                     \
    if (mode == FOVI_NEAREST) { if (pad == FOVI_PAD_ZEROS) RUN(TG, FOVI_NEAREST, FOVI_PAD_ZEROS); else RUN(TG, FOVI_NEAREST, FOVI_PAD_BORDER); } \
    else { if (pad == FOVI_PAD_ZEROS) RUN(TG, FOVI_BILINEAR, FOVI_PAD_ZEROS); else RUN(TG, FOVI_BILINEAR, FOVI_PAD_BORDER); }                  \
  } while (0)
  if (go_dtype == FOVI_F32) RUN_T(float); else RUN_T(__nv_bfloat16);
#undef RUN_T
#undef RUN
  return fovi::after_launch("fovi_sample_backward_kernel");
}
