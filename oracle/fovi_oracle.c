/* C restatement (POSIX threads) of the reference's sensor sampler and KNNConv forward.
 *
 * TEST INFRASTRUCTURE ONLY: used by the tests as a second, torch-free checker for cases too large for
 * the NumPy oracle, and by the benchmark as the timed CPU baseline.  Never part of the product path.
 * Parity status: pinned — tests/test_oracle_golden.py checks these functions against the outputs
 * recorded from the reference (bit-exact sampler, 1e-4 KNNConv: float accumulation order differs from BLAS).
 *
 * Sampler: fovi/sensing/coords.py:590-642 (grid transform, one float32 rounding per operation) followed by
 * torch's CPU grid_sample with align_corners=False as called at fovi/sensing/samplers.py:108
 * (unnormalise with one fused multiply-add, rounded weight products, NW/NE/SW/SE accumulated with fused
 * multiply-adds, zeros or border padding, nearest = round half to even).
 * KNNConv: fovi/arch/knn.py:484-557 collapsed to its closed form
 *   out[b,o,n] = bias[o] + sum_k sum_c Xpad[b,c,idx[k,n]] * W[o, c*V + tap[n,k]].
 * Build with -ffp-contract=off so that only the explicit fmaf calls fuse.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ---- a minimal parallel-for: [0,n) cut into contiguous blocks, one thread each ---- */
typedef void (*range_fn)(long lo, long hi, void* ctx);
typedef struct { range_fn fn; void* ctx; long lo, hi; } job_t;
static void* job_main(void* p) { job_t* j = (job_t*)p; j->fn(j->lo, j->hi, j->ctx); return NULL; }

int fovi_oracle_threads(void) {
  const char* e = getenv("FOVI_ORACLE_THREADS");
  long t = e ? atol(e) : sysconf(_SC_NPROCESSORS_ONLN);
  return (int)(t < 1 ? 1 : (t > 256 ? 256 : t));
}

static void parallel_for(long n, range_fn fn, void* ctx) {
  int T = fovi_oracle_threads();
  if (T > n) T = (int)(n > 0 ? n : 1);
  pthread_t th[256]; job_t jobs[256];
  for (int t = 0; t < T; ++t) {
    jobs[t].fn = fn; jobs[t].ctx = ctx; jobs[t].lo = n * t / T; jobs[t].hi = n * (t + 1) / T;
    if (t + 1 < T) pthread_create(&th[t], NULL, job_main, &jobs[t]);
  }
  job_main(&jobs[T - 1]);
  for (int t = 0; t + 1 < T; ++t) pthread_join(th[t], NULL);
}

static inline float fetch(const float* plane, int W, int H, long x, long y) {
  return (x >= 0 && x < W && y >= 0 && y < H) ? plane[y * (long)W + x] : 0.0f;
}

/* img [B,C,H,W]; grid_xy [N,2]; fix_rc, fix_hw [B,F,2]; out [B,F,C,N].  mode 0 nearest / 1 bilinear; pad 0 zeros / 1 border. */
typedef struct { const float* img; int B, C, H, W; const float* grid_xy; int N; const float* fix_rc; const float* fix_hw; int F, mode, pad; float* out; } sample_ctx;

static void sample_range(long lo, long hi, void* p) {
  const sample_ctx* a = (const sample_ctx*)p;
  const float* img = a->img; const int C = a->C, H = a->H, W = a->W, N = a->N, F = a->F, mode = a->mode, pad = a->pad;
  const float* grid_xy = a->grid_xy; const float* fix_rc = a->fix_rc; const float* fix_hw = a->fix_hw; float* out = a->out;
  const float Wf = (float)W, Hf = (float)H;
  for (long bf = lo; bf < hi; ++bf) {
    const int b = (int)(bf / F), f = (int)(bf % F);
    {
      const float* rc = fix_rc + ((size_t)b * F + f) * 2;
      const float* hw = fix_hw + ((size_t)b * F + f) * 2;
      const float cy = rc[0] * Hf, cx = rc[1] * Wf;
      const float half_h = hw[0] / 2.0f, half_w = hw[1] / 2.0f;
      float* o = out + ((size_t)b * F + f) * C * N;
      for (int n = 0; n < N; ++n) {
        float gx = grid_xy[2 * n] * half_w; gx = gx + cx;
        float gy = grid_xy[2 * n + 1] * half_h; gy = gy + cy;
        gx = (2.0f * gx) / Wf - 1.0f;
        gy = (2.0f * gy) / Hf - 1.0f;
        float ix = fmaf(gx + 1.0f, Wf * 0.5f, -0.5f);
        float iy = fmaf(gy + 1.0f, Hf * 0.5f, -0.5f);
        if (pad == 1) {
          ix = fminf(fmaxf(ix, 0.0f), Wf - 1.0f);
          iy = fminf(fmaxf(iy, 0.0f), Hf - 1.0f);
        }
        if (mode == 0) {
          const long x = lrintf(ix), y = lrintf(iy); /* default rounding mode: half to even */
          for (int c = 0; c < C; ++c) o[(size_t)c * N + n] = fetch(img + ((size_t)b * C + c) * H * W, W, H, x, y);
        } else {
          const float x0f = floorf(ix), y0f = floorf(iy);
          const float tx = ix - x0f, ty = iy - y0f, ux = 1.0f - tx, uy = 1.0f - ty;
          const float w_nw = uy * ux, w_ne = uy * tx, w_sw = ty * ux, w_se = ty * tx;
          const long x0 = (long)x0f, y0 = (long)y0f;
          for (int c = 0; c < C; ++c) {
            const float* plane = img + ((size_t)b * C + c) * H * W;
            float acc = fetch(plane, W, H, x0, y0) * w_nw;
            acc = fmaf(fetch(plane, W, H, x0 + 1, y0), w_ne, acc);
            acc = fmaf(fetch(plane, W, H, x0, y0 + 1), w_sw, acc);
            acc = fmaf(fetch(plane, W, H, x0 + 1, y0 + 1), w_se, acc);
            o[(size_t)c * N + n] = acc;
          }
        }
      }
    }
  }
}

void fovi_oracle_sample(const float* img, int B, int C, int H, int W, const float* grid_xy, int N, const float* fix_rc,
                        const float* fix_hw, int F, int mode, int pad, float* out) {
  sample_ctx a = {img, B, C, H, W, grid_xy, N, fix_rc, fix_hw, F, mode, pad, out};
  parallel_for((long)B * F, sample_range, &a);
}

/* X [B,Cin,Nin]; idx [K,Nout] (value Nin = pad); tap [Nout,K]; Wm [Cout, Cin*V]; Y [B,Cout,Nout]. */
typedef struct { const float* X; int B, Cin, Nin; const int32_t* idx; const int64_t* tap; int K, Nout, V; const float* Wm; const float* bias; int Cout, relu; float* Y; float* Wt; } conv_ctx;

static void transpose_range(long lo, long hi, void* p) {
  const conv_ctx* a = (const conv_ctx*)p;
  for (long v = lo; v < hi; ++v)
    for (int c = 0; c < a->Cin; ++c)
      for (int o = 0; o < a->Cout; ++o)
        a->Wt[((size_t)v * a->Cin + c) * a->Cout + o] = a->Wm[(size_t)o * a->Cin * a->V + (size_t)c * a->V + v];
}

static void conv_range(long lo, long hi, void* p) {
  const conv_ctx* a = (const conv_ctx*)p;
  const int Cin = a->Cin, Nin = a->Nin, K = a->K, Nout = a->Nout, Cout = a->Cout;
  float* acc = (float*)malloc((size_t)Cout * sizeof(float));
  for (long it = lo; it < hi; ++it) {
    const int b = (int)(it / Nout), n = (int)(it % Nout);
    for (int o = 0; o < Cout; ++o) acc[o] = 0.0f;
    for (int k = 0; k < K; ++k) {
      const int j = a->idx[(size_t)k * Nout + n];
      if (j >= Nin) continue; /* pad neighbour */
      const float* w = a->Wt + (size_t)a->tap[(size_t)n * K + k] * Cin * Cout;
      for (int c = 0; c < Cin; ++c) {
        const float x = a->X[((size_t)b * Cin + c) * Nin + j];
        const float* wc = w + (size_t)c * Cout;
        for (int o = 0; o < Cout; ++o) acc[o] += x * wc[o];
      }
    }
    for (int o = 0; o < Cout; ++o) {
      float v = acc[o] + (a->bias ? a->bias[o] : 0.0f);
      if (a->relu && v < 0.0f) v = 0.0f;
      a->Y[((size_t)b * Cout + o) * Nout + n] = v;
    }
  }
  free(acc);
}

void fovi_oracle_knnconv(const float* X, int B, int Cin, int Nin, const int32_t* idx, const int64_t* tap, int K, int Nout,
                         int V, const float* Wm, const float* bias, int Cout, int relu, float* Y) {
  conv_ctx a = {X, B, Cin, Nin, idx, tap, K, Nout, V, Wm, bias, Cout, relu, Y, NULL};
  /* tap-major, channel-minor copy of the weights: the Cout values of one (tap, channel) are contiguous */
  a.Wt = (float*)malloc((size_t)V * Cin * Cout * sizeof(float));
  parallel_for(V, transpose_range, &a);
  parallel_for((long)B * Nout, conv_range, &a);
  free(a.Wt);
}
