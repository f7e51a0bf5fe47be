// KNNConv: plan construction, operand packing and the exact float32 (CUDA-core) forward.
#include <algorithm>
#include <vector>

#include "knnconv_plan.cuh"

namespace {

// W [c_out, c_in*V] (c-major, v-minor)  ->  slabs [V, c_out, cp]
template <typename TW, typename TD>
__global__ void pack_weights_kernel(const TW* __restrict__ W, TD* __restrict__ dst, int V, int c_out, int c_in, int cp) {
  const long long total = (long long)V * c_out * cp;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cp);
    const int o = (int)((i / cp) % c_out);
    const int v = (int)(i / ((long long)cp * c_out));
    const float w = c < c_in ? ld_as_float(W + ((long long)o * c_in + c) * V + v) : 0.f;
    dst[i] = from_float<TD>(w);
  }
}

// Pair mode: W [c_out, c_in*V] -> per-output-point slabs [n_out, c_out/ct, sp, ct, 8] (so the eight
// slots of one stage of one c_out tile are contiguous); element (h, c) of a slot row is the weight
// of channel c (< 4) for the even (h = 0) or odd (h = 1) point of the pair.
template <typename TW>
__global__ void pack_weights_pairs_kernel(const TW* __restrict__ W, __nv_bfloat16* __restrict__ dst,
                                          const uint16_t* __restrict__ pair_tap, int n_out, int sp, int V, int c_out, int c_in, int ct) {
  const long long total = (long long)n_out * sp * c_out * 8;
  const int n_ct = c_out / ct;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int e = (int)(i & 7);
    long long r = i >> 3;
    const int oc = (int)(r % ct); r /= ct;
    const int sl = (int)(r % sp); r /= sp;
    const int tile = (int)(r % n_ct);
    const long long n = r / n_ct;
    const int o = tile * ct + oc;
    const long long slot = n * sp + sl;
    const int h = e >> 2, c = e & 3;
    const int t = pair_tap[slot * 2 + h];
    const float w = (c < c_in && t != 0xFFFF) ? ld_as_float(W + ((long long)o * c_in + c) * V + t) : 0.f;
    dst[i] = __float2bfloat16_rn(w);
  }
}

// Packed weights of a GROUPED pair-mode plan: the plan's "output points" are groups of G consecutive output points of the
// layer and its "output channels" are the G members' channels side by side (c_out = G * co), so the group's one
// neighbour list is the union of its members' lists.  The plan was created with tap[g][k] = k, i.e. pair_tap holds each
// slot's position in the union list; member_tap[g][k][j] is the filter tap member j gives that neighbour (0xFFFF: it
// is not a neighbour of member j, the weight is zero).  Same destination layout as pack_weights_pairs_kernel.
template <typename TW>
__global__ void pack_weights_grouped_kernel(const TW* __restrict__ W, __nv_bfloat16* __restrict__ dst,
                                            const uint16_t* __restrict__ pair_tap, const uint16_t* __restrict__ member_tap, int n_groups,
                                            int sp, int K, int G, int V, int co, int c_in, int ct) {
  // one thread per 16-byte row of the destination (a pair slot of one output channel: 2 points x 4 channels), so the
  // index arithmetic and the two table look-ups are paid once per eight values and the store is a whole 16-byte piece
  const int c_out = G * co;
  const long long total = (long long)n_groups * sp * c_out;
  const int n_ct = c_out / ct;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    long long r = i;
    const int oc = (int)(r % ct); r /= ct;
    const int sl = (int)(r % sp); r /= sp;
    const int tile = (int)(r % n_ct);
    const long long g = r / n_ct;
    const int op = tile * ct + oc;          // channel of the group: member j, its channel o
    const int j = op / co, o = op - j * co;
    __align__(16) __nv_bfloat16 v[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int k = pair_tap[(g * sp + sl) * 2 + h];
      int t = 0xFFFF;
      if (k != 0xFFFF) t = member_tap[(g * K + k) * G + j];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        v[h * 4 + c] = __float2bfloat16_rn((c < c_in && t != 0xFFFF) ? ld_as_float(W + ((long long)o * c_in + c) * V + t) : 0.f);
    }
    *reinterpret_cast<uint4*>(dst + i * 8) = *reinterpret_cast<const uint4*>(v);
  }
}

// X [B,C,N] -> [ceil(B/128), ceil(N/2), 128, 2, 4] bf16 (pair layout), one thread per (pair, image).
template <typename TX>
__global__ void pack_points_pairs_kernel(const TX* __restrict__ x, __nv_bfloat16* __restrict__ dst, int B, int C, int N) {
  const int n_pairs = (N + 1) / 2;
  const long long total = (long long)n_pairs * B;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int pr = (int)(i % n_pairs), b = (int)(i / n_pairs);
    __align__(16) __nv_bfloat16 v[8];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int n = 2 * pr + h;
        v[h * 4 + c] = __float2bfloat16_rn((c < C && n < N) ? ld_as_float(x + ((long long)b * C + c) * N + n) : 0.f);
      }
    *reinterpret_cast<uint4*>(dst + (((long long)(b >> 7) * n_pairs + pr) * 128 + (b & 127)) * 8) = *reinterpret_cast<const uint4*>(v);
  }
}

// X [B,C,N] -> [B,N,cp] bf16, transposing 32x32 tiles through shared memory.
template <typename TX>
__global__ void pack_points_kernel(const TX* __restrict__ x, __nv_bfloat16* __restrict__ dst, int C, int N, int cp) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z;
  const int n0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const TX* xb = x + (long long)b * C * N;
  __nv_bfloat16* db = dst + (long long)b * N * cp;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int c = c0 + r, n = n0 + threadIdx.x;
    tile[r][threadIdx.x] = (c < C && n < N) ? ld_as_float(xb + (long long)c * N + n) : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, c = c0 + threadIdx.x;
    if (n < N && c < cp) db[(long long)n * cp + c] = __float2bfloat16_rn(tile[threadIdx.x][r]);
  }
}

// Exact float32 forward.  One CTA: one output point, BT batch rows, all output channels.
template <typename TX, bool X_BNC, bool Y_BNC>
__global__ void __launch_bounds__(128) knnconv_f32_kernel(const TX* __restrict__ X, const float* __restrict__ Wt,
                                                          const float* __restrict__ bias, float* __restrict__ Y,
                                                          const int* __restrict__ nbr_idx, const uint16_t* __restrict__ nbr_tap,
                                                          const int* __restrict__ nbr_cnt, int kp, int B, int n_in, int n_out,
                                                          int c_in, int c_out, int cp, int relu, int BT) {
  const int n = blockIdx.x;
  const int b0 = blockIdx.y * BT;
  const int cnt = nbr_cnt[n];
  const int* idx = nbr_idx + (long long)n * kp;
  const uint16_t* tp = nbr_tap + (long long)n * kp;
  const int bt = min(BT, B - b0);
  for (int p = threadIdx.x; p < bt * c_out; p += blockDim.x) {
    const int o = p % c_out, b = b0 + p / c_out;
    float acc = 0.f;
    for (int k = 0; k < cnt; ++k) {
      const int j = idx[k];
      const float* w = Wt + ((long long)tp[k] * c_out + o) * cp;
      for (int c = 0; c < c_in; ++c) {
        const float xv = X_BNC ? ld_as_float(X + ((long long)b * n_in + j) * c_in + c)
                               : ld_as_float(X + ((long long)b * c_in + c) * n_in + j);
        acc = fmaf(xv, __ldg(w + c), acc);
      }
    }
    if (bias) acc += __ldg(bias + o);
    if (relu) acc = fmaxf(acc, 0.f);
    if (Y_BNC) Y[((long long)b * n_out + n) * c_out + o] = acc;
    else Y[((long long)b * c_out + o) * n_out + n] = acc;
  }
}

}  // namespace

extern "C" int fovi_knnconv_plan_create(const int32_t* knn_idx_pad, const uint16_t* tap, int n_in, int n_out, int K, int V,
                                        int c_in, int c_out, fovi_knnconv_plan** out) {
  if (!knn_idx_pad || !tap || !out) return FOVI_ERR_INVALID_ARGUMENT;
  if (n_in <= 0 || n_out <= 0 || K <= 0 || V <= 0 || c_in <= 0 || c_out <= 0 || V > 65535) return FOVI_ERR_INVALID_ARGUMENT;
  const int kp = (K + 7) / 8 * 8;
  std::vector<int> idx((size_t)n_out * kp, n_in), cnt(n_out, 0);
  std::vector<uint16_t> tp((size_t)n_out * kp, 0);
  int64_t nnz = 0;
  for (int n = 0; n < n_out; ++n) {
    int m = 0;
    for (int k = 0; k < K; ++k) {
      const int j = knn_idx_pad[(size_t)k * n_out + n];
      const int t = tap[(size_t)n * K + k];
      if (j < 0 || j > n_in || t >= V) return FOVI_ERR_TABLE_RANGE;
      if (j == n_in) continue;  // pad neighbour: contributes nothing
      idx[(size_t)n * kp + m] = j;
      tp[(size_t)n * kp + m] = (uint16_t)t;
      ++m;
    }
    cnt[n] = m;
    nnz += m;
  }
  auto* p = new fovi_knnconv_plan();
  p->n_in = n_in; p->n_out = n_out; p->K = K; p->V = V; p->c_in = c_in; p->c_out = c_out; p->kp = kp; p->nnz = nnz;
  p->cin_packed = (c_in % 64 == 0) ? c_in : (c_in + 7) / 8 * 8;
  p->ct = (c_out % 16 == 0) ? fovi::pick_cout_tile(c_out) : 0;
  // Pair mode for tiny channel counts: group each point's neighbours into aligned input pairs
  // (2p, 2p+1).  A neighbour takes the free half of a slot of its pair, or opens a new slot (so a
  // table that lists the same input point twice still adds both taps).
  std::vector<int> pidx, pcnt;
  std::vector<uint16_t> ptap, prun;
  if (c_in <= 4) {
    p->x_layout = FOVI_X_PAIRS;
    p->n_pairs = (n_in + 1) / 2;
    std::vector<std::vector<int>> slots_idx(n_out);
    std::vector<std::vector<uint16_t>> slots_tap(n_out);
    int max_slots = 0;
    for (int n = 0; n < n_out; ++n) {
      auto& si = slots_idx[n];
      auto& st = slots_tap[n];
      for (int m = 0; m < cnt[n]; ++m) {
        const int j = idx[(size_t)n * kp + m], pr = j >> 1, h = j & 1;
        size_t s = 0;
        for (; s < si.size(); ++s)
          if (si[s] == pr && st[2 * s + h] == 0xFFFF) break;
        if (s == si.size()) { si.push_back(pr); st.push_back(0xFFFF); st.push_back(0xFFFF); }
        st[2 * s + h] = tp[(size_t)n * kp + m];
      }
      max_slots = std::max<int>(max_slots, (int)si.size());
    }
    p->sp = std::max(8, (max_slots + 7) / 8 * 8);
    pidx.assign((size_t)n_out * p->sp, p->n_pairs);
    ptap.assign((size_t)n_out * p->sp * 2, 0xFFFF);
    pcnt.assign(n_out, 0);
    for (int n = 0; n < n_out; ++n) {
      // visit pairs in ascending order: neighbouring slots then read neighbouring memory
      std::vector<int> order(slots_idx[n].size());
      for (size_t s = 0; s < order.size(); ++s) order[s] = (int)s;
      std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return slots_idx[n][a] < slots_idx[n][b]; });
      for (size_t s = 0; s < order.size(); ++s) {
        pidx[(size_t)n * p->sp + s] = slots_idx[n][order[s]];
        ptap[((size_t)n * p->sp + s) * 2] = slots_tap[n][2 * order[s]];
        ptap[((size_t)n * p->sp + s) * 2 + 1] = slots_tap[n][2 * order[s] + 1];
      }
      pcnt[n] = (int)order.size();
    }
    // Copy plan: inside every 8-slot stage, consecutive pair indices are consecutive 2 KB blocks of the
    // activations, so each run moves with one copy; the unused tail of the last stage is one run of zeros.
    prun.assign((size_t)n_out * p->sp, 0);
    for (int n = 0; n < n_out; ++n) {
      const int* row = &pidx[(size_t)n * p->sp];
      for (int s0 = 0; s0 < p->sp; s0 += 8) {
        int j = 0;
        while (j < 8) {
          int len = 1;
          if (row[s0 + j] >= p->n_pairs) len = 8 - j;
          else while (j + len < 8 && row[s0 + j + len] == row[s0 + j] + len && row[s0 + j + len] < p->n_pairs) ++len;
          prun[(size_t)n * p->sp + s0 + j] = (uint16_t)len;
          j += len;
        }
      }
    }
  }
  cudaError_t e = cudaGetDevice(&p->device);
  if (e == cudaSuccess && p->x_layout == FOVI_X_PAIRS) {
    e = cudaMalloc(&p->pair_idx, sizeof(int) * pidx.size());
    if (e == cudaSuccess) e = cudaMalloc(&p->pair_cnt, sizeof(int) * n_out);
    if (e == cudaSuccess) e = cudaMalloc(&p->pair_tap, sizeof(uint16_t) * ptap.size());
    if (e == cudaSuccess) e = cudaMalloc(&p->pair_run, sizeof(uint16_t) * prun.size());
    if (e == cudaSuccess) e = cudaMemcpy(p->pair_run, prun.data(), sizeof(uint16_t) * prun.size(), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&p->zero_block, 16384);
    if (e == cudaSuccess) e = cudaMemset(p->zero_block, 0, 16384);
    if (e == cudaSuccess) e = cudaMemcpy(p->pair_idx, pidx.data(), sizeof(int) * pidx.size(), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(p->pair_cnt, pcnt.data(), sizeof(int) * n_out, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(p->pair_tap, ptap.data(), sizeof(uint16_t) * ptap.size(), cudaMemcpyHostToDevice);
  }
  if (e == cudaSuccess) e = cudaMalloc(&p->nbr_idx, sizeof(int) * idx.size());
  if (e == cudaSuccess) e = cudaMalloc(&p->nbr_tap, sizeof(uint16_t) * tp.size());
  if (e == cudaSuccess) e = cudaMalloc(&p->nbr_cnt, sizeof(int) * n_out);
  if (e == cudaSuccess) e = cudaMalloc(&p->status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpy(p->nbr_idx, idx.data(), sizeof(int) * idx.size(), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(p->nbr_tap, tp.data(), sizeof(uint16_t) * tp.size(), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(p->nbr_cnt, cnt.data(), sizeof(int) * n_out, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(p->status, 0, sizeof(int));
  if (e != cudaSuccess) {
    fovi_knnconv_plan_destroy(p);
    return fovi::cuda_fail(e, "fovi_knnconv_plan_create");
  }
  *out = p;
  return FOVI_OK;
}

extern "C" void fovi_knnconv_plan_destroy(fovi_knnconv_plan* p) {
  if (!p) return;
  if (p->nbr_idx) cudaFree(p->nbr_idx);
  if (p->nbr_tap) cudaFree(p->nbr_tap);
  if (p->nbr_cnt) cudaFree(p->nbr_cnt);
  if (p->status) cudaFree(p->status);
  if (p->pair_idx) cudaFree(p->pair_idx);
  if (p->pair_cnt) cudaFree(p->pair_cnt);
  if (p->pair_tap) cudaFree(p->pair_tap);
  if (p->zero_block) cudaFree(p->zero_block);
  if (p->pair_run) cudaFree(p->pair_run);
  delete p;
}

extern "C" int fovi_knnconv_cin_packed(const fovi_knnconv_plan* p) { return p ? p->cin_packed : -1; }
extern "C" int64_t fovi_knnconv_nnz(const fovi_knnconv_plan* p) { return p ? p->nnz : -1; }
extern "C" int fovi_knnconv_x_layout(const fovi_knnconv_plan* p) { return p ? p->x_layout : -1; }
extern "C" int fovi_knnconv_tc_supported(const fovi_knnconv_plan* p) {
  if (!p || !p->ct) return 0;
  return (p->x_layout == FOVI_X_PAIRS ? p->sp : p->kp) <= 256 ? 1 : 0;
}

extern "C" int64_t fovi_knnconv_packed_weight_bytes(const fovi_knnconv_plan* p, int dst_dtype) {
  if (!p || !fovi::valid_dtype(dst_dtype)) return -1;
  if (p->x_layout == FOVI_X_PAIRS && dst_dtype == FOVI_BF16) return (int64_t)p->n_out * p->sp * p->c_out * 8 * 2;
  return (int64_t)p->V * p->c_out * p->cin_packed * (int64_t)fovi::dtype_size(dst_dtype);
}

extern "C" int fovi_knnconv_pack_weights(const fovi_knnconv_plan* p, const void* W, int w_dtype, void* dst, int dst_dtype,
                                         void* stream) {
  if (!p || !W || !dst || !fovi::valid_dtype(w_dtype) || !fovi::valid_dtype(dst_dtype)) return FOVI_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (p->x_layout == FOVI_X_PAIRS && dst_dtype == FOVI_BF16) {
    if (!p->ct) return FOVI_ERR_UNSUPPORTED;
    const long long tot = (long long)p->n_out * p->sp * p->c_out * 8;
    const int g = (int)std::min<long long>((tot + 255) / 256, 148 * 32);
    if (w_dtype == FOVI_F32)
      pack_weights_pairs_kernel<float><<<g, 256, 0, st>>>((const float*)W, (__nv_bfloat16*)dst, p->pair_tap, p->n_out, p->sp, p->V, p->c_out, p->c_in, p->ct);
    else
      pack_weights_pairs_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)W, (__nv_bfloat16*)dst, p->pair_tap, p->n_out, p->sp, p->V, p->c_out, p->c_in, p->ct);
    return fovi::after_launch("pack_weights_pairs_kernel");
  }
  const long long total = (long long)p->V * p->c_out * p->cin_packed;
  const int grid = (int)std::min<long long>((total + 255) / 256, 148 * 16);
#define PACK(TW, TD) \
  pack_weights_kernel<TW, TD><<<grid, 256, 0, st>>>((const TW*)W, (TD*)dst, p->V, p->c_out, p->c_in, p->cin_packed)
  if (w_dtype == FOVI_F32 && dst_dtype == FOVI_F32) PACK(float, float);
  else if (w_dtype == FOVI_F32 && dst_dtype == FOVI_BF16) PACK(float, __nv_bfloat16);
  else if (w_dtype == FOVI_BF16 && dst_dtype == FOVI_F32) PACK(__nv_bfloat16, float);
  else PACK(__nv_bfloat16, __nv_bfloat16);
#undef PACK
  return fovi::after_launch("pack_weights_kernel");
}

extern "C" int fovi_knnconv_pack_weights_grouped(const fovi_knnconv_plan* p, const void* W, int w_dtype, const uint16_t* member_tap, int G,
                                                 int V, void* dst, void* stream) {
  if (!p || !W || !member_tap || !dst || !fovi::valid_dtype(w_dtype) || G <= 0 || V <= 0) return FOVI_ERR_INVALID_ARGUMENT;
  if (p->x_layout != FOVI_X_PAIRS || !p->ct || p->c_out % G) return FOVI_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long tot = (long long)p->n_out * p->sp * p->c_out;   // 16-byte rows
  const int grid = (int)std::min<long long>((tot + 255) / 256, 148 * 32);
  if (w_dtype == FOVI_F32)
    pack_weights_grouped_kernel<float><<<grid, 256, 0, st>>>((const float*)W, (__nv_bfloat16*)dst, p->pair_tap, member_tap, p->n_out, p->sp, p->K,
                                                             G, V, p->c_out / G, p->c_in, p->ct);
  else
    pack_weights_grouped_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)W, (__nv_bfloat16*)dst, p->pair_tap, member_tap, p->n_out,
                                                                     p->sp, p->K, G, V, p->c_out / G, p->c_in, p->ct);
  return fovi::after_launch("pack_weights_grouped_kernel");
}

extern "C" int fovi_pack_points(const void* x, int x_dtype, int B, int C, int N, void* dst, int cp, int x_layout, void* stream) {
  if (!fovi::valid_dtype(x_dtype) || B < 0 || C <= 0 || N <= 0) return FOVI_ERR_INVALID_ARGUMENT;
  if (x_layout != FOVI_X_BNC && x_layout != FOVI_X_PAIRS) return FOVI_ERR_INVALID_ARGUMENT;
  if (x_layout == FOVI_X_BNC && (cp < C || cp % 8)) return FOVI_ERR_INVALID_ARGUMENT;
  if (x_layout == FOVI_X_PAIRS && C > 4) return FOVI_ERR_INVALID_ARGUMENT;
  if (B == 0) return FOVI_OK;
  if (!x || !dst) return FOVI_ERR_INVALID_ARGUMENT;
  if (B > 65535) return FOVI_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (x_layout == FOVI_X_PAIRS) {
    const long long tot = (long long)((N + 1) / 2) * B;
    const int g = (int)std::min<long long>((tot + 255) / 256, 148 * 32);
    if (x_dtype == FOVI_F32) pack_points_pairs_kernel<float><<<g, 256, 0, st>>>((const float*)x, (__nv_bfloat16*)dst, B, C, N);
    else pack_points_pairs_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)dst, B, C, N);
    return fovi::after_launch("pack_points_pairs_kernel");
  }
  dim3 grid((N + 31) / 32, (cp + 31) / 32, B), block(32, 8);
  if (x_dtype == FOVI_F32) pack_points_kernel<float><<<grid, block, 0, st>>>((const float*)x, (__nv_bfloat16*)dst, C, N, cp);
  else pack_points_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)dst, C, N, cp);
  return fovi::after_launch("pack_points_kernel");
}

extern "C" int fovi_knnconv_forward_f32(const fovi_knnconv_plan* p, const void* X, int x_dtype, int x_layout, const float* Wt,
                                        const float* bias, float* Y, int y_layout, int B, int relu, void* stream) {
  if (!p || !fovi::valid_dtype(x_dtype) || B < 0) return FOVI_ERR_INVALID_ARGUMENT;
  if (B > 0 && (!X || !Wt || !Y)) return FOVI_ERR_INVALID_ARGUMENT;
  if ((x_layout != FOVI_ACT_BCN && x_layout != FOVI_ACT_BNC) || (y_layout != FOVI_ACT_BCN && y_layout != FOVI_ACT_BNC))
    return FOVI_ERR_INVALID_ARGUMENT;
  if (B == 0) return FOVI_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int BT = 4;
  if ((B + BT - 1) / BT > 65535) return FOVI_ERR_UNSUPPORTED;
  dim3 grid(p->n_out, (B + BT - 1) / BT);
#define RUN(TX, XL, YL)                                                                                                   \
  knnconv_f32_kernel<TX, XL, YL><<<grid, 128, 0, st>>>((const TX*)X, Wt, bias, Y, p->nbr_idx, p->nbr_tap, p->nbr_cnt, p->kp, B, \
                                                       p->n_in, p->n_out, p->c_in, p->c_out, p->cin_packed, relu, BT)
  const bool xb = x_layout == FOVI_ACT_BNC, yb = y_layout == FOVI_ACT_BNC;
  if (x_dtype == FOVI_F32) {
    if (xb && yb) RUN(float, true, true); else if (xb) RUN(float, true, false);
    else if (yb) RUN(float, false, true); else RUN(float, false, false);
  } else {
    if (xb && yb) RUN(__nv_bfloat16, true, true); else if (xb) RUN(__nv_bfloat16, true, false);
    else if (yb) RUN(__nv_bfloat16, false, true); else RUN(__nv_bfloat16, false, false);
  }
#undef RUN
  return fovi::after_launch("knnconv_f32_kernel");
}

// ------------------------------------------------------------------------------------------------
// Allocation-free forward from the reference's [B, c_in, n_in] layout.
//
// Some hosts may not allocate device memory at the point where they run a layer: code inside a
// real-time loop or a serving thread that was handed a fixed memory budget at start-up, or a
// plug-in whose host application owns the allocator and forbids allocation calls from callbacks
// (cudaMalloc also synchronises the whole device, which such hosts cannot afford).  For them the
// repacked copy of the activations that the tensor-core kernel reads lives in the fixed array
// below instead of a caller-provided or freshly allocated buffer.
//
// The array is part of the library image: every GPU that loads the library holds these bytes
// until the process exits.  All calls on a device share it and it keeps the last call's contents,
// so two calls that overlap on the GPU (different streams) race; issue them on one stream.
#define FOVI_STATIC_SCRATCH_BYTES (32u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[FOVI_STATIC_SCRATCH_BYTES];

namespace {
// Device address of g_static_scratch on each device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use, so it is resolved once per device.
int static_scratch_address(unsigned char** out) {
  static unsigned char* addr[64] = {nullptr};
  int dev = -1;
  FOVI_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FOVI_ERR_UNSUPPORTED;
  if (!addr[dev]) {
    void* p = nullptr;
    FOVI_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));  // the current device is `dev`
    addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = addr[dev];
  return FOVI_OK;
}
}  // namespace

extern "C" int64_t fovi_static_scratch_bytes(void) { return (int64_t)FOVI_STATIC_SCRATCH_BYTES; }

extern "C" int fovi_knnconv_forward_bcn_static(fovi_knnconv_plan* p, const void* X, int x_dtype, const void* Wt,
                                               const float* bias, void* Y, int y_dtype, int B, int relu, void* stream) {
  if (!p || !fovi::valid_dtype(x_dtype) || !fovi::valid_dtype(y_dtype) || B < 0) return FOVI_ERR_INVALID_ARGUMENT;
  if (B == 0) return FOVI_OK;
  if (!X || !Wt || !Y) return FOVI_ERR_INVALID_ARGUMENT;
  const bool pairs = p->x_layout == FOVI_X_PAIRS;
  const long long need = pairs ? (long long)((B + 127) / 128) * p->n_pairs * 2048
                               : (long long)B * p->n_in * p->cin_packed * 2;
  if (need > (long long)FOVI_STATIC_SCRATCH_BYTES) {
    fovi::g_last_cuda_error = "fovi_knnconv_forward_bcn_static: the packed activations need " + std::to_string(need) +
                              " bytes, the static scratch holds " + std::to_string(FOVI_STATIC_SCRATCH_BYTES) +
                              "; use a smaller batch or fovi_pack_points + fovi_knnconv_forward";
    return FOVI_ERR_UNSUPPORTED;
  }
  unsigned char* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (pairs && (B & 127)) {
    // The pad rows of the last 128-row tile are never written by the repack: clear them, so that no
    // bit pattern left by an earlier call is fed to the tensor cores.
    const int r0 = B & 127;
    unsigned char* tile = scratch + (size_t)(B / 128) * p->n_pairs * 2048;
    FOVI_CUDA(cudaMemset2DAsync(tile + (size_t)r0 * 16, 2048, 0, (size_t)(128 - r0) * 16, p->n_pairs, st));
  }
  rc = fovi_pack_points(X, x_dtype, B, p->c_in, p->n_in, scratch, p->cin_packed, p->x_layout, stream);
  if (rc) return rc;
  return fovi_knnconv_forward(p, scratch, Wt, bias, Y, y_dtype, B, relu, stream);
}
