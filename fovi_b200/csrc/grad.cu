// Layout change used by the weight-gradient contraction of KNNConv: the batch index becomes the innermost
// (contiguous) one, so that it can play the role of the channels in the tensor-core kernel.
#include <algorithm>

#include <cuda_bf16.h>

#include "common.cuh"

namespace {

// src: logical [B, I, J], element (b,i,j) at b*sb + i*si + j*sj, with si == 1 (FAST_I) or sj == 1 (!FAST_I).
// dst: [I, Jp, Bp] bf16, zero where j >= J or b >= B.  32x32 tiles of (batch, fast index) go through shared memory:
// reads run along the source's contiguous index, writes along the batch.
template <typename T, bool FAST_I>
__global__ void batch_to_inner_kernel(const T* __restrict__ src, __nv_bfloat16* __restrict__ dst, int B, int I, int J, int Jp, int Bp,
                                      long long sb, long long si, long long sj) {
  __shared__ float tile[32][33];
  const int b0 = blockIdx.x * 32, f0 = blockIdx.y * 32, slow = blockIdx.z;
  const int F = FAST_I ? I : J;   // extent of the fast index in the source
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int b = b0 + r, f = f0 + threadIdx.x;
    const int i = FAST_I ? f : slow, j = FAST_I ? slow : f;
    tile[r][threadIdx.x] = (b < B && f < F && j < J) ? ld_as_float(src + b * sb + i * si + j * sj) : 0.f;
  }
  __syncthreads();
  const int Fd = FAST_I ? I : Jp;  // extent of the fast index in the destination
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int f = f0 + r, b = b0 + threadIdx.x;
    if (f < Fd && b < Bp) {
      const int i = FAST_I ? f : slow, j = FAST_I ? slow : f;
      dst[((long long)i * Jp + j) * Bp + b] = __float2bfloat16_rn(tile[threadIdx.x][r]);
    }
  }
}

// Same, 64x64 tiles with two elements per access: a warp reads 64 consecutive source elements per row and writes 64 consecutive
// batch entries (128 bytes) per row.  Needs an even fast extent and even strides (so that pairs are aligned).
// Optionally fused, for the backward pass of a layer with a fused ReLU (src = upstream gradient, `act` = the layer's
// output, same layout): the gradient is masked where the output is not positive before it is transposed, the masked
// gradient is also written back in the source layout (`masked`, for the input-gradient GEMM) and its sums over
// everything but the fast index (the channels: the bias gradient) are added into `colsum` -- one read of the gradient
// instead of three.
constexpr int X2_SLOW = 4;   // consecutive values of the slow index one block works through

template <typename T, bool FAST_I>
__global__ void __launch_bounds__(256) batch_to_inner_x2_kernel(const T* __restrict__ src, __nv_bfloat16* __restrict__ dst, int B, int I, int J,
                                                               int Jp, int Bp, long long sb, long long si, long long sj,
                                                               const T* __restrict__ act, T* __restrict__ masked, float* __restrict__ colsum) {
  __shared__ __nv_bfloat16 tile[64][66];
  __shared__ float part[8][64];
  const int b0 = blockIdx.x * 64, f0 = blockIdx.y * 64;
  const int F = FAST_I ? I : J, n_slow = FAST_I ? Jp : I;
  const int tx = threadIdx.x, ty = threadIdx.y;
  float s0 = 0.f, s1 = 0.f;
  for (int sl = 0; sl < X2_SLOW; ++sl) {
    const int slow = blockIdx.z * X2_SLOW + sl;
    if (slow >= n_slow) break;           // uniform over the block
    if (sl) __syncthreads();             // the tile is free again
    for (int r = ty; r < 64; r += 8) {
      const int b = b0 + r, f = f0 + 2 * tx;
      const int i = FAST_I ? f : slow, j = FAST_I ? slow : f;
      float v0 = 0.f, v1 = 0.f;
      if (b < B && f < F && j < J) {   // F is even: f + 1 < F as well
        const long long off = b * sb + i * si + j * sj;
        const T* p = src + off;
        if (sizeof(T) == 2) {
          const __nv_bfloat162 q = *reinterpret_cast<const __nv_bfloat162*>(p);
          v0 = __bfloat162float(q.x); v1 = __bfloat162float(q.y);
        } else {
          const float2 q = *reinterpret_cast<const float2*>(p);
          v0 = q.x; v1 = q.y;
        }
        if (act) {
          float a0, a1;
          if (sizeof(T) == 2) {
            const __nv_bfloat162 q = *reinterpret_cast<const __nv_bfloat162*>(act + off);
            a0 = __bfloat162float(q.x); a1 = __bfloat162float(q.y);
          } else {
            const float2 q = *reinterpret_cast<const float2*>(act + off);
            a0 = q.x; a1 = q.y;
          }
          v0 = a0 > 0.f ? v0 : 0.f; v1 = a1 > 0.f ? v1 : 0.f;
        }
        if (masked) {
          if (sizeof(T) == 2) {
            __nv_bfloat162 q;
            q.x = __float2bfloat16_rn(v0); q.y = __float2bfloat16_rn(v1);
            *reinterpret_cast<__nv_bfloat162*>(masked + off) = q;
          } else {
            *reinterpret_cast<float2*>(masked + off) = make_float2(v0, v1);
          }
        }
        s0 += v0; s1 += v1;
      }
      __nv_bfloat162 t2;
      t2.x = __float2bfloat16_rn(v0); t2.y = __float2bfloat16_rn(v1);
      *reinterpret_cast<__nv_bfloat162*>(&tile[r][2 * tx]) = t2;
    }
    __syncthreads();
    const int Fd = FAST_I ? I : Jp;
    for (int r = ty; r < 64; r += 8) {
      const int f = f0 + r, b = b0 + 2 * tx;
      if (f < Fd && b < Bp) {          // Bp is even
        const int i = FAST_I ? f : slow, j = FAST_I ? slow : f;
        __nv_bfloat162 q;
        q.x = tile[2 * tx][r]; q.y = tile[2 * tx + 1][r];
        *reinterpret_cast<__nv_bfloat162*>(dst + ((long long)i * Jp + j) * Bp + b) = q;
      }
    }
  }
  if (colsum) {
    // in the FAST_I == false orientation the fast index (the channel) is the same for every slow index of the block, and in
    // the FAST_I orientation too: the sums of all X2_SLOW passes belong to the same 64 channels
    part[ty][2 * tx] = s0; part[ty][2 * tx + 1] = s1;
    __syncthreads();
    if (ty == 0) {
      for (int e = 0; e < 2; ++e) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += part[w][2 * tx + e];
        const int f = f0 + 2 * tx + e;
        if (f < F) atomicAdd(colsum + f, t);
      }
    }
  }
}

// Column sums of a row-major [R, C] matrix (C even) into float32 dst[C] (zeroed by the caller's launch order: see the entry
// point).  A warp reads 64 consecutive columns of a row (128 bytes of bf16); rows are strided over the 8 warps of a block
// and over grid.y; partial sums meet in shared memory and leave with one atomic per column and block.
template <typename T>
__global__ void __launch_bounds__(256) column_sum_kernel(const T* __restrict__ src, float* __restrict__ dst, long long R, int C,
                                                        long long rows_per_block) {
  __shared__ float part[8][64];
  const int c = blockIdx.x * 64 + 2 * threadIdx.x;
  const long long r0 = blockIdx.y * rows_per_block, r1 = min(R, r0 + rows_per_block);
  float s0 = 0.f, s1 = 0.f;
  if (c < C) {
    for (long long r = r0 + threadIdx.y; r < r1; r += 8) {
      const T* p = src + r * C + c;
      if (sizeof(T) == 2) {
        const __nv_bfloat162 q = *reinterpret_cast<const __nv_bfloat162*>(p);
        s0 += __bfloat162float(q.x); s1 += __bfloat162float(q.y);
      } else {
        const float2 q = *reinterpret_cast<const float2*>(p);
        s0 += q.x; s1 += q.y;
      }
    }
  }
  part[threadIdx.y][2 * threadIdx.x] = s0;
  part[threadIdx.y][2 * threadIdx.x + 1] = s1;
  __syncthreads();
  if (threadIdx.y == 0) {
    for (int e = 0; e < 2; ++e) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += part[w][2 * threadIdx.x + e];
      if (c + e < C) atomicAdd(dst + c + e, t);
    }
  }
}

// Segment sums for the weight gradient of a layer with few input channels.  prod [R][S][4] float32 holds, per output
// channel o (row) and per slot s = (output point, neighbour), the four channel products of that pair; every slot
// belongs to one filter tap.  dst[o][v*4 + c] += sum over the slots of tap v (listed in seg_slot[seg_start[v] ..
// seg_start[v+1])) of prod[o][s][c].  One block per (tap, 64 rows): 4 groups of 64 threads walk the list, each thread
// keeps the float4 of its row, the groups meet in shared memory.  Every dst element has one owner, so no atomics.
__global__ void __launch_bounds__(256) tap_segment_sum_kernel(const float4* __restrict__ prod, long long S, const int* __restrict__ seg_start,
                                                             const int* __restrict__ seg_slot, int R, float* __restrict__ dst, int dst_pitch) {
  __shared__ float4 part[4][64];
  const int v = blockIdx.x, o = blockIdx.y * 64 + (threadIdx.x & 63), g = threadIdx.x >> 6;
  const int p0 = __ldg(seg_start + v), p1 = __ldg(seg_start + v + 1);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (o < R) {
    const float4* row = prod + (long long)o * S;
    for (int p = p0 + g; p < p1; p += 4) {
      const float4 q = __ldg(row + __ldg(seg_slot + p));
      acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
    }
  }
  part[g][threadIdx.x & 63] = acc;
  __syncthreads();
  if (g == 0 && o < R) {
    for (int w = 1; w < 4; ++w) { const float4 q = part[w][threadIdx.x]; acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w; }
    float* d = dst + (long long)o * dst_pitch + 4 * v;
    d[0] += acc.x; d[1] += acc.y; d[2] += acc.z; d[3] += acc.w;
  }
}

}  // namespace

extern "C" int fovi_tap_segment_sum(const float* prod, int R, long long S, const int* seg_start, const int* seg_slot, int V, float* dst,
                                    int dst_pitch, void* stream) {
  if (!prod || !seg_start || !seg_slot || !dst || R <= 0 || S <= 0 || V <= 0 || dst_pitch < 4 * V) return FOVI_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(prod) & 15) return FOVI_ERR_ALIGNMENT;
  if ((R + 63) / 64 > 65535) return FOVI_ERR_UNSUPPORTED;
  dim3 grid(V, (R + 63) / 64);
  tap_segment_sum_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const float4*>(prod), S, seg_start, seg_slot, R, dst,
                                                                                    dst_pitch);
  return fovi::after_launch("tap_segment_sum_kernel");
}

extern "C" int fovi_column_sum(const void* src, int dtype, long long R, int C, float* dst, void* stream) {
  if (!fovi::valid_dtype(dtype) || R < 0 || C <= 0 || !dst) return FOVI_ERR_INVALID_ARGUMENT;
  if (C % 2 || (R > 0 && (!src || reinterpret_cast<uintptr_t>(src) % (2 * fovi::dtype_size(dtype))))) return FOVI_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  FOVI_CUDA(cudaMemsetAsync(dst, 0, sizeof(float) * (size_t)C, st));
  if (R == 0) return FOVI_OK;
  const long long rows_per_block = std::max<long long>(256, (R + 4095) / 4096);
  dim3 grid((C + 63) / 64, (unsigned)((R + rows_per_block - 1) / rows_per_block)), block(32, 8);
  if (dtype == FOVI_F32) column_sum_kernel<float><<<grid, block, 0, st>>>((const float*)src, dst, R, C, rows_per_block);
  else column_sum_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)src, dst, R, C, rows_per_block);
  return fovi::after_launch("column_sum_kernel");
}

static int batch_to_inner_impl(const void* src, int dtype, int B, int I, int J, long long sb, long long si, long long sj, void* dst, int Jp, int Bp,
                               const void* act, void* masked, float* colsum, void* stream) {
  if (!fovi::valid_dtype(dtype) || B < 0 || I <= 0 || J <= 0 || Jp < J || Bp < B || Bp <= 0) return FOVI_ERR_INVALID_ARGUMENT;
  if (!src || !dst) return FOVI_ERR_INVALID_ARGUMENT;
  if (si != 1 && sj != 1) return FOVI_ERR_UNSUPPORTED;
  const bool fused = act || masked || colsum;
  const bool fast_i = si == 1 && !(sj == 1 && J >= I);
  const int fast = fast_i ? I : Jp, slow = fast_i ? Jp : I;
  if (slow > 65535 || (fast + 31) / 32 > 65535) return FOVI_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int F = fast_i ? I : J;
  const size_t esz = fovi::dtype_size(dtype);
  const bool x2 = F % 2 == 0 && Bp % 2 == 0 && sb % 2 == 0 && (fast_i ? sj : si) % 2 == 0 &&
                  reinterpret_cast<uintptr_t>(src) % (2 * esz) == 0 && reinterpret_cast<uintptr_t>(dst) % 4 == 0 && (fast + 63) / 64 <= 65535;
  if (fused) {
    // the fused form exists for the two-element kernel only; the masked copy and the activations share the source's layout
    if (!x2 || (act && reinterpret_cast<uintptr_t>(act) % (2 * esz)) || (masked && reinterpret_cast<uintptr_t>(masked) % (2 * esz)))
      return FOVI_ERR_UNSUPPORTED;
    if (colsum) FOVI_CUDA(cudaMemsetAsync(colsum, 0, sizeof(float) * (size_t)F, st));
  }
  if (x2) {
    dim3 grid2((Bp + 63) / 64, (fast + 63) / 64, (slow + X2_SLOW - 1) / X2_SLOW), block2(32, 8);
#define RUN2(T, FI) batch_to_inner_x2_kernel<T, FI><<<grid2, block2, 0, st>>>((const T*)src, (__nv_bfloat16*)dst, B, I, J, Jp, Bp, sb, si, sj, \
                                                                              (const T*)act, (T*)masked, colsum)
    if (dtype == FOVI_F32) { if (fast_i) RUN2(float, true); else RUN2(float, false); }
    else { if (fast_i) RUN2(__nv_bfloat16, true); else RUN2(__nv_bfloat16, false); }
#undef RUN2
    return fovi::after_launch("batch_to_inner_x2_kernel");
  }
  dim3 grid((Bp + 31) / 32, (fast + 31) / 32, slow), block(32, 8);
#define RUN(T, FI) batch_to_inner_kernel<T, FI><<<grid, block, 0, st>>>((const T*)src, (__nv_bfloat16*)dst, B, I, J, Jp, Bp, sb, si, sj)
  if (dtype == FOVI_F32) { if (fast_i) RUN(float, true); else RUN(float, false); }
  else { if (fast_i) RUN(__nv_bfloat16, true); else RUN(__nv_bfloat16, false); }
#undef RUN
  return fovi::after_launch("batch_to_inner_kernel");
}

extern "C" int fovi_batch_to_inner(const void* src, int dtype, int B, int I, int J, long long sb, long long si, long long sj, void* dst,
                                   int Jp, int Bp, void* stream) {
  return batch_to_inner_impl(src, dtype, B, I, J, sb, si, sj, dst, Jp, Bp, nullptr, nullptr, nullptr, stream);
}

extern "C" int fovi_relu_backward_to_inner(const void* grad, const void* act, int dtype, int B, int I, int J, long long sb, long long si,
                                           long long sj, void* masked, void* dst, int Jp, int Bp, float* colsum, void* stream) {
  if (!act && !masked && !colsum) return FOVI_ERR_INVALID_ARGUMENT;
  return batch_to_inner_impl(grad, dtype, B, I, J, sb, si, sj, dst, Jp, Bp, act, masked, colsum, stream);
}
