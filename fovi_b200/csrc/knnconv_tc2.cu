// KNNConv, 64-channel mode, on CTA PAIRS (tcgen05 cta_group::2).
//
// Same table-driven gather-GEMM as knnconv_tc.cu, but one work item is 256 batch rows x one c_out tile,
// computed by a cluster of two CTAs on neighbouring SMs with a single M=256 MMA: each CTA stages its own
// 128 batch rows of the activations (A) and only HALF of the weight slab (B: c_out tile / 2 rows), and the
// tensor cores of both SMs read both halves.  The single-CTA kernel is bound by the L2 -> shared-memory
// stream (16 KB of A + 24-32 KB of B per 64-channel chunk, at the 64 B/clk/SM limit); halving B per SM
// cuts that stream by 30-33 % for the same MMA work.
//
// Roles per CTA (6 warps as before): warp 0 producer (both CTAs; loads land in the CTA's own shared memory
// but complete on the LEADER's "full" barrier), warp 1 MMA issuer (leader CTA only; both CTAs allocate and
// free tensor memory), warps 2-5 epilogue (both CTAs, each for its own 128 rows).
// Barriers: full[s] and acc_empty[a] are used in the leader's shared memory only (the peer's copies and
// epilogue threads signal them through cluster addresses); empty[s] and acc_full[a] exist in both CTAs and
// are signalled by the leader's tcgen05.commit, multicast to both.  No TMA load here is multicast.
// All waits are bounded; both CTAs always reach the closing cluster barrier.
#include "tc_common.cuh"

namespace {

struct Tc2Args {
  const int* nbr_idx; const uint16_t* nbr_tap; const int* nbr_cnt;
  const float* bias; void* Y; int* status;
  int kp, B, n_in, n_out, c_out, cp;
  int ct, n_ct, n_mt2, nstage, relu, y_f32, total_items;
  uint32_t stage_bytes, table_bytes;
  uint32_t wait_limit; int skip_loads;   // as in TcArgs
  const int* out_map; int n_out_y; int accumulate;   // see OutMode
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n barrier.cluster.wait.acquire;" ::: "memory");
}
// TMA load whose completion is counted on a barrier that may live in the peer CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs once the MMAs issued so far have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}

__device__ __forceinline__ void decode_item2(const Tc2Args& a, int item, int& n, int& mt2, int& ctile) {
  ctile = item % a.n_ct;
  const int t = item / a.n_ct;
  n = t % a.n_out;
  mt2 = t / a.n_out;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
fovi_knnconv_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Tc2Args a) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* basep = smem_raw + (base - raw);
  SmemHeader* hdr = reinterpret_cast<SmemHeader*>(basep);
  const uint32_t tbl_pitch = ((uint32_t)a.kp * 6u + 15u) & ~15u;
  unsigned char* tbl0 = basep + 1024;
  float* bias_s = reinterpret_cast<float*>(basep + 1024 + 2 * tbl_pitch);
  const uint32_t stages0 = base + 1024u + a.table_bytes;
  volatile int* abort_flag = &hdr->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0 = leader (issues the MMAs), 1 = peer
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int chunks = (a.cp + 63) / 64;   // a last box reaching past cp is zero-filled by the tensor copy
  const int half = a.ct / 2;                    // rows of B this CTA stages

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.nstage; ++s) { mbar_init(smem_u32(&hdr->full[s]), 1); mbar_init(smem_u32(&hdr->empty[s]), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&hdr->acc_full[i]), 1); mbar_init(smem_u32(&hdr->acc_empty[i]), 8); }
    mbar_init(smem_u32(&hdr->drain), 1);
    hdr->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // both CTAs of the pair allocate together: 512 columns = two accumulators of up to 256
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&hdr->tmem_base)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  // Programmatic dependent launch: let the next kernel of the stream be scheduled onto SMs as they free up (its
  // prologue then overlaps this kernel's tail), and hold this kernel's own first read of global data until the
  // kernel before it has completed.  Everything above (barriers, tensor memory) needed no global data.  Both are
  // no-ops when the kernel was launched without the attribute.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int i = threadIdx.x; i < a.c_out; i += blockDim.x) bias_s[i] = a.bias ? __ldg(a.bias + i) : 0.f;
  tc_fence_before();
  cluster_sync_all();   // barriers of both CTAs are initialised before anyone signals across
  tc_fence_after();
  const uint32_t tmem = hdr->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    uint32_t s = 0, ph = 0;
    bool ok = true;
    int item = a.skip_loads ? a.total_items : pair, buf = 0, cnt = 0;
    if (item < a.total_items) {
      int n, mt2, ctile;
      decode_item2(a, item, n, mt2, ctile);
      int* ti = reinterpret_cast<int*>(tbl0);
      uint16_t* tt = reinterpret_cast<uint16_t*>(tbl0 + (size_t)a.kp * 4);
      for (int k = lane; k < a.kp; k += 32) {
        ti[k] = __ldg(a.nbr_idx + (size_t)n * a.kp + k);
        tt[k] = __ldg(a.nbr_tap + (size_t)n * a.kp + k);
      }
      cnt = __ldg(a.nbr_cnt + n);
    }
    __syncwarp();
    while (item < a.total_items && ok) {
      const int next = item + n_pairs;
      int n, mt2, ctile;
      decode_item2(a, item, n, mt2, ctile);
      int r_idx[TBQ], cnt_next = 0;
      uint16_t r_tap[TBQ];
      if (next < a.total_items) {
        int n2, m2, c2;
        decode_item2(a, next, n2, m2, c2);
#pragma unroll
        for (int q = 0; q < TBQ; ++q) {
          const int k = lane + 32 * q;
          r_idx[q] = k < a.kp ? __ldg(a.nbr_idx + (size_t)n2 * a.kp + k) : 0;
          r_tap[q] = k < a.kp ? __ldg(a.nbr_tap + (size_t)n2 * a.kp + k) : (uint16_t)0;
        }
        cnt_next = __ldg(a.nbr_cnt + n2);
      }
      const int* tb_idx = reinterpret_cast<const int*>(tbl0 + buf * tbl_pitch);
      const uint16_t* tb_tap = reinterpret_cast<const uint16_t*>(tbl0 + buf * tbl_pitch + (size_t)a.kp * 4);
      if (lane == 0) {
        const int m0 = (mt2 * 2 + (int)rank) * BM;            // this CTA's 128 batch rows
        const int o0 = ctile * a.ct + (int)rank * half;       // this CTA's half of the c_out tile
        const int steps = cnt * chunks;
        int k = 0, cc = 0;
        for (int st = 0; st < steps; ++st) {
          if (!mbar_wait(smem_u32(&hdr->empty[s]), ph ^ 1u, abort_flag, a.status, 11, a.wait_limit)) { ok = false; break; }
          const uint32_t full_leader = map_to_cta(smem_u32(&hdr->full[s]), 0);
          if (rank == 0) mbar_expect_tx(smem_u32(&hdr->full[s]), 2u * a.stage_bytes);   // both CTAs' bytes
          const uint32_t sa = stages0 + s * a.stage_bytes;
          tma_load_3d_pair(sa, &tmA, full_leader, cc * 64, tb_idx[k], m0);
          tma_load_3d_pair(sa + A_STAGE_BYTES, &tmB, full_leader, cc * 64, o0, tb_tap[k]);
          if (++cc == chunks) { cc = 0; ++k; }
          if (++s == (uint32_t)a.nstage) { s = 0; ph ^= 1u; }
        }
      }
      __syncwarp();
      if (next < a.total_items) {
        int* ti = reinterpret_cast<int*>(tbl0 + (buf ^ 1) * tbl_pitch);
        uint16_t* tt = reinterpret_cast<uint16_t*>(tbl0 + (buf ^ 1) * tbl_pitch + (size_t)a.kp * 4);
#pragma unroll
        for (int q = 0; q < TBQ; ++q) {
          const int k = lane + 32 * q;
          if (k < a.kp) { ti[k] = r_idx[q]; tt[k] = r_tap[q]; }
        }
      }
      __syncwarp();
      s = __shfl_sync(0xffffffffu, s, 0); ph = __shfl_sync(0xffffffffu, ph, 0);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      buf ^= 1; cnt = cnt_next; item = next;
    }
    if (lane == 0 && *abort_flag) {
      // Give copies that are still in flight time to land before this CTA's shared memory goes away.
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.ct >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
      uint32_t s = 0, ph = 0, acc = 0, aph = 0;
      bool ok = true;
      int cnt = pair < a.total_items ? __ldg(a.nbr_cnt + (pair / a.n_ct) % a.n_out) : 0;
      for (int item = pair; item < a.total_items && ok; item += n_pairs) {
        const int next = item + n_pairs;
        const int cnt_next = next < a.total_items ? __ldg(a.nbr_cnt + (next / a.n_ct) % a.n_out) : 0;
        const int steps = cnt * chunks;
        if (!mbar_wait(smem_u32(&hdr->acc_empty[acc]), aph ^ 1u, abort_flag, a.status, 12, a.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem + acc * 256u;
        for (int st = 0; st < steps; ++st) {
          if (!mbar_wait(smem_u32(&hdr->full[s]), ph, abort_flag, a.status, 13, a.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = stages0 + s * a.stage_bytes, sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma_bf16_pair(d_tmem, smem_desc(sa + kk * 32u, 16u, 1024u, 2u), smem_desc(sb + kk * 32u, 16u, 1024u, 2u), idesc,
                             (st | kk) ? 1u : 0u);
          tc_commit_pair(smem_u32(&hdr->empty[s]));      // frees the stage in both CTAs
          if (++s == (uint32_t)a.nstage) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        tc_commit_pair(smem_u32(&hdr->acc_full[acc]));   // accumulator halves complete in both CTAs
        if (++acc == 2) { acc = 0; aph ^= 1u; }
        cnt = cnt_next;
      }
      if (*abort_flag) {
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&hdr->drain)) : "memory");
        for (uint32_t it = 0; it < (1u << 20); ++it)
          if (mbar_try_wait(smem_u32(&hdr->drain), 0)) break;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    uint32_t acc = 0, aph = 0;
    bool ok = true;
    int cnt = pair < a.total_items ? __ldg(a.nbr_cnt + (pair / a.n_ct) % a.n_out) : 0;
    for (int item = pair; item < a.total_items && ok; item += n_pairs) {
      int n, mt2, ctile;
      decode_item2(a, item, n, mt2, ctile);
      const int next = item + n_pairs;
      const int cnt_next = next < a.total_items ? __ldg(a.nbr_cnt + (next / a.n_ct) % a.n_out) : 0;
      ok = mbar_wait(smem_u32(&hdr->acc_full[acc]), aph, abort_flag, a.status, 14, a.wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = (mt2 * 2 + (int)rank) * BM + q * 32 + lane;
      const int o0 = ctile * a.ct;
      const int n_y = a.out_map ? __ldg(a.out_map + n) : n;
      const size_t y_off = ((size_t)row * a.n_out_y + n_y) * a.c_out + o0;
      const uint32_t t_base = tmem + ((uint32_t)(q * 32) << 16) + acc * 256u;
      for (int c0 = 0; c0 < a.ct; c0 += 64) {
        uint32_t r[64];
        const int w = min(64, a.ct - c0);   // 32 or 64 (ct is a multiple of 32 here)
        tc_ld32(t_base + c0, r);
        if (w == 64) tc_ld32(t_base + c0 + 32, r + 32);
        tc_ld_wait();
        if (cnt <= 0) {   // a point without neighbours: nothing was accumulated, the columns hold an earlier item's values
#pragma unroll
          for (int i = 0; i < 64; ++i) r[i] = 0u;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (g * 16 < w) {
            float v[16];
            const float4* b4 = reinterpret_cast<const float4*>(bias_s + o0 + c0 + g * 16);   // 64-byte aligned
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 bb = b4[i];
              v[4 * i] = __uint_as_float(r[g * 16 + 4 * i]) + bb.x;
              v[4 * i + 1] = __uint_as_float(r[g * 16 + 4 * i + 1]) + bb.y;
              v[4 * i + 2] = __uint_as_float(r[g * 16 + 4 * i + 2]) + bb.z;
              v[4 * i + 3] = __uint_as_float(r[g * 16 + 4 * i + 3]) + bb.w;
            }
            if (a.relu) {
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.f);
            }
            if (row < a.B) {
              if (a.accumulate) {
                float* dst = reinterpret_cast<float*>(a.Y) + y_off + c0 + g * 16;
                if (cnt > 0) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) red_add_f32x4(dst + 4 * i, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                }
              } else if (a.y_f32) {
                float* dst = reinterpret_cast<float*>(a.Y) + y_off + c0 + g * 16;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                  uint32_t w8[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) w8[e] = __float_as_uint(v[8 * i + e]);
                  st_global_32(dst + 8 * i, w8);
                }
              } else {
                uint32_t pk[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                  pk[i] = *reinterpret_cast<uint32_t*>(&h);
                }
                st_global_32(reinterpret_cast<__nv_bfloat16*>(a.Y) + y_off + c0 + g * 16, pk);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();   // every lane has finished reading the accumulator; one arrival per warp (8 in the pair)
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&hdr->acc_empty[acc]), 0));   // the leader's MMA thread waits for all 8
      if (++acc == 2) { acc = 0; aph ^= 1u; }
      cnt = cnt_next;
    }
  }

  tc_fence_before();
  cluster_sync_all();   // nobody frees tensor memory or leaves while the other CTA may still signal or read
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
  }
}

}  // namespace

int fovi::launch_knnconv_tc_pair(const fovi_knnconv_plan* p, const void* X, const void* Wt, const float* bias, void* Y, int y_dtype,
                                 int B, int relu, cudaStream_t st, int skip_loads, uint32_t wait_limit, const OutMode& om) {
  const int ct = p->ct, cp = p->cin_packed;
  if (p->x_layout != FOVI_X_BNC || cp < 16 || !ct || ct % 32 || ct < 32 || B <= BM) return FOVI_ERR_UNSUPPORTED;
  const int sms = fovi::sm_count();
  if (sms < 2) return FOVI_ERR_UNSUPPORTED;
  Tc2Args a;
  a.nbr_idx = p->nbr_idx; a.nbr_tap = p->nbr_tap; a.nbr_cnt = p->nbr_cnt;
  a.bias = bias; a.Y = Y; a.status = p->status;
  a.kp = p->kp; a.B = B; a.n_in = p->n_in; a.n_out = p->n_out; a.c_out = p->c_out; a.cp = cp;
  a.ct = ct; a.n_ct = p->c_out / ct; a.n_mt2 = (B + 2 * BM - 1) / (2 * BM);
  a.relu = relu; a.y_f32 = y_dtype == FOVI_F32;
  a.wait_limit = wait_limit; a.skip_loads = skip_loads;
  a.out_map = om.out_map; a.n_out_y = om.out_map ? om.n_out_y : p->n_out; a.accumulate = om.accumulate;
  const long long items = (long long)a.n_mt2 * p->n_out * a.n_ct;
  if (items >= (1ll << 31) || a.kp > 32 * TBQ) return FOVI_ERR_UNSUPPORTED;
  a.total_items = (int)items;
  a.stage_bytes = A_STAGE_BYTES + (uint32_t)(ct / 2) * 128u;
  a.table_bytes = (2u * (((uint32_t)a.kp * 6u + 15u) & ~15u) + (uint32_t)p->c_out * 4u + 1023u) & ~1023u;
  const uint32_t budget = 220u * 1024u - 2048u - a.table_bytes;
  a.nstage = (int)std::min<uint32_t>(MAX_STAGES, budget / a.stage_bytes);
  if (a.nstage < 2) return FOVI_ERR_UNSUPPORTED;
  const size_t smem = 1024 + 1024 + a.table_bytes + (size_t)a.nstage * a.stage_bytes;

  CUtensorMap tmA, tmB;
  int rc = fovi::encode_3d(&tmA, X, (uint64_t)cp, (uint64_t)p->n_in, (uint64_t)B, (uint64_t)cp * 2, (uint64_t)p->n_in * cp * 2, 64, 1, BM, true);
  if (rc) return rc;
  rc = fovi::encode_3d(&tmB, Wt, (uint64_t)cp, (uint64_t)p->c_out, (uint64_t)p->V, (uint64_t)cp * 2, (uint64_t)p->c_out * cp * 2, 64, (uint32_t)(ct / 2), 1, true);
  if (rc) return rc;

  FOVI_CUDA(cudaFuncSetAttribute(fovi_knnconv_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int pairs = (int)std::min<long long>(items, sms / 2);
  FOVI_CUDA(fovi::launch_pdl(fovi_knnconv_tc_pair_kernel, 2 * pairs, 192, smem, st, tmA, tmB, a));   // cluster size 2 comes from __cluster_dims__
  return fovi::after_launch("fovi_knnconv_tc_pair_kernel");
}
