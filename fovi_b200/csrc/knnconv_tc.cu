// KNNConv on the 5th-generation tensor cores (tcgen05 MMA, accumulators in tensor memory).
//
//   out[b, n, o] = bias[o] + sum_k sum_c X[b, idx[n,k], c] * Wt[tap[n,k]][o][c]
//
// For one output point n the sum over (k, c) is an ordinary GEMM whose M dimension is the
// batch: D[128 batch rows, c_out tile] += A_k[128, c] * B_k[c, c_out tile], where
//   A_k = X[b0:b0+128, idx[n,k], :]   a strided 2-D box of the channels-last activations,
//   B_k = Wt[tap[n,k]]                one slab of the tap-major packed weights.
// Both operands are therefore plain tiled TMA boxes chosen by the neighbour table, no element
// gather is needed, pad neighbours are skipped (the plan compacted them away) and the V/K-fold
// zero work of a one-hot scatter formulation never exists.
//
// CTA = 6 warps, persistent over work items (batch tile, output point, c_out tile):
//   warp 0      producer: stages the item's (idx, tap) list in shared memory, then one lane
//               issues the TMA loads into a ring of shared-memory stages;
//   warp 1      one lane issues tcgen05.mma (M=128, N=c_out tile, K=16) and commits to
//               mbarriers; the warp owns the tensor-memory allocation;
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (double-buffered in tensor
//               memory so the next item's MMAs overlap), add bias, ReLU, convert, store.
//
// Three operand modes:
//   C64    channels packed to a multiple of 64: a stage is one 64-channel chunk of one neighbour,
//          128-byte-swizzled K-major tiles (4 MMAs of K=16 per stage);
//   C8     any other multiple of 8 channels: a stage is eight (neighbour, 8-channel chunk) boxes
//          of 16-byte rows in the un-swizzled core-matrix layout; one MMA (K=16) consumes two
//          boxes.  Tail boxes read the out-of-range point index n_in, which TMA fills with zeros;
//   PAIRS  c_in <= 4 (RGB first layers, patch embeddings): activations are stored pair-major,
//          [point pair][batch row][2 points x 4 channels], so the 128 batch rows of one pair are
//          ONE contiguous 2 KB block that already is the un-swizzled core-matrix layout, and the
//          weights are pre-gathered per output point and c_out tile so the eight slabs of a stage
//          are one contiguous block too.  Both move with plain bulk copies (cp.async.bulk): the plan
//          precomputed the runs of consecutive pairs of every stage, one copy each, and the lanes of the
//          producer warp issue a stage's copies together (the copy-issue rate is what bounds this mode).
//          One MMA (K=16) consumes two pairs = four neighbours.  Unused slots read a block of
//          zeros; rows past the batch keep stale shared memory, which only reaches output rows
//          that are never stored.
//
// Every wait is bounded: a wait that gives up raises a CTA-wide abort flag and a status word in
// global memory (read back by fovi_knnconv_check); all roles then drain and leave normally, the
// tensor memory is freed and the context stays usable.
#include "tc_common.cuh"

// Tuning constants (compile-time; a comparison build overrides them with -D).
#ifndef FOVI_TC_C64_MIN
#define FOVI_TC_C64_MIN 16          // packed channel count from which 64-channel swizzled boxes are used
#endif
#ifndef FOVI_TC_SINGLE_CTA_ONLY
#define FOVI_TC_SINGLE_CTA_ONLY 0   // 1: never use the CTA-pair kernel
#endif
#ifndef FOVI_TC_PAIR_CTAS
#define FOVI_TC_PAIR_CTAS 3         // pair mode: CTAs per SM at most
#endif
#ifndef FOVI_TC_PAIR_GROUPS
#define FOVI_TC_PAIR_GROUPS 2       // pair mode: stages the producer warp fills per pass
#endif

namespace {

template <int MODE>
__global__ void __launch_bounds__(192, MODE == MODE_PAIRS ? 3 : 1)
fovi_knnconv_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcArgs a) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* basep = smem_raw + (base - raw);
  SmemHeader* hdr = reinterpret_cast<SmemHeader*>(basep);
  // two table buffers (the next item's list is prefetched while the current one is issued), then the bias
  const uint32_t tbl_pitch = ((uint32_t)a.kp * 6u + 15u) & ~15u;
  unsigned char* tbl0 = basep + 1024;
  float* bias_s = reinterpret_cast<float*>(basep + 1024 + 2 * tbl_pitch);
  const uint32_t stages0 = base + 1024u + a.table_bytes;  // 1024-aligned
  volatile int* abort_flag = &hdr->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t b_stage_off = A_STAGE_BYTES;
  constexpr bool C64 = MODE == MODE_C64;
  // operand boxes per list entry; a last 64-channel box that reaches past cp is zero-filled by the tensor copy
  const int chunks = C64 ? (a.cp + 63) / 64 : (MODE == MODE_PAIRS ? 1 : a.cp / 8);

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.nstage; ++s) { mbar_init(smem_u32(&hdr->full[s]), 1); mbar_init(smem_u32(&hdr->empty[s]), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&hdr->acc_full[i]), 1); mbar_init(smem_u32(&hdr->acc_empty[i]), 4); }
    mbar_init(smem_u32(&hdr->drain), 1);
    hdr->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory for two accumulators (all 512 columns when the c_out tile is wider than 128)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&hdr->tmem_base)), "r"(a.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Programmatic dependent launch: let the next kernel of the stream be scheduled onto SMs as they free up (its
  // prologue then overlaps this kernel's tail), and hold this kernel's own first read of global data until the
  // kernel before it has completed.  Everything above (barriers, tensor memory) needed no global data.  Both are
  // no-ops when the kernel was launched without the attribute.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int i = threadIdx.x; i < a.c_out; i += blockDim.x) bias_s[i] = a.bias ? __ldg(a.bias + i) : 0.f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = hdr->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    uint32_t s = 0, ph = 0;
    uint32_t issued = 0;
    bool ok = true;
    int item = a.skip_loads ? a.total_items : blockIdx.x, buf = 0, cnt = 0;
    if (item < a.total_items) {  // first item's list straight into buffer 0
      int n, mt, ctile;
      decode_item(a, item, n, mt, ctile);
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
      const int next = item + gridDim.x;
      int n, mt, ctile;
      decode_item(a, item, n, mt, ctile);
      // prefetch the next item's list into registers: the loads are in flight while lane 0 issues copies
      int r_idx[TBQ], cnt_next = 0;
      uint16_t r_tap[TBQ];
      if (next < a.total_items) {
        int n2, mt2, ct2;
        decode_item(a, next, n2, mt2, ct2);
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
      const int m0 = mt * BM, o0 = ctile * a.ct;
      if (MODE == MODE_PAIRS) {
        // The whole warp issues, several stages per pass: the warp is cut into groups of nine lanes, group j takes stage
        // st0 + j; its first lane waits for that stage to be free and arms its barrier, then lane i < 8 copies the 2 KB
        // blocks starting at slot i and lane 8 the eight weight slabs.  (A single thread pays the wait and the full issue
        // cost of every copy in sequence, about a thousand cycles per stage; here a pass costs that once for a.pgroups
        // stages.  pgroups < nstage, so the consumer always has a loaded stage while the producer waits;
        // two stages per pass measured best: 154 / 126 / 148 us with 1 / 2 / 3 on the grouped 3->64 first layer.)
        const int steps = (cnt + 7) / 8;
        const uint32_t b_bytes = 8u * (uint32_t)a.ct * 16u;
        const unsigned char* wn = a.Wt + ((size_t)n * a.n_ct + ctile) * a.kp * ((size_t)a.ct * 16);
        const unsigned char* xt = a.X + (size_t)mt * a.n_pairs * 2048;  // this batch tile's pair blocks
        const int grp = lane / 9, gl = lane - grp * 9;
        for (int st0 = 0; st0 < steps; st0 += a.pgroups) {
          const int my_st = st0 + grp;
          const bool active = grp < a.pgroups && my_st < steps;
          uint32_t my_s = s + (uint32_t)grp, my_ph = ph;
          if (my_s >= (uint32_t)a.nstage) { my_s -= (uint32_t)a.nstage; my_ph ^= 1u; }
          const uint32_t full = smem_u32(&hdr->full[my_s]);
          // what this lane will copy, worked out before the wait (one copy per lane, all issued by the same instruction)
          uint32_t dst = 0, bytes = 0;
          const unsigned char* src = nullptr;
          if (active) {
            const uint32_t sa = stages0 + my_s * a.stage_bytes;
            if (gl < 8) {
              // the plan marked the first slot of every run of consecutive pairs with the run's length (the unused
              // tail, whose slots hold n_pairs, is one run of zeros): one copy per run
              const uint32_t len = tb_tap[my_st * 8 + gl];
              if (len) {
                const int pr = tb_idx[my_st * 8 + gl];
                dst = sa + gl * 2048u; src = pr < a.n_pairs ? xt + (size_t)pr * 2048 : a.zero_block; bytes = len * 2048u;
              }
            } else {
              dst = sa + b_stage_off; src = wn + (size_t)my_st * b_bytes; bytes = b_bytes;
            }
          }
          bool mine = true;
          if (active && gl == 0) {
            mine = mbar_wait(smem_u32(&hdr->empty[my_s]), my_ph ^ 1u, abort_flag, a.status, 1, a.wait_limit);
            if (mine) mbar_expect_tx(full, a.stage_bytes);
          }
          ok = __all_sync(0xffffffffu, mine);   // also: nobody copies into a stage before its group's first lane saw it free
          if (!ok) break;
          if (bytes) bulk_load(dst, src, bytes, full);
          const uint32_t done = (uint32_t)min(a.pgroups, steps - st0);
          issued += done;
          s += done;
          if (s >= (uint32_t)a.nstage) { s -= (uint32_t)a.nstage; ph ^= 1u; }
        }
      } else if (MODE == MODE_C8) {
        // Eight 16-byte-row boxes of each operand per stage: lanes 0-7 issue the activation boxes, lanes 8-15 the weight
        // boxes, all with one instruction (a single thread would pay the issue cost of sixteen tensor copies in sequence).
        const int boxes = cnt * chunks;
        const int steps = (boxes + 7) / 8;
        const int j = lane & 7;
        const bool is_b = lane >= 8;
        for (int st = 0; st < steps; ++st) {
          const uint32_t full = smem_u32(&hdr->full[s]);
          bool mine = true;
          if (lane == 0) {
            mine = mbar_wait(smem_u32(&hdr->empty[s]), ph ^ 1u, abort_flag, a.status, 1, a.wait_limit);
            if (mine) mbar_expect_tx(full, a.stage_bytes);
          }
          ok = __all_sync(0xffffffffu, mine);
          if (!ok) break;
          if (lane < 16) {
            const int b = st * 8 + j;
            const int k = b / chunks, cc = b - k * chunks;
            const bool live = k < cnt;                       // boxes past the list read the zero row / tap 0
            const uint32_t sa = stages0 + s * a.stage_bytes;
            const uint32_t dst = is_b ? sa + b_stage_off + j * (uint32_t)a.ct * 16u : sa + j * 2048u;
            const int c1 = is_b ? o0 : (live ? tb_idx[k] : a.n_in);
            const int c2 = is_b ? (live ? (int)tb_tap[k] : 0) : m0;
            tma_load_3d(dst, is_b ? &tmB : &tmA, full, cc * 8, c1, c2);
          }
          ++issued;
          if (++s == (uint32_t)a.nstage) { s = 0; ph ^= 1u; }
        }
      } else if (lane == 0) {
        const int steps = cnt * chunks;
        int k = 0, cc = 0;
        for (int st = 0; st < steps; ++st) {
          const uint32_t full = smem_u32(&hdr->full[s]);
          if (!mbar_wait(smem_u32(&hdr->empty[s]), ph ^ 1u, abort_flag, a.status, 1, a.wait_limit)) { ok = false; break; }
          mbar_expect_tx(full, a.stage_bytes);
          const uint32_t sa = stages0 + s * a.stage_bytes;
          tma_load_3d(sa, &tmA, full, cc * 64, tb_idx[k], m0);
          tma_load_3d(sa + b_stage_off, &tmB, full, cc * 64, o0, tb_tap[k]);
          ++issued;
          if (++cc == chunks) { cc = 0; ++k; }
          if (++s == (uint32_t)a.nstage) { s = 0; ph ^= 1u; }
        }
      }
      if (MODE != MODE_PAIRS) {  // lane 0 carried the ring position and the outcome
        s = __shfl_sync(0xffffffffu, s, 0); ph = __shfl_sync(0xffffffffu, ph, 0); issued = __shfl_sync(0xffffffffu, issued, 0);
      }
      __syncwarp();
      if (next < a.total_items) {  // park the prefetched list in the other buffer
        int* ti = reinterpret_cast<int*>(tbl0 + (buf ^ 1) * tbl_pitch);
        uint16_t* tt = reinterpret_cast<uint16_t*>(tbl0 + (buf ^ 1) * tbl_pitch + (size_t)a.kp * 4);
#pragma unroll
        for (int q = 0; q < TBQ; ++q) {
          const int k = lane + 32 * q;
          if (k < a.kp) { ti[k] = r_idx[q]; tt[k] = r_tap[q]; }
        }
      }
      __syncwarp();
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      buf ^= 1; cnt = cnt_next; item = next;
    }
    if (lane == 0 && *abort_flag) {
      // Drain: wait (bounded, errors ignored) for the loads this thread armed and nobody consumed.
      const uint32_t back = issued < (uint32_t)a.nstage ? issued : (uint32_t)a.nstage;
      uint32_t ds = s, dph = ph;
      for (uint32_t i = 0; i < back; ++i) {
        if (ds == 0) { ds = a.nstage - 1; dph ^= 1u; } else { --ds; }
        for (uint32_t it = 0; it < (1u << 16); ++it)
          if (mbar_try_wait(smem_u32(&hdr->full[ds]), dph)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.ct >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      uint32_t s = 0, ph = 0, acc = 0, aph = 0;
      bool ok = true;
      int cnt = blockIdx.x < a.total_items ? __ldg(a.nbr_cnt + item_point(a, blockIdx.x)) : 0;
      for (int item = blockIdx.x; item < a.total_items && ok; item += gridDim.x) {
        const int next = item + gridDim.x;
        const int cnt_next = next < a.total_items ? __ldg(a.nbr_cnt + item_point(a, next)) : 0;  // consumed next round
        const int steps = C64 ? cnt * chunks : (cnt * chunks + 7) / 8;
        if (!mbar_wait(smem_u32(&hdr->acc_empty[acc]), aph ^ 1u, abort_flag, a.status, 2, a.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem + acc * a.acc_cols;
        for (int st = 0; st < steps; ++st) {
          if (!mbar_wait(smem_u32(&hdr->full[s]), ph, abort_flag, a.status, 3, a.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = stages0 + s * a.stage_bytes, sb = sa + b_stage_off;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            uint64_t da, db;
            if (C64) {
              da = smem_desc(sa + kk * 32u, 16u, 1024u, 2u);
              db = smem_desc(sb + kk * 32u, 16u, 1024u, 2u);
            } else {
              da = smem_desc(sa + kk * 4096u, 2048u, 128u, 0u);
              db = smem_desc(sb + kk * 2u * (uint32_t)a.ct * 16u, (uint32_t)a.ct * 16u, 128u, 0u);
            }
            tc_mma_bf16(d_tmem, da, db, idesc, (st | kk) ? 1u : 0u);
          }
          tc_commit(smem_u32(&hdr->empty[s]));  // frees the stage once these MMAs have read it
          if (++s == (uint32_t)a.nstage) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        tc_commit(smem_u32(&hdr->acc_full[acc]));  // accumulator complete
        if (++acc == 2) { acc = 0; aph ^= 1u; }
        cnt = cnt_next;
      }
      if (*abort_flag) {  // make sure no MMA is still reading shared memory / writing tensor memory
        tc_commit(smem_u32(&hdr->drain));
        for (uint32_t it = 0; it < (1u << 20); ++it)
          if (mbar_try_wait(smem_u32(&hdr->drain), 0)) break;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    uint32_t acc = 0, aph = 0;
    bool ok = true;
    int cnt = blockIdx.x < a.total_items ? __ldg(a.nbr_cnt + item_point(a, blockIdx.x)) : 0;
    for (int item = blockIdx.x; item < a.total_items && ok; item += gridDim.x) {
      int n, mt, ctile;
      decode_item(a, item, n, mt, ctile);
      const int next = item + gridDim.x;
      const int cnt_next = next < a.total_items ? __ldg(a.nbr_cnt + item_point(a, next)) : 0;
      ok = mbar_wait(smem_u32(&hdr->acc_full[acc]), aph, abort_flag, a.status, 4, a.wait_limit);
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below is warp-collective: leave as a whole warp or not at all
      if (!ok) break;
      tc_fence_after();
      const int row = mt * BM + q * 32 + lane;
      const int o0 = ctile * a.ct;
      const int n_y = a.out_map ? __ldg(a.out_map + n) : n;
      const size_t y_off = ((size_t)row * a.n_out_y + n_y) * a.c_out + o0;
      const uint32_t t_base = tmem + ((uint32_t)(q * 32) << 16) + acc * a.acc_cols;
      // 64 accumulator columns per round: two 32-column tensor-memory loads in flight, one wait
      for (int c0 = 0; c0 < a.ct; c0 += 64) {
        uint32_t r[64];
        const int w = min(64, a.ct - c0);  // 16, 32, 48 or 64 (ct is a multiple of 16)
        if (w >= 32) tc_ld32(t_base + c0, r); else tc_ld16(t_base + c0, *reinterpret_cast<uint32_t(*)[16]>(r));
        if (w == 64) tc_ld32(t_base + c0 + 32, r + 32);
        else if (w == 48) tc_ld16(t_base + c0 + 32, *reinterpret_cast<uint32_t(*)[16]>(r + 32));
        tc_ld_wait();
        if (cnt <= 0) {   // a point without neighbours: nothing was accumulated, the columns hold an earlier item's values
#pragma unroll
          for (int i = 0; i < 64; ++i) r[i] = 0u;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {  // groups of 16 columns
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
      __syncwarp();   // every lane has finished reading the accumulator; one arrival per epilogue warp
      if (lane == 0) mbar_arrive(smem_u32(&hdr->acc_empty[acc]));
      if (++acc == 2) { acc = 0; aph ^= 1u; }
      cnt = cnt_next;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(a.tmem_cols) : "memory");
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

}  // namespace

int fovi::encode_3d(CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                    uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2, bool swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { fovi::g_last_cuda_error = "cuTensorMapEncodeTiled entry point not available"; return FOVI_ERR_CUDA; }
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fovi::g_last_cuda_error = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r);
    return FOVI_ERR_CUDA;
  }
  return FOVI_OK;
}

static int knnconv_forward_impl(fovi_knnconv_plan* p, const void* X, const void* Wt, const float* bias, void* Y, int y_dtype, int B,
                                int relu, void* stream, int skip_loads, uint32_t wait_limit, const OutMode& om = OutMode()) {
  if (!p || B < 0 || !fovi::valid_dtype(y_dtype)) return FOVI_ERR_INVALID_ARGUMENT;
  if (B == 0) return FOVI_OK;  // an empty batch has no buffers to look at
  if (!X || !Wt || !Y) return FOVI_ERR_INVALID_ARGUMENT;
  if (p->c_out % 16) return FOVI_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(Wt) | reinterpret_cast<uintptr_t>(Y)) & 15) return FOVI_ERR_ALIGNMENT;
  const int ct = p->ct;
  if (!ct) return FOVI_ERR_UNSUPPORTED;
  const int cp = p->cin_packed;
  // 64-channel swizzled boxes for every layer of at least 16 channels: when cp is not a multiple of 64 the last box of a
  // neighbour reaches past the tensor's channel extent and the copy fills those columns with zeros.  Wasted MMA columns are
  // cheap next to 16-byte-row boxes, whose stages take 1.7 us (96 -> 256 channels, 1024 rows: 0.81 -> 0.25 ms; 16 / 32 / 48
  // -> 64 channels: 97 / 86 / 110 -> 54 / 56 / 56 us).
  const bool c64 = cp >= FOVI_TC_C64_MIN && p->x_layout != FOVI_X_PAIRS;
  // 64-channel layers with more than one batch tile run on CTA pairs (half the weight traffic per SM).
  if (c64 && !FOVI_TC_SINGLE_CTA_ONLY && B > BM && ct % 32 == 0) {
    const int rc2 = fovi::launch_knnconv_tc_pair(p, X, Wt, bias, Y, y_dtype, B, relu, reinterpret_cast<cudaStream_t>(stream), skip_loads, wait_limit, om);
    if (rc2 != FOVI_ERR_UNSUPPORTED) return rc2;
  }

  TcArgs a;
  const bool pairs = p->x_layout == FOVI_X_PAIRS;
  a.nbr_idx = pairs ? p->pair_idx : p->nbr_idx; a.nbr_tap = pairs ? p->pair_run : p->nbr_tap; a.nbr_cnt = pairs ? p->pair_cnt : p->nbr_cnt;
  a.bias = bias; a.Y = Y; a.status = p->status;
  a.kp = pairs ? p->sp : p->kp; a.B = B; a.n_in = p->n_in; a.n_out = p->n_out; a.c_out = p->c_out; a.cp = cp;
  a.ct = ct; a.n_ct = p->c_out / ct; a.n_mt = (B + BM - 1) / BM;
  a.relu = relu; a.y_f32 = y_dtype == FOVI_F32;
  a.wait_limit = wait_limit; a.skip_loads = skip_loads;
  a.out_map = om.out_map; a.n_out_y = om.out_map ? om.n_out_y : p->n_out; a.accumulate = om.accumulate;
  a.mt_fastest = pairs ? 1 : 0;
  const long long items = (long long)a.n_mt * p->n_out * a.n_ct;
  if (items >= (1ll << 31)) return FOVI_ERR_UNSUPPORTED;
  a.total_items = (int)items;
  a.stage_bytes = A_STAGE_BYTES + (uint32_t)ct * 128u;  // A: 128 rows x 128 B;  B: ct rows x 128 B (any mode)
  if (a.kp > 32 * TBQ) return FOVI_ERR_UNSUPPORTED;  // neighbour lists longer than 256 entries
  a.table_bytes = (2u * (((uint32_t)a.kp * 6u + 15u) & ~15u) + (uint32_t)p->c_out * 4u + 1023u) & ~1023u;
  a.acc_cols = 32;
  while ((int)a.acc_cols < ct) a.acc_cols <<= 1;
  a.tmem_cols = 2 * a.acc_cols;
  // Pair mode with a narrow c_out tile is bound by per-item latencies (copy issue, short neighbour lists, small MMAs),
  // not by bandwidth: up to three CTAs per SM, each with fewer stages and a share of the tensor memory, overlap them
  // (measured on the 3->64 first layer: 0.29 / 0.17 / 0.16 ms with 1 / 2 / 3 CTAs per SM).
  constexpr int pair_ctas = FOVI_TC_PAIR_CTAS;
  const int ctas_per_sm = !pairs ? 1 : (a.tmem_cols <= 128 && pair_ctas >= 3) ? 3 : (a.tmem_cols <= 256 && pair_ctas >= 2) ? 2 : 1;
  const uint32_t budget = (ctas_per_sm == 3 ? 73u : ctas_per_sm == 2 ? 110u : 220u) * 1024u - 2048u - a.table_bytes;
  a.nstage = (int)std::min<uint32_t>(MAX_STAGES, budget / a.stage_bytes);
  if (a.nstage < 2) return FOVI_ERR_UNSUPPORTED;
  a.pgroups = std::max(1, std::min(std::min(FOVI_TC_PAIR_GROUPS, 3), a.nstage - 1));
  const size_t smem = 1024 /*align slack*/ + 1024 /*header*/ + a.table_bytes + (size_t)a.nstage * a.stage_bytes;

  CUtensorMap tmA, tmB;
  const uint32_t kc = c64 ? 64 : 8;
  int rc;
  a.X = static_cast<const unsigned char*>(X); a.Wt = static_cast<const unsigned char*>(Wt);
  a.zero_block = static_cast<const unsigned char*>(p->zero_block); a.n_pairs = p->n_pairs;
  if (pairs) {
    // operands move with plain bulk copies; the tensor maps are unused placeholders
    memset(&tmA, 0, sizeof(tmA)); memset(&tmB, 0, sizeof(tmB));
    rc = FOVI_OK;
  } else {
    rc = fovi::encode_3d(&tmA, X, (uint64_t)cp, (uint64_t)p->n_in, (uint64_t)B, (uint64_t)cp * 2, (uint64_t)p->n_in * cp * 2, kc, 1, BM, c64);
    if (rc) return rc;
    rc = fovi::encode_3d(&tmB, Wt, (uint64_t)cp, (uint64_t)p->c_out, (uint64_t)p->V, (uint64_t)cp * 2, (uint64_t)p->c_out * cp * 2, kc, (uint32_t)ct, 1, c64);
  }
  if (rc) return rc;

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = std::min(a.total_items, ctas_per_sm * fovi::sm_count());
  if (pairs) {
    FOVI_CUDA(cudaFuncSetAttribute(fovi_knnconv_tc_kernel<MODE_PAIRS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FOVI_CUDA(fovi::launch_pdl(fovi_knnconv_tc_kernel<MODE_PAIRS>, grid, 192, smem, st, tmA, tmB, a));
  } else if (c64) {
    FOVI_CUDA(cudaFuncSetAttribute(fovi_knnconv_tc_kernel<MODE_C64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FOVI_CUDA(fovi::launch_pdl(fovi_knnconv_tc_kernel<MODE_C64>, grid, 192, smem, st, tmA, tmB, a));
  } else {
    FOVI_CUDA(cudaFuncSetAttribute(fovi_knnconv_tc_kernel<MODE_C8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FOVI_CUDA(fovi::launch_pdl(fovi_knnconv_tc_kernel<MODE_C8>, grid, 192, smem, st, tmA, tmB, a));
  }
  return fovi::after_launch("fovi_knnconv_tc_kernel");
}

extern "C" int fovi_knnconv_forward(fovi_knnconv_plan* p, const void* X, const void* Wt, const float* bias, void* Y,
                                    int y_dtype, int B, int relu, void* stream) {
  return knnconv_forward_impl(p, X, Wt, bias, Y, y_dtype, B, relu, stream, 0, WAIT_LIMIT);
}

extern "C" int fovi_knnconv_forward_scatter_add(fovi_knnconv_plan* p, const void* X, const void* Wt, float* Y, int B, const int* out_map,
                                               int n_out_y, void* stream) {
  if (!out_map || n_out_y <= 0) return FOVI_ERR_INVALID_ARGUMENT;
  OutMode om;
  om.out_map = out_map; om.n_out_y = n_out_y; om.accumulate = 1;
  return knnconv_forward_impl(p, X, Wt, nullptr, Y, FOVI_F32, B, 0, stream, 0, WAIT_LIMIT, om);
}

extern "C" int fovi_knnconv_selftest_wait_timeout(fovi_knnconv_plan* p, const void* X, const void* Wt, void* Y, int y_dtype, int B,
                                                  void* stream) {
  // the kernel's consumers wait for operands that never come; after 4096 attempts each wait gives up
  return knnconv_forward_impl(p, X, Wt, nullptr, Y, y_dtype, B, 0, stream, 1, 4096u);
}

extern "C" int fovi_knnconv_check(fovi_knnconv_plan* p, void* stream) {
  if (!p) return FOVI_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int h = 0;
  FOVI_CUDA(cudaMemcpyAsync(&h, p->status, sizeof(int), cudaMemcpyDeviceToHost, st));
  FOVI_CUDA(cudaStreamSynchronize(st));
  if (h != 0) {
    FOVI_CUDA(cudaMemsetAsync(p->status, 0, sizeof(int), st));
    FOVI_CUDA(cudaStreamSynchronize(st));
    fovi::g_last_cuda_error = "tensor-core KNNConv kernel gave up on wait site " + std::to_string(h);
    return FOVI_ERR_DEVICE_TIMEOUT;
  }
  return FOVI_OK;
}
