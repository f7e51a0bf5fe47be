// Device-side building blocks shared by the tensor-core KNNConv kernels: launch arguments, mbarrier / TMA /
// tcgen05 PTX wrappers (every wait bounded), shared-memory descriptors.  Everything has internal linkage.
#pragma once
#include <cuda.h>
#include <stdlib.h>
#include <string.h>
#include <utility>

#include "knnconv_plan.cuh"

namespace fovi {
// Where an output point's result goes.  Normally point n of the plan is point n of Y.  The weight-gradient contraction
// (one "output point" per part of a filter tap's pair list) instead ADDS every part into its tap's row of a float32 Y:
// out_map[n] is the row, n_out_y the number of rows of Y, and the stores become float32 reductions.
struct OutMode { const int* out_map = nullptr; int n_out_y = 0; int accumulate = 0; };
}  // namespace fovi
using fovi::OutMode;

namespace {

constexpr int BM = 128;            // batch rows per tile (UMMA M)
constexpr int MAX_STAGES = 8;
constexpr uint32_t A_STAGE_BYTES = 16384;
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // try_wait attempts before giving up

enum { MODE_C8 = 0, MODE_C64 = 1, MODE_PAIRS = 2 };

struct TcArgs {
  // per-output-point lists: neighbours (idx, tap) in C8/C64 mode, input pairs (idx only) in PAIRS mode
  const int* nbr_idx; const uint16_t* nbr_tap; const int* nbr_cnt;
  const float* bias; void* Y; int* status;
  int kp, B, n_in, n_out, c_out, cp;
  int ct, n_ct, n_mt, nstage, relu, y_f32, total_items;
  uint32_t wait_limit;   // try_wait attempts before a wait gives up
  int skip_loads;        // self-test: the producer withholds every operand load, so the first consumer wait must give up
  int mt_fastest;        // item order, see decode_item
  int pgroups;           // pair mode: stages the producer warp fills per pass
  uint32_t acc_cols, tmem_cols;  // columns per accumulator (power of two >= ct) and allocated in total (two accumulators)
  const unsigned char* X; const unsigned char* Wt; const unsigned char* zero_block; int n_pairs;  // PAIRS mode
  uint32_t stage_bytes, table_bytes;
  const int* out_map; int n_out_y; int accumulate;   // see OutMode
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when it gave up or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          uint32_t limit = WAIT_LIMIT) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// Contiguous global -> shared bulk copy (16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One 32-byte store (a whole sector) when the address allows it, else two 16-byte stores.
__device__ __forceinline__ void st_global_32(void* p, const uint32_t (&w)[8]) {
  if ((reinterpret_cast<uintptr_t>(p) & 31u) == 0) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
  } else {
    uint4* d = reinterpret_cast<uint4*>(p);
    d[0] = make_uint4(w[0], w[1], w[2], w[3]);
    d[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// Four float32 reductions in one instruction (16-byte aligned).
__device__ __forceinline__ void red_add_f32x4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Shared-memory matrix descriptor (K-major operand).  layout: 0 = no swizzle, 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of this architecture
  d |= (uint64_t)layout << 61;
  return d;
}

// Shared-memory header at the 1024-aligned base of the dynamic allocation.
struct SmemHeader {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int TBQ = 8;  // table entries prefetched per producer lane: list pitch <= 32 * TBQ

// Work item -> (output point, batch tile, c_out tile).  Consecutive items run at the same time on neighbouring SMs:
// with the point varying fastest they share activations (neighbouring points read the same inputs), with the batch
// tile varying fastest (mt_fastest, pair mode) they share the point's packed weights, which are the larger operand there.
__device__ __forceinline__ void decode_item(const TcArgs& a, int item, int& n, int& mt, int& ctile) {
  ctile = item % a.n_ct;
  const int t = item / a.n_ct;
  if (a.mt_fastest) { mt = t % a.n_mt; n = t / a.n_mt; }
  else { n = t % a.n_out; mt = t / a.n_out; }
}
__device__ __forceinline__ int item_point(const TcArgs& a, int item) {
  const int t = item / a.n_ct;
  return a.mt_fastest ? t / a.n_mt : t % a.n_out;
}


}  // namespace

namespace fovi {
// Launch with the programmatic-stream-serialization attribute (see the griddepcontrol note in the kernels):
// the kernel may start while the previous kernel of the stream drains.  A build with -DFOVI_TC_NO_PDL launches plainly.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t st, Args&&... args) {
#ifdef FOVI_TC_NO_PDL
  constexpr bool plain = true;
#else
  constexpr bool plain = false;
#endif
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(block); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = plain ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Tiled 3-D bf16 tensor map (box b0 x b1 x b2 of a tensor d0 x d1 x d2 with byte strides for d1, d2).
int encode_3d(CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
              uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2, bool swizzle128);
// CTA-pair variant of the 64-channel mode (knnconv_tc2.cu).  Returns FOVI_ERR_UNSUPPORTED when it does not apply.
int launch_knnconv_tc_pair(const fovi_knnconv_plan* p, const void* X, const void* Wt, const float* bias, void* Y, int y_dtype,
                           int B, int relu, cudaStream_t st, int skip_loads, uint32_t wait_limit, const OutMode& om);
}  // namespace fovi
