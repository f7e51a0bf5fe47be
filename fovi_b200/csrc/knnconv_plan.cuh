// Plan object shared by the KNNConv translation units.
#pragma once
#include "common.cuh"

namespace fovi {
// Largest c_out tile <= 256 that divides c_out and is a multiple of 16 (0 if none).
inline int pick_cout_tile(int c_out) {
  for (int n_ct = 1; n_ct <= c_out / 16; ++n_ct) {
    if (c_out % n_ct) continue;
    const int ct = c_out / n_ct;
    if (ct <= 256 && ct % 16 == 0) return ct;
  }
  return 0;
}
}  // namespace fovi

struct fovi_knnconv_plan {
  int n_in = 0, n_out = 0, K = 0, V = 0, c_in = 0, c_out = 0;
  int cin_packed = 0;  // channel count of the packed bf16/f32 operands
  int kp = 0;          // compacted neighbour-list pitch: K rounded up to a multiple of 8
  int device = -1;
  int64_t nnz = 0;     // non-pad (n,k) entries
  // Compacted per-output-point neighbour lists: entries [0,cnt[n]) are the non-pad neighbours in
  // their original order; the rest of the row holds idx = n_in (reads as zero), tap = 0.
  int* nbr_idx = nullptr;       // [n_out, kp]
  uint16_t* nbr_tap = nullptr;  // [n_out, kp]
  int* nbr_cnt = nullptr;       // [n_out]
  int* status = nullptr;        // device word written by a tensor-core kernel whose wait gave up
  // Pair mode (c_in <= 4): neighbours grouped into aligned point pairs (2p, 2p+1).
  int x_layout = FOVI_X_BNC;
  int n_pairs = 0;              // ceil(n_in / 2)
  int sp = 0;                   // pair-slot pitch per output point (multiple of 8)
  int* pair_idx = nullptr;      // [n_out, sp] pair index; unused slots hold n_pairs (reads as zero)
  int* pair_cnt = nullptr;      // [n_out]
  uint16_t* pair_tap = nullptr; // [n_out, sp, 2] tap of the even / odd member, 0xFFFF = not a neighbour
  uint16_t* pair_run = nullptr; // [n_out, sp] at the first slot of a run of consecutive pairs inside an 8-slot stage: the run's length; else 0
  void* zero_block = nullptr;   // 16 KB of zeros: the operand blocks read for unused pair slots
  int ct = 0;                   // c_out tile of the tensor-core path (UMMA N), 0 = unsupported c_out
};
