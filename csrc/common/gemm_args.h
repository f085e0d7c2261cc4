// Argument blocks of the GEMM entry points (mirrored by ctypes.Structure classes in Python), shared by the translation
// units that implement them.
#pragma once

constexpr int kDptbMaxRanks = 8;

// Argument block of dptb_gemm (mirrored by a ctypes.Structure in Python).
struct DptbGemmArgs {
  const void* A;
  const void* B;
  void* C;
  const void* bias;
  const void* residual;
  void* aux_out;
  const void* aux_in;
  long long lda, ldb, ldc, ldr, ld_aux_out, ld_aux_in;
  int M, N, K;
  int trans_a;   // 0: A stored [M, K] row-major; 1: A stored [K, M] row-major
  int trans_b;   // 0: B stored [K, N] row-major; 1: B stored [N, K] row-major (nn.Linear weight)
  int a_f32, b_f32;  // inputs are fp32 (SIMT path only)
  int bias_f32, out_f32, accumulate, act;
  float alpha;
  int force_simt;
  int bn;        // 0 = choose, else 128 or 256
  int splits;    // split-K factor: 0 = choose, 1 = off
  void* ws;      // fp32 scratch for split-K partial tiles (may be null: no split-K)
  long long ws_bytes;
  int* counters; // zero-initialised per-tile arrival counters (they return to zero after every launch)
  int num_counters;
};

// Peer-memory description of the all-reduce epilogue (see TpAr).  `partial_elems` / `max_tiles` are capacities that
// the launcher checks against the tiling it picks.
struct DptbTpArArgs {
  int world, rank, use_nvls, max_tiles;
  void* partial;
  long long partial_elems;
  const void* peer_partial[kDptbMaxRanks];
  const void* mc_partial;
  void* out_peer[kDptbMaxRanks];
  void* mc_out;
  void* flags_peer[kDptbMaxRanks];
  void* epoch;
  void* exit_counter;
  int mode;   // 0 = all-reduce into every rank's output, 1 = reduce-scatter by rows into this rank's output
};
