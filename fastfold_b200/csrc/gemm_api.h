// Argument block of the tcgen05 GEMM launcher (mirrored field-for-field by the
// ctypes structure in fastfold_b200/ops/_lib.py).
#pragma once
#include <cuda.h>

enum GemmAct { ACT_NONE = 0, ACT_RELU = 1, ACT_SIGMOID = 2 };
enum GemmOut { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ATOMIC = 2 };

struct GemmArgs {
  int M, N, K;              // per-batch problem; K is the contraction extent
  int splits;               // split-K factor (needs OUT_F32_ATOMIC when > 1)
  int kblocks_per_split;    // filled by the launcher
  int out_mode;             // GemmOut
  int trans_out;            // store C^T: element (m, n) -> C[n * ldc + m]
  int act;                  // GemmAct, applied after bias
  int glu;                  // columns are interleaved (value, gate) pairs -> value * sigmoid(gate); N_out = N / 2
  int dm_div, dm_mod;       // dropout-mask row = (m / dm_div) % dm_mod
  int a_zmul, b_zmul;       // 0: operand is shared by all batches, 1: indexed by batch
  float alpha;
  void* C;
  long long ldc, c_bstride;
  const void* bias;         // bf16 [N], added to alpha * acc
  const float* rowscale;    // fp32 [batch][M], multiplies the row
  long long rs_bstride;
  const void* mul;          // bf16, same indexing as the (non-transposed) output
  long long ldmul, mul_bstride;
  const void* dmask;        // bf16 [dm_mod][lddm]
  long long lddm;
  const void* resid;        // bf16 residual added last
  long long ldres, res_bstride;
  int peer_slab;            // gathered-operand GEMMs: extent of one rank's slab along the gathered (M or N) dimension
  // Block-permuted bf16 output: with m = 32 * m1 + m0 and n = 32 * n1 + n0, element (m, n) goes to
  // C[(m1 / cq_mdiv) * cq_sr2 + (m1 % cq_mdiv) * cq_sr1 + n1 * cq_sc1 + m0 * 32 + n0], i.e. every 32 x 32 block is
  // contiguous (2 KB) and the blocks are placed by three free strides (d = e = 32 below):
  //   [(i d), (j e)] -> [i][j][d][e]:      cq_mdiv = 1, cq_sr2 = J * 1024, cq_sr1 = 0, cq_sc1 = 1024
  //   [(i j), (d e)] -> [(i d)][(j e)]:    cq_mdiv = J / 32, cq_sr2 = J * 1024, cq_sr1 = 1024, cq_sc1 = 32 * J
  int cq, cq_mdiv;
  long long cq_sr2, cq_sr1, cq_sc1;
};

// Tensor maps of the slabs of a gathered operand, one per rank of the DAP group (peer memory, plain TMA loads).
struct PeerMaps {
  CUtensorMap m[8];
};
