// bf16 GEMM on the 5th-generation tensor cores (tcgen05) with TMA-fed operands
// and the accumulator in tensor memory (TMEM).
//
//   C[b] (M x N) = epilogue( alpha * A[b] (M x K) * B[b]^T (N x K) )
//
// Both operands may be stored "K-major" (the contraction index is the
// contiguous one, e.g. activations [tokens, c_in] and weights [c_out, c_in]) or
// "MN-major" (the contraction index is the strided one, e.g. the same weight
// used for a data-gradient GEMM, or activations contracted over tokens for a
// weight-gradient GEMM).  That covers forward, dgrad and wgrad of every Linear,
// the per-channel triangle-multiplication contraction and the outer-product-
// mean contraction without a transposed copy of any operand.
//
// One CTA computes one 128 x BN output tile:
//   warp 0      : TMA producer (one elected lane) - fills a STAGES-deep ring of
//                 128B-swizzled operand tiles, completion via mbarrier tx-count
//   warp 1      : MMA issuer (one lane) - tcgen05.mma, 128 x BN x 16 per
//                 instruction, tcgen05.commit releases ring slots and finally
//                 signals "accumulator ready"
//   warps 2..5  : epilogue - tcgen05.ld of their 32-lane TMEM quadrant, fused
//                 bias / activation / gating / mask / dropout / residual, bf16
//                 or fp32 stores (optionally transposed, optionally atomic for
//                 split-K)
// Several CTAs are resident per SM (smem permitting) so that one tile's
// epilogue overlaps the next tile's loads and MMAs.
//
// Covers what the reference leaves to cuBLAS through torch.matmul / einsum /
// nn.Linear (fastfold/model/fastnn/ops.py:79-82,143-160,275-324,393-404) plus
// the TorchScript elementwise fusions that follow those calls
// (fastfold/model/fastnn/kernel/jit/fused_ops.py:5-22).
#include "common.cuh"
#include "gemm_api.h"

namespace ffb {

__device__ int g_status[8];

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = 128 B = one swizzle row
constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = (BN >= 256) ? 4 : ((BN >= 128) ? 3 : 4);
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
};

__device__ __forceinline__ void load8(const bf16* p, bool vec, int n, float* o) {
  if (vec) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      o[2 * i] = f.x;
      o[2 * i + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = (i < n) ? __bfloat162float(p[i]) : 0.f;
  }
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS) gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                 const __grid_constant__ CUtensorMap tmB,
                                                                 const GemmArgs g) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024 B alignment for the 128B swizzle atoms
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + STAGES * Cfg::STAGE_BYTES);
  const uint32_t bar_full = smem_u32(bars);                 // STAGES barriers
  const uint32_t bar_empty = bar_full + 8 * STAGES;         // STAGES barriers
  const uint32_t bar_acc = bar_empty + 8 * STAGES;          // 1 barrier
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int m0 = blockIdx.y * BM;
  const int batch = blockIdx.z / g.splits;
  const int split = blockIdx.z - batch * g.splits;
  const int kb_total = (g.K + BK - 1) / BK;
  const int kb_begin = split * g.kblocks_per_split;
  int kb_end = kb_begin + g.kblocks_per_split;
  if (kb_end > kb_total) kb_end = kb_total;
  const int nkb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (nkb > 0) {
    if (warp == 0) {
      if (lane == 0) {
        // ---------------- TMA producer ----------------
        for (int i = 0; i < nkb; ++i) {
          const int s = i % STAGES;
          const int it = i / STAGES;
          if (it > 0) {
            if (!mbar_wait(bar_empty + 8 * s, (it - 1) & 1)) {
              report(ST_TIMEOUT_MMA, i);
              *abort_flag = 1;
              break;
            }
          }
          const int k0 = (kb_begin + i) * BK;
          const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(bar_full + 8 * s, Cfg::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_3d(sa + c * (BK * 128), &tmA, bar_full + 8 * s, m0 + c * 64, k0, batch * g.a_zmul);
          } else {
            tma_load_3d(sa, &tmA, bar_full + 8 * s, k0, m0, batch * g.a_zmul);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_3d(sb + c * (BK * 128), &tmB, bar_full + 8 * s, n0 + c * 64, k0, batch * g.b_zmul);
          } else {
            tma_load_3d(sb, &tmB, bar_full + 8 * s, k0, n0, batch * g.b_zmul);
          }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      if (lane == 0) {
        // ---------------- MMA issuer ----------------
        constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
        bool ok = true;
        for (int i = 0; i < nkb && ok; ++i) {
          const int s = i % STAGES;
          const int it = i / STAGES;
          if (!mbar_wait(bar_full + 8 * s, it & 1)) {
            report(ST_TIMEOUT_TMA, i);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16(tmem_acc, ad, bd, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty + 8 * s);   // slot reusable once these MMAs retire
        }
        if (ok) umma_commit(bar_acc);       // accumulator complete
      }
      __syncwarp();
    } else {
      // ---------------- epilogue (warps 2..5) ----------------
      const int quad = warp & 3;            // TMEM lane quadrant this warp may read
      const int row = m0 + quad * 32 + lane;
      bool ok = mbar_wait(bar_acc, 0);
      if (!ok && lane == 0) {
        if (*abort_flag == 0) report(ST_TIMEOUT_EPI, 0);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        const bool row_ok = row < g.M;
        const int Nout = g.glu ? (g.N >> 1) : g.N;
        float rs = 1.f;
        if (g.rowscale && row_ok) rs = g.rowscale[(long long)batch * g.rs_bstride + row];
        const bf16* dm_row = nullptr;
        if (g.dmask && row_ok) dm_row = reinterpret_cast<const bf16*>(g.dmask) + (long long)((row / g.dm_div) % g.dm_mod) * g.lddm;
        const bf16* mul_row = (g.mul && row_ok) ? reinterpret_cast<const bf16*>(g.mul) + (long long)batch * g.mul_bstride + (long long)row * g.ldmul : nullptr;
        const bf16* res_row = (g.resid && row_ok) ? reinterpret_cast<const bf16*>(g.resid) + (long long)batch * g.res_bstride + (long long)row * g.ldres : nullptr;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float v[32];
          tmem_ld_32x32(tmem_acc + ((uint32_t)(quad * 32) << 16) + c * 32, v);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (!row_ok || col0 >= g.N) continue;
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= g.alpha;
          if (g.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < g.N) v[j] += __bfloat162float(reinterpret_cast<const bf16*>(g.bias)[col0 + j]);
          }
          if (g.act == ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
          } else if (g.act == ACT_SIGMOID) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = sigmoidf_(v[j]);
          }
          int ncols = 32;
          int ocol0 = col0;
          if (g.glu) {
            // interleaved (value, gate) column pairs -> value * sigmoid(gate)
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = v[2 * j] * sigmoidf_(v[2 * j + 1]);
            ncols = 16;
            ocol0 = col0 >> 1;
          }
          // elementwise tail: mul, row scale, dropout mask, residual
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (q * 8 >= ncols) break;
            const int oc = ocol0 + q * 8;
            if (oc >= Nout) break;
            const int nvalid = (Nout - oc) < 8 ? (Nout - oc) : 8;
            float t[8];
            if (mul_row) {
              const bool vec = nvalid == 8 && ((reinterpret_cast<uintptr_t>(mul_row + oc) & 15) == 0);
              load8(mul_row + oc, vec, nvalid, t);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[q * 8 + j] *= t[j];
            }
            if (g.rowscale) {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[q * 8 + j] *= rs;
            }
            if (dm_row) {
              const bool vec = nvalid == 8 && ((reinterpret_cast<uintptr_t>(dm_row + oc) & 15) == 0);
              load8(dm_row + oc, vec, nvalid, t);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[q * 8 + j] *= t[j];
            }
            if (res_row) {
              const bool vec = nvalid == 8 && ((reinterpret_cast<uintptr_t>(res_row + oc) & 15) == 0);
              load8(res_row + oc, vec, nvalid, t);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[q * 8 + j] += t[j];
            }
            // ---- store ----
            if (g.trans_out) {
              // C^T: element (row, col) goes to C[col * ldc + row]; a warp
              // writes 32 consecutive rows of one column -> coalesced
              if (g.out_mode == OUT_BF16) {
                bf16* C = reinterpret_cast<bf16*>(g.C) + (long long)batch * g.c_bstride;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (j < nvalid) C[(long long)(oc + j) * g.ldc + row] = __float2bfloat16(v[q * 8 + j]);
              } else {
                float* C = reinterpret_cast<float*>(g.C) + (long long)batch * g.c_bstride;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (j < nvalid) {
                    if (g.out_mode == OUT_F32_ATOMIC) atomicAdd(&C[(long long)(oc + j) * g.ldc + row], v[q * 8 + j]);
                    else C[(long long)(oc + j) * g.ldc + row] = v[q * 8 + j];
                  }
              }
            } else if (g.out_mode == OUT_BF16) {
              bf16* dst = reinterpret_cast<bf16*>(g.C) + (long long)batch * g.c_bstride + (long long)row * g.ldc + oc;
              if (nvalid == 8 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
                uint4 u;
                bf162* h = reinterpret_cast<bf162*>(&u);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
                *reinterpret_cast<uint4*>(dst) = u;
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (j < nvalid) dst[j] = __float2bfloat16(v[q * 8 + j]);
              }
            } else {
              float* dst = reinterpret_cast<float*>(g.C) + (long long)batch * g.c_bstride + (long long)row * g.ldc + oc;
              if (g.out_mode == OUT_F32_ATOMIC) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (j < nvalid) atomicAdd(dst + j, v[q * 8 + j]);
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (j < nvalid) dst[j] = v[q * 8 + j];
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Host side: tensor-map encoding through the driver entry point (no link-time
// dependency on libcuda) and the launcher.
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess || !p) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// bf16 matrix [batch][rows][cols] (cols contiguous, row stride ld, batch stride
// bstride, all in elements); box = box_cols x box_rows, 128B swizzle.
int make_tmap_bf16(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, long long batch,
                   long long bstride, int box_cols, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)(batch > 0 ? batch : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? bstride : rows * ld) * 2};
  if (strides[1] == 0) strides[1] = (cuuint64_t)ld * 2 * rows;
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_cfg(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int batch, cudaStream_t st) {
  using Cfg = GemmCfg<BN>;
  static bool attr_set = false;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) return -2;
    attr_set = true;
  }
  dim3 grid((g.N + BN - 1) / BN, (g.M + BM - 1) / BM, batch * g.splits);
  kern<<<grid, GEMM_THREADS, Cfg::SMEM, st>>>(ta, tb, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

template <bool A_MN, bool B_MN>
static int launch_bn(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int batch, cudaStream_t st) {
  switch (bn) {
    case 64: return launch_cfg<64, A_MN, B_MN>(ta, tb, g, batch, st);
    case 128: return launch_cfg<128, A_MN, B_MN>(ta, tb, g, batch, st);
    case 256: return launch_cfg<256, A_MN, B_MN>(ta, tb, g, batch, st);
    default: return -4;
  }
}

}  // namespace ffb

using namespace ffb;

extern "C" {

// A: a_mn == 0 -> [batch][M][K] (ld = lda); a_mn == 1 -> [batch][K][M].
// B: b_mn == 0 -> [batch][N][K] (ld = ldb); b_mn == 1 -> [batch][K][N].
// A batch stride of 0 broadcasts the operand over the batch.
int ffb_gemm_bf16(const void* A, const void* B, int a_mn, int b_mn, long long lda, long long ldb, long long a_bstride,
                  long long b_bstride, int batch, int bn, GemmArgs* args, void* stream) {
  GemmArgs g = *args;
  if (g.M <= 0 || g.N <= 0 || g.K <= 0 || batch <= 0) return -10;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -11;
  if (g.glu && (g.N & 1)) return -12;
  if (bn == 0) {
    if (g.N > 128 && !g.glu && (long long)((g.M + 127) / 128) * ((g.N + 255) / 256) * batch >= 148) bn = 256;
    else if (g.N > 64) bn = 128;
    else bn = 64;
  }
  const int kb_total = (g.K + BK - 1) / BK;
  if (g.splits < 1) g.splits = 1;
  if (g.splits > kb_total) g.splits = kb_total;
  g.kblocks_per_split = (kb_total + g.splits - 1) / g.splits;
  g.splits = (kb_total + g.kblocks_per_split - 1) / g.kblocks_per_split;
  if (g.splits > 1 && g.out_mode != OUT_F32_ATOMIC) return -13;
  CUtensorMap ta, tb;
  int r;
  g.a_zmul = (batch > 1 && a_bstride != 0) ? 1 : 0;
  g.b_zmul = (batch > 1 && b_bstride != 0) ? 1 : 0;
  if ((a_bstride % 8) || (b_bstride % 8)) return -14;
  if ((a_mn || b_mn) && bn < 64) return -15;
  const int abatch = g.a_zmul ? batch : 1, bbatch = g.b_zmul ? batch : 1;
  if (a_mn) r = make_tmap_bf16(&ta, A, g.K, g.M, lda, abatch, a_bstride, 64, BK);
  else r = make_tmap_bf16(&ta, A, g.M, g.K, lda, abatch, a_bstride, BK, BM);
  if (r) return 1000 + r;
  if (b_mn) r = make_tmap_bf16(&tb, B, g.K, g.N, ldb, bbatch, b_bstride, 64, BK);
  else r = make_tmap_bf16(&tb, B, g.N, g.K, ldb, bbatch, b_bstride, BK, bn);
  if (r) return 2000 + r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn) {
    if (b_mn) return launch_bn<true, true>(bn, ta, tb, g, batch, st);
    return launch_bn<true, false>(bn, ta, tb, g, batch, st);
  }
  if (b_mn) return launch_bn<false, true>(bn, ta, tb, g, batch, st);
  return launch_bn<false, false>(bn, ta, tb, g, batch, st);
}

// Reads and clears the device status word; out[0] != 0 means a kernel gave up
// on a wait (out[1..3] = block index, out[4] = detail).
int ffb_read_status(int* out, int clear) {
  int h[8];
  if (cudaMemcpyFromSymbol(h, g_status, sizeof(h)) != cudaSuccess) return -1;
  for (int i = 0; i < 8; ++i) out[i] = h[i];
  if (clear && h[0] != 0) {
    int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (cudaMemcpyToSymbol(g_status, z, sizeof(z)) != cudaSuccess) return -1;
  }
  return 0;
}

}  // extern "C"
