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
// Persistent kernel, one CTA per SM, each CTA walks 128 x BN output tiles
// (tile = blockIdx.x, + gridDim.x, ...; N-tiles fastest so that CTAs running at
// the same time share A rows in L2):
//   warp 0      : TMA producer (one elected lane) - fills a STAGES-deep ring of
//                 128B-swizzled operand tiles, completion via mbarrier tx-count;
//                 the ring keeps running across tile boundaries
//   warp 1      : MMA issuer (one lane) - tcgen05.mma, 128 x BN x 16 per
//                 instruction, into one of TWO accumulator stages in TMEM;
//                 tcgen05.commit releases ring slots and signals "stage full"
//   warps 2..5  : epilogue - tcgen05.ld of their 32-lane TMEM quadrant, a
//                 32 x 64 transpose through shared memory so that 8 lanes
//                 cover 128 contiguous bytes of an output row, then fused
//                 bias / activation / GLU / gate / mask / dropout / residual
//                 and 16-byte stores (or vector fp32 reductions for split-K);
//                 transposed (channel-major) stores use the thread-per-row
//                 mapping directly.  The epilogue of tile t overlaps the MMAs
//                 of tile t+1 through the second accumulator stage.
// Every wait is bounded; a wait that runs out records a code in the status
// word and the CTA unwinds (TMEM is always released).
//
// Covers what the reference leaves to cuBLAS through torch.matmul / einsum /
// nn.Linear (fastfold/model/fastnn/ops.py:79-82,143-160,275-324,393-404) plus
// the TorchScript elementwise fusions that follow those calls
// (fastfold/model/fastnn/kernel/jit/fused_ops.py:5-22).
#include "common.cuh"
#include "gemm_api.h"
#include "tmap.h"

namespace ffb {

__device__ int g_status[8];

// Optional phase timeline of CTA 0 (compiled in only for profiling builds: -DFFB_GEMM_TRACE).
#ifdef FFB_GEMM_TRACE
__device__ unsigned long long g_gemm_trace[256 + 8 * 160];     // [15 tiles][16 slots] of CTA 0, then [CTA][8] phase stamps
// the "memory" clobber keeps the timer read on its side of barriers and waits
__device__ __forceinline__ unsigned long long trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
  return t;
}
#define GEMM_TRACE(tile_local, slot)                                                        \
  do {                                                                                      \
    if (blockIdx.x == 0 && (tile_local) < 15) g_gemm_trace[(tile_local) * 16 + (slot)] = trace_now(); \
  } while (0)
#define GEMM_TRACE_CTA(slot)                                                                \
  do {                                                                                      \
    if (threadIdx.x == 0 && blockIdx.x < 160) g_gemm_trace[256 + blockIdx.x * 8 + (slot)] = trace_now(); \
  } while (0)
#else
#define GEMM_TRACE(tile_local, slot) do {} while (0)
#define GEMM_TRACE_CTA(slot) do {} while (0)
#endif

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = 128 B = one swizzle row
constexpr int GEMM_THREADS = 320;   // producer warp, MMA warp, 8 epilogue warps
constexpr int EPI_WARPS = 8;
constexpr int STG_LD = 65;       // staging row pitch in floats (odd -> conflict-free column access)
constexpr int FAST_BIAS_MAX_N = 1024;                          // widest output whose bias the fast epilogue keeps in shared memory
constexpr int BIAS_SMEM_BYTES = (FAST_BIAS_MAX_N + 64) * 4;    // fp32, zero-padded by one column chunk

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = (BN >= 256) ? 3 : 4;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_WARP_BYTES = 9216;               // per epilogue warp: 2 x 4 KB TMA tiles (the 32 x 65 fp32 transpose
  static constexpr int STG_BYTES = EPI_WARPS * EPI_WARP_BYTES;  // buffer of the generic path aliases them)
  static constexpr int SMEM = STAGES * STAGE_BYTES + STG_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + BIAS_SMEM_BYTES;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulator stages
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

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

struct TileCoord {
  int m0, n0, batch, split;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int tiles_n, int tiles_m, int splits) {
  TileCoord t;
  const int tn = tile % tiles_n;
  int r = tile / tiles_n;
  const int tm = r % tiles_m;
  r /= tiles_m;
  t.split = r % splits;
  t.batch = r / splits;
  t.m0 = tm * BM;
  t.n0 = tn;   // scaled by BN by the caller
  return t;
}

// Epilogue arithmetic on 8 consecutive output columns of one row (everything after bias/activation/glu).
__device__ __forceinline__ void epi_tail8(float* v, const GemmArgs& g, int batch, int row, int oc, int nvalid, float rs) {
  float t[8];
  if (g.mul) {
    const bf16* p = reinterpret_cast<const bf16*>(g.mul) + (long long)batch * g.mul_bstride + (long long)row * g.ldmul + oc;
    load8(p, nvalid == 8 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0), nvalid, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= t[j];
  }
  if (g.rowscale) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= rs;
  }
  if (g.dmask) {
    const bf16* p = reinterpret_cast<const bf16*>(g.dmask) + (long long)((row / g.dm_div) % g.dm_mod) * g.lddm + oc;
    load8(p, nvalid == 8 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0), nvalid, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= t[j];
  }
  if (g.resid) {
    const bf16* p = reinterpret_cast<const bf16*>(g.resid) + (long long)batch * g.res_bstride + (long long)row * g.ldres + oc;
    load8(p, nvalid == 8 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0), nvalid, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] += t[j];
  }
}

__device__ __forceinline__ void epi_store8(const float* v, const GemmArgs& g, int batch, int row, int oc, int nvalid) {
  if (g.out_mode == OUT_BF16) {
    bf16* dst = reinterpret_cast<bf16*>(g.C) + (long long)batch * g.c_bstride + (long long)row * g.ldc + oc;
    if (nvalid == 8 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
      uint4 u;
      bf162* h = reinterpret_cast<bf162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      *reinterpret_cast<uint4*>(dst) = u;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nvalid) dst[j] = __float2bfloat16(v[j]);
    }
  } else {
    float* dst = reinterpret_cast<float*>(g.C) + (long long)batch * g.c_bstride + (long long)row * g.ldc + oc;
    const bool vec = nvalid == 8 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
    if (g.out_mode == OUT_F32_ATOMIC) {
      if (vec) {
        red_add_v4(dst, v[0], v[1], v[2], v[3]);
        red_add_v4(dst + 4, v[4], v[5], v[6], v[7]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nvalid) atomicAdd(dst + j, v[j]);
      }
    } else if (vec) {
      *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nvalid) dst[j] = v[j];
    }
  }
}

// Persistent kernel: every CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...
// PEER: 0 = both operands local; 1 = the A operand is gathered along M, 2 = the B operand is gathered along N: the
// slab of rank r lives in r's memory and its tiles are fetched with TMA straight over NVLink (all-gather fused into
// the GEMM's load stage; the gathered operand is never materialised).
template <int BN, bool A_MN, bool B_MN, int PEER>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                    const __grid_constant__ CUtensorMap tmB,
                                                                    const __grid_constant__ CUtensorMap tmC,
                                                                    const __grid_constant__ CUtensorMap tmMul,
                                                                    const __grid_constant__ CUtensorMap tmRes,
                                                                    const __grid_constant__ PeerMaps pm,
                                                                    const GemmArgs g, int num_tiles, int tiles_m, int tiles_n, int tma_epi) {
  pdl_launch_dependents();
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  GEMM_TRACE_CTA(0);
  // operand tiles need 1024 B alignment for the 128B swizzle atoms
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  float* staging = reinterpret_cast<float*>(smem_al + STAGES * Cfg::STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + STAGES * Cfg::STAGE_BYTES + Cfg::STG_BYTES);
  const uint32_t bar_full = smem_u32(bars);                 // STAGES: operand tile landed
  const uint32_t bar_empty = bar_full + 8 * STAGES;         // STAGES: operand tile consumed
  const uint32_t bar_accf = bar_empty + 8 * STAGES;         // 2: accumulator stage complete
  const uint32_t bar_acce = bar_accf + 16;                  // 2: accumulator stage drained
  const uint32_t bar_epld = bar_acce + 16;                  // 8: per-epilogue-warp TMA loads of mul / residual tiles
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + EPI_WARPS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_bias = reinterpret_cast<float*>(smem_al + STAGES * Cfg::STAGE_BYTES + Cfg::STG_BYTES + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kb_total = (g.K + BK - 1) / BK;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_accf + 8 * s, 1);
      mbar_init(bar_acce + 8 * s, EPI_WARPS);     // one arrival per epilogue warp
    }
    for (int s = 0; s < EPI_WARPS; ++s) mbar_init(bar_epld + 8 * s, 1);
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
  const uint32_t tmem_base = *tmem_slot;
  GEMM_TRACE_CTA(1);   // barriers initialised, tensor memory allocated
  // everything above touches only this CTA's shared and tensor memory; from here on global memory is read
  pdl_wait();
  if (warp >= 2 && tma_epi && g.bias && g.N <= FAST_BIAS_MAX_N) {
    // fast epilogue: the whole bias vector as fp32 in shared memory, read back as broadcast 16-byte loads.  Only the
    // epilogue warps fill and wait for it (named barrier 1), so the producer's first loads do not queue behind it.
    const bf16* bp = reinterpret_cast<const bf16*>(g.bias);
    for (int i = threadIdx.x - 64; i < FAST_BIAS_MAX_N + 64; i += EPI_WARPS * 32) s_bias[i] = (i < g.N) ? __bfloat162float(bp[i]) : 0.f;
    asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
  }
  GEMM_TRACE_CTA(2);   // start of the main phase

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t it = 0;   // k-block counter over all tiles of this CTA
      uint32_t plt = 0;  // local tile counter
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++plt) {
        const TileCoord tc = tile_coord(tile, tiles_n, tiles_m, g.splits);
        const int n0 = tc.n0 * BN;
        const int kb_begin = tc.split * g.kblocks_per_split;
        int kb_end = kb_begin + g.kblocks_per_split;
        if (kb_end > kb_total) kb_end = kb_total;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(bar_empty + 8 * s, ((it / STAGES) & 1) ^ 1)) {
            report(ST_TIMEOUT_MMA, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const int k0 = kb * BK;
          const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + Cfg::A_BYTES;
          const CUtensorMap* mapA = &tmA;
          const CUtensorMap* mapB = &tmB;
          int am0 = tc.m0, bn0 = n0;
          if (PEER == 1) {
            const int r = tc.m0 / g.peer_slab;
            mapA = &pm.m[r];
            am0 = tc.m0 - r * g.peer_slab;
          } else if (PEER == 2) {
            const int r = n0 / g.peer_slab;
            mapB = &pm.m[r];
            bn0 = n0 - r * g.peer_slab;
          }
          if (kb == kb_begin) GEMM_TRACE(plt, 0);      // producer: slot free, first loads of the tile go out
          mbar_expect_tx(bar_full + 8 * s, Cfg::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_3d(sa + c * (BK * 128), mapA, bar_full + 8 * s, am0 + c * 64, k0, tc.batch * g.a_zmul);
          } else {
            tma_load_3d(sa, mapA, bar_full + 8 * s, k0, am0, tc.batch * g.a_zmul);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_3d(sb + c * (BK * 128), mapB, bar_full + 8 * s, bn0 + c * 64, k0, tc.batch * g.b_zmul);
          } else {
            tma_load_3d(sb, mapB, bar_full + 8 * s, k0, bn0, tc.batch * g.b_zmul);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0, lt = 0;   // k-block counter, local tile counter
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++lt) {
        const TileCoord tc = tile_coord(tile, tiles_n, tiles_m, g.splits);
        const int kb_begin = tc.split * g.kblocks_per_split;
        int kb_end = kb_begin + g.kblocks_per_split;
        if (kb_end > kb_total) kb_end = kb_total;
        const uint32_t as = lt & 1;
        if (!mbar_wait(bar_acce + 8 * as, ((lt >> 1) & 1) ^ 1)) {
          report(ST_TIMEOUT_EPI, 1);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + as * BN;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(bar_full + 8 * s, (it / STAGES) & 1)) {
            report(ST_TIMEOUT_TMA, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          if (kb == kb_begin) GEMM_TRACE(lt, 1);       // issuer: first operand tile landed
          const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16(tmem_acc, ad, bd, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty + 8 * s);   // slot reusable once these MMAs retire
        }
        if (ok) umma_commit(bar_accf + 8 * as);   // accumulator stage complete
        GEMM_TRACE(lt, 2);                         // issuer: all MMAs of the tile issued
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..9): two warps per TMEM lane quadrant, alternating column chunks ----------------
    const int half = (warp - 2) >> 2;
    const int quad = warp & 3;            // TMEM lane quadrant this warp may read
    float* stg = staging + (warp - 2) * (Cfg::EPI_WARP_BYTES / 4);
    const uint32_t epi_smem = smem_u32(stg);              // 1024-aligned: [tile0 4 KB][tile1 4 KB]
    const uint32_t my_ldbar = bar_epld + 8 * (warp - 2);
    uint32_t ld_phase = 0, out_buf = 0;
    const int Nout = g.glu ? (g.N >> 1) : g.N;
    uint32_t lt = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++lt) {
      const TileCoord tc = tile_coord(tile, tiles_n, tiles_m, g.splits);
      const int n0 = tc.n0 * BN;
      const uint32_t as = lt & 1;
      // TMA epilogue with mul / residual tiles: the loads of this warp's first chunk go out BEFORE the wait for the
      // accumulator, so their latency hides behind the MMAs of the tile instead of sitting inside the epilogue
      bool pre_issued = false;
      if (tma_epi == 1 && (g.mul != nullptr || g.resid != nullptr)) {
        const int prow0 = tc.m0 + quad * 32, pcol0 = n0 + half * 64;
        if (half < BN / 64 && pcol0 < g.N && prow0 < g.M) {
          if (lane == 0) {
            if (g.mul) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            mbar_expect_tx(my_ldbar, (g.mul ? 4096u : 0u) + (g.resid ? 4096u : 0u));
            if (g.resid) tma_load_3d(epi_smem + out_buf * 4096, &tmRes, my_ldbar, pcol0, prow0, tc.batch);
            if (g.mul) tma_load_3d(epi_smem + (out_buf ^ 1) * 4096, &tmMul, my_ldbar, pcol0, prow0, tc.batch);
          }
          pre_issued = true;
        }
      }
      bool ok = mbar_wait(bar_accf + 8 * as, (lt >> 1) & 1);
      if (!ok && lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_EPI, 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (warp == 2 && lane == 0) GEMM_TRACE(lt, 3);   // epilogue: accumulator complete
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + as * BN;
      if (tma_epi == 2) {
        // Fast path (bf16 output, row-major or block-permuted, at most bias + activation): TMEM -> registers -> shared
        // tile -> bulk store, with no per-element branches.  The common projection / gradient GEMMs of the model land here.
        const int row0 = tc.m0 + quad * 32;
#pragma unroll 1
        for (int c = half; c < BN / 64; c += 2) {
          const int col0 = n0 + c * 64;
          if (col0 >= g.N || row0 >= g.M) break;           // warp-uniform
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the store that last read this tile is done
          __syncwarp();
          float v[64];
          tmem_ld_32x32(taddr + c * 64, v);
          tmem_ld_32x32(taddr + c * 64 + 32, v + 32);
          tmem_ld_wait();
          if (g.bias) {
            if (g.N <= FAST_BIAS_MAX_N) {
              const float4* bp = reinterpret_cast<const float4*>(s_bias + col0);
#pragma unroll
              for (int q = 0; q < 16; ++q) {
                const float4 b4 = bp[q];
                v[4 * q] += b4.x;
                v[4 * q + 1] += b4.y;
                v[4 * q + 2] += b4.z;
                v[4 * q + 3] += b4.w;
              }
            } else {
              // wide outputs: the chunk's 64 bias values straight from global memory (same address in every lane)
              const bf16* bp = reinterpret_cast<const bf16*>(g.bias) + col0;
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                float t[8];
                load8(bp + q * 8, (g.N - col0 - q * 8) >= 8 && ((reinterpret_cast<uintptr_t>(bp + q * 8) & 15) == 0), g.N - col0 - q * 8, t);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[q * 8 + j] += t[j];
              }
            }
          }
          if (g.act == ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = fmaxf(v[j], 0.f);
          } else if (g.act == ACT_SIGMOID) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = sigmoidf_(v[j]);
          }
          uint8_t* obuf = reinterpret_cast<uint8_t*>(stg) + out_buf * 4096;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            uint4 pk;
            bf162* hp = reinterpret_cast<bf162*>(&pk);
#pragma unroll
            for (int j = 0; j < 4; ++j) hp[j] = __floats2bfloat162_rn(v[u * 8 + 2 * j], v[u * 8 + 2 * j + 1]);
            // row-major: 128-byte swizzled rows; block-permuted: two linear [32][32] blocks
            uint8_t* slot = g.cq ? obuf + (u >> 2) * 2048 + lane * 64 + ((u & 3) << 4) : obuf + lane * 128 + ((u ^ (lane & 7)) << 4);
            *reinterpret_cast<uint4*>(slot) = pk;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (g.cq) {
              const int m1 = row0 >> 5;
              bf16* dst = reinterpret_cast<bf16*>(g.C) + (long long)tc.batch * g.c_bstride + (long long)(m1 / g.cq_mdiv) * g.cq_sr2 +
                          (long long)(m1 % g.cq_mdiv) * g.cq_sr1 + (long long)(col0 >> 5) * g.cq_sc1;
              asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 2048;" ::"l"(dst), "r"(epi_smem + out_buf * 4096)
                           : "memory");
              asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 2048;" ::"l"(dst + g.cq_sc1),
                           "r"(epi_smem + out_buf * 4096 + 2048)
                           : "memory");
            } else {
              asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(&tmC),
                           "r"(epi_smem + out_buf * 4096), "r"(col0), "r"(row0), "r"(tc.batch)
                           : "memory");
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          out_buf ^= 1;
        }
      } else if (tma_epi == 3) {
        // Fast transposed path (bf16 C^T; bias, activation, GLU pairing, row scale): the 32 x 64 warp tile is transposed on
        // its way into shared memory ([64 columns][32 rows], 64-byte lines written by whole warps) and leaves as one TMA
        // store.  With GLU the 64 accumulator columns are 32 (value, gate) pairs and the tile that leaves is [32][32].
        const int row0 = tc.m0 + quad * 32;
        const float rs3 = (g.rowscale && row0 + lane < g.M) ? g.rowscale[(long long)tc.batch * g.rs_bstride + row0 + lane] : 1.f;
#pragma unroll 1
        for (int c = half; c < BN / 64; c += 2) {
          const int col0 = n0 + c * 64;
          if (col0 >= g.N || row0 >= g.M) break;           // warp-uniform
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          __syncwarp();
          float v[64];
          tmem_ld_32x32(taddr + c * 64, v);
          tmem_ld_32x32(taddr + c * 64 + 32, v + 32);
          tmem_ld_wait();
          if (g.bias) {
            const float4* bp = reinterpret_cast<const float4*>(s_bias + col0);
#pragma unroll
            for (int q = 0; q < 16; ++q) {
              const float4 b4 = bp[q];
              v[4 * q] += b4.x;
              v[4 * q + 1] += b4.y;
              v[4 * q + 2] += b4.z;
              v[4 * q + 3] += b4.w;
            }
          }
          if (g.act == ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = fmaxf(v[j], 0.f);
          } else if (g.act == ACT_SIGMOID) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = sigmoidf_(v[j]);
          }
          bf16* obuf = reinterpret_cast<bf16*>(reinterpret_cast<uint8_t*>(stg) + out_buf * 4096) + lane;
          if (g.glu) {
#pragma unroll
            for (int j = 0; j < 32; ++j) obuf[j * 32] = __float2bfloat16(v[2 * j] * sigmoidf_(v[2 * j + 1]) * rs3);
          } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) obuf[j * 32] = __float2bfloat16(v[j] * rs3);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(&tmC),
                         "r"(epi_smem + out_buf * 4096), "r"(row0), "r"(g.glu ? (col0 >> 1) : col0), "r"(tc.batch)
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          out_buf ^= 1;
        }
      } else if (tma_epi) {
        // TMA path (bf16 row-major output): thread = row; mul / residual tiles arrive by TMA, the result tile leaves
        // by TMA, so every global access is a full-line bulk transfer and the warp only touches shared memory
        const int row0 = tc.m0 + quad * 32;
        const int row = row0 + lane;
        const float rs = (g.rowscale && row < g.M) ? g.rowscale[(long long)tc.batch * g.rs_bstride + row] : 1.f;
        const bf16* dm_row = (g.dmask && row < g.M) ? reinterpret_cast<const bf16*>(g.dmask) + (long long)((row / g.dm_div) % g.dm_mod) * g.lddm : nullptr;
        const bool has_ld = (g.mul != nullptr) || (g.resid != nullptr);
#pragma unroll 1
        for (int c = half; c < BN / 64; c += 2) {
          const int col0 = n0 + c * 64;
          if (col0 >= g.N || row0 >= g.M) break;           // warp-uniform
          // tile[out_buf] receives the residual (if any) and then the result; tile[out_buf ^ 1] receives mul (if any).
          // A tile may be refilled only after the bulk store that last read it has finished reading.
          if (lane == 0 && !(pre_issued && c == half)) {
            if (g.mul) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            if (has_ld) {
              mbar_expect_tx(my_ldbar, (g.mul ? 4096u : 0u) + (g.resid ? 4096u : 0u));
              if (g.resid) tma_load_3d(epi_smem + out_buf * 4096, &tmRes, my_ldbar, col0, row0, tc.batch);
              if (g.mul) tma_load_3d(epi_smem + (out_buf ^ 1) * 4096, &tmMul, my_ldbar, col0, row0, tc.batch);
            }
          }
          __syncwarp();
          float v[64];
          tmem_ld_32x32(taddr + c * 64, v);
          tmem_ld_32x32(taddr + c * 64 + 32, v + 32);
          tmem_ld_wait();
          if (g.alpha != 1.0f) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] *= g.alpha;
          }
          if (g.bias) {
            if (g.N <= FAST_BIAS_MAX_N) {
              const float4* bp = reinterpret_cast<const float4*>(s_bias + col0);
#pragma unroll
              for (int q = 0; q < 16; ++q) {
                const float4 b4 = bp[q];
                v[4 * q] += b4.x;
                v[4 * q + 1] += b4.y;
                v[4 * q + 2] += b4.z;
                v[4 * q + 3] += b4.w;
              }
            } else {
              const bf16* bp = reinterpret_cast<const bf16*>(g.bias) + col0;
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                float t[8];
                load8(bp + q * 8, (g.N - col0 - q * 8) >= 8 && ((reinterpret_cast<uintptr_t>(bp + q * 8) & 15) == 0), g.N - col0 - q * 8, t);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[q * 8 + j] += t[j];
              }
            }
          }
          if (g.act == ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = fmaxf(v[j], 0.f);
          } else if (g.act == ACT_SIGMOID) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = sigmoidf_(v[j]);
          }
          if (has_ld) {
            const bool w = mbar_wait(my_ldbar, ld_phase);
            ld_phase ^= 1;
            if (!w && lane == 0) report(ST_TIMEOUT_TMA, 40);   // the status word carries the failure; the tile is still written
          }
          uint8_t* stg8 = reinterpret_cast<uint8_t*>(stg);
          uint8_t* obuf = stg8 + out_buf * 4096;
          if (g.mul) {
            const uint8_t* mbuf = stg8 + (out_buf ^ 1) * 4096;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              float t[8];
              load8(reinterpret_cast<const bf16*>(mbuf + lane * 128 + ((u ^ (lane & 7)) << 4)), true, 8, t);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[u * 8 + j] *= t[j];
            }
          }
          if (g.rowscale) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] *= rs;
          }
          if (dm_row) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int oc = col0 + u * 8;
              if (oc < g.N) {
                float t[8];
                const int nvalid = (g.N - oc) < 8 ? (g.N - oc) : 8;
                load8(dm_row + oc, nvalid == 8 && ((reinterpret_cast<uintptr_t>(dm_row + oc) & 15) == 0), nvalid, t);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[u * 8 + j] *= t[j];
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            // this thread's own row: read residual, write result.  Block-permuted output: two linear [32][32] blocks
            uint8_t* slot = g.cq ? obuf + (u >> 2) * 2048 + lane * 64 + ((u & 3) << 4) : obuf + lane * 128 + ((u ^ (lane & 7)) << 4);
            if (g.resid) {
              float t[8];
              load8(reinterpret_cast<const bf16*>(slot), true, 8, t);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[u * 8 + j] += t[j];
            }
            uint4 pk;
            bf162* hp = reinterpret_cast<bf162*>(&pk);
#pragma unroll
            for (int j = 0; j < 4; ++j) hp[j] = __floats2bfloat162_rn(v[u * 8 + 2 * j], v[u * 8 + 2 * j + 1]);
            *reinterpret_cast<uint4*>(slot) = pk;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (g.cq) {
              // each 32 x 32 block of the tile is one contiguous 2 KB run of the destination: plain bulk copies
              const int m1 = row0 >> 5;
              bf16* dst = reinterpret_cast<bf16*>(g.C) + (long long)tc.batch * g.c_bstride + (long long)(m1 / g.cq_mdiv) * g.cq_sr2 +
                          (long long)(m1 % g.cq_mdiv) * g.cq_sr1 + (long long)(col0 >> 5) * g.cq_sc1;
              asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 2048;" ::"l"(dst), "r"(epi_smem + out_buf * 4096)
                           : "memory");
              asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 2048;" ::"l"(dst + g.cq_sc1),
                           "r"(epi_smem + out_buf * 4096 + 2048)
                           : "memory");
            } else {
              asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(&tmC),
                           "r"(epi_smem + out_buf * 4096), "r"(col0), "r"(row0), "r"(tc.batch)
                           : "memory");
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          out_buf ^= 1;
        }
      } else if (g.trans_out) {
        // direct path: thread = row, so a warp writes 32 consecutive rows of one output column
        const int row = tc.m0 + quad * 32 + lane;
        const bool row_ok = row < g.M;
        const float rs = (g.rowscale && row_ok) ? g.rowscale[(long long)tc.batch * g.rs_bstride + row] : 1.f;
#pragma unroll 1
        for (int c = half; c < BN / 32; c += 2) {
          float v[32];
          tmem_ld_32x32(taddr + c * 32, v);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (!row_ok || col0 >= g.N) continue;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] *= g.alpha;
            if (g.bias && col0 + j < g.N) v[j] += __bfloat162float(reinterpret_cast<const bf16*>(g.bias)[col0 + j]);
            if (g.act == ACT_RELU) v[j] = fmaxf(v[j], 0.f);
            else if (g.act == ACT_SIGMOID) v[j] = sigmoidf_(v[j]);
          }
          int ncols = 32, ocol0 = col0;
          if (g.glu) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = v[2 * j] * sigmoidf_(v[2 * j + 1]);
            ncols = 16;
            ocol0 = col0 >> 1;
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (q * 8 >= ncols) break;
            const int oc = ocol0 + q * 8;
            if (oc >= Nout) break;
            const int nvalid = (Nout - oc) < 8 ? (Nout - oc) : 8;
            epi_tail8(v + q * 8, g, tc.batch, row, oc, nvalid, rs);
            if (g.out_mode == OUT_BF16) {
              bf16* C = reinterpret_cast<bf16*>(g.C) + (long long)tc.batch * g.c_bstride;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (j < nvalid) C[(long long)(oc + j) * g.ldc + row] = __float2bfloat16(v[q * 8 + j]);
            } else {
              float* C = reinterpret_cast<float*>(g.C) + (long long)tc.batch * g.c_bstride;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (j < nvalid) {
                  if (g.out_mode == OUT_F32_ATOMIC) atomicAdd(&C[(long long)(oc + j) * g.ldc + row], v[q * 8 + j]);
                  else C[(long long)(oc + j) * g.ldc + row] = v[q * 8 + j];
                }
            }
          }
        }
      } else {
        // staged path: transpose 32 rows x 64 columns through shared memory so that 8 lanes cover 128 B of a row
        const int g8 = (lane & 7) * 8;
        const int sub = lane >> 3;
#pragma unroll 1
        for (int c = half; c < BN / 64; c += 2) {
          {
            float v[32];
            tmem_ld_32x32(taddr + c * 64, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) stg[lane * STG_LD + j] = v[j];
            tmem_ld_32x32(taddr + c * 64 + 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) stg[lane * STG_LD + 32 + j] = v[j];
          }
          __syncwarp();
          const int col = n0 + c * 64 + g8;       // raw accumulator column of this lane's group
          if (col < g.N) {
            float bv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) bv[j] = 0.f;
            if (g.bias) {
              const bf16* bp = reinterpret_cast<const bf16*>(g.bias) + col;
              load8(bp, (g.N - col) >= 8 && ((reinterpret_cast<uintptr_t>(bp) & 15) == 0), g.N - col, bv);
            }
#pragma unroll 2
            for (int i = 0; i < 8; ++i) {
              const int rl = 4 * i + sub;
              const int row = tc.m0 + quad * 32 + rl;
              if (row >= g.M) continue;
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = stg[rl * STG_LD + g8 + j] * g.alpha + bv[j];
              if (g.act == ACT_RELU) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.f);
              } else if (g.act == ACT_SIGMOID) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = sigmoidf_(v[j]);
              }
              const float rs = g.rowscale ? g.rowscale[(long long)tc.batch * g.rs_bstride + row] : 1.f;
              if (g.glu) {
                float w[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) w[j] = v[2 * j] * sigmoidf_(v[2 * j + 1]);
#pragma unroll
                for (int j = 4; j < 8; ++j) w[j] = 0.f;
                const int oc = col >> 1;
                int nvalid = Nout - oc;
                if (nvalid > 4) nvalid = 4;
                // 4 outputs per lane: tail and store work on a half-filled group of 8 (never vectorised)
                float t[8];
                if (g.mul) {
                  const bf16* p = reinterpret_cast<const bf16*>(g.mul) + (long long)tc.batch * g.mul_bstride + (long long)row * g.ldmul + oc;
                  load8(p, false, nvalid, t);
#pragma unroll
                  for (int j = 0; j < 4; ++j) w[j] *= t[j];
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) w[j] *= rs;
                if (g.dmask) {
                  const bf16* p = reinterpret_cast<const bf16*>(g.dmask) + (long long)((row / g.dm_div) % g.dm_mod) * g.lddm + oc;
                  load8(p, false, nvalid, t);
#pragma unroll
                  for (int j = 0; j < 4; ++j) w[j] *= t[j];
                }
                if (g.resid) {
                  const bf16* p = reinterpret_cast<const bf16*>(g.resid) + (long long)tc.batch * g.res_bstride + (long long)row * g.ldres + oc;
                  load8(p, false, nvalid, t);
#pragma unroll
                  for (int j = 0; j < 4; ++j) w[j] += t[j];
                }
                if (g.out_mode == OUT_BF16) {
                  bf16* dst = reinterpret_cast<bf16*>(g.C) + (long long)tc.batch * g.c_bstride + (long long)row * g.ldc + oc;
#pragma unroll
                  for (int j = 0; j < 4; ++j)
                    if (j < nvalid) dst[j] = __float2bfloat16(w[j]);
                } else {
                  float* dst = reinterpret_cast<float*>(g.C) + (long long)tc.batch * g.c_bstride + (long long)row * g.ldc + oc;
#pragma unroll
                  for (int j = 0; j < 4; ++j)
                    if (j < nvalid) {
                      if (g.out_mode == OUT_F32_ATOMIC) atomicAdd(dst + j, w[j]);
                      else dst[j] = w[j];
                    }
                }
              } else {
                const int nvalid = (g.N - col) < 8 ? (g.N - col) : 8;
                epi_tail8(v, g, tc.batch, row, col, nvalid, rs);
                epi_store8(v, g, tc.batch, row, col, nvalid);
              }
            }
          }
          __syncwarp();
        }
      }
      // all TMEM reads of this accumulator stage are complete: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acce + 8 * as);
      if (warp == 2 && lane == 0) GEMM_TRACE(lt, 4);   // epilogue: tile handed to the store engine, accumulator released
    }
    if (tma_epi && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  GEMM_TRACE_CTA(3);   // end of the main phase
#ifdef FFB_GEMM_TRACE_EXTRA
  // The same moment stamped by an epilogue thread: the assembler may schedule thread 0's timer read above the barrier
  // (thread 0 is the producer lane and reaches the barrier microseconds before the epilogue warps), so slot 3 can read
  // early; slot 6 cannot, because the epilogue warps arrive last.
  if (threadIdx.x == 64 && blockIdx.x < 160) g_gemm_trace[256 + blockIdx.x * 8 + 6] = trace_now();
#endif
#ifdef FFB_GEMM_TRACE_EXTRA
  // where does the time between the end of the main phase and the exit go: the bulk stores still in flight
  // (slot 4: when they have completed) or the TMEM release (slot 5)?
  if (warp >= 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  __syncthreads();
  GEMM_TRACE_CTA(4);
#endif
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  GEMM_TRACE_CTA(5);
}

// ---------------------------------------------------------------------------
// Host side: tensor-map encoding through the driver entry point (no link-time
// dependency on libcuda) and the launcher.
// ---------------------------------------------------------------------------
// bf16 matrix [batch][rows][cols] (cols contiguous, row stride ld, batch stride bstride, all in elements);
// box = box_cols x box_rows, 128B swizzle.
int make_tmap_bf16(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, long long batch,
                   long long bstride, int box_cols, int box_rows) {
  return encode_tmap3_bf16(map, base, cols, rows, batch > 0 ? batch : 1, ld, bstride, box_cols, box_rows, 128);
}

template <int BN, bool A_MN, bool B_MN, int PEER = 0>
static int launch_cfg(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap* epi, int tma_epi, const GemmArgs& g, int batch,
                      cudaStream_t st, const PeerMaps* pm = nullptr) {
  using Cfg = GemmCfg<BN>;
  static bool attr_set = false;
  static PeerMaps no_peers;
  if (!pm) pm = &no_peers;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, PEER>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) return -2;
    attr_set = true;
  }
  const int tiles_n = (g.N + BN - 1) / BN, tiles_m = (g.M + BM - 1) / BM;
  const long long num_tiles = (long long)tiles_n * tiles_m * batch * g.splits;
  if (num_tiles > 0x7fffffffLL) return -5;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
  }
  const int grid = (int)(num_tiles < sm_count ? num_tiles : sm_count);
  launch_k(kern, grid, GEMM_THREADS, Cfg::SMEM, st, ta, tb, epi[0], epi[1], epi[2], *pm, g, (int)num_tiles, tiles_m, tiles_n, tma_epi);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

template <bool A_MN, bool B_MN>
static int launch_bn(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap* epi, int tma_epi, const GemmArgs& g,
                     int batch, cudaStream_t st) {
  switch (bn) {
    case 64: return launch_cfg<64, A_MN, B_MN>(ta, tb, epi, tma_epi, g, batch, st);
    case 128: return launch_cfg<128, A_MN, B_MN>(ta, tb, epi, tma_epi, g, batch, st);
    case 256: return launch_cfg<256, A_MN, B_MN>(ta, tb, epi, tma_epi, g, batch, st);
    default: return -4;
  }
}

}  // namespace ffb

using namespace ffb;

// Common front end of the two entry points.  peer_which: 0 none, 1 = A gathered (peer_ptrs = base of every rank's
// A slab), 2 = B gathered.  For a gathered operand the pointer / strides describe ONE slab and M (or N) is the full
// gathered extent.
static int gemm_launch(const void* A, const void* B, int a_mn, int b_mn, long long lda, long long ldb, long long a_bstride,
                       long long b_bstride, int batch, int bn, GemmArgs* args, void* stream, int peer_which, const void* const* peer_ptrs,
                       int n_peers) {
  GemmArgs g = *args;
  if (g.M <= 0 || g.N <= 0 || g.K <= 0 || batch <= 0) return -10;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -11;
  if (g.glu && (g.N & 1)) return -12;
  if (peer_which) bn = 128;
  if (bn == 0) {
    // 256-wide tiles halve the A re-reads; measured faster than 128-wide as soon as they fill one wave of the 148 SMs
    // (32768 x 256 x 1024: 27.5 vs 34.7 us; 32768 x 256 x 256: 12.0 vs 13.3 us)
    if (g.N > 128 && (long long)((g.M + 127) / 128) * ((g.N + 255) / 256) * batch * (g.splits > 0 ? g.splits : 1) >= 148) bn = 256;
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
  // extents of one slab of the gathered operand
  int a_rows = g.M, b_rows = g.N;
  if (peer_which) {
    if (n_peers < 1 || n_peers > 8 || g.peer_slab <= 0) return -16;
    if (peer_which == 1) {
      if (g.peer_slab % BM || g.peer_slab * n_peers != g.M) return -17;
      a_rows = g.peer_slab;
    } else {
      if (g.peer_slab % bn || g.peer_slab * n_peers != g.N) return -17;
      b_rows = g.peer_slab;
    }
  }
  if (a_mn) r = make_tmap_bf16(&ta, A, g.K, a_rows, lda, abatch, a_bstride, 64, BK);
  else r = make_tmap_bf16(&ta, A, a_rows, g.K, lda, abatch, a_bstride, BK, BM);
  if (r) return 1000 + r;
  if (b_mn) r = make_tmap_bf16(&tb, B, g.K, b_rows, ldb, bbatch, b_bstride, 64, BK);
  else r = make_tmap_bf16(&tb, B, b_rows, g.K, ldb, bbatch, b_bstride, BK, bn);
  if (r) return 2000 + r;
  PeerMaps pm;
  if (peer_which) {
    for (int p = 0; p < n_peers; ++p) {
      const void* base = peer_ptrs[p];
      if (reinterpret_cast<uintptr_t>(base) & 15) return -18;
      if (peer_which == 1) {
        if (a_mn) r = make_tmap_bf16(&pm.m[p], base, g.K, a_rows, lda, abatch, a_bstride, 64, BK);
        else r = make_tmap_bf16(&pm.m[p], base, a_rows, g.K, lda, abatch, a_bstride, BK, BM);
      } else {
        if (b_mn) r = make_tmap_bf16(&pm.m[p], base, g.K, b_rows, ldb, bbatch, b_bstride, 64, BK);
        else r = make_tmap_bf16(&pm.m[p], base, b_rows, g.K, ldb, bbatch, b_bstride, BK, bn);
      }
      if (r) return 3000 + r;
    }
    for (int p = n_peers; p < 8; ++p) pm.m[p] = pm.m[0];
  }
  // TMA epilogue: bf16 row-major output whose rows (and those of mul / residual) are 16-byte aligned
  CUtensorMap epi[3];
  epi[0] = ta; epi[1] = ta; epi[2] = ta;
  auto al16 = [](const void* p, long long ld, long long bs) { return p && !(reinterpret_cast<uintptr_t>(p) & 15) && !(ld % 8) && !(bs % 8); };
  int tma_epi = (g.out_mode == OUT_BF16 && !g.trans_out && !g.glu && g.N >= 64 && al16(g.C, g.ldc, g.c_bstride) && (batch == 1 || g.c_bstride != 0)) ? 1 : 0;
  if (tma_epi && g.mul && !(al16(g.mul, g.ldmul, g.mul_bstride) && (batch == 1 || g.mul_bstride != 0))) tma_epi = 0;
  if (tma_epi && g.resid && !(al16(g.resid, g.ldres, g.res_bstride) && (batch == 1 || g.res_bstride != 0))) tma_epi = 0;
  if (g.cq) {
    // block-permuted store: bf16, whole 32 x 64 warp tiles only, no mul / residual tiles (they would be fetched in matrix layout)
    if (g.out_mode != OUT_BF16 || g.trans_out || g.glu || g.mul || g.resid || (g.M % 32) || (g.N % 64)) return -23;
    if ((reinterpret_cast<uintptr_t>(g.C) & 15) || (g.cq_sr1 % 8) || (g.cq_sr2 % 8) || (g.cq_sc1 % 8) || (g.c_bstride % 8) || g.cq_mdiv < 1) return -23;
    tma_epi = 1;
  } else if (tma_epi) {
    if (make_tmap_bf16(&epi[0], g.C, g.M, g.N, g.ldc, batch, g.c_bstride, 64, 32)) tma_epi = 0;
    if (tma_epi && g.mul && make_tmap_bf16(&epi[1], g.mul, g.M, g.N, g.ldmul, batch, g.mul_bstride, 64, 32)) tma_epi = 0;
    if (tma_epi && g.resid && make_tmap_bf16(&epi[2], g.resid, g.M, g.N, g.ldres, batch, g.res_bstride, 64, 32)) tma_epi = 0;
  }
  if (tma_epi && !g.mul && !g.resid && !g.rowscale && !g.dmask && g.alpha == 1.0f) tma_epi = 2;   // fast epilogue
  if (!tma_epi && g.trans_out && g.out_mode == OUT_BF16 && !g.mul && !g.resid && !g.dmask && g.alpha == 1.0f &&
      (!g.bias || g.N <= FAST_BIAS_MAX_N) && al16(g.C, g.ldc, g.c_bstride) && (batch == 1 || g.c_bstride != 0) && g.M >= 32) {
    // fast transposed epilogue: C^T is a [N][M] matrix ([N / 2][M] with GLU) with row stride ldc; tiles of 64 (32) rows x
    // 32 contiguous elements
    const int n_out = g.glu ? (g.N >> 1) : g.N;
    if (encode_tmap3_bf16(&epi[0], g.C, g.M, n_out, batch, g.ldc, g.c_bstride, 32, g.glu ? 32 : 64, 0) == 0) tma_epi = 3;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (peer_which == 1) {
    if (a_mn && b_mn) return launch_cfg<128, true, true, 1>(ta, tb, epi, tma_epi, g, batch, st, &pm);
    return -19;
  }
  if (peer_which == 2) {
    if (!a_mn && !b_mn) return launch_cfg<128, false, false, 2>(ta, tb, epi, tma_epi, g, batch, st, &pm);
    if (a_mn && b_mn) return launch_cfg<128, true, true, 2>(ta, tb, epi, tma_epi, g, batch, st, &pm);
    return -19;
  }
  if (a_mn) {
    if (b_mn) return launch_bn<true, true>(bn, ta, tb, epi, tma_epi, g, batch, st);
    return launch_bn<true, false>(bn, ta, tb, epi, tma_epi, g, batch, st);
  }
  if (b_mn) return launch_bn<false, true>(bn, ta, tb, epi, tma_epi, g, batch, st);
  return launch_bn<false, false>(bn, ta, tb, epi, tma_epi, g, batch, st);
}

extern "C" {

// A: a_mn == 0 -> [batch][M][K] (ld = lda); a_mn == 1 -> [batch][K][M].
// B: b_mn == 0 -> [batch][N][K] (ld = ldb); b_mn == 1 -> [batch][K][N].
// A batch stride of 0 broadcasts the operand over the batch.
int ffb_gemm_bf16(const void* A, const void* B, int a_mn, int b_mn, long long lda, long long ldb, long long a_bstride,
                  long long b_bstride, int batch, int bn, GemmArgs* args, void* stream) {
  return gemm_launch(A, B, a_mn, b_mn, lda, ldb, a_bstride, b_bstride, batch, bn, args, stream, 0, nullptr, 0);
}

// All-gather fused into the GEMM: operand `peer_which` (1 = A along M, 2 = B along N) is the concatenation of
// n_peers slabs of args->peer_slab rows each, slab p starting at peer_ptrs[p] (addresses of peer GPUs' memory as
// mapped on this GPU; same strides for every slab).  The caller orders this launch behind the peers' writes.
int ffb_gemm_bf16_peer(const void* A, const void* B, int a_mn, int b_mn, long long lda, long long ldb, long long a_bstride,
                       long long b_bstride, int batch, GemmArgs* args, int peer_which, const void* const* peer_ptrs, int n_peers,
                       void* stream) {
  if (peer_which != 1 && peer_which != 2) return -20;
  return gemm_launch(A, B, a_mn, b_mn, lda, ldb, a_bstride, b_bstride, batch, 128, args, stream, peer_which, peer_ptrs, n_peers);
}

#ifdef FFB_GEMM_TRACE
int ffb_gemm_trace_read(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_gemm_trace, sizeof(unsigned long long) * (256 + 8 * 160)) == cudaSuccess ? 0 : -1;
}
#endif

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
