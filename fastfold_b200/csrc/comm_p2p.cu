// Collectives of Dynamic Axial Parallelism as kernels over NVLink / NVSwitch peer memory.
//
// Every rank owns a slab of a *symmetric heap* (same size and layout on every GPU of the DAP group, all peers
// mapped into this GPU's address space) plus a symmetric pad of 32-bit flags.  A collective is two kernels:
//
//   publish   the rank's contribution is copied into its own slot of the heap (or a producer kernel wrote it
//             there directly) and the rank raises ready[slot][rank] = epoch in every peer's flag pad;
//   consume   a kernel that needs peer data polls ready[slot][peer] in its OWN pad (local memory), then reads
//             the peer's slot with plain loads over NVLink - as a copy (all-gather, all-to-all), fused with the
//             transpose + LayerNorm that follows an all-to-all, or as TMA tiles of a GEMM operand
//             (gemm_tcgen05.cu) - and finally raises done[slot][rank] = epoch in every peer's pad, which is what a
//             later publish into the same slot waits for.
//
// Epochs are device-side counters (one per slot, advanced by the consumer), never kernel arguments, so a CUDA
// graph that contains these kernels can be replayed.  Every wait has a time limit; when it runs out the kernel
// records ST_TIMEOUT_PEER in the status word, skips the data it could not get and returns - it never spins
// forever and never traps.  Only plain peer loads / stores are used (no multimem, no multicast loads).
//
// The reference performs the same exchanges with NCCL calls through torch.distributed
// (fastfold/distributed/comm.py:42-65,146-173, comm_async.py:66-147) followed by separate rearrange / cat copies.
#include "common.cuh"
#include "comm_api.h"

namespace ffb {

// Optional phase stamps of block 0 of the copy kernels (profiling builds only: -DFFB_COMM_TRACE).
#ifdef FFB_COMM_TRACE
__device__ unsigned long long g_comm_trace[16];
#define COMM_TRACE(slot_) do { if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) g_comm_trace[slot_] = globaltimer_ns(); } while (0)
#else
#define COMM_TRACE(slot_) do {} while (0)
#endif

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Raises one flag word on every rank: ONE system-scope fence orders everything this thread has observed (its block's
// accesses through the CTA barrier, the other blocks' through the block counter) before the flag stores, which then go
// out back to back.  A release store per rank instead would serialise one NVLink round trip per rank - measured 39 us
// per small collective at 8 ranks against 15 us at 2.
__device__ __forceinline__ void signal_all(const SymmCtx& c, int word, uint32_t value) {
  __threadfence_system();
  for (int r = 0; r < c.world; ++r) st_relaxed_sys(c.flags[r] + word, value);
}

// flag pad layout (uint32 words)
__device__ __forceinline__ int w_ready(int slot, int r) { return slot * 16 + r; }
__device__ __forceinline__ int w_done(int slot, int r) { return slot * 16 + 8 + r; }
__device__ __forceinline__ int w_epoch(int slot) { return SYMM_MAX_SLOTS * 16 + slot; }             // local only
__device__ __forceinline__ int w_blocks(int slot) { return SYMM_MAX_SLOTS * 17 + slot; }            // local only

// Bounded poll of a flag in local memory; returns false on timeout.
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t want, uint64_t limit_ns) {
  if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
      __nanosleep(64);
    }
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}

// One thread: wait until flag word `base(slot, r)` reached `want` for every peer r != rank.
__device__ __forceinline__ bool wait_peers(const SymmCtx& c, bool ready_not_done, int slot, uint32_t want) {
  bool ok = true;
  for (int r = 0; r < c.world; ++r) {
    if (r == c.rank) continue;
    const uint32_t* p = c.flags[c.rank] + (ready_not_done ? w_ready(slot, r) : w_done(slot, r));
    if (!wait_flag(p, want, c.wait_ns)) {
      report(ST_TIMEOUT_PEER, (slot << 8) | r);
      ok = false;
    }
  }
  return ok;
}

// The block that finishes last raises this rank's flag in every peer's pad (and, for `done`, advances the epoch).
// Ordering: the block's accesses are collected by the CTA barrier, thread 0 orders them at GPU scope before its
// counter increment, and only the last block pays for the system-scope fence in front of the remote flag stores
// (a system-scope fence in every thread cost 3-6 us per kernel).
__device__ __forceinline__ void last_block_signal(const SymmCtx& c, int slot, uint32_t epoch, bool ready_not_done) {
  __shared__ int s_last;
  COMM_TRACE(8);
  __syncthreads();
  COMM_TRACE(9);
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t* blk = c.flags[c.rank] + w_blocks(slot);
    const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
    s_last = (atomicAdd(blk, 1u) == total - 1) ? 1 : 0;
    if (s_last) {
      *blk = 0;
      signal_all(c, ready_not_done ? w_ready(slot, c.rank) : w_done(slot, c.rank), epoch);
      if (!ready_not_done) c.flags[c.rank][w_epoch(slot)] = epoch;
    }
  }
}

constexpr int COPY_U = 8;   // independent 16-byte transfers in flight per thread in the copy kernels
constexpr int A2A_U = 4;    // rows in flight per warp in the all-to-all + LayerNorm kernel

__device__ __forceinline__ uint32_t next_epoch(const SymmCtx& c, int slot) {
  return reinterpret_cast<volatile uint32_t*>(c.flags[c.rank])[w_epoch(slot)] + 1u;
}

// ---------------------------------------------------------------------------
// publish: src -> own heap slot, then ready[slot][rank] = epoch on every peer
// ---------------------------------------------------------------------------
__global__ void symm_publish_k(SymmCtx c, int slot, long long heap_off, const uint4* __restrict__ src, long long n16) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ uint32_t s_epoch;
  COMM_TRACE(0);
  if (threadIdx.x == 0) {
    s_epoch = next_epoch(c, slot);
    // the previous use of this slot must have been read by every peer before it is overwritten
    wait_peers(c, false, slot, s_epoch - 1u);
  }
  __syncthreads();
  COMM_TRACE(1);
  uint4* dst = reinterpret_cast<uint4*>(c.heap[c.rank] + heap_off);
  if (src != nullptr) {
    // COPY_U independent 16-byte loads in flight per thread before the first store
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride * COPY_U) {
      uint4 v[COPY_U];
#pragma unroll
      for (int u = 0; u < COPY_U; ++u)
        if (i + u * stride < n16) v[u] = src[i + u * stride];
#pragma unroll
      for (int u = 0; u < COPY_U; ++u)
        if (i + u * stride < n16) dst[i + u * stride] = v[u];
    }
  }
  COMM_TRACE(2);
  last_block_signal(c, slot, s_epoch, true);
  COMM_TRACE(3);
}

// ---------------------------------------------------------------------------
// all-gather: dst[r] = slot of peer r (each of n16 16-byte units)
// all-to-all: every rank published P chunks; dst[r] = chunk `rank` of peer r
// ---------------------------------------------------------------------------
__global__ void symm_pull_k(SymmCtx c, int slot, long long heap_off, uint4* __restrict__ dst, long long n16, int all_to_all) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_epoch = next_epoch(c, slot);
    s_ok = wait_peers(c, true, slot, s_epoch) ? 1 : 0;
  }
  __syncthreads();
  if (s_ok) {
    // blockIdx.y = source rank (starting with the farthest data in flight first does not matter: every rank is one
    // NVSwitch hop away); COPY_U independent peer loads per thread are issued before the first store
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (int r = blockIdx.y; r < c.world; r += gridDim.y) {
      const uint4* src = reinterpret_cast<const uint4*>(c.heap[r] + heap_off) + (all_to_all ? (long long)c.rank * n16 : 0);
      uint4* d = dst + (long long)r * n16;
      for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride * COPY_U) {
        uint4 v[COPY_U];
#pragma unroll
        for (int u = 0; u < COPY_U; ++u)
          if (i + u * stride < n16) v[u] = src[i + u * stride];
#pragma unroll
        for (int u = 0; u < COPY_U; ++u)
          if (i + u * stride < n16) d[i + u * stride] = v[u];
      }
    }
  }
  last_block_signal(c, slot, s_epoch, false);
}

// ---------------------------------------------------------------------------
// all-to-all fused with (optional transpose and) LayerNorm.
//
// Every rank published its shard X_r in its natural layout.  mode 0 ("row -> column"): X_r is [A/P][B][C] and the
// result on this rank is Y [A][B/P][C] with Y[a][bl] = X_{a / (A/P)}[a % (A/P)][rank * B/P + bl].  mode 1
// ("column -> row"): X_r is [A][B/P][C], Y [A/P][B][C] with Y[al][b] = X_{b / (B/P)}[rank * A/P + al][b % (B/P)].
// One warp per output row of C channels: the row is read once over NVLink, written raw (the residual stream) and,
// when gamma is given, written normalised - optionally at the transposed position [b][a] (column attention and
// the "ending node" triangle attention normalise the transposed tensor).
// ---------------------------------------------------------------------------
template <int VPL>
__global__ void __launch_bounds__(128) symm_a2a_ln_k(SymmCtx c, int slot, long long heap_off, int mode, int A, int B, int C,
                                                     bf16* __restrict__ y_raw, bf16* __restrict__ y_norm, const bf16* __restrict__ gamma,
                                                     const bf16* __restrict__ beta, float eps, int transpose_norm) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_epoch = next_epoch(c, slot);
    s_ok = wait_peers(c, true, slot, s_epoch) ? 1 : 0;
  }
  __syncthreads();
  const int P = c.world;
  const int Ad = mode == 0 ? A : A / P, Bd = mode == 0 ? B / P : B;       // output extents
  const long long rows = (long long)Ad * Bd;
  const int lane = threadIdx.x & 31;
  constexpr int NV = VPL / 8;
  if (s_ok) {
    // A2A_U rows per warp and step: all their peer loads are issued before the first one is consumed
    const long long wstride = (long long)gridDim.x * 4;
    for (long long row0 = (long long)blockIdx.x * 4 + (threadIdx.x >> 5); row0 < rows; row0 += wstride * A2A_U) {
      uint4 raw[A2A_U][NV];
#pragma unroll
      for (int u = 0; u < A2A_U; ++u) {
        const long long row = row0 + u * wstride;
        if (row < rows) {
          const int a = (int)(row / Bd), b = (int)(row - (long long)a * Bd);
          int r;
          long long src_row;
          if (mode == 0) {
            const int ap = A / P;
            r = a / ap;
            src_row = (long long)(a - r * ap) * B + (long long)c.rank * Bd + b;
          } else {
            const int bp = B / P;
            r = b / bp;
            src_row = (long long)(c.rank * Ad + a) * bp + (b - r * bp);
          }
          const bf16* src = reinterpret_cast<const bf16*>(c.heap[r] + heap_off) + src_row * C;
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            const int c0 = (i * 32 + lane) * 8;
            raw[u][i] = c0 < C ? *reinterpret_cast<const uint4*>(src + c0) : make_uint4(0, 0, 0, 0);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < A2A_U; ++u) {
        const long long row = row0 + u * wstride;
        if (row >= rows) break;                                   // warp-uniform
        const int a = (int)(row / Bd), b = (int)(row - (long long)a * Bd);
        float v[VPL];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int c0 = (i * 32 + lane) * 8;
          if (c0 < C && y_raw) *reinterpret_cast<uint4*>(y_raw + row * C + c0) = raw[u][i];
          const bf162* h = reinterpret_cast<const bf162*>(&raw[u][i]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            v[i * 8 + 2 * j] = f.x;
            v[i * 8 + 2 * j + 1] = f.y;
            s += f.x + f.y;
          }
        }
        if (y_norm) {
          const float mean = warp_sum(s) / C;
          float q = 0.f;
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            const int c0 = (i * 32 + lane) * 8;
            if (c0 < C) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float d = v[i * 8 + j] - mean;
                q += d * d;
              }
            }
          }
          const float rstd = rsqrtf(warp_sum(q) / C + eps);
          const long long orow = transpose_norm ? ((long long)b * Ad + a) : row;
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            const int c0 = (i * 32 + lane) * 8;
            if (c0 < C) {
              const uint4 ug = *reinterpret_cast<const uint4*>(gamma + c0), ub = *reinterpret_cast<const uint4*>(beta + c0);
              const bf162 *hg = reinterpret_cast<const bf162*>(&ug), *hb = reinterpret_cast<const bf162*>(&ub);
              uint4 uo;
              bf162* ho = reinterpret_cast<bf162*>(&uo);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 g2 = __bfloat1622float2(hg[j]), b2 = __bfloat1622float2(hb[j]);
                ho[j] = __floats2bfloat162_rn((v[i * 8 + 2 * j] - mean) * rstd * g2.x + b2.x, (v[i * 8 + 2 * j + 1] - mean) * rstd * g2.y + b2.y);
              }
              *reinterpret_cast<uint4*>(y_norm + orow * C + c0) = uo;
            }
          }
        }
      }
    }
  }
  last_block_signal(c, slot, s_epoch, false);
}

// ---------------------------------------------------------------------------
// Two-shot all-reduce (sum) of a bf16 vector that lives at the same heap offset on every rank (the flat gradient
// buffer): rank q sums element range q over all peers in fp32 and stores the result back into every peer's copy.
// Ranges are disjoint, so no rank reads what another one is writing.  `scale` is applied to the sum.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) symm_allreduce_bf16_k(SymmCtx c, int slot, long long heap_off, long long n8, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_epoch = next_epoch(c, slot);
    // entry: every rank announces that its gradients are complete (this kernel runs after backward on the stream)
    if (blockIdx.x == 0) signal_all(c, w_ready(slot, c.rank), s_epoch);
    s_ok = wait_peers(c, true, slot, s_epoch) ? 1 : 0;
  }
  __syncthreads();
  const int P = c.world;
  const long long per = (n8 + P - 1) / P;
  const long long lo = per * c.rank;
  long long hi = lo + per;
  if (hi > n8) hi = n8;
  if (s_ok) {
    for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (long long)gridDim.x * blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int r = 0; r < P; ++r) {
        const uint4 u = *(reinterpret_cast<const uint4*>(c.heap[r] + heap_off) + i);
        const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      bf162* ho = reinterpret_cast<bf162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) ho[j] = __floats2bfloat162_rn(acc[2 * j] * scale, acc[2 * j + 1] * scale);
      for (int r = 0; r < P; ++r) *(reinterpret_cast<uint4*>(c.heap[r] + heap_off) + i) = o;
    }
  }
  // exit: every rank's range has been written everywhere before anyone reads the result (the block's remote stores
  // are collected by the barrier and ordered by ONE system-scope fence per block)
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* blk = c.flags[c.rank] + w_blocks(slot);
    s_last = (atomicAdd(blk, 1u) == gridDim.x - 1) ? 1 : 0;
    if (s_last) {
      *blk = 0;
      signal_all(c, w_done(slot, c.rank), s_epoch);
      wait_peers(c, false, slot, s_epoch);
      c.flags[c.rank][w_epoch(slot)] = s_epoch;
    }
  }
}

// ---------------------------------------------------------------------------
// One-kernel collectives ("push").  The rank's contribution is viewed as [X][Ps][Y] 16-byte units, Ps = P when chunk
// q of the middle axis is meant for rank q (all-to-all, reduce-scatter) and 1 when every rank gets everything
// (all-gather).  Phase 1 stores the units straight into the destination ranks' slots over NVLink (a store needs no
// round trip, so a thread keeps many in flight), laid out [source rank][X][Y] there; the block that finishes last
// raises ready[slot][rank] on every rank.  Phase 2 waits (bounded) for every rank's ready flag and then reads only
// LOCAL memory: it copies the slot into the result in the layout the consumer wants, sums the P partial tensors in
// fp32 (the reduce-scatter of a gathered operand's gradient), or normalises rows on the way (axis switch + LayerNorm).
// One launch per collective instead of two to five; the grid is capped so that all blocks are resident at once
// (blocks of phase 2 wait for flags that other ranks raise only after ALL of their blocks finished phase 1).
// ---------------------------------------------------------------------------
__device__ __forceinline__ int w_blocks2(int slot) { return SYMM_MAX_SLOTS * 18 + slot; }                        // local only

struct XchgArgs {
  const uint4* src;
  long long X, Y;          // units: src is [X][Ps][Y]
  long long X2, Y2;        // what arrived from one rank (X * Y units) seen as [X2][Y2] for the placement below
  int scatter;             // 1: Ps = world, chunk q -> rank q;  0: Ps = 1, everything -> every rank
  int mode;                // 0: dst[r][x2][y2]   1: dst[x2][r][y2]   2: dst[x2][y2] = sum over r (bf16 in, fp32 accumulate, bf16 out)
  uint4* dst;
};

constexpr int XCHG_THREADS = 256;
constexpr int XCHG_U = 4;

// Whole block: wait until every rank (this one included) raised ready[slot] for `epoch`.  Thread r polls rank r's flag,
// so the polls of the (up to 8) flags overlap instead of running one after the other; returns the verdict to all threads.
__device__ __forceinline__ bool wait_all_ready(const SymmCtx& c, int slot, uint32_t epoch) {
  int ok = 1;
  if ((int)threadIdx.x < c.world) {
    const int r = threadIdx.x;
    if (!wait_flag(c.flags[c.rank] + w_ready(slot, r), epoch, c.wait_ns)) {
      report(ST_TIMEOUT_PEER, (slot << 8) | r | 0x80);
      ok = 0;
    }
  }
  return __syncthreads_and(ok) != 0;
}

// Whole block: wait until every peer has raised done[slot] for `want` (the slot's previous contents have been consumed).
__device__ __forceinline__ bool wait_all_done(const SymmCtx& c, int slot, uint32_t want) {
  int ok = 1;
  if ((int)threadIdx.x < c.world && (int)threadIdx.x != c.rank) {
    const int r = threadIdx.x;
    if (!wait_flag(c.flags[c.rank] + w_done(slot, r), want, c.wait_ns)) {
      report(ST_TIMEOUT_PEER, (slot << 8) | r);
      ok = 0;
    }
  }
  return __syncthreads_and(ok) != 0;
}

// Phase 1 of a push collective; returns the epoch (all threads).  On return this block's stores have been issued and the
// last block of the grid has raised (or will raise) the ready flags.
__device__ __forceinline__ uint32_t xchg_push(const SymmCtx& c, int slot, long long heap_off, const uint4* __restrict__ src, long long X,
                                              long long Y, int scatter) {
  const uint32_t s_epoch = next_epoch(c, slot);       // the epoch word only changes when the LAST block of a kernel finishes
  wait_all_done(c, slot, s_epoch - 1u);              // every rank has finished with what its slot held before
  const int P = c.world;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (scatter) {
    const long long n = X * P * Y;
    const bool small = n < (1ll << 31);
    const uint32_t Y32 = (uint32_t)Y;
    for (long long i = t0; i < n; i += stride * XCHG_U) {
      uint4 v[XCHG_U];
#pragma unroll
      for (int u = 0; u < XCHG_U; ++u)
        if (i + u * stride < n) v[u] = src[i + u * stride];
#pragma unroll
      for (int u = 0; u < XCHG_U; ++u) {
        const long long k = i + u * stride;
        if (k < n) {
          long long x, y;
          int q;
          if (small) {                                   // 32-bit divisions: a fifth of the instructions of the 64-bit ones
            const uint32_t k32 = (uint32_t)k, xq = k32 / Y32;
            y = k32 - xq * Y32;
            x = xq / (uint32_t)P;
            q = (int)(xq - (uint32_t)x * (uint32_t)P);
          } else {
            const long long xq = k / Y;
            y = k - xq * Y;
            x = xq / P;
            q = (int)(xq - x * P);
          }
          reinterpret_cast<uint4*>(c.heap[q] + heap_off)[((long long)c.rank * X + x) * Y + y] = v[u];
        }
      }
    }
  } else {
    const long long n = X * Y;
    const long long base = (long long)c.rank * n;
    for (long long i = t0; i < n; i += stride * XCHG_U) {
      uint4 v[XCHG_U];
#pragma unroll
      for (int u = 0; u < XCHG_U; ++u)
        if (i + u * stride < n) v[u] = src[i + u * stride];
      for (int qq = 0; qq < P; ++qq) {
        const int q = (c.rank + qq) % P;               // ranks start on different destinations
        uint4* d = reinterpret_cast<uint4*>(c.heap[q] + heap_off) + base;
#pragma unroll
        for (int u = 0; u < XCHG_U; ++u)
          if (i + u * stride < n) d[i + u * stride] = v[u];
      }
    }
  }
  last_block_signal(c, slot, s_epoch, true);
  return s_epoch;
}

// End of phase 2: the last block raises done[slot][rank] on every rank and advances the slot's epoch.
__device__ __forceinline__ void xchg_finish(const SymmCtx& c, int slot, uint32_t epoch) {
  __shared__ int s_last2;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t* blk = c.flags[c.rank] + w_blocks2(slot);
    s_last2 = (atomicAdd(blk, 1u) == gridDim.x - 1) ? 1 : 0;
    if (s_last2) {
      *blk = 0;
      // `done` tells the peers that this rank has finished READING its slot; no remote access of this kernel is still
      // outstanding here, so the fence inside is cheap
      signal_all(c, w_done(slot, c.rank), epoch);
      c.flags[c.rank][w_epoch(slot)] = epoch;
    }
  }
}

__device__ __forceinline__ void acc8(float* a, const uint4& u) {
  const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(h[j]);
    a[2 * j] += f.x;
    a[2 * j + 1] += f.y;
  }
}

__global__ void __launch_bounds__(XCHG_THREADS) symm_xchg_k(SymmCtx c, int slot, long long heap_off, XchgArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t epoch = xchg_push(c, slot, heap_off, a.src, a.X, a.Y, a.scatter);
  const bool s_ok = wait_all_ready(c, slot, epoch);
  if (s_ok) {
    const int P = c.world;
    const uint4* in = reinterpret_cast<const uint4*>(c.heap[c.rank] + heap_off);
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (a.mode == 2) {
      const long long n = a.X2 * a.Y2;
      for (long long i = t0; i < n; i += stride) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int r = 0; r < P; ++r) acc8(acc, in[(long long)r * n + i]);
        uint4 o;
        bf162* ho = reinterpret_cast<bf162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ho[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        a.dst[i] = o;
      }
    } else {
      const long long n = a.X2 * a.Y2 * P;
      for (long long i = t0; i < n; i += stride * XCHG_U) {
        uint4 v[XCHG_U];
#pragma unroll
        for (int u = 0; u < XCHG_U; ++u)
          if (i + u * stride < n) v[u] = in[i + u * stride];
#pragma unroll
        for (int u = 0; u < XCHG_U; ++u) {
          const long long k = i + u * stride;
          if (k < n) {
            long long o = k;
            if (a.mode == 1) {
              if (n < (1ll << 31)) {
                const uint32_t k32 = (uint32_t)k, y2 = (uint32_t)a.Y2, x2 = (uint32_t)a.X2;
                const uint32_t rx = k32 / y2, y = k32 - rx * y2;
                const uint32_t r = rx / x2, x = rx - r * x2;
                o = ((long long)x * P + r) * a.Y2 + y;
              } else {
                const long long rx = k / a.Y2, y = k - rx * a.Y2;
                const long long r = rx / a.X2, x = rx - r * a.X2;
                o = (x * P + r) * a.Y2 + y;
              }
            }
            a.dst[o] = v[u];
          }
        }
      }
    }
  }
  xchg_finish(c, slot, epoch);
}

// Axis switch + LayerNorm as one push collective.  mode 0 ("row -> column"): this rank holds X_r [A/P][B][C], the
// result is Y [A][B/P][C]; mode 1 ("column -> row"): X_r [A][B/P][C] -> Y [A/P][B][C].  The slot receives
// [source rank][A/P][B/P][C]; phase 2 walks the output rows (one warp per row of C channels), writes the raw row (the
// residual stream) and, when gamma is given, the normalised row - optionally at the transposed position.
template <int VPL>
__global__ void __launch_bounds__(128) symm_xchg_ln_k(SymmCtx c, int slot, long long heap_off, const uint4* __restrict__ src, int mode, int A,
                                                      int B, int C, bf16* __restrict__ y_raw, bf16* __restrict__ y_norm,
                                                      const bf16* __restrict__ gamma, const bf16* __restrict__ beta, float eps, int transpose_norm) {
  pdl_launch_dependents();
  pdl_wait();
  const int P = c.world;
  const int Al = A / P, Bl = B / P;
  const long long yu = (long long)Bl * (C / 8);
  // mode 0: src [Al][P][Bl*C]; mode 1: src [P][Al][Bl*C] = X 1 with chunks of Al * Bl * C
  const uint32_t epoch = mode == 0 ? xchg_push(c, slot, heap_off, src, Al, yu, 1) : xchg_push(c, slot, heap_off, src, 1, (long long)Al * yu, 1);
  const bool s_ok = wait_all_ready(c, slot, epoch);
  const int Ad = mode == 0 ? A : Al, Bd = mode == 0 ? Bl : B;       // output extents
  const long long rows = (long long)Ad * Bd;
  const int lane = threadIdx.x & 31;
  constexpr int NV = VPL / 8;
  // lanes per row: a row of C channels is C / 8 16-byte units; narrow rows share a warp (C = 128: two rows per warp,
  // C = 64: four), so that every lane carries data.  LN_U row groups are in flight per warp and step.
  int lpr = 32;
  if (NV == 1) {
    while (lpr > 1 && (lpr >> 1) * 8 >= C) lpr >>= 1;
  }
  const int rpw = 32 / lpr;                                           // rows per warp and step
  const int sub = lane / lpr, l = lane - sub * lpr;
  constexpr int LN_U = 4;
  if (s_ok) {
    const bf16* in = reinterpret_cast<const bf16*>(c.heap[c.rank] + heap_off);
    const long long wstride = (long long)gridDim.x * 4 * rpw;
    // the loop bound depends on the warp's first row only, so all lanes of a warp run the same iterations (the
    // shuffles below are warp-wide)
    for (long long base = ((long long)blockIdx.x * 4 + (threadIdx.x >> 5)) * rpw; base < rows; base += wstride * LN_U) {
      const long long row0 = base + sub;
      uint4 raw[LN_U][NV];
#pragma unroll
      for (int u = 0; u < LN_U; ++u) {
        const long long row = row0 + u * wstride;
#pragma unroll
        for (int i = 0; i < NV; ++i) raw[u][i] = make_uint4(0, 0, 0, 0);
        if (row < rows) {
          long long srow = row;                                        // mode 0: the slot IS the result layout
          if (mode == 1) {
            const int a = (int)(row / Bd), b = (int)(row - (long long)a * Bd);
            const int r = b / Bl;
            srow = ((long long)r * Al + a) * Bl + (b - r * Bl);
          }
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            const int c0 = (i * lpr + l) * 8;
            if (c0 < C) raw[u][i] = *reinterpret_cast<const uint4*>(in + srow * C + c0);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < LN_U; ++u) {
        const long long row = row0 + u * wstride;
        const bool live = row < rows;                                  // lanes of a finished row group still take part in the shuffles
        const int a = live ? (int)(row / Bd) : 0, b = live ? (int)(row - (long long)a * Bd) : 0;
        float v[VPL];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int c0 = (i * lpr + l) * 8;
          if (live && c0 < C && y_raw) *reinterpret_cast<uint4*>(y_raw + row * C + c0) = raw[u][i];
          const bf162* h = reinterpret_cast<const bf162*>(&raw[u][i]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            v[i * 8 + 2 * j] = f.x;
            v[i * 8 + 2 * j + 1] = f.y;
            s += f.x + f.y;
          }
        }
        if (y_norm) {
          for (int o = lpr >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
          const float mean = s / C;
          float q = 0.f;
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            const int c0 = (i * lpr + l) * 8;
            if (c0 < C) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float d = v[i * 8 + j] - mean;
                q += d * d;
              }
            }
          }
          for (int o = lpr >> 1; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
          const float rstd = rsqrtf(q / C + eps);
          const long long orow = transpose_norm ? ((long long)b * Ad + a) : row;
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            const int c0 = (i * lpr + l) * 8;
            if (live && c0 < C) {
              const uint4 ug = *reinterpret_cast<const uint4*>(gamma + c0), ub = *reinterpret_cast<const uint4*>(beta + c0);
              const bf162 *hg = reinterpret_cast<const bf162*>(&ug), *hb = reinterpret_cast<const bf162*>(&ub);
              uint4 uo;
              bf162* ho = reinterpret_cast<bf162*>(&uo);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 g2 = __bfloat1622float2(hg[j]), b2 = __bfloat1622float2(hb[j]);
                ho[j] = __floats2bfloat162_rn((v[i * 8 + 2 * j] - mean) * rstd * g2.x + b2.x, (v[i * 8 + 2 * j + 1] - mean) * rstd * g2.y + b2.y);
              }
              *reinterpret_cast<uint4*>(y_norm + orow * C + c0) = uo;
            }
          }
        }
      }
    }
  }
  xchg_finish(c, slot, epoch);
}

// Raises ready[slot][rank] after a producer kernel wrote the slot directly (stream-ordered behind it), waiting first
// (pre = 1, run BEFORE the producer) for the peers to have finished with the slot's previous contents.
__global__ void symm_slot_fence_k(SymmCtx c, int slot, int pre) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint32_t e = next_epoch(c, slot);
  if (pre) {
    wait_peers(c, false, slot, e - 1u);
  } else {
    signal_all(c, w_ready(slot, c.rank), e);
  }
}

// Consumer-side bookkeeping for a kernel that read peer slots itself (e.g. the GEMM reading operand tiles through
// peer tensor maps): pre = 1 waits for every peer's ready flag (run before the consumer), pre = 0 raises done and
// advances the epoch (run after it).
__global__ void symm_consume_fence_k(SymmCtx c, int slot, int pre) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint32_t e = next_epoch(c, slot);
  if (pre) {
    wait_peers(c, true, slot, e);
  } else {
    signal_all(c, w_done(slot, c.rank), e);
    c.flags[c.rank][w_epoch(slot)] = e;
  }
}

// Test hook: waits on a ready flag that nothing raises, with a short limit; must time out and report, not hang.
__global__ void symm_wait_never_k(SymmCtx c, int slot) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const uint32_t* p = c.flags[c.rank] + w_ready(slot, (c.rank + 1) % (c.world > 1 ? c.world : 2));
    if (!wait_flag(p, 0x7fffffffu, c.wait_ns)) report(ST_TIMEOUT_PEER, slot << 8);
  }
}

}  // namespace ffb

using namespace ffb;

extern "C" {

static int grid_for(long long n, int threads, int cap) {
  long long g = (n + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return (int)g;
}

int ffb_symm_publish(const SymmCtx* c, int slot, long long heap_off, const void* src, long long bytes, void* stream) {
  if (bytes % 16 || heap_off % 16 || slot < 0 || slot >= SYMM_MAX_SLOTS) return -2;
  const long long n16 = bytes / 16;
  launch_light(symm_publish_k, grid_for((n16 + COPY_U - 1) / COPY_U, 256, 296), 256, 0, reinterpret_cast<cudaStream_t>(stream), *c, slot, heap_off, (const uint4*)src, n16);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int ffb_symm_pull(const SymmCtx* c, int slot, long long heap_off, void* dst, long long bytes_per_rank, int all_to_all, void* stream) {
  if (bytes_per_rank % 16 || heap_off % 16 || slot < 0 || slot >= SYMM_MAX_SLOTS) return -2;
  const long long n16 = bytes_per_rank / 16;
  {
    const int gx = grid_for((n16 + COPY_U - 1) / COPY_U, 256, 592 / c->world > 0 ? 592 / c->world : 1);
    launch_light(symm_pull_k, dim3(gx, c->world), 256, 0, reinterpret_cast<cudaStream_t>(stream), *c, slot, heap_off, (uint4*)dst, n16, all_to_all);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int ffb_symm_a2a_layernorm(const SymmCtx* c, int slot, long long heap_off, int mode, int A, int B, int C, void* y_raw, void* y_norm,
                           const void* gamma, const void* beta, float eps, int transpose_norm, void* stream) {
  if (C % 8 || C > 1024 || heap_off % 16 || slot < 0 || slot >= SYMM_MAX_SLOTS) return -2;
  if ((mode == 0 && (A % c->world || B % c->world)) || (mode == 1 && (A % c->world || B % c->world))) return -3;
  const long long rows = (long long)(mode == 0 ? A : A / c->world) * (mode == 0 ? B / c->world : B);
  const int grid = grid_for(rows, 4, 1184);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (C <= 256) launch_light(symm_a2a_ln_k<8>, grid, 128, 0, st, *c, slot, heap_off, mode, A, B, C, (bf16*)y_raw, (bf16*)y_norm, (const bf16*)gamma, (const bf16*)beta, eps, transpose_norm);
  else if (C <= 512) launch_light(symm_a2a_ln_k<16>, grid, 128, 0, st, *c, slot, heap_off, mode, A, B, C, (bf16*)y_raw, (bf16*)y_norm, (const bf16*)gamma, (const bf16*)beta, eps, transpose_norm);
  else launch_light(symm_a2a_ln_k<32>, grid, 128, 0, st, *c, slot, heap_off, mode, A, B, C, (bf16*)y_raw, (bf16*)y_norm, (const bf16*)gamma, (const bf16*)beta, eps, transpose_norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// One-kernel collectives.  The source is [x1][Ps][bytes_chunk / x1] (Ps = world when `scatter`, else 1); what arrives from
// one rank (bytes_chunk) is placed as [x2][bytes_chunk / x2]:  mode 0: dst [P][x2][.];  1: dst [x2][P][.];
// 2: dst [x2][.] = sum over source ranks (bf16).  The slot must hold world * bytes_chunk bytes.
int ffb_symm_xchg(const SymmCtx* c, int slot, long long heap_off, const void* src, long long x1, long long x2, long long bytes_chunk,
                  int scatter, int mode, void* dst, void* stream) {
  if (bytes_chunk % 16 || heap_off % 16 || slot < 0 || slot >= SYMM_MAX_SLOTS || x1 < 1 || x2 < 1 || mode < 0 || mode > 2) return -2;
  const long long units = bytes_chunk / 16;
  if (units % x1 || units % x2) return -3;
  XchgArgs a;
  a.src = (const uint4*)src;
  a.X = x1;
  a.Y = units / x1;
  a.X2 = x2;
  a.Y2 = units / x2;
  a.scatter = scatter;
  a.mode = mode;
  a.dst = (uint4*)dst;
  const long long work = units * c->world;
  const int grid = grid_for((work + XCHG_U - 1) / XCHG_U, XCHG_THREADS, 296);
  launch_light(symm_xchg_k, grid, XCHG_THREADS, 0, reinterpret_cast<cudaStream_t>(stream), *c, slot, heap_off, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Axis switch (+ transpose) + LayerNorm in one kernel; same arguments as ffb_symm_a2a_layernorm plus the source shard.
int ffb_symm_xchg_layernorm(const SymmCtx* c, int slot, long long heap_off, const void* src, int mode, int A, int B, int C, void* y_raw,
                            void* y_norm, const void* gamma, const void* beta, float eps, int transpose_norm, void* stream) {
  if (C % 8 || C > 1024 || heap_off % 16 || slot < 0 || slot >= SYMM_MAX_SLOTS) return -2;
  if (A % c->world || B % c->world) return -3;
  const long long rows = (long long)(mode == 0 ? A : A / c->world) * (mode == 0 ? B / c->world : B);
  // all blocks must be resident at once (they wait for flags that peers raise after ALL of their blocks pushed): four
  // 128-thread blocks per SM for the narrow instantiation (92 registers), fewer for the wide ones
  const int grid = grid_for(rows, 4, C <= 256 ? 592 : (C <= 512 ? 296 : 148));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (C <= 256) launch_light(symm_xchg_ln_k<8>, grid, 128, 0, st, *c, slot, heap_off, (const uint4*)src, mode, A, B, C, (bf16*)y_raw, (bf16*)y_norm, (const bf16*)gamma, (const bf16*)beta, eps, transpose_norm);
  else if (C <= 512) launch_light(symm_xchg_ln_k<16>, grid, 128, 0, st, *c, slot, heap_off, (const uint4*)src, mode, A, B, C, (bf16*)y_raw, (bf16*)y_norm, (const bf16*)gamma, (const bf16*)beta, eps, transpose_norm);
  else launch_light(symm_xchg_ln_k<32>, grid, 128, 0, st, *c, slot, heap_off, (const uint4*)src, mode, A, B, C, (bf16*)y_raw, (bf16*)y_norm, (const bf16*)gamma, (const bf16*)beta, eps, transpose_norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int ffb_symm_allreduce_bf16(const SymmCtx* c, int slot, long long heap_off, long long n_elems, float scale, void* stream) {
  if (n_elems % 8 || heap_off % 16 || slot < 0 || slot >= SYMM_MAX_SLOTS) return -2;
  const long long n8 = n_elems / 8;
  const long long per = (n8 + c->world - 1) / c->world;
  launch_light(symm_allreduce_bf16_k, grid_for(per, 256, 296), 256, 0, reinterpret_cast<cudaStream_t>(stream), *c, slot, heap_off, n8, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int ffb_symm_slot_fence(const SymmCtx* c, int slot, int pre, void* stream) {
  launch_light(symm_slot_fence_k, 1, 32, 0, reinterpret_cast<cudaStream_t>(stream), *c, slot, pre);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int ffb_symm_consume_fence(const SymmCtx* c, int slot, int pre, void* stream) {
  launch_light(symm_consume_fence_k, 1, 32, 0, reinterpret_cast<cudaStream_t>(stream), *c, slot, pre);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

#ifdef FFB_COMM_TRACE
int ffb_comm_trace_read(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_comm_trace, sizeof(unsigned long long) * 16) == cudaSuccess ? 0 : -1;
}
#endif

int ffb_symm_wait_never(const SymmCtx* c, int slot, void* stream) {
  launch_light(symm_wait_never_k, 1, 32, 0, reinterpret_cast<cudaStream_t>(stream), *c, slot);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
