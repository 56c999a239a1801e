// Fused gated-attention core for the Evoformer's axial attentions (forward):
//
//   O[b,i,h,:] = softmax_j( scale * <Q[b,i,h,:], K[b,j,h,:]> + bias[h,i,j]  |  key mask[b,j] ) V[b,j,h,:]
//
// in one kernel, flash style: logits never reach global memory.  The pair bias
// is shared by every batch row b (MSA row attention: all N_seq rows; triangle
// attention: all N_res rows), so a CTA owns one (head, 128-query tile) and
// walks over batch rows; for sequences of up to 256 keys the bias tiles are
// loaded once and stay resident in shared memory for the whole walk.
//
// Per CTA (320 threads):
//   warp 0     TMA producer: Q tile, K/V key blocks (64B-swizzled, straight out of
//              the fused QKV projection output, no head transposes), bias tiles
//   warp 1     MMA issuer: S = Q K^T (tcgen05, 128 x 128 x 32) into one of two TMEM
//              stages; per key half, PV = P V (128 x 32 x 64) into its own TMEM stage
//   warps 2-9  softmax: two threads per query row, each owning one 64-key half of
//              every 128-key block (warps 2-5: keys 0-63, warps 6-9: keys 64-127).
//              A thread runs its own online softmax over its keys: tcgen05.ld of S,
//              scale + bias (+ mask), running max / sum, P written as bf16 into the
//              128B-swizzled shared tile that its half's PV MMA reads; its partial
//              output row lives in registers.  The two halves of a row are merged
//              once per item through shared memory (flash-decoding style), each
//              thread finishing 16 of the 32 output channels.
// The issuer runs one block ahead across item boundaries, so S of block g+1 and
// the PV products of block g overlap the softmax of block g.
// Masked keys get a huge negative logit (replaced, not added; -2^30 here, -1e9 in the reference's
// softmax kernels, softmax_cuda_kernel.cu:338-423,618-706 - same weights); keys beyond the
// sequence end get -inf.  The kernel also stores log2-domain row statistics
// L2 = m * log2(e) + log2(l) for the backward kernel.
//
// Replaces logits matmul + fused_softmax + weights*v of the reference
// (fastfold/model/fastnn/ops.py:304-319) and its unused Triton forward-only
// attention core (kernel/triton/attention_core.py:12-121).
#include "common.cuh"
#include "tmap.h"

namespace ffb {

constexpr int AT_BQ = 128;      // queries per tile
constexpr int AT_BK = 128;      // keys per block
constexpr int AT_THREADS = 320; // producer warp, MMA warp, 8 softmax / gradient warps
constexpr int AT_KV_STAGES = 3;
constexpr float LOG2E = 1.4426950408889634f;

struct AttnArgs {
  int B, H, n_q, n_k;            // batch rows, heads, query / key lengths
  int n_qt, n_kb;                // query tiles, key blocks
  int items;                     // H * n_qt * B work items
  int bias_resident;             // 1: n_kb <= 2, bias tiles stay in shared memory across batch rows
  float scale;                   // logit scale
  const bf16* mask;              // [B][n_k] or null
  long long mask_bstride;
  bf16* out;                     // [B][n_q][H*D]
  long long out_bstride, out_rstride;
  float* lse2;                   // [B][H][n_q] or null
  int has_bias;
};

// descriptor with explicit layout code: 2 = 128B swizzle, 4 = 64B swizzle
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(layout) << 61;
  return d;
}

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// two bf16 packed in a word -> two floats (low half first)
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Keep-bits of 64 consecutive keys starting at kbase: bit c of (lo | hi << 32) is set when key kbase + c is inside the
// sequence and its mask entry is non-zero.  `valid` gets the in-sequence bits alone.  One warp-wide call.
__device__ __forceinline__ void key_bits(const bf16* mrow, int kbase, int n_k, int lane, uint32_t& keep_lo, uint32_t& keep_hi,
                                         uint32_t& valid_lo, uint32_t& valid_hi) {
  const int k_a = kbase + lane, k_b = kbase + 32 + lane;
  const bool in_a = k_a < n_k, in_b = k_b < n_k;
  bool on_a = in_a, on_b = in_b;
  if (mrow) {
    if (in_a) on_a = __bfloat162float(mrow[k_a]) != 0.f;
    if (in_b) on_b = __bfloat162float(mrow[k_b]) != 0.f;
  }
  valid_lo = __ballot_sync(0xffffffffu, in_a);
  valid_hi = __ballot_sync(0xffffffffu, in_b);
  keep_lo = __ballot_sync(0xffffffffu, on_a);
  keep_hi = __ballot_sync(0xffffffffu, on_b);
}

// Masked keys take this logit (replaced, not added).  -2^30 instead of the reference's -1e9: its product with log2(e) is
// exact in fp32, so a fully masked row still comes out as exactly uniform weights from the fused multiply-add form
// exp2(v * log2e - m * log2e); any finite logit next to it underflows to weight 0 either way.
constexpr float MASKED_LOGIT = -1073741824.f;

// Per-warp table of the 64 keys of a half block: (keep, penalty) with logit' = logit * keep + penalty, i.e. (1, 0) for a
// normal key, (0, MASKED_LOGIT) for a masked one, (0, -inf) past the end of the sequence.  One FMA per logit instead of
// bit tests and selects.
__device__ __forceinline__ void write_key_table(float2* kp, int lane, uint32_t keep_lo, uint32_t keep_hi, uint32_t valid_lo,
                                                uint32_t valid_hi) {
  __syncwarp();                                   // the previous block's reads of the table are done
  const bool k0 = (keep_lo >> lane) & 1u, v0 = (valid_lo >> lane) & 1u, k1 = (keep_hi >> lane) & 1u, v1 = (valid_hi >> lane) & 1u;
  kp[lane] = v0 ? (k0 ? make_float2(1.f, 0.f) : make_float2(0.f, MASKED_LOGIT)) : make_float2(0.f, -INFINITY);
  kp[lane + 32] = v1 ? (k1 ? make_float2(1.f, 0.f) : make_float2(0.f, MASKED_LOGIT)) : make_float2(0.f, -INFINITY);
  __syncwarp();
}

struct AttnSmem {
  // offsets (bytes) from the 1024-aligned base
  static constexpr int Q = 0;                                  // 2 x [128][64 B]            16 KB
  static constexpr int KV = Q + 2 * 8192;                      // STAGES x (K 8 KB + V 8 KB) 48 KB
  static constexpr int BIAS = KV + AT_KV_STAGES * 16384;       // 2 x [2 boxes][128][128 B]  64 KB
  static constexpr int P = BIAS + 2 * 32768;                   // 2 x [2 chunks][128][128 B] 64 KB
  static constexpr int XCH = P + 2 * 32768;                    // [2 halves][18][128] floats 18 KB
  static constexpr int KP = XCH + 2 * 18 * 128 * 4;            // [8 warps][64] (keep, penalty) pairs 4 KB
  static constexpr int BARS = KP + 8 * 64 * 8;
  static constexpr int TOTAL = BARS + 512 + 1024;
};

template <int D>   // head dim: 32 (64-byte rows)
__global__ void __launch_bounds__(AT_THREADS, 1) attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                 const __grid_constant__ CUtensorMap tmK,
                                                                 const __grid_constant__ CUtensorMap tmV,
                                                                 const __grid_constant__ CUtensorMap tmBias, const AttnArgs a) {
  pdl_launch_dependents();
  static_assert(D == 32, "head dim 32");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + AttnSmem::BARS);
  // barrier map (8 bytes each)
  const uint32_t b0 = smem_u32(bars);
  const uint32_t q_full = b0, q_empty = b0 + 16;                       // 2 + 2
  const uint32_t kv_full = b0 + 32, kv_empty = kv_full + 8 * AT_KV_STAGES;
  const uint32_t bias_full = kv_empty + 8 * AT_KV_STAGES, bias_empty = bias_full + 16;
  const uint32_t s_full = bias_empty + 16, s_empty = s_full + 16;
  const uint32_t p_full = s_empty + 16;                                // [stage][half]
  const uint32_t o_full = p_full + 32;                                 // [stage][half]
  const uint32_t x_ready = o_full + 32, x_done = x_ready + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + AttnSmem::BARS + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(q_full + 8 * s, 1);
      mbar_init(q_empty + 8 * s, 1);
      mbar_init(bias_full + 8 * s, 1);
      mbar_init(bias_empty + 8 * s, 8);
      mbar_init(s_full + 8 * s, 1);
      mbar_init(s_empty + 8 * s, 8);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(p_full + 8 * s, 4);
      mbar_init(o_full + 8 * s, 1);
    }
    for (int s = 0; s < AT_KV_STAGES; ++s) {
      mbar_init(kv_full + 8 * s, 1);
      mbar_init(kv_empty + 8 * s, 1);
    }
    mbar_init(x_ready, 8);
    mbar_init(x_done, 8);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    if (a.has_bias) prefetch_tmap(&tmBias);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  pdl_wait();          // the prologue above touched no global memory; everything below may
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t TM_S = 0, TM_O = 256;       // S: 2 stages x 128 columns; O: [stage][half] x 32 columns

  // contiguous range of work items for this CTA; item = (h * n_qt + qt) * B + b
  const int per = (a.items + gridDim.x - 1) / gridDim.x;
  const int it_begin = blockIdx.x * per;
  int it_end = it_begin + per;
  if (it_end > a.items) it_end = a.items;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t jt = 0, qi = 0, bt = 0;     // key-block, item and streamed-bias counters
      uint32_t gidx = 0;                   // index of the current (head, query tile) group within this CTA
      int prev_group = -1;
      bool ok = true;
      for (int item = it_begin; item < it_end && ok; ++item, ++qi) {
        const int b = item % a.B;
        const int grp = item / a.B;
        const int qt = grp % a.n_qt, h = grp / a.n_qt;
        const int q0 = qt * AT_BQ;
        const uint32_t qs = qi & 1;
        if (!mbar_wait(q_empty + 8 * qs, ((qi >> 1) & 1) ^ 1)) { report(ST_TIMEOUT_MMA, 10); *abort_flag = 1; break; }
        mbar_expect_tx(q_full + 8 * qs, 8192);
        tma_load_3d(base + AttnSmem::Q + qs * 8192, &tmQ, q_full + 8 * qs, h * D, q0, b);
        const bool load_bias = a.has_bias && (!a.bias_resident || grp != prev_group);
        if (a.bias_resident && grp != prev_group) gidx = (prev_group < 0) ? 0 : gidx + 1;
        prev_group = grp;
        for (int j = 0; j < a.n_kb && ok; ++j, ++jt) {
          const int k0 = j * AT_BK;
          if (load_bias) {
            const uint32_t bs = a.bias_resident ? (uint32_t)j : (bt & 1);
            if (!a.bias_resident) {
              if (!mbar_wait(bias_empty + 8 * bs, ((bt >> 1) & 1) ^ 1)) { report(ST_TIMEOUT_EPI, 11); *abort_flag = 1; ok = false; break; }
            } else if (gidx > 0) {
              // resident slot j is released by the softmax warps once per group, after their last read of it
              if (!mbar_wait(bias_empty + 8 * bs, (gidx - 1) & 1)) { report(ST_TIMEOUT_EPI, 13); *abort_flag = 1; ok = false; break; }
            }
            mbar_expect_tx(bias_full + 8 * bs, 32768);
            tma_load_3d(base + AttnSmem::BIAS + bs * 32768, &tmBias, bias_full + 8 * bs, k0, q0, h);
            tma_load_3d(base + AttnSmem::BIAS + bs * 32768 + 16384, &tmBias, bias_full + 8 * bs, k0 + 64, q0, h);
            ++bt;
          }
          const uint32_t s = jt % AT_KV_STAGES;
          if (!mbar_wait(kv_empty + 8 * s, ((jt / AT_KV_STAGES) & 1) ^ 1)) { report(ST_TIMEOUT_MMA, 12); *abort_flag = 1; ok = false; break; }
          mbar_expect_tx(kv_full + 8 * s, 16384);
          tma_load_3d(base + AttnSmem::KV + s * 16384, &tmK, kv_full + 8 * s, h * D, k0, b);
          tma_load_3d(base + AttnSmem::KV + s * 16384 + 8192, &tmV, kv_full + 8 * s, h * D, k0, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc_s = make_idesc_bf16(128, AT_BK, 0, 0);     // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);         // P (K-major) x V (MN-major)
      const uint32_t total = (uint32_t)(it_end > it_begin ? it_end - it_begin : 0) * (uint32_t)a.n_kb;
      bool ok = true;
      uint32_t s_g = 0, s_qi = 0, s_j = 0;     // next S product: global block, item and block-in-item counters
      auto issue_s = [&]() -> bool {
        const uint32_t s = s_g % AT_KV_STAGES, sb = s_g & 1, qs = s_qi & 1;
        if (s_j == 0 && !mbar_wait(q_full + 8 * qs, (s_qi >> 1) & 1)) { report(ST_TIMEOUT_TMA, 22); return false; }
        if (!mbar_wait(kv_full + 8 * s, (s_g / AT_KV_STAGES) & 1)) { report(ST_TIMEOUT_TMA, 20); return false; }
        if (!mbar_wait(s_empty + 8 * sb, ((s_g >> 1) & 1) ^ 1)) { report(ST_TIMEOUT_EPI, 21); return false; }
        tc_fence_after();
        const uint32_t qa = base + AttnSmem::Q + qs * 8192;
        const uint32_t ka = base + AttnSmem::KV + s * 16384;
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem + TM_S + sb * 128, make_desc(qa + k * 32, 16, 512, 4), make_desc(ka + k * 32, 16, 512, 4), idesc_s, k > 0 ? 1u : 0u);
        umma_commit(s_full + 8 * sb);
        ++s_g;
        if (++s_j == (uint32_t)a.n_kb) {
          umma_commit(q_empty + 8 * qs);      // all S products of this item issued: the Q slot drains with them
          s_j = 0;
          ++s_qi;
        }
        return true;
      };
      if (total > 0) ok = issue_s();
      for (uint32_t g = 0; g < total && ok; ++g) {
        if (g + 1 < total) ok = issue_s();
        if (!ok) break;
        const uint32_t pb = g & 1, s = g % AT_KV_STAGES;
        const uint32_t pa = base + AttnSmem::P + pb * 32768;
        const uint32_t va = base + AttnSmem::KV + s * 16384 + 8192;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (!mbar_wait(p_full + 8 * (pb * 2 + half), (g >> 1) & 1)) { report(ST_TIMEOUT_EPI, 23); ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem + TM_O + (pb * 2 + half) * 32, make_desc(pa + half * 16384 + k * 32, 16, 1024, 2),
                      make_desc(va + (half * 4 + k) * 1024, 16, 512, 4), idesc_o, k > 0 ? 1u : 0u);
          umma_commit(o_full + 8 * (pb * 2 + half));
        }
        if (!ok) break;
        umma_commit(kv_empty + 8 * s);
      }
      if (!ok) *abort_flag = 1;
    }
    __syncwarp();
  } else {
    // ---------------- softmax / output (warps 2..9): thread = (query row, key half) ----------------
    const int quad = warp & 3;                      // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;               // which 64 keys of every block
    const int r = quad * 32 + lane;                 // row within the query tile
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    float* xch_mine = reinterpret_cast<float*>(sm + AttnSmem::XCH) + half * (18 * 128) + r;
    const float* xch_other = reinterpret_cast<const float*>(sm + AttnSmem::XCH) + (half ^ 1) * (18 * 128) + r;
    uint32_t jt = 0, bt = 0, ic = 0;
    int prev_group = -1;
    bool ok = true;
    for (int item = it_begin; item < it_end && ok; ++item, ++ic) {
      const int b = item % a.B;
      const int grp = item / a.B;
      const int qt = grp % a.n_qt, h = grp / a.n_qt;
      const int q0 = qt * AT_BQ;
      const bool new_bias = a.has_bias && (!a.bias_resident || grp != prev_group);
      prev_group = grp;
      const bool last_of_group = (item + 1 >= it_end) || ((item + 1) / a.B != grp);
      float o[D];
#pragma unroll
      for (int c = 0; c < D; ++c) o[c] = 0.f;
      float m = -INFINITY, l = 0.f, alpha_prev = 1.f;       // m in natural-log units
      const bf16* mrow = a.mask ? a.mask + (long long)b * a.mask_bstride : nullptr;
      for (int j = 0; j < a.n_kb; ++j, ++jt) {
        const int kbase = j * AT_BK + half * 64;
        const uint32_t sb = jt & 1;
        // key bits first: their global loads overlap the wait for S
        uint32_t keep_lo, keep_hi, valid_lo, valid_hi;
        key_bits(mrow, kbase, a.n_k, lane, keep_lo, keep_hi, valid_lo, valid_hi);
        const bool plain = (keep_lo & keep_hi) == 0xffffffffu;         // every key of this half in range and unmasked
        uint32_t bs = 0;
        if (a.has_bias) {
          bs = a.bias_resident ? (uint32_t)j : (bt & 1);
          if (new_bias) {
            // resident tiles: loaded once per (head, tile) group, parity advances once per group change
            const uint32_t par = a.bias_resident ? ((bt / a.n_kb) & 1) : ((bt >> 1) & 1);
            if (!mbar_wait(bias_full + 8 * bs, par)) { if (lane == 0) report(ST_TIMEOUT_TMA, 30); ok = false; }
            ++bt;
          }
        }
        if (ok && !mbar_wait(s_full + 8 * sb, (jt >> 1) & 1)) { if (lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_MMA, 31); ok = false; }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // ---- logits of this row's 64 keys in registers ----
        float s[64];
        tmem_ld_32x32(lane_base + TM_S + sb * 128 + half * 64, s);
        tmem_ld_32x32(lane_base + TM_S + sb * 128 + half * 64 + 32, s + 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty + 8 * sb);          // S stage may be overwritten by the next-but-one block
        if (a.has_bias) {
          const uint8_t* brow = sm + AttnSmem::BIAS + bs * 32768 + half * 16384 + r * 128;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint4 raw = *reinterpret_cast<const uint4*>(brow + ((u ^ (r & 7)) << 4));
            s[u * 8 + 0] = fmaf(s[u * 8 + 0], a.scale, bf_lo(raw.x));
            s[u * 8 + 1] = fmaf(s[u * 8 + 1], a.scale, bf_hi(raw.x));
            s[u * 8 + 2] = fmaf(s[u * 8 + 2], a.scale, bf_lo(raw.y));
            s[u * 8 + 3] = fmaf(s[u * 8 + 3], a.scale, bf_hi(raw.y));
            s[u * 8 + 4] = fmaf(s[u * 8 + 4], a.scale, bf_lo(raw.z));
            s[u * 8 + 5] = fmaf(s[u * 8 + 5], a.scale, bf_hi(raw.z));
            s[u * 8 + 6] = fmaf(s[u * 8 + 6], a.scale, bf_lo(raw.w));
            s[u * 8 + 7] = fmaf(s[u * 8 + 7], a.scale, bf_hi(raw.w));
          }
          if (!a.bias_resident || last_of_group) {
            __syncwarp();
            if (lane == 0) mbar_arrive(bias_empty + 8 * bs);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 64; ++c) s[c] *= a.scale;
        }
        if (!plain) {
          float2* kp = reinterpret_cast<float2*>(sm + AttnSmem::KP) + (warp - 2) * 64;
          write_key_table(kp, lane, keep_lo, keep_hi, valid_lo, valid_hi);
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            const float4 e = *reinterpret_cast<const float4*>(kp + c);       // same address in every lane: broadcast
            s[c] = fmaf(s[c], e.x, e.y);
            s[c + 1] = fmaf(s[c + 1], e.z, e.w);
          }
        }
        float mx0 = m, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
          mx0 = fmaxf(mx0, s[c]);
          mx1 = fmaxf(mx1, s[c + 1]);
          mx2 = fmaxf(mx2, s[c + 2]);
          mx3 = fmaxf(mx3, s[c + 3]);
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        const float mxs = (mx == -INFINITY) ? 0.f : mx;        // a half with no key in range yet: all p = 0
        const float alpha = ex2f((m - mxs) * LOG2E);            // m = -inf on the first block -> 0
        m = mx;
        // ---- P = exp(s - m) as bf16 into the swizzled A-operand tile ----
        uint8_t* prow = sm + AttnSmem::P + sb * 32768 + half * 16384 + r * 128;
        float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
        {
          const float nm = -mxs * LOG2E;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            float p[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) p[e] = ex2f(fmaf(s[u * 8 + e], LOG2E, nm));
            sum0 += p[0] + p[4];
            sum1 += p[1] + p[5];
            sum2 += p[2] + p[6];
            sum3 += p[3] + p[7];
            uint4 pk;
            bf162* hp = reinterpret_cast<bf162*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e) hp[e] = __floats2bfloat162_rn(p[2 * e], p[2 * e + 1]);
            *reinterpret_cast<uint4*>(prow + ((u ^ (r & 7)) << 4)) = pk;
          }
        }
        l = l * alpha + ((sum0 + sum1) + (sum2 + sum3));
        fence_proxy_async_smem();                              // generic-proxy P stores -> visible to the MMA (async proxy)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + 8 * (sb * 2 + half));
        // previous block's PV (if any) joins the register accumulator with the scaling that preceded this block
        if (j > 0) {
          const uint32_t ob = (jt - 1) & 1;
          bool w = mbar_wait(o_full + 8 * (ob * 2 + half), ((jt - 1) >> 1) & 1);
          if (!w && lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_MMA, 32);
          w = __all_sync(0xffffffffu, w);
          if (!w) { ok = false; break; }
          tc_fence_after();
          float pv[D];
          tmem_ld_32x32(lane_base + TM_O + (ob * 2 + half) * 32, pv);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < D; ++c) o[c] = o[c] * alpha_prev + pv[c];
        }
        alpha_prev = alpha;
      }
      if (!ok) break;
      // last block's PV
      {
        const uint32_t ob = (jt - 1) & 1;
        bool w = mbar_wait(o_full + 8 * (ob * 2 + half), ((jt - 1) >> 1) & 1);
        if (!w && lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_MMA, 33);
        w = __all_sync(0xffffffffu, w);
        if (!w) { ok = false; break; }
        tc_fence_after();
        float pv[D];
        tmem_ld_32x32(lane_base + TM_O + (ob * 2 + half) * 32, pv);
        tmem_ld_wait();
        tc_fence_before();
#pragma unroll
        for (int c = 0; c < D; ++c) o[c] = o[c] * alpha_prev + pv[c];
      }
      // ---- merge the two key halves of the row: this thread finishes channels [half * 16, half * 16 + 16) ----
      if (ic > 0) {
        bool w = mbar_wait(x_done, (ic - 1) & 1);              // the previous item's exchange has been read
        if (!w && lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_EPI, 34);
        w = __all_sync(0xffffffffu, w);
        if (!w) { ok = false; break; }
      }
      xch_mine[0] = m;
      xch_mine[128] = l;
#pragma unroll
      for (int c = 0; c < 16; ++c) xch_mine[(2 + c) * 128] = half ? o[c] : o[16 + c];
      __syncwarp();
      if (lane == 0) mbar_arrive(x_ready);
      {
        bool w = mbar_wait(x_ready, ic & 1);
        if (!w && lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_EPI, 35);
        w = __all_sync(0xffffffffu, w);
        if (!w) { ok = false; break; }
      }
      const float pm = xch_other[0], pl = xch_other[128];
      float po[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) po[c] = xch_other[(2 + c) * 128];
      __syncwarp();
      if (lane == 0) mbar_arrive(x_done);
      const float mt = fmaxf(m, pm);                           // finite: block 0 of half 0 always holds a key in range
      const float w_me = ex2f((m - mt) * LOG2E), w_ot = ex2f((pm - mt) * LOG2E);
      const float lt = l * w_me + pl * w_ot;
      const int qrow = q0 + r;
      if (qrow < a.n_q) {
        const float inv = 1.f / lt;
        const float f_me = w_me * inv, f_ot = w_ot * inv;
        bf16* dst = a.out + (long long)b * a.out_bstride + (long long)qrow * a.out_rstride + h * D + half * 16;
#pragma unroll
        for (int c = 0; c < 16; c += 8) {
          uint4 pk;
          bf162* hp = reinterpret_cast<bf162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int cc = c + 2 * e;
            const float mine0 = half ? o[16 + cc] : o[cc], mine1 = half ? o[16 + cc + 1] : o[cc + 1];
            hp[e] = __floats2bfloat162_rn(mine0 * f_me + po[cc] * f_ot, mine1 * f_me + po[cc + 1] * f_ot);
          }
          *reinterpret_cast<uint4*>(dst + c) = pk;
        }
        // A row whose keys are all masked has uniform weights; its statistic m * log2e + log2(l) would lose log2(l) to
        // rounding (|m| = 2^30), so such rows are flagged with -inf and the backward pass uses 1 / n_k for them.
        if (a.lse2 && half == 0)
          a.lse2[((long long)b * a.H + h) * a.n_q + qrow] = (mt == MASKED_LOGIT) ? -INFINITY : mt * LOG2E + log2f(lt);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------
static int make_tmap3(CUtensorMap* map, const void* ptr, long long d0, long long d1, long long d2, long long s1, long long s2, int b0,
                      int b1, int swizzle_bytes) {
  return encode_tmap3_bf16(map, ptr, d0, d1, d2, s1, s2, b0, b1, swizzle_bytes);
}

}  // namespace ffb

using namespace ffb;

extern "C" {

// q, k, v: bf16, element (b, i, h, c) at ptr[b * bstride + i * rstride + h * D + c]; D = 32.
// bias: bf16 [H][n_q][n_k] or null; mask: bf16 [B][n_k] or null (0 = masked key).
// out: bf16 (b, i, h, c) at out[b * out_bstride + i * out_rstride + h * D + c]; lse2: fp32 [B][H][n_q] or null.
int ffb_attention_fwd(const void* q, const void* k, const void* v, long long q_bstride, long long q_rstride, long long kv_bstride,
                      long long kv_rstride, const void* bias, const void* mask, long long mask_bstride, void* out,
                      long long out_bstride, long long out_rstride, float* lse2, int B, int H, int n_q, int n_k, int D, float scale,
                      void* stream) {
  if (D != 32) return -2;
  if ((q_rstride % 8) || (kv_rstride % 8) || (q_bstride % 8) || (kv_bstride % 8) || (out_rstride % 8) || (out_bstride % 8)) return -3;
  if (bias && (n_k % 8)) return -4;
  if (mask && (mask_bstride % 8)) return -5;
  AttnArgs a;
  a.B = B; a.H = H; a.n_q = n_q; a.n_k = n_k;
  a.n_qt = (n_q + AT_BQ - 1) / AT_BQ;
  a.n_kb = (n_k + AT_BK - 1) / AT_BK;
  const long long items = (long long)H * a.n_qt * B;
  if (items <= 0 || items > 0x7fffffffLL) return -6;
  a.items = (int)items;
  a.bias_resident = (bias && a.n_kb <= 2) ? 1 : 0;
  a.scale = scale;
  a.mask = (const bf16*)mask;
  a.mask_bstride = mask_bstride;
  a.out = (bf16*)out;
  a.out_bstride = out_bstride;
  a.out_rstride = out_rstride;
  a.lse2 = lse2;
  a.has_bias = bias ? 1 : 0;
  CUtensorMap tq, tk, tv, tb;
  // the q/k/v views are addressed as [B][n][H*D] slabs of a possibly wider row (fused qkv projection output)
  if (make_tmap3(&tq, q, (long long)H * D, n_q, B, q_rstride, q_bstride, D, AT_BQ, 64)) return -10;
  if (make_tmap3(&tk, k, (long long)H * D, n_k, B, kv_rstride, kv_bstride, D, AT_BK, 64)) return -11;
  if (make_tmap3(&tv, v, (long long)H * D, n_k, B, kv_rstride, kv_bstride, D, AT_BK, 64)) return -12;
  if (bias) {
    if (make_tmap3(&tb, bias, n_k, n_q, H, n_k, (long long)n_q * n_k, 64, AT_BQ, 128)) return -13;
  } else {
    tb = tq;
  }
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem::TOTAL) != cudaSuccess) return -14;
    attr = true;
  }
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
  }
  // groups of B consecutive items share their bias tiles: give every CTA whole multiples of a sensible chunk
  int grid = items < sm_count ? (int)items : sm_count;
  launch_k(attn_fwd_kernel<32>, grid, AT_THREADS, AttnSmem::TOTAL, reinterpret_cast<cudaStream_t>(stream), tq, tk, tv, tb, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -15;
}

}  // extern "C"

// ===========================================================================
// Backward.
//
// One CTA owns one (batch row, head) at a time and keeps every gradient of it
// on chip: for each key block j (outer) and query tile i (inner)
//     S  = Q_i K_j^T,  dP = dO_i V_j^T                  (tcgen05 -> TMEM)
//     P  = exp2(S * scale*log2e + bias*log2e - L2_i),   dS = P o (dP - D_i)
//     dV_j += P^T dO_i,  dK_j += scale dS^T Q_i,  dQ_i += scale dS K_j
// with dK_j / dV_j (current j) and dQ_i (all i, n_q <= 512) accumulating in
// TMEM.  P and dS are written once into 128B-swizzled shared tiles and are
// read by the tensor core in both orientations (K-major for dQ, MN-major for
// dK / dV), so nothing is transposed.  Q_i, K_j, V_j, dO_i tiles are loaded
// once by TMA (64B swizzle) and serve as K-major operands of the S / dP
// products and as MN-major operands of the gradient products.  The unscaled
// dS is also stored (bf16) for the pair-bias gradient, which is its sum over
// batch rows.  D_i = rowsum(dO o O) is computed at the start of each item.
//
// The reference has no attention backward of its own: autograd differentiates
// its unfused matmul / softmax chain (fastfold/model/fastnn/ops.py:304-319,
// kernel/softmax.py:39-59).
// ===========================================================================
namespace ffb {

struct AttnBwdArgs {
  int B, H, n_q, n_k, n_qt, n_kb, items;
  float scale, scale_log2e;
  const bf16* mask;
  long long mask_bstride;
  const bf16* o;      // forward output and its gradient: element (b, row, h, c) at ptr[b * o_bstride + row * o_rstride + h * D + c]
  const bf16* dout;
  long long o_bstride, o_rstride;
  const float* lse2;  // [B][H][n_q]
  bf16 *dq, *dk, *dv; // element (b, row, h, c) at ptr[b * bstride + row * rstride + h * D + c]
  long long dq_bstride, dkv_bstride, dq_rstride, dkv_rstride;
  bf16* ds;           // [B][H][n_q][n_k] or null
  int has_bias;
};

struct BwdSmem {
  static constexpr int QDO = 0;                         // 2 x (Q 8 KB + dO 8 KB)
  static constexpr int KV = QDO + 2 * 16384;            // 2 x (K 8 KB + V 8 KB)
  static constexpr int BIAS = KV + 2 * 16384;           // 2 x 32 KB
  static constexpr int P = BIAS + 2 * 32768;            // 32 KB
  static constexpr int DS = P + 32768;                  // 32 KB
  static constexpr int DROW = DS + 32768;               // float[512] D_i, float[512] L2_i
  static constexpr int KP = DROW + 4096;                // [8 warps][64] (keep, penalty) pairs 4 KB
  static constexpr int BARS = KP + 8 * 64 * 8;
  static constexpr int TOTAL = BARS + 512 + 1024;
};

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1) attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                 const __grid_constant__ CUtensorMap tmK,
                                                                 const __grid_constant__ CUtensorMap tmV,
                                                                 const __grid_constant__ CUtensorMap tmDO,
                                                                 const __grid_constant__ CUtensorMap tmBias, const AttnBwdArgs a) {
  pdl_launch_dependents();
  static_assert(D == 32, "head dim 32");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  float* drow = reinterpret_cast<float*>(sm + BwdSmem::DROW);
  float* lrow = drow + 512;
  const uint32_t b0 = smem_u32(sm + BwdSmem::BARS);
  const uint32_t qdo_full = b0, qdo_empty = b0 + 16, kv_full = b0 + 32, kv_empty = b0 + 48;
  const uint32_t bias_full = b0 + 64, bias_empty = b0 + 80;
  const uint32_t sdp_full = b0 + 96, sdp_empty = b0 + 104, pds_full = b0 + 112, pds_empty = b0 + 120;
  const uint32_t dkv_full = b0 + 128, dkv_empty = b0 + 136, dq_full = b0 + 144, dq_empty = b0 + 152;
  const uint32_t drow_ready = b0 + 160;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + BwdSmem::BARS + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(qdo_full + 8 * s, 1);
      mbar_init(qdo_empty + 8 * s, 1);
      mbar_init(kv_full + 8 * s, 1);
      mbar_init(kv_empty + 8 * s, 1);
      mbar_init(bias_full + 8 * s, 1);
      mbar_init(bias_empty + 8 * s, 8);
    }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_empty, 8);
    mbar_init(pds_full, 8);
    mbar_init(pds_empty, 1);
    mbar_init(dkv_full, 1);
    mbar_init(dkv_empty, 8);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 8);
    mbar_init(drow_ready, 8);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  pdl_wait();          // the prologue above touched no global memory; everything below may
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 288, TM_DQ = 320;

  const int steps_per_item = a.n_kb * a.n_qt;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      uint32_t t = 0, jc = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < a.items && ok; item += gridDim.x) {
        const int b = item / a.H, h = item % a.H;
        for (int j = 0; j < a.n_kb && ok; ++j, ++jc) {
          const uint32_t ks = jc & 1;
          if (!mbar_wait(kv_empty + 8 * ks, ((jc >> 1) & 1) ^ 1)) { report(ST_TIMEOUT_MMA, 50); ok = false; break; }
          mbar_expect_tx(kv_full + 8 * ks, 16384);
          tma_load_3d(base + BwdSmem::KV + ks * 16384, &tmK, kv_full + 8 * ks, h * D, j * AT_BK, b);
          tma_load_3d(base + BwdSmem::KV + ks * 16384 + 8192, &tmV, kv_full + 8 * ks, h * D, j * AT_BK, b);
          for (int i = 0; i < a.n_qt && ok; ++i, ++t) {
            const uint32_t s = t & 1;
            if (!mbar_wait(qdo_empty + 8 * s, ((t >> 1) & 1) ^ 1)) { report(ST_TIMEOUT_MMA, 51); ok = false; break; }
            mbar_expect_tx(qdo_full + 8 * s, 16384);
            tma_load_3d(base + BwdSmem::QDO + s * 16384, &tmQ, qdo_full + 8 * s, h * D, i * AT_BQ, b);
            tma_load_3d(base + BwdSmem::QDO + s * 16384 + 8192, &tmDO, qdo_full + 8 * s, h * D, i * AT_BQ, b);
            if (a.has_bias) {
              if (!mbar_wait(bias_empty + 8 * s, ((t >> 1) & 1) ^ 1)) { report(ST_TIMEOUT_EPI, 52); ok = false; break; }
              mbar_expect_tx(bias_full + 8 * s, 32768);
              tma_load_3d(base + BwdSmem::BIAS + s * 32768, &tmBias, bias_full + 8 * s, j * AT_BK, i * AT_BQ, h);
              tma_load_3d(base + BwdSmem::BIAS + s * 32768 + 16384, &tmBias, bias_full + 8 * s, j * AT_BK + 64, i * AT_BQ, h);
            }
          }
        }
      }
      if (!ok) *abort_flag = 1;
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t id_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t id_kv = make_idesc_bf16(128, D, 1, 1);      // (P^T | dS^T) MN-major x (dO | Q) MN-major
      constexpr uint32_t id_q = make_idesc_bf16(128, D, 0, 1);       // dS K-major x K_j MN-major
      uint32_t t = 0, jc = 0, ic = 0;
      bool ok = true;
      // first half of a step: S and dP
      auto issue_a = [&](uint32_t tt, uint32_t jcc, bool first_i) -> bool {
        const uint32_t s = tt & 1, ks = jcc & 1;
        if (!mbar_wait(qdo_full + 8 * s, (tt >> 1) & 1)) { report(ST_TIMEOUT_TMA, 60); return false; }
        if (first_i && !mbar_wait(kv_full + 8 * ks, (jcc >> 1) & 1)) { report(ST_TIMEOUT_TMA, 61); return false; }
        if (!mbar_wait(sdp_empty, (tt & 1) ^ 1)) { report(ST_TIMEOUT_EPI, 62); return false; }
        tc_fence_after();
        const uint32_t qa = base + BwdSmem::QDO + s * 16384, da = qa + 8192;
        const uint32_t ka = base + BwdSmem::KV + ks * 16384, va = ka + 8192;
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem + TM_S, make_desc(qa + k * 32, 16, 512, 4), make_desc(ka + k * 32, 16, 512, 4), id_s, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem + TM_DP, make_desc(da + k * 32, 16, 512, 4), make_desc(va + k * 32, 16, 512, 4), id_s, k > 0 ? 1u : 0u);
        umma_commit(sdp_full);
        return true;
      };
      for (int item = blockIdx.x; item < a.items && ok; item += gridDim.x, ++ic) {
        for (int j = 0; j < a.n_kb && ok; ++j, ++jc) {
          for (int i = 0; i < a.n_qt && ok; ++i, ++t) {
            if (t == 0) ok = issue_a(0, 0, true);
            if (!ok) break;
            if (!mbar_wait(pds_full, t & 1)) { report(ST_TIMEOUT_EPI, 63); ok = false; break; }
            if (i == 0 && !mbar_wait(dkv_empty, (jc & 1) ^ 1)) { report(ST_TIMEOUT_EPI, 64); ok = false; break; }
            if (i == 0 && j == 0 && !mbar_wait(dq_empty, (ic & 1) ^ 1)) { report(ST_TIMEOUT_EPI, 65); ok = false; break; }
            tc_fence_after();
            const uint32_t s = t & 1, ks = jc & 1;
            const uint32_t qa = base + BwdSmem::QDO + s * 16384, da = qa + 8192;
            const uint32_t ka = base + BwdSmem::KV + ks * 16384;
            const uint32_t pa = base + BwdSmem::P, dsa = base + BwdSmem::DS;
#pragma unroll
            for (int k = 0; k < AT_BQ / 16; ++k) {   // contraction over the 128 queries of tile i
              umma_bf16(tmem + TM_DV, make_desc(pa + k * 2048, 16384, 1024, 2), make_desc(da + k * 1024, 16, 512, 4), id_kv, (i > 0 || k > 0) ? 1u : 0u);
              umma_bf16(tmem + TM_DK, make_desc(dsa + k * 2048, 16384, 1024, 2), make_desc(qa + k * 1024, 16, 512, 4), id_kv, (i > 0 || k > 0) ? 1u : 0u);
            }
#pragma unroll
            for (int k = 0; k < AT_BK / 16; ++k)     // contraction over the 128 keys of block j
              umma_bf16(tmem + TM_DQ + i * 32, make_desc(dsa + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024, 2),
                        make_desc(ka + k * 1024, 16, 512, 4), id_q, (j > 0 || k > 0) ? 1u : 0u);
            umma_commit(pds_empty);
            umma_commit(qdo_empty + 8 * s);
            const bool last_i = (i + 1 == a.n_qt);
            if (last_i) {
              umma_commit(dkv_full);
              umma_commit(kv_empty + 8 * ks);
              if (j + 1 == a.n_kb) umma_commit(dq_full);
            }
            // next step's S / dP right away (its operands are usually already in shared memory)
            const bool more = !(last_i && j + 1 == a.n_kb) || (item + (int)gridDim.x < a.items);
            if (more) ok = issue_a(t + 1, last_i ? jc + 1 : jc, last_i);
          }
        }
      }
      if (!ok) *abort_flag = 1;
    }
    __syncwarp();
  } else {
    // ---------------- softmax-gradient warps: thread = (row, 64-key half of the block) ----------------
    const int quad = warp & 3;                      // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    const int HD = a.H * D;
    uint32_t t = 0, jc = 0, ic = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < a.items && ok; item += gridDim.x, ++ic) {
      const int b = item / a.H, h = item % a.H;
      // D_i = rowsum(dO o O) and L2_i for every query row of this (b, h): 8 warps x 32 rows per sweep
      for (int row = half * 128 + r; row < a.n_qt * AT_BQ; row += 256) {
        float dsum = 0.f, l2 = 0.f;
        if (row < a.n_q) {
          const bf16* op = a.o + (long long)b * a.o_bstride + (long long)row * a.o_rstride + h * D;
          const bf16* dp = a.dout + (long long)b * a.o_bstride + (long long)row * a.o_rstride + h * D;
#pragma unroll
          for (int c = 0; c < D; c += 8) {
            const uint4 uo = *reinterpret_cast<const uint4*>(op + c), ud = *reinterpret_cast<const uint4*>(dp + c);
            const bf162 *ho = reinterpret_cast<const bf162*>(&uo), *hd = reinterpret_cast<const bf162*>(&ud);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 fo = __bfloat1622float2(ho[e]), fd = __bfloat1622float2(hd[e]);
              dsum += fo.x * fd.x + fo.y * fd.y;
            }
          }
          l2 = a.lse2[((long long)b * a.H + h) * a.n_q + row];
        }
        drow[row] = dsum;
        lrow[row] = l2;
      }
      // the warps read each other's rows later: make the writes visible to all of them
      __syncwarp();
      if (lane == 0) mbar_arrive(drow_ready);
      if (!mbar_wait(drow_ready, ic & 1)) { if (lane == 0) report(ST_TIMEOUT_EPI, 70); ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const bf16* mrow = a.mask ? a.mask + (long long)b * a.mask_bstride : nullptr;
      for (int j = 0; j < a.n_kb && ok; ++j, ++jc) {
        const int k0 = j * AT_BK;
        for (int i = 0; i < a.n_qt; ++i, ++t) {
          const uint32_t s = t & 1;
          const int qrow = i * AT_BQ + r;
          // key bits first: their global loads overlap the waits below
          const int kbase = k0 + half * 64;
          uint32_t keep_lo, keep_hi, valid_lo, valid_hi;
          key_bits(mrow, kbase, a.n_k, lane, keep_lo, keep_hi, valid_lo, valid_hi);
          const bool plain = (keep_lo & keep_hi) == 0xffffffffu;
          bool w = true;
          if (a.has_bias) w = mbar_wait(bias_full + 8 * s, (t >> 1) & 1);
          if (w) w = mbar_wait(sdp_full, t & 1);
          if (w) w = mbar_wait(pds_empty, (t & 1) ^ 1);        // previous step's gradient MMAs have read P / dS
          if (!w && lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_MMA, 71);
          w = __all_sync(0xffffffffu, w);
          if (!w) { ok = false; break; }
          tc_fence_after();
          const bool row_ok = qrow < a.n_q;
          const float Di = drow[qrow];
          // rows past the end: p = exp2(-inf) = 0.  Fully masked rows (flag -inf): every valid key has the logit MASKED_LOGIT,
          // p = exp2(MASKED_LOGIT * log2e - MASKED_LOGIT * log2e - log2(n_k)) = 1 / n_k exactly.
          const float lse_row = row_ok ? lrow[qrow] : INFINITY;
          const bool row_full = lse_row == -INFINITY;
          const float nL2 = row_full ? -(MASKED_LOGIT * LOG2E) : -lse_row;
          const float nL2b = row_full ? -log2f((float)a.n_k) : 0.f;
          float2* kp = reinterpret_cast<float2*>(sm + BwdSmem::KP) + (warp - 2) * 64;
          if (!plain) write_key_table(kp, lane, keep_lo, keep_hi, valid_lo, valid_hi);
          const uint8_t* brow = sm + BwdSmem::BIAS + s * 32768 + half * 16384 + r * 128;
          uint8_t* prow = sm + BwdSmem::P + half * 16384 + r * 128;
          uint8_t* dsrow = sm + BwdSmem::DS + half * 16384 + r * 128;
          bf16* ds_g = (a.ds && row_ok) ? a.ds + (((long long)b * a.H + h) * a.n_q + qrow) * a.n_k + kbase : nullptr;
          float sv[64], dpv[64];
          tmem_ld_32x32(lane_base + TM_S + half * 64, sv);
          tmem_ld_32x32(lane_base + TM_S + half * 64 + 32, sv + 32);
          tmem_ld_32x32(lane_base + TM_DP + half * 64, dpv);
          tmem_ld_32x32(lane_base + TM_DP + half * 64 + 32, dpv + 32);
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            float v[8];
            if (a.has_bias) {
              const uint4 raw = *reinterpret_cast<const uint4*>(brow + ((u ^ (r & 7)) << 4));
              v[0] = fmaf(sv[u * 8 + 0], a.scale, bf_lo(raw.x));
              v[1] = fmaf(sv[u * 8 + 1], a.scale, bf_hi(raw.x));
              v[2] = fmaf(sv[u * 8 + 2], a.scale, bf_lo(raw.y));
              v[3] = fmaf(sv[u * 8 + 3], a.scale, bf_hi(raw.y));
              v[4] = fmaf(sv[u * 8 + 4], a.scale, bf_lo(raw.z));
              v[5] = fmaf(sv[u * 8 + 5], a.scale, bf_hi(raw.z));
              v[6] = fmaf(sv[u * 8 + 6], a.scale, bf_lo(raw.w));
              v[7] = fmaf(sv[u * 8 + 7], a.scale, bf_hi(raw.w));
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = sv[u * 8 + e] * a.scale;
            }
            float pe[8], g[8];
            if (plain) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                pe[e] = ex2f(fmaf(v[e], LOG2E, nL2));
                g[e] = pe[e] * (dpv[u * 8 + e] - Di);
              }
            } else {
              // masked keys: logit * keep + penalty; keys past the end have penalty -inf, hence p = 0.  The clamp keeps
              // p <= 1 whatever rounding does to a masked key's exponent.
#pragma unroll
              for (int e = 0; e < 8; e += 2) {
                const float4 kk = *reinterpret_cast<const float4*>(kp + u * 8 + e);
                pe[e] = ex2f(fminf(fmaf(fmaf(v[e], kk.x, kk.y), LOG2E, nL2) + nL2b, 0.f));
                pe[e + 1] = ex2f(fminf(fmaf(fmaf(v[e + 1], kk.z, kk.w), LOG2E, nL2) + nL2b, 0.f));
                // a masked logit is a constant: no gradient flows through it (matters in fully masked rows, where p != 0)
                g[e] = pe[e] * (dpv[u * 8 + e] - Di) * kk.x;
                g[e + 1] = pe[e + 1] * (dpv[u * 8 + e + 1] - Di) * kk.z;
              }
            }
            uint4 pp, dd, dg;
            bf162 *hpp = reinterpret_cast<bf162*>(&pp), *hdd = reinterpret_cast<bf162*>(&dd), *hdg = reinterpret_cast<bf162*>(&dg);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              hpp[e] = __floats2bfloat162_rn(pe[2 * e], pe[2 * e + 1]);
              hdg[e] = __floats2bfloat162_rn(g[2 * e], g[2 * e + 1]);
              hdd[e] = __floats2bfloat162_rn(g[2 * e] * a.scale, g[2 * e + 1] * a.scale);
            }
            const uint32_t off = (u ^ (r & 7)) << 4;
            *reinterpret_cast<uint4*>(prow + off) = pp;
            *reinterpret_cast<uint4*>(dsrow + off) = dd;
            if (ds_g) {
              const int kk = kbase + u * 8;
              if (kk + 8 <= a.n_k) *reinterpret_cast<uint4*>(ds_g + u * 8) = dg;
              else {
                const bf16* src = reinterpret_cast<const bf16*>(&dg);
                for (int e = 0; e < 8; ++e)
                  if (kk + e < a.n_k) ds_g[u * 8 + e] = src[e];
              }
            }
          }
          tc_fence_before();
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(sdp_empty);
            if (a.has_bias) mbar_arrive(bias_empty + 8 * s);
            mbar_arrive(pds_full);
          }
        }
        if (!ok) break;
        // dK_j / dV_j complete: thread = key row
        {
          bool w = mbar_wait(dkv_full, jc & 1);
          if (!w && lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_MMA, 72);
          w = __all_sync(0xffffffffu, w);
          if (!w) { ok = false; break; }
          tc_fence_after();
          float gg[D];
          tmem_ld_32x32(lane_base + (half ? TM_DK : TM_DV), gg);     // keys 0-63 group stores dV, the other dK
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(dkv_empty);
          const int krow = k0 + r;
          if (krow < a.n_k) {
            bf16* pg = (half ? a.dk : a.dv) + (long long)b * a.dkv_bstride + (long long)krow * a.dkv_rstride + h * D;
#pragma unroll
            for (int c = 0; c < D; c += 8) {
              uint4 x;
              bf162* hx = reinterpret_cast<bf162*>(&x);
#pragma unroll
              for (int e = 0; e < 4; ++e) hx[e] = __floats2bfloat162_rn(gg[c + 2 * e], gg[c + 2 * e + 1]);
              *reinterpret_cast<uint4*>(pg + c) = x;
            }
          }
        }
      }
      if (!ok) break;
      // dQ_i complete for every query tile of this item
      {
        bool w = mbar_wait(dq_full, ic & 1);
        if (!w && lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_MMA, 73);
        w = __all_sync(0xffffffffu, w);
        if (!w) { ok = false; break; }
        tc_fence_after();
        for (int i = half; i < a.n_qt; i += 2) {
          float gq[D];
          tmem_ld_32x32(lane_base + TM_DQ + i * 32, gq);
          tmem_ld_wait();
          const int qrow = i * AT_BQ + r;
          if (qrow < a.n_q) {
            bf16* pq = a.dq + (long long)b * a.dq_bstride + (long long)qrow * a.dq_rstride + h * D;
#pragma unroll
            for (int c = 0; c < D; c += 8) {
              uint4 x;
              bf162* hx = reinterpret_cast<bf162*>(&x);
#pragma unroll
              for (int e = 0; e < 4; ++e) hx[e] = __floats2bfloat162_rn(gq[c + 2 * e], gq[c + 2 * e + 1]);
              *reinterpret_cast<uint4*>(pq + c) = x;
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_empty);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace ffb

extern "C" {

// Gradients of ffb_attention_fwd.  o / dout: element (b, row, h, c) at ptr[b * o_bstride + row * o_rstride + h * D + c]
// (the forward's out_bstride / out_rstride); dq / dk / dv: element (b, row, h, c) at
// ptr[b * bstride + row * rstride + h * D + c], so the three gradients can be written straight into a packed
// [B][n][3][H*D] tensor; ds: bf16 [B][H][n_q][n_k] (unscaled dS, for the bias gradient) or null.
int ffb_attention_bwd_strided(const void* q, const void* k, const void* v, long long q_bstride, long long q_rstride,
                              long long kv_bstride, long long kv_rstride, const void* bias, const void* mask, long long mask_bstride,
                              const void* o, const void* dout, long long o_bstride, long long o_rstride, const float* lse2, void* dq,
                              void* dk, void* dv, long long dq_bstride,
                              long long dq_rstride, long long dkv_bstride, long long dkv_rstride, void* ds, int B, int H, int n_q,
                              int n_k, int D, float scale, void* stream) {
  using namespace ffb;
  if (D != 32) return -2;
  if (n_q > 512) return -3;
  if ((q_rstride % 8) || (kv_rstride % 8) || (q_bstride % 8) || (kv_bstride % 8) || (n_k % 8)) return -4;
  if ((dq_rstride % 8) || (dkv_rstride % 8) || (dq_bstride % 8) || (dkv_bstride % 8) || (o_bstride % 8) || (o_rstride % 8)) return -5;
  AttnBwdArgs a;
  a.B = B; a.H = H; a.n_q = n_q; a.n_k = n_k;
  a.n_qt = (n_q + AT_BQ - 1) / AT_BQ;
  a.n_kb = (n_k + AT_BK - 1) / AT_BK;
  a.items = B * H;
  a.scale = scale;
  a.scale_log2e = scale * LOG2E;
  a.mask = (const bf16*)mask;
  a.mask_bstride = mask_bstride;
  a.o = (const bf16*)o;
  a.dout = (const bf16*)dout;
  a.o_bstride = o_bstride;
  a.o_rstride = o_rstride;
  a.lse2 = lse2;
  const long long HD = (long long)H * D;
  a.dq = (bf16*)dq;
  a.dk = (bf16*)dk;
  a.dv = (bf16*)dv;
  a.dq_bstride = dq_bstride;
  a.dkv_bstride = dkv_bstride;
  a.dq_rstride = dq_rstride;
  a.dkv_rstride = dkv_rstride;
  a.ds = (bf16*)ds;
  a.has_bias = bias ? 1 : 0;
  CUtensorMap tq, tk, tv, tdo, tb;
  { int rc = make_tmap3(&tq, q, HD, n_q, B, q_rstride, q_bstride, D, AT_BQ, 64); if (rc) return -100000 - rc; }
  if (make_tmap3(&tk, k, HD, n_k, B, kv_rstride, kv_bstride, D, AT_BK, 64)) return -11;
  if (make_tmap3(&tv, v, HD, n_k, B, kv_rstride, kv_bstride, D, AT_BK, 64)) return -12;
  { int rc = make_tmap3(&tdo, dout, HD, n_q, B, o_rstride, o_bstride, D, AT_BQ, 64); if (rc) return -130000 - rc; }
  if (bias) {
    if (make_tmap3(&tb, bias, n_k, n_q, H, n_k, (long long)n_q * n_k, 64, AT_BQ, 128)) return -14;
  } else {
    tb = tq;
  }
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::TOTAL) != cudaSuccess) return -15;
    attr = true;
  }
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
  }
  const int grid = a.items < sm_count ? a.items : sm_count;
  launch_k(attn_bwd_kernel<32>, grid, AT_THREADS, BwdSmem::TOTAL, reinterpret_cast<cudaStream_t>(stream), tq, tk, tv, tdo, tb, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -16;
}


// Same, with the gradients in three [B][n_max][H*D] slabs (dq, dk, dv; n_max = max(n_q, n_k)) of one buffer.
int ffb_attention_bwd(const void* q, const void* k, const void* v, long long q_bstride, long long q_rstride, long long kv_bstride,
                      long long kv_rstride, const void* bias, const void* mask, long long mask_bstride, const void* o, const void* dout,
                      const float* lse2, void* dqkv, void* ds, int B, int H, int n_q, int n_k, int D, float scale, void* stream) {
  const long long HD = (long long)H * D;
  const long long n_max = n_q > n_k ? n_q : n_k;
  ffb::bf16* g = (ffb::bf16*)dqkv;
  return ffb_attention_bwd_strided(q, k, v, q_bstride, q_rstride, kv_bstride, kv_rstride, bias, mask, mask_bstride, o, dout,
                                   (long long)n_q * HD, HD, lse2, g,
                                   g + (long long)B * n_max * HD, g + 2 * (long long)B * n_max * HD, n_max * HD, HD, n_max * HD, HD, ds,
                                   B, H, n_q, n_k, D, scale, stream);
}

}  // extern "C"
