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
// Per CTA (192 threads):
//   warp 0     TMA producer: Q tile, K/V key blocks (64B-swizzled, straight out of
//              the fused QKV projection output, no head transposes), bias tiles
//   warp 1     MMA issuer: S = Q K^T (tcgen05, 128 x 128 x 32) into one of two TMEM
//              stages; PV = P V (128 x 32 x 128) into one of two TMEM stages
//   warps 2-5  softmax: thread = query row.  tcgen05.ld of S, scale + bias + mask,
//              online max / sum, P written as bf16 into the 128B-swizzled shared
//              tile that the PV MMA reads; the running output row lives in
//              registers and is rescaled there (no TMEM read-modify-write)
// S MMA of block j+1 and the PV MMA of block j overlap the softmax of block j.
// Masked keys get the logit -1e9 (replaced, not added), as in the reference's
// softmax kernels (softmax_cuda_kernel.cu:338-423,618-706); keys beyond the
// sequence end get -inf.  The kernel also stores log2-domain row statistics
// L2 = m2 + log2(l) for the backward kernel.
//
// Replaces logits matmul + fused_softmax + weights*v of the reference
// (fastfold/model/fastnn/ops.py:304-319) and its unused Triton forward-only
// attention core (kernel/triton/attention_core.py:12-121).
#include "common.cuh"

namespace ffb {

constexpr int AT_BQ = 128;      // queries per tile
constexpr int AT_BK = 128;      // keys per block
constexpr int AT_THREADS = 192;
constexpr int AT_KV_STAGES = 3;
constexpr float LOG2E = 1.4426950408889634f;

struct AttnArgs {
  int B, H, n_q, n_k;            // batch rows, heads, query / key lengths
  int n_qt, n_kb;                // query tiles, key blocks
  int items;                     // H * n_qt * B work items
  int bias_resident;             // 1: n_kb <= 2, bias tiles stay in shared memory across batch rows
  float scale_log2e;             // scale * log2(e)
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

struct AttnSmem {
  // offsets (bytes) from the 1024-aligned base
  static constexpr int Q = 0;                                  // 2 x [128][64 B]            16 KB
  static constexpr int KV = Q + 2 * 8192;                      // STAGES x (K 8 KB + V 8 KB) 48 KB
  static constexpr int BIAS = KV + AT_KV_STAGES * 16384;       // 2 x [2 boxes][128][128 B]  64 KB
  static constexpr int P = BIAS + 2 * 32768;                   // 2 x [2 chunks][128][128 B] 64 KB
  static constexpr int BARS = P + 2 * 32768;
  static constexpr int TOTAL = BARS + 512 + 1024;
};

template <int D>   // head dim: 32 (64-byte rows)
__global__ void __launch_bounds__(AT_THREADS, 1) attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                 const __grid_constant__ CUtensorMap tmK,
                                                                 const __grid_constant__ CUtensorMap tmV,
                                                                 const __grid_constant__ CUtensorMap tmBias, const AttnArgs a) {
  static_assert(D == 32, "head dim 32");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + AttnSmem::BARS);
  // barrier map
  const uint32_t b0 = smem_u32(bars);
  const uint32_t q_full = b0, q_empty = b0 + 16;                       // 2 + 2
  const uint32_t kv_full = b0 + 32, kv_empty = kv_full + 8 * AT_KV_STAGES;
  const uint32_t bias_full = kv_empty + 8 * AT_KV_STAGES, bias_empty = bias_full + 16;
  const uint32_t s_full = bias_empty + 16, s_empty = s_full + 16;
  const uint32_t p_full = s_empty + 16, o_full = p_full + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + AttnSmem::BARS + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(q_full + 8 * s, 1);
      mbar_init(q_empty + 8 * s, 1);
      mbar_init(bias_full + 8 * s, 1);
      mbar_init(bias_empty + 8 * s, 4);
      mbar_init(s_full + 8 * s, 1);
      mbar_init(s_empty + 8 * s, 4);
      mbar_init(p_full + 8 * s, 4);
      mbar_init(o_full + 8 * s, 1);
    }
    for (int s = 0; s < AT_KV_STAGES; ++s) {
      mbar_init(kv_full + 8 * s, 1);
      mbar_init(kv_empty + 8 * s, 1);
    }
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
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t TM_S = 0, TM_O = 256;

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
      uint32_t jt = 0, qi = 0;
      bool ok = true;
      auto issue_s = [&](uint32_t jglob, uint32_t qs) -> bool {
        const uint32_t s = jglob % AT_KV_STAGES, sb = jglob & 1;
        if (!mbar_wait(kv_full + 8 * s, (jglob / AT_KV_STAGES) & 1)) { report(ST_TIMEOUT_TMA, 20); return false; }
        if (!mbar_wait(s_empty + 8 * sb, ((jglob >> 1) & 1) ^ 1)) { report(ST_TIMEOUT_EPI, 21); return false; }
        tc_fence_after();
        const uint32_t qa = base + AttnSmem::Q + qs * 8192;
        const uint32_t ka = base + AttnSmem::KV + s * 16384;
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem + TM_S + sb * 128, make_desc(qa + k * 32, 16, 512, 4), make_desc(ka + k * 32, 16, 512, 4), idesc_s, k > 0 ? 1u : 0u);
        umma_commit(s_full + 8 * sb);
        return true;
      };
      for (int item = it_begin; item < it_end && ok; ++item, ++qi) {
        const uint32_t qs = qi & 1;
        if (!mbar_wait(q_full + 8 * qs, (qi >> 1) & 1)) { report(ST_TIMEOUT_TMA, 22); *abort_flag = 1; break; }
        ok = issue_s(jt, qs);
        for (int j = 0; j < a.n_kb && ok; ++j, ++jt) {
          if (j + 1 < a.n_kb) ok = issue_s(jt + 1, qs);
          if (!ok) break;
          if (j + 1 == a.n_kb) umma_commit(q_empty + 8 * qs);    // all S MMAs of this item issued: Q slot drains with them
          const uint32_t pb = jt & 1;
          if (!mbar_wait(p_full + 8 * pb, (jt >> 1) & 1)) { report(ST_TIMEOUT_EPI, 23); ok = false; break; }
          tc_fence_after();
          const uint32_t s = jt % AT_KV_STAGES;
          const uint32_t pa = base + AttnSmem::P + pb * 32768;
          const uint32_t va = base + AttnSmem::KV + s * 16384 + 8192;
#pragma unroll
          for (int k = 0; k < AT_BK / 16; ++k)
            umma_bf16(tmem + TM_O + pb * 32, make_desc(pa + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024, 2),
                      make_desc(va + k * 1024, 16, 512, 4), idesc_o, k > 0 ? 1u : 0u);
          umma_commit(o_full + 8 * pb);
          umma_commit(kv_empty + 8 * s);
        }
      }
      if (!ok) *abort_flag = 1;
    }
    __syncwarp();
  } else {
    // ---------------- softmax / output (warps 2..5): thread = query row ----------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                 // row within the query tile
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    uint32_t jt = 0, bt = 0;
    int prev_group = -1;
    bool ok = true;
    for (int item = it_begin; item < it_end && ok; ++item) {
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
      float m2 = -INFINITY, l = 0.f, alpha_prev = 1.f;
      const bf16* mrow = a.mask ? a.mask + (long long)b * a.mask_bstride : nullptr;
      for (int j = 0; j < a.n_kb; ++j, ++jt) {
        const int k0 = j * AT_BK;
        const uint32_t sb = jt & 1;
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
        // ---- logits of this row: 128 keys in registers ----
        float s[AT_BK];
#pragma unroll
        for (int c = 0; c < AT_BK / 32; ++c) tmem_ld_32x32(lane_base + TM_S + sb * 128 + c * 32, s + c * 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty + 8 * sb);          // S stage may be overwritten by the next-but-one block
        const uint8_t* btile = sm + AttnSmem::BIAS + bs * 32768;
        float mx = m2;
#pragma unroll
        for (int u = 0; u < AT_BK / 8; ++u) {
          float bv[8];
          if (a.has_bias) {
            const uint4 raw = *reinterpret_cast<const uint4*>(btile + (u >> 3) * 16384 + r * 128 + (((u & 7) ^ (r & 7)) << 4));
            const bf162* hp = reinterpret_cast<const bf162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(hp[e]);
              bv[2 * e] = f.x;
              bv[2 * e + 1] = f.y;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) bv[e] = 0.f;
          }
          float mk[8];
          if (mrow) {
            const int kk = k0 + u * 8;
            if (kk + 8 <= a.n_k) {
              const uint4 raw = *reinterpret_cast<const uint4*>(mrow + kk);
              const bf162* hp = reinterpret_cast<const bf162*>(&raw);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(hp[e]);
                mk[2 * e] = f.x;
                mk[2 * e + 1] = f.y;
              }
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) mk[e] = (kk + e < a.n_k) ? __bfloat162float(mrow[kk + e]) : 0.f;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) mk[e] = 1.f;
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int c = u * 8 + e;
            float v = s[c] * a.scale_log2e + bv[e] * LOG2E;
            if (mk[e] == 0.f) v = -1e9f * LOG2E;
            if (k0 + c >= a.n_k) v = -INFINITY;
            s[c] = v;
            mx = fmaxf(mx, v);
          }
        }
        if (a.has_bias && (!a.bias_resident || last_of_group)) {
          __syncwarp();
          if (lane == 0) mbar_arrive(bias_empty + 8 * bs);
        }
        const float alpha = ex2f(m2 - mx);                      // m2 = -inf on the first block -> 0
        m2 = mx;
        float rowsum = 0.f;
        // ---- P = exp2(s - m) as bf16 into the swizzled A-operand tile ----
        uint8_t* ptile = sm + AttnSmem::P + sb * 32768;
#pragma unroll
        for (int u = 0; u < AT_BK / 8; ++u) {
          uint4 pk;
          bf162* hp = reinterpret_cast<bf162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float p0 = ex2f(s[u * 8 + 2 * e] - mx), p1 = ex2f(s[u * 8 + 2 * e + 1] - mx);
            hp[e] = __floats2bfloat162_rn(p0, p1);
            const float2 back = __bfloat1622float2(hp[e]);     // sum what the MMA will actually see
            rowsum += back.x + back.y;
          }
          *reinterpret_cast<uint4*>(ptile + (u >> 3) * 16384 + r * 128 + (((u & 7) ^ (r & 7)) << 4)) = pk;
        }
        l = l * alpha + rowsum;
        // previous block's PV (if any) joins the register accumulator before this block's scaling is applied
        if (j > 0) {
          const uint32_t ob = (jt - 1) & 1;
          bool w = mbar_wait(o_full + 8 * ob, ((jt - 1) >> 1) & 1);
          if (!w && lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_MMA, 32);
          w = __all_sync(0xffffffffu, w);
          if (!w) { ok = false; break; }
          tc_fence_after();
          float pv[D];
          tmem_ld_32x32(lane_base + TM_O + ob * 32, pv);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < D; ++c) o[c] = o[c] * alpha_prev + pv[c];
        }
        alpha_prev = alpha;
        fence_proxy_async_smem();                              // generic-proxy P stores -> visible to the MMA (async proxy)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + 8 * sb);
      }
      if (!ok) break;
      // last block's PV
      {
        const uint32_t ob = (jt - 1) & 1;
        bool w = mbar_wait(o_full + 8 * ob, ((jt - 1) >> 1) & 1);
        if (!w && lane == 0 && *abort_flag == 0) report(ST_TIMEOUT_MMA, 33);
        w = __all_sync(0xffffffffu, w);
        if (!w) { ok = false; break; }
        tc_fence_after();
        float pv[D];
        tmem_ld_32x32(lane_base + TM_O + ob * 32, pv);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < D; ++c) o[c] = o[c] * alpha_prev + pv[c];
      }
      const int qrow = q0 + r;
      if (qrow < a.n_q) {
        const float inv = 1.f / l;
        bf16* dst = a.out + (long long)b * a.out_bstride + (long long)qrow * a.out_rstride + h * D;
#pragma unroll
        for (int c = 0; c < D; c += 8) {
          uint4 pk;
          bf162* hp = reinterpret_cast<bf162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) hp[e] = __floats2bfloat162_rn(o[c + 2 * e] * inv, o[c + 2 * e + 1] * inv);
          *reinterpret_cast<uint4*>(dst + c) = pk;
        }
        if (a.lse2) a.lse2[((long long)b * a.H + h) * a.n_q + qrow] = m2 + log2f(l);
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
typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn2 get_encode2() {
  static EncodeTiledFn2 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess || !p) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn2>(p);
  }
  return fn;
}

// bf16 tensor [d2][d1][d0] (d0 contiguous) with element strides s1, s2; box b0 x b1 x 1.
int make_tmap3(CUtensorMap* map, const void* ptr, long long d0, long long d1, long long d2, long long s1, long long s2, int b0,
               int b1, int swizzle_bytes) {
  EncodeTiledFn2 enc = get_encode2();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)(d2 > 0 ? d2 : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)s1 * 2, (cuuint64_t)(d2 > 1 ? s2 : d1 * s1) * 2};
  cuuint32_t box[3] = {(cuuint32_t)b0, (cuuint32_t)b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                 : (swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE));
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
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
  a.scale_log2e = scale * LOG2E;
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
  attn_fwd_kernel<32><<<grid, AT_THREADS, AttnSmem::TOTAL, reinterpret_cast<cudaStream_t>(stream)>>>(tq, tk, tv, tb, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -15;
}

}  // extern "C"
