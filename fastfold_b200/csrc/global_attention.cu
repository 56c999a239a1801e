// Global column attention of the extra-MSA stack, core part in one kernel.
//
// Per MSA column r there is ONE query per head (the masked mean over the sequences, projected), and keys / values are
// shared by all heads (fastfold/model/fastnn/ops.py:1175-1236, openfold-style GlobalAttention).  With S_e sequences of
// c = 8 channels per head this is a bandwidth problem: per column  logits[h][s] = q[h] . k[s],  softmax over s (masked keys
// get the logit -1e9, replaced), o[h] = sum_s w[h][s] v[s], and then the gate  out[s][h*c + i] = sigmoid(g[s][h*c+i] + b) * o[h][i].
// The kernel makes one pass over (k | v) with an online softmax per (head, sequence lane), folds the lanes through
// shared memory, and streams the gate tensor once: no logits, weights or broadcast copies of o reach memory.
//
// One CTA per column (or several, each gating a slice of the sequences, when there are few columns), 256 threads;
// thread t works on head t % H and sequence lane t / H (H divides 256).
#include <cooperative_groups.h>

#include "common.cuh"

namespace ffb {

constexpr int GA_THREADS = 256;
constexpr float GA_MASKED = -1e9f;

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int C>
__global__ void __launch_bounds__(GA_THREADS) global_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv,
                                                                      const bf16* __restrict__ mask, const bf16* __restrict__ gate,
                                                                      const bf16* __restrict__ gate_bias, bf16* __restrict__ out,
                                                                      int S, int H) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int lanes = GA_THREADS / H;
  float* s_m = sm;                       // [lanes][H]
  float* s_l = s_m + GA_THREADS;         // [lanes][H]
  float* s_acc = s_l + GA_THREADS;       // [lanes][H][C]
  float* s_o = s_acc + GA_THREADS * C;   // [H][C]
  float* s_b = s_o + H * C;              // [H][C] gate bias
  const long long r = blockIdx.x;
  const int part = blockIdx.y, parts = gridDim.y;     // every part recomputes o (kv comes from L2) and gates its share of the rows
  const int h = threadIdx.x % H, sl = threadIdx.x / H;
  const int HC = H * C;

  float qv[C];
#pragma unroll
  for (int i = 0; i < C; ++i) qv[i] = __bfloat162float(q[(r * H + h) * C + i]);
  for (int i = threadIdx.x; i < HC; i += GA_THREADS) s_b[i] = __bfloat162float(gate_bias[i]);

  float m = -INFINITY, l = 0.f, acc[C];
#pragma unroll
  for (int i = 0; i < C; ++i) acc[i] = 0.f;
  const bf16* kvr = kv + r * (long long)S * 2 * C;
  const bf16* mr = mask + r * (long long)S;
  constexpr int U = 4;      // keys per iteration: their loads are in flight together, and one rescale serves all four
  for (int s0 = sl; s0 < S; s0 += U * lanes) {
    // the H threads of one sequence lane read the same 4 * C bytes: one transaction, broadcast
    bf16 kk[U][C], vv[U][C];
    float mk[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = s0 + u * lanes;
      const long long off = (long long)(s < S ? s : s0) * 2 * C;
      if constexpr (C % 8 == 0) {
#pragma unroll
        for (int i = 0; i < C / 8; ++i) {
          reinterpret_cast<uint4*>(kk[u])[i] = reinterpret_cast<const uint4*>(kvr + off)[i];
          reinterpret_cast<uint4*>(vv[u])[i] = reinterpret_cast<const uint4*>(kvr + off + C)[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < C; ++i) {
          kk[u][i] = kvr[off + i];
          vv[u][i] = kvr[off + C + i];
        }
      }
      mk[u] = __bfloat162float(mr[s < S ? s : s0]);
    }
    float lg[U];
    float mn = m;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < C; ++i) d = fmaf(qv[i], __bfloat162float(kk[u][i]), d);
      if (mk[u] == 0.f) d = GA_MASKED;
      if (s0 + u * lanes >= S) d = -INFINITY;          // past the end: weight 0
      lg[u] = d;
      mn = fmaxf(mn, d);
    }
    const float a = __expf(m - mn);                    // m = -inf on the first iteration: a = 0
    l *= a;
#pragma unroll
    for (int i = 0; i < C; ++i) acc[i] *= a;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const float p = __expf(lg[u] - mn);
      l += p;
#pragma unroll
      for (int i = 0; i < C; ++i) acc[i] = fmaf(p, __bfloat162float(vv[u][i]), acc[i]);
    }
    m = mn;
  }
  s_m[sl * H + h] = m;
  s_l[sl * H + h] = l;
#pragma unroll
  for (int i = 0; i < C; ++i) s_acc[(sl * H + h) * C + i] = acc[i];
  __syncthreads();
  // fold the sequence lanes: thread (h, i) for i < C
  if (threadIdx.x < HC) {
    const int hh = threadIdx.x / C, i = threadIdx.x - hh * C;
    float mx = -INFINITY;
    for (int j = 0; j < lanes; ++j) mx = fmaxf(mx, s_m[j * H + hh]);
    float lt = 0.f, at = 0.f;
    for (int j = 0; j < lanes; ++j) {
      const float mj = s_m[j * H + hh];
      const float w = (mj == -INFINITY) ? 0.f : __expf(mj - mx);        // lanes that saw no key (S < lanes)
      lt = fmaf(s_l[j * H + hh], w, lt);
      at = fmaf(s_acc[(j * H + hh) * C + i], w, at);
    }
    s_o[threadIdx.x] = lt > 0.f ? at / lt : 0.f;
  }
  __syncthreads();
  // gate: out[s][j] = sigmoid(gate[s][j] + b[j]) * o[j]
  const bf16* gr = gate + r * (long long)S * HC;
  bf16* orow = out + r * (long long)S * HC;
  const int s_per = (S + parts - 1) / parts;
  const int s_lo = part * s_per, s_hi = min(S, s_lo + s_per);
  if (HC % 8 == 0) {
    const long long v_lo = (long long)s_lo * HC / 8, v_hi = (long long)s_hi * HC / 8;
    constexpr int V = 4;                                // 16-byte loads in flight per thread
    // H * C is a power of two <= 256, so 8 * GA_THREADS is a multiple of it and a slice starts on a row boundary: the eight
    // channels a thread handles never change, and their o and bias live in registers
    const int j0 = (int)(((v_lo + threadIdx.x) * 8) % HC);
    float o8[8], b8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      o8[e] = 0.5f * s_o[j0 + e];
      b8[e] = 0.5f * s_b[j0 + e];
    }
    for (long long v0 = v_lo + threadIdx.x; v0 < v_hi; v0 += (long long)V * GA_THREADS) {
      uint4 gv[V];
#pragma unroll
      for (int u = 0; u < V; ++u) {
        const long long v = v0 + (long long)u * GA_THREADS;
        gv[u] = v < v_hi ? reinterpret_cast<const uint4*>(gr)[v] : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < V; ++u) {
        const long long v = v0 + (long long)u * GA_THREADS;
        if (v >= v_hi) break;
        const bf16* ge = reinterpret_cast<const bf16*>(&gv[u]);
        uint4 ov;
        bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          // o * sigmoid(x) = (o / 2) * tanh(x / 2) + o / 2: one special-function instruction per element
          const float t = tanh_approx(fmaf(0.5f, __bfloat162float(ge[e]), b8[e]));
          oe[e] = __float2bfloat16(fmaf(o8[e], t, o8[e]));
        }
        reinterpret_cast<uint4*>(orow)[v] = ov;
      }
    }
  } else {
    for (long long v = (long long)s_lo * HC + threadIdx.x; v < (long long)s_hi * HC; v += GA_THREADS) {
      const int j = (int)(v % HC);
      const float x = __bfloat162float(gr[v]) + s_b[j];
      orow[v] = __float2bfloat16(s_o[j] / (1.f + __expf(-x)));
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Cluster version for the model's shape (H = 8 heads of C = 8 channels).  The CTAs of a thread-block cluster share one
// column: each runs the online softmax over ITS slice of the sequences with two threads per key (four heads each; the
// version above converts k and v once per head), the partial (max, sum, weighted values) of
// every CTA are merged through distributed shared memory, and each CTA gates its slice.  No part of the column is read
// twice and nothing but the result reaches global memory.
constexpr int GC_H = 8, GC_C = 8, GC_HC = GC_H * GC_C;
constexpr int GC_REC = 2 + GC_C;          // per head: max, sum, C weighted values

__global__ void __launch_bounds__(GA_THREADS, 2) global_attention_cluster_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv,
                                                                                 const bf16* __restrict__ mask, const bf16* __restrict__ gate,
                                                                                 const bf16* __restrict__ gate_bias, bf16* __restrict__ out,
                                                                                 int S) {
  pdl_launch_dependents();
  pdl_wait();
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float s_q[GC_HC];
  __shared__ float s_warp[GA_THREADS / 32][GC_H][GC_REC];
  __shared__ float s_part[GC_H][GC_REC];            // this CTA's partial, read by the whole cluster
  __shared__ float s_o[GC_HC], s_b[GC_HC];
  const long long r = blockIdx.x;
  const int part = blockIdx.y, parts = gridDim.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < GC_HC) {
    s_q[threadIdx.x] = __bfloat162float(q[r * GC_HC + threadIdx.x]);
    s_b[threadIdx.x] = __bfloat162float(gate_bias[threadIdx.x]);
  }
  __syncthreads();
  const int s_per = (S + parts - 1) / parts;
  const int s_lo = part * s_per, s_hi = min(S, s_lo + s_per);
  // two threads per key, four heads each: k and v are converted twice instead of eight times, and the running state
  // (4 x (max, sum, 8 values)) fits the registers of two CTAs per SM
  constexpr int HG = GC_H / 2;
  const int hg = threadIdx.x & 1;
  float m[HG], l[HG], acc[HG][GC_C];
#pragma unroll
  for (int h = 0; h < HG; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < GC_C; ++i) acc[h][i] = 0.f;
  }
  const bf16* kvr = kv + r * (long long)S * 2 * GC_C;
  const bf16* mr = mask + r * (long long)S;
  for (int s = s_lo + (threadIdx.x >> 1); s < s_hi; s += GA_THREADS / 2) {
    const uint4 kraw = *reinterpret_cast<const uint4*>(kvr + (long long)s * 2 * GC_C);
    const uint4 vraw = *reinterpret_cast<const uint4*>(kvr + (long long)s * 2 * GC_C + GC_C);
    const bool masked = __bfloat162float(mr[s]) == 0.f;
    float kf[GC_C], vf[GC_C];
    {
      const bf162* kh = reinterpret_cast<const bf162*>(&kraw);
      const bf162* vh = reinterpret_cast<const bf162*>(&vraw);
#pragma unroll
      for (int i = 0; i < GC_C / 2; ++i) {
        const float2 a = __bfloat1622float2(kh[i]), b = __bfloat1622float2(vh[i]);
        kf[2 * i] = a.x; kf[2 * i + 1] = a.y;
        vf[2 * i] = b.x; vf[2 * i + 1] = b.y;
      }
    }
#pragma unroll
    for (int h = 0; h < HG; ++h) {
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < GC_C; ++i) d = fmaf(s_q[(hg * HG + h) * GC_C + i], kf[i], d);
      if (masked) d = GA_MASKED;
      if (d > m[h]) {                         // the running maximum settles after a few keys: the rescale is rare
        const float a = __expf(m[h] - d);     // m = -inf on the first key: a = 0
        l[h] *= a;
#pragma unroll
        for (int i = 0; i < GC_C; ++i) acc[h][i] *= a;
        m[h] = d;
      }
      const float pw = __expf(d - m[h]);
      l[h] += pw;
#pragma unroll
      for (int i = 0; i < GC_C; ++i) acc[h][i] = fmaf(pw, vf[i], acc[h][i]);
    }
  }
  // warp level, over the 16 lanes of each head group (even / odd lanes): common maximum, rescaled sums
#pragma unroll
  for (int h = 0; h < HG; ++h) {
    float wm = m[h];
#pragma unroll
    for (int o = 16; o > 1; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
    const float sc = (m[h] == -INFINITY) ? 0.f : __expf(m[h] - wm);
    float v = l[h] * sc;
#pragma unroll
    for (int o = 16; o > 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane < 2) {
      s_warp[warp][hg * HG + h][0] = wm;
      s_warp[warp][hg * HG + h][1] = v;
    }
#pragma unroll
    for (int i = 0; i < GC_C; ++i) {
      float a = acc[h][i] * sc;
#pragma unroll
      for (int o = 16; o > 1; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      if (lane < 2) s_warp[warp][hg * HG + h][2 + i] = a;
    }
  }
  __syncthreads();
  // CTA level: thread (h, i) folds the eight warps
  if (threadIdx.x < GC_HC) {
    const int h = threadIdx.x / GC_C, i = threadIdx.x - h * GC_C;
    float mx = -INFINITY;
    for (int w = 0; w < GA_THREADS / 32; ++w) mx = fmaxf(mx, s_warp[w][h][0]);
    float lt = 0.f, at = 0.f;
    for (int w = 0; w < GA_THREADS / 32; ++w) {
      const float mw = s_warp[w][h][0];
      const float sc = (mw == -INFINITY) ? 0.f : __expf(mw - mx);
      lt = fmaf(s_warp[w][h][1], sc, lt);
      at = fmaf(s_warp[w][h][2 + i], sc, at);
    }
    if (i == 0) {
      s_part[h][0] = mx;
      s_part[h][1] = lt;
    }
    s_part[h][2 + i] = at;
  }
  cluster.sync();                              // every CTA's partial is in its shared memory
  if (threadIdx.x < GC_HC) {
    const int h = threadIdx.x / GC_C, i = threadIdx.x - h * GC_C;
    float mx = -INFINITY;
    for (int p = 0; p < parts; ++p) mx = fmaxf(mx, cluster.map_shared_rank(&s_part[0][0], p)[h * GC_REC]);
    float lt = 0.f, at = 0.f;
    for (int p = 0; p < parts; ++p) {
      const float* rp = cluster.map_shared_rank(&s_part[0][0], p) + h * GC_REC;
      const float mp = rp[0];
      const float sc = (mp == -INFINITY) ? 0.f : __expf(mp - mx);
      lt = fmaf(rp[1], sc, lt);
      at = fmaf(rp[2 + i], sc, at);
    }
    s_o[threadIdx.x] = lt > 0.f ? at / lt : 0.f;
  }
  cluster.sync();                              // nobody leaves (or goes on) while its partial may still be read
  // gate this CTA's slice
  const bf16* gr = gate + r * (long long)S * GC_HC;
  bf16* orow = out + r * (long long)S * GC_HC;
  const long long v_lo = (long long)s_lo * GC_HC / 8, v_hi = (long long)s_hi * GC_HC / 8;
  const int j0 = (int)(((v_lo + threadIdx.x) * 8) % GC_HC);
  float o8[8], b8[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    o8[e] = 0.5f * s_o[j0 + e];
    b8[e] = 0.5f * s_b[j0 + e];
  }
  constexpr int V = 8;                                  // 128 bytes in flight per thread
  for (long long v0 = v_lo + threadIdx.x; v0 < v_hi; v0 += (long long)V * GA_THREADS) {
    uint4 gv[V];
#pragma unroll
    for (int u = 0; u < V; ++u) {
      const long long v = v0 + (long long)u * GA_THREADS;
      gv[u] = v < v_hi ? reinterpret_cast<const uint4*>(gr)[v] : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < V; ++u) {
      const long long v = v0 + (long long)u * GA_THREADS;
      if (v >= v_hi) break;
      const bf162* ge = reinterpret_cast<const bf162*>(&gv[u]);
      uint4 ov;
      bf162* oe = reinterpret_cast<bf162*>(&ov);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 g2 = __bfloat1622float2(ge[e]);
        const float t0 = tanh_approx(fmaf(0.5f, g2.x, b8[2 * e])), t1 = tanh_approx(fmaf(0.5f, g2.y, b8[2 * e + 1]));
        oe[e] = __floats2bfloat162_rn(fmaf(o8[2 * e], t0, o8[2 * e]), fmaf(o8[2 * e + 1], t1, o8[2 * e + 1]));
      }
      reinterpret_cast<uint4*>(orow)[v] = ov;
    }
  }
}

// ---------------------------------------------------------------------------
// Backward of the kernel above (training of the extra-MSA stack).  Per column r, with g = sigmoid(gate + b),
// w = softmax over s of q[h].k[s] (masked keys at -1e9) and o[h] = sum_s w[h][s] v[s]:
//     d_o[h][i]    = sum_s dout[s][h*c+i] * g[s][h*c+i]
//     d_gate[s][j] = dout[s][j] * o[j] * g (1 - g)            (gradient w.r.t. the pre-activation; the bias gradient is its column sum)
//     d_w[h][s]    = d_o[h] . v[s],   d_logit[h][s] = w[h][s] (d_w[h][s] - d_o[h] . o[h])        (0 for masked keys: their logit is a constant)
//     d_q[h]       = sum_s d_logit[h][s] k[s],   d_k[s] = sum_h d_logit[h][s] q[h],   d_v[s] = sum_h w[h][s] d_o[h]
// Pass A streams (k | v) for the softmax statistics and o (as the forward does) and gate / dout for d_o; pass B streams
// them again and writes d_kv and d_gate.  One CTA per column; thread t works on head t % H and sequence lane t / H in the
// attention parts and on channel t % (H c) in the gating parts.  The PyTorch composite this replaces materialises the
// [R, H, S] logits and weights and a broadcast copy of o (fastfold/model/fastnn/ops.py:1175-1236).
// ---------------------------------------------------------------------------
template <int C>
__global__ void __launch_bounds__(GA_THREADS) global_attention_bwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv,
                                                                          const bf16* __restrict__ mask, const bf16* __restrict__ gate,
                                                                          const bf16* __restrict__ gate_bias, const bf16* __restrict__ dout,
                                                                          float* __restrict__ dq, bf16* __restrict__ dkv,
                                                                          bf16* __restrict__ dgate, int S, int H) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int lanes = GA_THREADS / H;
  const int HC = H * C;
  float* s_m = sm;                        // [lanes][H]
  float* s_l = s_m + GA_THREADS;          // [lanes][H]
  float* s_acc = s_l + GA_THREADS;        // [lanes][H][C]   (also the d_q fold buffer)
  float* s_o = s_acc + GA_THREADS * C;    // [H][C]
  float* s_do = s_o + HC;                 // [H][C]
  float* s_b = s_do + HC;                 // [H][C]
  float* s_mt = s_b + HC;                 // [H] final max
  float* s_il = s_mt + H;                 // [H] 1 / final sum
  float* s_dl = s_il + H;                 // [H] d_o . o
  float* s_dofold = s_dl + H;             // [GA_THREADS / HC][HC] partial d_o
  const long long r = blockIdx.x;
  const int h = threadIdx.x % H, sl = threadIdx.x / H;
  float qv[C];
#pragma unroll
  for (int i = 0; i < C; ++i) qv[i] = __bfloat162float(q[(r * H + h) * C + i]);
  for (int i = threadIdx.x; i < HC; i += GA_THREADS) s_b[i] = __bfloat162float(gate_bias[i]);
  const bf16* kvr = kv + r * (long long)S * 2 * C;
  const bf16* mr = mask + r * (long long)S;
  const bf16* gr = gate + r * (long long)S * HC;
  const bf16* dor = dout + r * (long long)S * HC;
  __syncthreads();
  // ---- pass A.1: softmax statistics and o ----
  float m = -INFINITY, l = 0.f, acc[C];
#pragma unroll
  for (int i = 0; i < C; ++i) acc[i] = 0.f;
  for (int s = sl; s < S; s += lanes) {
    float d = 0.f, vv[C];
#pragma unroll
    for (int i = 0; i < C; ++i) {
      d = fmaf(qv[i], __bfloat162float(kvr[(long long)s * 2 * C + i]), d);
      vv[i] = __bfloat162float(kvr[(long long)s * 2 * C + C + i]);
    }
    if (__bfloat162float(mr[s]) == 0.f) d = GA_MASKED;
    const float mn = fmaxf(m, d);
    const float a = __expf(m - mn), p = __expf(d - mn);
    l = l * a + p;
#pragma unroll
    for (int i = 0; i < C; ++i) acc[i] = fmaf(p, vv[i], acc[i] * a);
    m = mn;
  }
  s_m[sl * H + h] = m;
  s_l[sl * H + h] = l;
#pragma unroll
  for (int i = 0; i < C; ++i) s_acc[(sl * H + h) * C + i] = acc[i];
  // ---- pass A.2: d_o[j] = sum_s dout[s][j] * sigmoid(gate[s][j] + b[j]) ----
  {
    const int j = threadIdx.x % HC, gl = threadIdx.x / HC, gls = GA_THREADS / HC;
    float part = 0.f;
    const float bj = s_b[j];
    for (int s = gl; s < S; s += gls) {
      const float g = sigmoidf_(__bfloat162float(gr[(long long)s * HC + j]) + bj);
      part = fmaf(__bfloat162float(dor[(long long)s * HC + j]), g, part);
    }
    s_dofold[gl * HC + j] = part;
  }
  __syncthreads();
  if (threadIdx.x < HC) {
    const int hh = threadIdx.x / C, i = threadIdx.x - hh * C;
    float mx = -INFINITY;
    for (int j = 0; j < lanes; ++j) mx = fmaxf(mx, s_m[j * H + hh]);
    float lt = 0.f, at = 0.f;
    for (int j = 0; j < lanes; ++j) {
      const float mj = s_m[j * H + hh];
      const float w = (mj == -INFINITY) ? 0.f : __expf(mj - mx);
      lt = fmaf(s_l[j * H + hh], w, lt);
      at = fmaf(s_acc[(j * H + hh) * C + i], w, at);
    }
    s_o[threadIdx.x] = lt > 0.f ? at / lt : 0.f;
    float dsum = 0.f;
    for (int gl = 0; gl < GA_THREADS / HC; ++gl) dsum += s_dofold[gl * HC + threadIdx.x];
    s_do[threadIdx.x] = dsum;
    if (i == 0) {
      s_mt[hh] = mx;
      s_il[hh] = lt > 0.f ? 1.f / lt : 0.f;
    }
  }
  __syncthreads();
  if (threadIdx.x < H) {
    float d = 0.f;
    for (int i = 0; i < C; ++i) d = fmaf(s_do[threadIdx.x * C + i], s_o[threadIdx.x * C + i], d);
    s_dl[threadIdx.x] = d;
  }
  __syncthreads();
  // ---- pass B.1: d_logit, d_q (thread-local), d_k / d_v (folded over the H threads of a sequence: consecutive lanes) ----
  {
    float dov[C], dqa[C];
#pragma unroll
    for (int i = 0; i < C; ++i) {
      dov[i] = s_do[h * C + i];
      dqa[i] = 0.f;
    }
    const float mt = s_mt[h], il = s_il[h], dl = s_dl[h];
    const int s_iters = (S + lanes - 1) / lanes;
    for (int it = 0; it < s_iters; ++it) {
      const int s = it * lanes + sl;
      const bool in = s < S;                         // every thread runs every iteration, so the shuffles below are warp-wide
      float kk[C], vv[C], d = 0.f, dw = 0.f;
#pragma unroll
      for (int i = 0; i < C; ++i) {
        kk[i] = in ? __bfloat162float(kvr[(long long)s * 2 * C + i]) : 0.f;
        vv[i] = in ? __bfloat162float(kvr[(long long)s * 2 * C + C + i]) : 0.f;
        d = fmaf(qv[i], kk[i], d);
        dw = fmaf(dov[i], vv[i], dw);
      }
      const bool masked = in && (__bfloat162float(mr[s]) == 0.f);
      if (masked) d = GA_MASKED;
      const float w = in ? __expf(d - mt) * il : 0.f;
      const float dlg = masked ? 0.f : w * (dw - dl);
      float dk[C], dv[C];
#pragma unroll
      for (int i = 0; i < C; ++i) {
        dqa[i] = fmaf(dlg, kk[i], dqa[i]);
        dk[i] = dlg * qv[i];
        dv[i] = w * dov[i];
      }
      // sum over the H heads: threads sl * H + 0 .. H - 1 are consecutive lanes of one warp (H divides 32)
      for (int off = H >> 1; off > 0; off >>= 1) {
#pragma unroll
        for (int i = 0; i < C; ++i) {
          dk[i] += __shfl_xor_sync(0xffffffffu, dk[i], off);
          dv[i] += __shfl_xor_sync(0xffffffffu, dv[i], off);
        }
      }
      if (in && h == 0) {
#pragma unroll
        for (int i = 0; i < C; ++i) {
          dkv[(r * S + s) * 2 * C + i] = __float2bfloat16(dk[i]);
          dkv[(r * S + s) * 2 * C + C + i] = __float2bfloat16(dv[i]);
        }
      }
    }
    __syncthreads();                                  // s_acc (read in the fold above) is reused
#pragma unroll
    for (int i = 0; i < C; ++i) s_acc[(sl * H + h) * C + i] = dqa[i];
  }
  __syncthreads();
  if (threadIdx.x < HC) {
    const int hh = threadIdx.x / C, i = threadIdx.x - hh * C;
    float t = 0.f;
    for (int j = 0; j < lanes; ++j) t += s_acc[(j * H + hh) * C + i];
    dq[r * HC + threadIdx.x] = t;
  }
  // ---- pass B.2: d_gate[s][j] = dout[s][j] * o[j] * g (1 - g) ----
  {
    const int j = threadIdx.x % HC, gl = threadIdx.x / HC, gls = GA_THREADS / HC;
    const float bj = s_b[j], oj = s_o[j];
    bf16* dgr = dgate + r * (long long)S * HC;
    for (int s = gl; s < S; s += gls) {
      const float g = sigmoidf_(__bfloat162float(gr[(long long)s * HC + j]) + bj);
      dgr[(long long)s * HC + j] = __float2bfloat16(__bfloat162float(dor[(long long)s * HC + j]) * oj * g * (1.f - g));
    }
  }
}

}  // namespace ffb

extern "C" {

// q: bf16 [R][H][C] (projected, scaled); kv: bf16 [R][S][2C] (keys | values); mask: bf16 [R][S] (0 = masked key);
// gate: bf16 [R][S][H*C] (gating projection, before bias and sigmoid); gate_bias: bf16 [H*C]; out: bf16 [R][S][H*C].
// H must divide 256, C is 8, 16 or 32, H*C <= 256.  Returns 0, -2 for unsupported sizes, -1 for a launch error.
int ffb_global_attention_fwd(const void* q, const void* kv, const void* mask, const void* gate, const void* gate_bias, void* out,
                             long long R, int S, int H, int C, void* stream) {
  using namespace ffb;
  if (R < 0 || S < 1 || H < 1 || GA_THREADS % H || H * C > GA_THREADS || (C != 8 && C != 16 && C != 32)) return -2;
  if (R == 0) return 0;
  if (R > 0x7fffffffLL) return -2;
  auto st = reinterpret_cast<cudaStream_t>(stream);
  // enough CTAs for ~6 per SM; a column is split over at most 8 CTAs (the portable cluster size), each gating at least 64 sequences
  int parts = (int)((148 * 6 + R - 1) / R);
  parts = parts < 1 ? 1 : (parts > 8 ? 8 : parts);
  while (parts > 1 && S / parts < 64) --parts;
  if (H == GC_H && C == GC_C) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)R, (unsigned)parts);
    cfg.blockDim = dim3(GA_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)parts;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, global_attention_cluster_kernel, (const bf16*)q, (const bf16*)kv, (const bf16*)mask,
                                             (const bf16*)gate, (const bf16*)gate_bias, (bf16*)out, S);
    return e == cudaSuccess ? 0 : -1;
  }
  const size_t smem = (size_t)(2 * GA_THREADS + GA_THREADS * C + 2 * H * C) * sizeof(float);
#define FFB_GA_LAUNCH(CC)                                                                                                          \
  do {                                                                                                                             \
    if (smem > 48 * 1024) cudaFuncSetAttribute(global_attention_kernel<CC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_light(global_attention_kernel<CC>, dim3((unsigned)R, (unsigned)parts), GA_THREADS, smem, st, (const bf16*)q, (const bf16*)kv, (const bf16*)mask,           \
                                                                       (const bf16*)gate, (const bf16*)gate_bias, (bf16*)out, S, H); \
  } while (0)
  if (C == 8) FFB_GA_LAUNCH(8);
  else if (C == 16) FFB_GA_LAUNCH(16);
  else FFB_GA_LAUNCH(32);
#undef FFB_GA_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Gradients of ffb_global_attention_fwd: dq fp32 [R][H][C], dkv bf16 [R][S][2C], dgate bf16 [R][S][H*C] (w.r.t. the gate
// before bias and sigmoid).  H must divide 32 and H * C must divide 256.
int ffb_global_attention_bwd(const void* q, const void* kv, const void* mask, const void* gate, const void* gate_bias, const void* dout,
                             float* dq, void* dkv, void* dgate, long long R, int S, int H, int C, void* stream) {
  using namespace ffb;
  if (R <= 0 || S <= 0) return 0;
  if (H <= 0 || (32 % H) || (GA_THREADS % (H * C)) || !(C == 8 || C == 16 || C == 32)) return -2;
  auto st = reinterpret_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)(2 * GA_THREADS + GA_THREADS * C + 3 * H * C + 3 * H + GA_THREADS) * sizeof(float);
#define FFB_GAB_LAUNCH(CC)                                                                                                              \
  do {                                                                                                                                  \
    if (smem > 48 * 1024) cudaFuncSetAttribute(global_attention_bwd_kernel<CC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    launch_light(global_attention_bwd_kernel<CC>, dim3((unsigned)R), GA_THREADS, smem, st, (const bf16*)q, (const bf16*)kv, (const bf16*)mask, \
             (const bf16*)gate, (const bf16*)gate_bias, (const bf16*)dout, dq, (bf16*)dkv, (bf16*)dgate, S, H);                         \
  } while (0)
  if (C == 8) FFB_GAB_LAUNCH(8);
  else if (C == 16) FFB_GAB_LAUNCH(16);
  else FFB_GAB_LAUNCH(32);
#undef FFB_GAB_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
