// Global column attention of the extra-MSA stack, core part in one kernel.
//
// Per MSA column r there is ONE query per head (the masked mean over the sequences, projected), and keys / values are
// shared by all heads (fastfold/model/fastnn/ops.py:1175-1236, openfold-style GlobalAttention).  With S_e sequences of
// c = 8 channels per head this is a bandwidth problem: per column  logits[h][s] = q[h] . k[s],  softmax over s (masked keys
// get the logit -1e9, replaced), o[h] = sum_s w[h][s] v[s], and then the gate  out[s][h*c + i] = sigmoid(g[s][h*c+i] + b) * o[h][i].
// The kernel makes one pass over (k | v) with an online softmax per (head, sequence lane), folds the lanes through
// shared memory, and streams the gate tensor once: no logits, weights or broadcast copies of o reach memory.
//
// One CTA per column, 256 threads; thread t works on head t % H and sequence lane t / H (H divides 256).
#include "common.cuh"

namespace ffb {

constexpr int GA_THREADS = 256;
constexpr float GA_MASKED = -1e9f;

template <int C>
__global__ void __launch_bounds__(GA_THREADS) global_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv,
                                                                      const bf16* __restrict__ mask, const bf16* __restrict__ gate,
                                                                      const bf16* __restrict__ gate_bias, bf16* __restrict__ out,
                                                                      int S, int H) {
  extern __shared__ float sm[];
  const int lanes = GA_THREADS / H;
  float* s_m = sm;                       // [lanes][H]
  float* s_l = s_m + GA_THREADS;         // [lanes][H]
  float* s_acc = s_l + GA_THREADS;       // [lanes][H][C]
  float* s_o = s_acc + GA_THREADS * C;   // [H][C]
  float* s_b = s_o + H * C;              // [H][C] gate bias
  const long long r = blockIdx.x;
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
  for (int s = sl; s < S; s += lanes) {
    // the H threads of one sequence lane read the same 4 * C bytes: one transaction, broadcast
    bf16 kk[C], vv[C];
    if constexpr (C % 8 == 0) {
#pragma unroll
      for (int i = 0; i < C / 8; ++i) {
        reinterpret_cast<uint4*>(kk)[i] = reinterpret_cast<const uint4*>(kvr + (long long)s * 2 * C)[i];
        reinterpret_cast<uint4*>(vv)[i] = reinterpret_cast<const uint4*>(kvr + (long long)s * 2 * C + C)[i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < C; ++i) {
        kk[i] = kvr[(long long)s * 2 * C + i];
        vv[i] = kvr[(long long)s * 2 * C + C + i];
      }
    }
    float lg = 0.f;
#pragma unroll
    for (int i = 0; i < C; ++i) lg = fmaf(qv[i], __bfloat162float(kk[i]), lg);
    if (__bfloat162float(mr[s]) == 0.f) lg = GA_MASKED;
    const float mn = fmaxf(m, lg);
    const float a = __expf(m - mn), p = __expf(lg - mn);      // m = -inf on the first key: a = 0
    l = l * a + p;
#pragma unroll
    for (int i = 0; i < C; ++i) acc[i] = fmaf(acc[i], a, p * __bfloat162float(vv[i]));
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
  if (HC % 8 == 0) {
    const long long nvec = (long long)S * HC / 8;
    for (long long v = threadIdx.x; v < nvec; v += GA_THREADS) {
      const int j0 = (int)((v * 8) % HC);
      const uint4 gv = reinterpret_cast<const uint4*>(gr)[v];
      const bf16* ge = reinterpret_cast<const bf16*>(&gv);
      uint4 ov;
      bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float x = __bfloat162float(ge[e]) + s_b[j0 + e];
        oe[e] = __float2bfloat16(s_o[j0 + e] / (1.f + __expf(-x)));
      }
      reinterpret_cast<uint4*>(orow)[v] = ov;
    }
  } else {
    const long long n = (long long)S * HC;
    for (long long v = threadIdx.x; v < n; v += GA_THREADS) {
      const int j = (int)(v % HC);
      const float x = __bfloat162float(gr[v]) + s_b[j];
      orow[v] = __float2bfloat16(s_o[j] / (1.f + __expf(-x)));
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
  const size_t smem = (size_t)(2 * GA_THREADS + GA_THREADS * C + 2 * H * C) * sizeof(float);
  auto st = reinterpret_cast<cudaStream_t>(stream);
#define FFB_GA_LAUNCH(CC)                                                                                                          \
  do {                                                                                                                             \
    if (smem > 48 * 1024) cudaFuncSetAttribute(global_attention_kernel<CC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    global_attention_kernel<CC><<<(unsigned)R, GA_THREADS, smem, st>>>((const bf16*)q, (const bf16*)kv, (const bf16*)mask,           \
                                                                       (const bf16*)gate, (const bf16*)gate_bias, (bf16*)out, S, H); \
  } while (0)
  if (C == 8) FFB_GA_LAUNCH(8);
  else if (C == 16) FFB_GA_LAUNCH(16);
  else FFB_GA_LAUNCH(32);
#undef FFB_GA_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
