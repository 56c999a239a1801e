// Recycling embedder, pair part, in one pass (inference):
//
//   out[i][j][:] = LayerNorm(z_prev[i][j][:]) + W[:, bin(|x_i - x_j|^2)] + b
//
// The reference builds a one-hot [N, N, no_bins] distogram of the previous iteration's pseudo-beta distances, runs it
// through a Linear(no_bins, c_z) and adds the normalised previous pair representation (fastfold/model/fastnn/embedders.py:
// 100-137, nn/embedders.py RecyclingEmbedder).  A one-hot times a matrix is a gather: the kernel computes the squared
// distance, finds the bin (strict inequalities on both edges, so a distance outside every bin contributes the bias only),
// and adds that column of the weight to the LayerNorm of the row - z_prev is read once, the output written once, and no
// [N, N, no_bins] tensor exists.
//
// One warp per (i, j) row of C = 128 channels (4 per lane, 8-byte accesses); weight (transposed to [bin][C], fp32), bias,
// gamma, beta staged in shared memory per CTA.
#include "common.cuh"

namespace ffb {

constexpr int RE_C = 128;
constexpr int RE_MAX_BINS = 64;
constexpr int RE_WARPS = 8;

__device__ __forceinline__ float re_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float re_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

__global__ void __launch_bounds__(RE_WARPS * 32) recycle_pair_embed_kernel(const bf16* __restrict__ z, const float* __restrict__ x,
                                                                          const float* __restrict__ sq_bins, const bf16* __restrict__ w,
                                                                          const bf16* __restrict__ bias, const bf16* __restrict__ gamma,
                                                                          const bf16* __restrict__ beta, bf16* __restrict__ out,
                                                                          int n_i, int i0, int N, int nb, float eps, float inf) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* s_w = sm;                      // [nb][C]
  float* s_b = s_w + nb * RE_C;         // [C]
  float* s_g = s_b + RE_C;              // [C]
  float* s_be = s_g + RE_C;             // [C]
  float* s_lo = s_be + RE_C;            // [nb] lower edges, squared
  for (int t = threadIdx.x; t < nb * RE_C; t += blockDim.x) {
    const int k = t / RE_C, c = t - k * RE_C;
    s_w[t] = __bfloat162float(w[c * nb + k]);          // w: [C][nb] as stored by nn.Linear
  }
  for (int t = threadIdx.x; t < RE_C; t += blockDim.x) {
    s_b[t] = __bfloat162float(bias[t]);
    s_g[t] = __bfloat162float(gamma[t]);
    s_be[t] = __bfloat162float(beta[t]);
  }
  for (int t = threadIdx.x; t < nb; t += blockDim.x) s_lo[t] = sq_bins[t];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long rows = (long long)n_i * N;
  for (long long r = (long long)blockIdx.x * RE_WARPS + warp; r < rows; r += (long long)gridDim.x * RE_WARPS) {
    const int il = (int)(r / N), j = (int)(r - (long long)il * N);
    const int i = i0 + il;
    const float dx = x[i * 3 + 0] - x[j * 3 + 0], dy = x[i * 3 + 1] - x[j * 3 + 1], dz = x[i * 3 + 2] - x[j * 3 + 2];
    const float d2 = (dx * dx + dy * dy) + dz * dz;
    int bin = -1;
    for (int k = 0; k < nb; ++k) {
      const float hi = (k + 1 < nb) ? s_lo[k + 1] : inf;
      if (d2 > s_lo[k] && d2 < hi) bin = k;
    }
    const uint2 raw = *reinterpret_cast<const uint2*>(z + r * RE_C + lane * 4);
    float v[4] = {re_lo(raw.x), re_hi(raw.x), re_lo(raw.y), re_hi(raw.y)};
    const float mean = warp_sum(v[0] + v[1] + v[2] + v[3]) * (1.f / RE_C);
    float q = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[e] -= mean;
      q += v[e] * v[e];
    }
    const float rstd = rsqrtf(warp_sum(q) * (1.f / RE_C) + eps);
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int c = lane * 4 + e;
      // the reference rounds the LayerNorm output and the linear output to bf16 before adding them
      const float ln = __bfloat162float(__float2bfloat16(v[e] * rstd * s_g[c] + s_be[c]));
      const float lin = __bfloat162float(__float2bfloat16((bin >= 0 ? s_w[bin * RE_C + c] : 0.f) + s_b[c]));
      o[e] = lin + ln;
    }
    uint2 res;
    *reinterpret_cast<bf162*>(&res.x) = __floats2bfloat162_rn(o[0], o[1]);
    *reinterpret_cast<bf162*>(&res.y) = __floats2bfloat162_rn(o[2], o[3]);
    *reinterpret_cast<uint2*>(out + r * RE_C + lane * 4) = res;
  }
}

}  // namespace ffb

extern "C" {

// z, out: bf16 [n_i][N][128] (rows i0 .. i0 + n_i of the pair representation); x: fp32 [N][3]; sq_bins: fp32 [nb] squared
// lower bin edges (ascending; the last bin is open up to `inf`); w: bf16 [128][nb]; bias, gamma, beta: bf16 [128].
// Returns 0, -2 for unsupported sizes, -1 for a launch error.
int ffb_recycle_pair_embed(const void* z, const void* x, const void* sq_bins, const void* w, const void* bias, const void* gamma,
                           const void* beta, void* out, int n_i, int i0, int N, int C, int nb, float eps, float inf, void* stream) {
  using namespace ffb;
  if (C != RE_C || nb < 1 || nb > RE_MAX_BINS || n_i < 0 || N < 1 || i0 < 0 || i0 + n_i > N) return -2;
  if (n_i == 0) return 0;
  const long long rows = (long long)n_i * N;
  const long long want = (rows + RE_WARPS - 1) / RE_WARPS;
  const unsigned grid = (unsigned)(want < 148 * 8 ? want : 148 * 8);
  const size_t smem = (size_t)(nb * RE_C + 3 * RE_C + nb) * sizeof(float);
  launch_light(recycle_pair_embed_kernel, grid, RE_WARPS * 32, smem, reinterpret_cast<cudaStream_t>(stream), (const bf16*)z, (const float*)x, (const float*)sq_bins, (const bf16*)w, (const bf16*)bias, (const bf16*)gamma, (const bf16*)beta,
      (bf16*)out, n_i, i0, N, nb, eps, inf);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
