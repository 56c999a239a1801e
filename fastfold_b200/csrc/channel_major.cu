// Kernels for activations kept channel-major ([C][rows], row index contiguous) on the training path of the
// triangle multiplication, so that the per-channel contraction GEMMs read and write them without transposed copies:
//
//   ln_bwd_transposed   backward of the LayerNorm whose input is channel-major and whose output is row-major
//                       (forward: ln_fwd_transposed_kernel in layernorm.cu): dy [rows][C], x [C][rows] -> dx [C][rows]
//   glu_mask_t          lr[ch][x] = pre[ch][x] * sigmoid(pre[C2 + ch][x]) * mask[x]   (forward and backward)
//
// The reference keeps everything channel-last and pays permute copies around its einsum-style contractions
// (fastfold/model/fastnn/ops.py:372-411); its LayerNorm backward is layer_norm_cuda_kernel.cu:316-399.
#include "common.cuh"

namespace ffb {

constexpr int LTB_ROWS = 32;

// Block = 256 threads = 8 warps, tile = 32 rows x C channels (C <= 256).  tx = row in tile, ty = warp.
// part: [gridDim.x][2][C] partial (dgamma, dbeta) sums, reduced by a second kernel.
__global__ void __launch_bounds__(256) ln_bwd_transposed_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                               const bf16* __restrict__ gamma, const float* __restrict__ mean,
                                                               const float* __restrict__ rstd, bf16* __restrict__ dx,
                                                               float* __restrict__ part, long long rows, int C) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* t_x = sm;                              // [C][33] normalised input
  float* t_g = sm + C * (LTB_ROWS + 1);         // [C][33] dy * gamma
  __shared__ float s_a[8][LTB_ROWS], s_b[8][LTB_ROWS];
  const long long r0 = (long long)blockIdx.x * LTB_ROWS;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long r = r0 + tx;
  const bool rok = r < rows;
  const float mu = rok ? mean[r] : 0.f, rs = rok ? rstd[r] : 0.f;
  // x: lanes along rows (contiguous in memory)
  for (int c = ty; c < C; c += 8) t_x[c * (LTB_ROWS + 1) + tx] = rok ? (__bfloat162float(x[(long long)c * rows + r]) - mu) * rs : 0.f;
  // dy: lanes along channels (contiguous in memory); stored transposed
  for (int idx = threadIdx.x; idx < LTB_ROWS * C; idx += 256) {
    const int rr = idx / C, c = idx - rr * C;
    const float v = (r0 + rr < rows) ? __bfloat162float(dy[(r0 + rr) * C + c]) : 0.f;
    t_g[c * (LTB_ROWS + 1) + rr] = v;
  }
  __syncthreads();
  // per channel: dgamma / dbeta partials over the tile's rows (warp reduction over tx), then scale dy by gamma in place
  float a = 0.f, b = 0.f;     // per row: sum_c dy*gamma, sum_c dy*gamma*xhat (this warp's channels)
  for (int c = ty; c < C; c += 8) {
    const float g = t_g[c * (LTB_ROWS + 1) + tx], xh = t_x[c * (LTB_ROWS + 1) + tx];
    const float dg = warp_sum(g * xh), db = warp_sum(g);
    if (tx == 0) {
      part[((long long)blockIdx.x * 2) * C + c] = dg;
      part[((long long)blockIdx.x * 2 + 1) * C + c] = db;
    }
    const float gg = g * __bfloat162float(gamma[c]);
    t_g[c * (LTB_ROWS + 1) + tx] = gg;
    a += gg;
    b += gg * xh;
  }
  s_a[ty][tx] = a;
  s_b[ty][tx] = b;
  __syncthreads();
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    s1 += s_a[w][tx];
    s2 += s_b[w][tx];
  }
  const float inv_c = 1.f / C;
  s1 *= inv_c;
  s2 *= inv_c;
  if (rok)
    for (int c = ty; c < C; c += 8) {
      const float gg = t_g[c * (LTB_ROWS + 1) + tx], xh = t_x[c * (LTB_ROWS + 1) + tx];
      dx[(long long)c * rows + r] = __float2bfloat16(rs * (gg - s1 - xh * s2));
    }
}

// dgamma[c] = sum_b part[b][0][c], dbeta[c] = sum_b part[b][1][c]; block = 32 columns x 32 slices of blocks
__global__ void __launch_bounds__(1024) ltb_reduce_kernel(const float* __restrict__ part, int nblocks, int C, float* __restrict__ dgamma,
                                                          float* __restrict__ dbeta, int accumulate) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float acc[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < 2 * C)
    for (int b = ty; b < nblocks; b += 32) s += part[(long long)b * 2 * C + c];
  acc[ty][tx] = s;
  __syncthreads();
  const float v = warp_sum(acc[tx][ty]);
  const int co = blockIdx.x * 32 + ty;
  if (tx == 0 && co < 2 * C) {
    float* dst = co < C ? dgamma + co : dbeta + (co - C);
    *dst = accumulate ? *dst + v : v;
  }
}

// 8 bf16 per thread along the contiguous index
__global__ void glu_mask_t_fwd_kernel(const bf16* __restrict__ pre, const bf16* __restrict__ mask, bf16* __restrict__ out, int C2,
                                      long long R) {
  pdl_launch_dependents();
  pdl_wait();
  const long long vec_per_row = R >> 3;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= vec_per_row * C2) return;
  const long long ch = i / vec_per_row, xv = (i - ch * vec_per_row) << 3;
  const uint4 uv = *reinterpret_cast<const uint4*>(pre + ch * R + xv);
  const uint4 ug = *reinterpret_cast<const uint4*>(pre + (ch + C2) * R + xv);
  const uint4 um = *reinterpret_cast<const uint4*>(mask + xv);
  const bf162 *hv = reinterpret_cast<const bf162*>(&uv), *hg = reinterpret_cast<const bf162*>(&ug), *hm = reinterpret_cast<const bf162*>(&um);
  uint4 uo;
  bf162* ho = reinterpret_cast<bf162*>(&uo);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 v = __bfloat1622float2(hv[e]), g = __bfloat1622float2(hg[e]), m = __bfloat1622float2(hm[e]);
    ho[e] = __floats2bfloat162_rn(v.x * sigmoidf_(g.x) * m.x, v.y * sigmoidf_(g.y) * m.y);
  }
  *reinterpret_cast<uint4*>(out + ch * R + xv) = uo;
}

__global__ void glu_mask_t_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ pre, const bf16* __restrict__ mask,
                                      bf16* __restrict__ dpre, int C2, long long R) {
  pdl_launch_dependents();
  pdl_wait();
  const long long vec_per_row = R >> 3;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= vec_per_row * C2) return;
  const long long ch = i / vec_per_row, xv = (i - ch * vec_per_row) << 3;
  const uint4 ud = *reinterpret_cast<const uint4*>(dout + ch * R + xv);
  const uint4 uv = *reinterpret_cast<const uint4*>(pre + ch * R + xv);
  const uint4 ug = *reinterpret_cast<const uint4*>(pre + (ch + C2) * R + xv);
  const uint4 um = *reinterpret_cast<const uint4*>(mask + xv);
  const bf162 *hd = reinterpret_cast<const bf162*>(&ud), *hv = reinterpret_cast<const bf162*>(&uv), *hg = reinterpret_cast<const bf162*>(&ug),
              *hm = reinterpret_cast<const bf162*>(&um);
  uint4 o1, o2;
  bf162 *h1 = reinterpret_cast<bf162*>(&o1), *h2 = reinterpret_cast<bf162*>(&o2);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 d = __bfloat1622float2(hd[e]), v = __bfloat1622float2(hv[e]), g = __bfloat1622float2(hg[e]), m = __bfloat1622float2(hm[e]);
    const float sx = sigmoidf_(g.x), sy = sigmoidf_(g.y);
    const float dx_ = d.x * m.x, dy_ = d.y * m.y;
    h1[e] = __floats2bfloat162_rn(dx_ * sx, dy_ * sy);
    h2[e] = __floats2bfloat162_rn(dx_ * v.x * sx * (1.f - sx), dy_ * v.y * sy * (1.f - sy));
  }
  *reinterpret_cast<uint4*>(dpre + ch * R + xv) = o1;
  *reinterpret_cast<uint4*>(dpre + (ch + C2) * R + xv) = o2;
}

}  // namespace ffb

using namespace ffb;

extern "C" {

// Number of fp32 words of the `part` workspace the backward needs for `rows` rows.
long long ffb_layernorm_bwd_transposed_workspace(long long rows, int C) {
  return ((rows + LTB_ROWS - 1) / LTB_ROWS) * 2 * (long long)C;
}

// dy: bf16 [rows][C]; x: bf16 [C][rows]; mean / rstd: fp32 [rows] (saved by the forward); dx: bf16 [C][rows];
// dgamma / dbeta: fp32 [C]; part: fp32 workspace (ffb_layernorm_bwd_transposed_workspace words).
static int layernorm_bwd_transposed_impl(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                                         float* part, float* dgamma, float* dbeta, long long rows, int C, int accumulate, void* stream) {
  if (C > 256 || C < 1) return -2;
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t smem = sizeof(float) * 2 * C * (LTB_ROWS + 1);
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(ln_bwd_transposed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(float) * 2 * 256 * (LTB_ROWS + 1))) !=
        cudaSuccess)
      return -3;
    attr = true;
  }
  const long long nb = (rows + LTB_ROWS - 1) / LTB_ROWS;
  if (nb > 0x7fffffffLL) return -4;
  launch_light(ln_bwd_transposed_kernel, (unsigned)nb, 256, smem, st, (const bf16*)dy, (const bf16*)x, (const bf16*)gamma, mean, rstd, (bf16*)dx, part,
                                                           rows, C);
  launch_light(ltb_reduce_kernel, (2 * C + 31) / 32, 1024, 0, st, part, (int)nb, C, dgamma, dbeta, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int ffb_layernorm_bwd_transposed(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                                 float* part, float* dgamma, float* dbeta, long long rows, int C, void* stream) {
  return layernorm_bwd_transposed_impl(dy, x, gamma, mean, rstd, dx, part, dgamma, dbeta, rows, C, 0, stream);
}

// Same, but the column sums are ADDED to dgamma / dbeta (a trainer's fp32 gradient buffer).
int ffb_layernorm_bwd_transposed_acc(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                                     float* part, float* dgamma, float* dbeta, long long rows, int C, void* stream) {
  return layernorm_bwd_transposed_impl(dy, x, gamma, mean, rstd, dx, part, dgamma, dbeta, rows, C, 1, stream);
}

// pre: bf16 [2 * C2][R] (rows [0, C2) values, rows [C2, 2 C2) gates); mask: bf16 [R]; out: bf16 [C2][R].  R % 8 == 0.
int ffb_glu_mask_t_fwd(const void* pre, const void* mask, void* out, int C2, long long R, void* stream) {
  if (R % 8 || C2 < 1) return -2;
  const long long n = (R >> 3) * C2;
  if (n <= 0) return 0;
  launch_light(glu_mask_t_fwd_kernel, (unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream), (const bf16*)pre, (const bf16*)mask,
                                                                                                        (bf16*)out, C2, R);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// dout: bf16 [C2][R]; dpre: bf16 [2 * C2][R].
int ffb_glu_mask_t_bwd(const void* dout, const void* pre, const void* mask, void* dpre, int C2, long long R, void* stream) {
  if (R % 8 || C2 < 1) return -2;
  const long long n = (R >> 3) * C2;
  if (n <= 0) return 0;
  launch_light(glu_mask_t_bwd_kernel, (unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream), (const bf16*)dout, (const bf16*)pre, (const bf16*)mask, (bf16*)dpre, C2, R);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
