// LayerNorm over the last dimension, forward and backward, for bf16 / fp16 /
// fp32 activations with fp32 statistics.
//
// The op is bandwidth-bound, so the design is about bytes: one warp owns one
// row, the row is read once with 16-byte loads and kept in registers for the
// mean, the variance (two-pass in registers, no cancellation) and the
// normalisation; the backward kernel reads x and dy once, writes dx once and
// folds the per-column sums for dgamma / dbeta into per-block partials that a
// second tiny kernel reduces.  Rows up to 1024 elements take the register path
// (c_m = 256, c_z = 128, c_s = 384, c_e = c_t = 64 all do); longer rows fall to
// a looped path.  The optional `transposed input` variant normalises over the
// leading dimension of a [C, rows] tensor and writes [rows, C]: it is the
// LayerNorm that follows the per-channel triangle-multiplication GEMM, whose
// output is channel-major.
//
// Replaces fastfold/model/fastnn/kernel/cuda_native/csrc/layer_norm_cuda_kernel.cu
// (forward :61-152, gamma/beta partial sums :224-333, input gradient :335-443)
// and the Triton twins in kernel/triton/layer_norm.py.
#include "common.cuh"

namespace ffb {

constexpr int LN_WARPS = 4;

template <typename T, int VPL>  // VPL = values per lane (multiple of 8 for 16-bit types, 4 for fp32)
__global__ void __launch_bounds__(LN_WARPS * 32) ln_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                              const T* __restrict__ beta, T* __restrict__ y,
                                                              float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                              long long rows, int C, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  constexpr int VEC = 16 / sizeof(T);
  constexpr int NV = VPL / VEC;
  float v[VPL];
  const T* xr = x + row * C;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c0 = (i * 32 + lane) * VEC;
    if (c0 < C) {
      uint4 u = *reinterpret_cast<const uint4*>(xr + c0);
      const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        v[i * VEC + j] = to_f<T>(e[j]);
        s += v[i * VEC + j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[i * VEC + j] = 0.f;
    }
  }
  const float mean = warp_sum(s) / C;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c0 = (i * 32 + lane) * VEC;
    if (c0 < C) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float d = v[i * VEC + j] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / C + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  T* yr = y + row * C;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c0 = (i * 32 + lane) * VEC;
    if (c0 < C) {
      uint4 ug = *reinterpret_cast<const uint4*>(gamma + c0);
      uint4 ub = *reinterpret_cast<const uint4*>(beta + c0);
      const T* ge = reinterpret_cast<const T*>(&ug);
      const T* be = reinterpret_cast<const T*>(&ub);
      uint4 uo;
      T* oe = reinterpret_cast<T*>(&uo);
#pragma unroll
      for (int j = 0; j < VEC; ++j) oe[j] = from_f<T>((v[i * VEC + j] - mean) * rstd * to_f<T>(ge[j]) + to_f<T>(be[j]));
      *reinterpret_cast<uint4*>(yr + c0) = uo;
    }
  }
}

// Any C, any alignment: three passes over the row from global memory / L2.
template <typename T>
__global__ void __launch_bounds__(LN_WARPS * 32) ln_fwd_generic_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                                      const T* __restrict__ beta, T* __restrict__ y,
                                                                      float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                      long long rows, int C, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * C;
  float s = 0.f;
  for (int c = lane; c < C; c += 32) s += to_f<T>(xr[c]);
  const float mean = warp_sum(s) / C;
  float q = 0.f;
  for (int c = lane; c < C; c += 32) {
    const float d = to_f<T>(xr[c]) - mean;
    q += d * d;
  }
  const float rstd = rsqrtf(warp_sum(q) / C + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  T* yr = y + row * C;
  for (int c = lane; c < C; c += 32) yr[c] = from_f<T>((to_f<T>(xr[c]) - mean) * rstd * to_f<T>(gamma[c]) + to_f<T>(beta[c]));
}

// Backward.  Block = LN_WARPS warps, each block walks rows blockIdx.x, +gridDim.x, ...
// Per-lane column ownership is fixed, so dgamma/dbeta partial sums stay in
// registers over the whole walk and are combined across the block's warps at
// the end: part[blockIdx.x][0][c] = sum dy*xhat, part[blockIdx.x][1][c] = sum dy.
template <typename T, int VPL>
__global__ void __launch_bounds__(LN_WARPS * 32) ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                              const T* __restrict__ gamma, const float* __restrict__ mean,
                                                              const float* __restrict__ rstd, T* __restrict__ dx,
                                                              float* __restrict__ part, long long rows, int C) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int VEC = 16 / sizeof(T);
  constexpr int NV = VPL / VEC;
  __shared__ float red[LN_WARPS][2];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  float g[VPL], dg[VPL], db[VPL];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c0 = (i * 32 + lane) * VEC;
    if (c0 < C) {
      uint4 ug = *reinterpret_cast<const uint4*>(gamma + c0);
      const T* ge = reinterpret_cast<const T*>(&ug);
#pragma unroll
      for (int j = 0; j < VEC; ++j) g[i * VEC + j] = to_f<T>(ge[j]);
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) g[i * VEC + j] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) dg[i * VEC + j] = db[i * VEC + j] = 0.f;
  }
  (void)red;
  for (long long row = (long long)blockIdx.x * LN_WARPS + warp; row < rows; row += (long long)gridDim.x * LN_WARPS) {
    const float mu = mean[row], rs = rstd[row];
    float xh[VPL], d[VPL];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c0 = (i * 32 + lane) * VEC;
      if (c0 < C) {
        uint4 ux = *reinterpret_cast<const uint4*>(x + row * C + c0);
        uint4 ud = *reinterpret_cast<const uint4*>(dy + row * C + c0);
        const T* xe = reinterpret_cast<const T*>(&ux);
        const T* de = reinterpret_cast<const T*>(&ud);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const int k = i * VEC + j;
          xh[k] = (to_f<T>(xe[j]) - mu) * rs;
          d[k] = to_f<T>(de[j]);
          dg[k] += d[k] * xh[k];
          db[k] += d[k];
          const float gd = g[k] * d[k];
          s1 += gd;
          s2 += gd * xh[k];
        }
      } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) xh[i * VEC + j] = d[i * VEC + j] = 0.f;
      }
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c0 = (i * 32 + lane) * VEC;
      if (c0 < C) {
        uint4 uo;
        T* oe = reinterpret_cast<T*>(&uo);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const int k = i * VEC + j;
          oe[j] = from_f<T>(rs * (g[k] * d[k] - s1 - xh[k] * s2));
        }
        *reinterpret_cast<uint4*>(dx + row * C + c0) = uo;
      }
    }
  }
  // combine the block's warps through global atomics on the block's partial row
  float* p0 = part + (long long)blockIdx.x * 2 * C;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c0 = (i * 32 + lane) * VEC;
    if (c0 < C) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        atomicAdd(p0 + c0 + j, dg[i * VEC + j]);
        atomicAdd(p0 + C + c0 + j, db[i * VEC + j]);
      }
    }
  }
}

template <typename T>
__global__ void ln_bwd_generic_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                                      const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                                      float* __restrict__ part, long long rows, int C) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  float* p0 = part + (long long)blockIdx.x * 2 * C;
  for (long long row = (long long)blockIdx.x * LN_WARPS + warp; row < rows; row += (long long)gridDim.x * LN_WARPS) {
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane; c < C; c += 32) {
      const float xh = (to_f<T>(x[row * C + c]) - mu) * rs;
      const float d = to_f<T>(dy[row * C + c]);
      const float gd = to_f<T>(gamma[c]) * d;
      s1 += gd;
      s2 += gd * xh;
      atomicAdd(p0 + c, d * xh);
      atomicAdd(p0 + C + c, d);
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
    for (int c = lane; c < C; c += 32) {
      const float xh = (to_f<T>(x[row * C + c]) - mu) * rs;
      const float d = to_f<T>(dy[row * C + c]);
      dx[row * C + c] = from_f<T>(rs * (to_f<T>(gamma[c]) * d - s1 - xh * s2));
    }
  }
}

// dgamma[c] = sum_b part[b][0][c], dbeta[c] = sum_b part[b][1][c]
template <typename T>
__global__ void __launch_bounds__(1024) ln_bwd_reduce_kernel(const float* __restrict__ part, int nblocks, int C,
                                                             T* __restrict__ dgamma, T* __restrict__ dbeta) {
  pdl_launch_dependents();
  pdl_wait();
  // block = 32 columns x 32 row slices: coalesced 128-byte reads, 32 partial sums per column folded through shared memory
  __shared__ float acc[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < 2 * C)
    for (int b = ty; b < nblocks; b += 32) s += part[(long long)b * 2 * C + c];
  acc[ty][tx] = s;
  __syncthreads();
  // warp ty now owns column ty of the tile: lanes hold its 32 slices
  float v = warp_sum(acc[tx][ty]);
  const int co = blockIdx.x * 32 + ty;
  if (tx == 0 && co < 2 * C) {
    if (co < C) dgamma[co] = from_f<T>(v);
    else dbeta[co - C] = from_f<T>(v);
  }
}

// Same reduction, ADDED into fp32 vectors (a trainer's flat gradient buffer): one writer per column, no atomics.
__global__ void __launch_bounds__(1024) ln_bwd_reduce_acc_kernel(const float* __restrict__ part, int nblocks, int C,
                                                                 float* __restrict__ dgamma, float* __restrict__ dbeta) {
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
    if (co < C) dgamma[co] += v;
    else dbeta[co - C] += v;
  }
}

// LayerNorm over the leading dimension of x[C][rows] (row index contiguous),
// output y[rows][C].  One thread per row for the statistics (coalesced across
// the warp), staged through shared memory so that the [rows, C] writes are
// 16-byte coalesced too.  C <= 256, bf16.
constexpr int LNT_ROWS = 32;
__global__ void __launch_bounds__(256) ln_fwd_transposed_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gamma,
                                                               const bf16* __restrict__ beta, bf16* __restrict__ y,
                                                               float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                               long long rows, int C, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float tile[];  // [C][LNT_ROWS + 1]
  __shared__ float s_mean[LNT_ROWS], s_rstd[LNT_ROWS];
  const long long r0 = (long long)blockIdx.x * LNT_ROWS;
  const int tx = threadIdx.x & 31;   // row within the tile
  const int ty = threadIdx.x >> 5;   // 0..7
  for (int c = ty; c < C; c += 8) {
    const long long r = r0 + tx;
    tile[c * (LNT_ROWS + 1) + tx] = (r < rows) ? __bfloat162float(x[(long long)c * rows + r]) : 0.f;
  }
  __syncthreads();
  // statistics: every warp sums its share of the channels for row tx, shares are folded through shared memory
  __shared__ float s_part[8][LNT_ROWS];
  {
    float s = 0.f;
    for (int c = ty; c < C; c += 8) s += tile[c * (LNT_ROWS + 1) + tx];
    s_part[ty][tx] = s;
  }
  __syncthreads();
  float mu = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) mu += s_part[w][tx];
  mu /= C;
  __syncthreads();
  {
    float q = 0.f;
    for (int c = ty; c < C; c += 8) {
      const float d = tile[c * (LNT_ROWS + 1) + tx] - mu;
      q += d * d;
    }
    s_part[ty][tx] = q;
  }
  __syncthreads();
  if (ty == 0) {
    float q = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) q += s_part[w][tx];
    const float rs = rsqrtf(q / C + eps);
    s_mean[tx] = mu;
    s_rstd[tx] = rs;
    if (r0 + tx < rows) {
      if (mean_out) mean_out[r0 + tx] = mu;
      if (rstd_out) rstd_out[r0 + tx] = rs;
    }
  }
  __syncthreads();
  // write: consecutive threads -> consecutive channels of one row
  for (int idx = threadIdx.x; idx < LNT_ROWS * C; idx += blockDim.x) {
    const int r = idx / C, c = idx - r * C;
    if (r0 + r < rows)
      y[(r0 + r) * C + c] = __float2bfloat16((tile[c * (LNT_ROWS + 1) + r] - s_mean[r]) * s_rstd[r] * __bfloat162float(gamma[c]) +
                                             __bfloat162float(beta[c]));
  }
}

// 64-row tiles: a warp reads 128 contiguous bytes per channel (two rows per lane), four channels in flight per warp,
// and the normalised rows leave as 16-byte stores.  rows % 2 == 0, C % 8 == 0, C <= 256.
constexpr int LNT64 = 64;
__global__ void __launch_bounds__(256) ln_fwd_transposed64_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gamma,
                                                                 const bf16* __restrict__ beta, bf16* __restrict__ y,
                                                                 float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                 long long rows, int C, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float tile[];  // [C][LNT64 + 1]
  __shared__ float s_part[8][LNT64], s_mean[LNT64], s_rstd[LNT64];
  constexpr int P = LNT64 + 1;
  const long long r0 = (long long)blockIdx.x * LNT64;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long r = r0 + 2 * tx;
  const bool ok = r < rows;                      // rows is even: the pair is in range together
  for (int c = ty; c < C; c += 32) {
    bf162 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int cc = c + 8 * k;
      v[k] = (ok && cc < C) ? *reinterpret_cast<const bf162*>(x + (long long)cc * rows + r) : __floats2bfloat162_rn(0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int cc = c + 8 * k;
      if (cc < C) {
        const float2 f = __bfloat1622float2(v[k]);
        tile[cc * P + 2 * tx] = f.x;
        tile[cc * P + 2 * tx + 1] = f.y;
      }
    }
  }
  __syncthreads();
  {
    float a = 0.f, b = 0.f;
    for (int c = ty; c < C; c += 8) {
      a += tile[c * P + tx];
      b += tile[c * P + tx + 32];
    }
    s_part[ty][tx] = a;
    s_part[ty][tx + 32] = b;
  }
  __syncthreads();
  float mu0 = 0.f, mu1 = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    mu0 += s_part[w][tx];
    mu1 += s_part[w][tx + 32];
  }
  mu0 /= C;
  mu1 /= C;
  __syncthreads();
  {
    float a = 0.f, b = 0.f;
    for (int c = ty; c < C; c += 8) {
      const float d0 = tile[c * P + tx] - mu0, d1 = tile[c * P + tx + 32] - mu1;
      a += d0 * d0;
      b += d1 * d1;
    }
    s_part[ty][tx] = a;
    s_part[ty][tx + 32] = b;
  }
  __syncthreads();
  if (ty < 2) {
    const int rr = tx + 32 * ty;
    float q = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) q += s_part[w][rr];
    const float mu = ty == 0 ? mu0 : mu1;
    const float rs = rsqrtf(q / C + eps);
    s_mean[rr] = mu;
    s_rstd[rr] = rs;
    if (r0 + rr < rows) {
      if (mean_out) mean_out[r0 + rr] = mu;
      if (rstd_out) rstd_out[r0 + rr] = rs;
    }
  }
  __syncthreads();
  const int groups = C >> 3;
  for (int idx = threadIdx.x; idx < LNT64 * groups; idx += 256) {
    const int rr = idx / groups, c0 = (idx - rr * groups) * 8;
    if (r0 + rr >= rows) continue;
    const float mu = s_mean[rr], rs = s_rstd[rr];
    const uint4 ug = *reinterpret_cast<const uint4*>(gamma + c0), ub = *reinterpret_cast<const uint4*>(beta + c0);
    const bf162 *hg = reinterpret_cast<const bf162*>(&ug), *hb = reinterpret_cast<const bf162*>(&ub);
    uint4 uo;
    bf162* ho = reinterpret_cast<bf162*>(&uo);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g2 = __bfloat1622float2(hg[j]), b2 = __bfloat1622float2(hb[j]);
      ho[j] = __floats2bfloat162_rn((tile[(c0 + 2 * j) * P + rr] - mu) * rs * g2.x + b2.x, (tile[(c0 + 2 * j + 1) * P + rr] - mu) * rs * g2.y + b2.y);
    }
    *reinterpret_cast<uint4*>(y + (r0 + rr) * C + c0) = uo;
  }
}

// ---------------------------------------------------------------------------
// bf16 rows of C = 8 * L elements, L in {8, 16, 32} lanes per row (C = 64, 128, 256 - every LayerNorm of the
// Evoformer): a warp works on 32 / L rows side by side and on MR_U such groups per step, so that every lane has
// MR_U independent 16-byte loads in flight (the one-row-per-warp kernels above leave half the lanes idle at C = 128
// and have a single load in flight per lane).
// ---------------------------------------------------------------------------
constexpr int MR_U = 4;

template <int L>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = L / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  bf162* h = reinterpret_cast<bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

template <int L>
__global__ void __launch_bounds__(LN_WARPS * 32) ln_fwd_mr_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gamma,
                                                                 const bf16* __restrict__ beta, bf16* __restrict__ y,
                                                                 float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                 long long rows, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int C = 8 * L, G = 32 / L;
  const int lane = threadIdx.x & 31, li = lane % L, grp = lane / L;
  const long long base = ((long long)blockIdx.x * LN_WARPS + (threadIdx.x >> 5)) * (G * MR_U) + grp;
  float g[8], b[8];
  unpack8(*reinterpret_cast<const uint4*>(gamma + li * 8), g);
  unpack8(*reinterpret_cast<const uint4*>(beta + li * 8), b);
  uint4 raw[MR_U];
#pragma unroll
  for (int u = 0; u < MR_U; ++u) {
    const long long row = base + u * G;
    raw[u] = row < rows ? *reinterpret_cast<const uint4*>(x + row * C + li * 8) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int u = 0; u < MR_U; ++u) {
    const long long row = base + u * G;
    float v[8];
    unpack8(raw[u], v);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[j];
    const float mean = group_sum<L>(s) * (1.f / C);
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] -= mean;
      q += v[j] * v[j];
    }
    const float rstd = rsqrtf(group_sum<L>(q) * (1.f / C) + eps);
    if (row < rows) {
      if (li == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = v[j] * rstd * g[j] + b[j];
      *reinterpret_cast<uint4*>(y + row * C + li * 8) = pack8(v);
    }
  }
}

// part: [gridDim.x][2][C], written with plain stores (every block writes its whole row of partials)
template <int L>
__global__ void __launch_bounds__(LN_WARPS * 32) ln_bwd_mr_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                                 const bf16* __restrict__ gamma, const float* __restrict__ mean,
                                                                 const float* __restrict__ rstd, bf16* __restrict__ dx,
                                                                 float* __restrict__ part, long long rows) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int C = 8 * L, G = 32 / L;
  __shared__ float red[LN_WARPS][2][C];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, li = lane % L, grp = lane / L;
  float g[8], dg[8], db[8];
  unpack8(*reinterpret_cast<const uint4*>(gamma + li * 8), g);
#pragma unroll
  for (int j = 0; j < 8; ++j) dg[j] = db[j] = 0.f;
  const long long step = (long long)gridDim.x * LN_WARPS * (G * MR_U);
  for (long long base = ((long long)blockIdx.x * LN_WARPS + warp) * (G * MR_U) + grp; base - grp < rows; base += step) {
    uint4 rx[MR_U], rd[MR_U];
    float mu[MR_U], rs[MR_U];
#pragma unroll
    for (int u = 0; u < MR_U; ++u) {
      const long long row = base + u * G;
      const bool ok = row < rows;
      rx[u] = ok ? *reinterpret_cast<const uint4*>(x + row * C + li * 8) : make_uint4(0, 0, 0, 0);
      rd[u] = ok ? *reinterpret_cast<const uint4*>(dy + row * C + li * 8) : make_uint4(0, 0, 0, 0);
      mu[u] = ok ? mean[row] : 0.f;
      rs[u] = ok ? rstd[row] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < MR_U; ++u) {
      const long long row = base + u * G;
      float xh[8], d[8];
      unpack8(rx[u], xh);
      unpack8(rd[u], d);
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[j] = (xh[j] - mu[u]) * rs[u];
        dg[j] += d[j] * xh[j];
        db[j] += d[j];
        d[j] *= g[j];
        s1 += d[j];
        s2 += d[j] * xh[j];
      }
      s1 = group_sum<L>(s1) * (1.f / C);
      s2 = group_sum<L>(s2) * (1.f / C);
      if (row < rows) {
#pragma unroll
        for (int j = 0; j < 8; ++j) d[j] = rs[u] * (d[j] - s1 - xh[j] * s2);
        *reinterpret_cast<uint4*>(dx + row * C + li * 8) = pack8(d);
      }
    }
  }
  // fold the row groups of the warp (lanes li, li + L, ...), then the warps of the block
#pragma unroll
  for (int j = 0; j < 8; ++j) {
#pragma unroll
    for (int o = L; o < 32; o <<= 1) {
      dg[j] += __shfl_xor_sync(0xffffffffu, dg[j], o);
      db[j] += __shfl_xor_sync(0xffffffffu, db[j], o);
    }
  }
  if (grp == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      red[warp][0][li * 8 + j] = dg[j];
      red[warp][1][li * 8 + j] = db[j];
    }
  }
  __syncthreads();
  float* p0 = part + (long long)blockIdx.x * 2 * C;
  for (int i = threadIdx.x; i < 2 * C; i += LN_WARPS * 32) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < LN_WARPS; ++w) t += (&red[w][0][0])[i];
    p0[i] = t;
  }
}

template <typename T>
struct IsBf16 { static constexpr bool value = false; };
template <>
struct IsBf16<bf16> { static constexpr bool value = true; };

template <typename T>
static int ln_fwd_dispatch(const T* x, const T* g, const T* b, T* y, float* mean, float* rstd, long long rows, int C, float eps,
                           cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(T);
  const dim3 grid((unsigned)((rows + LN_WARPS - 1) / LN_WARPS));
  const bool aligned = (C % VEC == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                                           reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(b)) % 16 == 0);
  if (IsBf16<T>::value && aligned && (C == 64 || C == 128 || C == 256)) {
    const bf16 *xb = reinterpret_cast<const bf16*>(x), *gb = reinterpret_cast<const bf16*>(g), *bb = reinterpret_cast<const bf16*>(b);
    bf16* yb = reinterpret_cast<bf16*>(y);
    const int rows_per_block = LN_WARPS * MR_U * (256 / C);
    const dim3 gmr((unsigned)((rows + rows_per_block - 1) / rows_per_block));
    if (C == 64) launch_light(ln_fwd_mr_kernel<8>, gmr, LN_WARPS * 32, 0, st, xb, gb, bb, yb, mean, rstd, rows, eps);
    else if (C == 128) launch_light(ln_fwd_mr_kernel<16>, gmr, LN_WARPS * 32, 0, st, xb, gb, bb, yb, mean, rstd, rows, eps);
    else launch_light(ln_fwd_mr_kernel<32>, gmr, LN_WARPS * 32, 0, st, xb, gb, bb, yb, mean, rstd, rows, eps);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
  }
  if (aligned && C <= 32 * VEC) launch_light(ln_fwd_kernel<T, VEC>, grid, LN_WARPS * 32, 0, st, x, g, b, y, mean, rstd, rows, C, eps);
  else if (aligned && C <= 64 * VEC) launch_light(ln_fwd_kernel<T, 2 * VEC>, grid, LN_WARPS * 32, 0, st, x, g, b, y, mean, rstd, rows, C, eps);
  else if (aligned && C <= 128 * VEC) launch_light(ln_fwd_kernel<T, 4 * VEC>, grid, LN_WARPS * 32, 0, st, x, g, b, y, mean, rstd, rows, C, eps);
  else launch_light(ln_fwd_generic_kernel<T>, grid, LN_WARPS * 32, 0, st, x, g, b, y, mean, rstd, rows, C, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

template <typename T>
static int ln_bwd_dispatch(const T* dy, const T* x, const T* g, const float* mean, const float* rstd, T* dx, float* part,
                           int nblocks, T* dgamma, T* dbeta, long long rows, int C, cudaStream_t st, float* dgamma_acc = nullptr,
                           float* dbeta_acc = nullptr) {
  constexpr int VEC = 16 / sizeof(T);
  const bool aligned0 = (C % VEC == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) |
                                            reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(g)) % 16 == 0);
  const bool multi_row = IsBf16<T>::value && aligned0 && (C == 64 || C == 128 || C == 256);     // writes every partial itself
  if (!multi_row && cudaMemsetAsync(part, 0, sizeof(float) * 2 * C * nblocks, st) != cudaSuccess) return -1;
  const bool aligned = (C % VEC == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) |
                                           reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(g)) % 16 == 0);
  if (IsBf16<T>::value && aligned && (C == 64 || C == 128 || C == 256)) {
    const bf16 *db_ = reinterpret_cast<const bf16*>(dy), *xb = reinterpret_cast<const bf16*>(x), *gb = reinterpret_cast<const bf16*>(g);
    bf16* dxb = reinterpret_cast<bf16*>(dx);
    if (C == 64) launch_light(ln_bwd_mr_kernel<8>, nblocks, LN_WARPS * 32, 0, st, db_, xb, gb, mean, rstd, dxb, part, rows);
    else if (C == 128) launch_light(ln_bwd_mr_kernel<16>, nblocks, LN_WARPS * 32, 0, st, db_, xb, gb, mean, rstd, dxb, part, rows);
    else launch_light(ln_bwd_mr_kernel<32>, nblocks, LN_WARPS * 32, 0, st, db_, xb, gb, mean, rstd, dxb, part, rows);
  } else if (aligned && C <= 32 * VEC) launch_light(ln_bwd_kernel<T, VEC>, nblocks, LN_WARPS * 32, 0, st, dy, x, g, mean, rstd, dx, part, rows, C);
  else if (aligned && C <= 64 * VEC) launch_light(ln_bwd_kernel<T, 2 * VEC>, nblocks, LN_WARPS * 32, 0, st, dy, x, g, mean, rstd, dx, part, rows, C);
  else if (aligned && C <= 128 * VEC) launch_light(ln_bwd_kernel<T, 4 * VEC>, nblocks, LN_WARPS * 32, 0, st, dy, x, g, mean, rstd, dx, part, rows, C);
  else launch_light(ln_bwd_generic_kernel<T>, nblocks, LN_WARPS * 32, 0, st, dy, x, g, mean, rstd, dx, part, rows, C);
  if (dgamma_acc) launch_light(ln_bwd_reduce_acc_kernel, (2 * C + 31) / 32, 1024, 0, st, part, nblocks, C, dgamma_acc, dbeta_acc);
  else launch_light(ln_bwd_reduce_kernel<T>, (2 * C + 31) / 32, 1024, 0, st, part, nblocks, C, dgamma, dbeta);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace ffb

using namespace ffb;

extern "C" {

// dtype: 0 = fp32, 1 = fp16, 2 = bf16
int ffb_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, long long rows,
                      int C, float eps, int dtype, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (rows <= 0) return 0;
  switch (dtype) {
    case 0: return ln_fwd_dispatch<float>((const float*)x, (const float*)gamma, (const float*)beta, (float*)y, mean, rstd, rows, C, eps, st);
    case 1: return ln_fwd_dispatch<__half>((const __half*)x, (const __half*)gamma, (const __half*)beta, (__half*)y, mean, rstd, rows, C, eps, st);
    case 2: return ln_fwd_dispatch<bf16>((const bf16*)x, (const bf16*)gamma, (const bf16*)beta, (bf16*)y, mean, rstd, rows, C, eps, st);
  }
  return -2;
}

// part: fp32 workspace of 2 * C * nblocks floats (zeroed here).
int ffb_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                      float* part, int nblocks, void* dgamma, void* dbeta, long long rows, int C, int dtype, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (rows <= 0) return 0;
  switch (dtype) {
    case 0: return ln_bwd_dispatch<float>((const float*)dy, (const float*)x, (const float*)gamma, mean, rstd, (float*)dx, part, nblocks, (float*)dgamma, (float*)dbeta, rows, C, st);
    case 1: return ln_bwd_dispatch<__half>((const __half*)dy, (const __half*)x, (const __half*)gamma, mean, rstd, (__half*)dx, part, nblocks, (__half*)dgamma, (__half*)dbeta, rows, C, st);
    case 2: return ln_bwd_dispatch<bf16>((const bf16*)dy, (const bf16*)x, (const bf16*)gamma, mean, rstd, (bf16*)dx, part, nblocks, (bf16*)dgamma, (bf16*)dbeta, rows, C, st);
  }
  return -2;
}

// bf16 backward whose dgamma / dbeta are ADDED into fp32 vectors (a trainer's flat gradient buffer).
int ffb_layernorm_bwd_acc(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                          float* part, int nblocks, float* dgamma_acc, float* dbeta_acc, long long rows, int C, void* stream) {
  if (rows <= 0) return 0;
  if (!dgamma_acc || !dbeta_acc) return -2;
  return ln_bwd_dispatch<bf16>((const bf16*)dy, (const bf16*)x, (const bf16*)gamma, mean, rstd, (bf16*)dx, part, nblocks, nullptr, nullptr, rows,
                               C, reinterpret_cast<cudaStream_t>(stream), dgamma_acc, dbeta_acc);
}

// x: [C][rows] bf16 -> y: [rows][C] bf16, normalised over C (C <= 256).
int ffb_layernorm_fwd_transposed(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                                 long long rows, int C, float eps, void* stream) {
  if (C > 256) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (rows % 2 == 0 && C % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(gamma) |
                                       reinterpret_cast<uintptr_t>(beta)) & 15) == 0) {
    static bool attr = false;
    if (!attr) {
      if (cudaFuncSetAttribute(ln_fwd_transposed64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(float) * 256 * (LNT64 + 1))) !=
          cudaSuccess)
        return -3;
      attr = true;
    }
    const size_t smem64 = sizeof(float) * C * (LNT64 + 1);
    launch_light(ln_fwd_transposed64_kernel, (unsigned)((rows + LNT64 - 1) / LNT64), 256, smem64, st, (const bf16*)x, (const bf16*)gamma, (const bf16*)beta, (bf16*)y, mean, rstd, rows, C, eps);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
  }
  const size_t smem = sizeof(float) * C * (LNT_ROWS + 1);
  launch_light(ln_fwd_transposed_kernel, (unsigned)((rows + LNT_ROWS - 1) / LNT_ROWS), 256, smem, st, (const bf16*)x, (const bf16*)gamma, (const bf16*)beta, (bf16*)y, mean, rstd, rows, C, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free variant of the backward (see layernorm_noalloc.h).
// ---------------------------------------------------------------------------
#include <stdio.h>

#include "layernorm_noalloc.h"

// Partial dgamma / dbeta sums of FFB_LN_NOALLOC_BLOCKS blocks.  In host code this name is only a handle for
// cudaGetSymbolAddress - never a pointer to hand to a kernel.
static __device__ __align__(256) float g_ln_noalloc_scratch[FFB_LN_NOALLOC_BLOCKS * 2 * FFB_LN_NOALLOC_MAX_C];

// Device address of the array on each device of the process, resolved on first use with that device current.
static float* ln_noalloc_scratch_ptr() {
  static float* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_ln_noalloc_scratch) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<float*>(p);
  }
  return ptrs[dev];
}

extern "C" int ffb_layernorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                                         void* dgamma, void* dbeta, long long rows, int C, int dtype, void* stream) {
  if (C > FFB_LN_NOALLOC_MAX_C || C <= 0) {
    fprintf(stderr, "ffb_layernorm_bwd_noalloc: C = %d exceeds the built-in scratch capacity (C <= %d)\n", C, FFB_LN_NOALLOC_MAX_C);
    return FFB_LN_NOALLOC_TOO_WIDE;
  }
  if (rows <= 0) return 0;
  float* part = ln_noalloc_scratch_ptr();
  if (!part) return -1;
  long long want = (rows + LN_WARPS - 1) / LN_WARPS;
  const int nblocks = (int)(want < FFB_LN_NOALLOC_BLOCKS ? want : FFB_LN_NOALLOC_BLOCKS);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // ln_bwd_dispatch clears the 2 * C * nblocks floats it is about to accumulate into, on the same stream
  switch (dtype) {
    case 0: return ln_bwd_dispatch<float>((const float*)dy, (const float*)x, (const float*)gamma, mean, rstd, (float*)dx, part, nblocks, (float*)dgamma, (float*)dbeta, rows, C, st);
    case 1: return ln_bwd_dispatch<__half>((const __half*)dy, (const __half*)x, (const __half*)gamma, mean, rstd, (__half*)dx, part, nblocks, (__half*)dgamma, (__half*)dbeta, rows, C, st);
    case 2: return ln_bwd_dispatch<bf16>((const bf16*)dy, (const bf16*)x, (const bf16*)gamma, mean, rstd, (bf16*)dx, part, nblocks, (bf16*)dgamma, (bf16*)dbeta, rows, C, st);
  }
  return -2;
}
