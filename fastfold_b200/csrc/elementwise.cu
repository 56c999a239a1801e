// Fused elementwise regions of the Evoformer (bf16 storage, fp32 math), each
// with its backward:
//
//   bias_sigmoid_mul        y = sigmoid(g + b) * o                      attention gate
//   bias_dropout_add        y = r + (x + b) * m                         row / column attention output
//   bias_ele_dropout_res    y = r + m * (g * (ab + b))                  triangle multiplication output
//   glu_mask                y = rowmask * p * sigmoid(q)                triangle multiplication projections
//   act_bwd                 relu / sigmoid derivative applied to dy
//   colsum                  fp32 column sums (bias gradients)
//
// The dropout mask m is shared along one axis of the activation, so it is a
// small [mod, C] tensor indexed by (row / div) % mod; it already contains the
// 1/(1-p) scale.  All kernels move 16 bytes per thread per tensor; C must be a
// multiple of 8 and pointers 16-byte aligned (the Python wrappers route other
// shapes to a composite implementation).
//
// These are the reference's TorchScript fusions
// (fastfold/model/fastnn/kernel/jit/fused_ops.py:5-22) written as explicit
// kernels together with their gradients, which the reference leaves to
// autograd over the unfused ops.
#include "common.cuh"

namespace ffb {

struct V8 {
  float v[8];
};
__device__ __forceinline__ V8 ld8(const bf16* p) {
  V8 r;
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    r.v[2 * i] = f.x;
    r.v[2 * i + 1] = f.y;
  }
  return r;
}
__device__ __forceinline__ void st8(bf16* p, const V8& r) {
  uint4 u;
  bf162* h = reinterpret_cast<bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(r.v[2 * i], r.v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

#define FFB_EW_INDEX                                                          \
  const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x);  \
  const int cv = C >> 3;                                                      \
  const long long row = idx / cv;                                             \
  if (row >= rows) return;                                                    \
  const int c = (int)(idx - row * cv) << 3;                                   \
  const long long off = row * C + c;

__global__ void bias_sigmoid_mul_fwd_k(const bf16* g, const bf16* b, const bf16* o, bf16* y, long long rows, int C) {
  pdl_launch_dependents();
  pdl_wait();
  FFB_EW_INDEX
  V8 gv = ld8(g + off), bv = ld8(b + c), ov = ld8(o + off), r;
#pragma unroll
  for (int i = 0; i < 8; ++i) r.v[i] = sigmoidf_(gv.v[i] + bv.v[i]) * ov.v[i];
  st8(y + off, r);
}

__global__ void bias_sigmoid_mul_bwd_k(const bf16* dy, const bf16* g, const bf16* b, const bf16* o, bf16* dg, bf16* dob,
                                       long long rows, int C) {
  pdl_launch_dependents();
  pdl_wait();
  FFB_EW_INDEX
  V8 d = ld8(dy + off), gv = ld8(g + off), bv = ld8(b + c), ov = ld8(o + off), r1, r2;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float s = sigmoidf_(gv.v[i] + bv.v[i]);
    r1.v[i] = d.v[i] * ov.v[i] * s * (1.f - s);
    r2.v[i] = d.v[i] * s;
  }
  st8(dg + off, r1);
  st8(dob + off, r2);
}

__global__ void bias_dropout_add_fwd_k(const bf16* x, const bf16* b, const bf16* m, const bf16* r, bf16* y, long long rows,
                                       int C, int div, int mod) {
  pdl_launch_dependents();
  pdl_wait();
  FFB_EW_INDEX
  V8 xv = ld8(x + off), rv = ld8(r + off), o;
  V8 bv, mv;
#pragma unroll
  for (int i = 0; i < 8; ++i) bv.v[i] = 0.f, mv.v[i] = 1.f;
  if (b) bv = ld8(b + c);
  if (m) mv = ld8(m + (long long)((row / div) % mod) * C + c);
#pragma unroll
  for (int i = 0; i < 8; ++i) o.v[i] = rv.v[i] + (xv.v[i] + bv.v[i]) * mv.v[i];
  st8(y + off, o);
}

// dx = dy * m
__global__ void mask_mul_k(const bf16* dy, const bf16* m, bf16* dx, long long rows, int C, int div, int mod) {
  pdl_launch_dependents();
  pdl_wait();
  FFB_EW_INDEX
  V8 d = ld8(dy + off), mv = ld8(m + (long long)((row / div) % mod) * C + c), o;
#pragma unroll
  for (int i = 0; i < 8; ++i) o.v[i] = d.v[i] * mv.v[i];
  st8(dx + off, o);
}

__global__ void bias_ele_dropout_res_fwd_k(const bf16* ab, const bf16* b, const bf16* g, const bf16* m, const bf16* r, bf16* y,
                                           long long rows, int C, int div, int mod) {
  pdl_launch_dependents();
  pdl_wait();
  FFB_EW_INDEX
  V8 av = ld8(ab + off), bv = ld8(b + c), gv = ld8(g + off), rv = ld8(r + off), mv, o;
#pragma unroll
  for (int i = 0; i < 8; ++i) mv.v[i] = 1.f;
  if (m) mv = ld8(m + (long long)((row / div) % mod) * C + c);
#pragma unroll
  for (int i = 0; i < 8; ++i) o.v[i] = rv.v[i] + mv.v[i] * (gv.v[i] * (av.v[i] + bv.v[i]));
  st8(y + off, o);
}

__global__ void bias_ele_dropout_res_bwd_k(const bf16* dy, const bf16* ab, const bf16* b, const bf16* g, const bf16* m,
                                           bf16* dab, bf16* dg, long long rows, int C, int div, int mod) {
  pdl_launch_dependents();
  pdl_wait();
  FFB_EW_INDEX
  V8 d = ld8(dy + off), av = ld8(ab + off), bv = ld8(b + c), gv = ld8(g + off), mv, o1, o2;
#pragma unroll
  for (int i = 0; i < 8; ++i) mv.v[i] = 1.f;
  if (m) mv = ld8(m + (long long)((row / div) % mod) * C + c);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float t = d.v[i] * mv.v[i];
    o1.v[i] = t * gv.v[i];
    o2.v[i] = t * (av.v[i] + bv.v[i]);
  }
  st8(dab + off, o1);
  st8(dg + off, o2);
}

// y = rowmask[row] * p * sigmoid(q); p, q, y: [rows, C]
__global__ void glu_mask_fwd_k(const bf16* p, const bf16* q, const bf16* rowmask, bf16* y, long long rows, int C) {
  pdl_launch_dependents();
  pdl_wait();
  FFB_EW_INDEX
  V8 pv = ld8(p + off), qv = ld8(q + off), o;
  const float mk = rowmask ? __bfloat162float(rowmask[row]) : 1.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) o.v[i] = mk * pv.v[i] * sigmoidf_(qv.v[i]);
  st8(y + off, o);
}

__global__ void glu_mask_bwd_k(const bf16* dy, const bf16* p, const bf16* q, const bf16* rowmask, bf16* dp, bf16* dq,
                               long long rows, int C) {
  pdl_launch_dependents();
  pdl_wait();
  FFB_EW_INDEX
  V8 d = ld8(dy + off), pv = ld8(p + off), qv = ld8(q + off), o1, o2;
  const float mk = rowmask ? __bfloat162float(rowmask[row]) : 1.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float s = sigmoidf_(qv.v[i]);
    const float t = d.v[i] * mk;
    o1.v[i] = t * s;
    o2.v[i] = t * pv.v[i] * s * (1.f - s);
  }
  st8(dp + off, o1);
  st8(dq + off, o2);
}

// mode 1: relu (dx = dy where y > 0), mode 2: sigmoid (dx = dy * y * (1 - y))
__global__ void act_bwd_k(const bf16* dy, const bf16* y, bf16* dx, long long rows, int C, int mode) {
  pdl_launch_dependents();
  pdl_wait();
  FFB_EW_INDEX
  V8 d = ld8(dy + off), yv = ld8(y + off), o;
#pragma unroll
  for (int i = 0; i < 8; ++i) o.v[i] = mode == 1 ? (yv.v[i] > 0.f ? d.v[i] : 0.f) : d.v[i] * yv.v[i] * (1.f - yv.v[i]);
  st8(dx + off, o);
}

// out[c] += sum_rows x[row][c]; grid = (ceil(C/256), nchunks); fp32 atomics.
__global__ void colsum_k(const bf16* x, float* out, long long rows, int C, long long rows_per_block) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= C) return;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block;
  if (r1 > rows) r1 = rows;
  float s0 = 0.f, s1 = 0.f;
  for (long long r = r0; r < r1; ++r) {
    float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(x + r * C + c));
    s0 += f.x;
    s1 += f.y;
  }
  atomicAdd(out + c, s0);
  atomicAdd(out + c + 1, s1);
}

// Same sums for C % 8 == 0, C <= 2048 with 16-byte loads: a block of 256 threads is (C/8 column groups) x (row lanes);
// every thread keeps 8 running sums over its rows (4 independent loads in flight), the row lanes are folded through
// shared memory and one thread per column adds the block's result to `out`.
__global__ void __launch_bounds__(256) colsum_v8_k(const bf16* __restrict__ x, float* __restrict__ out, long long rows, int C,
                                                   long long rows_per_block) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float red[];                 // [row lanes][C]
  const int groups = C >> 3;                     // column groups of 8
  const int lanes = 256 / groups;                // row lanes per block (groups <= 256)
  const int gidx = threadIdx.x % groups, lane = threadIdx.x / groups;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (lane < lanes) {
    const long long r0 = (long long)blockIdx.x * rows_per_block;
    long long r1 = r0 + rows_per_block;
    if (r1 > rows) r1 = rows;
    const bf16* p = x + gidx * 8;
    long long r = r0 + lane;
    for (; r + 3LL * lanes < r1; r += 4LL * lanes) {
      uint4 u[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) u[k] = *reinterpret_cast<const uint4*>(p + (r + (long long)k * lanes) * C);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const bf162* h = reinterpret_cast<const bf162*>(&u[k]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
    }
    for (; r < r1; r += lanes) {
      const uint4 u = *reinterpret_cast<const uint4*>(p + r * C);
      const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) red[lane * C + gidx * 8 + j] = acc[j];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += 256) {
    float t = 0.f;
    for (int l = 0; l < lanes; ++l) t += red[l * C + c];
    atomicAdd(out + c, t);
  }
}

// Adam on flat buffers: fp32 master weights and moments, bf16 gradients (already
// reduced over ranks), bf16 working copy refreshed in the same pass.  The step
// dependent scalars (learning rate, bias corrections) are read from device
// memory so that a captured CUDA graph can be replayed with new values.
//   hp[0] = lr, hp[1] = 1 - beta1^t, hp[2] = 1 - beta2^t, hp[3] = gradient scale
__global__ void adam_k(float* w, float* m, float* v, const bf16* grad, bf16* w16, long long n, const float* hp, float b1,
                       float b2, float eps, float wd) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float lr = hp[0], bc1 = hp[1], bc2 = hp[2], gscale = hp[3];
  float gg = __bfloat162float(grad[i]) * gscale;
  float ww = w[i];
  if (wd != 0.f) gg += wd * ww;
  const float mm = b1 * m[i] + (1.f - b1) * gg;
  const float vv = b2 * v[i] + (1.f - b2) * gg * gg;
  m[i] = mm;
  v[i] = vv;
  ww -= lr * (mm / bc1) / (sqrtf(vv / bc2) + eps);
  w[i] = ww;
  w16[i] = __float2bfloat16(ww);
}

}  // namespace ffb

using namespace ffb;

#define FFB_EW_LAUNCH(kern, ...)                                                        \
  do {                                                                                  \
    if (rows <= 0) return 0;                                                            \
    if (C % 8) return -2;                                                               \
    const long long n = rows * (C / 8);                                                 \
    launch_light(kern, (unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream), __VA_ARGS__); \
    return cudaGetLastError() == cudaSuccess ? 0 : -1;                                  \
  } while (0)

extern "C" {

int ffb_bias_sigmoid_mul_fwd(const void* g, const void* b, const void* o, void* y, long long rows, int C, void* stream) {
  FFB_EW_LAUNCH(bias_sigmoid_mul_fwd_k, (const bf16*)g, (const bf16*)b, (const bf16*)o, (bf16*)y, rows, C);
}
int ffb_bias_sigmoid_mul_bwd(const void* dy, const void* g, const void* b, const void* o, void* dg, void* dob, long long rows,
                             int C, void* stream) {
  FFB_EW_LAUNCH(bias_sigmoid_mul_bwd_k, (const bf16*)dy, (const bf16*)g, (const bf16*)b, (const bf16*)o, (bf16*)dg, (bf16*)dob, rows, C);
}
int ffb_bias_dropout_add_fwd(const void* x, const void* b, const void* m, const void* r, void* y, long long rows, int C, int div,
                             int mod, void* stream) {
  FFB_EW_LAUNCH(bias_dropout_add_fwd_k, (const bf16*)x, (const bf16*)b, (const bf16*)m, (const bf16*)r, (bf16*)y, rows, C, div, mod);
}
int ffb_mask_mul(const void* dy, const void* m, void* dx, long long rows, int C, int div, int mod, void* stream) {
  FFB_EW_LAUNCH(mask_mul_k, (const bf16*)dy, (const bf16*)m, (bf16*)dx, rows, C, div, mod);
}
int ffb_bias_ele_dropout_res_fwd(const void* ab, const void* b, const void* g, const void* m, const void* r, void* y,
                                 long long rows, int C, int div, int mod, void* stream) {
  FFB_EW_LAUNCH(bias_ele_dropout_res_fwd_k, (const bf16*)ab, (const bf16*)b, (const bf16*)g, (const bf16*)m, (const bf16*)r, (bf16*)y, rows, C, div, mod);
}
int ffb_bias_ele_dropout_res_bwd(const void* dy, const void* ab, const void* b, const void* g, const void* m, void* dab, void* dg,
                                 long long rows, int C, int div, int mod, void* stream) {
  FFB_EW_LAUNCH(bias_ele_dropout_res_bwd_k, (const bf16*)dy, (const bf16*)ab, (const bf16*)b, (const bf16*)g, (const bf16*)m, (bf16*)dab, (bf16*)dg, rows, C, div, mod);
}
int ffb_glu_mask_fwd(const void* p, const void* q, const void* rowmask, void* y, long long rows, int C, void* stream) {
  FFB_EW_LAUNCH(glu_mask_fwd_k, (const bf16*)p, (const bf16*)q, (const bf16*)rowmask, (bf16*)y, rows, C);
}
int ffb_glu_mask_bwd(const void* dy, const void* p, const void* q, const void* rowmask, void* dp, void* dq, long long rows, int C,
                     void* stream) {
  FFB_EW_LAUNCH(glu_mask_bwd_k, (const bf16*)dy, (const bf16*)p, (const bf16*)q, (const bf16*)rowmask, (bf16*)dp, (bf16*)dq, rows, C);
}
int ffb_act_bwd(const void* dy, const void* y, void* dx, long long rows, int C, int mode, void* stream) {
  FFB_EW_LAUNCH(act_bwd_k, (const bf16*)dy, (const bf16*)y, (bf16*)dx, rows, C, mode);
}

// out (fp32 [C]) must be zeroed by the caller (or hold a running sum).
int ffb_colsum(const void* x, float* out, long long rows, int C, void* stream) {
  if (rows <= 0) return 0;
  if (C % 2) return -2;
  if (C % 8 == 0 && C <= 2048 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int groups = C / 8, lanes = 256 / groups;
    long long blocks = (rows + (long long)lanes * 8 - 1) / ((long long)lanes * 8);
    if (blocks > 592) blocks = 592;
    if (blocks < 1) blocks = 1;
    const long long rpb = (rows + blocks - 1) / blocks;
    const size_t smem = sizeof(float) * lanes * C;          // = 8 KB
    launch_light(colsum_v8_k, (unsigned)((rows + rpb - 1) / rpb), 256, smem, reinterpret_cast<cudaStream_t>(stream), (const bf16*)x, out, rows, C, rpb);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
  }
  long long chunks = (rows + 255) / 256;
  if (chunks > 512) chunks = 512;
  const long long rpb = (rows + chunks - 1) / chunks;
  dim3 grid((C / 2 + 127) / 128, (unsigned)((rows + rpb - 1) / rpb));
  launch_light(colsum_k, grid, 128, 0, reinterpret_cast<cudaStream_t>(stream), (const bf16*)x, out, rows, C, rpb);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int ffb_adam(float* w, float* m, float* v, const void* grad, void* w16, long long n, const float* hp, float b1, float b2,
             float eps, float wd, void* stream) {
  if (n <= 0) return 0;
  launch_light(adam_k, (unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream), w, m, v, (const bf16*)grad, (bf16*)w16, n, hp,
                                                                                          b1, b2, eps, wd);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
