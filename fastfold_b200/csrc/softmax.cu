// Row softmax with optional key mask and optional broadcast pair bias, forward
// and backward, bf16 / fp16 / fp32 storage with fp32 math.
//
//   y[b1,b2,h,q,:] = softmax( where(mask[b1,b2,:] == 0, -1e9, x[b1,b2,h,q,:] + bias[b1,0,h,q,:]) )
//
// One warp per row; rows up to 1024 keys live in registers (template on the
// number of keys per lane), longer rows use the looped kernel which re-reads
// the row from L2.  The mask row is found from (b1, b2), not from
// row / (H * K): logits need not be square, so the global-attention shape
// [b1, b2, H, 1, S] indexes its mask correctly.  The backward kernel
// (dx = (dy - sum(y * dy)) * y) has the same two paths, so rows longer than
// 1024 are differentiated correctly as well.
//
// Replaces fastfold/model/fastnn/kernel/cuda_native/csrc/softmax_cuda_kernel.cu
// (:84-161 plain, :338-522 masked, :618-810 masked + bias, :252-334 and
// :524-614 gradients) and kernel/triton/softmax.py.
#include "common.cuh"

namespace ffb {

constexpr int SM_WARPS = 4;
constexpr float MASK_FILL = -1e9f;

struct SoftmaxShape {
  long long rows;     // B1 * B2 * H * Q
  int K;
  long long hq;       // H * Q           (rows per (b1, b2))
  long long b2hq;     // B2 * H * Q      (rows per b1)
};

template <typename T, int CPT>
__global__ void __launch_bounds__(SM_WARPS * 32) softmax_fwd_kernel(const T* __restrict__ x, const T* __restrict__ mask,
                                                                   const T* __restrict__ bias, T* __restrict__ y, SoftmaxShape s) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * SM_WARPS + (threadIdx.x >> 5);
  if (row >= s.rows) return;
  const T* xr = x + row * s.K;
  const T* mr = mask ? mask + (row / s.hq) * s.K : nullptr;
  const T* br = bias ? bias + ((row / s.b2hq) * s.hq + row % s.hq) * s.K : nullptr;
  float v[CPT];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    const int k = i * 32 + lane;
    if (k < s.K) {
      float t = to_f<T>(xr[k]);
      if (br) t += to_f<T>(br[k]);
      if (mr && to_f<T>(mr[k]) == 0.f) t = MASK_FILL;
      v[i] = t;
      mx = fmaxf(mx, t);
    } else {
      v[i] = -INFINITY;
    }
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    v[i] = __expf(v[i] - mx);
    sum += v[i];
  }
  const float inv = 1.f / warp_sum(sum);
  T* yr = y + row * s.K;
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    const int k = i * 32 + lane;
    if (k < s.K) yr[k] = from_f<T>(v[i] * inv);
  }
}

template <typename T>
__global__ void __launch_bounds__(SM_WARPS * 32) softmax_fwd_loop_kernel(const T* __restrict__ x, const T* __restrict__ mask,
                                                                        const T* __restrict__ bias, T* __restrict__ y, SoftmaxShape s) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * SM_WARPS + (threadIdx.x >> 5);
  if (row >= s.rows) return;
  const T* xr = x + row * s.K;
  const T* mr = mask ? mask + (row / s.hq) * s.K : nullptr;
  const T* br = bias ? bias + ((row / s.b2hq) * s.hq + row % s.hq) * s.K : nullptr;
  auto logit = [&](int k) {
    float t = to_f<T>(xr[k]);
    if (br) t += to_f<T>(br[k]);
    if (mr && to_f<T>(mr[k]) == 0.f) t = MASK_FILL;
    return t;
  };
  float mx = -INFINITY;
  for (int k = lane; k < s.K; k += 32) mx = fmaxf(mx, logit(k));
  mx = warp_max(mx);
  float sum = 0.f;
  for (int k = lane; k < s.K; k += 32) sum += __expf(logit(k) - mx);
  const float inv = 1.f / warp_sum(sum);
  T* yr = y + row * s.K;
  for (int k = lane; k < s.K; k += 32) yr[k] = from_f<T>(__expf(logit(k) - mx) * inv);
}

template <typename T, int CPT>
__global__ void __launch_bounds__(SM_WARPS * 32) softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                                                   T* __restrict__ dx, long long rows, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * SM_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  float yv[CPT], dv[CPT];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    const int k = i * 32 + lane;
    if (k < K) {
      yv[i] = to_f<T>(y[row * K + k]);
      dv[i] = to_f<T>(dy[row * K + k]);
      dot += yv[i] * dv[i];
    } else {
      yv[i] = dv[i] = 0.f;
    }
  }
  dot = warp_sum(dot);
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
    const int k = i * 32 + lane;
    if (k < K) dx[row * K + k] = from_f<T>((dv[i] - dot) * yv[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(SM_WARPS * 32) softmax_bwd_loop_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                                                        T* __restrict__ dx, long long rows, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * SM_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  float dot = 0.f;
  for (int k = lane; k < K; k += 32) dot += to_f<T>(y[row * K + k]) * to_f<T>(dy[row * K + k]);
  dot = warp_sum(dot);
  for (int k = lane; k < K; k += 32) dx[row * K + k] = from_f<T>((to_f<T>(dy[row * K + k]) - dot) * to_f<T>(y[row * K + k]));
}

template <typename T>
static int softmax_fwd_t(const T* x, const T* mask, const T* bias, T* y, SoftmaxShape s, cudaStream_t st) {
  const unsigned grid = (unsigned)((s.rows + SM_WARPS - 1) / SM_WARPS);
  const int cpt = (s.K + 31) / 32;
#define FFB_SM_CASE(N)                                                                 \
  if (cpt <= N) {                                                                      \
    launch_light(softmax_fwd_kernel<T, N>, grid, SM_WARPS * 32, 0, st, x, mask, bias, y, s);     \
    return cudaGetLastError() == cudaSuccess ? 0 : -1;                                 \
  }
  FFB_SM_CASE(1) FFB_SM_CASE(2) FFB_SM_CASE(4) FFB_SM_CASE(8) FFB_SM_CASE(16) FFB_SM_CASE(32)
#undef FFB_SM_CASE
  launch_light(softmax_fwd_loop_kernel<T>, grid, SM_WARPS * 32, 0, st, x, mask, bias, y, s);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

template <typename T>
static int softmax_bwd_t(const T* dy, const T* y, T* dx, long long rows, int K, cudaStream_t st) {
  const unsigned grid = (unsigned)((rows + SM_WARPS - 1) / SM_WARPS);
  const int cpt = (K + 31) / 32;
#define FFB_SM_CASE(N)                                                                 \
  if (cpt <= N) {                                                                      \
    launch_light(softmax_bwd_kernel<T, N>, grid, SM_WARPS * 32, 0, st, dy, y, dx, rows, K);      \
    return cudaGetLastError() == cudaSuccess ? 0 : -1;                                 \
  }
  FFB_SM_CASE(1) FFB_SM_CASE(2) FFB_SM_CASE(4) FFB_SM_CASE(8) FFB_SM_CASE(16) FFB_SM_CASE(32)
#undef FFB_SM_CASE
  launch_light(softmax_bwd_loop_kernel<T>, grid, SM_WARPS * 32, 0, st, dy, y, dx, rows, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace ffb

using namespace ffb;

extern "C" {

// x, y: [B1][B2][H][Q][K]; mask: [B1][B2][K] or null; bias: [B1][H][Q][K] or null.
// dtype: 0 = fp32, 1 = fp16, 2 = bf16.
int ffb_softmax_fwd(const void* x, const void* mask, const void* bias, void* y, long long B1, long long B2, long long H,
                    long long Q, int K, int dtype, void* stream) {
  SoftmaxShape s;
  s.rows = B1 * B2 * H * Q;
  s.K = K;
  s.hq = H * Q;
  s.b2hq = B2 * H * Q;
  if (s.rows <= 0 || K <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case 0: return softmax_fwd_t<float>((const float*)x, (const float*)mask, (const float*)bias, (float*)y, s, st);
    case 1: return softmax_fwd_t<__half>((const __half*)x, (const __half*)mask, (const __half*)bias, (__half*)y, s, st);
    case 2: return softmax_fwd_t<bf16>((const bf16*)x, (const bf16*)mask, (const bf16*)bias, (bf16*)y, s, st);
  }
  return -2;
}

int ffb_softmax_bwd(const void* dy, const void* y, void* dx, long long rows, int K, int dtype, void* stream) {
  if (rows <= 0 || K <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case 0: return softmax_bwd_t<float>((const float*)dy, (const float*)y, (float*)dx, rows, K, st);
    case 1: return softmax_bwd_t<__half>((const __half*)dy, (const __half*)y, (__half*)dx, rows, K, st);
    case 2: return softmax_bwd_t<bf16>((const bf16*)dy, (const bf16*)y, (bf16*)dx, rows, K, st);
  }
  return -2;
}

}  // extern "C"
