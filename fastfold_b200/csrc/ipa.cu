// Invariant point attention core (AlphaFold Algorithm 22, lines 7-11) as one flash-style kernel.
//
// For every query residue i (one CTA per query row) the kernel streams the keys j in chunks and keeps, per head h,
// an online softmax over
//     logit[h][j] = w_C * q_i.k_j  +  sqrt(1/3) * (z[i][j] . W_b[h] + b_b[h])
//                   - 0.5 * gamma_h * sum_p |q_pt[i][h][p] - k_pt[j][h][p]|^2  +  inf * (mask_i * mask_j - 1)
// and the three weighted sums   o[h] = sum_j a v_j,   o_pt[h][p] = sum_j a v_pt[j][h][p] (global frame),
// o_pair[h] = sum_j a z[i][j].  The pair row z[i][:] is read ONCE from HBM (bf16) and serves both the bias projection
// and o_pair; the [H, N, N] attention tensor, the [N, N, H, P, 3] point differences and the [N, N, H] bias of the
// composite implementation never exist.  All arithmetic is fp32 (point terms must not lose the cancellation in
// |q - k|^2).  `row0` / `rows` select a block of query rows, so a rank that holds only its row shard of z computes its
// own residues (row-parallel IPA under Dynamic Axial Parallelism).
//
// Replaces the PyTorch composite of the reference (fastfold/model/nn/structure_module.py:383-505), which materialises
// all of the above through cuBLAS and elementwise kernels.
#include "common.cuh"

namespace ffb {

constexpr int IPA_THREADS = 256;
constexpr int IPA_J = 64;          // keys per chunk
constexpr int IPA_MAXH = 16;
constexpr int IPA_ZP = 8;          // padding (bf16) of a z row in shared memory: consecutive keys fall into different banks

struct IpaArgs {
  const float* q;       // [N][H][C]
  const float* k;       // [N][H][C]
  const float* v;       // [N][H][C]
  const float* q_pts;   // [N][H][Pq][3]
  const float* k_pts;   // [N][H][Pq][3]
  const float* v_pts;   // [N][H][Pv][3]
  const bf16* z;        // [rows][N][CZ]  (row r = query row0 + r)
  const float* wb;      // [H][CZ]
  const float* bb;      // [H]
  const float* gamma;   // [H]  softplus(head_weights) * sqrt(1 / (3 * Pq * 9 / 2))
  const float* mask;    // [N]
  float* o;             // [rows][H][C]
  float* o_pt;          // [rows][H][Pv][3]
  float* o_pair;        // [rows][H][CZ]
  int N, H, C, Pq, Pv, CZ, row0, rows;
  float w_c, w_b, inf;
};

template <int H, int C, int PQ, int PV, int CZ>
__global__ void __launch_bounds__(IPA_THREADS) ipa_fwd_kernel(const IpaArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int ZROW = CZ + IPA_ZP;
  constexpr int VC = C + 3 * PV;                 // value channels per head that do not come from z
  extern __shared__ uint8_t ipa_smem[];
  bf16* zs = reinterpret_cast<bf16*>(ipa_smem);                                  // [J][ZROW]
  float* wbt = reinterpret_cast<float*>(ipa_smem + IPA_J * ZROW * 2);            // [CZ][H + 1]  (transposed, padded)
  float* qs = wbt + CZ * (H + 1);                                                // [H][C]
  float* qp = qs + H * C;                                                        // [H][PQ * 3]
  float* ps = qp + H * PQ * 3;                                                   // [H][J]  logits, then probabilities
  float* mrun = ps + H * IPA_J;                                                  // [H] running max
  float* lrun = mrun + H;                                                        // [H] running sum
  float* alph = lrun + H;                                                        // [H] rescale factor of this chunk
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = blockIdx.x;
  if (r >= a.rows) return;
  const int i = a.row0 + r;
  const int N = a.N;
  for (int t = tid; t < H * CZ; t += IPA_THREADS) {
    const int h = t / CZ, c = t - h * CZ;
    wbt[c * (H + 1) + h] = a.wb[t];
  }
  for (int t = tid; t < H * C; t += IPA_THREADS) qs[t] = a.q[(long long)i * H * C + t];
  for (int t = tid; t < H * PQ * 3; t += IPA_THREADS) qp[t] = a.q_pts[(long long)i * H * PQ * 3 + t];
  if (tid < H) {
    mrun[tid] = -INFINITY;
    lrun[tid] = 0.f;
  }
  const float mask_i = a.mask ? a.mask[i] : 1.f;
  // accumulators: threads [0, CZ) own pair channel `tid` for every head; threads [CZ, 256) own the scalar / point channels
  float acc_z[H];
#pragma unroll
  for (int h = 0; h < H; ++h) acc_z[h] = 0.f;
  constexpr int NV_T = IPA_THREADS - CZ;                      // threads on the value channels
  constexpr int NVA = (H * VC + NV_T - 1) / NV_T;             // accumulators per such thread
  float acc_v[NVA];
#pragma unroll
  for (int u = 0; u < NVA; ++u) acc_v[u] = 0.f;
  const bf16* zrow = a.z + (long long)r * N * CZ;
  __syncthreads();

  for (int j0 = 0; j0 < N; j0 += IPA_J) {
    const int jn = (N - j0) < IPA_J ? (N - j0) : IPA_J;
    // ---- stage the chunk of the pair row: [jn][CZ] bf16, 16-byte loads ----
    for (int t = tid; t < IPA_J * (CZ / 8); t += IPA_THREADS) {
      const int j = t / (CZ / 8), c8 = t - j * (CZ / 8);
      uint4 val = make_uint4(0, 0, 0, 0);
      if (j < jn) val = *reinterpret_cast<const uint4*>(zrow + (long long)(j0 + j) * CZ + c8 * 8);
      *reinterpret_cast<uint2*>(zs + j * ZROW + c8 * 8) = make_uint2(val.x, val.y);
      *reinterpret_cast<uint2*>(zs + j * ZROW + c8 * 8 + 4) = make_uint2(val.z, val.w);
    }
    __syncthreads();
    // ---- logits: one (key, head) pair per thread and step ----
    for (int t = tid; t < IPA_J * H; t += IPA_THREADS) {
      const int j = t / H, h = t - j * H;
      float logit = -INFINITY;
      if (j < jn) {
        const int jj = j0 + j;
        const float4* kp = reinterpret_cast<const float4*>(a.k + ((long long)jj * H + h) * C);
        float qk = 0.f;
#pragma unroll
        for (int c = 0; c < C / 4; ++c) {
          const float4 kv = kp[c];
          qk += qs[h * C + 4 * c] * kv.x + qs[h * C + 4 * c + 1] * kv.y + qs[h * C + 4 * c + 2] * kv.z + qs[h * C + 4 * c + 3] * kv.w;
        }
        const float* kpt = a.k_pts + ((long long)jj * H + h) * PQ * 3;
        float d2 = 0.f;
#pragma unroll
        for (int p = 0; p < PQ * 3; ++p) {
          const float d = qp[h * PQ * 3 + p] - kpt[p];
          d2 += d * d;
        }
        float bz = a.bb[h];
        const bf16* zr = zs + j * ZROW;
#pragma unroll 8
        for (int c = 0; c < CZ; c += 2) {
          const float2 zf = __bfloat1622float2(*reinterpret_cast<const bf162*>(zr + c));
          bz += zf.x * wbt[c * (H + 1) + h] + zf.y * wbt[(c + 1) * (H + 1) + h];
        }
        const float mj = a.mask ? a.mask[jj] : 1.f;
        logit = a.w_c * qk + a.w_b * bz - 0.5f * a.gamma[h] * d2 + a.inf * (mask_i * mj - 1.f);
      }
      ps[h * IPA_J + j] = logit;
    }
    __syncthreads();
    // ---- online softmax: warp w handles heads w, w + 8, ... ----
    for (int h = warp; h < H; h += IPA_THREADS / 32) {
      const float s0 = ps[h * IPA_J + lane], s1 = ps[h * IPA_J + 32 + lane];
      const float mold = mrun[h];
      const float mnew = fmaxf(mold, warp_max(fmaxf(s0, s1)));
      const float p0 = __expf(s0 - mnew), p1 = __expf(s1 - mnew);      // -inf logits (beyond N) give 0
      ps[h * IPA_J + lane] = p0;
      ps[h * IPA_J + 32 + lane] = p1;
      const float sum = warp_sum(p0 + p1);
      if (lane == 0) {
        const float al = __expf(mold - mnew);                            // 0 on the first chunk (mold = -inf)
        alph[h] = al;
        mrun[h] = mnew;
        lrun[h] = lrun[h] * al + sum;
      }
    }
    __syncthreads();
    // ---- weighted sums ----
    if (tid < CZ) {
#pragma unroll
      for (int h = 0; h < H; ++h) acc_z[h] *= alph[h];
      for (int j = 0; j < IPA_J; j += 4) {
        const float z0 = __bfloat162float(zs[(j + 0) * ZROW + tid]), z1 = __bfloat162float(zs[(j + 1) * ZROW + tid]);
        const float z2 = __bfloat162float(zs[(j + 2) * ZROW + tid]), z3 = __bfloat162float(zs[(j + 3) * ZROW + tid]);
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const float4 p = *reinterpret_cast<const float4*>(ps + h * IPA_J + j);     // same address in every lane
          acc_z[h] += p.x * z0 + p.y * z1 + p.z * z2 + p.w * z3;
        }
      }
    } else {
      const int u0 = tid - CZ;
#pragma unroll
      for (int u = 0; u < NVA; ++u) {
        const int ch = u0 + u * NV_T;
        if (ch < H * VC) {
          const int h = ch / VC, c = ch - h * VC;
          const float* base = c < C ? a.v + (long long)h * C + c : a.v_pts + (long long)h * PV * 3 + (c - C);
          const long long jstride = c < C ? (long long)H * C : (long long)H * PV * 3;
          float acc = acc_v[u] * alph[h];
          for (int j = 0; j < jn; ++j) acc += ps[h * IPA_J + j] * base[(long long)(j0 + j) * jstride];
          acc_v[u] = acc;
        }
      }
    }
    __syncthreads();
  }
  // ---- normalise and store ----
  if (tid < CZ) {
#pragma unroll
    for (int h = 0; h < H; ++h) a.o_pair[((long long)r * H + h) * CZ + tid] = acc_z[h] / lrun[h];
  } else {
    const int u0 = tid - CZ;
#pragma unroll
    for (int u = 0; u < NVA; ++u) {
      const int ch = u0 + u * NV_T;
      if (ch < H * VC) {
        const int h = ch / VC, c = ch - h * VC;
        const float val = acc_v[u] / lrun[h];
        if (c < C) a.o[((long long)r * H + h) * C + c] = val;
        else a.o_pt[((long long)r * H + h) * PV * 3 + (c - C)] = val;
      }
    }
  }
}

}  // namespace ffb

using namespace ffb;

extern "C" {

// All pointers are device memory; q / k / v / points / weights / outputs fp32, z bf16 (layouts in IpaArgs).
// Supported configuration: H = 12 heads, C = 16 channels, 4 query / key points, 8 value points, c_z = 128 (AlphaFold's
// structure module); anything else returns -2 and the caller uses its PyTorch composite.
int ffb_ipa_fwd(const float* q, const float* k, const float* v, const float* q_pts, const float* k_pts, const float* v_pts, const void* z,
                const float* wb, const float* bb, const float* gamma, const float* mask, float* o, float* o_pt, float* o_pair, int N, int H,
                int C, int Pq, int Pv, int CZ, int row0, int rows, float w_c, float w_b, float inf, void* stream) {
  if (H != 12 || C != 16 || Pq != 4 || Pv != 8 || CZ != 128) return -2;
  if (rows <= 0) return 0;
  if (N <= 0 || row0 < 0 || row0 + rows > N || (reinterpret_cast<uintptr_t>(z) & 15) || (reinterpret_cast<uintptr_t>(k) & 15)) return -3;
  IpaArgs a;
  a.q = q; a.k = k; a.v = v; a.q_pts = q_pts; a.k_pts = k_pts; a.v_pts = v_pts;
  a.z = reinterpret_cast<const bf16*>(z);
  a.wb = wb; a.bb = bb; a.gamma = gamma; a.mask = mask;
  a.o = o; a.o_pt = o_pt; a.o_pair = o_pair;
  a.N = N; a.H = H; a.C = C; a.Pq = Pq; a.Pv = Pv; a.CZ = CZ; a.row0 = row0; a.rows = rows;
  a.w_c = w_c; a.w_b = w_b; a.inf = inf;
  constexpr int HH = 12, CC = 16, PQ = 4, PV = 8, CZZ = 128;
  const size_t smem = IPA_J * (CZZ + IPA_ZP) * 2 + sizeof(float) * (CZZ * (HH + 1) + HH * CC + HH * PQ * 3 + HH * IPA_J + 3 * HH);
  launch_light(ipa_fwd_kernel<HH, CC, PQ, PV, CZZ>, rows, IPA_THREADS, smem, reinterpret_cast<cudaStream_t>(stream), a);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
