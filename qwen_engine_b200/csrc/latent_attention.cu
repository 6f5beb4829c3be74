// Attention over a latent cache: every token keeps one normed latent of R channels and one rotated key part of
// Dr channels that all heads share; keys and values of a head are projections of the latent.  With W_uk (per
// head, [dn, R]) folded into the query and W_uv (per head, [dv, R]) applied after the softmax,
//
//   score_h(i, j) = scale * ((W_uk_h^T q_plain_h,i) . c_j + q_rot_h,i . k_rot_j)
//   o_h,i = W_uv_h (sum_j p_h(i, j) c_j)
//
// this is attention with ONE key/value head of R + Dr channels whose values are the keys' first R channels: the
// paged kernels run it on a cache of one plane per page.  Here are the two kernels around them:
//
//   qe_latent_prepare   per token: RMS norm of the latent and rotation of the shared key part, both written to the
//                       token's cache slot; rotation of every head's rotated query part into the packed query
//   qe_head_linear      out[t, h, :N] = W[h] x[t, h, :K], one matrix per head (the two folds above)
//
// Norm, angles and rotation in float32; one rounding into the cache and into the packed query.
#include "tile_product.cuh"
#include <math.h>

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ down, long ld_down, const T* __restrict__ q, long ldq,
                      const float* __restrict__ norm_w, float eps, const int* __restrict__ positions,
                      const float* __restrict__ inv_freq, int rot_dims, T* __restrict__ cache,
                      const int* __restrict__ slot_mapping, T* __restrict__ qlat, int H, int dn, int R, int Dr,
                      int write_kv) {
  __shared__ float red[33];
  extern __shared__ float lp_cs[];                  // the token's cosines [half], then its sines [half]
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int D = R + Dr;
  const int half = rot_dims / 2;
  // positions and frequencies come from the host's copy and the weights: the angles are ready before the wait
  const float pos = (float)positions[t];
  for (int f = threadIdx.x; f < half; f += blockDim.x) sincosf(pos * inv_freq[f], &lp_cs[half + f], &lp_cs[f]);
  pdl_wait();
  __syncthreads();
  const T* row = down + (size_t)t * ld_down;
  if (write_kv) {
    float ss = 0.f;
    for (int d = threadIdx.x; d < R; d += blockDim.x) { const float v = to_f32(row[d]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)R + eps);
    T* dst = cache + (size_t)slot_mapping[t] * D;
    for (int d = threadIdx.x; d < R; d += blockDim.x) dst[d] = from_f32<T>(to_f32(row[d]) * rstd * norm_w[d]);
    // the shared key part: pairs (i, i + half) of its first rot_dims channels turn, the rest pass
    for (int i = threadIdx.x; i < Dr; i += blockDim.x) {
      float v = to_f32(row[R + i]);
      if (i < rot_dims) {
        const int f = i < half ? i : i - half;
        const float cs = lp_cs[f], sn = lp_cs[half + f];
        const float other = to_f32(row[R + (i < half ? i + half : i - half)]);
        v = i < half ? v * cs - other * sn : v * cs + other * sn;
      }
      dst[R + i] = from_f32<T>(v);
    }
  }
  // every head's rotated query part, behind the room for its folded plain part
#pragma unroll 4
  for (int e = threadIdx.x; e < H * Dr; e += blockDim.x) {
    const int h = e / Dr, i = e - h * Dr;
    const T* qr = q + (size_t)t * ldq + (size_t)h * (dn + Dr) + dn;
    float v = to_f32(qr[i]);
    if (i < rot_dims) {
      const int f = i < half ? i : i - half;
      const float cs = lp_cs[f], sn = lp_cs[half + f];
      const float other = to_f32(qr[i < half ? i + half : i - half]);
      v = i < half ? v * cs - other * sn : v * cs + other * sn;
    }
    qlat[((size_t)t * H + h) * D + R + i] = from_f32<T>(v);
  }
}

extern "C" int qe_latent_prepare(const void* down, long ld_down, const void* q, long ldq, const float* norm_w, float eps,
                                 const int* positions, const float* inv_freq, int rot_dims, void* cache,
                                 const int* slot_mapping, void* qlat, int T, int H, int dn, int R, int Dr, int write_kv,
                                 int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot_dims < 0 || rot_dims > Dr || rot_dims % 2) QE_REFUSE("latent_prepare: %d rotated dimensions of %d", rot_dims, Dr);
  if (H < 1 || dn < 0 || R < 1 || Dr < 0) QE_REFUSE("latent_prepare: sizes %d %d %d %d", H, dn, R, Dr);
  const size_t lp_smem = (size_t)(rot_dims > 0 ? rot_dims : 2) * sizeof(float);
  if (lp_smem > 40 * 1024) QE_REFUSE("latent_prepare: %d rotated dimensions", rot_dims);
#define LP(TT) qe_launch(latent_prepare_kernel<TT>, dim3(T), dim3(128), lp_smem, stream, (const TT*)down, ld_down, (const TT*)q, ldq, \
                         norm_w, eps, positions, inv_freq, rot_dims, (TT*)cache, slot_mapping, (TT*)qlat, H, dn, R, Dr, write_kv)
  if (dtype == QE_DTYPE_F32) LP(float);
  else if (dtype == QE_DTYPE_BF16) LP(__nv_bfloat16);
  else QE_REFUSE("latent_prepare: unknown dtype %d", dtype);
#undef LP
  QE_CHECK_LAUNCH("latent_prepare");
  return 0;
}

// out[t * ldo + h * ldo_h + n] = sum_k w[h][n][k] * x[t * ldx + h * ldx_h + k]
template <typename T>
__global__ void __launch_bounds__(TP_THREADS)
head_linear_kernel(const T* __restrict__ x, long ldx, long ldx_h, const T* __restrict__ w, T* __restrict__ out, long ldo,
                   long ldo_h, int M, int N, int K) {
  __shared__ TpSmem<T, 1> sm;
  TpAcc<T, 1> acc;
  const int m0 = blockIdx.x * TP_BM, n0 = blockIdx.y * TP_BN, h = blockIdx.z;
  pdl_launch_dependents();
  pdl_wait();
  const T* wh = w + (size_t)h * N * K;
  tile_product<T, 1>(sm, acc, K,
      [&](int r) -> const T* { return m0 + r < M ? x + (size_t)(m0 + r) * ldx + (size_t)h * ldx_h : nullptr; },
      [&](int, int n) -> const T* { return n0 + n < N ? wh + (size_t)(n0 + n) * K : nullptr; });
  tile_for_each<T, 1>(acc, [&](int r, int n, float v, float) {
    if (m0 + r < M && n0 + n < N) out[(size_t)(m0 + r) * ldo + (size_t)h * ldo_h + n0 + n] = from_f32<T>(v);
  });
}

__global__ void __launch_bounds__(FP_THREADS)
head_linear_fast_kernel(const __nv_bfloat16* __restrict__ x, long ldx, long ldx_h, const __nv_bfloat16* __restrict__ w,
                        __nv_bfloat16* __restrict__ out, long ldo, long ldo_h, int M, int N, int K) {
  extern __shared__ __align__(16) unsigned char fp_smem[];
  FpAcc acc;
  constexpr int BN = FpShape<1>::BN;
  const int m0 = blockIdx.x * FP_BM, n0 = blockIdx.y * BN, h = blockIdx.z;
  pdl_launch_dependents();
  pdl_wait();
  const __nv_bfloat16* wh = w + (size_t)h * N * K;
  fast_tile_product<1>(fp_smem, acc, K, w, min(FP_BM, M - m0),
      [&](int r) -> const __nv_bfloat16* { return m0 + r < M ? x + (size_t)(m0 + r) * ldx + (size_t)h * ldx_h : nullptr; },
      [&](int, int n) -> const __nv_bfloat16* { return n0 + n < N ? wh + (size_t)(n0 + n) * K : nullptr; });
  fast_tile_for_each<1>(acc, [&](int r, int n, float v, float) {
    if (m0 + r < M && n0 + n < N) out[(size_t)(m0 + r) * ldo + (size_t)h * ldo_h + n0 + n] = __float2bfloat16_rn(v);
  });
}

extern "C" int qe_head_linear(const void* x, long ldx, long ldx_h, const void* w, void* out, long ldo, long ldo_h,
                              int M, int H, int N, int K, int dtype, cudaStream_t stream) {
  if (M <= 0 || H <= 0 || N <= 0) return 0;
  if (K < 1 || H > 65535) QE_REFUSE("head_linear: K = %d, %d heads", K, H);
  if (dtype == QE_DTYPE_BF16 && K % 8 == 0 && ldx % 8 == 0 && ldx_h % 8 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0) {
    // every row on a 16-byte boundary: the pipelined kernel
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(head_linear_fast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FP_SMEM_BYTES);
      if (e != cudaSuccess) QE_REFUSE("head_linear: shared memory: %s", cudaGetErrorString(e));
      configured = true;
    }
    dim3 fgrid((M + FP_BM - 1) / FP_BM, (N + FpShape<1>::BN - 1) / FpShape<1>::BN, H);
    if (fgrid.y > 65535) QE_REFUSE("head_linear: N = %d is too wide", N);
    qe_launch(head_linear_fast_kernel, fgrid, dim3(FP_THREADS), FP_SMEM_BYTES, stream, (const __nv_bfloat16*)x, ldx, ldx_h,
              (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ldo, ldo_h, M, N, K);
    QE_CHECK_LAUNCH("head_linear");
    return 0;
  }
  dim3 grid((M + TP_BM - 1) / TP_BM, (N + TP_BN - 1) / TP_BN, H);
  if (grid.y > 65535) QE_REFUSE("head_linear: N = %d is too wide", N);
#define HL(TT) qe_launch(head_linear_kernel<TT>, grid, dim3(TP_THREADS), 0, stream, (const TT*)x, ldx, ldx_h, (const TT*)w, \
                         (TT*)out, ldo, ldo_h, M, N, K)
  if (dtype == QE_DTYPE_F32) HL(float);
  else if (dtype == QE_DTYPE_BF16) HL(__nv_bfloat16);
  else QE_REFUSE("head_linear: unknown dtype %d", dtype);
#undef HL
  QE_CHECK_LAUNCH("head_linear");
  return 0;
}
