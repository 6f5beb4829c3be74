// Gated linear attention with a decay per key channel, as a recurrence over tokens with its state in
// float32, for any mixture of prompt portions and single decoded tokens:
//
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        (S: key channels x value channels, one per head and request)
//   o_t = S_t^T (q_scale q_t)
//
// and the two small kernels around it: the decay alpha = sigmoid(z)^(1/tau) from a low-rank projection, and
// the per-head RMS norm of o with an output gate.  Everything that enters the recurrence besides q, k, v is
// float32 (z, its log-sigmoid, alpha, the state, o); q, k, v come in the step's compute type.
//
// The scan: one CTA per (request, head, tile of value channels).  A value channel's column of S evolves on
// its own, so the columns are dealt to threads: thread (j, l) keeps DC consecutive key channels of column j
// in registers (L = threads per column, L * DC >= key channels), multiplies, adds and reduces over l by
// shuffles; the order of every sum is fixed by the sizes alone, so a token's output does not depend on how
// the request was cut into steps or on what else the step carries.  Four producer warps stage the next
// chunk of tokens (q scaled, k, alpha, v, as float32) in shared memory while the others compute.
// State in memory: [slot][head][value channel][key channel] float32; a request whose context is empty
// starts from zero whatever its slot holds.
#include "common.cuh"
#include <math.h>

// ---------------------------------------------------------------------------------------------------------
// alpha[t, n] = exp(logsigmoid(z) / tau),  z = sum_r a[t, r] w[n, r] + bias[n]
// ---------------------------------------------------------------------------------------------------------
#define DEC_COLS 128
#define DEC_ROWS 16
template <typename T>
__global__ void __launch_bounds__(DEC_COLS)
channel_decay_kernel(const T* __restrict__ a, long lda, const T* __restrict__ w, const float* __restrict__ bias,
                     float inv_tau, float* __restrict__ out, int T_tokens, int N, int R,
                     const float* __restrict__ log_rate, int per_rate) {
  extern __shared__ float smem[];
  float* ws = smem;                          // [DEC_COLS][R + 1]
  float* as = ws + DEC_COLS * (R + 1);       // [DEC_ROWS][R]
  const int n0 = blockIdx.x * DEC_COLS, t0 = blockIdx.y * DEC_ROWS;
  pdl_launch_dependents();
#pragma unroll 8
  for (int e = threadIdx.x; e < DEC_COLS * R; e += blockDim.x) {       // weights: nothing of the step writes them
    const int n = e / R, r = e - n * R;
    ws[n * (R + 1) + r] = n0 + n < N ? to_f32(w[(size_t)(n0 + n) * R + r]) : 0.f;
  }
  pdl_wait();
  const int rows = min(DEC_ROWS, T_tokens - t0);
  for (int e = threadIdx.x; e < rows * R; e += blockDim.x) {
    const int t = e / R, r = e - t * R;
    as[e] = to_f32(a[(size_t)(t0 + t) * lda + r]);
  }
  __syncthreads();
  const int n = n0 + threadIdx.x;
  if (n >= N) return;
  const float b = bias ? bias[n] : 0.f;
  const float* wr = ws + threadIdx.x * (R + 1);
  // the second form: exp(-rate softplus(z)) with one rate = exp(log_rate) per `per_rate` neighbouring channels
  const float rate = log_rate ? expf(log_rate[n / per_rate]) : 0.f;
  for (int t = 0; t < rows; ++t) {
    float z = b;
    const float* ar = as + t * R;
    for (int r = 0; r < R; ++r) z = fmaf(ar[r], wr[r], z);
    if (log_rate) {
      const float softplus = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
      out[(size_t)(t0 + t) * N + n] = expf(-rate * softplus);
    } else {
      const float logsig = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
      out[(size_t)(t0 + t) * N + n] = expf(logsig * inv_tau);
    }
  }
}

// log_rate null: out = sigmoid(z)^(1/tau).  log_rate float32 [N / per_rate]: out = exp(-exp(log_rate[n / per_rate]) softplus(z)).
extern "C" int qe_channel_decay(const void* a, long lda, const void* w, const float* bias, float tau, float* out,
                                int T, int N, int R, int dtype, const float* log_rate, int per_rate, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (R < 1 || R > 256) QE_REFUSE("channel_decay: rank %d is outside 1..256", R);
  if (!log_rate && !(tau > 0.f)) QE_REFUSE("channel_decay: tau must be positive");
  if (log_rate && (per_rate < 1 || N % per_rate)) QE_REFUSE("channel_decay: %d channels do not share rates in groups of %d", N, per_rate);
  const size_t smem = ((size_t)DEC_COLS * (R + 1) + (size_t)DEC_ROWS * R) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    const int max_smem = (int)(((size_t)DEC_COLS * 257 + (size_t)DEC_ROWS * 256) * sizeof(float));
    cudaError_t e = cudaFuncSetAttribute(channel_decay_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(channel_decay_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e != cudaSuccess) QE_REFUSE("channel_decay: shared memory %d: %s", max_smem, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((N + DEC_COLS - 1) / DEC_COLS, (T + DEC_ROWS - 1) / DEC_ROWS);
  if (dtype == QE_DTYPE_F32)
    qe_launch(channel_decay_kernel<float>, grid, dim3(DEC_COLS), smem, stream, (const float*)a, lda, (const float*)w, bias,
              log_rate ? 0.f : 1.f / tau, out, T, N, R, log_rate, per_rate);
  else if (dtype == QE_DTYPE_BF16)
    qe_launch(channel_decay_kernel<__nv_bfloat16>, grid, dim3(DEC_COLS), smem, stream, (const __nv_bfloat16*)a, lda,
              (const __nv_bfloat16*)w, bias, log_rate ? 0.f : 1.f / tau, out, T, N, R, log_rate, per_rate);
  else QE_REFUSE("channel_decay: unknown dtype %d", dtype);
  QE_CHECK_LAUNCH("channel_decay");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// the scan
// ---------------------------------------------------------------------------------------------------------
#define GLA_PRODUCERS 128          // threads that stage the next chunk
#define GLA_MAX_COMPUTE 128        // threads that hold state (with the producers 256 a CTA: registers enough for eight tokens a turn)

struct GlaArgs {
  const void* q; const void* k; const void* v;        // rows of the step's tokens; heads side by side
  long ldq, ldk, ldv;                                 // row strides in elements
  const float* alpha;                                 // [T, H * dk]
  float* state;                                       // [slots, H, dv, dk]
  const int* cu_q; const int* ctx_lens; const int* slot_ids;
  float* out;                                         // [T, H * dv]
  float q_scale;
  int H, dk, dv, L, VT, chunk, write_state;
  int vec;                                            // q, k, v, alpha can be staged in pieces of 16 bytes
  int single;                                         // every request brings one token
  // single tokens may bring the decay's inputs instead of alpha: alpha = exp(logsigmoid(a . w[c] + bias[c]) / tau)
  const void* da; long lda; const void* dw; const float* dbias; float inv_tau; int R;
  int fast;                                           // ... and a chunk is at most 8 pieces a producer
  const float* head_decay;                            // null, or [H]: alpha is this one number for every token and key channel of a head
};

// index of key channel c in a staged row: blocks of DC channels, 4 floats of padding between them (banks)
template <int DC> __device__ __forceinline__ int gla_pad(int c) { return c + (c / DC) * 4; }

// SINGLE: a step of single tokens (one chunk of one token a request): no producers, no turns of eight tokens, few
// registers, many CTAs an SM.
template <typename T, int DC, bool SINGLE>
__global__ void __launch_bounds__(SINGLE ? GLA_MAX_COMPUTE : GLA_MAX_COMPUTE + GLA_PRODUCERS, SINGLE ? 4 : 1)
gla_scan_kernel(GlaArgs A) {
  extern __shared__ float smem[];
  const int req = blockIdx.x, head = blockIdx.y, j0 = blockIdx.z * A.VT;
  const int dk = A.dk, dv = A.dv, L = A.L, VT = A.VT, H = A.H;
  const int n_compute = VT * L;
  const int row_w = gla_pad<DC>(L * DC);               // floats of one staged row of q, k or alpha
  const int tok_w = 3 * row_w + ((VT + 3) & ~3);       // floats of one staged token (rows stay 16-byte aligned)
  float* buf[2] = {smem, smem + (size_t)A.chunk * tok_w};
  const bool producer = threadIdx.x >= n_compute;
  const int tid = threadIdx.x;
  const int j = j0 + tid / L, l = tid % L;
  const bool owns = !producer && j < dv;
  // the L threads of a column are neighbours within one warp; only they meet in the shuffles
  const unsigned col_mask = L >= 32 ? 0xffffffffu : (((1u << L) - 1u) << ((threadIdx.x & 31) & ~(L - 1)));
  pdl_launch_dependents();
  pdl_wait();
  const int row0 = A.cu_q[req];
  const int n = A.cu_q[req + 1] - row0;
  if (n <= 0) return;
  const int ctx = A.ctx_lens[req];
  const int slot = A.slot_ids[req];
  float* st = A.state + (((size_t)slot * H + head) * dv + (owns ? j : 0)) * dk;

  float s[DC];
#pragma unroll
  for (int i = 0; i < DC; ++i) s[i] = 0.f;
  if (owns && ctx > 0) {
    if (dk % 4 == 0) {
#pragma unroll
      for (int i = 0; i < DC; i += 4) {
        const int c = l * DC + i;
        if (c < dk) { const float4 x = *reinterpret_cast<const float4*>(st + c); s[i] = x.x; s[i + 1] = x.y; s[i + 2] = x.z; s[i + 3] = x.w; }
      }
    } else {
#pragma unroll
      for (int i = 0; i < DC; ++i) { const int c = l * DC + i; if (c < dk) s[i] = st[c]; }
    }
  }

  const T* q = (const T*)A.q + (size_t)head * dk;
  const T* k = (const T*)A.k + (size_t)head * dk;
  const T* v = (const T*)A.v + (size_t)head * dv;
  const float* al = A.alpha + (size_t)head * dk;
  const float hd = A.head_decay ? A.head_decay[head] : 0.f;
  const int n_chunks = (n + A.chunk - 1) / A.chunk;
  const int ptid = tid - n_compute, n_prod = blockDim.x - n_compute;
  const int padded = L * DC;

  // stage chunk `ch` into buf[ch & 1], element by element (any sizes and strides): by the producers, or by everybody
  // for the first chunk
  auto stage = [&](int ch, int t_id, int t_n) {
    float* b = buf[ch & 1];
    const int t_first = ch * A.chunk;
    const int rows = min(A.chunk, n - t_first);
    const int per_tok = 3 * padded + VT;
    for (int e = t_id; e < rows * per_tok; e += t_n) {
      const int t = e / per_tok, x = e - t * per_tok;
      const size_t row = (size_t)(row0 + t_first + t);
      float* dst = b + (size_t)t * tok_w;
      if (x < 3 * padded) {
        const int which = x / padded, c = x - which * padded;
        if (which == 2 && c < dk && A.alpha == nullptr && A.head_decay == nullptr) continue;      // the kernel forms this decay itself, below
        float val;
        if (c >= dk) val = which == 2 ? 1.f : 0.f;                     // channels beyond the head: nothing in, nothing out
        else if (which == 0) val = to_f32(q[row * A.ldq + c]) * A.q_scale;
        else if (which == 1) val = to_f32(k[row * A.ldk + c]);
        else val = A.head_decay ? hd : al[row * ((size_t)H * dk) + c];
        dst[which * row_w + gla_pad<DC>(c)] = val;
      } else {
        const int jj = x - 3 * padded;
        dst[3 * row_w + jj] = j0 + jj < dv ? to_f32(v[row * A.ldv + j0 + jj]) : 0.f;
      }
    }
  };

  // The same in pieces of 16 bytes where sizes, strides and addresses allow (A.vec).  A thread's pieces of a chunk sit
  // at the same places in every chunk, so what describes them (which row of the chunk, where from, where to) is worked
  // out once; all of a thread's loads are on their way before the first is converted and stored.
  constexpr int VEC = 16 / (int)sizeof(T);             // elements of q, k, v in a piece
  constexpr int NI = 8;                                // pieces a thread has on their way at a time
  const int pieces_qk = dk / VEC, pieces_a = dk / 4, pieces_v = VT / VEC;
  const int per_tok_v = 2 * pieces_qk + pieces_a + pieces_v;
  // piece e of a chunk: token e / per_tok_v; then q, k, alpha, v in turn.  kind 0..3 (4: v columns beyond the head,
  // zeros); `off`: bytes from the kind's base to the piece within its row; so, so2: where its two groups of four go
  const char* const base_of[4] = {(const char*)q, (const char*)k, (const char*)al, (const char*)(v + j0)};
  const long row_bytes_of[4] = {A.ldq * (long)sizeof(T), A.ldk * (long)sizeof(T), (long)H * dk * (long)sizeof(float),
                                A.ldv * (long)sizeof(T)};
  auto describe = [&](int e, int& t, int& off, int& so, int& so2, int& kind) {
    t = e / per_tok_v;
    int x = e - t * per_tok_v;
    if (x < pieces_qk) {
      kind = 0; off = x * 16;
      so = t * tok_w + gla_pad<DC>(x * VEC); so2 = t * tok_w + gla_pad<DC>(x * VEC + 4);
    } else if ((x -= pieces_qk) < pieces_qk) {
      kind = 1; off = x * 16;
      so = t * tok_w + row_w + gla_pad<DC>(x * VEC); so2 = t * tok_w + row_w + gla_pad<DC>(x * VEC + 4);
    } else if ((x -= pieces_qk) < pieces_a) {
      kind = 2; off = x * 16;
      so = so2 = t * tok_w + 2 * row_w + gla_pad<DC>(x * 4);
    } else {
      x -= pieces_a;
      kind = j0 + x * VEC >= dv ? 4 : 3; off = x * 16;
      so = t * tok_w + 3 * row_w + x * VEC; so2 = so + 4;
    }
  };
  auto fetch = [&](int kind, int off, size_t row) -> uint4 {
    if (kind == 2 && A.head_decay) { const unsigned u = __float_as_uint(hd); return make_uint4(u, u, u, u); }
    if (kind > 3 || (kind == 2 && A.alpha == nullptr)) return make_uint4(0, 0, 0, 0);
    const char* base = kind == 0 ? base_of[0] : kind == 1 ? base_of[1] : kind == 2 ? base_of[2] : base_of[3];
    const long rb = kind == 0 ? row_bytes_of[0] : kind == 1 ? row_bytes_of[1] : kind == 2 ? row_bytes_of[2] : row_bytes_of[3];
    return __ldg(reinterpret_cast<const uint4*>(base + row * rb + off));
  };
  auto put = [&](float* b, const uint4& r, int so, int so2, int kind) {
    if (kind == 2) { if (A.alpha || A.head_decay) *reinterpret_cast<uint4*>(b + so) = r; return; }      // (absent: the kernel forms the decay itself)
    float f[VEC];
    if constexpr (sizeof(T) == 2) {
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int u = 0; u < 4; ++u) { const float2 x2 = __bfloat1622float2(h2[u]); f[2 * u] = x2.x; f[2 * u + 1] = x2.y; }
    } else {
      f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
    }
    const float sc = kind == 0 ? A.q_scale : 1.f;
    // groups of four channels never straddle a thread's block of DC (a multiple of four): the padding falls between
    *reinterpret_cast<float4*>(b + so) = make_float4(f[0] * sc, f[1] * sc, f[2] * sc, f[3] * sc);
    if constexpr (VEC == 8) *reinterpret_cast<float4*>(b + so2) = make_float4(f[4] * sc, f[5] * sc, f[6] * sc, f[7] * sc);
  };
  // any number of pieces, described as they come (the first chunk, by all threads; chunks too large for the fast form)
  auto stage_vec = [&](int ch, int t_id, int t_n) {
    float* b = buf[ch & 1];
    const int t_first = ch * A.chunk;
    const int total = min(A.chunk, n - t_first) * per_tok_v;
    for (int e0 = t_id; e0 < total; e0 += NI * t_n) {
      uint4 r[NI];
      int so[NI], so2[NI], kind[NI];
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const int e = e0 + i * t_n;
        kind[i] = -1;
        if (e < total) {
          int t, off;
          describe(e, t, off, so[i], so2[i], kind[i]);
          r[i] = fetch(kind[i], off, (size_t)(row0 + t_first + t));
        }
      }
#pragma unroll
      for (int i = 0; i < NI; ++i) if (kind[i] >= 0) put(b, r[i], so[i], so2[i], kind[i]);
    }
  };
  // the producers' fast form: a chunk is at most NI pieces a producer (A.fast), each described once
  int p_meta[NI], p_off[NI], p_so[NI], p_so2[NI];          // p_meta: the chunk's row * 8 + kind
  if (!SINGLE && A.vec && A.fast && producer) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int e = ptid + i * n_prod;
      p_meta[i] = 1 << 30; p_off[i] = p_so[i] = p_so2[i] = 0;
      if (e < A.chunk * per_tok_v) {
        int t, kind;
        describe(e, t, p_off[i], p_so[i], p_so2[i], kind);
        p_meta[i] = t * 8 + kind;
      }
    }
  }
  auto stage_fast = [&](int ch) {
    float* b = buf[ch & 1];
    const int t_first = ch * A.chunk;
    const int rows = min(A.chunk, n - t_first);
    const size_t base_row = (size_t)(row0 + t_first);
    uint4 r[NI];
#pragma unroll
    for (int i = 0; i < NI; ++i)
      if ((p_meta[i] >> 3) < rows) r[i] = fetch(p_meta[i] & 7, p_off[i], base_row + (p_meta[i] >> 3));
#pragma unroll
    for (int i = 0; i < NI; ++i) if ((p_meta[i] >> 3) < rows) put(b, r[i], p_so[i], p_so2[i], p_meta[i] & 7);
  };

  if (A.vec) {
    // channels beyond the head (L * DC > dk) are never staged by pieces: nothing in, nothing kept, nothing out
    if (padded > dk)
      for (int e = tid; e < 2 * A.chunk * (padded - dk); e += blockDim.x) {
        const int t = e / (padded - dk), c = dk + e - t * (padded - dk);
        float* dst = smem + (size_t)t * tok_w + gla_pad<DC>(c);
        dst[0] = 0.f; dst[row_w] = 0.f; dst[2 * row_w] = 1.f;
      }
    stage_vec(0, tid, blockDim.x);
  } else {
    stage(0, tid, blockDim.x);
  }
  if (SINGLE && A.da) {
    // the request's one token: the decay of this head's channels from the low-rank pair's second half, in the order
    // of sums of the kernel that does this for many tokens (the same bits)
    const T* a = (const T*)A.da + (size_t)row0 * A.lda;
    for (int c = tid; c < dk; c += blockDim.x) {
      const T* wr = (const T*)A.dw + ((size_t)head * dk + c) * A.R;
      float z = A.dbias ? A.dbias[head * dk + c] : 0.f;
      for (int r = 0; r < A.R; ++r) z = fmaf(to_f32(a[r]), to_f32(wr[r]), z);
      const float logsig = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
      smem[2 * row_w + gla_pad<DC>(c)] = expf(logsig * A.inv_tau);
    }
  }
  __syncthreads();
  const size_t o_ld = (size_t)H * dv;
  for (int ch = 0; ch < n_chunks; ++ch) {
    if (producer) {
      if (!SINGLE && ch + 1 < n_chunks) {
        if (A.vec && A.fast) stage_fast(ch + 1);
        else if (A.vec) stage_vec(ch + 1, ptid, n_prod);
        else stage(ch + 1, ptid, n_prod);
      }
    } else if (owns) {
      const int rows = min(A.chunk, n - ch * A.chunk);
      const float* r = buf[ch & 1] + l * (DC + 4);
      const float* rv = buf[ch & 1] + 3 * row_w + (j - j0);
      float* o = A.out + (size_t)(row0 + ch * A.chunk) * o_ld + (size_t)head * dv + j;
      int t0 = 0;
      // Eight tokens a turn.  The state's chain runs through them one after the other; their eight sums over the column's
      // threads are then formed together: in each round a thread keeps half of its tokens and hands the other half to its
      // partner (1, 2, 4 lanes away), so that after three rounds every thread holds one token's sum (7 exchanges for 8
      // tokens instead of 24), which it stores.  Columns of fewer than 8 threads stop earlier and keep several tokens
      // each; columns of more go on with whole sums.  The order of every sum depends on the sizes alone.
      for (; !SINGLE && t0 + 8 <= rows; t0 += 8) {
        float acc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float vj = rv[0];
          float a0 = 0.f, a1 = 0.f;
#pragma unroll
          for (int i = 0; i < DC; i += 4) {
            const float4 q4 = *reinterpret_cast<const float4*>(r + i);
            const float4 k4 = *reinterpret_cast<const float4*>(r + row_w + i);
            const float4 a4 = *reinterpret_cast<const float4*>(r + 2 * row_w + i);
            s[i] = fmaf(a4.x, s[i], k4.x * vj);             a0 = fmaf(q4.x, s[i], a0);
            s[i + 1] = fmaf(a4.y, s[i + 1], k4.y * vj);     a1 = fmaf(q4.y, s[i + 1], a1);
            s[i + 2] = fmaf(a4.z, s[i + 2], k4.z * vj);     a0 = fmaf(q4.z, s[i + 2], a0);
            s[i + 3] = fmaf(a4.w, s[i + 3], k4.w * vj);     a1 = fmaf(q4.w, s[i + 3], a1);
          }
          acc[u] = a0 + a1;
          r += tok_w; rv += tok_w;
        }
        int mine = 0, held = 8;                       // the first token this thread ends up with, and how many
        if (L > 1) {
          const bool up = l & 1;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float give = up ? acc[i] : acc[i + 4], keep = up ? acc[i + 4] : acc[i];
            acc[i] = keep + __shfl_xor_sync(col_mask, give, 1);
          }
          mine += up ? 4 : 0; held = 4;
        }
        if (L > 2) {
          const bool up = l & 2;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const float give = up ? acc[i] : acc[i + 2], keep = up ? acc[i + 2] : acc[i];
            acc[i] = keep + __shfl_xor_sync(col_mask, give, 2);
          }
          mine += up ? 2 : 0; held = 2;
        }
        if (L > 4) {
          const bool up = l & 4;
          const float give = up ? acc[0] : acc[1], keep = up ? acc[1] : acc[0];
          acc[0] = keep + __shfl_xor_sync(col_mask, give, 4);
          mine += up ? 1 : 0; held = 1;
        }
        for (int off = 8; off < L; off <<= 1) acc[0] += __shfl_xor_sync(col_mask, acc[0], off);
        if (l < 8) {
#pragma unroll
          for (int i = 0; i < 8; ++i) if (i < held) o[(size_t)(t0 + mine + i) * o_ld] = acc[i];
        }
      }
      // what is left of the chunk, token by token
      for (; t0 < rows; ++t0) {
        const float vj = rv[0];
        float a0 = 0.f, a1 = 0.f;                 // (the same order of sums as in a turn of eight: the bits do not depend on the cut)
#pragma unroll
        for (int i = 0; i < DC; i += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(r + i);
          const float4 k4 = *reinterpret_cast<const float4*>(r + row_w + i);
          const float4 a4 = *reinterpret_cast<const float4*>(r + 2 * row_w + i);
          s[i] = fmaf(a4.x, s[i], k4.x * vj);             a0 = fmaf(q4.x, s[i], a0);
          s[i + 1] = fmaf(a4.y, s[i + 1], k4.y * vj);     a1 = fmaf(q4.y, s[i + 1], a1);
          s[i + 2] = fmaf(a4.z, s[i + 2], k4.z * vj);     a0 = fmaf(q4.z, s[i + 2], a0);
          s[i + 3] = fmaf(a4.w, s[i + 3], k4.w * vj);     a1 = fmaf(q4.w, s[i + 3], a1);
        }
        float acc1 = a0 + a1;
        for (int off = 1; off < L; off <<= 1) acc1 += __shfl_xor_sync(col_mask, acc1, off);
        if (l == 0) o[(size_t)t0 * o_ld] = acc1;
        r += tok_w; rv += tok_w;
      }
    }
    if (n_chunks > 1) __syncthreads();
  }
  if (owns && A.write_state) {
    if (dk % 4 == 0) {
#pragma unroll
      for (int i = 0; i < DC; i += 4) {
        const int c = l * DC + i;
        if (c < dk) *reinterpret_cast<float4*>(st + c) = make_float4(s[i], s[i + 1], s[i + 2], s[i + 3]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < DC; ++i) { const int c = l * DC + i; if (c < dk) st[c] = s[i]; }
    }
  }
}

template <typename T, int DC>
static int gla_launch(const GlaArgs& A, int R, cudaStream_t stream, size_t smem) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gla_scan_kernel<T, DC, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gla_scan_kernel<T, DC, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e != cudaSuccess) QE_REFUSE("linear_attention_scan: shared memory: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int n_compute = ((A.VT * A.L + 31) / 32) * 32;
  dim3 grid(R, A.H, (A.dv + A.VT - 1) / A.VT);
  // steps of single tokens have one chunk: nobody stages ahead, the CTA is its computing threads alone
  if (A.single) qe_launch(gla_scan_kernel<T, DC, true>, grid, dim3(n_compute), smem, stream, A);
  else qe_launch(gla_scan_kernel<T, DC, false>, grid, dim3(n_compute + GLA_PRODUCERS), smem, stream, A);
  QE_CHECK_LAUNCH("linear_attention_scan");
  return 0;
}

// How the key channels of a head are dealt to threads: DC channels a thread, L threads a column.
static void gla_shape(int dk, int* DC, int* L) {
  int dc = dk <= 16 ? 4 : dk <= 64 ? 8 : dk <= 128 ? 16 : 32;
  int l = 1;
  while (l * dc < dk) l <<= 1;
  *DC = dc; *L = l;
}

// alpha null (steps of single tokens only): the decay comes from decay_a [T, rank] (rows of lda elements), decay_w
// [H dk, rank] in the type of q, decay_bias float32 [H dk] and tau, as qe_channel_decay computes it.
extern "C" int qe_linear_attention_scan(const void* q, const void* k, const void* v, long ldq, long ldk, long ldv,
                                        const float* alpha, float* state, const int* cu_q, const int* ctx_lens,
                                        const int* slot_ids, float* out, float q_scale, int R, int max_q_len, int H,
                                        int dk, int dv, int write_state, int dtype, const void* decay_a, long lda,
                                        const void* decay_w, const float* decay_bias, float tau, int rank,
                                        const float* head_decay, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (head_decay != nullptr && alpha != nullptr) QE_REFUSE("linear_attention_scan: a decay per head or per channel, not both");
  if (alpha == nullptr && head_decay == nullptr && (decay_a == nullptr || decay_w == nullptr || rank < 1 || !(tau > 0.f) || max_q_len > 1))
    QE_REFUSE("linear_attention_scan: without alpha, a step of single tokens must bring the decay's inputs");
  if (dk < 1 || dk > 1024 || dv < 1) QE_REFUSE("linear_attention_scan: key size %d must be 1..1024, value size %d positive", dk, dv);
  if (H < 1 || H > 65535) QE_REFUSE("linear_attention_scan: %d heads", H);
  int DC, L;
  gla_shape(dk, &DC, &L);
  if (L > 32) QE_REFUSE("linear_attention_scan: key size %d is too large", dk);
  GlaArgs A;
  A.q = q; A.k = k; A.v = v; A.ldq = ldq; A.ldk = ldk; A.ldv = ldv; A.alpha = alpha; A.state = state;
  A.cu_q = cu_q; A.ctx_lens = ctx_lens; A.slot_ids = slot_ids; A.out = out; A.q_scale = q_scale;
  A.H = H; A.dk = dk; A.dv = dv; A.L = L; A.write_state = write_state;
  A.head_decay = head_decay;
  if (head_decay) decay_a = nullptr;
  A.da = alpha ? nullptr : decay_a; A.lda = lda; A.dw = decay_w; A.dbias = decay_bias; A.inv_tau = (alpha || head_decay) ? 0.f : 1.f / tau; A.R = rank;
  // a column's threads lie within one warp (L divides 32); a tile of value channels fills up to 256 threads,
  // and is narrower where few requests would leave SMs idle
  int VT = GLA_MAX_COMPUTE / L;
  if (VT > dv) VT = dv;
  while (VT > 8 && (long)R * H * ((dv + VT - 1) / VT) < 296 && VT * L > 64) VT = (VT + 1) / 2;
  A.VT = VT;
  const int row_w = L * DC + ((L * DC) / DC) * 4;
  const int tok_w = 3 * row_w + ((VT + 3) & ~3);
  // tokens a chunk: up to 24, and for longer prompts few enough that a producer has at most eight pieces of 16 bytes
  // of a chunk to fetch, which it then describes once for all chunks (measured at 2 048 tokens of 8 heads, 64 key and
  // 128 value channels: 242 us with chunks of 8, 212 with 16, 206 with 24, 299 with 32, where the pieces are too many;
  // 128 key channels: 327 us with chunks of 8, 571 with 16)
  const int vec_n0 = dtype == QE_DTYPE_F32 ? 4 : 8;
  int chunk_max = 24;
  while (chunk_max > 8 && chunk_max * (2 * (dk / vec_n0) + dk / 4 + VT / vec_n0) > 8 * GLA_PRODUCERS) chunk_max -= 8;
  int chunk = max_q_len < chunk_max ? (max_q_len < 1 ? 1 : max_q_len) : chunk_max;
  while (chunk > 1 && (size_t)2 * chunk * tok_w * sizeof(float) > 96 * 1024) chunk >>= 1;
  A.chunk = chunk;
  A.single = max_q_len <= 1;      // (a chunk of one token can also be all that fits shared memory: that is not this case)
  // pieces of 16 bytes: whole pieces per head and per tile of value channels, rows and bases on 16-byte boundaries
  const int vec_n = dtype == QE_DTYPE_F32 ? 4 : 8;
  const int per_tok_pieces = 2 * (dk / vec_n) + dk / 4 + VT / vec_n;
  A.fast = chunk * per_tok_pieces <= 8 * GLA_PRODUCERS;
  A.vec = dk % vec_n == 0 && dk % 4 == 0 && VT % vec_n == 0 && dv % vec_n == 0 && ldq % vec_n == 0 && ldk % vec_n == 0 &&
          ldv % vec_n == 0 && (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)alpha) & 15) == 0;
  const size_t smem = (size_t)2 * chunk * tok_w * sizeof(float);
  if (smem > 96 * 1024) QE_REFUSE("linear_attention_scan: key size %d needs %zu bytes of shared memory", dk, smem);
#define GLA_CASE(TT, DCC) return gla_launch<TT, DCC>(A, R, stream, smem)
  if (dtype == QE_DTYPE_F32) {
    switch (DC) { case 4: GLA_CASE(float, 4); case 8: GLA_CASE(float, 8); case 16: GLA_CASE(float, 16); default: GLA_CASE(float, 32); }
  } else if (dtype == QE_DTYPE_BF16) {
    switch (DC) { case 4: GLA_CASE(__nv_bfloat16, 4); case 8: GLA_CASE(__nv_bfloat16, 8); case 16: GLA_CASE(__nv_bfloat16, 16);
                  default: GLA_CASE(__nv_bfloat16, 32); }
  }
#undef GLA_CASE
  QE_REFUSE("linear_attention_scan: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------------------------
// out[t, h, j] = o[t, h, j] * rsqrt(mean_j o[t, h, :]^2 + eps) * w[j] * gate(g[t, h, j]) * scale
// o float32 [T, H * D]; g and out in the compute type, with row strides; one warp per (token, head).
// gate: 0 none, 1 silu (g / (1 + exp(-g))), 2 sigmoid.  w may be null (no norm: out = o * gate * scale).
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float gate_value(float g, int kind) {
  if (kind == 1) return g / (1.f + expf(-g));
  if (kind == 2) return 1.f / (1.f + expf(-g));
  return 1.f;
}

template <typename T, typename TI>
__global__ void head_norm_gate_kernel(const TI* __restrict__ o, long ldo, const T* __restrict__ g, long ldg,
                                      const float* __restrict__ w, float eps, T* __restrict__ out, long ldout, float scale,
                                      int gate, long items, int H, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * warps + warp;
  if (item >= items) return;
  const long t = item / H;
  const int h = (int)(item - t * H);
  const TI* x = o + (size_t)t * ldo + (size_t)h * D;
  float rstd = 1.f;
  if (w) {
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) { const float val = to_f32(x[d]); ss = fmaf(val, val, ss); }
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)D + eps);
  }
  const T* gr = g ? g + (size_t)t * ldg + (size_t)h * D : nullptr;
  T* dst = out + (size_t)t * ldout + (size_t)h * D;
  for (int d = lane; d < D; d += 32) {
    float val = to_f32(x[d]) * rstd;
    if (w) val *= w[d];
    if (gr) val *= gate_value(to_f32(gr[d]), gate);
    dst[d] = from_f32<T>(val * scale);
  }
}

// The same for long rows (heads joined into one, a whole projection): a CTA per (token, head), so that a step of a few
// tokens does not leave a row of thousands of channels to one warp.
template <typename T, typename TI>
__global__ void __launch_bounds__(256)
head_norm_gate_block_kernel(const TI* __restrict__ o, long ldo, const T* __restrict__ g, long ldg, const float* __restrict__ w,
                            float eps, T* __restrict__ out, long ldout, float scale, int gate, int H, int D) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const long t = blockIdx.x / H;
  const int h = (int)(blockIdx.x - t * H);
  const TI* x = o + (size_t)t * ldo + (size_t)h * D;
  float rstd = 1.f;
  if (w) {
    float ss = 0.f;
#pragma unroll 4
    for (int d = threadIdx.x; d < D; d += blockDim.x) { const float val = to_f32(x[d]); ss = fmaf(val, val, ss); }
    ss = block_sum(ss, red);
    rstd = rsqrtf(ss / (float)D + eps);
  }
  const T* gr = g ? g + (size_t)t * ldg + (size_t)h * D : nullptr;
  T* dst = out + (size_t)t * ldout + (size_t)h * D;
#pragma unroll 4
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float val = to_f32(x[d]) * rstd;
    if (w) val *= w[d];
    if (gr) val *= gate_value(to_f32(gr[d]), gate);
    dst[d] = from_f32<T>(val * scale);
  }
}

// The same for bfloat16 gates and outputs where a head is a multiple of 128 channels and everything lies on 16-byte
// boundaries: a lane takes four neighbouring channels of every 128 (16 bytes of float32 o, 8 bytes of gate and of
// output), all loads on their way before the sum of squares.
template <typename TI, int NV>
__global__ void head_norm_gate_vec_kernel(const TI* __restrict__ o, long ldo, const __nv_bfloat16* __restrict__ g, long ldg,
                                          const float* __restrict__ w, float eps, __nv_bfloat16* __restrict__ out, long ldout,
                                          float scale, int gate, long items, int H) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int D = NV * 128;
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * warps + warp;
  if (item >= items) return;
  const long t = item / H;
  const int h = (int)(item - t * H);
  const TI* x = o + (size_t)t * ldo + (size_t)h * D;
  float v[NV][4], gv[NV][4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int d = i * 128 + lane * 4;
    if constexpr (sizeof(TI) == 4) {
      const float4 f = *reinterpret_cast<const float4*>(x + d);
      v[i][0] = f.x; v[i][1] = f.y; v[i][2] = f.z; v[i][3] = f.w;
    } else {
      const uint2 r = *reinterpret_cast<const uint2*>(x + d);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = b.x; v[i][3] = b.y;
    }
    if (g) {
      const uint2 r = *reinterpret_cast<const uint2*>(g + (size_t)t * ldg + (size_t)h * D + d);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
      gv[i][0] = a.x; gv[i][1] = a.y; gv[i][2] = b.x; gv[i][3] = b.y;
    }
  }
  float rstd = 1.f;
  if (w) {
    // (the sum runs over a lane's channels in the order of the channels, then over the lanes: fixed by the sizes)
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int u = 0; u < 4; ++u) ss = fmaf(v[i][u], v[i][u], ss);
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)D + eps);
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int d = i * 128 + lane * 4;
    float r4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float val = v[i][u] * rstd;
      if (w) val *= w[d + u];
      if (g) val *= gate_value(gv[i][u], gate);
      r4[u] = val * scale;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(r4[0], r4[1]), hi = __floats2bfloat162_rn(r4[2], r4[3]);
    uint2 st;
    st.x = *reinterpret_cast<uint32_t*>(&lo);
    st.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + (size_t)t * ldout + (size_t)h * D + d) = st;
  }
}

extern "C" int qe_head_norm_gate(const void* o, long ldo, int o_f32, const void* g, long ldg, const float* w, float eps,
                                 void* out, long ldout, float scale, int gate, int T, int H, int D, int dtype,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  const long items = (long)T * H;
  const int warps = 8;
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (dtype == QE_DTYPE_BF16 && (D == 128 || D == 256) && ldo % 4 == 0 && ldg % 4 == 0 && ldout % 4 == 0 &&
      (((uintptr_t)o & 15) | ((uintptr_t)g & 7) | ((uintptr_t)out & 7)) == 0) {
#define HNGV(TI, NV) qe_launch(head_norm_gate_vec_kernel<TI, NV>, dim3(blocks), dim3(warps * 32), 0, stream, (const TI*)o, ldo, \
                               (const __nv_bfloat16*)g, ldg, w, eps, (__nv_bfloat16*)out, ldout, scale, gate, items, H)
    if (o_f32) { if (D == 128) HNGV(float, 1); else HNGV(float, 2); }
    else { if (D == 128) HNGV(__nv_bfloat16, 1); else HNGV(__nv_bfloat16, 2); }
#undef HNGV
    QE_CHECK_LAUNCH("head_norm_gate");
    return 0;
  }
  if (D >= 512 && items <= 65535L * 32) {
#define HNGB(TT, TI) qe_launch(head_norm_gate_block_kernel<TT, TI>, dim3((unsigned)items), dim3(256), 0, stream, (const TI*)o, ldo, \
                               (const TT*)g, ldg, w, eps, (TT*)out, ldout, scale, gate, H, D)
    if (dtype == QE_DTYPE_F32) HNGB(float, float);
    else if (dtype == QE_DTYPE_BF16) { if (o_f32) HNGB(__nv_bfloat16, float); else HNGB(__nv_bfloat16, __nv_bfloat16); }
    else QE_REFUSE("head_norm_gate: unknown dtype %d", dtype);
#undef HNGB
    QE_CHECK_LAUNCH("head_norm_gate");
    return 0;
  }
#define HNG(TT, TI) qe_launch(head_norm_gate_kernel<TT, TI>, dim3(blocks), dim3(warps * 32), 0, stream, (const TI*)o, ldo, \
                              (const TT*)g, ldg, w, eps, (TT*)out, ldout, scale, gate, items, H, D)
  if (dtype == QE_DTYPE_F32) HNG(float, float);
  else if (dtype == QE_DTYPE_BF16) { if (o_f32) HNG(__nv_bfloat16, float); else HNG(__nv_bfloat16, __nv_bfloat16); }
  else QE_REFUSE("head_norm_gate: unknown dtype %d", dtype);
#undef HNG
  QE_CHECK_LAUNCH("head_norm_gate");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// acc = (first ? 0 : acc) + scale * x, in float32: the weighted sum of mixers that run side by side and
// cannot share one output product.
// ---------------------------------------------------------------------------------------------------------
template <typename TA, typename TX>
__global__ void scaled_add_kernel(TA* __restrict__ acc, const TX* __restrict__ x, float scale, int first, long n) {
  pdl_launch_dependents();
  pdl_wait();
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x)
    acc[e] = from_f32<TA>((first ? 0.f : to_f32(acc[e])) + scale * to_f32(x[e]));
}

extern "C" int qe_scaled_add(void* acc, int acc_dtype, const void* x, int x_dtype, float scale, int first, long n,
                             cudaStream_t stream) {
  if (n <= 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
#define SADD(TA, TX) qe_launch(scaled_add_kernel<TA, TX>, dim3(blocks), dim3(256), 0, stream, (TA*)acc, (const TX*)x, scale, first, n)
  if (acc_dtype == QE_DTYPE_F32 && x_dtype == QE_DTYPE_F32) SADD(float, float);
  else if (acc_dtype == QE_DTYPE_F32 && x_dtype == QE_DTYPE_BF16) SADD(float, __nv_bfloat16);
  else if (acc_dtype == QE_DTYPE_BF16 && x_dtype == QE_DTYPE_F32) SADD(__nv_bfloat16, float);
  else if (acc_dtype == QE_DTYPE_BF16 && x_dtype == QE_DTYPE_BF16) SADD(__nv_bfloat16, __nv_bfloat16);
  else QE_REFUSE("scaled_add: unknown dtypes %d, %d", acc_dtype, x_dtype);
#undef SADD
  QE_CHECK_LAUNCH("scaled_add");
  return 0;
}
