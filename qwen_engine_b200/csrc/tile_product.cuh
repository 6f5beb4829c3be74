// A 64 x 64 tile of C = A . B^T by one CTA of 128 threads, for products whose rows are gathered or whose
// matrices come one per head or per expert, so that they are no plain [M, K] x [N, K] product:
//
//   C[r][n] = sum_k A_r[k] * B_n[k]      r < 64 rows given by pointers (null: a row of zeros), n < 64 rows of B
//
// float: FFMA, a thread owns 4 rows x 8 columns.  bfloat16: mma.sync m16n8k16 with float32 accumulators, a warp owns
// 16 rows x 64 columns.  K is walked in steps of 32 through shared memory; the order of a row's sum depends on K
// alone, so a row's bits do not depend on which other rows share its tile.  NB = 2 runs two B matrices against the
// same rows (the gate and the up projection of a gated feed-forward).
#pragma once
#include "common.cuh"

#define TP_BM 64
#define TP_BN 64
#define TP_BK 32
#define TP_THREADS 128

template <typename T, int NB> struct TpSmem;
template <int NB> struct alignas(16) TpSmem<float, NB> {
  float a[TP_BK][TP_BM + 4];
  float b[NB][TP_BK][TP_BN + 4];
};
template <int NB> struct alignas(16) TpSmem<__nv_bfloat16, NB> {
  __nv_bfloat16 a[TP_BM][TP_BK + 8];
  __nv_bfloat16 b[NB][TP_BN][TP_BK + 8];
};

template <typename T, int NB> struct TpAcc;
template <int NB> struct TpAcc<float, NB> { float v[NB][4][8]; };              // rows ty*4 + i, columns tx*8 + j
template <int NB> struct TpAcc<__nv_bfloat16, NB> { float v[NB][8][4]; };      // n-tile, mma fragment

__device__ __forceinline__ void tp_mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// a_row(r): pointer to row r's K elements or nullptr; b_row(m, n): pointer to row n of B matrix m or nullptr.
template <typename T, int NB, typename ARow, typename BRow>
__device__ __forceinline__ void tile_product(TpSmem<T, NB>& sm, TpAcc<T, NB>& acc, int K, ARow a_row, BRow b_row) {
  const int tid = threadIdx.x;
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int m = 0; m < NB; ++m)
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc.v[m][i][j] = 0.f;
  } else {
#pragma unroll
    for (int m = 0; m < NB; ++m)
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc.v[m][i][j] = 0.f;
  }
  // a thread stages half a row of A and of every B per step: row tid / 2, columns (tid % 2) * 16 ...
  const int sr = tid >> 1, sc = (tid & 1) * 16;
  const T* ap = a_row(sr);
  const T* bp[NB];
#pragma unroll
  for (int m = 0; m < NB; ++m) bp[m] = b_row(m, sr);
  for (int k0 = 0; k0 < K; k0 += TP_BK) {
    __syncthreads();
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int k = k0 + sc + u;
      const T zero = from_f32<T>(0.f);
      const T av = (ap && k < K) ? ap[k] : zero;
      if constexpr (sizeof(T) == 4) sm.a[sc + u][sr] = av; else sm.a[sr][sc + u] = av;
#pragma unroll
      for (int m = 0; m < NB; ++m) {
        const T bv = (bp[m] && k < K) ? bp[m][k] : zero;
        if constexpr (sizeof(T) == 4) sm.b[m][sc + u][sr] = bv; else sm.b[m][sr][sc + u] = bv;
      }
    }
    __syncthreads();
    if constexpr (sizeof(T) == 4) {
      const int ty = tid >> 3, tx = tid & 7;
#pragma unroll 8
      for (int k = 0; k < TP_BK; ++k) {
        const float4 a4 = *reinterpret_cast<const float4*>(&sm.a[k][ty * 4]);
        const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
        for (int m = 0; m < NB; ++m) {
          const float4 b0 = *reinterpret_cast<const float4*>(&sm.b[m][k][tx * 8]);
          const float4 b1 = *reinterpret_cast<const float4*>(&sm.b[m][k][tx * 8 + 4]);
          const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc.v[m][i][j] = fmaf(av[i], bv[j], acc.v[m][i][j]);
        }
      }
    } else {
      const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
#pragma unroll
      for (int kk = 0; kk < TP_BK; kk += 16) {
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t*>(&sm.a[warp * 16 + g][kk + 2 * c]);
        a[1] = *reinterpret_cast<const uint32_t*>(&sm.a[warp * 16 + g + 8][kk + 2 * c]);
        a[2] = *reinterpret_cast<const uint32_t*>(&sm.a[warp * 16 + g][kk + 2 * c + 8]);
        a[3] = *reinterpret_cast<const uint32_t*>(&sm.a[warp * 16 + g + 8][kk + 2 * c + 8]);
#pragma unroll
        for (int m = 0; m < NB; ++m)
#pragma unroll
          for (int nt = 0; nt < 8; ++nt) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&sm.b[m][nt * 8 + g][kk + 2 * c]);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&sm.b[m][nt * 8 + g][kk + 2 * c + 8]);
            tp_mma_bf16(acc.v[m][nt], a, b0, b1);
          }
      }
    }
  }
}

// Every element of the tile that the thread holds: f(row in tile, column in tile, value of B matrix 0[, of 1]).
template <typename T, int NB, typename F>
__device__ __forceinline__ void tile_for_each(const TpAcc<T, NB>& acc, F f) {
  const int tid = threadIdx.x;
  if constexpr (sizeof(T) == 4) {
    const int ty = tid >> 3, tx = tid & 7;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) f(ty * 4 + i, tx * 8 + j, acc.v[0][i][j], NB > 1 ? acc.v[NB - 1][i][j] : 0.f);
  } else {
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e)
        f(warp * 16 + g + (e >> 1) * 8, nt * 8 + 2 * c + (e & 1), acc.v[0][nt][e], NB > 1 ? acc.v[NB - 1][nt][e] : 0.f);
  }
}

// ---------------------------------------------------------------------------------------------------------
// The same for bfloat16 where every row lies on a 16-byte boundary and K is a multiple of 8: a tile of 128 rows by
// one CTA of 256 threads, rows and weights copied 16 bytes at a time through a ring of four stages (cp.async, zero
// fill for rows that are not there and beyond K), fragments by ldmatrix.  NB = 1: 128 columns of one matrix, a warp
// owns 64 rows x 32 columns.  NB = 2: 64 columns of each of two matrices, a warp owns 64 rows x the same 16 columns
// of both.  The order of a row's sum depends on K alone.
// ---------------------------------------------------------------------------------------------------------
#define FP_BM 128
#define FP_BK 32
#define FP_LD 40                       // bfloat16 per staged row: 32 and 16 bytes of padding (ldmatrix without conflicts)
#define FP_STAGES 4
#define FP_THREADS 256
#define FP_STAGE_BYTES (2 * FP_BM * FP_LD * 2)
#define FP_SMEM_BYTES (FP_STAGES * FP_STAGE_BYTES)
template <int NB> struct FpShape { static constexpr int BN = NB == 1 ? 128 : 64; };

__device__ __forceinline__ void fp_cp16(void* dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n"
               :: "r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void fp_ldmatrix4(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}

struct FpAcc { float v[4][4][4]; };    // [16-row tile of the warp's 64 rows][8-column tile][fragment]

// One staged step of 32 channels for a warp: its 64 rows x four 8-column tiles.  FULL: all four 16-row tiles hold rows;
// otherwise only the first `tiles` of them do and the others are left out (the same for all lanes of the warp).
template <int NB, bool FULL>
__device__ __forceinline__ void fp_stage_mma(const __nv_bfloat16* sa, const __nv_bfloat16* sb, FpAcc& acc, int warp_m, int warp_n,
                                             int lane, int tiles) {
  constexpr int BN = FpShape<NB>::BN;
#pragma unroll
  for (int kk = 0; kk < FP_BK; kk += 16) {
    uint32_t b[2][4];
#pragma unroll
    for (int pr = 0; pr < 2; ++pr) {
      // two 8-column tiles: staged rows base .. base + 15; matrices (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
      const int base = NB == 1 ? warp_n * 32 + pr * 16 : pr * BN + warp_n * 16;
      const int mat = lane >> 3;
      fp_ldmatrix4(b[pr], sb + (base + (mat >> 1) * 8 + (lane & 7)) * FP_LD + kk + (mat & 1) * 8);
    }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      if (!FULL && mt >= tiles) break;
      uint32_t a[4];
      fp_ldmatrix4(a, sa + (warp_m * 64 + mt * 16 + (lane & 15)) * FP_LD + kk + (lane >> 4) * 8);
#pragma unroll
      for (int q = 0; q < 4; ++q) tp_mma_bf16(acc.v[mt][q], a, b[q >> 1][(q & 1) * 2], b[q >> 1][(q & 1) * 2 + 1]);
    }
  }
}

// a_row(r): row r's K elements or nullptr; b_row(m, n): row n of matrix m or nullptr; `valid`: any mapped address;
// `rows`: rows of the tile that are there (the first ones): a warp multiplies only its 16-row tiles that hold any, so a
// tile of a few rows (a decode step) costs its weights' copies and little else
template <int NB, typename ARow, typename BRow>
__device__ __forceinline__ void fast_tile_product(unsigned char* smem, FpAcc& acc, int K, const void* valid, int rows, ARow a_row,
                                                  BRow b_row) {
  using bf = __nv_bfloat16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int warp_m = warp >> 2, warp_n = warp & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc.v[i][j][e] = 0.f;
  // a thread copies two pieces of 16 bytes of A and two of B per stage: rows tid / 4 and tid / 4 + 64, piece tid % 4
  const int prow = tid >> 2, pk = (tid & 3) * 8;
  constexpr int BN = FpShape<NB>::BN;
  const bf* ap[2] = {a_row(prow), a_row(prow + 64)};
  const bf* bp[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = prow + 64 * i;                  // staged row of B: matrix r / BN, its row r % BN
    bp[i] = NB == 1 ? b_row(0, r) : b_row(r / BN, r % BN);
  }
  const int steps = (K + FP_BK - 1) / FP_BK;
  const int my_tiles = min(4, max(0, (rows - warp_m * 64 + 15) / 16));     // of this warp's four 16-row tiles
  auto issue = [&](int step) {
    bf* sa = reinterpret_cast<bf*>(smem + (size_t)(step % FP_STAGES) * FP_STAGE_BYTES);
    bf* sb = sa + FP_BM * FP_LD;
    const int k = step * FP_BK + pk;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const bool a_ok = ap[i] != nullptr && k < K, b_ok = bp[i] != nullptr && k < K;
      fp_cp16(sa + (prow + 64 * i) * FP_LD + pk, a_ok ? (const void*)(ap[i] + k) : valid, a_ok ? 16 : 0);
      fp_cp16(sb + (prow + 64 * i) * FP_LD + pk, b_ok ? (const void*)(bp[i] + k) : valid, b_ok ? 16 : 0);
    }
  };
#pragma unroll
  for (int s = 0; s < FP_STAGES - 1; ++s) {
    if (s < steps) issue(s);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  }
  for (int step = 0; step < steps; ++step) {
    asm volatile("cp.async.wait_group %0;\n" :: "n"(FP_STAGES - 2) : "memory");
    __syncthreads();                              // the stage has landed for everybody; the stage refilled below was read a step ago
    if (step + FP_STAGES - 1 < steps) issue(step + FP_STAGES - 1);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    const bf* sa = reinterpret_cast<const bf*>(smem + (size_t)(step % FP_STAGES) * FP_STAGE_BYTES);
    const bf* sb = sa + FP_BM * FP_LD;
    if (my_tiles == 4) fp_stage_mma<NB, true>(sa, sb, acc, warp_m, warp_n, lane, 4);
    else if (my_tiles > 0) fp_stage_mma<NB, false>(sa, sb, acc, warp_m, warp_n, lane, my_tiles);
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

// f(row in tile, column in tile, value of matrix 0, value of matrix 1 (NB = 2) or 0)
template <int NB, typename F>
__device__ __forceinline__ void fast_tile_for_each(const FpAcc& acc, F f) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int warp_m = warp >> 2, warp_n = warp & 3;
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int q = 0; q < (NB == 1 ? 4 : 2); ++q)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = warp_m * 64 + mt * 16 + g + (e >> 1) * 8;
        const int col = (NB == 1 ? warp_n * 32 : warp_n * 16) + q * 8 + 2 * c + (e & 1);
        f(row, col, acc.v[mt][q][e], NB == 1 ? 0.f : acc.v[mt][q + 2][e]);
      }
}
