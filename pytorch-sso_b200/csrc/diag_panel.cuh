// Diagonal block of a 128-column Cholesky panel, done by one CTA: L = chol(D) and L^-1 for a
// (<=128)x(<=128) SPD block D, all in fp32 FMA arithmetic.
//
// The block is distributed cyclically over a 16x16 thread grid: thread (ty, tx) holds the elements
// (ty + 16 i, tx + 16 j), i >= j, in registers, so that every thread owns a piece of every 16-column
// panel and of every trailing block (the work stays balanced while the trailing matrix shrinks, and
// the 16 threads of a row of the grid touch 16 consecutive shared-memory rows, which at a pitch of 132
// floats are 4 banks apart: 16-byte loads without conflicts).  Right-looking over panels of 16 columns:
//   publish : the owners write panel k (rows >= 16 k) into shared memory
//   factor  : one warp, lane = row, factorises the 16x16 diagonal block with shuffles (16 pivots, each a
//             broadcast of the pivot, an rsqrt, a column scale and a rank-1 update of the lane's row)
//   solve   : one thread per row below solves its 16 unknowns against that block (forward substitution)
//   update  : every thread subtracts the panel's outer product from its registers
// i.e. three block barriers per 16 columns instead of one per column.  The finished factor sits in shared
// memory; its inverse follows by the inverses of the eight 16x16 diagonal blocks (one warp each, lane =
// column) and three levels of doubling, Inv21 = -Inv22 * (L21 * Inv11), with the product L21 * Inv11
// parked in the (otherwise unused) upper triangle.  Rows and columns past the block's size behave as an
// identity block.  A non-positive or NaN pivot is recorded once per matrix (LAPACK numbering) and
// replaced by 1, like the 64-wide kernel does.
#pragma once
#include "common.cuh"

namespace sso {
namespace dpanel {

constexpr int PN = 128;        // rows / columns handled by one CTA
constexpr int PP = 132;        // pitch of the shared-memory matrices (floats)
constexpr int PK = 16;         // panel width inside the block
constexpr int THREADS = 256;
constexpr size_t SMEM_BYTES = (size_t)(2 * PN * PP + PN) * sizeof(float);

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float x, float y, float z, float w) {
  *reinterpret_cast<float4*>(p) = make_float4(x, y, z, w);
}

// One level of the doubling for the range [lo, lo + 2 SZ): first product (stage 0)
//     Y = L21 * Inv11      -> S rows lo.., columns lo + SZ..  (scratch above the diagonal)
// then (stage 1)            Inv21 = -Inv22 * Y.
// Thread (ty, tx) computes the outputs (ty + 16 a, tx + 16 b).  Inv11 and Inv22 are lower triangular: the
// half of the inner range that only meets zeros of a whole half of the output is skipped.
template <int SZ>
__device__ __forceinline__ void doubling_product(float* __restrict__ S, float* __restrict__ V, int lo, int stage,
                                                 int ty, int tx) {
  constexpr int NT = SZ / 16;
  constexpr int NH = NT >= 2 ? NT / 2 : NT;
  const int mid = lo + SZ;
  float acc[NT][NT];
#pragma unroll
  for (int a = 0; a < NT; ++a)
#pragma unroll
    for (int b = 0; b < NT; ++b) acc[a][b] = 0.f;
  if (stage == 0) {
    // Y[r][c] = sum_q L[mid + r][lo + q] * Inv[lo + q][lo + c], Inv11[q][c] = 0 for q < c
    const float* Lr = S + (mid + ty) * PP + lo;
    const float* Vc = V + lo * PP + lo + tx;
#pragma unroll 4
    for (int q = 0; q < SZ / 2; ++q) {      // meets the columns of the first half only (all of them if NT == 1)
      float l[NT];
#pragma unroll
      for (int a = 0; a < NT; ++a) l[a] = Lr[16 * a * PP + q];
#pragma unroll
      for (int b = 0; b < NH; ++b) {
        const float v = Vc[q * PP + 16 * b];
#pragma unroll
        for (int a = 0; a < NT; ++a) acc[a][b] = fmaf(l[a], v, acc[a][b]);
      }
    }
#pragma unroll 4
    for (int q = SZ / 2; q < SZ; ++q) {
      float l[NT];
#pragma unroll
      for (int a = 0; a < NT; ++a) l[a] = Lr[16 * a * PP + q];
#pragma unroll
      for (int b = 0; b < NT; ++b) {
        const float v = Vc[q * PP + 16 * b];
#pragma unroll
        for (int a = 0; a < NT; ++a) acc[a][b] = fmaf(l[a], v, acc[a][b]);
      }
    }
    float* Y = S + (lo + ty) * PP + mid + tx;
#pragma unroll
    for (int a = 0; a < NT; ++a)
#pragma unroll
      for (int b = 0; b < NT; ++b) Y[16 * a * PP + 16 * b] = acc[a][b];
  } else {
    // Inv21[r][c] = -sum_q Inv[mid + r][mid + q] * Y[q][c], Inv22[r][q] = 0 for q > r
    const float* Vr = V + (mid + ty) * PP + mid;
    const float* Yc = S + lo * PP + mid + tx;
#pragma unroll 4
    for (int q = 0; q < SZ / 2; ++q) {
      float y[NT];
#pragma unroll
      for (int b = 0; b < NT; ++b) y[b] = Yc[q * PP + 16 * b];
#pragma unroll
      for (int a = 0; a < NT; ++a) {
        const float v = Vr[16 * a * PP + q];
#pragma unroll
        for (int b = 0; b < NT; ++b) acc[a][b] = fmaf(v, y[b], acc[a][b]);
      }
    }
#pragma unroll 4
    for (int q = SZ / 2; q < SZ; ++q) {     // meets the rows of the second half only (all of them if NT == 1)
      float y[NT];
#pragma unroll
      for (int b = 0; b < NT; ++b) y[b] = Yc[q * PP + 16 * b];
#pragma unroll
      for (int a = NT - NH; a < NT; ++a) {
        const float v = Vr[16 * a * PP + q];
#pragma unroll
        for (int b = 0; b < NT; ++b) acc[a][b] = fmaf(v, y[b], acc[a][b]);
      }
    }
    float* O = V + (mid + ty) * PP + lo + tx;
#pragma unroll
    for (int a = 0; a < NT; ++a)
#pragma unroll
      for (int b = 0; b < NT; ++b) O[16 * a * PP + 16 * b] = -acc[a][b];
  }
}

template <int SZ>
__device__ __forceinline__ void doubling_level(float* S, float* V, int cols, int ty, int tx) {
  // ranges whose second half lies past the matrix (identity padding) keep Inv21 = 0
  for (int lo = 0; lo + SZ < cols; lo += 2 * SZ) doubling_product<SZ>(S, V, lo, 0, ty, tx);
  __syncthreads();
  for (int lo = 0; lo + SZ < cols; lo += 2 * SZ) doubling_product<SZ>(S, V, lo, 1, ty, tx);
  __syncthreads();
}

__global__ void __launch_bounds__(THREADS, 1) diag_panel_kernel(const sso_diag_rec* __restrict__ recs,
                                                               int* __restrict__ info) {
  extern __shared__ __align__(16) float psm[];
  float* S = psm;               // panels of the block as they are published, then L (lower triangle)
  float* V = psm + PN * PP;     // L^-1
  float* dinv = V + PN * PP;    // 1 / L_jj
  const sso_diag_rec rec = recs[blockIdx.x];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ty = tid >> 4, tx = tid & 15;
  const int n = rec.size;
  const int np = (n + PK - 1) / PK;     // panels that hold columns of the matrix
  const int cols = np * PK;

  float a[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j <= i; ++j) {
      const int r = ty + 16 * i, c = tx + 16 * j;
      float v = (r == c) ? 1.f : 0.f;
      if (r < n && c <= r) v = rec.L[(int64_t)r * rec.ld_l + c];
      a[i][j] = v;
    }
  for (int e = tid; e < PN * PP / 4; e += THREADS) st4(V + 4 * e, 0.f, 0.f, 0.f, 0.f);
  if (tid < PN) dinv[tid] = 1.f;

  for (int k = 0; k < np; ++k) {
    const int c0 = PK * k;
    // ---- publish panel k
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j == k) {
#pragma unroll
        for (int i = j; i < 8; ++i) S[(ty + 16 * i) * PP + c0 + tx] = a[i][j];
      }
    __syncthreads();
    // ---- 16x16 diagonal block: lane l (and its twin l + 16) holds row l
    if (warp == 0) {
      const int l = lane & 15;
      float* row = S + (c0 + l) * PP + c0;
      float r[PK];
#pragma unroll
      for (int q = 0; q < PK; q += 4) {
        const float4 v = ld4(row + q);
        r[q] = v.x; r[q + 1] = v.y; r[q + 2] = v.z; r[q + 3] = v.w;
      }
#pragma unroll
      for (int c = 0; c < PK; ++c)
        if (c > l) r[c] = 0.f;
#pragma unroll
      for (int j = 0; j < PK; ++j) {
        float pv = __shfl_sync(0xffffffffu, r[j], j);
        if (!(pv > 0.f)) {      // non-positive or NaN pivot: record once, continue with 1
          if (lane == 0 && info && c0 + j < n)
            atomicCAS(info + 2 * rec.mat + rec.info_slot, 0, rec.row0 + c0 + j + 1);
          pv = 1.f;
        }
        const float rs = rsqrtf(pv);
        const float lj = (l == j) ? sqrtf(pv) : r[j] * rs;      // rows above the pivot hold 0
        r[j] = lj;
        if (lane == j) dinv[c0 + j] = rs;
#pragma unroll
        for (int c = j + 1; c < PK; ++c) {
          const float t = __shfl_sync(0xffffffffu, lj, c);       // L[c][j]
          r[c] = fmaf(-lj, t, r[c]);                             // only columns c <= l are kept below
        }
      }
      if (lane < PK) {
#pragma unroll
        for (int q = 0; q < PK; q += 4)
          st4(row + q, q <= l ? r[q] : 0.f, q + 1 <= l ? r[q + 1] : 0.f, q + 2 <= l ? r[q + 2] : 0.f,
              q + 3 <= l ? r[q + 3] : 0.f);
      }
    }
    __syncthreads();
    // ---- rows below the diagonal block: x * L16^T = a, one thread per row
    {
      const int rowi = c0 + PK + tid;
      if (rowi < cols) {
        float* xr = S + rowi * PP + c0;
        float x[PK];
#pragma unroll
        for (int q = 0; q < PK; q += 4) {
          const float4 v = ld4(xr + q);
          x[q] = v.x; x[q + 1] = v.y; x[q + 2] = v.z; x[q + 3] = v.w;
        }
#pragma unroll
        for (int c = 0; c < PK; ++c) {
          const float* lrow = S + (c0 + c) * PP + c0;    // same address in every lane: broadcast
          float lr[PK];
#pragma unroll
          for (int q = 0; q < c; q += 4) {
            const float4 v = ld4(lrow + q);
            lr[q] = v.x; lr[q + 1] = v.y; lr[q + 2] = v.z; lr[q + 3] = v.w;
          }
          float s = x[c];
#pragma unroll
          for (int q = 0; q < c; ++q) s = fmaf(-x[q], lr[q], s);
          x[c] = s * dinv[c0 + c];
        }
#pragma unroll
        for (int q = 0; q < PK; q += 4) st4(xr + q, x[q], x[q + 1], x[q + 2], x[q + 3]);
      }
    }
    __syncthreads();
    // ---- trailing update: a[i][j] -= sum_q L[row_i][c0 + q] * L[col_j][c0 + q] for k < j <= i
    if (k + 1 < np) {
#pragma unroll
      for (int qc = 0; qc < PK / 4; ++qc) {
        float4 rv[8];
#pragma unroll
        for (int i = 1; i < 8; ++i) {
          rv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (i > k && i < np) rv[i] = ld4(S + (ty + 16 * i) * PP + c0 + 4 * qc);
        }
#pragma unroll
        for (int j = 1; j < 8; ++j)
          if (j > k && j < np) {
            const float4 cv = ld4(S + (tx + 16 * j) * PP + c0 + 4 * qc);
#pragma unroll
            for (int i = j; i < 8; ++i) {
              float t = a[i][j];
              t = fmaf(-rv[i].x, cv.x, t);
              t = fmaf(-rv[i].y, cv.y, t);
              t = fmaf(-rv[i].z, cv.z, t);
              t = fmaf(-rv[i].w, cv.w, t);
              a[i][j] = t;
            }
          }
      }
    }
  }
  // ---- identity padding of the factor (columns that hold no matrix column were never published)
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (j >= np) {
#pragma unroll
      for (int i = j; i < 8; ++i) S[(ty + 16 * i) * PP + 16 * j + tx] = (i == j && ty == tx) ? 1.f : 0.f;
    }
  __syncthreads();
  // ---- inverses of the 16x16 diagonal blocks: warp w, lane c = column c of block w
  if (lane < PK) {
    const int b0 = PK * warp, c = lane;
    if (warp < np) {
      float x[PK];
#pragma unroll
      for (int r = 0; r < PK; ++r) {
        const float* lrow = S + (b0 + r) * PP + b0;
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < r; ++q) s = fmaf(lrow[q], x[q], s);     // x[q] = 0 for q < c
        const float d = dinv[b0 + r];
        x[r] = (r < c) ? 0.f : (r == c ? d : -s * d);
      }
#pragma unroll
      for (int r = 0; r < PK; ++r) V[(b0 + r) * PP + b0 + c] = x[r];
    } else {
      V[(b0 + c) * PP + b0 + c] = 1.f;
    }
  }
  __syncthreads();
  doubling_level<16>(S, V, cols, ty, tx);
  doubling_level<32>(S, V, cols, ty, tx);
  doubling_level<64>(S, V, cols, ty, tx);
  // ---- results: L (lower, zeros above), L^-1 (same) and optionally its transpose
  for (int e = tid; e < n * PN; e += THREADS) {
    const int r = e >> 7, c = e & (PN - 1);
    if (c < n) {
      const bool low = c <= r;
      rec.L[(int64_t)r * rec.ld_l + c] = low ? S[r * PP + c] : 0.f;
      rec.Linv[(int64_t)r * rec.ld_inv + c] = low ? V[r * PP + c] : 0.f;
      if (rec.LinvT) rec.LinvT[(int64_t)r * rec.ld_invt + c] = (c >= r) ? V[c * PP + r] : 0.f;
    }
  }
}

}  // namespace dpanel
}  // namespace sso
