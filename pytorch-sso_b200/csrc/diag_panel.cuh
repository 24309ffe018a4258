// Diagonal block of a 128-column Cholesky panel, done by one CTA: L = chol(D) and L^-1 for a
// (<=128)x(<=128) SPD block D, all in fp32 FMA arithmetic.
//
// The block is distributed cyclically over a 16x16 thread grid: thread (ty, tx) holds the elements
// (ty + 16 i, tx + 16 j), i >= j, in registers, so that every thread owns a piece of every 16-column
// panel and of every trailing block (the work stays balanced while the trailing matrix shrinks, and
// the 16 threads of a row of the grid touch 16 consecutive shared-memory rows, which at a pitch of 132
// floats are 4 banks apart: 16-byte loads without conflicts).  Right-looking over panels of 16 columns:
//   publish : the owners write panel k (rows >= 16 k) into shared memory
//   factor  : one warp, lane = row, factorises the 16x16 diagonal block: per pivot one round of shuffles
//             (the raw column, and the next diagonal element so that the next pivot's rsqrt starts early)
//   solve   : one thread per row below solves its 16 unknowns against that block (forward substitution)
//   update  : every thread subtracts the panel's outer product from its registers
// i.e. three block barriers per 16 columns instead of one per column.  The finished factor sits in shared
// memory; its inverse follows by the inverses of the eight 16x16 diagonal blocks (one warp each, lane =
// column) and three levels of doubling, Inv21 = -Inv22 * (L21 * Inv11), with the product L21 * Inv11
// parked in the (otherwise unused) upper triangle.  Rows and columns past the block's size behave as an
// identity block.  A pivot that is not a positive normal number (non-positive, denormal or NaN) is recorded
// once per matrix (LAPACK numbering) and replaced by 1, like the 64-wide kernel does for non-positive ones.
// Measured (d = 4608, 36 panels): 24 us per launch against 2 x 44 us for the two 64-wide factorisations plus
// 2 x 14 us of 64-wide panel tasks it replaces; what is left is bound by shared-memory bandwidth (trailing
// update and doubling products: 16-byte loads cost four cycles each for the whole SM) and by the chain of
// 128 pivots (86 cycles each).
#pragma once
#include "common.cuh"

namespace sso {
namespace dpanel {

constexpr int PN = 128;        // rows / columns handled by one CTA
constexpr int PP = 132;        // pitch of the shared-memory matrices (floats)
constexpr int PK = 16;         // panel width inside the block
constexpr int THREADS = 256;
constexpr size_t SMEM_BYTES = (size_t)(2 * PN * PP + PN) * sizeof(float);

// MUFU.RSQ alone (2 ulp); the argument is a positive normal number wherever this is called
__device__ __forceinline__ float rsqrt_approx(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
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
#pragma unroll 8
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
#pragma unroll 8
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
#pragma unroll 8
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
#pragma unroll 8
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

// Panel K of the thread's elements goes to shared memory (rows >= 16 K).
template <int K>
__device__ __forceinline__ void publish_panel(const float (&a)[8][8], float* __restrict__ S, int ty, int tx) {
#pragma unroll
  for (int i = K; i < 8; ++i) S[(ty + 16 * i) * PP + PK * K + tx] = a[i][K];
}

// a[i][j] -= sum_q L[row_i][16 K + q] * L[col_j][16 K + q] for K < j <= i, four q at a time.  K is a template
// parameter so that the loop body is straight-line code: a branch per block column costs a single warp
// more than the multiply-adds it guards.  Rows past the matrix hold zeros in the published panel.
template <int K>
__device__ __forceinline__ void update_trailing(float (&a)[8][8], const float* __restrict__ S, int ty, int tx) {
  if (K >= 7) return;
  const float* rbase = S + ty * PP + PK * K;
  const float* cbase = S + tx * PP + PK * K;
#pragma unroll 1
  for (int qc = 0; qc < PK / 4; ++qc) {
    float4 rv[8], cv[8];
#pragma unroll
    for (int i = K + 1; i < 8; ++i) {
      rv[i] = ld4(rbase + 16 * i * PP + 4 * qc);
      cv[i] = ld4(cbase + 16 * i * PP + 4 * qc);
    }
    // one component of the four at a time over all pairs: consecutive multiply-adds are independent
#pragma unroll
    for (int j = K + 1; j < 8; ++j)
#pragma unroll
      for (int i = j; i < 8; ++i) a[i][j] = fmaf(-rv[i].x, cv[j].x, a[i][j]);
#pragma unroll
    for (int j = K + 1; j < 8; ++j)
#pragma unroll
      for (int i = j; i < 8; ++i) a[i][j] = fmaf(-rv[i].y, cv[j].y, a[i][j]);
#pragma unroll
    for (int j = K + 1; j < 8; ++j)
#pragma unroll
      for (int i = j; i < 8; ++i) a[i][j] = fmaf(-rv[i].z, cv[j].z, a[i][j]);
#pragma unroll
    for (int j = K + 1; j < 8; ++j)
#pragma unroll
      for (int i = j; i < 8; ++i) a[i][j] = fmaf(-rv[i].w, cv[j].w, a[i][j]);
  }
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
    switch (k) {
      case 0: publish_panel<0>(a, S, ty, tx); break;
      case 1: publish_panel<1>(a, S, ty, tx); break;
      case 2: publish_panel<2>(a, S, ty, tx); break;
      case 3: publish_panel<3>(a, S, ty, tx); break;
      case 4: publish_panel<4>(a, S, ty, tx); break;
      case 5: publish_panel<5>(a, S, ty, tx); break;
      case 6: publish_panel<6>(a, S, ty, tx); break;
      default: publish_panel<7>(a, S, ty, tx); break;
    }
    __syncthreads();
    // ---- 16x16 diagonal block by warp 0: lane l (and its twin l + 16) holds row l.  One exchange per pivot:
    // every lane fetches the raw column j (pivot included) from the lanes that own it, takes the rsqrt of
    // the pivot itself and applies the rank-1 update to its own row.
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
      // The pivot of step j + 1 is formed inside step j from the next raw diagonal element (fetched with
      // the column) by the same multiply-add its owner applies to it: the rsqrt of the next pivot then runs
      // while the shuffles of the next column are in flight, instead of after them.
      float pv = __shfl_sync(0xffffffffu, r[0], 0);
      int first_bad = -1;
#pragma unroll
      for (int j = 0; j < PK; ++j) {
        float t[PK];
#pragma unroll
        for (int c = j + 1; c < PK; ++c) t[c] = __shfl_sync(0xffffffffu, r[j], c);     // a[c][j], c > j
        float d1 = 0.f;
        if (j + 1 < PK) d1 = __shfl_sync(0xffffffffu, r[j + 1], j + 1);                // a[j+1][j+1] before this step
        // a pivot that is not a positive normal number (or is NaN) is remembered and replaced by 1; no branch
        // here: the chain from one pivot to the next is what bounds this kernel
        const bool bad = !(pv >= 1.17549435e-38f);
        if (bad && first_bad < 0) first_bad = j;
        pv = bad ? 1.f : pv;
        const float rs = rsqrt_approx(pv);
        const float lj = (l == j) ? pv * rs : r[j] * rs;      // L[l][j]; rows above the pivot hold 0
#pragma unroll
        for (int c = j + 1; c < PK; ++c) r[c] = fmaf(-lj, t[c] * rs, r[c]);            // kept for c <= l only
        r[j] = lj;
        if (lane == j) dinv[c0 + j] = rs;
        if (j + 1 < PK) {
          const float x = t[j + 1] * rs;
          pv = fmaf(-x, x, d1);
        }
      }
      if (first_bad >= 0 && lane == 0 && info && c0 + first_bad < n)
        atomicCAS(info + 2 * rec.mat + rec.info_slot, 0, rec.row0 + c0 + first_bad + 1);
      if (lane < PK) {
#pragma unroll
        for (int q = 0; q < PK; q += 4)
          st4(row + q, q <= l ? r[q] : 0.f, q + 1 <= l ? r[q + 1] : 0.f, q + 2 <= l ? r[q + 2] : 0.f,
              q + 3 <= l ? r[q + 3] : 0.f);
      }
    }
    __syncthreads();
    // ---- rows below the diagonal block: x * L16^T = a, one thread per row, right looking (each finished
    // unknown is subtracted from all later ones at once, so the dependent chain is two operations per step)
    {
      const int rowi = c0 + PK + tid;
      if (rowi < cols) {
        float* xr = S + rowi * PP + c0;
        const float* lblk = S + c0 * PP + c0;            // same addresses in every lane: broadcast
        float x[PK];
#pragma unroll
        for (int q = 0; q < PK; q += 4) {
          const float4 v = ld4(xr + q);
          x[q] = v.x; x[q + 1] = v.y; x[q + 2] = v.z; x[q + 3] = v.w;
        }
#pragma unroll
        for (int c = 0; c < PK; ++c) {
          x[c] *= dinv[c0 + c];
#pragma unroll
          for (int c2 = c + 1; c2 < PK; ++c2) x[c2] = fmaf(-x[c], lblk[c2 * PP + c], x[c2]);
        }
#pragma unroll
        for (int q = 0; q < PK; q += 4) st4(xr + q, x[q], x[q + 1], x[q + 2], x[q + 3]);
      }
    }
    __syncthreads();
    // ---- trailing update
    if (k + 1 < np) {
      switch (k) {
        case 0: update_trailing<0>(a, S, ty, tx); break;
        case 1: update_trailing<1>(a, S, ty, tx); break;
        case 2: update_trailing<2>(a, S, ty, tx); break;
        case 3: update_trailing<3>(a, S, ty, tx); break;
        case 4: update_trailing<4>(a, S, ty, tx); break;
        case 5: update_trailing<5>(a, S, ty, tx); break;
        default: update_trailing<6>(a, S, ty, tx); break;
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
  // ---- results: the lower triangle of L, L^-1 with zeros above its diagonal, and optionally the upper
  // triangle of the transpose of L^-1.  Nothing reads L above the diagonal, and the buffer of the transpose
  // is zeroed before the factorisation starts.
  for (int r = warp; r < n; r += THREADS / 32) {
    float* lrow = rec.L + (int64_t)r * rec.ld_l;
    float* vrow = rec.Linv + (int64_t)r * rec.ld_inv;
    float* trow = rec.LinvT ? rec.LinvT + (int64_t)r * rec.ld_invt : nullptr;
    float lv[4], vv[4], tv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {           // all loads of the row first, then all stores
      const int c = lane + 32 * u;
      lv[u] = S[r * PP + c];
      vv[u] = V[r * PP + c];
      tv[u] = V[c * PP + r];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = lane + 32 * u;
      if (c < n) {
        if (c <= r) lrow[c] = lv[u];
        vrow[c] = (c <= r) ? vv[u] : 0.f;     // read in full (K = 128) by the tasks of the rows below
        if (trow && c >= r) trow[c] = tv[u];
      }
    }
  }
}

}  // namespace dpanel
}  // namespace sso
