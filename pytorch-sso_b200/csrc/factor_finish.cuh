// Finishing step of the tensor-core factor kernels, done by the producing kernel itself.
//
// A factor launch is a grid of (tile, split) CTAs; every CTA leaves a 128x128 fp32 partial tile in
// the scratch.  Instead of a second launch that sums the splits, the CTA that finishes LAST for a
// tile does it: each CTA publishes its partial tile (store, __threadfence), takes a ticket from a
// counter of its tile, and the holder of the last ticket reads all partial tiles back IN SPLIT
// ORDER, so the sum does not depend on which CTA happens to be last (deterministic, and both
// halves of the symmetric result come from the same numbers: bitwise symmetric).  With many splits
// the sum runs in two levels - the last CTA of each group of ~sqrt(S) splits sums its group into the
// group's first slot, the last group to finish sums the group results - so that no single CTA has
// to stream all S tiles.  With one split the accumulator goes straight from registers to the
// output through shared memory and the scratch is not touched at all.
// Used for factors whose columns need no reordering (1x1 convolutions, Linear layers, every G
// factor) and that have few splits; factors of k x k convolutions keep the separate finishing
// kernel, whose job is the (kh,kw,c) -> (c,kh,kw) permutation across tiles, and so do problems with
// many splits of few tiles, where one CTA per tile streaming all partial tiles is slower than a
// kernel that spreads them over every SM (measured: d = 256 from 100352 rows, 49 splits of 3
// tiles, 33 us with the separate kernel against 62 us).
#pragma once
#include "common.cuh"
#include "factor_params.cuh"

namespace sso {
namespace fin {

constexpr int T = 128;
constexpr int CT_LD = T + 1;          // staging tile pitch (floats): conflict-free row and column walks
constexpr int MAX_GROUPS = 16;

__host__ __device__ inline int group_size(int splits) {
  if (splits <= 6) return splits;
  int g = 1;
  while (g * g < splits) ++g;
  return g;
}

// Sum `count` partial tiles that lie `stride` tiles apart, in index order, into the staging tile
// (or, for a group sum, back into the first of them).  Rows >= vr hold nothing.
template <int NT>
__device__ __forceinline__ void sum_tiles(const float* __restrict__ first, int count, int64_t stride_floats,
                                          int vr, float* __restrict__ ct, float* __restrict__ gdst, int tid) {
  for (int e = tid; e < vr * (T / 4); e += NT) {
    const int r = e / (T / 4), c4 = (e % (T / 4)) * 4;
    const float* src = first + r * T + c4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    // loads in batches of four (independent, all in flight together); the adds keep the index order
    for (int s0 = 0; s0 < count; s0 += 4) {
      float4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        v[k] = (s0 + k < count) ? __ldcg(reinterpret_cast<const float4*>(src + (int64_t)(s0 + k) * stride_floats))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k = 0; k < 4; ++k) { a.x += v[k].x; a.y += v[k].y; a.z += v[k].z; a.w += v[k].w; }
    }
    if (gdst) {
      *reinterpret_cast<float4*>(gdst + r * T + c4) = a;
    } else {
      float* d = ct + r * CT_LD + c4;
      d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w;
    }
  }
}

// out <- alpha * tile + beta * out for tile (bi, bj) of the lower triangle, plus its mirror.
template <int NT>
__device__ __forceinline__ void write_tile(const FactorParams& p, int bi, int bj, const float* __restrict__ ct, int tid) {
  const int warp = tid >> 5, lane = tid & 31, nw = NT / 32;
  const int vr = min(T, p.d - bi * T), vc = min(T, p.d - bj * T);
  const bool bad = p.status && *reinterpret_cast<volatile int*>(p.status) != 0;
  const float nanv = __int_as_float(0x7fc00000);
  const bool diag = (bi == bj);
  // Rows go four at a time: with beta != 0 the old values of all four (16 loads per lane) are fetched
  // before the first store; row by row, each load would wait behind the previous row's stores to the
  // same array, a chain of round trips to L2 as long as the tile is high.
  // pass 0: the tile itself (row r of the tile, lanes along its columns); pass 1: its mirror
  for (int pass = 0; pass < (diag ? 1 : 2); ++pass) {
    const int rows = pass == 0 ? vr : vc, cols = pass == 0 ? vc : vr;
    float* obase = pass == 0 ? p.out + (int64_t)(bi * T) * p.ldo + bj * T : p.out + (int64_t)(bj * T) * p.ldo + bi * T;
    for (int r0 = warp; r0 < rows; r0 += 4 * nw) {
      float old[4][T / 32];
      if (p.beta != 0.f) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int u = 0; u < T / 32; ++u) {
            const int r = r0 + j * nw, c = lane + 32 * u;
            old[j][u] = (r < rows && c < cols) ? obase[(int64_t)r * p.ldo + c] : 0.f;
          }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int u = 0; u < T / 32; ++u) {
          const int r = r0 + j * nw, c = lane + 32 * u;
          if (r < rows && c < cols) {
            // diagonal tile: the value above the diagonal is the mirrored one, so that out == out^T bit for bit
            float v = pass == 0 ? p.alpha * ((diag && c > r) ? ct[c * CT_LD + r] : ct[r * CT_LD + c])
                                : p.alpha * ct[c * CT_LD + r];
            if (bad) v = nanv;
            obase[(int64_t)r * p.ldo + c] = (p.beta == 0.f) ? v : fmaf(p.beta, old[j][u], v);
          }
        }
    }
  }
}

// Called by every thread of the CTA after its partial tile has been stored and fenced (or, with one
// split, after the accumulator has been placed in `ct`).  `flag` is a shared-memory word.
template <int NT>
__device__ __forceinline__ void finish_tile(const FactorParams& p, int tile, int bi, int bj, int split,
                                            float* __restrict__ ct, int* flag, int tid) {
  const int S = p.splits;
  if (S > 1) {
    const int gs = group_size(S), ng = ceil_div(S, gs);
    const int g = split / gs, gcount = min(gs, S - g * gs);
    float* tile0 = p.partial + (int64_t)tile * S * (T * T);
    const int vr = min(T, p.d - bi * T);
    int* t1 = p.tickets + p.ticket_tiles + tile * MAX_GROUPS + g;
    int* t2 = p.tickets + tile;
    __syncthreads();                 // every thread's partial-tile stores are fenced
    if (tid == 0) {
      const int t = atomicAdd(t1, 1);
      *flag = (t == gcount - 1);
      if (t == gcount - 1) *t1 = 0;  // leave the counter ready for the next launch
    }
    __syncthreads();
    if (!*flag) return;
    __threadfence();
    if (ng == 1) {
      sum_tiles<NT>(tile0, S, T * T, vr, ct, nullptr, tid);
    } else {
      float* gfirst = tile0 + (int64_t)g * gs * (T * T);
      sum_tiles<NT>(gfirst, gcount, T * T, vr, nullptr, gfirst, tid);
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int t = atomicAdd(t2, 1);
        *flag = (t == ng - 1);
        if (t == ng - 1) *t2 = 0;
      }
      __syncthreads();
      if (!*flag) return;
      __threadfence();
      sum_tiles<NT>(tile0, ng, (int64_t)gs * (T * T), vr, ct, nullptr, tid);
    }
  }
  __syncthreads();
  write_tile<NT>(p, bi, bj, ct, tid);
}

}  // namespace fin
}  // namespace sso
