// HBM-streaming kernels of the K-FAC path: EMA / scaled accumulation over flat factor pools,
// BatchNorm diagonal curvature, diagonal inverse + precondition, triangular pack / unpack.
// All are bandwidth bound: 16-byte vector accesses where alignment allows, grids sized as a
// multiple of the 148 SMs with a grid-stride loop.
#include <algorithm>

#include "common.cuh"

namespace sso {

constexpr int kSMs = 148;

__device__ __forceinline__ float ema_op(float data, float ema, float beta, float omb) {
  return fmaf(beta, data, omb * ema);
}

// dst <- a*src + b*dst  (b == 0: dst is not read)
__global__ void __launch_bounds__(256) axpby_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                    int64_t count, float a, float b) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
  if (vec) {
    const int64_t n4 = count >> 2;
    const float4* s4 = reinterpret_cast<const float4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
    for (int64_t i = tid; i < n4; i += stride) {
      const float4 s = __ldg(s4 + i);
      float4 o;
      if (b == 0.f) {
        o = make_float4(a * s.x, a * s.y, a * s.z, a * s.w);
      } else {
        const float4 d = d4[i];
        o = make_float4(fmaf(a, s.x, b * d.x), fmaf(a, s.y, b * d.y), fmaf(a, s.z, b * d.z), fmaf(a, s.w, b * d.w));
      }
      d4[i] = o;
    }
    for (int64_t i = (n4 << 2) + tid; i < count; i += stride)
      dst[i] = (b == 0.f) ? a * src[i] : fmaf(a, src[i], b * dst[i]);
  } else {
    for (int64_t i = tid; i < count; i += stride)
      dst[i] = (b == 0.f) ? a * src[i] : fmaf(a, src[i], b * dst[i]);
  }
}

static int grid_for(int64_t count, int per_thread) {
  const int64_t want = ceil_div64(count, (int64_t)256 * per_thread);
  const int64_t cap = (int64_t)kSMs * 8;
  return (int)std::max<int64_t>(1, std::min(want, cap));
}

// ------------------------------------------------------------------------------------------
// BatchNorm diagonal curvature
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) bn_plane_sums_pcontig(const T* __restrict__ y, const T* __restrict__ g,
                                                             int n, int c, int hw, int64_t syn, int64_t syc, int64_t syp,
                                                             int64_t sgn, int64_t sgc, int64_t sgp,
                                                             const float* __restrict__ scale,
                                                             const float* __restrict__ shift,
                                                             float* __restrict__ sx, float* __restrict__ sg) {
  // one warp per (n, c) plane
  const int warp = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (warp >= n * c) return;
  const int in = warp / c, ic = warp % c;
  const float inv_scale = scale ? 1.f / scale[ic] : 1.f, sh = shift ? shift[ic] : 0.f;
  const T* py = y + (int64_t)in * syn + (int64_t)ic * syc;
  const T* pg = g + (int64_t)in * sgn + (int64_t)ic * sgc;
  float ax = 0.f, ag = 0.f;
  for (int p = lane; p < hw; p += 32) {
    if (y) {
      const float xv = (to_f32<T>(py[(int64_t)p * syp]) - sh) * inv_scale;
      ax = fmaf(xv, xv, ax);
    }
    if (g) {
      const float gv = to_f32<T>(pg[(int64_t)p * sgp]);
      ag = fmaf(gv, gv, ag);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ax += __shfl_xor_sync(0xffffffffu, ax, o);
    ag += __shfl_xor_sync(0xffffffffu, ag, o);
  }
  if (lane == 0) {
    if (y) sx[warp] = ax;
    if (g) sg[warp] = ag;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) bn_plane_sums_ccontig(const T* __restrict__ y, const T* __restrict__ g,
                                                             int n, int c, int hw, int64_t syn, int64_t syc, int64_t syp,
                                                             int64_t sgn, int64_t sgc, int64_t sgp,
                                                             const float* __restrict__ scale,
                                                             const float* __restrict__ shift,
                                                             float* __restrict__ sx, float* __restrict__ sg) {
  // block = 32 channels x 8 pixel lanes; grid = (ceil(c/32), n)
  __shared__ float rx[8][33], rg[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int ic = blockIdx.x * 32 + tx, in = blockIdx.y;
  float ax = 0.f, ag = 0.f;
  if (ic < c) {
    const float inv_scale = scale ? 1.f / scale[ic] : 1.f, sh = shift ? shift[ic] : 0.f;
    const T* py = y + (int64_t)in * syn + (int64_t)ic * syc;
    const T* pg = g + (int64_t)in * sgn + (int64_t)ic * sgc;
    for (int p = ty; p < hw; p += 8) {
      if (y) {
        const float xv = (to_f32<T>(py[(int64_t)p * syp]) - sh) * inv_scale;
        ax = fmaf(xv, xv, ax);
      }
      if (g) {
        const float gv = to_f32<T>(pg[(int64_t)p * sgp]);
        ag = fmaf(gv, gv, ag);
      }
    }
  }
  rx[ty][tx] = ax;
  rg[ty][tx] = ag;
  __syncthreads();
  if (ty == 0 && ic < c) {
    float tx_sum = 0.f, tg_sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      tx_sum += rx[i][tx];
      tg_sum += rg[i][tx];
    }
    if (y) sx[(int64_t)in * c + ic] = tx_sum;
    if (g) sg[(int64_t)in * c + ic] = tg_sum;
  }
}

// Channels-contiguous planes, vectorised: a thread owns V = 16 bytes / sizeof(T) consecutive channels
// and walks pixels; LP lanes cover one pixel's channels (LP*V >= c), 256/LP pixels are processed in
// parallel per block, and the pixel range of one image is cut into `splits` blocks.  Partial sums go
// to out[(n*splits + split)*c + channel]; the finishing kernel adds the splits.
template <typename T, bool IS_Y>
__global__ void __launch_bounds__(256) bn_plane_sums_vec(const T* __restrict__ t, int c, int hw, int64_t sn,
                                                         int64_t sp, int lp, int splits,
                                                         const float* __restrict__ scale,
                                                         const float* __restrict__ shift,
                                                         float* __restrict__ out) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float red[256][V + 1];
  const int cv = threadIdx.x % lp, pp = threadIdx.x / lp, npp = 256 / lp;
  const int in = blockIdx.y, split = blockIdx.x;
  const int per = (hw + splits - 1) / splits;
  const int p0 = split * per, p1 = min(hw, p0 + per);
  const int c0 = cv * V;
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  if (c0 < c) {
    float isc[V], sh[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
      isc[i] = (IS_Y && scale) ? 1.f / scale[c0 + i] : 1.f;
      sh[i] = (IS_Y && shift) ? shift[c0 + i] : 0.f;
    }
    const T* base = t + (int64_t)in * sn + c0;
    auto add = [&](const uint4& raw) {
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float v = (to_f32<T>(e[i]) - sh[i]) * isc[i];
        acc[i] = fmaf(v, v, acc[i]);
      }
    };
    int p = p0 + pp;
    for (; p + 3 * npp < p1; p += 4 * npp) {      // four independent 16-byte loads in flight per thread
      const uint4 r0 = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)p * sp));
      const uint4 r1 = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)(p + npp) * sp));
      const uint4 r2 = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)(p + 2 * npp) * sp));
      const uint4 r3 = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)(p + 3 * npp) * sp));
      add(r0); add(r1); add(r2); add(r3);
    }
    for (; p < p1; p += npp) add(__ldg(reinterpret_cast<const uint4*>(base + (int64_t)p * sp)));
  }
#pragma unroll
  for (int i = 0; i < V; ++i) red[threadIdx.x][i] = acc[i];
  __syncthreads();
  if (pp == 0 && c0 < c) {
    float* o = out + ((int64_t)in * splits + split) * c + c0;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float sum = 0.f;
      for (int q = 0; q < npp; ++q) sum += red[q * lp + cv][i];
      o[i] = sum;
    }
  }
}

// block = 8 channels x 32 image lanes: with the usual 32..256 images a thread owns one to eight
// images, issues the loads of all their split partials back to back, and the 32 lanes are combined
// in shared memory (fixed order: deterministic).  Many small blocks keep this latency-bound step short.
__global__ void __launch_bounds__(256) bn_finish_kernel(const float* __restrict__ sx, const float* __restrict__ sg,
                                                        const float* __restrict__ weight, int n, int c,
                                                        int splits_x, int splits_g, float alpha, float beta,
                                                        float* __restrict__ w_out, float* __restrict__ b_out) {
  __shared__ float rw[32][9], rb[32][9];
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  const int ic = blockIdx.x * 8 + tx;
  float aw = 0.f, ab = 0.f;
  if (ic < c) {
    for (int in = ty; in < n; in += 32) {
      const float* px = sx + (int64_t)in * splits_x * c + ic;
      const float* pg = sg + (int64_t)in * splits_g * c + ic;
      float x0 = 0.f, x1 = 0.f, g0 = 0.f, g1 = 0.f;
      int q = 0;
      for (; q + 1 < splits_x; q += 2) { x0 += px[(int64_t)q * c]; x1 += px[(int64_t)(q + 1) * c]; }
      if (q < splits_x) x0 += px[(int64_t)q * c];
      for (q = 0; q + 1 < splits_g; q += 2) { g0 += pg[(int64_t)q * c]; g1 += pg[(int64_t)(q + 1) * c]; }
      if (q < splits_g) g0 += pg[(int64_t)q * c];
      const float gsum = (weight ? weight[in] : 1.f) * (g0 + g1);
      aw = fmaf(x0 + x1, gsum, aw);
      ab += gsum;
    }
  }
  rw[ty][tx] = aw;
  rb[ty][tx] = ab;
  __syncthreads();
  if (ty == 0 && ic < c) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) { tw += rw[i][tx]; tb += rb[i][tx]; }
    const float s = alpha / (float)n;
    w_out[ic] = (beta == 0.f) ? s * tw : fmaf(beta, w_out[ic], s * tw);
    if (b_out) b_out[ic] = (beta == 0.f) ? s * tb : fmaf(beta, b_out[ic], s * tb);
  }
}

// pixel-range splits of the vectorised kernel for a [n, c, hw] tensor (1 when it is not used)
static int bn_vec_lanes(int64_t c, int vec) {
  if (c % vec != 0 || c / vec > 256) return 0;
  int lp = 1;
  while (lp < c / vec) lp <<= 1;
  return lp;
}
static int bn_vec_splits(int64_t n, int64_t c, int64_t hw, int vec) {
  const int lp = bn_vec_lanes(c, vec);
  if (lp == 0 || hw <= 1) return 1;
  const int npp = 256 / lp;
  int64_t s = ceil_div64(4 * kSMs, n);                       // about four blocks per SM
  const int64_t most = std::max<int64_t>(1, hw / (8 * npp)); // at least eight pixels per lane
  if (s > most) s = most;
  return (int)std::max<int64_t>(1, s);
}

template <typename T>
static int bn_sums_typed(const void* y, const void* g, int64_t n, int64_t c, int64_t hw, int64_t syn,
                         int64_t syc, int64_t syp, int64_t sgn, int64_t sgc, int64_t sgp,
                         const float* scale, const float* shift, float* sx, float* sg, int splits,
                         cudaStream_t st) {
  const T* ty = reinterpret_cast<const T*>(y);
  const T* tg = reinterpret_cast<const T*>(g);
  constexpr int V = 16 / sizeof(T);
  const int lp = bn_vec_lanes(c, V);
  auto vec_ok = [&](const T* p, int64_t sc_, int64_t sn_, int64_t sp_) {
    return p != nullptr && sc_ == 1 && lp > 0 && hw > 1 && (reinterpret_cast<uintptr_t>(p) & 15) == 0 &&
           (sn_ * sizeof(T)) % 16 == 0 && (sp_ * sizeof(T)) % 16 == 0;
  };
  if (splits > 1 || (vec_ok(ty, syc, syn, syp) || !y) && (vec_ok(tg, sgc, sgn, sgp) || !g) && hw > 1 && lp > 0) {
    SSO_CHECK_ARG((!y || vec_ok(ty, syc, syn, syp)) && (!g || vec_ok(tg, sgc, sgn, sgp)),
                  "bn_plane_sums: splits > 1 needs channels-contiguous, 16-byte aligned planes");
    dim3 grid((unsigned)splits, (unsigned)n);
    if (y) {
      bn_plane_sums_vec<T, true><<<grid, 256, 0, st>>>(ty, (int)c, (int)hw, syn, syp, lp, splits, scale, shift, sx);
      SSO_LAUNCH_OK("bn_plane_sums_vec");
    }
    if (g) {
      bn_plane_sums_vec<T, false><<<grid, 256, 0, st>>>(tg, (int)c, (int)hw, sgn, sgp, lp, splits, nullptr, nullptr, sg);
      SSO_LAUNCH_OK("bn_plane_sums_vec");
    }
    return 0;
  }
  if (syc == 1 && sgc == 1 && hw > 1) {
    dim3 grid((unsigned)ceil_div64(c, 32), (unsigned)n);
    bn_plane_sums_ccontig<T><<<grid, 256, 0, st>>>(ty, tg, (int)n, (int)c, (int)hw, syn, syc, syp, sgn, sgc,
                                                    sgp, scale, shift, sx, sg);
  } else {
    const int64_t warps = n * c;
    bn_plane_sums_pcontig<T><<<(unsigned)ceil_div64(warps * 32, 256), 256, 0, st>>>(
        ty, tg, (int)n, (int)c, (int)hw, syn, syc, syp, sgn, sgc, sgp, scale, shift, sx, sg);
  }
  SSO_LAUNCH_OK("bn_plane_sums");
  return 0;
}

// ------------------------------------------------------------------------------------------
// diagonal inverse / precondition
// ------------------------------------------------------------------------------------------
__global__ void diag_inv_precond_kernel(const float* __restrict__ ema, float* __restrict__ inv,
                                        float* __restrict__ grad, int64_t count, float damping,
                                        int use_sqrt, int update_inv) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
    float v;
    if (update_inv) {
      float x = ema[i];
      if (use_sqrt) x = sqrtf(x);
      v = 1.f / (x + damping);
      inv[i] = v;
    } else {
      v = inv[i];
    }
    if (grad) grad[i] *= v;
  }
}

// ------------------------------------------------------------------------------------------
// triangular pack / unpack over a table of row runs
// ------------------------------------------------------------------------------------------
// Both kernels read through the read-only path in batches of four loads per thread: the source and the
// destination come out of one record, so with plain loads every load would wait for the previous store.
__global__ void __launch_bounds__(256) tri_pack_kernel(const sso_tri_rec* __restrict__ recs, float scale) {
  const sso_tri_rec r = recs[blockIdx.x];
  for (int row = r.row0; row < r.row0 + r.nrows; ++row) {
    const int64_t base = (int64_t)r.n * row - (int64_t)row * (row + 1) / 2;
    const float* src = r.m + (int64_t)row * r.ld;
    float* dst = r.packed + base;
    for (int x0 = row + threadIdx.x; x0 < r.n; x0 += 4 * 256) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = (x0 + 256 * u < r.n) ? __ldg(src + x0 + 256 * u) : 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (x0 + 256 * u < r.n) dst[x0 + 256 * u] = scale * v[u];
    }
  }
}
// A record of at most 32 rows: the part on and above the diagonal is copied row by row (contiguous in the
// packed form); the part below it is the transpose of packed rows, moved in 32 x 32 tiles through shared
// memory so that the packed rows are read and the matrix rows written in whole 128-byte lines.  Longer
// records take the element-wise path (strided reads below the diagonal).
__global__ void __launch_bounds__(256) tri_unpack_kernel(const sso_tri_rec* __restrict__ recs, float scale,
                                                         int symmetric) {
  __shared__ float tile[2][32][33];
  const sso_tri_rec r = recs[blockIdx.x];
  const int n = r.n, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* pk = r.packed;
  auto base = [n](int row) { return (int64_t)n * row - (int64_t)row * (row + 1) / 2; };
  if (r.nrows > 32) {
    if (blockIdx.y != 0) return;
    for (int row = r.row0; row < r.row0 + r.nrows; ++row) {
      float* dst = r.m + (int64_t)row * r.ld;
      for (int x = tid; x < n; x += 256) {
        const int lo = min(row, x), hi = max(row, x);
        const float v = scale * __ldg(pk + base(lo) + hi);
        dst[x] = (symmetric || x >= row) ? v : 0.f;
      }
    }
    return;
  }
  // gridDim.y CTAs share a record: rows of the upper part and tiles of the lower part are dealt round robin
  const int part = blockIdx.y, parts = gridDim.y;
  for (int rr = part; rr < r.nrows; rr += parts) {
    const int row = r.row0 + rr;
    const float* src = pk + base(row);
    float* dst = r.m + (int64_t)row * r.ld;
    for (int x0 = row + tid; x0 < n; x0 += 4 * 256) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = (x0 + 256 * u < n) ? __ldg(src + x0 + 256 * u) : 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (x0 + 256 * u < n) dst[x0 + 256 * u] = scale * v[u];
    }
  }
  const int xend = r.row0 + r.nrows - 1;        // columns x < xend have elements below the diagonal in this band
  int buf = 0;
  for (int x0 = 32 * part; x0 < xend; x0 += 32 * parts, buf ^= 1) {
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int x = x0 + warp + 8 * k, row = r.row0 + lane;
      v[k] = (symmetric && lane < r.nrows && x < row) ? __ldg(pk + base(x) + row) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) tile[buf][warp + 8 * k][lane] = v[k];
    __syncthreads();          // (two buffers: the next tile's stores cannot overtake this tile's reads)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int rr = warp + 8 * k, row = r.row0 + rr, x = x0 + lane;
      if (rr < r.nrows && x < row) r.m[(int64_t)row * r.ld + x] = scale * tile[buf][lane][rr];
    }
  }
}

// scaled copies of many flat segments in one launch (one CTA per record)
__global__ void __launch_bounds__(256) copy_segments_kernel(const sso_seg_rec* __restrict__ recs, float scale) {
  const sso_seg_rec r = recs[blockIdx.x];
  const bool vec = ((reinterpret_cast<uintptr_t>(r.src) | reinterpret_cast<uintptr_t>(r.dst)) & 15) == 0;
  if (vec) {
    const int64_t n4 = r.count >> 2;
    // four 16-byte loads in flight per thread: one at a time leaves an SM with ~10 KB on its way to it
    for (int64_t i0 = threadIdx.x; i0 < n4; i0 += 4 * 256) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + 256 * u < n4) v[u] = __ldg(reinterpret_cast<const float4*>(r.src) + i0 + 256 * u);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + 256 * u < n4)
          reinterpret_cast<float4*>(r.dst)[i0 + 256 * u] = make_float4(scale * v[u].x, scale * v[u].y, scale * v[u].z, scale * v[u].w);
    }
    for (int64_t i = (n4 << 2) + threadIdx.x; i < r.count; i += 256) r.dst[i] = scale * r.src[i];
  } else {
    for (int64_t i = threadIdx.x; i < r.count; i += 256) r.dst[i] = scale * r.src[i];
  }
}

__global__ void __launch_bounds__(256) optimizer_tail_kernel(const sso_tail_rec* __restrict__ recs) {
  const sso_tail_rec r = recs[blockIdx.x];
  for (int64_t i = threadIdx.x; i < r.count; i += 256) {
    const float pv = r.p[i];
    float g = r.g[i];
    g = fmaf(r.add, pv, g);
    if (r.mbuf) {
      g = fmaf(r.momentum, r.mbuf[i], g);
      r.mbuf[i] = g;
    }
    if (r.ebuf) {
      g = fmaf(r.ema, g, (1.f - r.ema) * r.ebuf[i]);
      r.ebuf[i] = g;
    }
    g *= r.scale;
    r.g[i] = g;
    if (r.lr != 0.f) r.p[i] = fmaf(-r.lr, g, pv);
  }
}

}  // namespace sso

using namespace sso;

// ---- 16-bit wire format of the exchange ---------------------------------------------------------
// A packed fp32 buffer is a sequence of arrays; a chunk record names a run of elements of one array.
// absmax: maxima[array] = max |x| (non-negative floats order like their bit patterns, so an integer
// atomicMax gives a deterministic result).  encode: out16 = cast(x * 65000 / sums[array]).
// decode: out32 = float(x16) * sums[array] / 65000.  `sums` holds the per-array maxima summed over
// the ranks, so that the sum of the scaled values of all ranks stays inside the fp16 range.
__global__ void __launch_bounds__(256) wire_absmax_kernel(const float* __restrict__ buf, const sso_wire_rec* __restrict__ recs,
                                                          float* __restrict__ maxima) {
  const sso_wire_rec r = recs[blockIdx.x];
  const float* src = buf + r.offset;
  float m = 0.f;
  for (int64_t i = threadIdx.x; i < r.count; i += 256) m = fmaxf(m, fabsf(src[i]));
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float sm[8];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) m = fmaxf(m, sm[w]);
    if (!(m == m)) m = __int_as_float(0x7f800000);     // a NaN in the array: scale by infinity's reciprocal
    atomicMax(reinterpret_cast<int*>(maxima + r.array), __float_as_int(m));
  }
}

template <typename T>
__device__ __forceinline__ T wire_cast(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 wire_cast<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half wire_cast<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) wire_encode_kernel(const float* __restrict__ buf, const sso_wire_rec* __restrict__ recs,
                                                          const float* __restrict__ sums, T* __restrict__ out) {
  const sso_wire_rec r = recs[blockIdx.x];
  const float s = sums[r.array];
  const float scale = (s > 0.f && s < __int_as_float(0x7f800000)) ? 65000.f / s : 1.f;
  const float* src = buf + r.offset;
  T* dst = out + r.offset;
  for (int64_t i = threadIdx.x; i < r.count; i += 256) dst[i] = wire_cast<T>(src[i] * scale);
}

template <typename T>
__global__ void __launch_bounds__(256) wire_decode_kernel(const T* __restrict__ in, const sso_wire_rec* __restrict__ recs,
                                                          const float* __restrict__ sums, float* __restrict__ out) {
  const sso_wire_rec r = recs[blockIdx.x];
  const float s = sums[r.array];
  const float scale = (s > 0.f && s < __int_as_float(0x7f800000)) ? s / 65000.f : 1.f;
  const T* src = in + r.offset;
  float* dst = out + r.offset;
  for (int64_t i = threadIdx.x; i < r.count; i += 256) dst[i] = to_f32<T>(src[i]) * scale;
}

extern "C" {

int sso_optimizer_tail(const sso_tail_rec* recs_dev, int n_recs, void* stream) {
  SSO_CHECK_ARG(recs_dev != nullptr && n_recs >= 0, "optimizer_tail: bad argument");
  if (n_recs == 0) return 0;
  optimizer_tail_kernel<<<n_recs, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(recs_dev);
  SSO_LAUNCH_OK("optimizer_tail_kernel");
  return 0;
}

int sso_axpby(const float* src, float* dst, int64_t count, float a, float b, void* stream) {
  SSO_CHECK_ARG(src && dst && count >= 0, "axpby: bad argument");
  if (count == 0) return 0;
  axpby_kernel<<<grid_for(count, 16), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(src, dst, count, a, b);
  SSO_LAUNCH_OK("axpby_kernel");
  return 0;
}

int sso_ema_update(const float* data, float* ema, int64_t count, float beta, int first, void* stream) {
  // first (or beta == 1): ema <- data; else ema <- beta*data + (1-beta)*ema
  if (first || beta == 1.f) return sso_axpby(data, ema, count, 1.f, 0.f, stream);
  return sso_axpby(data, ema, count, beta, 1.f - beta, stream);
}

int sso_bn_plane_splits(int dtype, int64_t n, int64_t c, int64_t hw, int64_t stride_c) {
  if (stride_c != 1) return 1;
  return bn_vec_splits(n, c, hw, dtype == SSO_F32 ? 4 : 8);
}

int sso_bn_plane_sums(const void* y, const void* g, int dtype, int64_t n, int64_t c, int64_t hw,
                      int64_t syn, int64_t syc, int64_t syp, int64_t sgn, int64_t sgc, int64_t sgp,
                      const float* scale, const float* shift, float* sx, float* sg, int splits, void* stream) {
  SSO_CHECK_ARG((y && sx) || (g && sg), "bn_plane_sums: nothing to do");
  SSO_CHECK_ARG(!y || sx, "bn_plane_sums: y without sx");
  SSO_CHECK_ARG(!g || sg, "bn_plane_sums: g without sg");
  SSO_CHECK_ARG(n > 0 && c > 0 && hw > 0 && n * c < (int64_t)1 << 26 && splits >= 1, "bn_plane_sums: bad shape");
  if (!y) { syn = sgn; syc = sgc; syp = sgp; }
  if (!g) { sgn = syn; sgc = syc; sgp = syp; }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SSO_F32:
      return bn_sums_typed<float>(y, g, n, c, hw, syn, syc, syp, sgn, sgc, sgp, scale, shift, sx, sg, splits, st);
    case SSO_BF16:
      return bn_sums_typed<__nv_bfloat16>(y, g, n, c, hw, syn, syc, syp, sgn, sgc, sgp, scale, shift, sx, sg, splits, st);
    case SSO_F16:
      return bn_sums_typed<__half>(y, g, n, c, hw, syn, syc, syp, sgn, sgc, sgp, scale, shift, sx, sg, splits, st);
  }
  return fail(-1, "bn_plane_sums: unknown dtype %d", dtype);
}

int sso_bn_diag_finish(const float* sx, const float* sg, const float* sample_weight, int64_t n, int64_t c,
                       int splits_x, int splits_g, float alpha, float beta, float* w_out, float* b_out,
                       void* stream) {
  SSO_CHECK_ARG(sx && sg && w_out && n > 0 && c > 0 && splits_x >= 1 && splits_g >= 1, "bn_diag_finish: bad argument");
  bn_finish_kernel<<<(unsigned)ceil_div64(c, 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      sx, sg, sample_weight, (int)n, (int)c, splits_x, splits_g, alpha, beta, w_out, b_out);
  SSO_LAUNCH_OK("bn_finish_kernel");
  return 0;
}

int sso_diag_inv_precondition(const float* ema, float* inv, float* grad, int64_t count, float damping,
                              int use_sqrt, int update_inv, void* stream) {
  SSO_CHECK_ARG(inv && count >= 0 && (ema || !update_inv), "diag_inv_precondition: bad argument");
  if (count == 0) return 0;
  diag_inv_precond_kernel<<<grid_for(count, 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ema, inv, grad, count, damping, use_sqrt, update_inv);
  SSO_LAUNCH_OK("diag_inv_precond_kernel");
  return 0;
}

int sso_tri_pack(const sso_tri_rec* recs_dev, int n_recs, float scale, void* stream) {
  SSO_CHECK_ARG(recs_dev && n_recs >= 0, "tri_pack: bad argument");
  if (n_recs == 0) return 0;
  tri_pack_kernel<<<n_recs, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(recs_dev, scale);
  SSO_LAUNCH_OK("tri_pack_kernel");
  return 0;
}

int sso_tri_unpack(const sso_tri_rec* recs_dev, int n_recs, float scale, int symmetric, void* stream) {
  SSO_CHECK_ARG(recs_dev && n_recs >= 0, "tri_unpack: bad argument");
  if (n_recs == 0) return 0;
  tri_unpack_kernel<<<dim3((unsigned)n_recs, 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(recs_dev, scale, symmetric);
  SSO_LAUNCH_OK("tri_unpack_kernel");
  return 0;
}

int sso_copy_segments(const sso_seg_rec* recs_dev, int n_recs, float scale, void* stream) {
  SSO_CHECK_ARG(recs_dev && n_recs >= 0, "copy_segments: bad argument");
  if (n_recs == 0) return 0;
  copy_segments_kernel<<<n_recs, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(recs_dev, scale);
  SSO_LAUNCH_OK("copy_segments_kernel");
  return 0;
}

int sso_wire_absmax(const float* buf, const sso_wire_rec* recs_dev, int n_recs, float* maxima, void* stream) {
  SSO_CHECK_ARG(buf && recs_dev && maxima && n_recs >= 0, "wire_absmax: bad argument");
  if (n_recs == 0) return 0;
  wire_absmax_kernel<<<n_recs, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(buf, recs_dev, maxima);
  SSO_LAUNCH_OK("wire_absmax_kernel");
  return 0;
}

int sso_wire_encode(const float* buf, const sso_wire_rec* recs_dev, int n_recs, const float* sums, void* out16,
                    int dtype, void* stream) {
  SSO_CHECK_ARG(buf && recs_dev && sums && out16 && n_recs >= 0, "wire_encode: bad argument");
  SSO_CHECK_ARG(dtype == SSO_BF16 || dtype == SSO_F16, "wire_encode: the wire type must be bf16 or fp16");
  if (n_recs == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == SSO_BF16)
    wire_encode_kernel<__nv_bfloat16><<<n_recs, 256, 0, st>>>(buf, recs_dev, sums, static_cast<__nv_bfloat16*>(out16));
  else
    wire_encode_kernel<__half><<<n_recs, 256, 0, st>>>(buf, recs_dev, sums, static_cast<__half*>(out16));
  SSO_LAUNCH_OK("wire_encode_kernel");
  return 0;
}

int sso_wire_decode(const void* in16, const sso_wire_rec* recs_dev, int n_recs, const float* sums, float* out32,
                    int dtype, void* stream) {
  SSO_CHECK_ARG(in16 && recs_dev && sums && out32 && n_recs >= 0, "wire_decode: bad argument");
  SSO_CHECK_ARG(dtype == SSO_BF16 || dtype == SSO_F16, "wire_decode: the wire type must be bf16 or fp16");
  if (n_recs == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == SSO_BF16)
    wire_decode_kernel<__nv_bfloat16><<<n_recs, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in16), recs_dev, sums, out32);
  else
    wire_decode_kernel<__half><<<n_recs, 256, 0, st>>>(static_cast<const __half*>(in16), recs_dev, sums, out32);
  SSO_LAUNCH_OK("wire_decode_kernel");
  return 0;
}

}  // extern "C"
