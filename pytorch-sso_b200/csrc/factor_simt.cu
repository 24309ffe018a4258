// Kronecker-factor construction, fp32 SIMT path:  out = alpha * sum_r w_r u_r u_r^T + beta * out
// with u_r gathered on the fly from the layer input (implicit im2col).  This is the exact-fp32
// path (plain FFMA accumulation); the tensor-core path lives in factor_tc.cu.
//
// Work decomposition: lower-triangle 128x128 output tiles x row splits.  Each CTA accumulates
// its split of the rows; if there is more than one split the partial tiles go to a workspace
// and a second kernel sums them in a fixed order (deterministic, no atomics), applies
// alpha/beta and writes both triangles.
#include "common.cuh"
#include "factor_params.cuh"

namespace sso {

template <typename T>
__device__ __forceinline__ float fetch(const FactorParams& p, const RowInfo& r, const ColInfo& c) {
  if (!r.valid || c.kind == 2) return 0.f;
  if (c.kind == 1) return 1.f;
  const int ih = r.ih0 + c.dh, iw = r.iw0 + c.dw;
  if ((unsigned)ih >= (unsigned)p.h || (unsigned)iw >= (unsigned)p.w) return 0.f;
  const T* px = reinterpret_cast<const T*>(p.x) + (r.base + c.off + (int64_t)ih * p.sh + (int64_t)iw * p.sw);
  return to_f32<T>(__ldg(px));
}

// ROW_CONTIG: consecutive im2col rows are (mostly) consecutive in memory (NCHW); otherwise
// consecutive columns are (channels_last, plain row-major matrices).
template <typename T, bool ROW_CONTIG>
__global__ void __launch_bounds__(256) factor_syrk_simt_kernel(const FactorParams p) {
  constexpr int MT = 8, TILE = 128, PER = TILE * KT / 256;  // 16 elements per thread per operand
  __shared__ __align__(16) float As[KT * TILE];
  __shared__ __align__(16) float Bs[KT * TILE];
  __shared__ RowInfo rinfo[2][KT];
  __shared__ ColInfo cinfo[2][TILE];

  const int tid = threadIdx.x;
  int bi, bj;
  tri_decode(blockIdx.x, bi, bj);
  const bool diag = (bi == bj);
  const bool share = diag && (p.weight == nullptr);  // B tile identical to A tile
  const int split = blockIdx.y;
  const int64_t r_begin = (int64_t)split * p.rows_per_split;
  const int64_t r_end = min(p.rows, r_begin + (int64_t)p.rows_per_split);
  const int nkt = (int)ceil_div64(max((int64_t)0, r_end - r_begin), KT);

  // column tables for both operands
  for (int i = tid; i < 2 * TILE; i += 256) {
    const int op = i / TILE, cl = i % TILE;
    const int col = (op == 0 ? bi : bj) * TILE + cl;
    ColInfo ci;
    ci.pad = 0;
    if (col < p.dcols) {
      const int kk = p.kh * p.kw;
      const int ch = col / kk, rem = col - ch * kk;
      const int ky = rem / p.kw, kx = rem - ky * p.kw;
      ci.off = (int64_t)ch * p.sc;
      ci.dh = ky * p.dil_h;
      ci.dw = kx * p.dil_w;
      ci.kind = 0;
    } else {
      ci.off = 0; ci.dh = 0; ci.dw = 0;
      ci.kind = (col < p.d) ? 1 : 2;
    }
    cinfo[op][cl] = ci;
  }
  auto fill_rows = [&](int kt, int buf) {
    if (tid < KT) {
      const int64_t r = r_begin + (int64_t)kt * KT + tid;
      RowInfo ri;
      if (r < r_end) {
        const int hw = p.ho * p.wo;
        const int nn = (int)(r / hw);
        const int rem = (int)(r - (int64_t)nn * hw);
        const int oy = rem / p.wo, ox = rem - oy * p.wo;
        ri.base = (int64_t)nn * p.sn;
        ri.ih0 = oy * p.stride_h - p.pad_h;
        ri.iw0 = ox * p.stride_w - p.pad_w;
        ri.wgt = p.weight ? p.weight[nn] : 1.f;
        ri.valid = 1;
      } else {
        ri.base = 0; ri.ih0 = 0; ri.iw0 = 0; ri.wgt = 0.f; ri.valid = 0;
      }
      rinfo[buf][tid] = ri;
    }
  };

  float ra[PER], rb[PER];
  auto load_regs = [&](int buf) {
    if (ROW_CONTIG) {
      const int k = tid & 31, cg = tid >> 5;  // 8 column groups of 4
      const RowInfo ri = rinfo[buf][k];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int cl = cg * 4 + 32 * i + q;
          ra[i * 4 + q] = fetch<T>(p, ri, cinfo[0][cl]) * ri.wgt;
          if (!share) rb[i * 4 + q] = fetch<T>(p, ri, cinfo[1][cl]);
        }
    } else {
      const int cl = tid & 127, k0 = tid >> 7;
      const ColInfo ca = cinfo[0][cl], cb = cinfo[1][cl];
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const RowInfo ri = rinfo[buf][k0 + 2 * i];
        ra[i] = fetch<T>(p, ri, ca) * ri.wgt;
        if (!share) rb[i] = fetch<T>(p, ri, cb);
      }
    }
  };
  auto store_smem = [&]() {
    if (ROW_CONTIG) {
      const int k = tid & 31, cg = tid >> 5;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int cl = cg * 4 + 32 * i;
        *reinterpret_cast<float4*>(As + k * TILE + swz(k, cl)) =
            make_float4(ra[i * 4], ra[i * 4 + 1], ra[i * 4 + 2], ra[i * 4 + 3]);
        if (!share)
          *reinterpret_cast<float4*>(Bs + k * TILE + swz(k, cl)) =
              make_float4(rb[i * 4], rb[i * 4 + 1], rb[i * 4 + 2], rb[i * 4 + 3]);
      }
    } else {
      const int cl = tid & 127, k0 = tid >> 7;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int k = k0 + 2 * i;
        As[k * TILE + swz(k, cl)] = ra[i];
        if (!share) Bs[k * TILE + swz(k, cl)] = rb[i];
      }
    }
  };

  float acc[MT][MT];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[i][j] = 0.f;
  const int ty = tid >> 4, tx = tid & 15;

  fill_rows(0, 0);
  __syncthreads();
  if (nkt > 0) {
    load_regs(0);
    fill_rows(1, 1);
    store_smem();
  }
  __syncthreads();
  for (int kt = 0; kt < nkt; ++kt) {
    if (kt + 1 < nkt) load_regs((kt + 1) & 1);
    TileCore<MT>::compute(As, share ? As : Bs, ty, tx, acc);
    __syncthreads();
    if (kt + 1 < nkt) {
      store_smem();
      fill_rows(kt + 2, kt & 1);
    }
    __syncthreads();
  }

  // epilogue
  if (p.splits > 1) {
    float* dst = p.partial + ((int64_t)blockIdx.x * p.splits + split) * (TILE * TILE);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const int r = TileCore<MT>::row_of(ty, i);
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const int c0 = g * 64 + tx * 4;
        *reinterpret_cast<float4*>(dst + r * TILE + c0) =
            make_float4(acc[i][g * 4], acc[i][g * 4 + 1], acc[i][g * 4 + 2], acc[i][g * 4 + 3]);
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    const int gr = bi * TILE + TileCore<MT>::row_of(ty, i);
    if (gr >= p.d) continue;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int gc = bj * TILE + TileCore<MT>::col_of(tx, j);
      if (gc >= p.d) continue;
      float* o = p.out + (int64_t)gr * p.ldo + gc;
      const float v = p.alpha * acc[i][j];
      // beta == 0 must not read (the buffer may hold NaNs from a fresh allocation)
      if (!diag) {
        float* o2 = p.out + (int64_t)gc * p.ldo + gr;
        *o2 = (p.beta == 0.f) ? v : fmaf(p.beta, *o2, v);
      }
      *o = (p.beta == 0.f) ? v : fmaf(p.beta, *o, v);
    }
  }
}

// Sum the split partials in split order and finish the tile.
__global__ void __launch_bounds__(256) factor_reduce_kernel(const FactorParams p) {
  constexpr int TILE = 128;
  int bi, bj;
  tri_decode(blockIdx.x, bi, bj);
  const float* src = p.partial + (int64_t)blockIdx.x * p.splits * (TILE * TILE);
  const int e0 = (blockIdx.y * 256 + threadIdx.x) * 4;  // 4 consecutive columns of one row
  const int r = e0 / TILE, c0 = e0 % TILE;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sp = 0; sp < p.splits; ++sp) {
    const float4 v = *reinterpret_cast<const float4*>(src + (int64_t)sp * (TILE * TILE) + e0);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  const int gr = bi * TILE + r;
  if (gr >= p.d) return;
  const float vals[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int gc = bj * TILE + c0 + q;
    if (gc >= p.d) continue;
    const float v = p.alpha * vals[q];
    float* o = p.out + (int64_t)gr * p.ldo + gc;
    if (bi != bj) {
      float* o2 = p.out + (int64_t)gc * p.ldo + gr;
      *o2 = (p.beta == 0.f) ? v : fmaf(p.beta, *o2, v);
    }
    *o = (p.beta == 0.f) ? v : fmaf(p.beta, *o, v);
  }
}

// rows per split: bounded above so that a sequential fp32 sum stays well inside the 1e-5
// factor tolerance, and chosen so that the grid covers the 148 SMs about twice.
static void choose_splits(int64_t rows, int tiles, int& splits, int& rows_per_split) {
  const int64_t kMaxRowsPerSplit = 4096;
  const int kTargetCtas = 2 * 148;
  int64_t s = ceil_div64(rows, kMaxRowsPerSplit);
  const int64_t want = ceil_div64(kTargetCtas, tiles);
  const int64_t most = ceil_div64(rows, 4 * KT);  // at least 128 rows per split
  if (s < want) s = want;
  if (s > most) s = most;
  if (s < 1) s = 1;
  int64_t rps = ceil_div64(rows, s);
  rps = ceil_div64(rps, KT) * KT;
  splits = (int)ceil_div64(rows, rps);
  if (splits < 1) splits = 1;
  rows_per_split = (int)rps;
}

size_t factor_simt_workspace_bytes(int64_t rows, int64_t d) {
  const int nb = (int)ceil_div64(d, 128);
  const int tiles = nb * (nb + 1) / 2;
  int splits, rps;
  choose_splits(rows, tiles, splits, rps);
  return splits > 1 ? (size_t)tiles * splits * 128 * 128 * sizeof(float) : 0;
}

template <typename T>
static int launch_typed(const FactorParams& p, int tiles, bool row_contig, cudaStream_t st) {
  dim3 grid(tiles, p.splits);
  if (row_contig)
    factor_syrk_simt_kernel<T, true><<<grid, 256, 0, st>>>(p);
  else
    factor_syrk_simt_kernel<T, false><<<grid, 256, 0, st>>>(p);
  SSO_LAUNCH_OK("factor_syrk_simt_kernel");
  if (p.splits > 1) {
    factor_reduce_kernel<<<dim3(tiles, 128 * 128 / (256 * 4)), 256, 0, st>>>(p);
    SSO_LAUNCH_OK("factor_reduce_kernel");
  }
  return 0;
}

int factor_simt_launch(FactorParams p, int dtype, void* workspace, size_t workspace_bytes,
                       cudaStream_t st) {
  const int nb = ceil_div(p.d, 128);
  const int tiles = nb * (nb + 1) / 2;
  choose_splits(p.rows, tiles, p.splits, p.rows_per_split);
  if (p.splits > 1) {
    const size_t need = (size_t)tiles * p.splits * 128 * 128 * sizeof(float);
    SSO_CHECK_ARG(workspace != nullptr && workspace_bytes >= need,
                  "factor workspace too small: need %zu bytes, got %zu", need, workspace_bytes);
    p.partial = reinterpret_cast<float*>(workspace);
  }
  // consecutive rows are consecutive in memory when the innermost stride is along w
  const bool row_contig = (p.sw == 1 && p.sc != 1);
  switch (dtype) {
    case SSO_F32: return launch_typed<float>(p, tiles, row_contig, st);
    case SSO_BF16: return launch_typed<__nv_bfloat16>(p, tiles, row_contig, st);
    case SSO_F16: return launch_typed<__half>(p, tiles, row_contig, st);
  }
  return fail(-1, "unknown dtype %d", dtype);
}

}  // namespace sso
