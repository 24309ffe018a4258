// Diagonal curvature of Linear / Conv2d layers: the mean over samples of the SQUARED per-sample
// weight gradient,
//     out_w[o][j] <- alpha * sum_b w_b * ( sum_l g[b,o,l] * u[b,l,j] )^2 + beta * out_w[o][j]
//     out_b[o]    <- alpha * sum_b w_b *   sum_l g[b,o,l]^2              + beta * out_b[o]
// with u the im2col rows of the layer input (never materialised), l the output pixels of one
// sample and j = (c, ky, kx) the weight's own column order; a Linear layer is the case of one
// pixel and a 1x1 kernel (then the square factorises into g^2 * a^2).
//
// Exact fp32 FFMA: one CTA owns a 64 x 64 tile of out_w and a range of the samples; per sample it
// accumulates the 64 x 64 per-sample gradient tile over the pixels (operands staged in shared
// memory, 4x4 register tile per thread), squares it into a second register tile and moves on.
// Sample ranges go to a workspace and are summed in a fixed order by a finishing kernel
// (deterministic, no atomics).
#include "common.cuh"

namespace sso {

struct DiagSqParams {
  const void* x;        // layer input  [n, c, h, w]   (element strides sxn, sxc, sxh, sxw)
  const void* g;        // output grad  [n, oc, ho, wo] (element strides sgn, sgc, sgh, sgw)
  const float* weight;  // per-sample weights, nullable
  float* partial;       // [splits][oc][d]
  int64_t sxn, sxc, sxh, sxw, sgn, sgc, sgh, sgw;
  int n, c, h, w, oc, ho, wo;
  int kh, kw, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int d;                // c*kh*kw
  int samples_per_split;
};

constexpr int DT = 64, DK = 16;

// ONE_PIXEL (a Linear layer): the square factorises, out[o][j] = sum_b w_b g[b,o]^2 x[b,j]^2, so
// the samples themselves are the contraction index and the operands are squared while staged.
template <typename T, bool ONE_PIXEL>
__global__ void __launch_bounds__(256) diag_sq_kernel(const DiagSqParams p) {
  __shared__ __align__(16) float Gs[DK][DT + 4];   // row pitch 68 floats: float4 rows stay 16-byte aligned
  __shared__ __align__(16) float Us[DK][DT + 4];
  __shared__ int64_t col_off[DT];
  __shared__ int col_dh[DT], col_dw[DT];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int o0 = blockIdx.x * DT, j0 = blockIdx.y * DT, split = blockIdx.z;
  const int b_begin = split * p.samples_per_split, b_end = min(p.n, b_begin + p.samples_per_split);
  const int L = p.ho * p.wo, kk = p.kh * p.kw;
  if (tid < DT) {
    const int j = j0 + tid;
    if (j < p.d) {
      const int ch = j / kk, rem = j - ch * kk, ky = rem / p.kw, kx = rem - ky * p.kw;
      col_off[tid] = (int64_t)ch * p.sxc;
      col_dh[tid] = ky * p.dil_h - p.pad_h;
      col_dw[tid] = kx * p.dil_w - p.pad_w;
    } else {
      col_off[tid] = -1; col_dh[tid] = 0; col_dw[tid] = 0;
    }
  }
  __syncthreads();
  const T* X = reinterpret_cast<const T*>(p.x);
  const T* G = reinterpret_cast<const T*>(p.g);
  float sq[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int q = 0; q < 4; ++q) sq[i][q] = 0.f;
  // staging map: thread -> (pixel ll = tid / 16, four consecutive tile columns 4*(tid % 16) ..)
  const int ll = tid >> 4, c4 = (tid & 15) * 4;
  if (ONE_PIXEL) {
    for (int b0 = b_begin; b0 < b_end; b0 += DK) {
      const int b = b0 + ll;
      const bool bv = b < b_end;
      const float wb = (bv && p.weight) ? p.weight[b] : 1.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int o = o0 + c4 + q;
        float gv = 0.f;
        if (bv && o < p.oc) gv = to_f32<T>(__ldg(G + (int64_t)b * p.sgn + (int64_t)o * p.sgc));
        Gs[ll][c4 + q] = wb * gv * gv;
        float uv = 0.f;
        const int64_t off = col_off[c4 + q];
        if (bv && off >= 0) uv = to_f32<T>(__ldg(X + (int64_t)b * p.sxn + off));
        Us[ll][c4 + q] = uv * uv;
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < DK; ++k) {
        const float4 g4 = *reinterpret_cast<const float4*>(&Gs[k][ty * 4]);
        const float4 u4 = *reinterpret_cast<const float4*>(&Us[k][tx * 4]);
        const float gr[4] = {g4.x, g4.y, g4.z, g4.w}, ur[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int q = 0; q < 4; ++q) sq[i][q] = fmaf(gr[i], ur[q], sq[i][q]);
      }
      __syncthreads();
    }
  }
  for (int b = ONE_PIXEL ? b_end : b_begin; b < b_end; ++b) {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[i][q] = 0.f;
    // the gathers of chunk l0 + DK are in flight while chunk l0 is multiplied
    T gv[4], uv[4];    // raw values: converted when stored, so that nothing waits on the loads here
    auto gather = [&](int l0) {
      const int l = l0 + ll;
      const bool lv = l < L;
      const int oy = lv ? l / p.wo : 0, ox = lv ? l - oy * p.wo : 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int o = o0 + c4 + q;
        gv[q] = T(0.f);
        if (lv && o < p.oc)
          gv[q] = __ldg(G + (int64_t)b * p.sgn + (int64_t)o * p.sgc + (int64_t)oy * p.sgh + (int64_t)ox * p.sgw);
        uv[q] = T(0.f);
        const int64_t off = col_off[c4 + q];
        if (lv && off >= 0) {
          const int ih = oy * p.stride_h + col_dh[c4 + q], iw = ox * p.stride_w + col_dw[c4 + q];
          if ((unsigned)ih < (unsigned)p.h && (unsigned)iw < (unsigned)p.w)
            uv[q] = __ldg(X + (int64_t)b * p.sxn + off + (int64_t)ih * p.sxh + (int64_t)iw * p.sxw);
        }
      }
    };
    gather(0);
    for (int l0 = 0; l0 < L; l0 += DK) {
      *reinterpret_cast<float4*>(&Gs[ll][c4]) = make_float4(to_f32<T>(gv[0]), to_f32<T>(gv[1]), to_f32<T>(gv[2]), to_f32<T>(gv[3]));
      *reinterpret_cast<float4*>(&Us[ll][c4]) = make_float4(to_f32<T>(uv[0]), to_f32<T>(uv[1]), to_f32<T>(uv[2]), to_f32<T>(uv[3]));
      __syncthreads();
      if (l0 + DK < L) gather(l0 + DK);
#pragma unroll
      for (int k = 0; k < DK; ++k) {
        const float4 g4 = *reinterpret_cast<const float4*>(&Gs[k][ty * 4]);
        const float4 u4 = *reinterpret_cast<const float4*>(&Us[k][tx * 4]);
        const float gr[4] = {g4.x, g4.y, g4.z, g4.w}, ur[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int q = 0; q < 4; ++q) acc[i][q] = fmaf(gr[i], ur[q], acc[i][q]);
      }
      __syncthreads();
    }
    const float wb = p.weight ? p.weight[b] : 1.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int q = 0; q < 4; ++q) sq[i][q] = fmaf(wb * acc[i][q], acc[i][q], sq[i][q]);
  }
  float* dst = p.partial + (int64_t)split * p.oc * p.d;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int o = o0 + ty * 4 + i;
    if (o >= p.oc) continue;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int j = j0 + tx * 4 + q;
      if (j < p.d) dst[(int64_t)o * p.d + j] = sq[i][q];
    }
  }
}

__global__ void __launch_bounds__(256) diag_sq_finish_kernel(const float* __restrict__ partial, int splits,
                                                             int64_t count, float alpha, float beta,
                                                             float* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= count) return;
  float s = 0.f;
  for (int sp = 0; sp < splits; ++sp) s += partial[(int64_t)sp * count + i];
  out[i] = (beta == 0.f) ? alpha * s : fmaf(beta, out[i], alpha * s);
}

// bias: one warp per output channel, samples and pixels summed in a fixed order
template <typename T>
__global__ void __launch_bounds__(256) diag_sq_bias_kernel(const DiagSqParams p, float alpha, float beta,
                                                           float* __restrict__ out_b) {
  const int o = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (o >= p.oc) return;
  const T* G = reinterpret_cast<const T*>(p.g);
  const int L = p.ho * p.wo;
  float tot = 0.f;
  for (int b = 0; b < p.n; ++b) {
    float s = 0.f;
    for (int l = lane; l < L; l += 32) {
      const int oy = l / p.wo, ox = l - oy * p.wo;
      const float v = to_f32<T>(__ldg(G + (int64_t)b * p.sgn + (int64_t)o * p.sgc + (int64_t)oy * p.sgh + (int64_t)ox * p.sgw));
      s = fmaf(v, v, s);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    tot = fmaf(p.weight ? p.weight[b] : 1.f, s, tot);
  }
  if (lane == 0) out_b[o] = (beta == 0.f) ? alpha * tot : fmaf(beta, out_b[o], alpha * tot);
}

static int diag_sq_splits(int n, int oc, int d) {
  const int64_t tiles = (int64_t)ceil_div(oc, DT) * ceil_div(d, DT);
  int s = (int)std::min<int64_t>(n, std::max<int64_t>(1, ceil_div64(2 * 148, tiles)));
  return s;
}

template <typename T>
static int diag_sq_typed(DiagSqParams p, float alpha, float beta, float* out_w, float* out_b, cudaStream_t st) {
  const int splits = ceil_div(p.n, p.samples_per_split);
  const dim3 grid(ceil_div(p.oc, DT), ceil_div(p.d, DT), splits);
  if (p.ho * p.wo == 1 && p.kh * p.kw == 1 && p.pad_h == 0 && p.pad_w == 0)
    diag_sq_kernel<T, true><<<grid, 256, 0, st>>>(p);
  else
    diag_sq_kernel<T, false><<<grid, 256, 0, st>>>(p);
  SSO_LAUNCH_OK("diag_sq_kernel");
  const int64_t count = (int64_t)p.oc * p.d;
  diag_sq_finish_kernel<<<(unsigned)ceil_div64(count, 256), 256, 0, st>>>(p.partial, splits, count, alpha, beta, out_w);
  SSO_LAUNCH_OK("diag_sq_finish_kernel");
  if (out_b) {
    diag_sq_bias_kernel<T><<<ceil_div(p.oc, 8), 256, 0, st>>>(p, alpha, beta, out_b);
    SSO_LAUNCH_OK("diag_sq_bias_kernel");
  }
  return 0;
}

}  // namespace sso

using namespace sso;

extern "C" {

size_t sso_diag_sq_workspace_bytes(int64_t n, int64_t oc, int64_t d) {
  if (n <= 0 || oc <= 0 || d <= 0) return 0;
  const int splits = diag_sq_splits((int)n, (int)oc, (int)d);
  const int per = ceil_div((int)n, splits);
  return (size_t)ceil_div((int)n, per) * (size_t)oc * (size_t)d * sizeof(float);
}

int sso_diag_sq_im2col(const void* x, const void* g, int dtype, int64_t n, int64_t c, int64_t h, int64_t w,
                       int64_t sxn, int64_t sxc, int64_t sxh, int64_t sxw, int64_t oc, int64_t sgn,
                       int64_t sgc, int64_t sgh, int64_t sgw, int kh, int kw, int stride_h, int stride_w,
                       int pad_h, int pad_w, int dil_h, int dil_w, const float* sample_weight, float alpha,
                       float beta, float* out_w, float* out_b, void* workspace, size_t workspace_bytes,
                       void* stream) {
  SSO_CHECK_ARG(x && g && out_w, "diag_sq: null pointer");
  SSO_CHECK_ARG(n > 0 && c > 0 && h > 0 && w > 0 && oc > 0, "diag_sq: bad dims");
  SSO_CHECK_ARG(kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 && dil_h > 0 && dil_w > 0 && pad_h >= 0 &&
                pad_w >= 0, "diag_sq: bad conv geometry");
  const int64_t ho = (h + 2 * pad_h - (int64_t)dil_h * (kh - 1) - 1) / stride_h + 1;
  const int64_t wo = (w + 2 * pad_w - (int64_t)dil_w * (kw - 1) - 1) / stride_w + 1;
  SSO_CHECK_ARG(ho > 0 && wo > 0, "diag_sq: empty output");
  const int64_t d = c * kh * kw;
  SSO_CHECK_ARG(d < ((int64_t)1 << 30) && n < ((int64_t)1 << 30) && ho * wo < ((int64_t)1 << 30), "diag_sq: shape too large");
  const size_t need = sso_diag_sq_workspace_bytes(n, oc, d);
  SSO_CHECK_ARG(workspace != nullptr && workspace_bytes >= need, "diag_sq: workspace too small: need %zu bytes, got %zu",
                need, workspace_bytes);
  DiagSqParams p{};
  p.x = x; p.g = g; p.weight = sample_weight; p.partial = reinterpret_cast<float*>(workspace);
  p.sxn = sxn; p.sxc = sxc; p.sxh = sxh; p.sxw = sxw; p.sgn = sgn; p.sgc = sgc; p.sgh = sgh; p.sgw = sgw;
  p.n = (int)n; p.c = (int)c; p.h = (int)h; p.w = (int)w; p.oc = (int)oc; p.ho = (int)ho; p.wo = (int)wo;
  p.kh = kh; p.kw = kw; p.stride_h = stride_h; p.stride_w = stride_w; p.pad_h = pad_h; p.pad_w = pad_w;
  p.dil_h = dil_h; p.dil_w = dil_w; p.d = (int)d;
  int splits = diag_sq_splits((int)n, (int)oc, (int)d);
  // a Linear layer contracts over the samples, 16 per staging step: no split shorter than that
  // (the workspace bound above is the one for the general case and covers this one)
  if (ho * wo == 1 && kh * kw == 1) splits = std::min(splits, std::max(1, (int)(n / 16)));
  p.samples_per_split = ceil_div((int)n, splits);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SSO_F32: return diag_sq_typed<float>(p, alpha, beta, out_w, out_b, st);
    case SSO_BF16: return diag_sq_typed<__nv_bfloat16>(p, alpha, beta, out_w, out_b, st);
    case SSO_F16: return diag_sq_typed<__half>(p, alpha, beta, out_w, out_b, st);
  }
  return fail(-1, "diag_sq: unknown dtype %d", dtype);
}

}  // extern "C"
