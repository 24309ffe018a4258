// Tile-task engine: batched pi-damped SPD inverse, Cholesky factor, Kronecker precondition and
// posterior sampling, each expressed as phases of independent tile tasks
//     C[m x n] <- alpha * op(A) * op(B) + beta * C
// (one kernel launch per phase, covering every matrix of every layer) plus a dense 64x64
// diagonal-block factorisation done by one CTA in shared memory.
//
// Blocked algorithm per SPD matrix M (panels of 128 columns, left looking):
//   Cholesky, panel p:
//       update : M_ip -= sum_{k<p} L_ik * L_pk^T         for i >= p (128-wide tile tasks, long K)
//       diag   : L_pp = chol(M_pp), also Linv_pp = L_pp^-1          (diag-panel kernel, one CTA)
//       panel  : L_ip = M_ip * Linv_pp^T                 for i > p  (128-wide tile tasks)
//     (with "chol_panel" off: the same with two 64-wide halves per panel and the 64x64 diag-block kernel)
//   Triangular inverse by recursive doubling over block ranges [first | second]:
//       Y   = L_21 * Inv_11          (into scratch)      Inv_21 = - Inv_22 * Y
//   Inverse:  M^-1 = Linv^T * Linv   (lower tiles computed, mirrored into the upper triangle)
#include <algorithm>
#include <map>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "diag_panel.cuh"

namespace sso {

int launch_tile_tasks_tc(const sso_tile_task* tasks_dev, int count, int* status_dev, cudaStream_t st);
int launch_tile_tasks_kc(const sso_tile_task* tasks_dev, int count, int* status_dev, cudaStream_t st);
int launch_tile_tasks_tma(const sso_tile_task* tasks_dev, const void* maps_dev, int count, int* status_dev, cudaStream_t st);
bool tma_encode_f32_rows(void* out, const float* base, int64_t rows, int64_t cols, int64_t ld);
int g_phase_lpt = 1;    // tasks of a 128-wide phase sorted by decreasing K
int g_chol_ksplit = 6;  // Cholesky panel updates from this panel index on are cut along K (0: never)
int g_engine_tma = 1;   // k-contiguous 128-wide tasks fetch their operands with TMA (tensor maps per task)
int g_engine_tc = 1;    // run 128-wide tile phases on the tensor cores (3xTF32) instead of FFMA
int g_chol_panel = 1;   // factorise a 128-column panel's diagonal block in one launch (else two 64-wide halves)

constexpr int NB = 64;  // algorithmic block size of the factorisations

// ------------------------------------------------------------------------------------------
// device records
// ------------------------------------------------------------------------------------------
using DiagRec = sso_diag_rec;
using CopyRec = sso_copy_rec;
struct MatRec {       // per-matrix data for the trace / pi kernel
  const float* src;
  int32_t d;
  int32_t partner;
  int32_t role;
  int32_t ld;
};

// ------------------------------------------------------------------------------------------
// tile GEMM kernel
// ------------------------------------------------------------------------------------------
template <int MT>
__global__ void __launch_bounds__(256) tile_task_kernel(const sso_tile_task* __restrict__ tasks) {
  constexpr int TILE = 16 * MT;
  constexpr int PER = TILE * KT / 256;  // elements per thread per operand per stage
  __shared__ __align__(16) float As[KT * TILE];
  __shared__ __align__(16) float Bs[KT * TILE];
  const sso_tile_task t = tasks[blockIdx.x];
  const int tid = threadIdx.x;
  const bool ta = t.flags & 1u, tb = t.flags & 2u;
  // operand element (idx, k):  A: ta ? A[k*lda+idx] : A[idx*lda+k];  B: tb ? B[idx*ldb+k] : B[k*ldb+idx]
  const bool a_kcontig = !ta, b_kcontig = tb;

  float ra[PER], rb[PER];
  auto load_op = [&](const float* __restrict__ P, int ld, bool kcontig, int lim, int k0, float (&r)[PER]) {
    if (kcontig) {
      const int k = k0 + (tid & 31), g = tid >> 5;
      const bool kok = k < t.k;
#pragma unroll
      for (int i = 0; i < PER / 4; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int idx = g * 4 + 32 * i + q;
          r[i * 4 + q] = (kok && idx < lim) ? __ldg(P + (int64_t)idx * ld + k) : 0.f;
        }
    } else {
      const int idx = tid % TILE, kb = tid / TILE;
      const bool iok = idx < lim;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int k = k0 + kb + (256 / TILE) * i;
        r[i] = (iok && k < t.k) ? __ldg(P + (int64_t)k * ld + idx) : 0.f;
      }
    }
  };
  auto store_op = [&](float* S, bool kcontig, const float (&r)[PER]) {
    if (kcontig) {
      const int k = tid & 31, g = tid >> 5;
#pragma unroll
      for (int i = 0; i < PER / 4; ++i)
        *reinterpret_cast<float4*>(S + k * TILE + swz(k, g * 4 + 32 * i)) =
            make_float4(r[i * 4], r[i * 4 + 1], r[i * 4 + 2], r[i * 4 + 3]);
    } else {
      const int idx = tid % TILE, kb = tid / TILE;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int k = kb + (256 / TILE) * i;
        S[k * TILE + swz(k, idx)] = r[i];
      }
    }
  };

  float acc[MT][MT];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[i][j] = 0.f;
  const int ty = tid >> 4, tx = tid & 15;
  const int nkt = ceil_div(t.k, KT);
  if (nkt > 0) {
    load_op(t.A, t.lda, a_kcontig, t.m, 0, ra);
    load_op(t.B, t.ldb, b_kcontig, t.n, 0, rb);
    store_op(As, a_kcontig, ra);
    store_op(Bs, b_kcontig, rb);
  }
  __syncthreads();
  for (int kt = 0; kt < nkt; ++kt) {
    if (kt + 1 < nkt) {
      load_op(t.A, t.lda, a_kcontig, t.m, (kt + 1) * KT, ra);
      load_op(t.B, t.ldb, b_kcontig, t.n, (kt + 1) * KT, rb);
    }
    TileCore<MT>::compute(As, Bs, ty, tx, acc);
    __syncthreads();
    if (kt + 1 < nkt) {
      store_op(As, a_kcontig, ra);
      store_op(Bs, b_kcontig, rb);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    const int r = TileCore<MT>::row_of(ty, i);
    if (r >= t.m) continue;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int c = TileCore<MT>::col_of(tx, j);
      if (c >= t.n) continue;
      if ((t.flags & 4u) && c > r) continue;   // symmetric tile: lower half computed, mirrored below
      float* o = t.C + (int64_t)r * t.ldc + c;
      float v = t.alpha * acc[i][j];
      if (t.beta != 0.f) v = fmaf(t.beta, *o, v);
      *o = v;
      if (t.C2) t.C2[(int64_t)c * t.ldc2 + r] = v;
      if ((t.flags & 4u) && c < r) t.C[(int64_t)c * t.ldc + r] = v;
    }
  }
}

// ------------------------------------------------------------------------------------------
// diagonal block: Cholesky of a (<=64)x(<=64) SPD block and the inverse of its factor
// ------------------------------------------------------------------------------------------
// The 64x64 block lives in registers: thread (ty, tx) of a 16x16 grid owns the 4x4 sub-block at
// rows 4ty.., columns 4tx...  Both the right-looking Cholesky and the right-looking triangular
// inverse then cost one __syncthreads per column: the owners of column j publish it (unscaled,
// pivot included) in a double-buffered shared vector, everybody applies the rank-1 update to its
// registers.  Padding rows/columns (block smaller than 64) behave as an identity block.
__global__ void __launch_bounds__(256) diag_block_kernel(const DiagRec* __restrict__ recs,
                                                         int* __restrict__ info) {
  __shared__ float Ls[NB][NB + 1];      // finished factor, column by column
  __shared__ float colbuf[2][NB];
  __shared__ float rowbuf[2][NB];
  __shared__ float dinv[NB];
  const DiagRec rec = recs[blockIdx.x];
  const int tid = threadIdx.x, n = rec.size;
  const int ty = tid >> 4, tx = tid & 15, r0 = ty * 4, c0 = tx * 4;
  float a[4][4], x[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = r0 + i, c = c0 + j;
      float v = (r == c) ? 1.f : 0.f;
      if (r < n && c < n) v = (c <= r) ? rec.L[(int64_t)r * rec.ld_l + c] : 0.f;
      a[i][j] = v;
      x[i][j] = (r == c) ? 1.f : 0.f;
    }
  // ---- Cholesky.  Columns are walked in groups of four so that the position of column j inside
  // a thread's 4x4 block (jj) is a compile-time constant and the selects below fold away.
  for (int jb = 0; jb < NB / 4; ++jb) {
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = 4 * jb + jj;
      if (tx == jb) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (r0 + i >= j) colbuf[j & 1][r0 + i] = a[i][jj];
      }
      __syncthreads();
      float pv = colbuf[j & 1][j];
      if (!(pv > 0.f)) {   // non-positive or NaN pivot: record once, continue with 1
        if (tid == 0 && info && j < n) atomicCAS(info + 2 * rec.mat + rec.info_slot, 0, rec.row0 + j + 1);
        pv = 1.f;
      }
      const float inv = 1.f / pv, rs = rsqrtf(pv);
      if (ty >= jb && tx >= jb && tx <= ty) {     // blocks that column j still touches (lower triangle)
        float cr[4], cc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          cr[i] = colbuf[j & 1][r0 + i];
          cc[i] = colbuf[j & 1][c0 + i] * inv;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int r = r0 + i, c = c0 + q;
            if (r > j && c > j && c <= r) a[i][q] -= cr[i] * cc[q];
          }
        if (tx == jb) {                           // finish column j of the factor
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = r0 + i;
            if (r >= j) {
              const float l = (r == j) ? sqrtf(pv) : a[i][jj] * rs;
              a[i][jj] = l;
              Ls[r][j] = l;
            }
          }
        }
      }
      if (tid == 0) dinv[j] = rs;
    }
  }
  __syncthreads();
  // ---- inverse of the factor: X starts as I; for k: row k of X /= L_kk, rows r > k -= L_rk * row k
  for (int kb = 0; kb < NB / 4; ++kb) {
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const int k = 4 * kb + kk;
      if (ty == kb) {
        const float d = dinv[k];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          x[kk][q] *= d;
          rowbuf[k & 1][c0 + q] = x[kk][q];
        }
      }
      __syncthreads();
      if (c0 <= k && ty >= kb) {
        float xr[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) xr[q] = rowbuf[k & 1][c0 + q];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = r0 + i;
          if (r > k) {
            const float l = Ls[r][k];
#pragma unroll
            for (int q = 0; q < 4; ++q) x[i][q] -= l * xr[q];
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = r0 + i, c = c0 + q;
      if (r < n && c < n) {
        rec.L[(int64_t)r * rec.ld_l + c] = (c <= r) ? a[i][q] : 0.f;
        rec.Linv[(int64_t)r * rec.ld_inv + c] = (c <= r) ? x[i][q] : 0.f;
        if (rec.LinvT) rec.LinvT[(int64_t)c * rec.ld_invt + r] = (c <= r) ? x[i][q] : 0.f;
      }
    }
}

// ------------------------------------------------------------------------------------------
// traces -> per-matrix diagonal shift v = r*pi or r/pi
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) trace_kernel(const MatRec* __restrict__ mats,
                                                    float* __restrict__ traces) {
  __shared__ float red[256];
  const MatRec m = mats[blockIdx.x];
  float s = 0.f;
  for (int i = threadIdx.x; i < m.d; i += 256) s += m.src[(int64_t)i * m.ld + i];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) traces[blockIdx.x] = red[0];
}
__global__ void shift_kernel(const MatRec* __restrict__ mats, const float* __restrict__ traces,
                             const float* __restrict__ damp_r, float* __restrict__ shift, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const MatRec m = mats[i];
  float pi = 1.f;
  if (m.partner >= 0) {
    const MatRec o = mats[m.partner];
    const float mine = traces[i] / (float)m.d, other = traces[m.partner] / (float)o.d;
    // pi = sqrt(mean-diag(A) / mean-diag(G)), A = the role-0 member of the pair
    pi = (m.role == 0) ? sqrtf(mine / other) : sqrtf(other / mine);
  }
  shift[i] = (m.role == 0) ? damp_r[i] * pi : damp_r[i] / pi;
}

__global__ void __launch_bounds__(256) copy_kernel(const CopyRec* __restrict__ recs,
                                                   const float* __restrict__ shift) {
  const CopyRec r = recs[blockIdx.x];
  const int ld = r.ld, d = r.d;
  if (r.mode == 3) {
    // dst (a tile of nrows x d) += its r.mat partial products, which sit side by side 128 columns
    // apart starting at src; summed in that order
    // Four elements per thread at a time, all their loads (up to 32) issued before the first store: one
    // element at a time, the loads of the next would wait behind the store of the previous to the same array.
    const int total = r.nrows * d;
    for (int e0 = threadIdx.x; e0 < total; e0 += 4 * 256) {
      float x[4], pv[4][7];     // at most 7 partial products (8 slices)
      int64_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = e0 + 256 * j;
        const int row = e / d, col = e - row * d;
        o[j] = (int64_t)row * ld + col;
        const bool in = e < total;
        x[j] = in ? r.dst[o[j]] : 0.f;
#pragma unroll
        for (int q = 0; q < 7; ++q) pv[j][q] = (in && q < r.mat) ? r.src[o[j] + q * 128] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int q = 0; q < 7; ++q) x[j] += pv[j][q];
        if (e0 + 256 * j < total) r.dst[o[j]] = x[j];
      }
    }
    return;
  }
  const float v = (r.mat >= 0) ? shift[r.mat] : 0.f;
  if (r.mode != 1 && (ld & 3) == 0 && ((reinterpret_cast<uintptr_t>(r.dst) | reinterpret_cast<uintptr_t>(r.src)) & 15) == 0) {
    // rows are 16-byte aligned: whole float4s, then the ragged end of each row
    const int d4 = d >> 2, per_row = d4 + (d & 3);
    const int total = r.nrows * per_row;
    for (int e = threadIdx.x; e < total; e += 256) {
      const int lr = e / per_row, i = e - lr * per_row, row = r.row0 + lr;
      float* drow = r.dst + (int64_t)row * ld;
      if (i < d4) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r.mode == 0) {
          x = *reinterpret_cast<const float4*>(r.src + (int64_t)row * ld + 4 * i);
          const int dc = row - 4 * i;
          if (dc == 0) x.x += v; else if (dc == 1) x.y += v; else if (dc == 2) x.z += v; else if (dc == 3) x.w += v;
        }
        *reinterpret_cast<float4*>(drow + 4 * i) = x;
      } else {
        const int col = 4 * d4 + (i - d4);
        float x = 0.f;
        if (r.mode == 0) {
          x = r.src[(int64_t)row * ld + col];
          if (row == col) x += v;
        }
        drow[col] = x;
      }
    }
    return;
  }
  const int64_t total = (int64_t)r.nrows * d;
  for (int64_t e = threadIdx.x; e < total; e += 256) {
    const int row = r.row0 + (int)(e / d), col = (int)(e % d);
    if (r.mode == 2) {
      r.dst[(int64_t)row * ld + col] = 0.f;
    } else if (r.mode == 1) {
      // dst = L^T restricted to the upper triangle (row <= col reads L[col][row])
      r.dst[(int64_t)row * ld + col] = (row <= col) ? r.src[(int64_t)col * ld + row] : 0.f;
    } else {
      float x = r.src[(int64_t)row * ld + col];
      if (row == col) x += v;
      r.dst[(int64_t)row * ld + col] = x;
    }
  }
}

// ------------------------------------------------------------------------------------------
// plans
// ------------------------------------------------------------------------------------------
struct Plan {
  std::vector<sso_tile_task> tasks;
  std::vector<DiagRec> diags;
  std::vector<CopyRec> copies;
  std::vector<MatRec> mats;
  std::vector<sso_phase> inv_phases, std_phases, run_phases;  // kron: inv/std; others: run
  // device tables
  sso_tile_task* d_tasks = nullptr;
  DiagRec* d_diags = nullptr;
  CopyRec* d_copies = nullptr;
  MatRec* d_mats = nullptr;
  float* d_traces = nullptr;
  float* d_shift = nullptr;
  int* d_status = nullptr;   // set by a tensor-core tile task whose wait gave up
  unsigned char* d_maps = nullptr;   // 256 bytes per task: tensor maps of A and B (k-contiguous tasks only)
  bool have_maps = false;
  int first_scaled_task = -1, n_scaled_tasks = 0;  // sample plan: tasks whose alpha is std_scale
  bool host_only = false;
};

static std::mutex g_mu;
static std::map<int64_t, Plan*> g_plans;
static int64_t g_next = 1;

static int64_t register_plan(Plan* p) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_plans[g_next] = p;
  return g_next++;
}
static Plan* find_plan(int64_t h) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_plans.find(h);
  return it == g_plans.end() ? nullptr : it->second;
}

static size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

struct Builder {
  Plan& p;
  std::vector<sso_phase>* phases;
  explicit Builder(Plan& plan, std::vector<sso_phase>* ph) : p(plan), phases(ph) {}
  int task_begin() const { return (int)p.tasks.size(); }
  void gemm(const float* A, int lda, bool ta, const float* B, int ldb, bool tb, float* C, int ldc,
            int m, int n, int k, float alpha, float beta, float* C2 = nullptr, int ldc2 = 0,
            bool symmetric = false) {
    sso_tile_task t;
    t.A = A; t.B = B; t.C = C; t.C2 = C2;
    t.lda = lda; t.ldb = ldb; t.ldc = ldc; t.ldc2 = ldc2;
    t.m = m; t.n = n; t.k = k;
    t.flags = (ta ? 1u : 0u) | (tb ? 2u : 0u) | (symmetric ? 4u : 0u);
    t.alpha = alpha; t.beta = beta;
    p.tasks.push_back(t);
  }
  // A 128-wide task qualifies for the cp.async kernel when both operands are read along k in
  // 16-byte aligned rows.
  static bool k_contiguous(const sso_tile_task& t) {
    auto al = [](const void* p, int ld) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && ld % 4 == 0; };
    return (t.flags & 3u) == 2u && al(t.A, t.lda) && al(t.B, t.ldb);
  }
  void push_phase(int kind, int first, int count) {
    if (count <= 0) return;
    sso_phase ph;
    ph.kind = kind; ph.first = first; ph.count = count; ph.reserved = 0;
    phases->push_back(ph);
  }
  void end_phase(int kind, int first, int count) {
    if (count <= 0) return;
    if (kind != 1) return push_phase(kind, first, count);
    // the tasks of a phase are independent: run the k-contiguous ones (kind 4) and the rest
    // (kind 1) as two launches
    auto mid = std::stable_partition(p.tasks.begin() + first, p.tasks.begin() + first + count, k_contiguous);
    const int nfast = (int)(mid - (p.tasks.begin() + first));
    // CTAs are handed out in task order: longest K first keeps the tail of each launch short
    if (g_phase_lpt) {
      auto longer = [](const sso_tile_task& a, const sso_tile_task& b) { return a.k > b.k; };
      std::stable_sort(p.tasks.begin() + first, mid, longer);
      std::stable_sort(mid, p.tasks.begin() + first + count, longer);
    }
    push_phase(4, first, nfast);
    push_phase(1, first + nfast, count - nfast);
  }
};

static inline int padded_ld(int d) { return (d + 3) / 4 * 4; }   // rows of plan-owned matrices start on 16 bytes

struct Mat {  // one square matrix being factorised
  int d, nb;
  int ld;      // leading dimension of W, Li and T (the caller's buffers)
  int ldx;     // leading dimension of X (plan-owned)
  float* W;    // holds M, then L (lower)
  float* Li;   // receives L^-1 (lower)
  float* X;    // receives L^-T (upper), or null: lets every product of the triangular inverse and of
               // L^-T L^-1 read both operands along k
  float* T;    // where the finished inverse goes
  int mat_index;
};
static inline int bsz(const Mat& m, int b) { return std::min(NB, m.d - b * NB); }
static inline float* blk(float* base, int d, int bi, int bj) { return base + (int64_t)bi * NB * d + (int64_t)bj * NB; }

// Cholesky of every matrix in `ms` (in place in W, block inverses into Li's diagonal blocks).
// Left-looking over panels of two blocks (128 columns): a panel first receives the update of
// all finished columns in one phase of 128x128 tasks with a long K (tensor cores), then its
// two block columns are factorised with 64-wide tasks.  The upper triangle of W is scratch.
static void emit_cholesky(Builder& b, const std::vector<Mat>& ms, int info_slot) {
  constexpr int PB = 2 * NB;
  int max_np = 0;
  for (auto& m : ms) max_np = std::max(max_np, (m.d + PB - 1) / PB);
  auto blk2 = [](float* base, int d, int pi, int pj) { return base + (int64_t)pi * PB * d + (int64_t)pj * PB; };
  for (int p = 0; p < max_np; ++p) {
    int first = b.task_begin();
    // Late panels have few tasks with a long K (one CTA each, most SMs idle): their K range is cut
    // into `ksplit` slices of whole 128-column blocks.  Slice 0 updates the tile itself, the
    // others write partial products into free 128x128 blocks of W's upper triangle (scratch
    // during the factorisation), and a copy phase adds them to the tile in a fixed order.
    int n_tasks = 0;
    if (p > 0)
      for (auto& m : ms) n_tasks += std::max(0, (m.d + PB - 1) / PB - p);
    int ksplit = 1;
    if (g_chol_ksplit > 0 && p >= g_chol_ksplit && n_tasks > 0) ksplit = std::max(1, std::min(std::min(8, 148 / n_tasks), p / 2));
    const int first_sum = (int)b.p.copies.size();
    if (p > 0)
      for (auto& m : ms) {
        const int np = (m.d + PB - 1) / PB;
        // free scratch blocks (r, c), r < c <= np - 2 (full 128x128 blocks above the diagonal), handed
        // out as runs of ksplit - 1 neighbours in one block row
        int sr = 0, sc = 1;
        auto take_run = [&](int len) -> float* {
          while (sr <= np - 3) {
            if (sc + len - 1 <= np - 2) {
              float* q = blk2(m.W, m.ld, sr, sc);
              sc += len;
              return q;
            }
            ++sr; sc = sr + 1;
          }
          return nullptr;
        };
        for (int i = p; i < np; ++i) {
          const int mi = std::min(PB, m.d - i * PB), nj = std::min(PB, m.d - p * PB);
          float* C = blk2(m.W, m.ld, i, p);
          float* run = ksplit > 1 ? take_run(ksplit - 1) : nullptr;
          const int parts = run ? ksplit : 1;
          const int per = (p + parts - 1) / parts;        // 128-column blocks of K per slice
          int used = 0;
          for (int s = 0; s < parts; ++s) {
            const int kb0 = s * per, kb1 = std::min(p, kb0 + per);
            if (kb0 >= kb1) break;
            float* dst = s == 0 ? C : run + (int64_t)(s - 1) * PB;
            b.gemm(blk2(m.W, m.ld, i, kb0), m.ld, false, blk2(m.W, m.ld, p, kb0), m.ld, true, dst, m.ld, mi, nj,
                   (kb1 - kb0) * PB, -1.f, s == 0 ? 1.f : 0.f);
            used = s;
          }
          // one record (one CTA of the copy phase) per 16 rows of the tile
          for (int r0 = 0; used > 0 && r0 < mi; r0 += 16) {
            CopyRec c;
            c.src = run + (int64_t)r0 * m.ld; c.dst = C + (int64_t)r0 * m.ld; c.d = nj; c.row0 = 0;
            c.nrows = std::min(16, mi - r0); c.mat = used; c.mode = 3; c.ld = m.ld;
            b.p.copies.push_back(c);
          }
        }
      }
    b.end_phase(1, first, b.task_begin() - first);
    b.end_phase(3, first_sum, (int)b.p.copies.size() - first_sum);
    if (g_chol_panel) {
      // the panel's 128x128 diagonal block in one launch (factor, inverse and its transpose), then the
      // rows below as 128-wide tasks with K = 128:  L_ip = M_ip * Linv_pp^T, in place
      first = (int)b.p.diags.size();
      for (auto& m : ms)
        if (p * PB < m.d) {
          DiagRec r;
          r.L = blk2(m.W, m.ld, p, p); r.Linv = blk2(m.Li, m.ld, p, p);
          r.ld_l = m.ld; r.ld_inv = m.ld; r.size = std::min(PB, m.d - p * PB); r.mat = m.mat_index; r.row0 = p * PB;
          r.info_slot = info_slot;
          r.LinvT = m.X ? blk2(m.X, m.ldx, p, p) : nullptr; r.ld_invt = m.ldx; r.pad = 0;
          b.p.diags.push_back(r);
        }
      b.end_phase(5, first, (int)b.p.diags.size() - first);
      first = b.task_begin();
      for (auto& m : ms) {
        const int np = (m.d + PB - 1) / PB;
        for (int i = p + 1; i < np; ++i)
          b.gemm(blk2(m.W, m.ld, i, p), m.ld, false, blk2(m.Li, m.ld, p, p), m.ld, true,
                 blk2(m.W, m.ld, i, p), m.ld, std::min(PB, m.d - i * PB), PB, PB, 1.f, 0.f);
      }
      b.end_phase(1, first, b.task_begin() - first);
      continue;
    }
    for (int half = 0; half < 2; ++half) {
      const int j = 2 * p + half;
      if (half == 1) {   // second block column of the panel: update by the first
        first = b.task_begin();
        for (auto& m : ms)
          for (int i = j; i < m.nb; ++i)
            b.gemm(blk(m.W, m.ld, i, j - 1), m.ld, false, blk(m.W, m.ld, j, j - 1), m.ld, true,
                   blk(m.W, m.ld, i, j), m.ld, bsz(m, i), bsz(m, j), NB, -1.f, 1.f);
        b.end_phase(0, first, b.task_begin() - first);
      }
      first = (int)b.p.diags.size();
      for (auto& m : ms)
        if (j < m.nb) {
          DiagRec r;
          r.L = blk(m.W, m.ld, j, j); r.Linv = blk(m.Li, m.ld, j, j);
          r.ld_l = m.ld; r.ld_inv = m.ld; r.size = bsz(m, j); r.mat = m.mat_index; r.row0 = j * NB;
          r.info_slot = info_slot;
          r.LinvT = m.X ? blk(m.X, m.ldx, j, j) : nullptr; r.ld_invt = m.ldx; r.pad = 0;
          b.p.diags.push_back(r);
        }
      b.end_phase(2, first, (int)b.p.diags.size() - first);
      first = b.task_begin();
      for (auto& m : ms)
        for (int i = j + 1; i < m.nb; ++i)
          b.gemm(blk(m.W, m.ld, i, j), m.ld, false, blk(m.Li, m.ld, j, j), m.ld, true,
                 blk(m.W, m.ld, i, j), m.ld, bsz(m, i), NB, NB, 1.f, 0.f);
      b.end_phase(0, first, b.task_begin() - first);
    }
  }
}

// T <- Li^T * Li (symmetric; lower tiles computed and mirrored).  128-wide tiles when they pay.
static void emit_lauum(Builder& b, const std::vector<Mat>& ms) {
  for (int pass = 0; pass < 2; ++pass) {
    const int tile = pass == 0 ? 64 : 128;
    const int first = b.task_begin();
    for (auto& m : ms) {
      const bool big = m.d >= 512;
      if (big != (pass == 1)) continue;
      const int nt = (m.d + tile - 1) / tile;
      for (int i = 0; i < nt; ++i)
        for (int j = 0; j <= i; ++j) {
          const int mi = std::min(tile, m.d - i * tile), nj = std::min(tile, m.d - j * tile);
          float* C = m.T + (int64_t)i * tile * m.ld + (int64_t)j * tile;
          float* C2 = (i == j) ? nullptr : m.T + (int64_t)j * tile * m.ld + (int64_t)i * tile;
          if (m.X) {   // T(i,j) = sum_{k >= i*tile} X(i,k) X(j,k): both operands read along k
            const float* A = m.X + (int64_t)i * tile * m.ldx + (int64_t)i * tile;
            const float* B = m.X + (int64_t)j * tile * m.ldx + (int64_t)i * tile;
            b.gemm(A, m.ldx, false, B, m.ldx, true, C, m.ld, mi, nj, m.d - i * tile, 1.f, 0.f, C2, m.ld, i == j);
            continue;
          }
          // rows k >= i*tile of Li contribute: A = Li[k, i-cols]^T, B = Li[k, j-cols]
          const float* A = m.Li + (int64_t)i * tile * m.ld + (int64_t)i * tile;
          const float* B = m.Li + (int64_t)i * tile * m.ld + (int64_t)j * tile;
          b.gemm(A, m.ld, true, B, m.ld, false, C, m.ld, mi, nj, m.d - i * tile, 1.f, 0.f, C2, m.ld, i == j);
        }
    }
    b.end_phase(pass == 0 ? 0 : 1, first, b.task_begin() - first);
  }
}

static void emit_copy(Builder& b, const float* src, float* dst, int d, int ld, int mat, int mode) {
  const int rows_per = std::max(1, 16384 / d);
  for (int r0 = 0; r0 < d; r0 += rows_per) {
    CopyRec c;
    c.src = src; c.dst = dst; c.d = d; c.row0 = r0; c.nrows = std::min(rows_per, d - r0);
    c.mat = mat; c.mode = mode; c.ld = ld;
    b.p.copies.push_back(c);
  }
}

static size_t plan_table_bytes(size_t tasks, size_t diags, size_t copies, size_t mats) {
  return align_up(tasks * 256) + align_up(tasks * sizeof(sso_tile_task)) + align_up(diags * sizeof(DiagRec)) +
         align_up(copies * sizeof(CopyRec)) + align_up(mats * sizeof(MatRec)) +
         2 * align_up(mats * sizeof(float)) + 256;
}

static int upload(Plan& p, void* dev_mem, size_t dev_bytes) {
  const size_t need = plan_table_bytes(p.tasks.size(), p.diags.size(), p.copies.size(), p.mats.size());
  SSO_CHECK_ARG(dev_mem != nullptr && dev_bytes >= need, "plan device memory too small: need %zu, got %zu",
                need, dev_bytes);
  char* q = reinterpret_cast<char*>(dev_mem);
  q = reinterpret_cast<char*>(align_up(reinterpret_cast<uintptr_t>(q)));
  p.d_maps = reinterpret_cast<unsigned char*>(q); q += align_up(p.tasks.size() * 256);
  p.d_tasks = reinterpret_cast<sso_tile_task*>(q); q += align_up(p.tasks.size() * sizeof(sso_tile_task));
  p.d_diags = reinterpret_cast<DiagRec*>(q); q += align_up(p.diags.size() * sizeof(DiagRec));
  p.d_copies = reinterpret_cast<CopyRec*>(q); q += align_up(p.copies.size() * sizeof(CopyRec));
  p.d_mats = reinterpret_cast<MatRec*>(q); q += align_up(p.mats.size() * sizeof(MatRec));
  p.d_traces = reinterpret_cast<float*>(q); q += align_up(p.mats.size() * sizeof(float));
  p.d_shift = reinterpret_cast<float*>(q); q += align_up(p.mats.size() * sizeof(float));
  p.d_status = reinterpret_cast<int*>(q);
  SSO_CUDA_OK(cudaMemset(p.d_status, 0, 256));
  if (!p.tasks.empty())
    SSO_CUDA_OK(cudaMemcpy(p.d_tasks, p.tasks.data(), p.tasks.size() * sizeof(sso_tile_task), cudaMemcpyHostToDevice));
  // tensor maps for the tasks of the k-contiguous phases (operand = rows of a row-major matrix)
  p.have_maps = false;
  if (g_engine_tma && !p.tasks.empty()) {
    std::vector<unsigned char> maps(p.tasks.size() * 256, 0);
    bool ok = true, any = false;
    auto encode_phase = [&](const sso_phase& ph) {
      if (ph.kind != 4) return;
      for (int i = ph.first; i < ph.first + ph.count && ok; ++i) {
        const sso_tile_task& t = p.tasks[i];
        ok = tma_encode_f32_rows(&maps[(size_t)i * 256], t.A, t.m, t.k, t.lda) &&
             tma_encode_f32_rows(&maps[(size_t)i * 256 + 128], t.B, t.n, t.k, t.ldb);
        any = true;
      }
    };
    for (auto& ph : p.inv_phases) encode_phase(ph);
    for (auto& ph : p.std_phases) encode_phase(ph);
    for (auto& ph : p.run_phases) encode_phase(ph);
    if (ok && any) {
      SSO_CUDA_OK(cudaMemcpy(p.d_maps, maps.data(), maps.size(), cudaMemcpyHostToDevice));
      p.have_maps = true;
    }
  }
  if (!p.diags.empty())
    SSO_CUDA_OK(cudaMemcpy(p.d_diags, p.diags.data(), p.diags.size() * sizeof(DiagRec), cudaMemcpyHostToDevice));
  if (!p.copies.empty())
    SSO_CUDA_OK(cudaMemcpy(p.d_copies, p.copies.data(), p.copies.size() * sizeof(CopyRec), cudaMemcpyHostToDevice));
  if (!p.mats.empty())
    SSO_CUDA_OK(cudaMemcpy(p.d_mats, p.mats.data(), p.mats.size() * sizeof(MatRec), cudaMemcpyHostToDevice));
  return 0;
}

// A tensor-core tile task whose bounded wait gave up has set the plan's status word (and written NaN
// tiles); surface it through the LAPACK-style info array the caller already reads: info[0] = -(1000 + code).
__global__ void fold_status_kernel(const int* __restrict__ status, int* __restrict__ info) {
  const int s = *status;
  if (s != 0) info[0] = -(1000 + s);
}

static int run_phases(const Plan& p, const std::vector<sso_phase>& phases, int* info, cudaStream_t st) {
  for (const sso_phase& ph : phases) {
    switch (ph.kind) {
      case 0: tile_task_kernel<4><<<ph.count, 256, 0, st>>>(p.d_tasks + ph.first); break;
      case 1:
        if (g_engine_tc) {
          const int rc = launch_tile_tasks_tc(p.d_tasks + ph.first, ph.count, p.d_status, st);
          if (rc) return rc;
          continue;
        }
        tile_task_kernel<8><<<ph.count, 256, 0, st>>>(p.d_tasks + ph.first);
        break;
      case 4:
        if (g_engine_tc) {
          const int rc = p.have_maps
              ? launch_tile_tasks_tma(p.d_tasks + ph.first, p.d_maps + (size_t)ph.first * 256, ph.count, p.d_status, st)
              : launch_tile_tasks_kc(p.d_tasks + ph.first, ph.count, p.d_status, st);
          if (rc) return rc;
          continue;
        }
        tile_task_kernel<8><<<ph.count, 256, 0, st>>>(p.d_tasks + ph.first);
        break;
      case 2: diag_block_kernel<<<ph.count, 256, 0, st>>>(p.d_diags + ph.first, info); break;
      case 5:
        SSO_ENSURE_SMEM((dpanel::diag_panel_kernel), dpanel::SMEM_BYTES);
        dpanel::diag_panel_kernel<<<ph.count, dpanel::THREADS, dpanel::SMEM_BYTES, st>>>(p.d_diags + ph.first, info);
        break;
      case 3: copy_kernel<<<ph.count, 256, 0, st>>>(p.d_copies + ph.first, p.d_shift); break;
      default: return fail(-1, "bad phase kind %d", ph.kind);
    }
    SSO_LAUNCH_OK("plan phase");
  }
  return 0;
}

// task-count estimate without building (used for the *_dev_bytes queries): build and measure.
static Plan* build_kron(int n, const int64_t* dims, float* const* src, float* const* dst,
                        float* const* work, float* const* std_out, const int32_t* partner,
                        const int32_t* role, float* const* xbuf, const int64_t* lds) {
  Plan* p = new Plan();
  std::vector<Mat> ms(n);
  for (int i = 0; i < n; ++i) {
    MatRec mr;
    mr.src = src ? src[i] : nullptr; mr.d = (int)dims[i];
    mr.partner = partner ? partner[i] : -1; mr.role = role ? role[i] : 0;
    mr.ld = lds ? (int)lds[i] : (int)dims[i];
    p->mats.push_back(mr);
    ms[i].d = (int)dims[i]; ms[i].nb = (ms[i].d + NB - 1) / NB;
    ms[i].ld = mr.ld; ms[i].ldx = padded_ld(ms[i].d);
    ms[i].W = dst ? dst[i] : nullptr;   // the output buffer first holds M + vI, then L
    ms[i].Li = work ? work[i] : nullptr;
    ms[i].X = xbuf ? xbuf[i] : nullptr;
    ms[i].T = nullptr;
    ms[i].mat_index = i;
  }
  // ---- inverse: dst <- (src + vI)^-1.
  // Buffers: W = dst holds M + vI, then its factor L in the lower blocks; Li = work (zeroed
  // first, because 128-wide tiles of the last stage also read the blocks just above the
  // diagonal) receives L^-1.  The triangular inverse needs scratch for Y = L21 * Inv11: block
  // Y(i,j), i > j, is stored transposed in W's block (j,i), which a lower-triangular L never
  // uses.  Finally Li^T Li overwrites W, i.e. lands in dst.
  {
    Builder b(*p, &p->inv_phases);
    int first = (int)p->copies.size();
    for (int i = 0; i < n; ++i) {
      emit_copy(b, src ? src[i] : nullptr, ms[i].W, ms[i].d, ms[i].ld, i, 0);
      emit_copy(b, nullptr, ms[i].Li, ms[i].d, ms[i].ld, -1, 2);
      if (ms[i].X) emit_copy(b, nullptr, ms[i].X, ms[i].d, ms[i].ldx, -1, 2);
    }
    b.end_phase(3, first, (int)p->copies.size() - first);
    emit_cholesky(b, ms, 0);
    // triangular inverse by recursive doubling over block ranges [lo,mid) | [mid,hi)
    int max_nb = 0;
    for (auto& m : ms) max_nb = std::max(max_nb, m.nb);
    // (the panel kernel has already inverted whole 128x128 diagonal blocks: the first level is done)
    for (int s = g_chol_panel ? 2 : 1; s < max_nb; s *= 2) {
      // from s = 2 on every range boundary is a multiple of two blocks: 128x128 tasks (the
      // zero blocks just above the diagonal of Li make the wider K ranges harmless)
      const int w = s == 1 ? 1 : 2;
      const int T = w * NB;
      first = b.task_begin();
      for (auto& m : ms)
        for (int lo = 0; lo + s < m.nb; lo += 2 * s) {
          const int mid = lo + s, hi = std::min(lo + 2 * s, m.nb);
          for (int i = mid; i < hi; i += w)
            for (int j = lo; j < mid; j += w)
              // Y(i,j)^T = sum_{k in [j,mid)} Inv11(k,j)^T * L(i,k)^T  -> W block (j,i);
              // Inv11(k,j)^T = X(j,k) when the transposed inverse is kept
              if (m.X)
                b.gemm(blk(m.X, m.ldx, j, j), m.ldx, false, blk(m.W, m.ld, i, j), m.ld, true,
                       blk(m.W, m.ld, j, i), m.ld, T, std::min(T, m.d - i * NB), (mid - j) * NB, 1.f, 0.f);
              else
                b.gemm(blk(m.Li, m.ld, j, j), m.ld, true, blk(m.W, m.ld, i, j), m.ld, true,
                       blk(m.W, m.ld, j, i), m.ld, T, std::min(T, m.d - i * NB), (mid - j) * NB, 1.f, 0.f);
        }
      b.end_phase(w == 1 ? 0 : 1, first, b.task_begin() - first);
      first = b.task_begin();
      for (auto& m : ms)
        for (int lo = 0; lo + s < m.nb; lo += 2 * s) {
          const int mid = lo + s, hi = std::min(lo + 2 * s, m.nb);
          for (int i = mid; i < hi; i += w)
            for (int j = lo; j < mid; j += w) {
              const int kk = std::min((i + w - mid) * NB, m.d - mid * NB);
              // Inv21(i,j) = - sum_k Inv22(i,k) * Y(k,j),  Y(k,j) stored at W(j,k) transposed
              b.gemm(blk(m.Li, m.ld, i, mid), m.ld, false, blk(m.W, m.ld, j, mid), m.ld, true,
                     blk(m.Li, m.ld, i, j), m.ld, std::min(T, m.d - i * NB), T, kk, -1.f, 0.f,
                     m.X ? blk(m.X, m.ldx, j, i) : nullptr, m.ldx);
            }
        }
      b.end_phase(w == 1 ? 0 : 1, first, b.task_begin() - first);
    }
    for (auto& m : ms) m.T = m.W;  // L is dead now; the inverse overwrites it
    emit_lauum(b, ms);
  }
  // ---- std: U = chol(dst)^T.  Work copy of dst into `work`, factor there, then write the
  // transposed factor into std_out.  Block inverses produced on the way land in std_out and
  // are overwritten by the final transposing copy.
  if (std_out) {
    Builder b(*p, &p->std_phases);
    std::vector<Mat> cs(n);
    int first = (int)p->copies.size();
    for (int i = 0; i < n; ++i) {
      cs[i] = ms[i];
      cs[i].W = work[i];
      cs[i].Li = std_out[i];
      cs[i].X = nullptr;
      emit_copy(b, dst[i], work[i], ms[i].d, ms[i].ld, -1, 0);
    }
    b.end_phase(3, first, (int)p->copies.size() - first);
    emit_cholesky(b, cs, 1);
    first = (int)p->copies.size();
    for (int i = 0; i < n; ++i) emit_copy(b, work[i], std_out[i], ms[i].d, ms[i].ld, -1, 1);
    b.end_phase(3, first, (int)p->copies.size() - first);
  }
  return p;
}

}  // namespace sso

using namespace sso;

extern "C" {

static size_t kron_scratch_bytes(int n_mats, const int64_t* dims) {
  size_t b = 0;
  for (int i = 0; i < n_mats; ++i) b += align_up((size_t)dims[i] * (size_t)padded_ld((int)dims[i]) * sizeof(float));
  return b;
}

size_t sso_kron_plan_dev_bytes(int n_mats, const int64_t* dims, int with_std) {
  if (n_mats <= 0 || !dims) return 0;
  std::vector<float*> fake(n_mats, nullptr);
  std::vector<float*> fake_x(n_mats, reinterpret_cast<float*>(4096));   // non-null: the scratch matrices exist
  Plan* p = build_kron(n_mats, dims, fake.data(), fake.data(), fake.data(),
                       with_std ? fake.data() : nullptr, nullptr, nullptr, fake_x.data(), nullptr);
  const size_t bytes = plan_table_bytes(p->tasks.size(), p->diags.size(), p->copies.size(), p->mats.size());
  delete p;
  return kron_scratch_bytes(n_mats, dims) + 256 + bytes;
}

int64_t sso_kron_plan_create(int n_mats, const int64_t* dims, float* const* src, float* const* dst,
                             float* const* work, float* const* std_out, const int32_t* partner,
                             const int32_t* role, void* dev_mem, size_t dev_mem_bytes, int host_only,
                             const int64_t* lds) {
  SSO_CHECK_ARG(n_mats > 0 && dims && src && dst && work, "kron plan: null argument");
  for (int i = 0; i < n_mats; ++i) {
    SSO_CHECK_ARG(dims[i] > 0 && dims[i] <= 32768, "kron plan: bad dim %lld", (long long)dims[i]);
    SSO_CHECK_ARG(src[i] && dst[i] && work[i], "kron plan: null matrix pointer at %d", i);
    if (partner && partner[i] >= 0) SSO_CHECK_ARG(partner[i] < n_mats, "kron plan: bad partner");
  }
  // the head of the plan's memory holds one scratch matrix per factor (the transposed triangular
  // inverse); the tables follow.  A host-only plan needs (host) memory for the scratch part only.
  const size_t scratch = kron_scratch_bytes(n_mats, dims) + 256;
  SSO_CHECK_ARG(dev_mem != nullptr && dev_mem_bytes >= scratch, "kron plan: plan memory too small for the scratch matrices");
  std::vector<float*> xb(n_mats);
  {
    char* q = reinterpret_cast<char*>(align_up(reinterpret_cast<uintptr_t>(dev_mem)));
    for (int i = 0; i < n_mats; ++i) {
      xb[i] = reinterpret_cast<float*>(q);
      q += align_up((size_t)dims[i] * (size_t)padded_ld((int)dims[i]) * sizeof(float));
    }
  }
  if (lds)
    for (int i = 0; i < n_mats; ++i) SSO_CHECK_ARG(lds[i] >= dims[i], "kron plan: leading dimension %lld < dim %lld", (long long)lds[i], (long long)dims[i]);
  Plan* p = build_kron(n_mats, dims, src, dst, work, std_out, partner, role, xb.data(), lds);
  p->host_only = host_only != 0;
  if (!p->host_only) {
    const int rc = upload(*p, reinterpret_cast<char*>(dev_mem) + scratch, dev_mem_bytes - scratch);
    if (rc != 0) { delete p; return rc; }
  }
  return register_plan(p);
}

int sso_kron_plan_run(int64_t plan, const float* damp_r_dev, int* info_dev, int do_inverse,
                      int do_std, void* stream) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr, "unknown plan %lld", (long long)plan);
  SSO_CHECK_ARG(!p->host_only, "plan %lld was built host-only", (long long)plan);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int n = (int)p->mats.size();
  if (info_dev) SSO_CUDA_OK(cudaMemsetAsync(info_dev, 0, 2 * n * sizeof(int), st));
  if (do_inverse) {
    SSO_CHECK_ARG(damp_r_dev != nullptr, "kron run: damping table is null");
    trace_kernel<<<n, 256, 0, st>>>(p->d_mats, p->d_traces);
    SSO_LAUNCH_OK("trace_kernel");
    shift_kernel<<<ceil_div(n, 128), 128, 0, st>>>(p->d_mats, p->d_traces, damp_r_dev, p->d_shift, n);
    SSO_LAUNCH_OK("shift_kernel");
    const int rc = run_phases(*p, p->inv_phases, info_dev, st);
    if (rc) return rc;
  }
  if (do_std) {
    SSO_CHECK_ARG(!p->std_phases.empty(), "plan %lld has no std program", (long long)plan);
    const int rc = run_phases(*p, p->std_phases, info_dev, st);
    if (rc) return rc;
  }
  if (info_dev && p->d_status) {
    fold_status_kernel<<<1, 1, 0, st>>>(p->d_status, info_dev);
    SSO_LAUNCH_OK("fold_status_kernel");
  }
  return 0;
}

// ---- precondition --------------------------------------------------------------------------
static Plan* build_precond(int n, const int64_t* dA, const int64_t* dG, float* const* A_inv,
                           float* const* G_inv, float* const* gw, float* const* gb, float* const* tmp,
                           const int64_t* ldA, const int64_t* ldG) {
  Plan* p = new Plan();
  Builder b(*p, &p->run_phases);
  constexpr int T = 128;
  // Both factors are symmetric, which lets every operand be read along its contiguous
  // direction (the fast path of the tensor-core tasks):
  //   tmp = U^T = A_inv[:, :wc] * gw^T (+ A_inv[:, wc] * gb^T),   [gw | gb] = G_inv * U.
  // la / lg: leading dimensions of A_inv / G_inv; tmp is [d_A x d_G] with leading dimension lg.
  int first = b.task_begin();
  for (int l = 0; l < n; ++l) {
    const int a = (int)dA[l], g = (int)dG[l];
    const int la = ldA ? (int)ldA[l] : a, lg = ldG ? (int)ldG[l] : g;
    const bool bias = gb && gb[l];
    const int wcols = bias ? a - 1 : a;
    for (int i = 0; i < a; i += T)
      for (int j = 0; j < g; j += T)
        b.gemm(A_inv[l] + (int64_t)i * la, la, false, gw[l] + (int64_t)j * wcols, wcols, true,
               tmp[l] + (int64_t)i * lg + j, lg, std::min(T, a - i), std::min(T, g - j), wcols, 1.f, 0.f);
  }
  b.end_phase(1, first, b.task_begin() - first);
  first = b.task_begin();
  for (int l = 0; l < n; ++l) {
    const int a = (int)dA[l], g = (int)dG[l];
    const int la = ldA ? (int)ldA[l] : a, lg = ldG ? (int)ldG[l] : g;
    if (!(gb && gb[l])) continue;
    for (int i = 0; i < a; i += NB)
      for (int j = 0; j < g; j += NB)
        b.gemm(A_inv[l] + (int64_t)i * la + (a - 1), la, false, gb[l] + j, g, false,
               tmp[l] + (int64_t)i * lg + j, lg, std::min(NB, a - i), std::min(NB, g - j), 1, 1.f, 1.f);
  }
  b.end_phase(0, first, b.task_begin() - first);
  first = b.task_begin();
  for (int l = 0; l < n; ++l) {
    const int a = (int)dA[l], g = (int)dG[l];
    const int lg = ldG ? (int)ldG[l] : g;
    const bool bias = gb && gb[l];
    const int wcols = bias ? a - 1 : a;
    for (int i = 0; i < g; i += T) {
      for (int j = 0; j < wcols; j += T)
        b.gemm(G_inv[l] + (int64_t)i * lg, lg, false, tmp[l] + (int64_t)j * lg, lg, true,
               gw[l] + (int64_t)i * wcols + j, wcols, std::min(T, g - i), std::min(T, wcols - j), g, 1.f, 0.f);
      if (bias)
        b.gemm(G_inv[l] + (int64_t)i * lg, lg, false, tmp[l] + (int64_t)wcols * lg, lg, true,
               gb[l] + i, 1, std::min(T, g - i), 1, g, 1.f, 0.f);
    }
  }
  b.end_phase(1, first, b.task_begin() - first);
  return p;
}

size_t sso_precond_plan_dev_bytes(int n_layers, const int64_t* dA, const int64_t* dG) {
  size_t tasks = 0;
  for (int l = 0; l < n_layers; ++l) {
    const size_t ti = (dG[l] + 127) / 128, tj = (dA[l] + 127) / 128 + 1;
    tasks += 2 * ti * tj + ((dG[l] + 63) / 64) * ((dA[l] + 63) / 64);
  }
  return plan_table_bytes(tasks, 0, 0, 0);
}

int64_t sso_precond_plan_create(int n_layers, const int64_t* dA, const int64_t* dG,
                                float* const* A_inv, float* const* G_inv, float* const* gw,
                                float* const* gb, float* const* tmp, void* dev_mem,
                                size_t dev_mem_bytes, int host_only, const int64_t* ldA, const int64_t* ldG) {
  SSO_CHECK_ARG(n_layers > 0 && dA && dG && A_inv && G_inv && gw && tmp, "precond plan: null argument");
  for (int l = 0; l < n_layers; ++l)
    SSO_CHECK_ARG(dA[l] > 0 && dG[l] > 0 && A_inv[l] && G_inv[l] && gw[l] && tmp[l],
                  "precond plan: bad layer %d", l);
  Plan* p = build_precond(n_layers, dA, dG, A_inv, G_inv, gw, gb, tmp, ldA, ldG);
  p->host_only = host_only != 0;
  if (!p->host_only) {
    const int rc = upload(*p, dev_mem, dev_mem_bytes);
    if (rc != 0) { delete p; return rc; }
  }
  return register_plan(p);
}

int sso_precond_plan_run(int64_t plan, void* stream) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr && !p->host_only, "unknown or host-only plan %lld", (long long)plan);
  return run_phases(*p, p->run_phases, nullptr, reinterpret_cast<cudaStream_t>(stream));
}

// ---- posterior sampling --------------------------------------------------------------------
static Plan* build_sample(int n, const int64_t* dA, const int64_t* dG, float* const* U_A,
                          float* const* U_G, float* const* noise, float* const* w, float* const* bvec,
                          float* const* tmp, const int64_t* ldA, const int64_t* ldG) {
  Plan* p = new Plan();
  Builder b(*p, &p->run_phases);
  constexpr int T = 128;
  // tmp = U_G * E : row block i only needs k >= i (upper triangular U_G)
  int first = b.task_begin();
  for (int l = 0; l < n; ++l) {
    const int a = (int)dA[l], g = (int)dG[l];
    for (int i = 0; i < g; i += T)
      for (int j = 0; j < a; j += T)
        b.gemm(U_G[l] + (int64_t)i * (ldG ? (int)ldG[l] : g) + i, ldG ? (int)ldG[l] : g, false, noise[l] + (int64_t)i * a + j, a, false,
               tmp[l] + (int64_t)i * a + j, a, std::min(T, g - i), std::min(T, a - j), g - i, 1.f, 0.f);
  }
  b.end_phase(1, first, b.task_begin() - first);
  // [w | b] += s * tmp * U_A : column block j only needs k < j + T (upper triangular U_A)
  first = b.task_begin();
  p->first_scaled_task = first;
  for (int l = 0; l < n; ++l) {
    const int a = (int)dA[l], g = (int)dG[l];
    const bool bias = bvec && bvec[l];
    const int wcols = bias ? a - 1 : a;
    for (int i = 0; i < g; i += T) {
      for (int j = 0; j < wcols; j += T)
        b.gemm(tmp[l] + (int64_t)i * a, a, false, U_A[l] + j, ldA ? (int)ldA[l] : a, false,
               w[l] + (int64_t)i * wcols + j, wcols, std::min(T, g - i), std::min(T, wcols - j),
               std::min(a, j + T), 1.f, 1.f);
      if (bias)
        b.gemm(tmp[l] + (int64_t)i * a, a, false, U_A[l] + wcols, ldA ? (int)ldA[l] : a, false, bvec[l] + i, 1,
               std::min(T, g - i), 1, a, 1.f, 1.f);
    }
  }
  p->n_scaled_tasks = b.task_begin() - first;
  b.end_phase(1, first, b.task_begin() - first);
  return p;
}

size_t sso_sample_plan_dev_bytes(int n_layers, const int64_t* dA, const int64_t* dG) {
  return sso_precond_plan_dev_bytes(n_layers, dA, dG);
}

int64_t sso_sample_plan_create(int n_layers, const int64_t* dA, const int64_t* dG, float* const* U_A,
                               float* const* U_G, float* const* noise, float* const* w,
                               float* const* b, float* const* tmp, void* dev_mem,
                               size_t dev_mem_bytes, int host_only, const int64_t* ldA, const int64_t* ldG) {
  SSO_CHECK_ARG(n_layers > 0 && dA && dG && U_A && U_G && noise && w && tmp, "sample plan: null argument");
  Plan* p = build_sample(n_layers, dA, dG, U_A, U_G, noise, w, b, tmp, ldA, ldG);
  p->host_only = host_only != 0;
  if (!p->host_only) {
    const int rc = upload(*p, dev_mem, dev_mem_bytes);
    if (rc != 0) { delete p; return rc; }
  }
  return register_plan(p);
}

__global__ void set_alpha_kernel(sso_tile_task* tasks, int count, float alpha) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) tasks[i].alpha = alpha;
}

int sso_sample_plan_run(int64_t plan, float std_scale, void* stream) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr && !p->host_only, "unknown or host-only plan %lld", (long long)plan);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (p->n_scaled_tasks > 0) {
    set_alpha_kernel<<<ceil_div(p->n_scaled_tasks, 256), 256, 0, st>>>(p->d_tasks + p->first_scaled_task,
                                                                     p->n_scaled_tasks, std_scale);
    SSO_LAUNCH_OK("set_alpha_kernel");
  }
  return run_phases(*p, p->run_phases, nullptr, st);
}

// ---- generic ---------------------------------------------------------------------------------
int sso_plan_destroy(int64_t plan) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_plans.find(plan);
  if (it == g_plans.end()) return fail(-1, "unknown plan %lld", (long long)plan);
  delete it->second;
  g_plans.erase(it);
  return 0;
}

static const std::vector<sso_phase> all_phases(const Plan& p) {
  std::vector<sso_phase> v(p.inv_phases);
  v.insert(v.end(), p.std_phases.begin(), p.std_phases.end());
  v.insert(v.end(), p.run_phases.begin(), p.run_phases.end());
  return v;
}

int sso_plan_num_phases(int64_t plan) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr, "unknown plan");
  return (int)all_phases(*p).size();
}
int sso_plan_get_phase(int64_t plan, int index, sso_phase* out) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr && out != nullptr, "unknown plan");
  const auto v = all_phases(*p);
  SSO_CHECK_ARG(index >= 0 && index < (int)v.size(), "phase index out of range");
  *out = v[index];
  return 0;
}
int sso_plan_num_tasks(int64_t plan) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr, "unknown plan");
  return (int)p->tasks.size();
}
int sso_plan_copy_tasks(int64_t plan, sso_tile_task* out, int capacity) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr && out != nullptr, "unknown plan");
  const int n = std::min(capacity, (int)p->tasks.size());
  std::copy(p->tasks.begin(), p->tasks.begin() + n, out);
  return n;
}

int sso_plan_num_diag_recs(int64_t plan) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr, "unknown plan");
  return (int)p->diags.size();
}
int sso_plan_copy_diag_recs(int64_t plan, sso_diag_rec* out, int capacity) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr && out != nullptr, "unknown plan");
  const int n = std::min(capacity, (int)p->diags.size());
  std::copy(p->diags.begin(), p->diags.begin() + n, out);
  return n;
}
int sso_plan_num_copy_recs(int64_t plan) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr, "unknown plan");
  return (int)p->copies.size();
}
int sso_plan_copy_copy_recs(int64_t plan, sso_copy_rec* out, int capacity) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr && out != nullptr, "unknown plan");
  const int n = std::min(capacity, (int)p->copies.size());
  std::copy(p->copies.begin(), p->copies.begin() + n, out);
  return n;
}

int sso_plan_status(int64_t plan) {
  Plan* p = find_plan(plan);
  SSO_CHECK_ARG(p != nullptr && !p->host_only && p->d_status != nullptr, "unknown or host-only plan");
  int v = 0;
  SSO_CUDA_OK(cudaMemcpy(&v, p->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  return v;
}

int sso_run_tile_tasks(const sso_tile_task* tasks_dev, int count, int tile, void* stream) {
  SSO_CHECK_ARG(tasks_dev != nullptr && count > 0, "run_tile_tasks: empty");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (tile == 64) tile_task_kernel<4><<<count, 256, 0, st>>>(tasks_dev);
  else if (tile == 128) tile_task_kernel<8><<<count, 256, 0, st>>>(tasks_dev);
  else return fail(-1, "tile must be 64 or 128");
  SSO_LAUNCH_OK("tile_task_kernel");
  return 0;
}

}  // extern "C"
