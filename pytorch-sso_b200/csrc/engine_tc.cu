// Tile tasks on the tensor cores:  C[m x n] <- alpha * op(A)[m x k] * op(B)[k x n] + beta * C  with
// m, n <= 128, fp32 in / fp32 out, computed as 3xTF32 on tcgen05 (x = hi + lo, hi = rna_tf32(x);
// lo*hi + hi*lo + hi*hi into one TMEM accumulator that is drained into fp32 registers every two
// stages, because the tensor core's own accumulation truncates).
//
// One CTA per task, 17 warps: 8 accumulate warps, 1 MMA warp, 8 load warps.  Both operands end up
// K-major in shared memory (canonical no-swizzle layout, core matrix = 8 rows x 16 bytes):
//   * operand contiguous along k in global memory (A not transposed, B transposed): a thread loads
//     16 bytes = 4 consecutive k of one row and stores them as they are; 8 lanes = one 128-byte line;
//     LBO = 144, SBO = 1152 rotate the 8 k-chunks of a row over the banks;
//   * operand contiguous along its row/column index (A transposed, B not transposed): a thread loads
//     4 consecutive indices of one k and scatters them with scalar stores; LBO = 128, SBO = 1040.
// Unaligned bases / leading dimensions (odd matrix sizes) fall back to element loads.
// Every wait is bounded; a timeout sets *status and the task writes nothing.
#include "common.cuh"
#include "tc_common.cuh"

namespace sso {
namespace etc {

using namespace tc;

constexpr int TILE = 128, KS = 32, STAGES = 3;
constexpr int EPI_WARPS = 8, MMA_WARP = 8, LOAD_WARPS = 8;
constexpr int THREADS = 32 * (EPI_WARPS + 1 + LOAD_WARPS);
constexpr uint32_t OPB = 16 * 1152;                 // bytes of one operand part (hi or lo) of one stage
constexpr uint32_t STAGE_BYTES = 4 * OPB;           // A_hi A_lo B_hi B_lo
constexpr uint32_t TMEM_COLS = 256;
constexpr int FLUSH = 2;

struct Layout {
  uint32_t lbo, sbo;
};
__device__ __forceinline__ Layout layout_of(bool kcontig) { return kcontig ? Layout{144u, 1152u} : Layout{128u, 1040u}; }

__device__ __forceinline__ void split_store4(uint32_t addr, float4 v) {
  const uint32_t h0 = rna_tf32(v.x), h1 = rna_tf32(v.y), h2 = rna_tf32(v.z), h3 = rna_tf32(v.w);
  const uint32_t l0 = __float_as_uint(v.x - __uint_as_float(h0)), l1 = __float_as_uint(v.y - __uint_as_float(h1));
  const uint32_t l2 = __float_as_uint(v.z - __uint_as_float(h2)), l3 = __float_as_uint(v.w - __uint_as_float(h3));
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(h0), "r"(h1), "r"(h2), "r"(h3) : "memory");
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr + OPB), "r"(l0), "r"(l1), "r"(l2), "r"(l3) : "memory");
}
__device__ __forceinline__ void split_store1(uint32_t addr, float x) {
  const uint32_t h = rna_tf32(x);
  const uint32_t l = __float_as_uint(x - __uint_as_float(h));
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(h) : "memory");
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr + OPB), "r"(l) : "memory");
}

// 4 consecutive elements along the contiguous direction starting at (fixed, first); elements whose
// contiguous index is >= lim_c or whose other index is out of range read as zero.
__device__ __forceinline__ float4 load4(const float* __restrict__ P, int64_t ld, int fixed, int first, bool fixed_ok,
                                        int lim_c, bool vec_ok) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!fixed_ok || first >= lim_c) return v;
  const float* q = P + (int64_t)fixed * ld + first;
  if (vec_ok && first + 3 < lim_c) return __ldg(reinterpret_cast<const float4*>(q));
  v.x = __ldg(q);
  if (first + 1 < lim_c) v.y = __ldg(q + 1);
  if (first + 2 < lim_c) v.z = __ldg(q + 2);
  if (first + 3 < lim_c) v.w = __ldg(q + 3);
  return v;
}

__global__ void __launch_bounds__(THREADS, 1) tile_task_tc_kernel(const sso_tile_task* __restrict__ tasks, int* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_base_slot;
  const sso_tile_task t = tasks[blockIdx.x];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool ta = t.flags & 1u, tb = t.flags & 2u;
  const bool a_kc = !ta, b_kc = tb;
  const Layout la = layout_of(a_kc), lb = layout_of(b_kc);
  const int nstages = ceil_div(t.k, KS);
  const int nchunks = ceil_div(nstages, FLUSH);

  const uint32_t smem0 = (smem_u32(smem_raw) + 127u) & ~127u;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto accfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto accempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), LOAD_WARPS);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accfull_bar(b), 1);
      mbar_init(accempty_bar(b), EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp < EPI_WARPS) {
    // ------------------------------------------------------------------ accumulate + epilogue
    const int q = warp & 3, half = warp >> 2;
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    bool ok = true;
    for (int c = 0; c < nchunks; ++c) {
      const int b = c & 1;
      if (!mbar_wait(accfull_bar(b), (c >> 1) & 1, status, 13)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * TILE + half * 64);
      uint32_t v0[32], v1[32];
      tmem_ld32(taddr, v0);
      tmem_ld32(taddr + 32, v1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(accempty_bar(b));
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        acc[i] += __uint_as_float(v0[i]);
        acc[32 + i] += __uint_as_float(v1[i]);
      }
    }
    const int r = q * 32 + lane;
    if (ok && r < t.m) {
      float* crow = t.C + (int64_t)r * t.ldc;
#pragma unroll 4
      for (int i = 0; i < 64; ++i) {
        const int c = half * 64 + i;
        if (c >= t.n) break;
        if ((t.flags & 4u) && c > r) break;      // symmetric tile: lower half computed, mirrored below
        float v = t.alpha * acc[i];
        if (t.beta != 0.f) v = fmaf(t.beta, crow[c], v);
        crow[c] = v;
        if (t.C2) t.C2[(int64_t)c * t.ldc2 + r] = v;
        if ((t.flags & 4u) && c < r) t.C[(int64_t)c * t.ldc + r] = v;
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(2u, 0u);   // tf32, K-major
      bool ok = true;
      for (int s = 0; s < nstages && ok; ++s) {
        const int slot = s % STAGES, c = s / FLUSH, b = c & 1;
        const bool first_of_chunk = (s % FLUSH) == 0;
        if (first_of_chunk && c >= 2) ok = mbar_wait(accempty_bar(b), ((c >> 1) - 1) & 1, status, 12);
        if (!ok) break;
        ok = mbar_wait(full_bar(slot), (s / STAGES) & 1, status, 11);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sb = smem0 + slot * STAGE_BYTES;
        const uint32_t ah = sb, al = sb + OPB, bh = sb + 2 * OPB, bl = sb + 3 * OPB;
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * TILE);
#pragma unroll
        for (int ks = 0; ks < KS / 8; ++ks) {
          const uint64_t adh = smem_desc(ah + ks * 2 * la.lbo, la.lbo, la.sbo), adl = smem_desc(al + ks * 2 * la.lbo, la.lbo, la.sbo);
          const uint64_t bdh = smem_desc(bh + ks * 2 * lb.lbo, lb.lbo, lb.sbo), bdl = smem_desc(bl + ks * 2 * lb.lbo, lb.lbo, lb.sbo);
          umma<true>(d_tmem, adl, bdh, idesc, (first_of_chunk && ks == 0) ? 0u : 1u);
          umma<true>(d_tmem, adh, bdl, idesc, 1u);
          umma<true>(d_tmem, adh, bdh, idesc, 1u);
        }
        umma_commit(empty_bar(slot));
        if ((s % FLUSH) == FLUSH - 1 || s == nstages - 1) umma_commit(accfull_bar(b));
      }
    }
  } else {
    // ------------------------------------------------------------------ load warps
    const int lt = tid - 32 * (MMA_WARP + 1);
    const int l8 = lt & 7, q = lt >> 3;               // q: 0..31
    const bool a_vec = ((reinterpret_cast<uintptr_t>(t.A) & 15) == 0) && (t.lda % 4 == 0);
    const bool b_vec = ((reinterpret_cast<uintptr_t>(t.B) & 15) == 0) && (t.ldb % 4 == 0);
    bool ok = true;
    for (int s = 0; s < nstages && ok; ++s) {
      const int slot = s % STAGES, k0 = s * KS;
      float4 va[4], vb[4];
      // operand A: rows i of op(A), contraction index k
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (a_kc) {        // A[i*lda + k]: row i = q + 32j, k-chunk l8
          const int i = q + 32 * j;
          va[j] = load4(t.A, t.lda, i, k0 + l8 * 4, i < t.m, t.k, a_vec);
        } else {           // A[k*lda + i]: k = k0 + q, index chunk l8 + 8j
          const int k = k0 + q;
          va[j] = load4(t.A, t.lda, k, (l8 + 8 * j) * 4, k < t.k, t.m, a_vec);
        }
        if (b_kc) {        // B[jcol*ldb + k]
          const int jc = q + 32 * j;
          vb[j] = load4(t.B, t.ldb, jc, k0 + l8 * 4, jc < t.n, t.k, b_vec);
        } else {           // B[k*ldb + jcol]
          const int k = k0 + q;
          vb[j] = load4(t.B, t.ldb, k, (l8 + 8 * j) * 4, k < t.k, t.n, b_vec);
        }
      }
      if (s >= STAGES) ok = mbar_wait(empty_bar(slot), ((s / STAGES) - 1) & 1, status, 14);
      if (!ok) break;
      const uint32_t sb = smem0 + slot * STAGE_BYTES;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (a_kc) {
          const int i = q + 32 * j;
          split_store4(sb + (i >> 3) * la.sbo + l8 * la.lbo + (i & 7) * 16, va[j]);
        } else {
          const float f[4] = {va[j].x, va[j].y, va[j].z, va[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = (l8 + 8 * j) * 4 + e;
            split_store1(sb + (col >> 3) * la.sbo + (q >> 2) * la.lbo + (col & 7) * 16 + (q & 3) * 4, f[e]);
          }
        }
        if (b_kc) {
          const int jc = q + 32 * j;
          split_store4(sb + 2 * OPB + (jc >> 3) * lb.sbo + l8 * lb.lbo + (jc & 7) * 16, vb[j]);
        } else {
          const float f[4] = {vb[j].x, vb[j].y, vb[j].z, vb[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = (l8 + 8 * j) * 4 + e;
            split_store1(sb + 2 * OPB + (col >> 3) * lb.sbo + (q >> 2) * lb.lbo + (col & 7) * 16 + (q & 3) * 4, f[e]);
          }
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar(slot));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace etc

int launch_tile_tasks_tc(const sso_tile_task* tasks_dev, int count, int* status_dev, cudaStream_t st) {
  const size_t smem = (size_t)etc::STAGES * etc::STAGE_BYTES + 128;
  static bool configured = false;
  if (!configured) {
    SSO_CUDA_OK(cudaFuncSetAttribute(etc::tile_task_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  etc::tile_task_tc_kernel<<<count, etc::THREADS, smem, st>>>(tasks_dev, status_dev);
  SSO_LAUNCH_OK("tile_task_tc_kernel");
  return 0;
}

}  // namespace sso
