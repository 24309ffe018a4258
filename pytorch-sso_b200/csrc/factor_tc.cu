// Kronecker-factor construction on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   partial[tile][split] = sum over this split's rows r of  u_r[I] u_r[J]^T      (128x128 fp32)
//
// One CTA owns one lower-triangle 128x128 output tile and one split of the rows.  17 warps:
//   warps 0-7   accumulate: drain the TMEM accumulator (tcgen05.ld) into fp32 registers every
//               `flush` stages -- the tensor core's own running sum is kept short, the long
//               sum is done with round-to-nearest FADDs -- and finally store the tile;
//   warp  8     one elected thread issues tcgen05.mma (M=128, N=128, operands in shared memory,
//               MN-major canonical layout without swizzle) and commits to mbarriers;
//   warps 9-16  gather: fused im2col.  16-byte global loads of consecutive channels
//               (channels-contiguous inputs: channels_last activations, row-major matrices),
//               conversion in registers, 16-byte shared stores straight into the UMMA operand
//               layout, fence.proxy.async, mbarrier arrive.
// bf16/fp16 inputs: one kind::f16 pass (products of 16-bit values are exact in fp32).
// fp32 inputs: 3xTF32 -- x = hi + lo with hi = rna_tf32(x); hi*hi + hi*lo + lo*hi as three
// kind::tf32 MMAs per k-slice into the same accumulator.
// Column order inside the kernel is (kh, kw, c) so that 16 bytes are one chunk of channels; the
// finishing kernel (factor_tc_reduce) permutes to the (c, kh, kw) order of the public result,
// sums the splits in a fixed order and applies alpha / beta and the mirror.
//
// Every wait is bounded: on a timeout the role records a code in the status word, leaves its
// loop and the finishing kernel poisons the output with NaN instead of returning wrong numbers.
#include <algorithm>

#include "common.cuh"
#include "factor_params.cuh"
#include "tc_common.cuh"

namespace sso {
int factor_tc_run_reduce(const FactorParams& p, int tiles, cudaStream_t st);
namespace tc {

constexpr int TILE = 128;
constexpr int EPI_WARPS = 8;
constexpr int LOAD_WARPS = 8;
constexpr int MMA_WARP = EPI_WARPS;
constexpr int THREADS = 32 * (EPI_WARPS + 1 + LOAD_WARPS);
constexpr int LOAD_THREADS = 32 * LOAD_WARPS;
constexpr uint32_t TMEM_COLS = 256;    // two 128-column accumulators

template <typename T>
struct Cfg;
// Operand layouts in shared memory (canonical UMMA layouts without swizzle; one "core matrix"
// is 8 rows of 16 bytes):
//  16-bit inputs, MN-major: 16 bytes = 8 consecutive columns (channels) of one row k;
//      addr(chunk, k) = chunk*SBO + (k/8)*LBO + (k%8)*16.  The 16 bytes a gather thread fetches
//      are stored as they are.
//  fp32 inputs, K-major (tf32 operands are transposed on the way in): 16 bytes = 4 consecutive
//      rows k of one column;  addr(col, k) = (col/8)*SBO + (k/4)*LBO + (col%8)*16 + (k%4)*4.
//  LBO = 128 and SBO = 1040 = 8*128 + 16 in both: the 16 extra bytes rotate consecutive chunks /
//  column groups across the banks, so the 8 chunks of one 128-byte global line (16-bit) and the
//  32 scalar stores of a warp (fp32) are bank-conflict free.
template <>
struct Cfg<float> {
  static constexpr int KS = 32, CH = 4, STAGES = 3, PARTS = 2, LAG = 0, FLUSH = 2;
  static constexpr uint32_t FMT = 2, MAJOR = 0;  // tf32, K-major
  static constexpr uint32_t LBO = 128, SBO = 1040, OPB = 16 * 1040, KSTEP = 2 * 128;
};
template <>
struct Cfg<__nv_bfloat16> {
  static constexpr int KS = 64, CH = 8, STAGES = 6, PARTS = 1, LAG = 4, FLUSH = 8;
  static constexpr uint32_t FMT = 1, MAJOR = 1;  // bf16, MN-major
  static constexpr uint32_t LBO = 128, SBO = 1040, OPB = 16 * 1040, KSTEP = 2 * 128;
};
template <>
struct Cfg<__half> {
  static constexpr int KS = 64, CH = 8, STAGES = 6, PARTS = 1, LAG = 4, FLUSH = 8;
  static constexpr uint32_t FMT = 0, MAJOR = 1;  // f16, MN-major
  static constexpr uint32_t LBO = 128, SBO = 1040, OPB = 16 * 1040, KSTEP = 2 * 128;
};

template <typename T>
__global__ void __launch_bounds__(THREADS, 1) factor_tc_kernel(const FactorParams p, int flush) {
  using C = Cfg<T>;
  constexpr int KS = C::KS, CH = C::CH, STAGES = C::STAGES, PARTS = C::PARTS;
  constexpr uint32_t OPB = C::OPB, SBO = C::SBO, LBO = C::LBO, KSTEP = C::KSTEP;
  constexpr uint32_t STAGE_BYTES = 2 * PARTS * OPB;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_base_slot;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int bi, bj;
  tri_decode(blockIdx.x, bi, bj);
  const bool share = (bi == bj) && (p.weight == nullptr);
  const int split = blockIdx.y;
  const int64_t r_begin = (int64_t)split * p.rows_per_split;
  const int64_t r_end = min(p.rows, r_begin + (int64_t)p.rows_per_split);
  // bits 16 / 17 of `flush` are timing experiments: skip the gather's copies / skip the MMAs
  const bool dbg_no_gather = (flush & 0x10000) != 0, dbg_no_mma = (flush & 0x20000) != 0;
  flush &= 0xFFFF;
  const int nstages = (int)ceil_div64(max((int64_t)0, r_end - r_begin), KS);
  const int nchunks = ceil_div(nstages, flush);
  int* status = p.status;

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
    // ------------------------------------------------------------------ accumulate warps
    const int q = warp & 3, half = warp >> 2;
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    for (int c = 0; c < nchunks; ++c) {
      const int b = c & 1;
      if (!mbar_wait(accfull_bar(b), (c >> 1) & 1, status, 3)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * TILE + half * 64);
      uint32_t v0[32], v1[32];
      tmem_ld32(taddr, v0);
      tmem_ld32(taddr + 32, v1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(accempty_bar(b));   // one arrival per warp
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        acc[i] += __uint_as_float(v0[i]);
        acc[32 + i] += __uint_as_float(v1[i]);
      }
    }
    float* dst = p.partial + ((int64_t)blockIdx.x * p.splits + split) * (TILE * TILE) +
                 (q * 32 + lane) * TILE + half * 64;
#pragma unroll
    for (int i = 0; i < 64; i += 4)
      *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(C::FMT, C::MAJOR);
      bool ok = true;
      for (int s = 0; s < nstages && ok; ++s) {
        const int slot = s % STAGES, c = s / flush, b = c & 1;
        const bool first_of_chunk = (s % flush) == 0;
        if (first_of_chunk && c >= 2) ok = mbar_wait(accempty_bar(b), ((c >> 1) - 1) & 1, status, 2);
        if (!ok) break;
        ok = mbar_wait(full_bar(slot), (s / STAGES) & 1, status, 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sb = smem0 + slot * STAGE_BYTES;
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * TILE);
        if (dbg_no_mma && s > 0) {
        } else if (PARTS == 1) {
          const uint32_t a0 = sb, b0 = share ? sb : sb + OPB;
#pragma unroll
          for (int ks = 0; ks < KS / 16; ++ks) {
            const uint64_t ad = smem_desc(a0 + ks * KSTEP, LBO, SBO);
            const uint64_t bd = smem_desc(b0 + ks * KSTEP, LBO, SBO);
            umma<false>(d_tmem, ad, bd, idesc, (first_of_chunk && ks == 0) ? 0u : 1u);
          }
        } else {
          const uint32_t ah = sb, al = sb + OPB;
          const uint32_t bh = share ? ah : sb + 2 * OPB, bl = share ? al : sb + 3 * OPB;
#pragma unroll
          for (int ks = 0; ks < KS / 8; ++ks) {
            const uint64_t adh = smem_desc(ah + ks * KSTEP, LBO, SBO), adl = smem_desc(al + ks * KSTEP, LBO, SBO);
            const uint64_t bdh = smem_desc(bh + ks * KSTEP, LBO, SBO), bdl = smem_desc(bl + ks * KSTEP, LBO, SBO);
            umma<true>(d_tmem, adl, bdh, idesc, (first_of_chunk && ks == 0) ? 0u : 1u);
            umma<true>(d_tmem, adh, bdl, idesc, 1u);
            umma<true>(d_tmem, adh, bdh, idesc, 1u);
          }
        }
        umma_commit(empty_bar(slot));
        if ((s % flush) == flush - 1 || s == nstages - 1) umma_commit(accfull_bar(b));
      }
    }
  } else {
    // ------------------------------------------------------------------ gather warps
    // Work item = (row k of the stage, group of 8 consecutive 16-byte chunks of one operand):
    // the 8 lanes of an item read one 128-byte line of one input pixel (coalesced) and write
    // 8 chunks whose shared addresses are SBO = 1040 bytes apart, i.e. 16 bytes apart modulo
    // 128 -> one conflict-free wavefront per line.  A warp instruction covers 4 consecutive rows.
    const int lt = tid - 32 * (MMA_WARP + 1);      // 0 .. 255
    const int l8 = lt & 7, q = lt >> 3;            // chunk within its group, item slot 0..31
    constexpr int GROUPS = TILE / (8 * CH);        // chunk groups per operand (2 or 4)
    constexpr int ROWS_PER_THREAD = KS / 32;       // rows q, q+32, ... of the stage: 1 (fp32) or 2 (16-bit)
    constexpr int G_PER_ROW = GROUPS;              // a thread covers chunk l8 of every group of its rows
    const T* xp = reinterpret_cast<const T*>(p.x);
    const int Cc = p.c;
    const int nops = share ? 1 : 2;
    const int hw = p.ho * p.wo;

    // per (operand, group) constants of this thread's chunk
    int koff[2][G_PER_ROW], kpos[2][G_PER_ROW];
#pragma unroll
    for (int op = 0; op < 2; ++op)
#pragma unroll
      for (int g = 0; g < G_PER_ROW; ++g) {
        const int ch = g * 8 + l8;
        const int j0 = (op == 0 ? bi : bj) * TILE + ch * CH;
        if (j0 < p.dcols) {
          const int pos = j0 / Cc, c0 = j0 - pos * Cc;
          const int ky = pos / p.kw, kx = pos - ky * p.kw;
          const int dh = ky * p.dil_h, dw = kx * p.dil_w;
          koff[op][g] = (int)(dh * p.sh + dw * p.sw) + c0;
          kpos[op][g] = dh | (dw << 16);
        } else {
          koff[op][g] = 0;
          kpos[op][g] = (j0 == p.dcols && j0 < p.d) ? -1 : -2;   // ones column / outside
        }
      }
    const bool no_halo = (p.kh == 1 && p.kw == 1 && p.pad_h == 0 && p.pad_w == 0);
    // row walkers: decode the first row once, then advance by KS rows per stage with carries
    int64_t rr[ROWS_PER_THREAD];
    int wn[ROWS_PER_THREAD], wy[ROWS_PER_THREAD], wx[ROWS_PER_THREAD];
#pragma unroll
    for (int j = 0; j < ROWS_PER_THREAD; ++j) {
      rr[j] = r_begin + q + 32 * j;
      wn[j] = (int)(rr[j] / hw);
      const int rem = (int)(rr[j] - (int64_t)wn[j] * hw);
      wy[j] = rem / p.wo;
      wx[j] = rem - wy[j] * p.wo;
    }
    const int step_n = KS / hw, step_rem = KS - step_n * hw;
    const int step_y = step_rem / p.wo, step_x = step_rem - step_y * p.wo;
    auto advance = [&](int j) {
      rr[j] += KS;
      wx[j] += step_x;
      if (wx[j] >= p.wo) { wx[j] -= p.wo; ++wy[j]; }
      wy[j] += step_y;
      if (wy[j] >= p.ho) { wy[j] -= p.ho; ++wn[j]; }
      wn[j] += step_n;
    };
    bool ok = true;
    if (PARTS == 1) {
      // 16-bit inputs need no conversion: cp.async copies 16 bytes global -> shared straight
      // into the operand layout (zero-filling where the patch leaves the image), with LAG
      // stages in flight per thread; a stage is handed to the MMA warp once its copies landed.
      constexpr int LAG = C::LAG;
      for (int s = 0; s < nstages + LAG && ok; ++s) {
        if (s < nstages) {
          const int slot = s % STAGES;
          if (s >= STAGES) ok = mbar_wait(empty_bar(slot), ((s / STAGES) - 1) & 1, status, 4);
          if (!ok) break;
          const uint32_t sb = smem0 + slot * STAGE_BYTES;
#pragma unroll
          for (int j = 0; j < ROWS_PER_THREAD; ++j) {
            const int krow = q + 32 * j;
            const bool rvalid = rr[j] < r_end;
            const int ih0 = wy[j] * p.stride_h - p.pad_h, iw0 = wx[j] * p.stride_w - p.pad_w;
            const T* pix = xp + ((int64_t)wn[j] * p.sn + (int64_t)ih0 * p.sh + (int64_t)iw0 * p.sw);
            const uint32_t arow = sb + l8 * SBO + (krow >> 3) * LBO + (krow & 7) * 16;
#pragma unroll
            for (int op = 0; op < 2; ++op) {
              if (op >= nops) continue;
#pragma unroll
              for (int g = 0; g < G_PER_ROW; ++g) {
                const uint32_t a = arow + op * OPB + g * 8 * SBO;
                const int kp = kpos[op][g];
                if (kp == -1) {
                  const uint32_t one = !rvalid ? 0u : (C::FMT == 1 ? 0x3F80u : 0x3C00u);
                  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%2,%2};" ::"r"(a), "r"(one), "r"(0u) : "memory");
                } else {
                  bool in = rvalid && kp >= 0;
                  if (!no_halo)
                    in = in && (unsigned)(ih0 + (kp & 0xFFFF)) < (unsigned)p.h &&
                         (unsigned)(iw0 + (kp >> 16)) < (unsigned)p.w;
                  if (dbg_no_gather) continue;
                  const T* src = in ? pix + koff[op][g] : xp;
                  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a), "l"(src), "r"(in ? 16 : 0) : "memory");
                }
              }
            }
            advance(j);
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (s >= LAG) {
          asm volatile("cp.async.wait_group %0;" ::"n"(LAG) : "memory");
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(full_bar((s - LAG) % STAGES));   // one arrival per warp
        }
      }
    } else {
      // fp32 inputs: 16-byte loads into registers, split into tf32 hi / lo, transposing scalar
      // stores into the K-major operand layout (bank-conflict free thanks to the padded SBO)
      for (int s = 0; s < nstages && ok; ++s) {
        const int slot = s % STAGES;
        const int krow = q;
        const bool rvalid = rr[0] < r_end;
        const int ih0 = wy[0] * p.stride_h - p.pad_h, iw0 = wx[0] * p.stride_w - p.pad_w;
        const T* pix = xp + ((int64_t)wn[0] * p.sn + (int64_t)ih0 * p.sh + (int64_t)iw0 * p.sw);
        const float wgt = (p.weight && rvalid) ? p.weight[wn[0]] : 1.f;
        uint4 v[2][G_PER_ROW];
#pragma unroll
        for (int op = 0; op < 2; ++op)
#pragma unroll
          for (int g = 0; g < G_PER_ROW; ++g) {
            v[op][g] = make_uint4(0u, 0u, 0u, 0u);
            if (op < nops && rvalid) {
              const int kp = kpos[op][g];
              if (kp >= 0) {
                if (no_halo || ((unsigned)(ih0 + (kp & 0xFFFF)) < (unsigned)p.h &&
                                (unsigned)(iw0 + (kp >> 16)) < (unsigned)p.w))
                  v[op][g] = __ldg(reinterpret_cast<const uint4*>(pix + koff[op][g]));
              } else if (kp == -1) {
                v[op][g].x = __float_as_uint(1.f);
              }
            }
          }
        advance(0);
        if (s >= STAGES) ok = mbar_wait(empty_bar(slot), ((s / STAGES) - 1) & 1, status, 4);
        if (!ok) break;
        const uint32_t sb = smem0 + slot * STAGE_BYTES + (krow >> 2) * LBO + (krow & 3) * 4;
#pragma unroll
        for (int op = 0; op < 2; ++op) {
          if (op >= nops) continue;
#pragma unroll
          for (int g = 0; g < G_PER_ROW; ++g) {
            float f[4] = {__uint_as_float(v[op][g].x), __uint_as_float(v[op][g].y), __uint_as_float(v[op][g].z),
                          __uint_as_float(v[op][g].w)};
            const int col0 = (g * 8 + l8) * 4;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              if (op == 0) f[t] *= wgt;
              const uint32_t hi = rna_tf32(f[t]);
              const uint32_t lo = __float_as_uint(f[t] - __uint_as_float(hi));
              const int col = col0 + t;
              const uint32_t a = sb + op * (PARTS * OPB) + (col >> 3) * SBO + (col & 7) * 16;
              asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(hi) : "memory");
              asm volatile("st.shared.b32 [%0], %1;" ::"r"(a + OPB), "r"(lo) : "memory");
            }
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(slot));
      }
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

// Sum the splits (fixed order), permute internal (kh,kw,c) columns to (c,kh,kw), apply
// alpha / beta, mirror.  A non-zero status (a wait gave up) poisons the result with NaN.
//
// One CTA produces 32 output rows x one group of columns that is CONTIGUOUS in the output:
// for permuted factors a block of up to 8 channels at all kernel positions (8*kk columns), else
// 32 consecutive columns.  Inside the partial tiles such a group is kk runs of 8 consecutive
// columns.  Elements on or below the diagonal are read from their own tile with the lanes along
// the run; elements above it are read from the mirrored position with the lanes along the rows,
// so global reads come in whole 32-byte sectors, writes in whole rows of the group, and both
// halves of the symmetric result come from the same numbers (bitwise symmetric).  The block is
// staged in shared memory.
constexpr int RED_ROWS = 32, RED_CB = 8, RED_W = 32;

// sum over the splits of element (r, c), r >= c, of the lower-triangle partial tiles; four
// independent partial sums keep several loads in flight, combined in a fixed order
__device__ __forceinline__ float reduce_fetch(const float* __restrict__ partial, int nsplit, int r, int c) {
  const int bi = r >> 7, bj = c >> 7;
  const float* src = partial + ((int64_t)(bi * (bi + 1) / 2 + bj) * nsplit) * (TILE * TILE) + (r & 127) * TILE + (c & 127);
  constexpr int64_t S = TILE * TILE;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int sp = 0;
  for (; sp + 4 <= nsplit; sp += 4) {
    a0 += src[sp * S];
    a1 += src[(sp + 1) * S];
    a2 += src[(sp + 2) * S];
    a3 += src[(sp + 3) * S];
  }
  for (; sp < nsplit; ++sp) a0 += src[sp * S];
  return (a0 + a1) + (a2 + a3);
}

__global__ void __launch_bounds__(256) factor_tc_reduce(const FactorParams p, int perm_groups, int pitch) {
  extern __shared__ float rs[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gi0 = blockIdx.x * RED_ROWS;
  const int grp = blockIdx.y;
  const int kk = p.perm_kk, C = p.perm_c, d = p.d;
  int ext0, n_ext;
  if (grp < perm_groups) {
    const int c0 = grp * RED_CB, len = min(RED_CB, C - c0);
    ext0 = c0 * kk;
    n_ext = len * kk;
    // below / on the diagonal: 4 rows x 8 columns per warp; above: 32 rows x 1 column per warp
    const int rrA = warp * 4 + (lane >> 3), eA = lane & 7, giA = gi0 + rrA;
    const int rrB = lane, eB = warp, giB = gi0 + rrB;
    const bool okA = eA < len && giA < d, okB = eB < len && giB < d;
#pragma unroll 3
    for (int run = 0; run < kk; ++run) {
      const int gjA = run * C + c0 + eA, gjB = run * C + c0 + eB;
      float vA = 0.f, vB = 0.f;
      const bool doA = okA && gjA <= giA, doB = okB && gjB > giB;
      if (doA) vA = reduce_fetch(p.partial, p.splits, giA, gjA);
      if (doB) vB = reduce_fetch(p.partial, p.splits, gjB, giB);
      if (doA) rs[rrA * pitch + eA * kk + run] = vA;
      if (doB) rs[rrB * pitch + eB * kk + run] = vB;
    }
  } else {
    ext0 = (perm_groups > 0 ? p.dcols : 0) + (grp - perm_groups) * RED_W;
    n_ext = min(RED_W, d - ext0);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int rrA = warp + 8 * k, giA = gi0 + rrA, gjA = ext0 + lane;
      const int eB = warp + 8 * k, giB = gi0 + lane, gjB = ext0 + eB;
      const bool doA = lane < n_ext && giA < d && gjA <= giA;
      const bool doB = eB < n_ext && giB < d && gjB > giB;
      float vA = 0.f, vB = 0.f;
      if (doA) vA = reduce_fetch(p.partial, p.splits, giA, gjA);
      if (doB) vB = reduce_fetch(p.partial, p.splits, gjB, giB);
      if (doA) rs[rrA * pitch + lane] = vA;
      if (doB) rs[lane * pitch + eB] = vB;
    }
  }
  __syncthreads();
  const bool bad = p.status && *p.status != 0;
  for (int rr = warp; rr < RED_ROWS; rr += 8) {
    const int gi = gi0 + rr;
    if (gi >= d) break;
    const int gr = (C > 0 && gi < p.dcols) ? (gi % C) * kk + gi / C : gi;
    float* orow = p.out + (int64_t)gr * p.ldo + ext0;
    for (int e = lane; e < n_ext; e += 32) {
      float v = p.alpha * rs[rr * pitch + e];
      if (bad) v = __int_as_float(0x7fc00000);
      orow[e] = (p.beta == 0.f) ? v : fmaf(p.beta, orow[e], v);
    }
  }
}

// Tile-wise variant of the finishing kernel: a CTA sums 1024/SL elements of one partial tile with
// 16-byte loads and scatters them (and their mirror) to the output.  It wins when many splits
// make the partial tiles, not the output, the bulk of the traffic.  With many splits and few
// tiles, SL = 2, 4 or 8 neighbouring lanes share an element group: lane l sums splits l, l+SL, ...
// and the lanes are combined by shuffles in a fixed tree, so the sum stays deterministic while
// the chains get shorter and SL times more CTAs are in flight.
__global__ void __launch_bounds__(256) factor_tc_reduce_tiles(const FactorParams p, int sl) {
  int bi, bj;
  tri_decode(blockIdx.x, bi, bj);
  const float* src = p.partial + (int64_t)blockIdx.x * p.splits * (TILE * TILE);
  const int group = (blockIdx.y * 256 + threadIdx.x) / sl, sub = threadIdx.x % sl;
  const int e0 = group * 4;
  const int r = e0 / TILE, c0 = e0 % TILE;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f), s2 = make_float4(0.f, 0.f, 0.f, 0.f);
  int sp = sub;
  for (; sp + sl < p.splits; sp += 2 * sl) {      // two independent chains per lane
    const float4 v = *reinterpret_cast<const float4*>(src + (int64_t)sp * (TILE * TILE) + e0);
    const float4 w = *reinterpret_cast<const float4*>(src + (int64_t)(sp + sl) * (TILE * TILE) + e0);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    s2.x += w.x; s2.y += w.y; s2.z += w.z; s2.w += w.w;
  }
  if (sp < p.splits) {
    const float4 v = *reinterpret_cast<const float4*>(src + (int64_t)sp * (TILE * TILE) + e0);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  s.x += s2.x; s.y += s2.y; s.z += s2.z; s.w += s2.w;
  for (int o = 1; o < sl; o <<= 1) {
    s.x += __shfl_xor_sync(0xffffffffu, s.x, o);
    s.y += __shfl_xor_sync(0xffffffffu, s.y, o);
    s.z += __shfl_xor_sync(0xffffffffu, s.z, o);
    s.w += __shfl_xor_sync(0xffffffffu, s.w, o);
  }
  if (sub != 0) return;
  const bool bad = p.status && *p.status != 0;
  auto ext = [&](int j) {
    if (p.perm_c > 0 && j < p.dcols) return (j % p.perm_c) * p.perm_kk + j / p.perm_c;
    return j;
  };
  const int gi = bi * TILE + r;
  if (gi >= p.d) return;
  const int gr = ext(gi);
  const float vals[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int gj = bj * TILE + c0 + q;
    if (gj >= p.d || gj > gi) continue;   // diagonal tiles: lower triangle only, mirrored below
    const int gc = ext(gj);
    float v = p.alpha * vals[q];
    if (bad) v = __int_as_float(0x7fc00000);
    float* o = p.out + (int64_t)gr * p.ldo + gc;
    if (gi != gj) {
      float* o2 = p.out + (int64_t)gc * p.ldo + gr;
      *o2 = (p.beta == 0.f) ? v : fmaf(p.beta, *o2, v);
    }
    *o = (p.beta == 0.f) ? v : fmaf(p.beta, *o, v);
  }
}

// Rows are split so that tiles*splits CTAs (one per SM at a time) fill whole waves of the 148 SMs
// as evenly as possible; more splits cost more partial-tile traffic, so a larger count must buy
// at least 4 % of wave efficiency.
static void choose_splits(int64_t rows, int tiles, int ks, int& splits, int& rows_per_split) {
  const int kSMs = 148;
  const int64_t most = std::max<int64_t>(1, rows / (4 * ks));   // at least 4 stages per split
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= 64 && s <= most; ++s) {
    const int64_t ctas = (int64_t)tiles * s;
    const double eff = (double)ctas / (double)(kSMs * ceil_div64(ctas, kSMs));
    if (eff > best_eff + 0.04) { best_eff = eff; best = s; }
  }
  int64_t rps = ceil_div64(ceil_div64(rows, best), ks) * ks;
  splits = (int)ceil_div64(rows, rps);
  if (splits < 1) splits = 1;
  rows_per_split = (int)rps;
}

}  // namespace tc

static int g_flush_stages = 0;   // stages between drains of the TMEM accumulator; 0 = per-dtype default

size_t factor_tc_workspace_bytes(int64_t rows, int64_t d) {
  const int nb = (int)ceil_div64(d, 128);
  const int tiles = nb * (nb + 1) / 2;
  int splits, rps;
  tc::choose_splits(rows, tiles, 32, splits, rps);   // the fp32 stage depth gives the larger count
  int s2, r2;
  tc::choose_splits(rows, tiles, 64, s2, r2);
  if (s2 > splits) splits = s2;
  // the TMA-fed kernel spreads one- and two-tile problems over all SMs (up to 148 splits); stay
  // below 12 MB of partial tiles for them
  const int64_t wide = std::min<int64_t>(std::min<int64_t>(148, 192 / tiles), std::max<int64_t>(1, rows / 512));
  if (wide > splits) splits = (int)wide;
  return factor_header_bytes(tiles) + (size_t)tiles * splits * 128 * 128 * sizeof(float);
}

bool factor_tc_supported(const FactorParams& p, int dtype) {
  const int ch = (dtype == SSO_F32) ? 4 : 8;
  const int esz = (dtype == SSO_F32) ? 4 : 2;
  if (p.sc != 1) return false;
  if (p.c % ch != 0) return false;
  if ((reinterpret_cast<uintptr_t>(p.x) & 15) != 0) return false;
  if ((p.sn * esz) % 16 != 0) return false;
  if (p.h > 1 && (p.sh * esz) % 16 != 0) return false;
  if (p.w > 1 && (p.sw * esz) % 16 != 0) return false;
  if (p.weight != nullptr && dtype != SSO_F32) return false;  // weights would round 16-bit operands
  return true;
}

template <typename T>
static int tc_launch_typed(FactorParams p, int tiles, cudaStream_t st) {
  using C = tc::Cfg<T>;
  tc::choose_splits(p.rows, tiles, C::KS, p.splits, p.rows_per_split);
  const size_t smem = (size_t)C::STAGES * 2 * C::PARTS * C::OPB + 128;
  SSO_ENSURE_SMEM((tc::factor_tc_kernel<T>), smem);
  tc::factor_tc_kernel<T><<<dim3(tiles, p.splits), tc::THREADS, smem, st>>>(
      p, g_flush_stages > 0 ? g_flush_stages : C::FLUSH);
  SSO_LAUNCH_OK("factor_tc_kernel");
  return factor_tc_run_reduce(p, tiles, st);
}

int factor_tc_launch(FactorParams p, int dtype, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  const int nb = ceil_div(p.d, 128);
  const int tiles = nb * (nb + 1) / 2;
  const size_t need = factor_tc_workspace_bytes(p.rows, p.d);
  SSO_CHECK_ARG(workspace != nullptr && workspace_bytes >= need,
                "factor workspace too small: need %zu bytes, got %zu", need, workspace_bytes);
  p.status = reinterpret_cast<int*>(workspace);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + factor_header_bytes(tiles));
  p.tickets = nullptr;
  SSO_CUDA_OK(cudaMemsetAsync(p.status, 0, sizeof(int), st));
  // internal column order (kh, kw, c); identity when there is a single kernel position
  p.perm_c = (p.kh * p.kw > 1) ? p.c : 0;
  p.perm_kk = p.kh * p.kw;
  switch (dtype) {
    case SSO_F32: return tc_launch_typed<float>(p, tiles, st);
    case SSO_BF16: return tc_launch_typed<__nv_bfloat16>(p, tiles, st);
    case SSO_F16: return tc_launch_typed<__half>(p, tiles, st);
  }
  return fail(-1, "unknown dtype %d", dtype);
}

// Permuted factors of at least 1024 columns with at most this many splits are finished row-wise (whole
// output rows through shared memory); the tile-wise kernel scatters 4-byte stores when columns are permuted.
// 8 instead of 3: VGG-16-style step 59.5 -> 58.3 ms, 5x5 ConvNet step unchanged.
static int g_rowwise_max_splits = 8;
void factor_tc_set_rowwise_max_splits(int s) { g_rowwise_max_splits = s; }

int factor_tc_run_reduce(const FactorParams& p, int tiles, cudaStream_t st) {
  // a large permuted factor with not too many splits: the output dominates, write it in whole rows
  if (!(p.perm_c > 0 && p.splits <= g_rowwise_max_splits && p.d >= 1024)) {
    // lanes per element group: enough CTAs to fill the GPU when there are few tiles, and chains
    // of at most ~8 partial tiles per lane
    int sl = 1;
    while (sl < 8 && (tiles * 16 * sl < 2 * 148 || p.splits > 8 * sl) && p.splits >= 4 * sl) sl <<= 1;
    tc::factor_tc_reduce_tiles<<<dim3(tiles, 16 * sl), 256, 0, st>>>(p, sl);
    SSO_LAUNCH_OK("factor_tc_reduce_tiles");
    return 0;
  }
  int perm_groups = 0, width = tc::RED_W;
  if (p.perm_c > 0) {
    perm_groups = ceil_div(p.perm_c, tc::RED_CB);
    width = std::max(tc::RED_CB * p.perm_kk, 1);
  }
  const int plain_groups = p.perm_c > 0 ? (p.d > p.dcols ? 1 : 0) : ceil_div(p.d, tc::RED_W);
  const int pitch = width | 1;
  const size_t smem = (size_t)tc::RED_ROWS * pitch * sizeof(float);
  SSO_CHECK_ARG(smem <= 200 * 1024, "factor: kernel window too large for the finishing kernel");
  SSO_ENSURE_SMEM(tc::factor_tc_reduce, 200 * 1024);
  tc::factor_tc_reduce<<<dim3(ceil_div(p.d, tc::RED_ROWS), perm_groups + plain_groups), 256, smem, st>>>(p, perm_groups, pitch);
  SSO_LAUNCH_OK("factor_tc_reduce");
  return 0;
}

int factor_tc_set_wait_controls(long long cycles, int stall) { return tc::set_wait_controls(cycles, stall); }

int factor_tc_flush_setting() { return g_flush_stages & 0xFFFF; }

void factor_tc_set_flush(int stages) { g_flush_stages = stages < 0 ? 0 : stages; }  // see kernel for bits 16/17

}  // namespace sso
