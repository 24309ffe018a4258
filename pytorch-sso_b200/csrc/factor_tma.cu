// Kronecker-factor construction with TMA-fed operands: the im2col gather IS the TMA tile load.
//
// For 16-bit channels-contiguous inputs (channels_last activations / row-major matrices) whose
// channel count is a multiple of 64, an operand block "64 channels of kernel position (ky,kx) for
// a rectangle of output pixels" is exactly one 4-D tiled TMA box of the NHWC tensor:
//     box = {64 channels, wo pixels, bh rows, bn images}, start = {c0, kx*dil - pad, oy0*stride +
//     ky*dil - pad, n0}, element strides {1, stride_w, stride_h, 1}; padding is the out-of-bounds
//     zero fill.  With the 128-byte swizzle the box lands in shared memory as rows of 128 bytes, which
//     is the canonical MN-major SWIZZLE_128B operand layout of tcgen05.mma, so no thread touches
//     the data: one producer thread issues up to four box loads per stage and the MMA warp
//     consumes them.
// One CTA = one lower-triangle 128x128 tile x one split of the stages; 8 accumulate warps (drain
// TMEM every few stages into fp32 registers), 1 MMA warp, 1 producer warp.  Partial tiles go to
// the same workspace layout as the gather kernel and are finished by the same reduction.
// No multicast, no peer memory.
#include <cuda.h>

#include <algorithm>
#include <vector>

#include "common.cuh"
#include "factor_finish.cuh"
#include "factor_params.cuh"
#include "tc_common.cuh"

namespace sso {

int factor_tc_run_reduce(const FactorParams& p, int tiles, cudaStream_t st);

namespace tma {

using namespace tc;

constexpr int TILE = 128;
constexpr int EPI_WARPS = 8;
constexpr int MMA_WARP = 8;
constexpr int PROD_WARP = 9;
constexpr int THREADS = 320;
constexpr int STAGES = 3;
constexpr int KPAD_MAX = 128;
constexpr uint32_t BLOCK_BYTES_MAX = KPAD_MAX * 128;       // one 64-column block of one stage
constexpr uint32_t STAGE_BYTES = 4 * BLOCK_BYTES_MAX;      // A0 A1 B0 B1
constexpr uint32_t TMEM_COLS = 256;

struct Geom {
  int bw, bh, bn;        // box in output pixels: width (= wo), rows, images
  int kstage, kpad;      // rows per stage, padded to a multiple of 16
  int ystages;           // stages per image group along the output height
  int total_stages;
  int stages_per_split;
  int flush;
  uint32_t fmt;          // 1 bf16, 0 fp16
};

__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) |
         ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

__global__ void __launch_bounds__(THREADS, 1)
factor_tma_kernel(const FactorParams p, const Geom g, const __grid_constant__ CUtensorMap tmap) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int fin_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int bi, bj;
  tri_decode(blockIdx.x, bi, bj);
  const bool share = (bi == bj);
  const bool fused = p.tickets != nullptr;
  const int split = blockIdx.y;
  const int s_begin = split * g.stages_per_split;
  const int s_end = min(g.total_stages, s_begin + g.stages_per_split);
  const int nstages = max(0, s_end - s_begin);
  const int flush = g.flush;
  const int nchunks = ceil_div(nstages, flush);
  int* status = p.status;

  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto accfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto accempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accfull_bar(b), 1);
      mbar_init(accempty_bar(b), EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // What TMA never writes must read as zeros: the padding rows kstage..kpad of every block, and
  // whole blocks past the matrix edge.  A row of a 64-column block is 128 bytes (the swizzle only
  // permutes 16-byte chunks inside a row), so both are plain byte ranges; nothing else is touched.
  const uint32_t blk_bytes = (uint32_t)g.kpad * 128u;
  for (int sb = 0; sb < 4 * STAGES; ++sb) {
    const int e = sb & 3, op = e >> 1;
    const int j0 = (op == 0 ? bi : bj) * TILE + (e & 1) * 64;
    const bool valid = (j0 < p.dcols) && !(share && op == 1);
    if (share && op == 1) continue;                         // never read on a diagonal tile
    const uint32_t base = smem0 + (sb >> 2) * STAGE_BYTES + op * 2 * BLOCK_BYTES_MAX + (e & 1) * blk_bytes;
    const uint32_t lo = valid ? (uint32_t)g.kstage * 128u : 0u;
    for (uint32_t o = lo + tid * 16u; o < blk_bytes; o += THREADS * 16u)
      asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(base + o), "r"(0u) : "memory");
  }
  fence_async_smem();
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
      if (lane == 0) mbar_arrive(accempty_bar(b));
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        acc[i] += __uint_as_float(v0[i]);
        acc[32 + i] += __uint_as_float(v1[i]);
      }
    }
    if (fused && p.splits == 1) {
      // one split: the accumulator is the result; it goes to the output through the staging tile
      // (the operand buffers are free: the last commit has fired, so every MMA has read them)
      float* ct = reinterpret_cast<float*>(smem_raw + (smem0 - smem_u32(smem_raw))) + (q * 32 + lane) * fin::CT_LD + half * 64;
#pragma unroll
      for (int i = 0; i < 64; ++i) ct[i] = acc[i];
    } else {
      float* dst = p.partial + ((int64_t)blockIdx.x * p.splits + split) * (TILE * TILE) +
                   (q * 32 + lane) * TILE + half * 64;
#pragma unroll
      for (int i = 0; i < 64; i += 4)
        *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
      if (fused) __threadfence();
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(g.fmt, 1u);
      const int nk = g.kpad / 16;
      bool ok = true;
      for (int s = 0; s < nstages && ok; ++s) {
        const int slot = s % STAGES, c = s / flush, b = c & 1;
        const bool first_of_chunk = (s % flush) == 0;
        if (first_of_chunk && c >= 2) ok = mbar_wait(accempty_bar(b), ((c >> 1) - 1) & 1, status, 2);
        if (!ok) break;
        ok = mbar_wait(full_bar(slot), (s / STAGES) & 1, status, 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a0 = smem0 + slot * STAGE_BYTES;
        const uint32_t b0 = share ? a0 : a0 + 2 * BLOCK_BYTES_MAX;
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * TILE);
        for (int ks = 0; ks < nk; ++ks) {
          // K = 16 rows = two 8-row swizzle atoms of 1024 bytes; the next 64-column block of the
          // operand starts blk_bytes further on
          const uint64_t ad = smem_desc_sw128(a0 + ks * 2048u, blk_bytes, 1024u);
          const uint64_t bd = smem_desc_sw128(b0 + ks * 2048u, blk_bytes, 1024u);
          umma<false>(d_tmem, ad, bd, idesc, (first_of_chunk && ks == 0) ? 0u : 1u);
        }
        umma_commit(empty_bar(slot));
        if ((s % flush) == flush - 1 || s == nstages - 1) umma_commit(accfull_bar(b));
      }
    }
  } else if (warp == PROD_WARP) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // the (up to) four 64-column blocks of this tile: A0 A1 (rows of the tile), B0 B1 (columns)
      int bc0[4], bx[4], by[4];
      bool bvalid[4];
      int nvalid = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int op = e >> 1;
        const int j0 = (op == 0 ? bi : bj) * TILE + (e & 1) * 64;
        bvalid[e] = (j0 < p.dcols) && !(share && op == 1);
        const int pos = j0 / p.c;
        const int ky = pos / p.kw, kx = pos - ky * p.kw;
        bc0[e] = j0 - pos * p.c;
        bx[e] = kx * p.dil_w - p.pad_w;
        by[e] = ky * p.dil_h - p.pad_h;
        nvalid += bvalid[e] ? 1 : 0;
      }
      const uint32_t box_bytes = (uint32_t)g.kstage * 128u;
      const uint64_t tmap_ptr = reinterpret_cast<uint64_t>(&tmap);
      bool ok = !g_inject_stall;       // stalled: nothing is ever loaded and the consumers' waits run out
      for (int s = 0; s < nstages && ok; ++s) {
        const int slot = s % STAGES;
        if (s >= STAGES) ok = mbar_wait(empty_bar(slot), ((s / STAGES) - 1) & 1, status, 4);
        if (!ok) break;
        const int sg = s_begin + s;
        const int n0 = (sg / g.ystages) * g.bn;
        const int oy0 = (sg % g.ystages) * g.bh;
        const uint32_t fb = full_bar(slot);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb), "r"(box_bytes * nvalid) : "memory");
        const uint32_t sb = smem0 + slot * STAGE_BYTES;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (!bvalid[e]) continue;
          const uint32_t dst = sb + (e >> 1) * 2 * BLOCK_BYTES_MAX + (e & 1) * blk_bytes;
          asm volatile(
              "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
              ::"r"(dst), "l"(tmap_ptr), "r"(bc0[e]), "r"(bx[e]), "r"(oy0 * p.stride_h + by[e]), "r"(n0), "r"(fb)
              : "memory");
        }
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
  if (fused)
    fin::finish_tile<THREADS>(p, blockIdx.x, bi, bj, split,
                              reinterpret_cast<float*>(smem_raw + (smem0 - smem_u32(smem_raw))), &fin_flag, tid);
}

// ---- CTA-pair variant ----------------------------------------------------------------------------
// Two CTAs of a cluster compute one 256x256 block of the result with tcgen05.mma.cta_group::2:
// CTA r of the pair stages columns [256I + 128r, +128) of the A side and columns [256J + 128r, +128)
// of the B side (its half of N) - the same four 64-column boxes per stage as the single-CTA
// kernel - but each byte in shared memory now feeds twice the tensor work (M = 256, N = 256), which
// is what the single-CTA kernel, bound by the L2 -> shared-memory feed, lacks.  The leader CTA
// (rank 0) issues the MMAs; all TMA loads of both CTAs complete on the leader's "full" barrier;
// tcgen05.commit with a cluster multicast releases the stage ("empty") and publishes the
// accumulator ("accfull") in both CTAs; every accumulate warp of both CTAs arrives on the leader's
// "accempty".  Each CTA keeps rows [128r, +128) x 256 columns of the block in its own TMEM
// (2 x 256 columns) and writes them as two ordinary 128x128 partial tiles, so the finishing
// kernels are shared with the other factor kernels.  No multicast loads, no peer-GPU memory.
constexpr uint32_t TMEM_COLS2 = 512;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
      "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at the same shared-memory offset in both CTAs of the pair once all MMAs
// issued so far have completed
__device__ __forceinline__ void umma2_commit_both(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask) : "memory");
}
// instruction descriptor: D fp32, A/B 16-bit format `fmt`, both MN-major, M = 256 (pair), N = 256
__device__ __forceinline__ uint32_t instr_desc_pair(uint32_t fmt) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(256 >> 3) << 17) |
         ((uint32_t)(256 >> 4) << 24);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
factor_tma_pair_kernel(const FactorParams p, const Geom g, const __grid_constant__ CUtensorMap tmap) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int fin_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool fused = p.tickets != nullptr;
  const uint32_t rank = cluster_ctarank();
  int bI, bJ;
  tri_decode(blockIdx.x >> 1, bI, bJ);        // 256-wide block row / column of the pair
  const bool share = (bI == bJ);
  const int split = blockIdx.y;
  const int s_begin = split * g.stages_per_split;
  const int s_end = min(g.total_stages, s_begin + g.stages_per_split);
  const int nstages = max(0, s_end - s_begin);
  const int flush = g.flush;
  const int nchunks = ceil_div(nstages, flush);
  int* status = p.status;

  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto accfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto accempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // two arrivals per stage: the leader's (with the byte count of both CTAs) and the peer's, so
      // that a peer with nothing to load (its columns lie past the matrix edge) stays in step with
      // the stages instead of being lapped by its "empty" barrier
      mbar_init(full_bar(s), 2);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accfull_bar(b), 1);
      mbar_init(accempty_bar(b), 2 * EPI_WARPS);   // the accumulate warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const uint32_t blk_bytes = (uint32_t)g.kpad * 128u;
  // valid 64-column blocks of a CTA of rank rr: A0 A1 (rows of the block), B0 B1 (its half of the columns)
  auto block_col = [&](uint32_t rr, int e) { return ((e >> 1) == 0 ? bI : bJ) * 256 + (int)rr * TILE + (e & 1) * 64; };
  auto block_valid = [&](uint32_t rr, int e) { return block_col(rr, e) < p.dcols && !(share && (e >> 1) == 1); };
  // zero what TMA never writes (see the single-CTA kernel): padding rows and blocks past the edge
  for (int sb = 0; sb < 4 * STAGES; ++sb) {
    const int e = sb & 3, op = e >> 1;
    if (share && op == 1) continue;
    const uint32_t base = smem0 + (sb >> 2) * STAGE_BYTES + op * 2 * BLOCK_BYTES_MAX + (e & 1) * blk_bytes;
    const uint32_t lo = block_valid(rank, e) ? (uint32_t)g.kstage * 128u : 0u;
    for (uint32_t o = lo + tid * 16u; o < blk_bytes; o += THREADS * 16u)
      asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(base + o), "r"(0u) : "memory");
  }
  fence_async_smem();
  if (warp == MMA_WARP) tmem_alloc2(smem_u32(&tmem_base_slot), TMEM_COLS2);
  tc_fence_before();
  cluster_sync_all();          // barriers of both CTAs are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp < EPI_WARPS) {
    // ------------------------------------------------------------------ accumulate warps
    // warp = 4*half + q: TMEM lanes 32q.., columns [128*half, +128) = one 128x128 tile of the result
    const int q = warp & 3, half = warp >> 2;
    float acc[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) acc[i] = 0.f;
    const uint32_t leader_accempty0 = map_to_cta(accempty_bar(0), 0u);
    for (int c = 0; c < nchunks; ++c) {
      const int b = c & 1;
      if (!mbar_wait(accfull_bar(b), (c >> 1) & 1, status, 33)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * 256 + half * 128);
#pragma unroll
      for (int part = 0; part < 4; ++part) {
        uint32_t v[32];
        tmem_ld32(taddr + part * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[part * 32 + i] += __uint_as_float(v[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_accempty0 + 8u * b);
    }
    const int ti = 2 * bI + (int)rank, tj = 2 * bJ + half;
    const int nb = ceil_div(p.d, TILE);
    if (ti < nb && tj <= ti) {
      if (fused && p.splits == 1) {
        // one staging tile per half, behind each other in the (now free) operand buffers
        float* ct = reinterpret_cast<float*>(smem_raw + (smem0 - smem_u32(smem_raw))) + half * (TILE * fin::CT_LD) +
                    (q * 32 + lane) * fin::CT_LD;
#pragma unroll
        for (int i = 0; i < 128; ++i) ct[i] = acc[i];
      } else {
        float* dst = p.partial + ((int64_t)(ti * (ti + 1) / 2 + tj) * p.splits + split) * (TILE * TILE) +
                     (q * 32 + lane) * TILE;
#pragma unroll
        for (int i = 0; i < 128; i += 4)
          *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
        if (fused) __threadfence();
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = instr_desc_pair(g.fmt);
      const int nk = g.kpad / 16;
      bool ok = true;
      for (int s = 0; s < nstages && ok; ++s) {
        const int slot = s % STAGES, c = s / flush, b = c & 1;
        const bool first_of_chunk = (s % flush) == 0;
        if (first_of_chunk && c >= 2) ok = mbar_wait(accempty_bar(b), ((c >> 1) - 1) & 1, status, 32);
        if (!ok) break;
        ok = mbar_wait(full_bar(slot), (s / STAGES) & 1, status, 31);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a0 = smem0 + slot * STAGE_BYTES;
        const uint32_t b0 = share ? a0 : a0 + 2 * BLOCK_BYTES_MAX;
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * 256);
        for (int ks = 0; ks < nk; ++ks) {
          const uint64_t ad = smem_desc_sw128(a0 + ks * 2048u, blk_bytes, 1024u);
          const uint64_t bd = smem_desc_sw128(b0 + ks * 2048u, blk_bytes, 1024u);
          umma2_f16(d_tmem, ad, bd, idesc, (first_of_chunk && ks == 0) ? 0u : 1u);
        }
        umma2_commit_both(empty_bar(slot));
        if ((s % flush) == flush - 1 || s == nstages - 1) umma2_commit_both(accfull_bar(b));
      }
    }
  } else if (warp == PROD_WARP) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int bc0[4], bx[4], by[4];
      bool bvalid[4];
      int nvalid_pair = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j0 = block_col(rank, e);
        bvalid[e] = block_valid(rank, e);
        const int pos = j0 / p.c;
        const int ky = pos / p.kw, kx = pos - ky * p.kw;
        bc0[e] = j0 - pos * p.c;
        bx[e] = kx * p.dil_w - p.pad_w;
        by[e] = ky * p.dil_h - p.pad_h;
        nvalid_pair += (block_valid(0u, e) ? 1 : 0) + (block_valid(1u, e) ? 1 : 0);
      }
      const uint32_t box_bytes = (uint32_t)g.kstage * 128u;
      const uint64_t tmap_ptr = reinterpret_cast<uint64_t>(&tmap);
      bool ok = !g_inject_stall;
      for (int s = 0; s < nstages && ok; ++s) {
        const int slot = s % STAGES;
        if (s >= STAGES) ok = mbar_wait(empty_bar(slot), ((s / STAGES) - 1) & 1, status, 34);
        if (!ok) break;
        const int sg = s_begin + s;
        const int n0 = (sg / g.ystages) * g.bn;
        const int oy0 = (sg % g.ystages) * g.bh;
        // the loads of both CTAs complete on the leader's barrier; the leader announces the bytes
        const uint32_t fb = map_to_cta(full_bar(slot), 0u);
        if (rank == 0)
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full_bar(slot)), "r"(box_bytes * nvalid_pair) : "memory");
        const uint32_t sb = smem0 + slot * STAGE_BYTES;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (!bvalid[e]) continue;
          const uint32_t dst = sb + (e >> 1) * 2 * BLOCK_BYTES_MAX + (e & 1) * blk_bytes;
          asm volatile(
              "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
              ::"r"(dst), "l"(tmap_ptr), "r"(bc0[e]), "r"(bx[e]), "r"(oy0 * p.stride_h + by[e]), "r"(n0), "r"(fb)
              : "memory");
        }
        if (rank != 0) mbar_arrive_cluster(fb);
      }
    }
  }
  tc_fence_before();
  cluster_sync_all();          // neither CTA leaves while its peer may still read its shared memory
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS2);
  }
  if (fused) {
    // this CTA's two tiles of the block: rows [128*rank, +128) x columns [128*h, +128), h = 0, 1
    const int nb = ceil_div(p.d, TILE);
    const int ti = 2 * bI + (int)rank;
    float* ct0 = reinterpret_cast<float*>(smem_raw + (smem0 - smem_u32(smem_raw)));
    for (int h = 0; h < 2; ++h) {
      const int tj = 2 * bJ + h;
      if (ti < nb && tj <= ti)
        fin::finish_tile<THREADS>(p, ti * (ti + 1) / 2 + tj, ti, tj, split,
                                  ct0 + (p.splits == 1 ? h * (TILE * fin::CT_LD) : 0), &fin_flag, tid);
      __syncthreads();
    }
  }
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

static int round16(int v) { return (v + 15) / 16 * 16; }

// Output-pixel box of one stage: full output rows, as many as fit in 128 pixels, or whole images
// when an image has at most 128 pixels; chosen to minimise zero-padded rows.
static bool choose_box(const FactorParams& p, Geom& g) {
  const int wo = p.wo, ho = p.ho, hw = wo * ho;
  if (wo > 128 || wo * p.stride_w > 256) return false;
  g.bw = wo;
  if (hw <= KPAD_MAX) {
    int best = 1;
    double best_cost = 1e30;
    for (int bn = 1; bn * hw <= KPAD_MAX && bn <= 256; ++bn) {
      const double cost = (double)round16(bn * hw) / bn;
      if (cost <= best_cost + 1e-9) { best_cost = cost; best = bn; }   // ties: the larger box
    }
    g.bn = best; g.bh = ho; g.ystages = 1;
  } else {
    int best = 1;
    double best_cost = 1e30;
    for (int bh = 1; bh * wo <= KPAD_MAX && bh <= ho; ++bh) {
      if (bh * p.stride_h > 256) break;
      // the box must not reach past the last output row: with a kernel offset or padding the
      // input rows of such phantom pixels can lie inside the image and would be counted
      if (ho % bh != 0) continue;
      const double cost = (double)ceil_div(ho, bh) * round16(bh * wo);
      if (cost <= best_cost + 1e-9) { best_cost = cost; best = bh; }   // ties: the larger box
    }
    g.bn = 1; g.bh = best; g.ystages = ceil_div(ho, best);
  }
  if (g.bh * p.stride_h > 256) return false;
  g.kstage = g.bw * g.bh * g.bn;
  g.kpad = round16(g.kstage);
  g.total_stages = ceil_div(p.n, g.bn) * g.ystages;
  return g.kpad <= KPAD_MAX;
}

// Splits of the stage range per tile.  More splits fill the 148 SMs more evenly but every split
// writes a 64 KB partial tile that the finishing kernel reads back.  Cost model (microseconds,
// constants fitted to measurements on B200): a CTA runs its stages at ~0.75 us each plus ~4 us
// of prologue / drain, CTAs run in waves of 148, and a partial tile costs ~0.03 us of the
// whole GPU's memory system (written once, read once).
static void choose_splits(int total_stages, int tiles, int& splits, int& stages_per_split) {
  const int kSMs = 148;
  const int most = std::max(1, total_stages / 4);
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 148 && s <= most; ++s) {
    const int sps = ceil_div(total_stages, s);
    const int real = ceil_div(total_stages, sps);
    const int64_t ctas = (int64_t)tiles * real;
    const double cost = (double)ceil_div64(ctas, kSMs) * (sps * 0.75 + 4.0) + (double)ctas * 0.03;
    if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
  }
  stages_per_split = ceil_div(total_stages, best);
  splits = ceil_div(total_stages, stages_per_split);
}

}  // namespace tma

// Tensor map of a row-major fp32 matrix [rows][cols] with leading dimension ld (elements), for
// boxes of 32 columns x 128 rows landing in the SWIZZLE_128B layout; out-of-range reads give zero.
// `out` must hold 128 bytes.  False if the driver entry point is missing or the encode fails.
bool tma_encode_f32_rows(void* out, const float* base, int64_t rows, int64_t cols, int64_t ld) {
  auto fn = tma::encode_fn();
  if (!fn) return false;
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstr[1] = {(cuuint64_t)ld * 4};
  const cuuint32_t box[2] = {32u, 128u};
  const cuuint32_t estr[2] = {1u, 1u};
  return fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), gdim,
            gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ---- fp32 inputs: TMA-fed 3xTF32 ---------------------------------------------------------------
// Same idea for fp32 channels-contiguous activations whose channel count is a multiple of 32: a
// box {32 channels, bw, bh, bn} of the NHWC tensor is 128-byte rows in shared memory, i.e. the
// MN-major operand of a kind::tf32 MMA in its 32-byte-chunk swizzle (32 columns per block, four blocks per 128-wide
// operand).  A stage is at most 32 pixels: 2 x 4 blocks x 4 KB = 32 KB land in a ring of five raw
// stages; eight warps then split the landed stage in place (hi = rna_tf32(x) overwrites x, lo = x - hi
// goes to a two-stage ring) and the MMA warp issues lo*hi + hi*lo + hi*hi per 8-pixel slice.  The
// accumulator is drained into fp32 registers every two stages.  Partial tiles and the finishing
// kernels are those of the other factor kernels.
namespace tmaf {

using namespace tc;

constexpr int TILE = 128;
constexpr int EPI_WARPS = 8, MMA_WARP = 8, SPLIT_WARPS = 8;
constexpr int THREADS = 32 * (EPI_WARPS + 1 + SPLIT_WARPS);
constexpr int RAW_SLOTS = 5, LO_SLOTS = 2, PREFETCH = 3, FLUSH = 2;
constexpr int KPAD_MAX = 32;
constexpr uint32_t BLOCK_BYTES_MAX = KPAD_MAX * 128;          // one 32-column block of one stage
constexpr uint32_t OPERAND_BYTES = 4 * BLOCK_BYTES_MAX;       // 128 columns
constexpr uint32_t STAGE_BYTES = 2 * OPERAND_BYTES;           // A and B
constexpr uint32_t TMEM_COLS = 256;

struct GeomF {
  int bw, bh, bn;            // box in output pixels
  int xchunks, ychunks;      // boxes per output row / per image column
  int kstage, kpad;          // pixels per stage, padded to a multiple of 8
  int total_stages, stages_per_split;
};

// MN-major 32-bit operands have one shared-memory layout: 128-byte rows swizzled in 32-byte chunks
// (chunk index XOR (row & 3)), atoms of 4 rows.  LBO = stride between 32-column blocks, SBO = stride
// between groups of 4 rows (512 bytes here), descriptor version 1, layout type 1.
__device__ __forceinline__ uint64_t desc_mn_sw128(uint32_t saddr, uint32_t lbo_bytes) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) |
         ((uint64_t)(512u >> 4) << 32) | (1ull << 46) | (1ull << 61);
}

__global__ void __launch_bounds__(THREADS, 1)
factor_tma_f32_kernel(const FactorParams p, const GeomF g, const __grid_constant__ CUtensorMap tmap) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * RAW_SLOTS + 2 * LO_SLOTS + 4];
  __shared__ uint32_t tmem_base_slot;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int bi, bj;
  tri_decode(blockIdx.x, bi, bj);
  const bool share = (bi == bj);
  const int split = blockIdx.y;
  const int s_begin = split * g.stages_per_split;
  const int s_end = min(g.total_stages, s_begin + g.stages_per_split);
  const int nstages = max(0, s_end - s_begin);
  const int nchunks = ceil_div(nstages, FLUSH);
  int* status = p.status;

  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t lo0 = smem0 + RAW_SLOTS * STAGE_BYTES;
  const uint32_t bar0 = smem_u32(bars);
  auto rawfree_bar = [&](int s) { return bar0 + 8u * s; };
  auto rawfull_bar = [&](int s) { return bar0 + 8u * (RAW_SLOTS + s); };
  auto full_bar = [&](int s) { return bar0 + 8u * (2 * RAW_SLOTS + s); };
  auto lofree_bar = [&](int s) { return bar0 + 8u * (2 * RAW_SLOTS + LO_SLOTS + s); };
  const uint32_t accfull0 = bar0 + 8u * (2 * RAW_SLOTS + 2 * LO_SLOTS), accempty0 = accfull0 + 16u;

  if (tid == 0) {
    for (int s = 0; s < RAW_SLOTS; ++s) {
      mbar_init(rawfree_bar(s), 1);
      mbar_init(rawfull_bar(s), 1);
    }
    for (int s = 0; s < LO_SLOTS; ++s) {
      mbar_init(full_bar(s), SPLIT_WARPS);
      mbar_init(lofree_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accfull0 + 8u * b, 1);
      mbar_init(accempty0 + 8u * b, EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // zero both rings once: padding pixels and blocks past the matrix edge are never written by TMA
  for (uint32_t o = tid * 16u; o < (RAW_SLOTS + LO_SLOTS) * STAGE_BYTES; o += THREADS * 16u)
    asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(smem0 + o), "r"(0u) : "memory");
  fence_async_smem();
  if (warp == MMA_WARP) tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t blk_bytes = (uint32_t)g.kpad * 128u;

  if (warp < EPI_WARPS) {
    // ------------------------------------------------------------------ accumulate warps
    const int q = warp & 3, half = warp >> 2;
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    for (int c = 0; c < nchunks; ++c) {
      const int b = c & 1;
      if (!mbar_wait(accfull0 + 8u * b, (c >> 1) & 1, status, 53)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * TILE + half * 64);
      uint32_t v0[32], v1[32];
      tmem_ld32(taddr, v0);
      tmem_ld32(taddr + 32, v1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(accempty0 + 8u * b);
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
      const uint32_t idesc = instr_desc(2u, 1u);     // tf32, MN-major operands
      const int nk = g.kpad / 8;
      bool ok = true;
      for (int s = 0; s < nstages && ok; ++s) {
        const int rs = s % RAW_SLOTS, ls = s % LO_SLOTS, c = s / FLUSH, b = c & 1;
        const bool first_of_chunk = (s % FLUSH) == 0;
        if (first_of_chunk && c >= 2) ok = mbar_wait(accempty0 + 8u * b, ((c >> 1) - 1) & 1, status, 52);
        if (!ok) break;
        ok = mbar_wait(full_bar(ls), (s / LO_SLOTS) & 1, status, 51);
        if (!ok) break;
        tc_fence_after();
        const uint32_t ah = smem0 + rs * STAGE_BYTES, al = lo0 + ls * STAGE_BYTES;
        const uint32_t bh = share ? ah : ah + OPERAND_BYTES, bl = share ? al : al + OPERAND_BYTES;
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * TILE);
        for (int ks = 0; ks < nk; ++ks) {
          // one slice = 8 pixels = one 1024-byte swizzle atom; the next 32-column block of the
          // operand starts blk_bytes further on
          const uint64_t adh = desc_mn_sw128(ah + ks * 1024u, blk_bytes), adl = desc_mn_sw128(al + ks * 1024u, blk_bytes);
          const uint64_t bdh = desc_mn_sw128(bh + ks * 1024u, blk_bytes), bdl = desc_mn_sw128(bl + ks * 1024u, blk_bytes);
          umma<true>(d_tmem, adl, bdh, idesc, (first_of_chunk && ks == 0) ? 0u : 1u);
          umma<true>(d_tmem, adh, bdl, idesc, 1u);
          umma<true>(d_tmem, adh, bdh, idesc, 1u);
        }
        umma_commit(rawfree_bar(rs));
        umma_commit(lofree_bar(ls));
        if ((s % FLUSH) == FLUSH - 1 || s == nstages - 1) umma_commit(accfull0 + 8u * b);
      }
    }
  } else {
    // ------------------------------------------------------------------ producer thread + split warps
    const int lt = tid - 32 * (MMA_WARP + 1);
    int bc0[8], bx[8], by[8];
    bool bvalid[8];
    int nvalid = 0;
    if (lt == 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int op = e >> 2;
        const int j0 = (op == 0 ? bi : bj) * TILE + (e & 3) * 32;
        bvalid[e] = (j0 < p.dcols) && !(share && op == 1);
        const int pos = j0 / p.c;
        const int ky = pos / p.kw, kx = pos - ky * p.kw;
        bc0[e] = j0 - pos * p.c;
        bx[e] = kx * p.dil_w - p.pad_w;
        by[e] = ky * p.dil_h - p.pad_h;
        nvalid += bvalid[e] ? 1 : 0;
      }
    }
    const uint32_t box_bytes = (uint32_t)g.kstage * 128u;
    const uint64_t tmap_ptr = reinterpret_cast<uint64_t>(&tmap);
    bool ok = true;
    auto issue = [&](int s) {
      const int rs = s % RAW_SLOTS;
      if (s >= RAW_SLOTS && !mbar_wait(rawfree_bar(rs), ((s / RAW_SLOTS) - 1) & 1, status, 54)) { ok = false; return; }
      const int sg = s_begin + s;
      const int per_img = g.xchunks * g.ychunks;
      const int n0 = (sg / per_img) * g.bn;
      const int rem = sg % per_img;
      const int oy0 = (rem / g.xchunks) * g.bh, ox0 = (rem % g.xchunks) * g.bw;
      const uint32_t fb = rawfull_bar(rs);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb), "r"(box_bytes * nvalid) : "memory");
      const uint32_t sb = smem0 + rs * STAGE_BYTES;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (!bvalid[e]) continue;
        const uint32_t dst = sb + (e >> 2) * OPERAND_BYTES + (e & 3) * blk_bytes;
        asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
            ::"r"(dst), "l"(tmap_ptr), "r"(bc0[e]), "r"(ox0 * p.stride_w + bx[e]), "r"(oy0 * p.stride_h + by[e]), "r"(n0), "r"(fb)
            : "memory");
      }
    };
    if (lt == 0)
      for (int s = 0; s < PREFETCH && s < nstages; ++s) issue(s);
    // the operand bytes of a stage that exist: A always, B unless the tile is on the diagonal
    const uint32_t split_bytes = share ? OPERAND_BYTES : STAGE_BYTES;
    for (int s = 0; s < nstages; ++s) {
      if (lt == 0 && s + PREFETCH < nstages) issue(s + PREFETCH);
      const int rs = s % RAW_SLOTS, ls = s % LO_SLOTS;
      if (!mbar_wait(rawfull_bar(rs), (s / RAW_SLOTS) & 1, status, 56)) break;
      if (s >= LO_SLOTS && !mbar_wait(lofree_bar(ls), ((s / LO_SLOTS) - 1) & 1, status, 55)) break;
      const uint32_t hi = smem0 + rs * STAGE_BYTES, lo = lo0 + ls * STAGE_BYTES;
      for (uint32_t off = (uint32_t)lt * 16u; off < split_bytes; off += 32u * SPLIT_WARPS * 16u) {
        float4 v;
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(hi + off) : "memory");
        const uint32_t h0 = rna_tf32(v.x), h1 = rna_tf32(v.y), h2 = rna_tf32(v.z), h3 = rna_tf32(v.w);
        const uint32_t l0 = __float_as_uint(v.x - __uint_as_float(h0)), l1 = __float_as_uint(v.y - __uint_as_float(h1));
        const uint32_t l2 = __float_as_uint(v.z - __uint_as_float(h2)), l3 = __float_as_uint(v.w - __uint_as_float(h3));
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(hi + off), "r"(h0), "r"(h1), "r"(h2), "r"(h3) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(lo + off), "r"(l0), "r"(l1), "r"(l2), "r"(l3) : "memory");
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar(ls));
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

static int round8(int v) { return (v + 7) / 8 * 8; }

// Output-pixel rectangle of one stage (at most 32 pixels): bw divides the output width, bh the
// height; whole images are grouped when an image has at most 32 pixels.  Chosen to minimise the
// padded pixel count, ties to the larger box.
static bool choose_box(const FactorParams& p, GeomF& g) {
  const int wo = p.wo, ho = p.ho, hw = wo * ho;
  double best_cost = 1e30;
  bool found = false;
  auto consider = [&](int bw, int bh, int bn) {
    if (bw * p.stride_w > 256 || bh * p.stride_h > 256 || bn > 256) return;
    const int ks = bw * bh * bn;
    if (ks > KPAD_MAX) return;
    const double stages = (double)(wo / bw) * (ho / bh) * ceil_div(p.n, bn);
    const double cost = stages * round8(ks) + stages * 4.0;     // padded pixels + a per-stage overhead
    if (cost < best_cost - 1e-9 || (cost < best_cost + 1e-9 && ks > g.kstage)) {
      best_cost = cost; found = true;
      g.bw = bw; g.bh = bh; g.bn = bn; g.kstage = ks;
    }
  };
  g.kstage = 0;
  if (hw <= KPAD_MAX)
    for (int bn = 1; bn * hw <= KPAD_MAX; ++bn) consider(wo, ho, bn);
  for (int bw = 1; bw <= wo && bw <= KPAD_MAX; ++bw) {
    if (wo % bw != 0) continue;
    for (int bh = 1; bh <= ho && bw * bh <= KPAD_MAX; ++bh)
      if (ho % bh == 0) consider(bw, bh, 1);
  }
  if (!found) return false;
  g.xchunks = wo / g.bw;
  g.ychunks = ho / g.bh;
  g.kpad = round8(g.kstage);
  g.total_stages = ceil_div(p.n, g.bn) * g.xchunks * g.ychunks;
  return true;
}

}  // namespace tmaf

int factor_tma_set_wait_controls(long long cycles, int stall) { return tc::set_wait_controls(cycles, stall); }

static int g_tma_f32 = 0;     // fp32 inputs may use the TMA-fed 3xTF32 kernel
void factor_tma_set_f32(int on) { g_tma_f32 = on != 0; }

static bool factor_tma_f32_supported(const FactorParams& p) {
  if (!g_tma_f32) return false;
  if (p.sc != 1 || p.c % 32 != 0 || p.weight != nullptr || p.d != p.dcols) return false;
  if ((reinterpret_cast<uintptr_t>(p.x) & 15) != 0) return false;
  if (p.stride_h > 8 || p.stride_w > 8) return false;
  if ((p.sn * 4) % 16 != 0 || (p.h > 1 && (p.sh * 4) % 16 != 0) || (p.w > 1 && (p.sw * 4) % 16 != 0)) return false;
  tmaf::GeomF g;
  if (!tmaf::choose_box(p, g)) return false;
  return tma::encode_fn() != nullptr;
}

static int factor_tma_f32_launch(FactorParams p, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  using namespace tmaf;
  GeomF g{};
  SSO_CHECK_ARG(choose_box(p, g), "factor (tma, fp32): unsupported geometry");
  const int nb = ceil_div(p.d, 128);
  const int tiles = nb * (nb + 1) / 2;
  tma::choose_splits(g.total_stages, tiles, p.splits, g.stages_per_split);
  const size_t hdr = factor_header_bytes(tiles);
  SSO_CHECK_ARG(workspace != nullptr && workspace_bytes >= hdr + (size_t)tiles * 65536,
                "factor workspace too small for the tensor-core path");
  const int max_splits = (int)((workspace_bytes - hdr) / ((size_t)tiles * 65536));
  if (p.splits > max_splits) {
    g.stages_per_split = ceil_div(g.total_stages, max_splits);
    p.splits = ceil_div(g.total_stages, g.stages_per_split);
  }
  p.rows_per_split = 0;
  p.status = reinterpret_cast<int*>(workspace);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + hdr);
  p.tickets = nullptr;
  SSO_CUDA_OK(cudaMemsetAsync(p.status, 0, sizeof(int), st));
  p.perm_c = (p.kh * p.kw > 1) ? p.c : 0;
  p.perm_kk = p.kh * p.kw;

  CUtensorMap tmap;
  const cuuint64_t gdim[4] = {(cuuint64_t)p.c, (cuuint64_t)p.w, (cuuint64_t)p.h, (cuuint64_t)p.n};
  const cuuint64_t sw_b = (cuuint64_t)(p.w > 1 ? p.sw : p.c) * 4, sh_b = (cuuint64_t)(p.h > 1 ? p.sh : p.sn) * 4;
  const cuuint64_t gstr[3] = {sw_b, sh_b, (cuuint64_t)p.sn * 4};
  const cuuint32_t box[4] = {32u, (cuuint32_t)(g.bw * p.stride_w), (cuuint32_t)(g.bh * p.stride_h), (cuuint32_t)g.bn};
  const cuuint32_t estr[4] = {1u, (cuuint32_t)p.stride_w, (cuuint32_t)p.stride_h, 1u};
  const CUresult cr = tma::encode_fn()(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(p.x), gdim, gstr, box,
                                       estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(-5, "cuTensorMapEncodeTiled failed with code %d", (int)cr);

  const size_t smem = (size_t)(RAW_SLOTS + LO_SLOTS) * STAGE_BYTES + 1024;
  SSO_ENSURE_SMEM(factor_tma_f32_kernel, (int)smem);
  factor_tma_f32_kernel<<<dim3(tiles, p.splits), THREADS, smem, st>>>(p, g, tmap);
  SSO_LAUNCH_OK("factor_tma_f32_kernel");
  return factor_tc_run_reduce(p, tiles, st);
}

bool factor_tma_supported(const FactorParams& p, int dtype) {
  if (dtype == SSO_F32) return factor_tma_f32_supported(p);
  if (dtype != SSO_BF16 && dtype != SSO_F16) return false;
  if (p.sc != 1 || p.c % 64 != 0 || p.weight != nullptr || p.d != p.dcols) return false;
  if ((reinterpret_cast<uintptr_t>(p.x) & 15) != 0) return false;
  if (p.stride_h > 8 || p.stride_w > 8) return false;
  if ((p.sn * 2) % 16 != 0 || (p.h > 1 && (p.sh * 2) % 16 != 0) || (p.w > 1 && (p.sw * 2) % 16 != 0)) return false;
  tma::Geom g;
  if (!tma::choose_box(p, g)) return false;
  return tma::encode_fn() != nullptr;
}

static int g_fused_finish = 1;  // unpermuted factors are finished by the producing kernel
void factor_tma_set_fused_finish(int on) { g_fused_finish = on != 0; }

static int g_pair_min_d = 512;  // factors at least this wide use the CTA-pair kernel; 0 = never
void factor_tma_set_pair_min_d(int d) { g_pair_min_d = d < 0 ? 0 : d; }

int factor_tma_launch(FactorParams p, int dtype, void* workspace, size_t workspace_bytes, int flush,
                      cudaStream_t st) {
  if (dtype == SSO_F32) return factor_tma_f32_launch(p, workspace, workspace_bytes, st);
  using namespace tma;
  Geom g{};
  SSO_CHECK_ARG(choose_box(p, g), "factor (tma): unsupported geometry");
  const int nb = ceil_div(p.d, 128);
  const int tiles = nb * (nb + 1) / 2;
  const bool pair = g_pair_min_d > 0 && p.d >= g_pair_min_d;
  const int nb2 = ceil_div(p.d, 256);
  const int pair_blocks = nb2 * (nb2 + 1) / 2;
  choose_splits(g.total_stages, pair ? 2 * pair_blocks : tiles, p.splits, g.stages_per_split);
  // fit the partial tiles into the scratch the caller sized with sso_factor_workspace_bytes
  const size_t hdr = factor_header_bytes(tiles);
  SSO_CHECK_ARG(workspace != nullptr && workspace_bytes >= hdr + (size_t)tiles * 65536,
                "factor workspace too small for the tensor-core path");
  const int max_splits = (int)((workspace_bytes - hdr) / ((size_t)tiles * 65536));
  if (p.splits > max_splits) {
    g.stages_per_split = ceil_div(g.total_stages, max_splits);
    p.splits = ceil_div(g.total_stages, g.stages_per_split);
  }
  p.rows_per_split = 0;
  g.flush = flush > 0 ? flush : 4;
  g.fmt = (dtype == SSO_BF16) ? 1u : 0u;
  p.status = reinterpret_cast<int*>(workspace);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + hdr);
  p.perm_c = (p.kh * p.kw > 1) ? p.c : 0;
  p.perm_kk = p.kh * p.kw;
  // columns in their public order already: the last CTA of every tile finishes it (factor_finish.cuh)
  const bool fused = g_fused_finish && p.perm_c == 0 && p.splits <= 4;
  p.tickets = fused ? reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + 256) : nullptr;
  p.ticket_tiles = tiles;
  SSO_CUDA_OK(cudaMemsetAsync(p.status, 0, fused ? hdr : sizeof(int), st));

  // NHWC view of the input: dims {C, W, H, N}
  CUtensorMap tmap;
  const cuuint64_t gdim[4] = {(cuuint64_t)p.c, (cuuint64_t)p.w, (cuuint64_t)p.h, (cuuint64_t)p.n};
  const cuuint64_t sw_b = (cuuint64_t)(p.w > 1 ? p.sw : p.c) * 2, sh_b = (cuuint64_t)(p.h > 1 ? p.sh : p.sn) * 2;
  const cuuint64_t gstr[3] = {sw_b, sh_b, (cuuint64_t)p.sn * 2};
  const cuuint32_t box[4] = {64u, (cuuint32_t)(g.bw * p.stride_w), (cuuint32_t)(g.bh * p.stride_h), (cuuint32_t)g.bn};
  const cuuint32_t estr[4] = {1u, (cuuint32_t)p.stride_w, (cuuint32_t)p.stride_h, 1u};
  const CUresult cr = encode_fn()(&tmap, dtype == SSO_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                  4, const_cast<void*>(p.x), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(-5, "cuTensorMapEncodeTiled failed with code %d", (int)cr);

  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
  SSO_ENSURE_SMEM(factor_tma_kernel, (int)smem);
  if (pair) {
    SSO_ENSURE_SMEM(factor_tma_pair_kernel, (int)smem);
    factor_tma_pair_kernel<<<dim3(2 * pair_blocks, p.splits), THREADS, smem, st>>>(p, g, tmap);
    SSO_LAUNCH_OK("factor_tma_pair_kernel");
    return fused ? 0 : factor_tc_run_reduce(p, tiles, st);
  }
  factor_tma_kernel<<<dim3(tiles, p.splits), THREADS, smem, st>>>(p, g, tmap);
  SSO_LAUNCH_OK("factor_tma_kernel");
  return fused ? 0 : factor_tc_run_reduce(p, tiles, st);
}

#include "factor_batch.cuh"

void factor_batch_set_pairs(int pairs) { batch::g_batch_pairs = pairs < 0 ? 0 : pairs; }
size_t factor_batch_scratch_bytes(const FactorParams* ps, const int* dtypes, int n) {
  return batch::factor_batch_scratch_bytes(ps, dtypes, n);
}
int factor_batch_launch(const FactorParams* ps, const int* dtypes, int n, unsigned char* done, void* workspace,
                        size_t workspace_bytes, int flush, cudaStream_t st) {
  return batch::factor_batch_launch(ps, dtypes, n, done, workspace, workspace_bytes, flush, st);
}

}  // namespace sso
