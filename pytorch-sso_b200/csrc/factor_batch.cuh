// Many factor problems in ONE launch (included by factor_tma.cu only, inside namespace sso).
//
// A training step builds ~100 Kronecker factors, most of them far too small to fill the GPU or to
// amortise a launch: per call, launch latency, pipeline fill, accumulator drain and a finishing
// launch cost more than the tensor-core work.  Here the factors that are ready at the same time
// (all A factors once the forward pass is done; all G factors once a backward pass is done) go to
// the device together:
//   * every problem is cut into work items "one 256x256 block of the result x one range of the
//     stages", all of about the same length, ordered longest problem first;
//   * a persistent grid of CTA pairs (one pair per two SMs, tcgen05.mma.cta_group::2 as in
//     factor_tma_pair_kernel) walks the items round-robin: barriers, tensor memory and the TMA / MMA /
//     accumulate pipelines are set up once per CTA and keep running across item boundaries (the
//     accumulate warps write the partial tiles of item k while the MMA warp is already in item k+1);
//   * the problem table - a tensor map and ~25 words per problem - travels in the kernel's parameter
//     space, so a launch captured in a CUDA graph carries it by value;
//   * one second launch finishes all problems (sum of the splits in fixed order, column permutation
//     of k x k convolutions, alpha / beta, mirror).
// No multicast loads, no peer memory; every wait is bounded.
namespace batch {

using namespace tc;
using namespace tma;

constexpr int MAX_PROBLEMS = 96;
constexpr int ITEM_STAGES_MIN = 32, ITEM_STAGES_MAX = 128;   // bounds of a work item's length, in pipeline stages

struct alignas(64) Prob {
  CUtensorMap tmap;          // NHWC view of the input, box {64, bw*stride_w, bh*stride_h, bn}
  float* partial;            // [tile][split][128*128]
  int dcols, d, c, kw;
  int dil_h, dil_w, pad_h, pad_w, stride_h;
  int kstage, kpad, ystages, bn, bh;
  int total_stages, stages_per_split, splits;
  int item0;                 // index of the problem's first work item
  uint32_t fmt;              // 1 bf16, 0 fp16
  int reserved[11];
};
static_assert(sizeof(Prob) == 256, "problem record must stay 256 bytes");

struct Params {
  int nprob, nitems, flush;
  int* status;
  int reserved[11];
  Prob prob[MAX_PROBLEMS];
};
static_assert(sizeof(Params) <= 32000, "kernel parameter space");

struct Item {
  int bI, bJ, split, nstages, s_begin;
  bool share;
};

__device__ __forceinline__ Item decode_item(const Prob& P, int item) {
  Item it;
  const int j = item - P.item0;
  const int blk = j / P.splits;
  it.split = j - blk * P.splits;
  tri_decode(blk, it.bI, it.bJ);
  it.share = (it.bI == it.bJ);
  it.s_begin = it.split * P.stages_per_split;
  it.nstages = max(0, min(P.total_stages, it.s_begin + P.stages_per_split) - it.s_begin);
  return it;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
factor_batch_kernel(const __grid_constant__ Params bp) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_base_slot;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int flush = bp.flush;
  int* status = bp.status;

  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto accfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto accempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // "full" takes two arrivals per stage: the leader's (which also announces the bytes of both
      // CTAs) and one from the peer's producer once it has dealt with the stage.  Without the second
      // a peer that has nothing to load for a stretch of stages (its half of the block lies past the
      // matrix edge) could fall two phases behind its "empty" barrier, whose parity it would then
      // misread; it also orders the peer's zero filling before the MMAs that read its shared memory.
      mbar_init(full_bar(s), 2);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accfull_bar(b), 1);
      mbar_init(accempty_bar(b), 2 * EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc2(smem_u32(&tmem_base_slot), TMEM_COLS2);
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp < EPI_WARPS) {
    // ------------------------------------------------------------------ accumulate warps
    const int q = warp & 3, half = warp >> 2;
    const uint32_t leader_accempty0 = map_to_cta(accempty_bar(0), 0u);
    int gc = 0, pi = 0;
    bool ok = true;
    for (int item = pair; item < bp.nitems && ok; item += npairs) {
      while (pi + 1 < bp.nprob && item >= bp.prob[pi + 1].item0) ++pi;
      const Prob& P = bp.prob[pi];
      const Item it = decode_item(P, item);
      const int nchunks = ceil_div(it.nstages, flush);
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      for (int c = 0; c < nchunks; ++c, ++gc) {
        const int b = gc & 1;
        if (!mbar_wait(accfull_bar(b), (gc >> 1) & 1, status, 63)) { ok = false; break; }
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
      const int ti = 2 * it.bI + (int)rank, tj = 2 * it.bJ + half;
      const int nb = ceil_div(P.d, TILE);
      if (ti < nb && tj <= ti) {
        float* dst = P.partial + ((int64_t)(ti * (ti + 1) / 2 + tj) * P.splits + it.split) * (TILE * TILE) +
                     (q * 32 + lane) * TILE;
#pragma unroll
        for (int i = 0; i < 128; i += 4)
          *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      int gs = 0, gc = 0, pi = 0;
      bool ok = true;
      for (int item = pair; item < bp.nitems && ok; item += npairs) {
        while (pi + 1 < bp.nprob && item >= bp.prob[pi + 1].item0) ++pi;
        const Prob& P = bp.prob[pi];
        const Item it = decode_item(P, item);
        const uint32_t idesc = instr_desc_pair(P.fmt);
        const int nk = P.kpad / 16;
        const uint32_t blk_bytes = (uint32_t)P.kpad * 128u;
        for (int s = 0; s < it.nstages && ok; ++s, ++gs) {
          const int slot = gs % STAGES, b = gc & 1;
          const bool first_of_chunk = (s % flush) == 0;
          if (first_of_chunk && gc >= 2) ok = mbar_wait(accempty_bar(b), ((gc >> 1) - 1) & 1, status, 62);
          if (!ok) break;
          ok = mbar_wait(full_bar(slot), (gs / STAGES) & 1, status, 61);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a0 = smem0 + slot * STAGE_BYTES;
          const uint32_t b0 = it.share ? a0 : a0 + 2 * BLOCK_BYTES_MAX;
          const uint32_t d_tmem = tmem_base + (uint32_t)(b * 256);
          for (int ks = 0; ks < nk; ++ks) {
            const uint64_t ad = smem_desc_sw128(a0 + ks * 2048u, blk_bytes, 1024u);
            const uint64_t bd = smem_desc_sw128(b0 + ks * 2048u, blk_bytes, 1024u);
            umma2_f16(d_tmem, ad, bd, idesc, (first_of_chunk && ks == 0) ? 0u : 1u);
          }
          umma2_commit_both(empty_bar(slot));
          if ((s % flush) == flush - 1 || s == it.nstages - 1) {
            umma2_commit_both(accfull_bar(b));
            ++gc;
          }
        }
      }
    }
  } else if (warp == PROD_WARP) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    // The whole warp walks the items: lane 0 issues the loads, all lanes zero what TMA will not write
    // (padding rows, blocks past the matrix edge) whenever a slot is first used with a new geometry.
    int gs = 0, pi = 0;
    uint32_t sig[STAGES];
#pragma unroll
    for (int s = 0; s < STAGES; ++s) sig[s] = 0xffffffffu;
    bool ok = !g_inject_stall;
    for (int item = pair; item < bp.nitems && ok; item += npairs) {
      while (pi + 1 < bp.nprob && item >= bp.prob[pi + 1].item0) ++pi;
      const Prob& P = bp.prob[pi];
      const Item it = decode_item(P, item);
      const uint32_t blk_bytes = (uint32_t)P.kpad * 128u;
      int bc0[4], bx[4], by[4];
      uint32_t vmask = 0, nvalid_pair = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int base = ((e >> 1) == 0 ? it.bI : it.bJ) * 256 + (e & 1) * 64;
        const bool v0 = base < P.dcols && !(it.share && (e >> 1) == 1);
        const bool v1 = base + TILE < P.dcols && !(it.share && (e >> 1) == 1);
        nvalid_pair += (v0 ? 1u : 0u) + (v1 ? 1u : 0u);
        if (rank == 0 ? v0 : v1) vmask |= 1u << e;
        const int j0 = base + (int)rank * TILE;
        const int pos = j0 / P.c;
        const int ky = pos / P.kw, kx = pos - ky * P.kw;
        bc0[e] = j0 - pos * P.c;
        bx[e] = kx * P.dil_w - P.pad_w;
        by[e] = ky * P.dil_h - P.pad_h;
      }
      // geometry signature of a slot: what has to be zero where
      const uint32_t want = ((uint32_t)P.kstage << 16) | ((uint32_t)P.kpad << 4) | vmask | (it.share ? 0x8000u : 0u);
      const uint32_t box_bytes = (uint32_t)P.kstage * 128u;
      const uint64_t tmap_ptr = reinterpret_cast<uint64_t>(&P.tmap);
      for (int s = 0; s < it.nstages && ok; ++s, ++gs) {
        const int slot = gs % STAGES;
        if (gs >= STAGES) ok = mbar_wait(empty_bar(slot), ((gs / STAGES) - 1) & 1, status, 64);
        if (!ok) break;
        const uint32_t sb = smem0 + slot * STAGE_BYTES;
        if (sig[slot] != want) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (it.share && (e >> 1) == 1) continue;          // never read on a diagonal block
            const uint32_t base = sb + (e >> 1) * 2 * BLOCK_BYTES_MAX + (e & 1) * blk_bytes;
            const uint32_t lo = ((vmask >> e) & 1u) ? box_bytes : 0u;
            for (uint32_t o = lo + lane * 16u; o < blk_bytes; o += 32u * 16u)
              asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(base + o), "r"(0u) : "memory");
          }
          fence_async_smem();
          sig[slot] = want;
        }
        __syncwarp();
        if (lane == 0) {
          const int sg = it.s_begin + s;
          const int n0 = (sg / P.ystages) * P.bn;
          const int oy0 = (sg % P.ystages) * P.bh;
          const uint32_t fb = map_to_cta(full_bar(slot), 0u);
          if (rank == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full_bar(slot)), "r"(box_bytes * nvalid_pair) : "memory");
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (!((vmask >> e) & 1u)) continue;
            const uint32_t dst = sb + (e >> 1) * 2 * BLOCK_BYTES_MAX + (e & 1) * blk_bytes;
            asm volatile(
                "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                ::"r"(dst), "l"(tmap_ptr), "r"(bc0[e]), "r"(bx[e]), "r"(oy0 * P.stride_h + by[e]), "r"(n0), "r"(fb)
                : "memory");
          }
          if (rank != 0) mbar_arrive_cluster(fb);       // the peer's arrival for this stage
        }
        __syncwarp();
      }
    }
  }
  tc_fence_before();
  cluster_sync_all();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS2);
  }
}

// ---- finishing of a whole batch ------------------------------------------------------------------
// Same work as factor_tc_reduce (factor_tc.cu) for every problem of the batch in one launch: a CTA
// produces 32 output rows x one group of output-contiguous columns (8 channels at all kernel
// positions for a k x k convolution, else 32 columns), summing the splits in fixed order, reading the
// partial tiles in 32-byte sectors below the diagonal and mirrored above it.
struct FinProb {
  const float* partial;
  float* out;
  int64_t ldo;
  int d, dcols, splits, perm_c, perm_kk;
  int perm_groups, groups, pitch;
  int block0;                // first CTA of this problem in the launch
  float alpha, beta;
  int reserved[2];
};
static_assert(sizeof(FinProb) == 80, "finishing record");

struct FinParams {
  int nprob;
  int* status;
  FinProb prob[MAX_PROBLEMS];
};

// sum over the splits of one element; `src` points at the element inside the first split's tile
__device__ __forceinline__ float sum_splits(const float* __restrict__ src, int nsplit) {
  constexpr int64_t S = TILE * TILE;
  if (nsplit == 1) return src[0];
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

constexpr int FIN_ROWS = 32, FIN_CB = 8, FIN_W = 32;

__global__ void __launch_bounds__(256) factor_batch_finish_kernel(const __grid_constant__ FinParams fp) {
  extern __shared__ float rs[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int pi = 0;
  {
    int lo = 0, hi = fp.nprob - 1;       // last problem whose block0 <= blockIdx.x
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (fp.prob[mid].block0 <= (int)blockIdx.x) lo = mid; else hi = mid - 1;
    }
    pi = lo;
  }
  // the record is read once into registers: every later use would be another indexed load from
  // parameter space
  const FinProb P = fp.prob[pi];
  const float* __restrict__ partial = P.partial;
  const int local = blockIdx.x - P.block0;
  const int rb = local / P.groups, grp = local - rb * P.groups;
  const int gi0 = rb * FIN_ROWS;
  const int kk = P.perm_kk, C = P.perm_c, d = P.d, pitch = P.pitch, nsplit = P.splits;
  const int64_t tile_floats = (int64_t)nsplit * (TILE * TILE);
  // element (r, c), r >= c, of the lower-triangle partial tiles (first split)
  auto at = [&](int r, int c) {
    const int bi = r >> 7, bj = c >> 7;
    return partial + (int64_t)(bi * (bi + 1) / 2 + bj) * tile_floats + ((r & 127) * TILE + (c & 127));
  };
  int ext0, n_ext;
  if (grp < P.perm_groups) {
    const int c0 = grp * FIN_CB, len = min(FIN_CB, C - c0);
    ext0 = c0 * kk;
    n_ext = len * kk;
    // below / on the diagonal: 4 rows x 8 columns per warp (lanes along the run of 8 channels);
    // above: 32 rows x 1 column per warp, read from the mirrored position (lanes along its columns)
    const int rrA = warp * 4 + (lane >> 3), eA = lane & 7, giA = gi0 + rrA;
    const int rrB = lane, eB = warp, giB = gi0 + rrB;
    const bool okA = eA < len && giA < d, okB = eB < len && giB < d;
    // fixed parts of the two addresses: A walks along its own row, B down a column of the mirrored tile
    const int biA = giA >> 7;
    const float* rowA = partial + (int64_t)(biA * (biA + 1) / 2) * tile_floats + (giA & 127) * TILE;
    const int bjB = giB >> 7, cjB = giB & 127;
    float* dstA = rs + rrA * pitch + eA * kk;
    float* dstB = rs + rrB * pitch + eB * kk;
#pragma unroll 3
    for (int run = 0; run < kk; ++run) {
      const int gjA = run * C + c0 + eA, gjB = run * C + c0 + eB;
      if (okA && gjA <= giA) dstA[run] = sum_splits(rowA + (int64_t)(gjA >> 7) * tile_floats + (gjA & 127), nsplit);
      if (okB && gjB > giB) {
        const int biB = gjB >> 7;
        dstB[run] = sum_splits(partial + (int64_t)(biB * (biB + 1) / 2 + bjB) * tile_floats + ((gjB & 127) * TILE + cjB), nsplit);
      }
    }
  } else {
    ext0 = (P.perm_groups > 0 ? P.dcols : 0) + (grp - P.perm_groups) * FIN_W;
    n_ext = min(FIN_W, d - ext0);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int rrA = warp + 8 * k, giA = gi0 + rrA, gjA = ext0 + lane;
      const int eB = warp + 8 * k, giB = gi0 + lane, gjB = ext0 + eB;
      if (lane < n_ext && giA < d && gjA <= giA) rs[rrA * pitch + lane] = sum_splits(at(giA, gjA), nsplit);
      if (eB < n_ext && giB < d && gjB > giB) rs[lane * pitch + eB] = sum_splits(at(gjB, giB), nsplit);
    }
  }
  __syncthreads();
  const bool bad = fp.status && *fp.status != 0;
  const float alpha = P.alpha, beta = P.beta;
  for (int rr = warp; rr < FIN_ROWS; rr += 8) {
    const int gi = gi0 + rr;
    if (gi >= d) break;
    const int gr = (C > 0 && gi < P.dcols) ? (gi % C) * kk + gi / C : gi;
    float* orow = P.out + (int64_t)gr * P.ldo + ext0;
    for (int e = lane; e < n_ext; e += 32) {
      float v = alpha * rs[rr * pitch + e];
      if (bad) v = __int_as_float(0x7fc00000);
      orow[e] = (beta == 0.f) ? v : fmaf(beta, orow[e], v);
    }
  }
}

// ---- host side -----------------------------------------------------------------------------------
static int g_batch_pairs = 0;        // CTA pairs of the persistent kernel; 0 = one per two SMs

struct Planned {
  FactorParams p;
  Geom g;
  int dtype;
  int tiles, nblk;
  size_t partial_bytes;
};

// true if the problem can ride in a batch (same conditions as the TMA-fed single launch)
static bool batchable(const FactorParams& p, int dtype) {
  return (dtype == SSO_BF16 || dtype == SSO_F16) && factor_tma_supported(p, dtype);
}

// Length of a work item for a set of problems: long enough that the partial tiles (one per item and
// tile, written and read back once) stay a small part of the traffic, short enough that every CTA pair
// gets several items (about six) and the round-robin walk ends evenly.
static int item_stages_for(const FactorParams* ps, const int* dtypes, int n, int pairs) {
  double work = 0;
  for (int i = 0; i < n; ++i) {
    if (!batchable(ps[i], dtypes[i])) continue;
    Geom g;
    choose_box(ps[i], g);
    const int nb2 = ceil_div(ps[i].d, 256);
    work += (double)(nb2 * (nb2 + 1) / 2) * g.total_stages;
  }
  const int want = (int)(work / (6.0 * std::max(1, pairs)));
  return std::max(ITEM_STAGES_MIN, std::min(ITEM_STAGES_MAX, want));
}

static void plan_problem(const FactorParams& p, int dtype, int item_stages, Planned& out) {
  out.p = p;
  out.dtype = dtype;
  choose_box(p, out.g);
  const int nb = ceil_div(p.d, 128), nb2 = ceil_div(p.d, 256);
  out.tiles = nb * (nb + 1) / 2;
  out.nblk = nb2 * (nb2 + 1) / 2;
  int splits = std::max(1, (out.g.total_stages + item_stages - 1) / item_stages);
  splits = std::min(splits, 64);
  out.g.stages_per_split = ceil_div(out.g.total_stages, splits);
  out.p.splits = ceil_div(out.g.total_stages, out.g.stages_per_split);
  out.p.perm_c = (p.kh * p.kw > 1) ? p.c : 0;
  out.p.perm_kk = p.kh * p.kw;
  out.partial_bytes = (size_t)out.tiles * out.p.splits * 65536;
}

size_t factor_batch_scratch_bytes(const FactorParams* ps, const int* dtypes, int n) {
  // sized for the shortest items (most splits), so that it holds for any grid size chosen later
  size_t total = 256;
  for (int i = 0; i < n; ++i) {
    if (!batchable(ps[i], dtypes[i])) continue;
    Planned pl;
    plan_problem(ps[i], dtypes[i], ITEM_STAGES_MIN, pl);
    total += pl.partial_bytes;
  }
  return total;
}

// Launches the batchable problems of ps[0..n) (marks them in done[]); the caller runs the rest one by one.
int factor_batch_launch(const FactorParams* ps, const int* dtypes, int n, unsigned char* done, void* workspace,
                        size_t workspace_bytes, int flush, cudaStream_t st) {
  int sm_count = 148;
  {
    int dev = 0;
    SSO_CUDA_OK(cudaGetDevice(&dev));
    static int cached[64] = {};
    if (dev >= 0 && dev < 64) {
      if (!cached[dev]) SSO_CUDA_OK(cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev));
      sm_count = cached[dev];
    }
  }
  // all SM pairs by default; fewer leave SMs to kernels of other streams that run beside the batch
  int max_pairs = sm_count / 2;
  if (g_batch_pairs > 0) max_pairs = std::min(max_pairs, g_batch_pairs);
  const int item_stages = item_stages_for(ps, dtypes, n, max_pairs);
  std::vector<Planned> plans;
  for (int i = 0; i < n; ++i) {
    done[i] = 0;
    if (!batchable(ps[i], dtypes[i])) continue;
    Planned pl;
    plan_problem(ps[i], dtypes[i], item_stages, pl);
    plans.push_back(pl);
    done[i] = 1;
  }
  if (plans.empty()) return 0;
  // longest items first: the round-robin walk then ends with the short ones
  std::stable_sort(plans.begin(), plans.end(), [](const Planned& a, const Planned& b) {
    return a.g.stages_per_split * a.g.kpad > b.g.stages_per_split * b.g.kpad;
  });
  SSO_CHECK_ARG(workspace != nullptr, "factor batch: no workspace");
  int* status = reinterpret_cast<int*>(workspace);
  SSO_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int), st));
  char* cursor = reinterpret_cast<char*>(workspace) + 256;
  char* const end = reinterpret_cast<char*>(workspace) + workspace_bytes;

  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
  SSO_ENSURE_SMEM(factor_batch_kernel, smem);
  size_t at = 0;
  while (at < plans.size()) {
    const size_t cnt = std::min<size_t>(MAX_PROBLEMS, plans.size() - at);
    static thread_local Params bp;
    static thread_local FinParams fpm;
    bp.nprob = (int)cnt; bp.flush = flush > 0 ? flush : 4; bp.status = status;
    fpm.nprob = (int)cnt; fpm.status = status;
    int items = 0, blocks = 0;
    size_t fin_smem = 0;
    for (size_t k = 0; k < cnt; ++k) {
      Planned& pl = plans[at + k];
      const FactorParams& p = pl.p;
      SSO_CHECK_ARG(cursor + pl.partial_bytes <= end, "factor batch: workspace too small (%zu bytes given)", workspace_bytes);
      Prob& P = bp.prob[k];
      const cuuint64_t gdim[4] = {(cuuint64_t)p.c, (cuuint64_t)p.w, (cuuint64_t)p.h, (cuuint64_t)p.n};
      const cuuint64_t sw_b = (cuuint64_t)(p.w > 1 ? p.sw : p.c) * 2, sh_b = (cuuint64_t)(p.h > 1 ? p.sh : p.sn) * 2;
      const cuuint64_t gstr[3] = {sw_b, sh_b, (cuuint64_t)p.sn * 2};
      const cuuint32_t box[4] = {64u, (cuuint32_t)(pl.g.bw * p.stride_w), (cuuint32_t)(pl.g.bh * p.stride_h), (cuuint32_t)pl.g.bn};
      const cuuint32_t estr[4] = {1u, (cuuint32_t)p.stride_w, (cuuint32_t)p.stride_h, 1u};
      const CUresult cr = encode_fn()(&P.tmap, pl.dtype == SSO_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                      4, const_cast<void*>(p.x), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (cr != CUDA_SUCCESS) return fail(-5, "cuTensorMapEncodeTiled failed with code %d", (int)cr);
      P.partial = reinterpret_cast<float*>(cursor);
      cursor += pl.partial_bytes;
      P.dcols = p.dcols; P.d = p.d; P.c = p.c; P.kw = p.kw;
      P.dil_h = p.dil_h; P.dil_w = p.dil_w; P.pad_h = p.pad_h; P.pad_w = p.pad_w; P.stride_h = p.stride_h;
      P.kstage = pl.g.kstage; P.kpad = pl.g.kpad; P.ystages = pl.g.ystages; P.bn = pl.g.bn; P.bh = pl.g.bh;
      P.total_stages = pl.g.total_stages; P.stages_per_split = pl.g.stages_per_split; P.splits = p.splits;
      P.item0 = items;
      P.fmt = (pl.dtype == SSO_BF16) ? 1u : 0u;
      items += pl.nblk * p.splits;

      FinProb& F = fpm.prob[k];
      F.partial = P.partial; F.out = p.out; F.ldo = p.ldo;
      F.d = p.d; F.dcols = p.dcols; F.splits = p.splits; F.perm_c = p.perm_c; F.perm_kk = p.perm_kk;
      int width = FIN_W;
      F.perm_groups = 0;
      if (p.perm_c > 0) {
        F.perm_groups = ceil_div(p.perm_c, FIN_CB);
        width = std::max(FIN_CB * p.perm_kk, 1);
      }
      const int plain = p.perm_c > 0 ? (p.d > p.dcols ? 1 : 0) : ceil_div(p.d, FIN_W);
      F.groups = F.perm_groups + plain;
      F.pitch = std::max(width, FIN_W) | 1;
      F.block0 = blocks;
      F.alpha = p.alpha; F.beta = p.beta;
      blocks += ceil_div(p.d, FIN_ROWS) * F.groups;
      fin_smem = std::max(fin_smem, (size_t)FIN_ROWS * F.pitch * sizeof(float));
    }
    bp.nitems = items;
    SSO_CHECK_ARG(fin_smem <= 200 * 1024, "factor batch: kernel window too large for the finishing kernel");
    const int pairs = std::max(1, std::min(max_pairs, items));
    factor_batch_kernel<<<2 * pairs, THREADS, smem, st>>>(bp);
    SSO_LAUNCH_OK("factor_batch_kernel");
    SSO_ENSURE_SMEM(factor_batch_finish_kernel, 200 * 1024);
    factor_batch_finish_kernel<<<blocks, 256, fin_smem, st>>>(fpm);
    SSO_LAUNCH_OK("factor_batch_finish_kernel");
    at += cnt;
  }
  return 0;
}

}  // namespace batch
