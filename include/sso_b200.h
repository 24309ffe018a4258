/*
 * sso_b200 -- C ABI of the B200 (sm_100a) K-FAC curvature kernels.
 *
 * The reference library (PyTorch-SSO) has no C ABI of its own: its native work is done by
 * torch ATen, CuPy/cuSOLVER and ChainerMN calls made from Python.  Each entry point below
 * names the reference call site(s) (path within the reference project : lines) whose work
 * it replaces.  The Python package `torchsso` in this repository binds these symbols with
 * ctypes; nothing here takes or returns a torch type.
 *
 * Conventions
 *   - every pointer named *_dev / x / out / ... is a DEVICE pointer unless the comment says
 *     host; matrices are row-major fp32 unless a dtype argument says otherwise;
 *   - `stream` is a cudaStream_t passed as void*; calls enqueue work and return without
 *     synchronising (plan creation is the exception: it uploads its tables synchronously);
 *   - return value 0 = success, negative = error (sso_last_error() gives the text);
 *   - no entry point allocates device memory unless its comment says so: callers size
 *     scratch with the *_bytes query and pass it in;
 *   - numerical failure (non-positive pivot) is reported asynchronously through an int
 *     `info` array on the device, LAPACK style (0 = ok, k > 0 = first bad pivot, 1-based).
 */
#ifndef SSO_B200_H_
#define SSO_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SSO_VERSION 100

enum { SSO_F32 = 0, SSO_BF16 = 1, SSO_F16 = 2 };
/* factor kernel implementations.  AUTO picks, in this order, the TMA-fed tcgen05 kernel (16-bit
 * channels-contiguous inputs with a multiple of 64 channels, no ones column, no weights), the
 * tcgen05 kernel with a register/cp.async gather (channels-contiguous inputs, 16-bit or fp32 as
 * 3xTF32), the fp32 SIMT kernel (anything). */
enum { SSO_IMPL_AUTO = 0, SSO_IMPL_SIMT = 1, SSO_IMPL_TCGEN05 = 2, SSO_IMPL_TMA = 3 };

int sso_version(void);
const char* sso_last_error(void);
/* kernels launched by this library since it was loaded (bookkeeping for benchmarks) */
uint64_t sso_launch_count(void);
/* process-wide switches: "tc_auto" / "tma_auto" (0/1: may SSO_IMPL_AUTO choose the tcgen05 kernels /
 * the TMA-fed one), "engine_tc" (0/1: 128-wide tile phases of the engine on tcgen05 3xTF32 or fp32 FFMA),
 * "tc_flush" (stages of tensor-core accumulation between drains into fp32 registers),
 * "chol_ksplit" (first 128-column panel of the blocked Cholesky whose update tasks are cut along K;
 * 0 = never; read when a plan is built), "rowwise_max_splits" (column-permuted factors of >= 1024 columns with
 * at most this many row splits are finished by the kernel that writes whole output rows), "chol_panel" (0/1: a panel's 128x128 diagonal block is factorised
 * and inverted by one launch, or as two 64-wide halves; read when a plan is built), "phase_lpt" (0/1: tasks
 * of a 128-wide phase ordered by decreasing K, so that the longest tasks of a launch start first; read when
 * a plan is built) */
int sso_configure(const char* key, int value);

/* ---------------------------------------------------------------------------------------
 * Kronecker factor construction (symmetric rank-k update with the im2col gather fused in).
 *
 *   out <- alpha * sum_r w[n(r)] * u_r u_r^T  +  beta * out,        out is d x d, ld = ldo
 *
 * u_r is row r = (n, ho, wo) of the im2col matrix of x (logical NCHW dims n,c,h,w with
 * element strides sn,sc,sh,sw -- channels_last and plain 2-D matrices are stride choices),
 * columns ordered (c, kh, kw); append_ones adds a trailing column of ones (bias).  w is an
 * optional per-sample weight (length n, fp32), NULL = 1.  Both triangles of out are written.
 * A plain matrix X[rows, cols] is the case n=rows, c=cols, h=w=kh=kw=1.
 *
 * Replaces: torchsso/curv/cov/linear.py:50-67 (einsum 'ki,kj->ij' + cat of ones),
 *           torchsso/curv/cov/conv.py:47-74 (F.unfold, transpose/reshape copy, cat, einsum),
 *           torchsso/curv/fisher/linear.py:44-53, torchsso/curv/fisher/conv.py:56-66
 *           (prob-weighted variants), the in-place rescale at torchsso/curv/curvature.py:299-300
 *           and the accumulation at torchsso/utils/accumulator.py:23-38 (through alpha/beta).
 * ------------------------------------------------------------------------------------- */
size_t sso_factor_workspace_bytes(int64_t rows, int64_t d, int impl);

int sso_factor_syrk_im2col(const void* x, int dtype,
                           int64_t n, int64_t c, int64_t h, int64_t w,
                           int64_t sn, int64_t sc, int64_t sh, int64_t sw,
                           int kh, int kw, int stride_h, int stride_w,
                           int pad_h, int pad_w, int dil_h, int dil_w,
                           int append_ones, const float* sample_weight,
                           float alpha, float beta, float* out, int64_t ldo,
                           void* workspace, size_t workspace_bytes, int impl, void* stream);

int sso_factor_syrk(const void* x, int dtype, int64_t rows, int64_t cols,
                    int64_t row_stride, int64_t col_stride,
                    int append_ones, const float* row_weight,
                    float alpha, float beta, float* out, int64_t ldo,
                    void* workspace, size_t workspace_bytes, int impl, void* stream);

/* Many factors in one call: every problem is what one sso_factor_syrk_im2col call describes (a plain
 * [rows, cols] matrix is n = rows, c = cols, h = w = 1 with a 1x1 window).  Problems with 16-bit
 * channels-contiguous inputs whose channel count is a multiple of 64 (no ones column, no per-sample
 * weights) are cut into equally long work items and processed by ONE persistent tcgen05 kernel plus
 * one finishing kernel; the others run one by one behind them.  The outputs must be distinct
 * matrices.  Scratch: sso_factor_batch_workspace_bytes bytes, contents irrelevant on entry.
 * Replaces: the per-layer loop of curvature updates that the hooks of
 *           torchsso/curv/curvature.py:118-155 run one layer at a time (each a full launch sequence
 *           of torchsso/curv/cov/conv.py:47-74 or torchsso/curv/cov/linear.py:50-67). */
typedef struct {
  const void* x;
  int32_t dtype, append_ones;
  int64_t n, c, h, w, sn, sc, sh, sw;
  int32_t kh, kw, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  const float* sample_weight;
  float alpha, beta;
  float* out;
  int64_t ldo;
} sso_factor_desc;
size_t sso_factor_batch_workspace_bytes(int n, const sso_factor_desc* descs);
int sso_factor_batch(int n, const sso_factor_desc* descs, void* workspace, size_t workspace_bytes, void* stream);

/* sso_factor_syrk for callers that are not allowed to allocate device memory when they need a
 * factor (all device memory already given to their own pool, a fixed memory budget after start-up,
 * or no tolerance for the implicit synchronisation of an allocation).  It has no counterpart in
 * the reference, which allocates freely on every call.
 * The split-partial scratch is a 16 MiB array inside the library image: every GPU that loads the
 * library holds it until the process exits.  Shapes whose scratch need (sso_factor_workspace_bytes)
 * is larger are rejected with an error and nothing is launched.  The first call on a device
 * resolves the array's device address; make it before any stream capture begins.  Where the CUDA
 * driver loads modules lazily, that first call is also when it sets the 16 MiB aside on the device
 * (free device memory drops by that amount, once; no later call changes it).  All calls on a
 * device share the array: calls whose GPU work can overlap (other streams or threads) race and
 * must be serialised by the caller; calls on one stream are safe.  Nothing on this path calls
 * cudaMalloc / cudaFree or an allocating library routine. */
int sso_factor_syrk_noalloc(const void* x, int dtype, int64_t rows, int64_t cols,
                            int64_t row_stride, int64_t col_stride,
                            int append_ones, const float* row_weight,
                            float alpha, float beta, float* out, int64_t ldo,
                            int impl, void* stream);

/* ---------------------------------------------------------------------------------------
 * BatchNorm diagonal curvature in two streaming stages, so that nothing activation-sized
 * is kept between forward and backward (in-place ReLU / residual adds may overwrite the
 * layer output afterwards):
 *   forward :  sx[n,c] = sum_hw ((y - shift[c]) / scale[c])^2       (y = layer output)
 *   backward:  sg[n,c] = sum_hw g^2                                  (g = grad of the output)
 *   finish  :  w_out[c] <- alpha/n * sum_n sx * p_n * sg + beta * w_out[c]
 *              b_out[c] <- alpha/n * sum_n      p_n * sg + beta * b_out[c]     (b_out nullable)
 * y / g are logical [n, c, hw] with element strides (s*n, s*c, s*p); either may be NULL to
 * run only the other half; scale/shift NULL mean 1/0; p = sample_weight or 1.
 * Channels-contiguous tensors may be reduced in `splits` pieces of the pixel range (more blocks
 * for large planes): sx / sg then hold [n, splits, c] partial sums, and the finishing call is told
 * the split count of each.  sso_bn_plane_splits gives the count to use (1 = no splitting).
 * Replaces: torchsso/curv/curvature.py:123-134 (restore normalised input),
 *           torchsso/curv/cov/batchnorm.py:10-49, torchsso/curv/fisher/batchnorm.py:11-32.
 * ------------------------------------------------------------------------------------- */
int sso_bn_plane_splits(int dtype, int64_t n, int64_t c, int64_t hw, int64_t stride_c);
int sso_bn_plane_sums(const void* y, const void* g, int dtype, int64_t n, int64_t c, int64_t hw,
                      int64_t syn, int64_t syc, int64_t syp, int64_t sgn, int64_t sgc, int64_t sgp,
                      const float* scale, const float* shift, float* sx, float* sg, int splits,
                      void* stream);
int sso_bn_diag_finish(const float* sx, const float* sg, const float* sample_weight,
                       int64_t n, int64_t c, int splits_x, int splits_g, float alpha, float beta,
                       float* w_out, float* b_out, void* stream);

/* ---------------------------------------------------------------------------------------
 * Streaming kernels over flat fp32 buffers.  The Python side keeps every factor of every
 * layer in one contiguous pool per role (data / ema / inverse), so one launch covers a model.
 * ------------------------------------------------------------------------------------- */
/* ema <- first ? data : beta*data + (1-beta)*ema      (beta weights the NEW data)
 * Replaces: torchsso/curv/curvature.py:174-191. */
int sso_ema_update(const float* data, float* ema, int64_t count, float beta, int first, void* stream);
/* dst <- a*src + b*dst (dst is not read when b == 0).  Replaces the scale/accumulate copies of
 * torchsso/utils/accumulator.py:23-53 and torchsso/optim/secondorder.py:174-182,213-223. */
int sso_axpby(const float* src, float* dst, int64_t count, float a, float b, void* stream);
/* Diagonal curvature:  inv <- 1/(ema [sqrt] + damping) if update_inv;  grad <- grad*inv if grad.
 * Replaces: torchsso/curv/curvature.py:226-238. */
int sso_diag_inv_precondition(const float* ema, float* inv, float* grad, int64_t count,
                              float damping, int use_sqrt, int update_inv, void* stream);

/* ---------------------------------------------------------------------------------------
 * Triangular packing for the factor exchange: packed[n*y - y*(y+1)/2 + x] = scale*m[y][x],
 * x >= y (row-major upper triangle); unpack writes both triangles.  One record = a run of
 * rows of one matrix, one CTA per record; the table lives in device memory.
 * Replaces: torchsso/utils/chainer_communicators/_utility.py:19-33 (unpack kernel),
 *           :59-86 (cuBLAS trttp pack) and the mean kernel at
 *           torchsso/utils/chainer_communicators/pure_nccl_communicator.py:184-199,430-435
 *           (through scale).
 * ------------------------------------------------------------------------------------- */
typedef struct {
  float* m;          /* matrix base (row-major, leading dimension ld) */
  float* packed;     /* base of this matrix's packed triangle */
  int32_t n, ld;
  int32_t row0, nrows;
} sso_tri_rec;
int sso_tri_pack(const sso_tri_rec* recs_dev, int n_recs, float scale, void* stream);
/* symmetric != 0: both triangles are written; 0: upper triangle only, zeros below (for the
 * triangular factors exchanged by the variational optimizer) */
int sso_tri_unpack(const sso_tri_rec* recs_dev, int n_recs, float scale, int symmetric, void* stream);

/* dst[0:count] <- scale * src[0:count] for a device table of flat segments, one launch.
 * Replaces the per-array device-to-device copies of Packer.pack / unpack for non-square arrays
 * (torchsso/utils/chainer_communicators/_utility.py:35-57). */
typedef struct {
  const float* src;
  float* dst;
  int64_t count;
} sso_seg_rec;
int sso_copy_segments(const sso_seg_rec* recs_dev, int n_recs, float scale, void* stream);

/* 16-bit wire format of the exchange with per-array scaling.  A packed fp32 buffer is a sequence of
 * arrays; the device table cuts it into runs of at most a few thousand elements of one array each.
 *   sso_wire_absmax : maxima[array] <- max(maxima[array], max |x|) over the array's runs (clear
 *                     `maxima` first); the caller sums the maxima over the ranks (one small all-reduce).
 *   sso_wire_encode : out16[i] <- cast(buf[i] * 65000 / sums[array(i)])   (bf16 or fp16)
 *   sso_wire_decode : out32[i] <- float(in16[i]) * sums[array(i)] / 65000
 * An array whose summed maximum is zero or not finite travels unscaled.
 * Replaces: torchsso/utils/chainer_communicators/pure_nccl_communicator.py:359-412
 *           (_communication_scale / _rescale: per-array max-abs on side streams, all-reduce of the
 *           maxima, scale to 65000 / sum before the cast, rescale after) and the cast kernels at
 *           :415-429; here scaling is fused into the cast in both directions. */
typedef struct {
  int64_t offset;    /* first element of the run inside the packed buffer */
  int64_t count;
  int32_t array;     /* index into maxima / sums */
  int32_t pad;
} sso_wire_rec;
int sso_wire_absmax(const float* buf, const sso_wire_rec* recs_dev, int n_recs, float* maxima, void* stream);
int sso_wire_encode(const float* buf, const sso_wire_rec* recs_dev, int n_recs, const float* sums, void* out16,
                    int dtype, void* stream);
int sso_wire_decode(const void* in16, const sso_wire_rec* recs_dev, int n_recs, const float* sums, float* out32,
                    int dtype, void* stream);

/* Diagonal curvature of Linear / Conv2d layers: mean over samples of the squared per-sample weight
 * gradient (torchsso/curv/cov/linear.py:28-45, torchsso/curv/cov/conv.py:15-42; the reference builds
 * it from F.unfold + a batched matmul + elementwise squares):
 *     out_w[o][j] <- alpha * sum_b w_b * ( sum_l g[b,o,l] * u[b,l,j] )^2 + beta * out_w[o][j]
 *     out_b[o]    <- alpha * sum_b w_b *   sum_l g[b,o,l]^2              + beta * out_b[o]   (out_b nullable)
 * x [n,c,h,w] and g [n,oc,ho,wo] with element strides; a Linear layer is h = w = 1 with a 1x1 kernel;
 * j runs over (c, ky, kx) like the weight itself.  Exact fp32 accumulation. */
size_t sso_diag_sq_workspace_bytes(int64_t n, int64_t oc, int64_t d);
int sso_diag_sq_im2col(const void* x, const void* g, int dtype, int64_t n, int64_t c, int64_t h, int64_t w,
                       int64_t sxn, int64_t sxc, int64_t sxh, int64_t sxw, int64_t oc,
                       int64_t sgn, int64_t sgc, int64_t sgh, int64_t sgw,
                       int kh, int kw, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                       const float* sample_weight /* [n] or NULL */, float alpha, float beta,
                       float* out_w /* [oc][c*kh*kw] */, float* out_b /* [oc] or NULL */,
                       void* workspace, size_t workspace_bytes, void* stream);

/* Optimizer tail over a table of parameter chunks: weight decay / l2, momentum, gradient moving
 * average, bias-correction scale and the parameter update in one launch
 * (replaces the per-group multi-tensor chains of torchsso/optim/secondorder.py:225-283,
 * update_preprocess + update):
 *     g += add * p
 *     if (mbuf) { mbuf = momentum * mbuf + g;  g = mbuf; }
 *     if (ebuf) { ebuf = (1 - ema) * ebuf + ema * g;  g = ebuf; }
 *     g *= scale
 *     if (lr != 0) p -= lr * g
 * The "raw" stage (before preconditioning) passes add = l2_reg and lr = 0, the "preconditioned"
 * stage add = weight_decay and the group's lr. */
typedef struct {
  float* p;
  float* g;
  float* mbuf;       /* nullable */
  float* ebuf;       /* nullable */
  int64_t count;
  float add, momentum, ema, scale, lr;
  int32_t pad;
} sso_tail_rec;
int sso_optimizer_tail(const sso_tail_rec* recs_dev, int n_recs, void* stream);

/* ---------------------------------------------------------------------------------------
 * Tile-task engine.  All dense algebra after factor construction (pi-damped SPD inverse,
 * Cholesky factor of the inverse, G^-1 dW A^-1, posterior sampling) is expressed as phases
 * of independent tile tasks   C[m x n] <- alpha * op(A)[m x k] * op(B)[k x n] + beta * C
 * plus a small dense diagonal-block factorisation; one kernel launch runs a whole phase for
 * every matrix of every layer.  A plan is built once for a fixed set of device buffers.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  const float* A;
  const float* B;
  float* C;
  float* C2;          /* optional transposed copy of the tile (mirror), NULL if unused */
  int32_t lda, ldb, ldc, ldc2;
  int32_t m, n, k;
  uint32_t flags;     /* bit0: A transposed, bit1: B transposed, bit2: symmetric square tile (only
                         its lower half is computed and it is mirrored inside the tile) */
  float alpha, beta;
} sso_tile_task;

/* diagonal-block record: factor block (<= 64 x 64 in a phase of kind 2, <= 128 x 128 in one of kind 5) in
   place, also write the inverse of its factor */
typedef struct {
  float* L;           /* block (j,j) of the working matrix; lower triangle valid on entry */
  float* Linv;        /* receives the inverse of the block's Cholesky factor */
  int32_t ld_l, ld_inv;
  int32_t size;       /* valid rows/cols of this block */
  int32_t mat;        /* matrix index (for info) */
  int32_t row0;       /* first global row of the block (for info) */
  int32_t info_slot;  /* 0 inverse pass, 1 Cholesky-of-inverse pass */
  float* LinvT;       /* optional: also receives the transpose of that inverse (upper triangular) */
  int32_t ld_invt;
  int32_t pad;
} sso_diag_rec;

/* copy record: a run of whole rows of one d x d matrix */
typedef struct {
  const float* src;
  float* dst;
  int32_t d;
  int32_t row0, nrows;
  int32_t mat;        /* index into the diagonal-shift table, or -1 */
  int32_t mode;       /* 0 dst = src (+ shift on the diagonal), 1 dst = upper-triangular transpose
                         of src's lower triangle, 2 dst = 0 */
  int32_t ld;         /* leading dimension of src and dst */
} sso_copy_rec;

typedef struct {
  int32_t kind;       /* 0 gemm64, 1 gemm128, 2 diag-block factor (<= 64), 3 copy, 4 gemm128 whose operands are both read along k,
                         5 diag-block factor of a 128-column panel (same records as 2, size <= 128) */
  int32_t first;      /* first record of this phase in its table */
  int32_t count;      /* number of records (= CTAs) */
  int32_t reserved;
} sso_phase;

/* Batched pi-damped SPD inverse (and optional upper Cholesky factor of the result).
 *   for matrix i:  M_i = src_i + v_i * I,  v_i = r_i * pi  (role 0, "A")  or  r_i / pi  (role 1, "G")
 *                  pi  = sqrt( (tr A / d_A) / (tr G / d_G) ) of the pair (i, partner_i); partner -1 => pi = 1
 *                  dst_i <- M_i^-1 (both triangles);   std_i <- U with U^T U = dst_i (upper), if requested
 * Replaces: torchsso/curv/curvature.py:302-312 and :334-340 (pi, add_value_to_diagonal),
 *           torchsso/utils/inv_cupy.py:27-132 (cuSOLVER potrf + potrs against identity),
 *           torchsso/curv/curvature.py:317-321 with torchsso/utils/cholesky_cupy.py:9-14.
 * All arrays are HOST arrays of length n_mats; work_i is d_i*d_i floats of scratch.
 * dev_mem (device, sso_kron_plan_dev_bytes bytes) receives the tables; host_only != 0 builds
 * the plan without touching the device (for inspecting the task program on a CPU).
 * Returns a plan handle > 0, or a negative error. */
size_t sso_kron_plan_dev_bytes(int n_mats, const int64_t* dims, int with_std);
int64_t sso_kron_plan_create(int n_mats, const int64_t* dims, float* const* src, float* const* dst,
                             float* const* work, float* const* std_out /* nullable */,
                             const int32_t* partner, const int32_t* role,
                             void* dev_mem, size_t dev_mem_bytes, int host_only,
                             const int64_t* lds /* nullable: leading dimensions of src/dst/work/std, default dims */);
/* damp_r_dev: per-matrix r = sqrt(damping); info_dev: per-matrix status (2 ints: inverse, std) */
int sso_kron_plan_run(int64_t plan, const float* damp_r_dev, int* info_dev,
                      int do_inverse, int do_std, void* stream);

/* Kronecker precondition  dW|db <- G^-1 [dW|db] A^-1  for a set of layers, in place.
 * Replaces: torchsso/curv/cov/linear.py:69-84, torchsso/curv/cov/conv.py:76-92 (cat, 2 mm, 2 copies).
 * HOST arrays of length n_layers; gb_i may be NULL (no bias => d_A is the weight's column
 * count, else columns + 1); tmp_i is dG_i*dA_i floats of scratch. */
size_t sso_precond_plan_dev_bytes(int n_layers, const int64_t* dA, const int64_t* dG);
int64_t sso_precond_plan_create(int n_layers, const int64_t* dA, const int64_t* dG,
                                float* const* A_inv, float* const* G_inv,
                                float* const* gw, float* const* gb, float* const* tmp,
                                void* dev_mem, size_t dev_mem_bytes, int host_only,
                                const int64_t* ldA, const int64_t* ldG /* nullable: leading dimensions of
                                A_inv / G_inv (default dA / dG); tmp is [dA x dG] with leading dimension ldG */);
int sso_precond_plan_run(int64_t plan, void* stream);

/* Posterior sampling  [W|b] <- [W|b] + s * U_G E U_A  (W, b pre-loaded with the mean by the
 * caller; E is dG x dA standard normal, supplied).  U_* upper triangular.
 * Replaces: torchsso/curv/cov/linear.py:86-100, torchsso/curv/cov/conv.py:94-108. */
size_t sso_sample_plan_dev_bytes(int n_layers, const int64_t* dA, const int64_t* dG);
int64_t sso_sample_plan_create(int n_layers, const int64_t* dA, const int64_t* dG,
                               float* const* U_A, float* const* U_G, float* const* noise,
                               float* const* w, float* const* b, float* const* tmp,
                               void* dev_mem, size_t dev_mem_bytes, int host_only,
                               const int64_t* ldA, const int64_t* ldG /* nullable: leading dimensions of U_A / U_G */);
int sso_sample_plan_run(int64_t plan, float std_scale, void* stream);

int sso_plan_destroy(int64_t plan);
/* 0, or the code of a bounded device-side wait that gave up in a tensor-core tile task of this
 * plan (synchronises; for diagnostics) */
int sso_plan_status(int64_t plan);

/* Plan introspection (host side; used to check the task program without a GPU). */
int sso_plan_num_phases(int64_t plan);
int sso_plan_get_phase(int64_t plan, int index, sso_phase* out);
int sso_plan_num_tasks(int64_t plan);
int sso_plan_copy_tasks(int64_t plan, sso_tile_task* out, int capacity);
int sso_plan_num_diag_recs(int64_t plan);
int sso_plan_copy_diag_recs(int64_t plan, sso_diag_rec* out, int capacity);
int sso_plan_num_copy_recs(int64_t plan);
int sso_plan_copy_copy_recs(int64_t plan, sso_copy_rec* out, int capacity);

/* Run one ad-hoc list of tile tasks that already sits in device memory. */
int sso_run_tile_tasks(const sso_tile_task* tasks_dev, int count, int tile /* 64 or 128 */, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SSO_B200_H_ */
