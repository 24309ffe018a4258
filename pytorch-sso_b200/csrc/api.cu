// extern "C" entry points for factor construction plus library-wide state.
#include <mutex>

#include "common.cuh"

namespace sso {

thread_local std::string g_last_error;
unsigned long long g_launches = 0;
}  // namespace sso

#include <algorithm>
#include <map>
#include <utility>
#include <vector>

namespace sso {
int ensure_dynamic_smem(const void* kernel, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> done;
  int dev = -1;
  SSO_CUDA_OK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(mu);
  int& have = done[std::make_pair(kernel, dev)];
  if (have >= bytes) return 0;
  SSO_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  have = bytes;
  return 0;
}
}  // namespace sso

#include "factor_params.cuh"

namespace sso {
int factor_tma_set_wait_controls(long long cycles, int stall);
int factor_tc_set_wait_controls(long long cycles, int stall);
int engine_tc_set_wait_controls(long long cycles, int stall);
static long long g_wait_kcycles = 0;   // 0 = default limit
static int g_stall = 0;
static int apply_wait_controls() {
  const long long cycles = g_wait_kcycles * 1024;
  int rc = factor_tma_set_wait_controls(cycles, g_stall);
  if (!rc) rc = factor_tc_set_wait_controls(cycles, 0);
  if (!rc) rc = engine_tc_set_wait_controls(cycles, g_stall);
  return rc;
}
size_t factor_simt_workspace_bytes(int64_t rows, int64_t d);
int factor_simt_launch(FactorParams p, int dtype, void* workspace, size_t workspace_bytes, cudaStream_t st);
size_t factor_tc_workspace_bytes(int64_t rows, int64_t d);
bool factor_tc_supported(const FactorParams& p, int dtype);
int factor_tc_launch(FactorParams p, int dtype, void* workspace, size_t workspace_bytes, cudaStream_t st);
void factor_tc_set_flush(int stages);
int factor_tc_flush_setting();
bool factor_tma_supported(const FactorParams& p, int dtype);
void factor_tma_set_pair_min_d(int d);
void factor_tma_set_f32(int on);
void factor_tma_set_fused_finish(int on);
void factor_batch_set_pairs(int pairs);
void factor_tc_set_rowwise_max_splits(int s);
int factor_tma_launch(FactorParams p, int dtype, void* workspace, size_t workspace_bytes, int flush, cudaStream_t st);
size_t factor_batch_scratch_bytes(const FactorParams* ps, const int* dtypes, int n);
int factor_batch_launch(const FactorParams* ps, const int* dtypes, int n, unsigned char* done, void* workspace,
                        size_t workspace_bytes, int flush, cudaStream_t st);
extern int g_engine_tc;
static int g_tc_auto = 1;    // whether SSO_IMPL_AUTO may pick the tcgen05 kernels
static int g_tma_auto = 1;   // whether SSO_IMPL_AUTO may pick the TMA-fed tcgen05 kernel
}  // namespace sso

using namespace sso;

namespace sso { extern int g_engine_tma; extern int g_chol_ksplit; extern int g_phase_lpt; extern int g_chol_panel; }

extern "C" {

int sso_version(void) { return SSO_VERSION; }
const char* sso_last_error(void) { return g_last_error.c_str(); }
uint64_t sso_launch_count(void) { return __atomic_load_n(&g_launches, __ATOMIC_RELAXED); }

int sso_configure(const char* key, int value) {
  SSO_CHECK_ARG(key != nullptr, "configure: null key");
  const std::string k(key);
  if (k == "tc_auto") { g_tc_auto = value != 0; return 0; }
  if (k == "tma_auto") { g_tma_auto = value != 0; return 0; }
  if (k == "engine_tc") { g_engine_tc = value != 0; return 0; }
  if (k == "tma_f32") { factor_tma_set_f32(value); return 0; }
  if (k == "batch_pairs") { factor_batch_set_pairs(value); return 0; }
  if (k == "rowwise_max_splits") { factor_tc_set_rowwise_max_splits(value); return 0; }
  if (k == "fused_finish") { factor_tma_set_fused_finish(value); return 0; }
  if (k == "tma_pair_min_d") { factor_tma_set_pair_min_d(value); return 0; }
  if (k == "engine_tma") { g_engine_tma = value != 0; return 0; }
  if (k == "phase_lpt") { g_phase_lpt = value != 0; return 0; }
  if (k == "chol_ksplit") { g_chol_ksplit = (int)value; return 0; }
  if (k == "chol_panel") { g_chol_panel = value != 0; return 0; }
  // failure-path controls, current device only: the limit of every bounded device-side wait in units of
  // 1024 clocks (0 = the default of ~2 s), and a switch that makes the TMA producers of the factor and
  // tile-task kernels issue no loads, so that the waits of their consumers run out
  if (k == "wait_kcycles") { g_wait_kcycles = value < 0 ? 0 : value; return apply_wait_controls(); }
  if (k == "inject_stall") { g_stall = value != 0; return apply_wait_controls(); }
  if (k == "tc_flush") { factor_tc_set_flush(value); return 0; }
  return fail(-1, "configure: unknown key %s", key);
}

size_t sso_factor_workspace_bytes(int64_t rows, int64_t d, int impl) {
  const size_t a = factor_simt_workspace_bytes(rows, d);
  const size_t b = factor_tc_workspace_bytes(rows, d);
  if (impl == SSO_IMPL_SIMT) return a;
  if (impl == SSO_IMPL_TCGEN05 || impl == SSO_IMPL_TMA) return b;
  return a > b ? a : b;
}

// Argument checks and launch parameters shared by the single-problem and the batched entry points.
static int make_factor_params(const void* x, int64_t n, int64_t c, int64_t h, int64_t w, int64_t sn, int64_t sc,
                              int64_t sh, int64_t sw, int kh, int kw, int stride_h, int stride_w, int pad_h, int pad_w,
                              int dil_h, int dil_w, int append_ones, const float* sample_weight, float alpha,
                              float beta, float* out, int64_t ldo, FactorParams& p) {
  SSO_CHECK_ARG(x != nullptr && out != nullptr, "factor: null pointer");
  SSO_CHECK_ARG(n > 0 && c > 0 && h > 0 && w > 0, "factor: bad input dims");
  SSO_CHECK_ARG(kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 && dil_h > 0 && dil_w > 0 && pad_h >= 0 &&
                    pad_w >= 0, "factor: bad conv geometry");
  const int64_t ho = (h + 2 * pad_h - (int64_t)dil_h * (kh - 1) - 1) / stride_h + 1;
  const int64_t wo = (w + 2 * pad_w - (int64_t)dil_w * (kw - 1) - 1) / stride_w + 1;
  SSO_CHECK_ARG(ho > 0 && wo > 0, "factor: empty output");
  const int64_t dcols = c * kh * kw;
  const int64_t d = dcols + (append_ones ? 1 : 0);
  SSO_CHECK_ARG(d <= 65536 && n < ((int64_t)1 << 31) && ho * wo < ((int64_t)1 << 31), "factor: shape too large");
  SSO_CHECK_ARG(ldo >= d, "factor: ldo < d");
  p = FactorParams{};
  p.x = x; p.weight = sample_weight; p.out = out; p.partial = nullptr;
  p.sn = sn; p.sc = sc; p.sh = sh; p.sw = sw; p.ldo = ldo;
  p.rows = n * ho * wo;
  p.n = (int)n; p.c = (int)c; p.h = (int)h; p.w = (int)w; p.ho = (int)ho; p.wo = (int)wo;
  p.kh = kh; p.kw = kw; p.stride_h = stride_h; p.stride_w = stride_w;
  p.pad_h = pad_h; p.pad_w = pad_w; p.dil_h = dil_h; p.dil_w = dil_w;
  p.d = (int)d; p.dcols = (int)dcols;
  p.alpha = alpha; p.beta = beta;
  return 0;
}

static int launch_one_factor(const FactorParams& p, int dtype, void* workspace, size_t workspace_bytes, int impl,
                             cudaStream_t st) {
  if (impl == SSO_IMPL_TMA) {
    SSO_CHECK_ARG(factor_tma_supported(p, dtype), "factor: shape not supported by the TMA-fed tcgen05 path");
    return factor_tma_launch(p, dtype, workspace, workspace_bytes, factor_tc_flush_setting(), st);
  }
  if (impl == SSO_IMPL_AUTO && g_tc_auto && g_tma_auto && factor_tma_supported(p, dtype))
    return factor_tma_launch(p, dtype, workspace, workspace_bytes, factor_tc_flush_setting(), st);
  if (impl == SSO_IMPL_TCGEN05) {
    SSO_CHECK_ARG(factor_tc_supported(p, dtype), "factor: shape not supported by the tcgen05 path");
    return factor_tc_launch(p, dtype, workspace, workspace_bytes, st);
  }
  if (impl == SSO_IMPL_AUTO && g_tc_auto && factor_tc_supported(p, dtype))
    return factor_tc_launch(p, dtype, workspace, workspace_bytes, st);
  return factor_simt_launch(p, dtype, workspace, workspace_bytes, st);
}

int sso_factor_syrk_im2col(const void* x, int dtype, int64_t n, int64_t c, int64_t h, int64_t w,
                           int64_t sn, int64_t sc, int64_t sh, int64_t sw, int kh, int kw,
                           int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                           int append_ones, const float* sample_weight, float alpha, float beta,
                           float* out, int64_t ldo, void* workspace, size_t workspace_bytes, int impl,
                           void* stream) {
  FactorParams p;
  const int rc = make_factor_params(x, n, c, h, w, sn, sc, sh, sw, kh, kw, stride_h, stride_w, pad_h, pad_w, dil_h,
                                    dil_w, append_ones, sample_weight, alpha, beta, out, ldo, p);
  if (rc) return rc;
  return launch_one_factor(p, dtype, workspace, workspace_bytes, impl, reinterpret_cast<cudaStream_t>(stream));
}

// ---- many factors in one call ----------------------------------------------------------------
static int batch_params(int n, const sso_factor_desc* descs, std::vector<FactorParams>& ps, std::vector<int>& dts) {
  SSO_CHECK_ARG(n >= 0 && (n == 0 || descs != nullptr), "factor batch: bad argument");
  ps.resize(n);
  dts.resize(n);
  for (int i = 0; i < n; ++i) {
    const sso_factor_desc& q = descs[i];
    const int rc = make_factor_params(q.x, q.n, q.c, q.h, q.w, q.sn, q.sc, q.sh, q.sw, q.kh, q.kw, q.stride_h, q.stride_w,
                                      q.pad_h, q.pad_w, q.dil_h, q.dil_w, q.append_ones, q.sample_weight, q.alpha, q.beta,
                                      q.out, q.ldo, ps[i]);
    if (rc) return rc;
    dts[i] = q.dtype;
  }
  return 0;
}

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

size_t sso_factor_batch_workspace_bytes(int n, const sso_factor_desc* descs) {
  std::vector<FactorParams> ps;
  std::vector<int> dts;
  if (batch_params(n, descs, ps, dts) != 0) return 0;
  size_t single = 0;
  for (int i = 0; i < n; ++i) single = std::max(single, sso_factor_workspace_bytes(ps[i].rows, ps[i].d, SSO_IMPL_AUTO));
  const size_t batched = (g_tc_auto && g_tma_auto) ? factor_batch_scratch_bytes(ps.data(), dts.data(), n) : 256;
  return align256(batched) + align256(single);
}

int sso_factor_batch(int n, const sso_factor_desc* descs, void* workspace, size_t workspace_bytes, void* stream) {
  std::vector<FactorParams> ps;
  std::vector<int> dts;
  const int rc = batch_params(n, descs, ps, dts);
  if (rc) return rc;
  if (n == 0) return 0;
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < i; ++j)
      SSO_CHECK_ARG(ps[i].out != ps[j].out, "factor batch: problems %d and %d write the same matrix", j, i);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  std::vector<unsigned char> done(n, 0);
  size_t batched = 256;
  if (g_tc_auto && g_tma_auto) {
    batched = factor_batch_scratch_bytes(ps.data(), dts.data(), n);
    SSO_CHECK_ARG(workspace != nullptr && workspace_bytes >= batched, "factor batch: workspace too small: need %zu bytes, got %zu",
                  batched, workspace_bytes);
    const int rb = factor_batch_launch(ps.data(), dts.data(), n, done.data(), workspace, batched, factor_tc_flush_setting(), st);
    if (rb) return rb;
  }
  // whatever the batched kernel does not take (fp32 inputs, odd channel counts, a ones column, per-sample
  // weights) runs through the single-problem path behind the batch's scratch
  char* tail = workspace ? reinterpret_cast<char*>(workspace) + align256(batched) : nullptr;
  const size_t tail_bytes = workspace_bytes > align256(batched) ? workspace_bytes - align256(batched) : 0;
  for (int i = 0; i < n; ++i) {
    if (done[i]) continue;
    const int r1 = launch_one_factor(ps[i], dts[i], tail, tail_bytes, SSO_IMPL_AUTO, st);
    if (r1) return r1;
  }
  return 0;
}

int sso_factor_syrk(const void* x, int dtype, int64_t rows, int64_t cols, int64_t row_stride,
                    int64_t col_stride, int append_ones, const float* row_weight, float alpha,
                    float beta, float* out, int64_t ldo, void* workspace, size_t workspace_bytes,
                    int impl, void* stream) {
  return sso_factor_syrk_im2col(x, dtype, rows, cols, 1, 1, row_stride, col_stride, 0, 0, 1, 1, 1, 1, 0, 0,
                                1, 1, append_ones, row_weight, alpha, beta, out, ldo, workspace,
                                workspace_bytes, impl, stream);
}

// ---------------------------------------------------------------------------------------------
// Factor construction for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc (or anything that may call it) at the point
// where they need a factor: an embedding runtime that handed all device memory to its own pool
// at start-up, a service with a hard memory budget that forbids growth after initialisation, or
// code running where an implicit device synchronisation (which cudaMalloc implies) is not
// acceptable.  sso_factor_syrk needs scratch for its split partial tiles, so those callers get
// this variant: the scratch is a fixed array that is part of the loaded library image.
//
//  * The array is kStaticScratchBytes (16 MiB) per GPU that loads the library and stays
//    resident until the process exits, whether or not this entry point is ever used.
//  * Problems whose scratch need (sso_factor_workspace_bytes) exceeds it are rejected with an
//    error; nothing is launched.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress,
//    with that device current).  Make that first call before starting any stream capture.  With
//    CUDA's lazy module loading that look-up is also the moment the driver sets the array's 16 MiB
//    aside on that device (free device memory drops by that much, once); no later call changes the
//    amount of free device memory.
//  * All calls on a device share the one array and it keeps the previous call's contents.  The
//    kernels overwrite every partial tile before reading it and the status word is cleared on the
//    stream at the start of each call, so back-to-back calls on ONE stream are safe; calls whose
//    GPU work may overlap (different streams, different host threads) race on the array and must
//    be serialised by the caller.
//  * No cudaMalloc, cudaFree or allocating library routine is called on this path.
constexpr size_t kStaticScratchBytes = (size_t)16 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_scratch_mu;
static void* g_scratch_addr[kMaxDevices] = {};

// In host code `g_static_scratch` is only a handle for the symbol, not a device address:
// the address a kernel can use has to be asked for, once per device.
static int static_scratch_address(void** out) {
  int dev = -1;
  SSO_CUDA_OK(cudaGetDevice(&dev));
  SSO_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    SSO_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
    SSO_CHECK_ARG(p != nullptr, "cudaGetSymbolAddress returned a null address");
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

int sso_factor_syrk_noalloc(const void* x, int dtype, int64_t rows, int64_t cols, int64_t row_stride,
                            int64_t col_stride, int append_ones, const float* row_weight, float alpha,
                            float beta, float* out, int64_t ldo, int impl, void* stream) {
  SSO_CHECK_ARG(rows > 0 && cols > 0, "factor (no-alloc): bad shape");
  const int64_t d = cols + (append_ones ? 1 : 0);
  const size_t need = sso_factor_workspace_bytes(rows, d, impl);
  SSO_CHECK_ARG(need <= kStaticScratchBytes,
                "factor (no-alloc): %lld rows x %lld columns needs %zu bytes of scratch but the built-in "
                "scratch holds %zu; use sso_factor_syrk with caller-provided scratch",
                (long long)rows, (long long)d, need, kStaticScratchBytes);
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != 0) return rc;
  return sso_factor_syrk(x, dtype, rows, cols, row_stride, col_stride, append_ones, row_weight, alpha, beta,
                         out, ldo, scratch, kStaticScratchBytes, impl, stream);
}

}  // extern "C"
