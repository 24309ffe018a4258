// Launch parameters shared by the factor-construction kernels.
#pragma once
#include <stdint.h>

namespace sso {

struct FactorParams {
  const void* x;
  const float* weight;  // per-sample, nullable
  float* out;
  float* partial;  // workspace [tile][split][128*128]
  int64_t sn, sc, sh, sw;
  int64_t ldo;
  int64_t rows;  // n*ho*wo
  int n, c, h, w, ho, wo;
  int kh, kw, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int d;        // columns incl. the ones column
  int dcols;    // c*kh*kw
  int splits;
  int rows_per_split;
  float alpha, beta;
  // tensor-core path only
  int* status;      // device word: 0 ok, else the code of the wait that gave up
  int perm_c;       // > 0: kernel columns are ordered (kh, kw, c) with c < perm_c; 0: natural order
  int perm_kk;      // kh*kw
  // finishing inside the producing kernel (factor_finish.cuh); tickets == nullptr: separate kernel
  int* tickets;     // [ticket_tiles] per-tile counters, then [ticket_tiles][16] per-group counters
  int ticket_tiles;
};

// Scratch layout of the tensor-core factor kernels: [status word, 256 bytes][ticket counters]
// [partial tiles].  The header is cleared on the stream by every launch.
inline size_t factor_header_bytes(int tiles) {
  return 256 + (((size_t)tiles * 17 * sizeof(int) + 255) / 256) * 256;
}

struct RowInfo {   // one im2col row (n, ho, wo)
  int64_t base;    // n*sn
  int ih0, iw0;    // top-left input coordinate of the patch
  float wgt;       // sample weight (A operand only)
  int valid;
};
struct ColInfo {   // one im2col column (c, kh, kw) or the ones column
  int64_t off;     // c*sc
  int dh, dw;      // kh*dil_h, kw*dil_w
  int kind;        // 0 data, 1 ones, 2 out of range
  int pad;
};

}  // namespace sso
