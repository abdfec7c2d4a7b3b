// KV-tile range a q-tile has to visit, as plain integer arithmetic shared by the host entry
// point, the prefill kernel and (through the C ABI) the Python analysis layer.
//
// The reference derives the same ranges symbolically (z3 + sympy) in
// loopfuse/compiler/passes/skip_loop_iterations.py:287-378 and rewrites Loop.start/end at
// :343-376. Here the range is defined directly as "every KV tile that holds at least one
// unmasked, in-bounds (row, column) pair of the q-tile", which is what a brute-force scan of
// the mask gives; it equals the reference's closed forms except for the reference's window
// lower bound when tile_k divides (iq*tile_q - window + 2), where the reference drops one
// live corner tile.
#pragma once

#include <stdint.h>

#include "../../include/lf_sm100.h"

#if defined(__CUDACC__)
#define LF_HD __host__ __device__ __forceinline__
#else
#define LF_HD inline
#endif

namespace lf {

LF_HD int32_t floor_div(int32_t a, int32_t b) {  // b > 0
  int32_t q = a / b;
  return (a % b != 0 && a < 0) ? q - 1 : q;
}

LF_HD void skip_range(int32_t mask_kind, int32_t window, int32_t causal_offset, int32_t Sq,
                      int32_t Skv, int32_t tile_q, int32_t tile_k, int32_t iq, int32_t* lo,
                      int32_t* hi) {
  const int32_t n_kt = (Skv + tile_k - 1) / tile_k;
  const int32_t row_first = iq * tile_q;
  int32_t row_last = row_first + tile_q - 1;
  if (row_last > Sq - 1) row_last = Sq - 1;
  int32_t l = 0, h = n_kt;
  if (row_first > row_last) {  // q-tile outside the sequence
    *lo = 0;
    *hi = 0;
    return;
  }
  if (mask_kind == LF_MASK_CAUSAL || mask_kind == LF_MASK_CAUSAL_WINDOW) {
    const int32_t last_col = row_last + causal_offset;  // largest visible column of the tile
    if (last_col < 0) {
      h = 0;
    } else {
      const int32_t hh = last_col / tile_k + 1;
      if (hh < h) h = hh;
    }
  }
  if (mask_kind == LF_MASK_CAUSAL_WINDOW) {
    const int32_t first_col = row_first + causal_offset - (window - 1);
    if (first_col > 0) {
      const int32_t ll = first_col / tile_k;
      if (ll > l) l = ll;
    }
  }
  if (h <= l) {  // nothing visible: the empty range is always reported as [0, 0)
    l = 0;
    h = 0;
  }
  *lo = l;
  *hi = h;
}

}  // namespace lf
