// Launchers shared between translation units of libt2t_b200.so (not part of the C ABI).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>

#include "t2t_b200.h"

namespace t2t {

// Tensor-core assignment with exact verification (assign_tc.cu).  `amb` is a
// scratch list of (H * N + 1) ints: a counter followed by the rows queued for
// the exact re-evaluation.
size_t assign_ws_bytes(int H, int N);
int launch_assign(const __nv_bfloat16* X, const __nv_bfloat16* cen, int* labels, int H, int N, int Cn,
                  int pin_begin, int pin_label, int* amb, int* d_status, cudaStream_t st);

// Exact warp-per-row selection of the rows queued in fixq (select.cu).  fixq: per
// head a count followed by (row, query cluster) pairs, H * (2 N + 1) ints.
int launch_select_fix(const __nv_bfloat16* QU, const __nv_bfloat16* cks, const int* kcounts, const int* ns,
                      int* unip, int* rowcnt, int H, int N, int CQ, const int* fixq, cudaStream_t st);

// Tensor map (128 bytes, written to map_out) over the bf16 matrix base [rows, 128]
// with a 64-column x 1-row box and 128-byte swizzle, for tma_gather4 (tma_rows.cu).
// False when the driver entry point is missing or the encoding is refused.
bool make_row_gather_map(void* map_out, const void* base, uint64_t rows);
// Same matrix, box of 64 columns x `box_rows` rows: plain tile loads of contiguous rows.
bool make_row_tile_map(void* map_out, const void* base, uint64_t rows, uint32_t box_rows);

// A bf16 tensor of `heads` x `rows_per_head` rows of 128 elements (row (h, n) at base + h * head_stride +
// n * row_stride, strides in elements) as a 3D tensor with a 64-column x `box_rows`-row x 1-head box: tile
// loads that never cross a head, rows past the head's last row read as zeros.
bool make_head_tile_map(void* map_out, const void* base, uint64_t rows_per_head, uint64_t heads, uint32_t box_rows,
                        uint64_t row_stride, uint64_t head_stride);

}  // namespace t2t
