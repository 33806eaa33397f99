// Host side of TMA: building the CUtensorMap a kernel reads its (bh, rows, width) operand through.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

namespace limn_b200 {

// Where element (batch b, head h, row t, column 0) of an operand lives: base + b * batch + h * head + t * row
// elements. Columns are always contiguous.
struct Strides {
  long long batch, head, row;
};
// Strides of a (batch, heads, rows, width) operand in the given limn_b200_layout.
Strides strides_of(int layout, int heads, int rows, int width);

// A 4-D map (column, row, head, batch) over an operand of 2-byte elements, fetched in boxes of `box_rows`
// rows by 64 elements (128 bytes) of one (batch, head) problem, written to shared memory with the 128-byte
// swizzle the tcgen05 operand descriptors expect. Rows past `rows` read as zero, so a ragged last tile
// never reaches another problem's rows.
int make_tile_map(CUtensorMap* map, const void* base, bool fp16, int batch, int heads, int rows, int width, int box_rows,
                  const Strides& strides);

}  // namespace limn_b200
