// Host side of TMA: building the CUtensorMap a kernel reads its (bh, rows, width) operand through.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "common.h"

namespace limn_b200 {

// A 4-D map (column, row, head, batch) over an operand of 2-byte elements, fetched in boxes of `box_rows`
// rows by 64 elements (128 bytes) of one (batch, head) problem, written to shared memory with the 128-byte
// swizzle the tcgen05 operand descriptors expect. Rows past `rows` read as zero, so a ragged last tile
// never reaches another problem's rows.
int make_tile_map(CUtensorMap* map, const void* base, bool fp16, int batch, int heads, int rows, int width, int box_rows,
                  const Strides& strides);

}  // namespace limn_b200
