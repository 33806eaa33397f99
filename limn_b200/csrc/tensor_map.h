// Host side of TMA: building the CUtensorMap a kernel reads its (bh, rows, width) operand through.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

namespace limn_b200 {

// A 3-D map over a dense (bh, rows, width) tensor of 2-byte elements, fetched in boxes of
// `box_rows` rows by 64 elements (128 bytes) of one problem, written to shared memory with
// the 128-byte swizzle the tcgen05 operand descriptors expect. Rows past `rows` read as
// zero, so a ragged last tile never reaches the next problem's rows.
int make_tile_map(CUtensorMap* map, const void* base, bool fp16, long long bh, int rows, int width, int box_rows);

}  // namespace limn_b200
