// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the
// runtime's driver entry point lookup, so the library does not link libcuda).
#pragma once
#include <cuda.h>
#include <stdint.h>

#include "common.cuh"

namespace evo {

// 16-bit [B,H,S,R,D] attention-view tensor -> 5-D map with dims (D, R, S, H, B).
// Box = (box_d, box_r, 1, 1, 1); rows of box_d*2 bytes are swizzled with the matching
// 32/64/128-byte pattern.  Elements beyond D or R read as zero.
bool make_qkv_map(CUtensorMap* out, const void* base, const Str4& stride_elems, int B, int H, int S, int R, int D,
                  int box_d, int box_r);

// fp32 [B,H,R,R] pair bias -> 4-D map with dims (R_j, R_i, H, B); box = (box_j, box_i, 1, 1)
// with box_j = 32 (rows of 128 bytes, 128-byte swizzle) or 16 (rows of 64 bytes, 64-byte swizzle).
bool make_bias_map(CUtensorMap* out, const float* base, const Str3& stride_elems, int B, int H, int R, int box_i,
                   int box_j);

// Contiguous fp32 [slabs, R, D] (the dQ accumulator: one slab per (b,h,s)) as a 3-D map
// (D, R, slabs) with box (box_d, box_r, 1); rows and columns beyond R and D are clipped.
bool make_rows_f32_map(CUtensorMap* out, const float* base, int D, int R, long long slabs, int box_d, int box_r);
// The same tensor with an unswizzled box (rows of box_d floats land back to back in shared memory).
bool make_rows_f32_plain_map(CUtensorMap* out, const float* base, int D, int R, long long slabs, int box_d, int box_r);

// fp32 [B,H,R,R] pair bias (or its dense gradient) as a 4-D map (R_j, R_i, H, B) with an
// unswizzled box (box_j, box_i, 1, 1): rows of box_j floats land back to back in shared memory.
bool make_bias_plain_map(CUtensorMap* out, const float* base, const Str3& stride_elems, int B, int H, int R, int box_i,
                         int box_j);

// 16-bit [B,H,R,R] pair bias as a 4-D map (R_j, R_i, H, B), box (box_j, box_i, 1, 1): rows of
// box_j*2 bytes, swizzled with the matching pattern when `swizzle` is set (box_j*2 <= 128), else
// back to back.
bool make_bias16_map(CUtensorMap* out, const void* base, const Str3& stride_elems, int B, int H, int R, int box_i,
                     int box_j, bool swizzle = true);

// Contiguous fp32 per-row statistics [B*H, S, R] as a 3-D map (R, S, B*H) with box (box_r, 1, 1);
// rows beyond R and MSA rows beyond S read as zero.
bool make_stats_map(CUtensorMap* out, const float* base, int BH, int S, int R, int box_r);

}  // namespace evo
