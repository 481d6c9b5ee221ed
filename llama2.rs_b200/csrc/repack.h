// Load-time re-ordering of QLinear records into the device layout (see repack.cpp).
#pragma once

#include <cstdint>
#include <vector>

#include "host_common.h"

namespace l2 {

// Device layout of one QLinear (IN, OUT, GS): the matrix is cut into tiles of 16 output rows and
// units of (tile, group).  W = GS/32 is the number of 32-bit weight words a lane holds per row.
struct PackedQ {
    int in = 0, out = 0, groups = 0, tiles = 0, w = 0;
    // [tiles][groups] unit records of 64*W + 20 words, contiguous so that one bulk copy moves a run:
    //   words [h][L][W]  half h, lane L=(r,t): weight words t*W..t*W+W-1 of row 16*tile+8h+r in the group
    //   16 f32 scales (row 16*tile+i), 2 zero words (nibble r of word h = zero nibble of row 16*tile+8h+r),
    //   2 words of padding (the record is a multiple of 16 bytes)
    std::vector<uint32_t> rec;
    int unit_words() const { return 64 * w + 20; }
};

// rows_order[j] = checkpoint row that becomes device row j (NULL = identity).  Rows beyond OUT in
// the last tile are zero (weights, scales and zero nibbles), so they contribute nothing.
void repack_qlinear(int in, int out, int gs, const int32_t* qweight, const int32_t* qzeros,
                    const float* scales, const int32_t* rows_order, PackedQ& dst);
void repack_compact(int in, int n, int gs, const uint32_t* qw, const float* sc, const uint8_t* zn, PackedQ& dst);
void gather_rows(int in, int gs, const uint32_t* qweight, const uint32_t* qzeros, const float* scales,
                 const int32_t* rows, int n, uint32_t* qw, float* sc, uint8_t* zn);
std::vector<int32_t> inverse_permutation(const int32_t* perm, int n);
bool is_permutation(const int32_t* perm, int n);

}  // namespace l2
