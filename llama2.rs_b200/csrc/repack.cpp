// Load-time re-ordering of one QLinear record into the device layout.  Every step is an
// exact re-ordering of the checkpoint's bits; nothing is re-quantised.
//
// The GEMV kernel feeds the weights to mma.sync.m16n8k32 (u8 x s8): a tile is 16 output rows, a
// unit is (tile, quantisation group).  Inside a unit the 32-bit words (8 nibbles each; nibble j
// of word i is the weight of permuted input 8i+j, as in the checkpoint) are stored in the order
// in which the 32 lanes of a warp consume them, so that a warp reads one unit with two fully
// coalesced loads per lane and the units of a tile are contiguous:
//   qw     [tile][group][half h][lane L][W]   row = 16*tile + 8*h + L/4, words (L%4)*W .. +W-1 of the group
//   meta   [tile][group][20]                  words 0-15: f32 scales of rows 16*tile + i; words 16,17:
//                                             zero nibbles (nibble r of word 16+h = row 16*tile + 8*h + r);
//                                             words 18,19 pad the record to 80 bytes (bulk copies move
//                                             multiples of 16 bytes)
#include <cstdlib>
#include <cstring>

#include "repack.h"

namespace l2 {

void repack_qlinear(int in, int out, int gs, const int32_t* qweight, const int32_t* qzeros,
                    const float* scales, const int32_t* rows_order, PackedQ& dst) {
    const int g = (int)Shape::groups(in, gs);
    const int w = gs / 32;
    const int wpr = in / 8;        // words per checkpoint row
    const int wpg = gs / 8;        // words per group
    const int tiles = (out + 15) / 16;
    dst.in = in; dst.out = out; dst.groups = g; dst.tiles = tiles; dst.w = w;
    dst.qw.assign((size_t)tiles * g * 64 * w, 0);
    dst.meta.assign((size_t)tiles * g * 20, 0);
    const uint32_t* qws = reinterpret_cast<const uint32_t*>(qweight);
    const uint32_t* qzs = reinterpret_cast<const uint32_t*>(qzeros);
    for (int j = 0; j < out; j++) {
        const int src = rows_order ? rows_order[j] : j;
        const int tile = j / 16, h = (j % 16) / 8, r = j % 8;
        for (int k = 0; k < g; k++) {
            const size_t unit = (size_t)tile * g + k;
            for (int t = 0; t < 4; t++)
                for (int i = 0; i < w; i++)
                    dst.qw[(unit * 2 + h) * 32 * w + (size_t)(r * 4 + t) * w + i] = qws[(size_t)src * wpr + (size_t)k * wpg + t * w + i];
            memcpy(&dst.meta[unit * 20 + (j % 16)], &scales[(size_t)src * g + k], 4);
            const uint32_t nib = (qzs[(size_t)(src / 8) * g + k] >> (4 * (src % 8))) & 15u;
            dst.meta[unit * 20 + 16 + h] |= nib << (4 * r);
        }
    }
}

std::vector<int32_t> inverse_permutation(const int32_t* perm, int n) {
    std::vector<int32_t> inv(n);
    for (int j = 0; j < n; j++) inv[perm[j]] = j;
    return inv;
}

bool is_permutation(const int32_t* perm, int n) {
    std::vector<char> seen(n, 0);
    for (int j = 0; j < n; j++) {
        if (perm[j] < 0 || perm[j] >= n || seen[perm[j]]) return false;
        seen[perm[j]] = 1;
    }
    return true;
}

}  // namespace l2

using namespace l2;

extern "C" int l2_debug_repack(int in, int out, int group_size, const int32_t* qweight, const int32_t* qzeros,
                               const float* scales, const int32_t* rows_order, uint32_t** qw_dev,
                               uint32_t** meta_dev, int* tiles) {
    clear_error();
    if (!qweight || !qzeros || !scales || !qw_dev || !meta_dev || !tiles)
        return fail(L2_EINVAL, "l2_debug_repack: null argument");
    if (in % 32 || out % 8 || in % group_size) return fail(L2_EINVAL, "l2_debug_repack: bad shape");
    if (rows_order && !is_permutation(rows_order, out)) return fail(L2_EINVAL, "l2_debug_repack: rows_order is not a permutation");
    PackedQ p;
    repack_qlinear(in, out, group_size, qweight, qzeros, scales, rows_order, p);
    *qw_dev = (uint32_t*)malloc(p.qw.size() * 4);
    *meta_dev = (uint32_t*)malloc(p.meta.size() * 4);
    memcpy(*qw_dev, p.qw.data(), p.qw.size() * 4);
    memcpy(*meta_dev, p.meta.data(), p.meta.size() * 4);
    *tiles = p.tiles;
    return L2_OK;
}
