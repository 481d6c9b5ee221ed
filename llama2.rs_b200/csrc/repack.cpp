// Load-time re-ordering of one QLinear record into the device layout.  Every step is an
// exact re-ordering of the checkpoint's bits; nothing is re-quantised.
//
// The GEMV kernel feeds the weights to mma.sync.m16n8k32 (u8 x s8): a tile is 16 output rows, a
// unit is (tile, quantisation group).  Inside a unit the 32-bit words (8 nibbles each; nibble j
// of word i is the weight of permuted input 8i+j, as in the checkpoint) are stored in the order
// in which the 32 lanes of a warp consume them, so that a warp reads one unit with two fully
// coalesced loads per lane and the units of a tile are contiguous:
//   rec [tile][group] = { words[half h][lane L][W]   row = 16*tile + 8*h + L/4, words (L%4)*W .. +W-1 of the group
//                         scales[16]                  f32, rows 16*tile + i
//                         zeros[2]                    nibble r of word h = zero nibble of row 16*tile + 8*h + r
//                         pad[2] }                    the record is a multiple of 16 bytes (bulk copies need that)
#include <cstdlib>
#include <cstring>

#include "repack.h"

namespace l2 {

// Core: rows given compactly -- qw [n][in/8] words, sc [n][groups] scales, zn [n][groups] zero nibbles
// (one byte each) -- in the order they take on the device.
void repack_compact(int in, int n, int gs, const uint32_t* qw, const float* sc, const uint8_t* zn, PackedQ& dst) {
    const int g = (int)Shape::groups(in, gs);
    const int w = gs / 32;
    const int wpr = in / 8;        // words per row
    const int wpg = gs / 8;        // words per group
    const int tiles = (n + 15) / 16;
    dst.in = in; dst.out = n; dst.groups = g; dst.tiles = tiles; dst.w = w;
    const size_t uw = (size_t)dst.unit_words();
    dst.rec.assign((size_t)tiles * g * uw, 0);
    for (int j = 0; j < n; j++) {
        const int tile = j / 16, h = (j % 16) / 8, r = j % 8;
        for (int k = 0; k < g; k++) {
            const size_t unit = (size_t)tile * g + k;
            for (int t = 0; t < 4; t++)
                for (int i = 0; i < w; i++)
                    dst.rec[unit * uw + (size_t)h * 32 * w + (size_t)(r * 4 + t) * w + i] = qw[(size_t)j * wpr + (size_t)k * wpg + t * w + i];
            memcpy(&dst.rec[unit * uw + 64 * w + (j % 16)], &sc[(size_t)j * g + k], 4);
            dst.rec[unit * uw + 64 * w + 16 + h] |= (uint32_t)(zn[(size_t)j * g + k] & 15u) << (4 * r);
        }
    }
}

// Rows `rows[0..n)` of a QLinear in checkpoint layout, compactly (see repack_compact).
void gather_rows(int in, int gs, const uint32_t* qweight, const uint32_t* qzeros, const float* scales,
                 const int32_t* rows, int n, uint32_t* qw, float* sc, uint8_t* zn) {
    const int g = (int)Shape::groups(in, gs), wpr = in / 8;
    for (int j = 0; j < n; j++) {
        const int src = rows[j];
        memcpy(qw + (size_t)j * wpr, qweight + (size_t)src * wpr, sizeof(uint32_t) * wpr);
        memcpy(sc + (size_t)j * g, scales + (size_t)src * g, sizeof(float) * g);
        for (int k = 0; k < g; k++) zn[(size_t)j * g + k] = (uint8_t)((qzeros[(size_t)(src / 8) * g + k] >> (4 * (src % 8))) & 15u);
    }
}

void repack_qlinear(int in, int out, int gs, const int32_t* qweight, const int32_t* qzeros,
                    const float* scales, const int32_t* rows_order, PackedQ& dst) {
    const int g = (int)Shape::groups(in, gs);
    std::vector<int32_t> rows(out);
    for (int j = 0; j < out; j++) rows[j] = rows_order ? rows_order[j] : j;
    std::vector<uint32_t> qw((size_t)out * (in / 8));
    std::vector<float> sc((size_t)out * g);
    std::vector<uint8_t> zn((size_t)out * g);
    gather_rows(in, gs, reinterpret_cast<const uint32_t*>(qweight), reinterpret_cast<const uint32_t*>(qzeros), scales,
                rows.data(), out, qw.data(), sc.data(), zn.data());
    repack_compact(in, out, gs, qw.data(), sc.data(), zn.data(), dst);
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
                               const float* scales, const int32_t* rows_order, uint32_t** rec_dev,
                               int* tiles, int* unit_words) {
    clear_error();
    if (!qweight || !qzeros || !scales || !rec_dev || !tiles || !unit_words)
        return fail(L2_EINVAL, "l2_debug_repack: null argument");
    if (in % 32 || out % 8 || in % group_size) return fail(L2_EINVAL, "l2_debug_repack: bad shape");
    if (rows_order && !is_permutation(rows_order, out)) return fail(L2_EINVAL, "l2_debug_repack: rows_order is not a permutation");
    PackedQ p;
    repack_qlinear(in, out, group_size, qweight, qzeros, scales, rows_order, p);
    *rec_dev = (uint32_t*)malloc(p.rec.size() * 4);
    memcpy(*rec_dev, p.rec.data(), p.rec.size() * 4);
    *tiles = p.tiles;
    *unit_words = p.unit_words();
    return L2_OK;
}
