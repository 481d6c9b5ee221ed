// Load-time re-ordering of one QLinear record into the device layout.  Every step is an
// exact re-ordering of the checkpoint's bits; nothing is re-quantised.
//
// Device layout of a QLinear (IN, OUT, GS), G = IN/GS groups, Gp = G rounded up to 4:
//   qw     [OUT][IN/8]  u32  the checkpoint's qweight rows (nibble j of word i is the
//                            weight of permuted input 8i+j), optionally with the output
//                            rows re-ordered;
//   scales [OUT][Gp]    f32  zero padded;
//   zeros  [OUT/8][Gp]  u32  nibble r of word [b][g] is the zero nibble of row 8b+r.
// Padding Gp keeps every 8-row block of scales/zeros 16-byte aligned.
#include <cstdlib>
#include <cstring>

#include "repack.h"

namespace l2 {

void repack_qlinear(int in, int out, int gs, const int32_t* qweight, const int32_t* qzeros,
                    const float* scales, const int32_t* rows_order, PackedQ& dst) {
    const int g = (int)Shape::groups(in, gs);
    const int gp = (g + 3) & ~3;
    const int wpr = in / 8;
    dst.in = in; dst.out = out; dst.groups = g; dst.gp = gp;
    dst.qw.assign((size_t)out * wpr, 0);
    dst.sc.assign((size_t)out * gp, 0.0f);
    dst.zr.assign((size_t)(out / 8) * gp, 0);
    for (int j = 0; j < out; j++) {
        const int src = rows_order ? rows_order[j] : j;
        memcpy(&dst.qw[(size_t)j * wpr], qweight + (size_t)src * wpr, sizeof(uint32_t) * wpr);
        memcpy(&dst.sc[(size_t)j * gp], scales + (size_t)src * g, sizeof(float) * g);
        const uint32_t* zsrc = reinterpret_cast<const uint32_t*>(qzeros) + (size_t)(src / 8) * g;
        uint32_t* zdst = &dst.zr[(size_t)(j / 8) * gp];
        const int sshift = 4 * (src % 8), dshift = 4 * (j % 8);
        for (int k = 0; k < g; k++) zdst[k] |= ((zsrc[k] >> sshift) & 15u) << dshift;
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
                               float** scales_dev, uint32_t** zeros_dev, int* groups_padded) {
    clear_error();
    if (!qweight || !qzeros || !scales || !qw_dev || !scales_dev || !zeros_dev || !groups_padded)
        return fail(L2_EINVAL, "l2_debug_repack: null argument");
    if (in % 32 || out % 8 || in % group_size) return fail(L2_EINVAL, "l2_debug_repack: bad shape");
    if (rows_order && !is_permutation(rows_order, out)) return fail(L2_EINVAL, "l2_debug_repack: rows_order is not a permutation");
    PackedQ p;
    repack_qlinear(in, out, group_size, qweight, qzeros, scales, rows_order, p);
    *qw_dev = (uint32_t*)malloc(p.qw.size() * 4);
    *scales_dev = (float*)malloc(p.sc.size() * 4);
    *zeros_dev = (uint32_t*)malloc(p.zr.size() * 4);
    memcpy(*qw_dev, p.qw.data(), p.qw.size() * 4);
    memcpy(*scales_dev, p.sc.data(), p.sc.size() * 4);
    memcpy(*zeros_dev, p.zr.data(), p.zr.size() * 4);
    *groups_padded = p.gp;
    return L2_OK;
}
