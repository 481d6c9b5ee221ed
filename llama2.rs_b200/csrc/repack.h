// Load-time re-ordering of QLinear records into the device layout (see repack.cpp).
#pragma once

#include <cstdint>
#include <vector>

#include "host_common.h"

namespace l2 {

struct PackedQ {
    int in = 0, out = 0, groups = 0, gp = 0;
    std::vector<uint32_t> qw;  // [OUT][IN/8]
    std::vector<float> sc;     // [OUT][gp]
    std::vector<uint32_t> zr;  // [OUT/8][gp]
};

// rows_order[j] = checkpoint row that becomes device row j (NULL = identity).
void repack_qlinear(int in, int out, int gs, const int32_t* qweight, const int32_t* qzeros,
                    const float* scales, const int32_t* rows_order, PackedQ& dst);
std::vector<int32_t> inverse_permutation(const int32_t* perm, int n);
bool is_permutation(const int32_t* perm, int n);

}  // namespace l2
