// The aggregation kernels for one combination of the template switches of spmm_kernels.cuh
// (UNIT = true, HOT = true); a translation unit of its own so that the combinations compile side by side.
#include "spmm_kernels.cuh"

#include <algorithm>

namespace drone {

int spmm_dispatch_unit_hot(const SpmmArgs &a, bool vec4) {
    return vec4 ? dispatch_width<4, true, true>(a) : dispatch_width<1, true, true>(a);
}

}  // namespace drone
