// The aggregation kernels for one combination of the template switches of spmm_kernels.cuh
// (UNIT = false, HOT = true); a translation unit of its own so that the combinations compile side by side.
#include "spmm_kernels.cuh"

#include <algorithm>

namespace drone {

int spmm_dispatch_hot(const SpmmArgs &a, bool vec4) {
    return vec4 ? dispatch_width<4, false, true>(a) : dispatch_width<1, false, true>(a);
}

}  // namespace drone
