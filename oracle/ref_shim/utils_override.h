/* Force-included INSTEAD of the reference's common/utils.h (its include guard UTILS_H is pre-defined on the command
 * line): the same declarations, with the two compile-time switches set to the lossless configuration the parity
 * runs need.  The reference ships batch_type = SEMI_BATCH and compress = true (cuda_gcn/src/common/utils.h:8,10),
 * which replace exchanged values by stale or 8-bit ones.  Test infrastructure for oracle/_ref only. */
#ifndef DRONE_ORACLE_UTILS_OVERRIDE_H
#define DRONE_ORACLE_UTILS_OVERRIDE_H
/* With a single worker the reference's exchange launches kernels over zero received rows; CUDA reports "invalid
 * configuration argument" for those and the reference's CUDA_CHECK answers with exit().  The aggregation result is
 * complete by then, so exit() inside the reference sources is turned into an exception the driver catches. */
#include <cstdlib>
#include <stdlib.h>
struct DroneRefExit { int code; };
/* The driver of a whole training epoch sets drone_ref_tolerate_exit: the launch error of a zero-row kernel is then
 * cleared where the reference checks it and the epoch carries on (the driver checks the device at the end). */
extern int drone_ref_tolerate_exit;
extern "C" int cudaGetLastError_for_ref_shim(void);
inline void drone_ref_exit(int code) {
    if (drone_ref_tolerate_exit) {
        cudaGetLastError_for_ref_shim();
        return;
    }
    throw DroneRefExit{code};
}
#define exit(code) drone_ref_exit(code)
typedef enum { FULL_BATCH, SEMI_BATCH } BatchType;
const BatchType batch_type = FULL_BATCH;
const bool compress = false;
const bool time_debug = false;
const int max_grid_size = 102400;
const bool sc = false;
extern long long master2mirror_forward_total[2], mirror2master_forward_total[2], master2mirror, mirror2master,
    master2mirror_backward_total[2], mirror2master_backward_total[2];
extern int current_epoch;
extern float mean_accuracy;
extern bool update_threshold;
#endif
