#include "common.cuh"
#include "host.h"
namespace trn {
int launch_colstats(const TrnColStatsArgs&, cudaStream_t, const DeviceState&) { return TRN_E_VARIANT; }
}
