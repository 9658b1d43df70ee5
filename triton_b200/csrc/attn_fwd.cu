#include "common.cuh"
#include "host.h"
namespace trn {
int launch_attention(const TrnAttnArgs&, cudaStream_t, const DeviceState&) { return TRN_E_VARIANT; }
}
