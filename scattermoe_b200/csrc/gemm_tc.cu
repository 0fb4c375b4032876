#include "smoe_common.cuh"
namespace smoe {
int launch_s2s_tc(const S2SArgs&) { return SMOE_ERR_UNSUPPORTED; }
int launch_wgrad_tc(const WGradArgs&) { return SMOE_ERR_UNSUPPORTED; }
}
