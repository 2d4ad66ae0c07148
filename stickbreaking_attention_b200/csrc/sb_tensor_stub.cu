// placeholder until the tcgen05 kernels are in
#include "sb_common.cuh"
namespace sb {
bool tensor_path_eligible(const SbParams&, bool, int* why) { *why = SBATTN_EUNSUPPORTED; return false; }
int launch_tensor_fwd(const SbParams&, const WsLayout&, const KArgs&, cudaStream_t) { return 1; }
int launch_tensor_bwd(const SbParams&, const WsLayout&, const KArgs&, cudaStream_t) { return 1; }
}
