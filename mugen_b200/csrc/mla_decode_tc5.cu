#include "mla_launch.h"
namespace mla {
int decode_tc5_configure() { return int(cudaErrorNotSupported); }
int launch_decode_tc5(int, const void*, const void*, uint32_t, uint32_t, const StepMeta&, float*, uint32_t, uint32_t*, cudaStream_t) { return int(cudaErrorNotSupported); }
}
