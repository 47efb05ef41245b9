/* prefill.cu — placeholder until the tcgen05 kernel lands: nothing fits, so callers take the three-door path. */
#include "kernels.h"
namespace sv {
bool prefill_fits(const PrefillCall&) { return false; }
cudaError_t prefill_launch(const PrefillCall&) { return cudaErrorNotSupported; }
}
