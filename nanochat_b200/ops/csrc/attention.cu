#include "attention.h"

namespace nc {

cudaError_t attention_fwd(const AttnDesc&, int*, cudaStream_t) { return cudaErrorNotSupported; }

}  // namespace nc
