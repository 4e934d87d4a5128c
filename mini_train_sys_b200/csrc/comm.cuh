// Peer-memory collectives for sm_100a (implemented in comm.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mts {
}  // namespace mts
