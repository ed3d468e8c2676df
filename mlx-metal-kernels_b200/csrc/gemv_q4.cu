// q4 instantiations of the tensor-core matvec kernel.
#include "gemv_params.cuh"

namespace b200q {
B200Q_DEFINE_STATUS_WORD(gemv_q4_read_status)
}

#include "gemv_fast.cuh"

namespace b200q {
int gemv_fast_q4(GemvParams& p, bool gate_up, cudaStream_t stream) { return dispatch_bits<4>(p, gate_up, stream); }
}  // namespace b200q
