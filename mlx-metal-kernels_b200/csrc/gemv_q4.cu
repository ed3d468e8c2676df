// q4 instantiations of the tensor-core matvec kernel.
#include "gemv_params.cuh"

namespace b200q {
B200Q_DEFINE_STATUS_WORD(gemv_q4_read_status)
}

#include "gemv_fast.cuh"

namespace b200q {
int gemv_fast_q4(GemvParams& p, bool gate_up, cudaStream_t stream) { return dispatch_bits<4>(p, gate_up, stream); }
}  // namespace b200q

#if defined(B200Q_DBG_TRACE)
extern "C" int b200q_dbg_read_events(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, b200q::g_events, sizeof(unsigned long long) * 32);
}
extern "C" int b200q_dbg_read_trace(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, b200q::g_trace, sizeof(unsigned long long) * 4 * 1024);
}
#endif
