// Parameters shared by the matvec kernels and their host-side dispatch.
#pragma once

#include "common.cuh"

namespace b200q {

#ifndef B200Q_GEMV_WARPS
#define B200Q_GEMV_WARPS 16
#endif
constexpr int kConsumerWarps = B200Q_GEMV_WARPS;
constexpr int kConsumerThreads = kConsumerWarps * 32;
#ifndef B200Q_GEMV_PRODUCERS
#define B200Q_GEMV_PRODUCERS 3
#endif
// Issuing a bulk copy costs the issuing warp about 40 ns per copy (measured), so the copies of a stage are
// shared by several producer warps.
constexpr int kProducerWarps = B200Q_GEMV_PRODUCERS;
constexpr int kFirstProducerWarp = kConsumerWarps;
constexpr int kEpilogueWarp = kConsumerWarps + kProducerWarps;
constexpr int kThreads = (kConsumerWarps + kProducerWarps + 1) * 32;
#ifndef B200Q_GEMV_MIN_CTAS
#define B200Q_GEMV_MIN_CTAS 1
#endif
// CTAs of this kernel (or of two kernels of a dependent chain) that fit on one SM: bounds registers and shared memory.
constexpr int kMinCtasPerSm = B200Q_GEMV_MIN_CTAS;
constexpr int kTileRows = 16;
constexpr int kUnitGroups = 8;
constexpr uint32_t kWaitLimit = 1u << 21;
constexpr int kMaxStages = 8;
constexpr int kMaxSlots = 16;

struct GemvParams {
    // activations
    const void* x;          // [B, K]
    const void* res_in;     // norm prologue: x := rmsnorm(x + res_in); may be null
    const void* norm_w;     // [K]; null = no prologue
    float eps;
    void* z_out;            // [B, K] or null
    void* normed_out;       // [B, K] or null
    // weights (index 1 only for the fused gate/up kernel)
    const uint8_t* w[2];
    const void* s[2];
    const void* z[2];
    // outputs
    const void* residual;   // plain: out = cast(residual + cast(y)); may be null
    void* y;
    void* gate_out;
    void* up_out;
    void* act_out;
    int B, N, K, G, Gn;
    int act_dtype, scale_dtype, norm_w_dtype;
    int row_bytes;          // bytes of one weight row
    int kc;                 // k per ring stage (a whole number of units)
    int n_kc;               // stages per (matrix, tile) over the whole K
    int nu;                 // units per full stage
    int stages;
    int xk;                 // k per staged activation chunk (a whole number of stages)
    int n_xc;               // activation chunks (1 unless B*K is too large for shared memory)
    int nslot;              // result slots: 2 (streamed) or one per tile of the CTA (n_xc > 1)
    int meta_depth;         // buffers for the scales / zero points of a (tile, matrix)
    int meta_vec;           // scales / zeros are fp16, 16-byte aligned, Gn % 8 == 0: vector loads
    int interleave;         // 1: CTA c takes tiles c, c + grid, ... instead of a contiguous row range
    int rows_lo, rem;       // CTA c owns rows_lo (+1 if c < rem) rows
    TpOut tp_out;           // tensor-parallel exchange: outputs go to every rank's full buffer (world == 0: off)
    TpIn tp_in;             // ... the activations are another exchange's full buffer: wait for its flags first
    uint32_t off_xs, off_xzero, off_xmx, off_xscale, off_part, off_meta, off_ring;
    uint32_t xstride, stage_bytes, row_stride;
};

// Tensor-core kernels, one translation unit per code width (gemv_q4.cu, gemv_q8.cu).  They return
// B200Q_ERR_UNSUPPORTED when the problem does not fit their shared-memory plan.
int gemv_fast_q4(GemvParams& p, bool gate_up, cudaStream_t stream);
int gemv_fast_q8(GemvParams& p, bool gate_up, cudaStream_t stream);
int gemv_q4_read_status(int reset, cudaStream_t stream);
int gemv_q8_read_status(int reset, cudaStream_t stream);

// tcgen05 kernel (qgemm_ts.cu): weights through tensor memory, any batch up to 64 rows per launch.  Returns
// B200Q_ERR_UNSUPPORTED when the problem is outside its plan.
int qgemm_ts(int bits, const GemvParams& p, bool gate_up, cudaStream_t stream);
int qgemm_ts_read_status(int reset, cudaStream_t stream);

}  // namespace b200q
