// Quantized matvec / skinny GEMM for decode: host-side dispatch and the general kernel.
//
//   y[b, n] = sum_k x[b, k] * (code[n, k] - zero[n, k/G]) * scale[n, k/G]
//
// The tensor-core kernel (gemv_fast.cuh) serves group sizes 32 / 64 / 128 with 16-byte aligned rows
// and up to 16 batch rows per launch.  Everything else runs the general kernel below, which follows
// the reference arithmetic literally.
#include "gemv_params.cuh"

#include <algorithm>
#include <cmath>

namespace b200q {

// Defined in api.cu
int rmsnorm_residual_launch(const void* x, const void* residual, const void* weight, void* y, void* z_out,
                            int64_t rows, int64_t D, float eps, int dtype, int w_dtype, cudaStream_t stream);

int gemv_read_status(int reset, cudaStream_t stream) {
    const int a = gemv_q4_read_status(reset, stream);
    const int b = gemv_q8_read_status(reset, stream);
    const int c = qgemm_ts_read_status(reset, stream);
    return a != 0 ? a : (b != 0 ? b : c);
}

namespace {

__device__ __forceinline__ float round_act(float v, int dtype) {
    return dtype == B200Q_F16 ? __half2float(__float2half_rn(v)) : __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------------------------
// Generic kernel: any K / group size / alignment.  One warp per (output row), all batch rows.
// Follows the reference: W = cast(fp32(code - zero) * scale) in the activation dtype, fp32 sum.
// ---------------------------------------------------------------------------------------------
template <bool GATE_UP>
__global__ void __launch_bounds__(256) qgemv_generic_kernel(const __grid_constant__ GemvParams p, int bits) {
    constexpr int MATS = GATE_UP ? 2 : 1;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= p.N) return;
    const float fmax_act = p.act_dtype == B200Q_F16 ? 65504.0f : 3.3895313892515355e38f;
    for (int b = 0; b < p.B; ++b) {
        float acc[MATS];
#pragma unroll
        for (int m = 0; m < MATS; ++m) acc[m] = 0.0f;
        for (int k = lane; k < p.K; k += 32) {
            const float xv = load_as_f32(p.x, p.act_dtype, (int64_t)b * p.K + k);
            const int gi = min(k / p.G, p.Gn - 1);
#pragma unroll
            for (int m = 0; m < MATS; ++m) {
                float q;
                if (bits == 4) {
                    const uint8_t byte = p.w[m][row * p.row_bytes + (k >> 1)];
                    q = (float)((k & 1) ? (byte >> 4) : (byte & 0x0F));
                } else {
                    q = (float)p.w[m][row * p.row_bytes + k];
                }
                const float s = load_as_f32(p.s[m], p.scale_dtype, row * p.Gn + gi);
                float w = p.z[m] != nullptr
                              ? __fmul_rn(__fsub_rn(q, load_as_f32(p.z[m], p.scale_dtype, row * p.Gn + gi)), s)
                              : __fmul_rn(q, s);
                w = round_act(w, p.act_dtype);
                acc[m] = fmaf(xv, w, acc[m]);
            }
        }
        float val[MATS];
#pragma unroll
        for (int m = 0; m < MATS; ++m) {
            const float s = warp_sum(acc[m]);
            val[m] = round_act(fminf(fmaxf(s, -fmax_act), fmax_act), p.act_dtype);
        }
        if (lane == 0) {
            const int64_t o = (int64_t)b * p.N + row;
            auto store = [&](void* base, float v) {
                if (p.act_dtype == B200Q_F16) reinterpret_cast<__half*>(base)[o] = __float2half_rn(v);
                else reinterpret_cast<__nv_bfloat16*>(base)[o] = __float2bfloat16_rn(v);
            };
            if (GATE_UP) {
                if (p.gate_out != nullptr) store(p.gate_out, val[0]);
                if (p.up_out != nullptr) store(p.up_out, val[MATS - 1]);
                if (p.act_out != nullptr) {
                    const float silu = val[0] / (1.0f + expf(-val[0]));
                    store(p.act_out, silu * val[MATS - 1]);
                }
            } else {
                float v = val[0];
                if (p.residual != nullptr) v = load_as_f32(p.residual, p.act_dtype, o) + v;
                store(p.y, v);
            }
        }
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <bool GATE_UP>
int launch_generic(const GemvParams& p, int bits, cudaStream_t stream) {
    const int warps = 8;
    const int grid = (int)((p.N + warps - 1) / warps);
    qgemv_generic_kernel<GATE_UP><<<grid, warps * 32, 0, stream>>>(p, bits);
    return finish_launch();
}

// The general kernel has no norm prologue: the caller runs the stand-alone rmsnorm kernel first when
// the tensor-core kernel does not apply.
bool fast_path_ok(const GemvParams& p) {
    if (tuning_get("gemv.force_generic")) return false;
    if (p.G != 32 && p.G != 64 && p.G != 128) return false;
    if (p.K % p.G != 0 || p.row_bytes % 16 != 0) return false;
    if (p.B > 64) return false;
    if (!aligned16(p.x) || !aligned16(p.w[0]) || (p.w[1] != nullptr && !aligned16(p.w[1]))) return false;
    if (p.res_in != nullptr && !aligned16(p.res_in)) return false;
    if (p.z_out != nullptr && !aligned16(p.z_out)) return false;
    if (p.normed_out != nullptr && !aligned16(p.normed_out)) return false;
    return true;
}

// Which kernel takes a launch: "gemv.ts" = 1 sends everything the tcgen05 kernel supports to it, -1 nothing,
// 0 (default) the batches of gemv.ts_min_batch rows and more (default 5: measured crossover at the Llama-3-8B
// shapes, where the mma.sync kernel pays its per-group affine step once per batch row tile).
bool prefer_ts(const GemvParams& p) {
    const int mode = tuning_get("gemv.ts");
    if (mode < 0) return false;
    if (mode > 0) return true;
    int min_b = tuning_get("gemv.ts_min_batch");
    if (min_b <= 0) min_b = 5;
    return p.B >= min_b;
}

// The rmsnorm prologue costs the tcgen05 kernel's activation warps more than a launch of the row kernel (measured,
// 4096 -> 2 x 14336: at batch 32 56 us fused against 33 + 3 us, at batch 8 40 us against 30 + 3 us), so when the caller
// provides the buffer for the normalised rows they are materialised first.
int split_norm_prologue(GemvParams& p, cudaStream_t stream) {
    if (p.norm_w == nullptr || p.normed_out == nullptr || !prefer_ts(p) || tuning_get("gemv.fuse_norm") > 0) return B200Q_OK;
    const int rc = rmsnorm_residual_launch(p.x, p.res_in, p.norm_w, p.normed_out, p.z_out, p.B, p.K, p.eps, p.act_dtype,
                                           p.norm_w_dtype, stream);
    if (rc != B200Q_OK) return rc;
    p.x = p.normed_out;
    p.norm_w = nullptr; p.res_in = nullptr; p.z_out = nullptr; p.normed_out = nullptr;
    return B200Q_OK;
}

int dispatch_fast(int bits, GemvParams& p, bool gate_up, cudaStream_t stream) {
    if (prefer_ts(p)) {
        const int rc = qgemm_ts(bits, p, gate_up, stream);
        if (rc != B200Q_ERR_UNSUPPORTED) return rc;
    }
    if (p.B > 16) return B200Q_ERR_UNSUPPORTED;
    return bits == 4 ? gemv_fast_q4(p, gate_up, stream) : gemv_fast_q8(p, gate_up, stream);
}

}  // namespace


int qmatvec_impl(int bits, const void* x, const uint8_t* codes, const void* scales, const void* zeros,
                 const void* residual, void* y, int B, int64_t N, int64_t K, int group_size, int act_dtype,
                 int scale_dtype, const void* residual_in, const void* norm_weight, int norm_w_dtype, float eps,
                 void* z_out, void* normed_out, cudaStream_t stream) {
    int tp_in_slot = -1, tp_out_slot = -1;
    tp_take(&tp_in_slot, &tp_out_slot);
    if ((bits != 4 && bits != 8) || x == nullptr || codes == nullptr || scales == nullptr ||
        (y == nullptr && tp_out_slot < 0))
        return B200Q_ERR_BAD_ARG;
    if ((tp_in_slot >= 0 || tp_out_slot >= 0) && B > 16) return B200Q_ERR_UNSUPPORTED;
    if (B <= 0 || N <= 0 || K <= 0 || group_size <= 0 || !is_act_dtype(act_dtype) || !is_scale_dtype(scale_dtype))
        return B200Q_ERR_BAD_ARG;
    if (norm_weight != nullptr && !is_scale_dtype(norm_w_dtype)) return B200Q_ERR_BAD_ARG;
    if (norm_weight == nullptr && (residual_in != nullptr || z_out != nullptr || normed_out != nullptr))
        return B200Q_ERR_BAD_ARG;
    if (N > INT32_MAX || K > INT32_MAX) return B200Q_ERR_UNSUPPORTED;
    const int esz = 2;
    auto off = [&](const void* base, size_t elems) -> const uint8_t* {
        return base ? reinterpret_cast<const uint8_t*>(base) + elems * esz : nullptr;
    };
    auto offw = [&](void* base, size_t elems) -> uint8_t* {
        return base ? reinterpret_cast<uint8_t*>(base) + elems * esz : nullptr;
    };
    int chunk = 64;      // batch rows per launch; halved when the kernels' shared-memory plans do not fit
    for (int b0 = 0; b0 < B;) {
        GemvParams p = {};
        const int bn = std::min(chunk, B - b0);
        p.x = off(x, (size_t)b0 * K);
        p.res_in = off(residual_in, (size_t)b0 * K);
        p.norm_w = norm_weight; p.eps = eps; p.norm_w_dtype = norm_w_dtype;
        p.z_out = offw(z_out, (size_t)b0 * K);
        p.normed_out = offw(normed_out, (size_t)b0 * K);
        p.w[0] = codes; p.s[0] = scales; p.z[0] = zeros;
        p.residual = off(residual, (size_t)b0 * N);
        p.y = offw(y, (size_t)b0 * N);
        p.B = bn; p.N = (int)N; p.K = (int)K; p.G = group_size; p.Gn = (int)((K + group_size - 1) / group_size);
        p.act_dtype = act_dtype; p.scale_dtype = scale_dtype;
        p.row_bytes = bits == 4 ? (int)((K + 1) / 2) : (int)K;
        if (tp_out_slot >= 0) p.tp_out = tp_slot(tp_out_slot)->out;
        if (tp_in_slot >= 0) {
            const TpOut& src = tp_slot(tp_in_slot)->out;
            p.tp_in.flags = src.flags[src.rank];
            p.tp_in.epoch = src.epoch;
            p.tp_in.world = src.world;
            p.tp_in.spin_limit = (uint32_t)std::max(0, tuning_get("tp.spin_limit"));
            p.tp_in.packets = src.packets;
        }
        const bool tp_used = tp_in_slot >= 0 || tp_out_slot >= 0;
        if (!tp_used && fast_path_ok(p)) {
            const int nrc = split_norm_prologue(p, stream);
            if (nrc != B200Q_OK) return nrc;
        }
        int rc = fast_path_ok(p) ? dispatch_fast(bits, p, false, stream) : B200Q_ERR_UNSUPPORTED;
        if (rc == B200Q_ERR_UNSUPPORTED && tp_used) return rc;      // exchanges exist only in the tensor-core kernel
        if (rc == B200Q_ERR_UNSUPPORTED && bn > 1 && fast_path_ok(p)) {
            chunk = (bn + 1) / 2;
            continue;
        }
        if (rc == B200Q_ERR_UNSUPPORTED) {
            if (norm_weight != nullptr) {
                // generic route: materialise the normalised rows first (normed_out is required as the buffer)
                if (p.normed_out == nullptr) return B200Q_ERR_UNSUPPORTED;
                rc = rmsnorm_residual_launch(p.x, p.res_in, norm_weight, p.normed_out, p.z_out, bn, K, eps, act_dtype,
                                             norm_w_dtype, stream);
                if (rc != B200Q_OK) return rc;
                p.x = p.normed_out;
                p.norm_w = nullptr; p.res_in = nullptr; p.z_out = nullptr; p.normed_out = nullptr;
            }
            rc = launch_generic<false>(p, bits, stream);
        }
        if (rc != B200Q_OK) return rc;
        b0 += bn;
    }
    return B200Q_OK;
}

int gate_up_impl(int bits, const void* x, const uint8_t* gate_codes, const uint8_t* up_codes, const void* gate_scales,
                 const void* up_scales, const void* gate_zeros, const void* up_zeros, void* gate_out, void* up_out,
                 void* act_out, const void* residual_in, const void* norm_weight, float eps, void* z_out,
                 void* normed_out, int rows, int64_t N, int64_t K, int group_size, int act_dtype, int scale_dtype,
                 int norm_w_dtype, cudaStream_t stream) {
    int tp_in_slot = -1, tp_out_slot = -1;
    tp_take(&tp_in_slot, &tp_out_slot);
    if ((bits != 4 && bits != 8) || x == nullptr || gate_codes == nullptr || up_codes == nullptr ||
        gate_scales == nullptr || up_scales == nullptr)
        return B200Q_ERR_BAD_ARG;
    if ((tp_in_slot >= 0 || tp_out_slot >= 0) && rows > 16) return B200Q_ERR_UNSUPPORTED;
    if (rows <= 0 || N <= 0 || K <= 0 || group_size <= 0 || !is_act_dtype(act_dtype) || !is_scale_dtype(scale_dtype))
        return B200Q_ERR_BAD_ARG;
    if (norm_weight != nullptr && !is_scale_dtype(norm_w_dtype)) return B200Q_ERR_BAD_ARG;
    if (norm_weight == nullptr && (residual_in != nullptr || z_out != nullptr || normed_out != nullptr))
        return B200Q_ERR_BAD_ARG;
    if (N > INT32_MAX || K > INT32_MAX) return B200Q_ERR_UNSUPPORTED;
    const int esz = 2;
    auto off = [&](const void* base, size_t elems) -> const uint8_t* {
        return base ? reinterpret_cast<const uint8_t*>(base) + elems * esz : nullptr;
    };
    auto offw = [&](void* base, size_t elems) -> uint8_t* {
        return base ? reinterpret_cast<uint8_t*>(base) + elems * esz : nullptr;
    };
    int chunk = 64;      // batch rows per launch; halved when the kernels' shared-memory plans do not fit
    for (int b0 = 0; b0 < rows;) {
        GemvParams p = {};
        const int bn = std::min(chunk, rows - b0);
        p.x = off(x, (size_t)b0 * K);
        p.res_in = off(residual_in, (size_t)b0 * K);
        p.norm_w = norm_weight; p.eps = eps; p.norm_w_dtype = norm_w_dtype;
        p.z_out = offw(z_out, (size_t)b0 * K);
        p.normed_out = offw(normed_out, (size_t)b0 * K);
        p.w[0] = gate_codes; p.w[1] = up_codes;
        p.s[0] = gate_scales; p.s[1] = up_scales;
        p.z[0] = gate_zeros; p.z[1] = up_zeros;
        p.gate_out = offw(gate_out, (size_t)b0 * N);
        p.up_out = offw(up_out, (size_t)b0 * N);
        p.act_out = offw(act_out, (size_t)b0 * N);
        p.B = bn; p.N = (int)N; p.K = (int)K; p.G = group_size; p.Gn = (int)((K + group_size - 1) / group_size);
        p.act_dtype = act_dtype; p.scale_dtype = scale_dtype;
        p.row_bytes = bits == 4 ? (int)((K + 1) / 2) : (int)K;
        if (tp_out_slot >= 0) p.tp_out = tp_slot(tp_out_slot)->out;
        if (tp_in_slot >= 0) {
            const TpOut& src = tp_slot(tp_in_slot)->out;
            p.tp_in.flags = src.flags[src.rank];
            p.tp_in.epoch = src.epoch;
            p.tp_in.world = src.world;
            p.tp_in.spin_limit = (uint32_t)std::max(0, tuning_get("tp.spin_limit"));
            p.tp_in.packets = src.packets;
        }
        const bool tp_used = tp_in_slot >= 0 || tp_out_slot >= 0;
        if (!tp_used && fast_path_ok(p)) {
            const int nrc = split_norm_prologue(p, stream);
            if (nrc != B200Q_OK) return nrc;
        }
        int rc;
        rc = fast_path_ok(p) ? dispatch_fast(bits, p, true, stream) : B200Q_ERR_UNSUPPORTED;
        if (rc == B200Q_ERR_UNSUPPORTED && tp_used) return rc;      // exchanges exist only in the tensor-core kernel
        if (rc == B200Q_ERR_UNSUPPORTED && bn > 1 && fast_path_ok(p)) {
            chunk = (bn + 1) / 2;
            continue;
        }
        if (rc == B200Q_ERR_UNSUPPORTED) {
            if (norm_weight != nullptr) {
                // generic route: materialise the normalised rows first (normed_out is required as the buffer)
                if (p.normed_out == nullptr) return B200Q_ERR_UNSUPPORTED;
                rc = rmsnorm_residual_launch(p.x, p.res_in, norm_weight, p.normed_out, p.z_out, bn, K, eps, act_dtype,
                                             norm_w_dtype, stream);
                if (rc != B200Q_OK) return rc;
                p.x = p.normed_out;
                p.norm_w = nullptr; p.res_in = nullptr; p.z_out = nullptr; p.normed_out = nullptr;
            }
            rc = launch_generic<true>(p, bits, stream);
        }
        if (rc != B200Q_OK) return rc;
        b0 += bn;
    }
    return B200Q_OK;
}

}  // namespace b200q
