// Weight-streaming quantized matvec / skinny GEMM for decode (sm_100a): the tensor-core kernel.
//
//   y[b, n] = sum_k x[b, k] * (code[n, k] - zero[n, k/G]) * scale[n, k/G]          b < B <= 16
//
// Design (one CTA per SM: 16 consumer warps, one producer warp, one epilogue warp):
//   * output rows are dealt out evenly to the CTAs; a CTA walks its rows in tiles of 16 (one
//     tensor-core M tile).
//   * the producer warp streams each tile through a ring of shared-memory stages with 1-D bulk
//     copies (TMA engine) signalled on mbarriers: one copy per weight row and k-chunk, sized
//     about 2 KB because the copy engine needs >= 2 KB per copy to saturate HBM.  It starts
//     before griddepcontrol.wait: weights do not depend on the previous kernel.
//   * the codes are NOT dequantised.  OR-ing a code into the mantissa of 1024.0 (or 64.0 for the
//     high nibbles) gives the exact half 1024 + q, which goes straight into mma.sync.m16n8k16 as
//     the A operand (16 output rows); the tensor core then produces, per quantisation group,
//         c = sum_k (off_k + q_k) x_k            (fp32)
//     and the affine part is applied once per group in fp32:
//         y += scale * (c - M - zero * X),   M = sum_k off_k x_k,   X = sum_k x_k
//     with M and X precomputed per group from the activations.  Nothing about the weights is
//     rounded, so the result is closer to exact arithmetic than a dequantise-to-fp16 kernel.
//   * the 8 columns of the tensor-core tile hold (quantisation group, batch row) pairs: with one
//     batch row, 8 consecutive groups accumulate side by side in one accumulator and the per-group
//     step above runs once per 8 groups; with 8 batch rows it runs once per group.  A lane's B
//     operand is the activation slice of its column's group, or zeros for the other groups.
//   * work unit = 16 rows x 8 groups; units are dealt round-robin to the 16 consumer warps, which
//     add their results into private shared-memory slots.  The epilogue warp sums the 16 slots in a
//     fixed order (bitwise reproducible), clamps, rounds, applies residual add or SwiGLU, stores.
//   * optional prologue: x := rmsnorm(x + residual) recomputed by every CTA from L2.
//
// This header is compiled into one translation unit per code width.
#pragma once

#include "gemv_params.cuh"

#include <algorithm>
#include <cmath>

namespace b200q {
namespace {

// ---- activation source: 8 consecutive values of batch row b at k, as the reference would hold them --------
__device__ __forceinline__ void load8_raw(const void* base, int dtype, int64_t idx, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + idx);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (dtype == B200Q_F16) {
            const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            v[2 * i] = __low2float(h);
            v[2 * i + 1] = __high2float(h);
        } else {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
}
__device__ __forceinline__ float round_act(float v, int dtype) {
    return dtype == B200Q_F16 ? __half2float(__float2half_rn(v)) : __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ void store8_act(void* base, int dtype, int64_t idx, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (dtype == B200Q_F16) {
            const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        } else {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
}
// z = cast(x + res) (res optional)
__device__ __forceinline__ void load8_z(const GemvParams& p, int b, int k, float (&zv)[8]) {
    load8_raw(p.x, p.act_dtype, (int64_t)b * p.K + k, zv);
    if (p.res_in != nullptr) {
        float r[8];
        load8_raw(p.res_in, p.act_dtype, (int64_t)b * p.K + k, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) zv[i] = round_act(zv[i] + r[i], p.act_dtype);
    }
}
// the activation row the matvec sees: x itself, or cast(z * inv_rms * w)
__device__ __forceinline__ void load8_act(const GemvParams& p, int b, int k, float inv_rms, bool write_side, float (&v)[8]) {
    if (p.norm_w == nullptr) {
        load8_raw(p.x, p.act_dtype, (int64_t)b * p.K + k, v);
        return;
    }
    float zv[8];
    load8_z(p, b, k, zv);
    if (write_side && p.z_out != nullptr) store8_act(p.z_out, p.act_dtype, (int64_t)b * p.K + k, zv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float w = load_as_f32(p.norm_w, p.norm_w_dtype, k + i);
        v[i] = round_act(zv[i] * inv_rms * w, p.act_dtype);
    }
    if (write_side && p.normed_out != nullptr) store8_act(p.normed_out, p.act_dtype, (int64_t)b * p.K + k, v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

template <int NWORDS>
__device__ __forceinline__ void load_words(const uint8_t* ptr, uint32_t (&w)[NWORDS]) {
    if constexpr (NWORDS == 1) {
        w[0] = *reinterpret_cast<const uint32_t*>(ptr);
    } else if constexpr (NWORDS == 2) {
        const uint2 u = *reinterpret_cast<const uint2*>(ptr);
        w[0] = u.x; w[1] = u.y;
    } else {
#pragma unroll
        for (int i = 0; i < NWORDS / 4; ++i) {
            const uint4 u = *reinterpret_cast<const uint4*>(ptr + 16 * i);
            w[4 * i] = u.x; w[4 * i + 1] = u.y; w[4 * i + 2] = u.z; w[4 * i + 3] = u.w;
        }
    }
}

__device__ __forceinline__ float half_lo(uint32_t u) { return __half2float(__ushort_as_half((unsigned short)(u & 0xFFFFu))); }
__device__ __forceinline__ float half_hi(uint32_t u) { return __half2float(__ushort_as_half((unsigned short)(u >> 16))); }

// BITS: code width.  LOGG: log2(group size) in {5, 6, 7}.  NB: tensor-core columns per quantisation group
// (batch rows rounded up to 1, 2, 4, 8).  NT: column tiles (2 only with NB == 8: 9..16 batch rows).
template <int BITS, int LOGG, int NB, int NT, bool GATE_UP>
__global__ void __launch_bounds__(kThreads, 1) qgemv_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MATS = GATE_UP ? 2 : 1;
    constexpr int G = 1 << LOGG;
    constexpr int GB = G * BITS / 8;              // bytes of one group in one weight row
    constexpr int LB = GB / 4;                    // bytes a lane holds per row and group
    constexpr int NW = LB / 4;                    // ... as 32-bit words
    constexpr int XB = G / 2;                     // activation bytes per lane and group (G/4 halves)
    constexpr int UK = kUnitGroups * G;           // k per unit
    constexpr int NP = NB;                        // passes over a unit
    constexpr int GS = kUnitGroups / NB;          // groups side by side in one accumulator
    constexpr int BC = NB * NT;                   // batch columns kept per row
    constexpr int MW = (NB < 2 ? 2 : NB) / 2;     // 32-bit words of scales (and of zeros) per lane and row
    constexpr float OFF_ODD = BITS == 4 ? 64.0f : 1024.0f;
    static_assert(NT == 1 || NB == 8, "two column tiles only with eight batch columns per group");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    uint64_t* tile_done = empty + kMaxStages;      // [kMaxSlots] all consumer warps have added their share
    uint64_t* slot_free = tile_done + kMaxSlots;   // [kMaxSlots] the epilogue has read (and zeroed) the slot

    const int cta = blockIdx.x;
    const int r_lo = cta * p.rows_lo + min(cta, p.rem);
    const int r_cnt = p.rows_lo + (cta < p.rem ? 1 : 0);
    const int r_hi = r_lo + r_cnt;
    const int n_tiles = (r_cnt + kTileRows - 1) / kTileRows;
    const int n_xc = p.n_xc;
    const int cpx = p.xk / p.kc;                   // stages per (matrix, tile, activation chunk)
    const int nslot = p.nslot;
    const int B = p.B;

    float* part = reinterpret_cast<float*>(smem + p.off_part);     // [nslot][MATS][16 warps][16 rows][BC]
    uint8_t* xzero = smem + p.off_xzero;
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        for (int s = 0; s < kMaxSlots; ++s) {
            mbar_init(&tile_done[s], kConsumerWarps);
            mbar_init(&slot_free[s], 1);
        }
        mbar_fence_init();
    }
    for (int i = threadIdx.x; i < nslot * MATS * kConsumerWarps * kTileRows * BC; i += kThreads) part[i] = 0.0f;
    for (int i = threadIdx.x; i < UK * 2 / 4; i += kThreads) reinterpret_cast<uint32_t*>(xzero)[i] = 0u;
    __syncthreads();
    pdl_launch_dependents();

    uint8_t* ring = smem + p.off_ring;

    // Producer and consumers walk the stages in the same order: activation chunk, tile, matrix, k-chunk.
    if (warp == kProducerWarp) {
        bool ok = true;
        int slot = 0;
        uint32_t phase = 1;
        bool first_pass = true;
        for (int xc = 0; xc < n_xc; ++xc) {
            const int c_begin = xc * cpx;
            const int c_end = min(p.n_kc, c_begin + cpx);
            for (int tl = 0; tl < n_tiles; ++tl) {
                const int row0 = r_lo + tl * kTileRows;
                const int rows = min(kTileRows, r_hi - row0);
                for (int m = 0; m < MATS; ++m) {
                    for (int c = c_begin; c < c_end; ++c) {
                        if (!first_pass)
                            ok = mbar_wait_bounded(&empty[slot], phase, &g_device_status, EV_GEMV_EMPTY_WAIT,
                                                   ok ? kWaitLimit : 64u) && ok;
                        const int k0 = c * p.kc;
                        const int kcur = min(p.kc, p.K - k0);
                        const uint32_t bytes_row = (uint32_t)(kcur * BITS / 8);
                        uint8_t* stage = ring + (size_t)slot * p.stage_bytes;
                        if (lane == 0) mbar_arrive_expect_tx(&full[slot], bytes_row * rows);
                        __syncwarp();
                        if (lane < rows) {
                            const uint8_t* src = ((MATS == 2 && m != 0) ? p.w[1] : p.w[0]) + (size_t)(row0 + lane) * p.row_bytes + (size_t)k0 * BITS / 8;
                            bulk_g2s(stage + (size_t)lane * p.row_stride, src, bytes_row, &full[slot]);
                        }
                        if (++slot == p.stages) { slot = 0; phase ^= 1; first_pass = false; }
                    }
                }
            }
        }
        return;
    }

    const float fmax_act = p.act_dtype == B200Q_F16 ? 65504.0f : 3.3895313892515355e38f;
    const bool need_row_pass = (p.norm_w != nullptr) || (p.act_dtype == B200Q_BF16);
    float* xscale = reinterpret_cast<float*>(smem + p.off_xscale);    // [B]: 2^e ; [B..2B): inv_rms

    if (warp == kEpilogueWarp) {
        // ------------------------------ epilogue warp ------------------------------------------
        pdl_wait();   // the output buffers may still be read by the previous kernel
        bool ok = true;
        for (int tl = 0; tl < n_tiles; ++tl) {
            const int ps = tl % nslot;
            ok = mbar_wait_bounded(&tile_done[ps], (uint32_t)(tl / nslot) & 1u, &g_device_status, EV_GEMV_FULL_WAIT,
                                   ok ? kWaitLimit : 64u) && ok;
            const int row0 = r_lo + tl * kTileRows;
            const int rows = min(kTileRows, r_hi - row0);
            float* slot_base = part + (size_t)ps * MATS * kConsumerWarps * kTileRows * BC;
            for (int it = lane; it < kTileRows * BC; it += 32) {
                const int r = it & (kTileRows - 1);
                const int b = it >> 4;
                float val[MATS];
#pragma unroll
                for (int m = 0; m < MATS; ++m) {
                    float* src = slot_base + ((size_t)m * kConsumerWarps * kTileRows + r) * BC + b;
                    float s = 0.0f;
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; ++w) {
                        s += src[w * kTileRows * BC];
                        src[w * kTileRows * BC] = 0.0f;
                    }
                    if (need_row_pass && b < B) s *= xscale[b];
                    val[m] = round_act(fminf(fmaxf(s, -fmax_act), fmax_act), p.act_dtype);
                }
                if (r < rows && b < B) {
                    const int64_t o = (int64_t)b * p.N + row0 + r;
                    auto store = [&](void* basep, float v) {
                        if (p.act_dtype == B200Q_F16) reinterpret_cast<__half*>(basep)[o] = __float2half_rn(v);
                        else reinterpret_cast<__nv_bfloat16*>(basep)[o] = __float2bfloat16_rn(v);
                    };
                    if (GATE_UP) {
                        if (p.gate_out != nullptr) store(p.gate_out, val[0]);
                        if (p.up_out != nullptr) store(p.up_out, val[MATS - 1]);
                        if (p.act_out != nullptr) {
                            const float gte = val[0];
                            const float silu = gte / (1.0f + expf(-gte));
                            store(p.act_out, silu * val[MATS - 1]);
                        }
                    } else {
                        float v = val[0];
                        if (p.residual != nullptr) v = load_as_f32(p.residual, p.act_dtype, o) + v;
                        store(p.y, v);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&slot_free[ps]);
        }
        return;
    }

    // ---------------------------------- consumer warps -----------------------------------------
    const int cw = warp;
    const int ctid = threadIdx.x;               // 0 .. kConsumerThreads-1
    const int g = lane >> 2;
    const int t = lane & 3;
    const int Gn = p.Gn;

    uint8_t* xs = smem + p.off_xs;                                    // [B] rows of xstride bytes, fp16, operand order
    float2* xmx = reinterpret_cast<float2*>(smem + p.off_xmx);        // [groups of the chunk (+ padding)][BC] {M, X}

    pdl_wait();   // activations belong to the previous kernel until here

    // per batch row: inv_rms (norm prologue) and the power of two that maps bf16 rows into fp16 range
    if (need_row_pass) {
        for (int b = cw; b < B; b += kConsumerWarps) {
            float inv = 1.0f;
            if (p.norm_w != nullptr) {
                float ss = 0.0f;
                for (int k = lane * 8; k < p.K; k += 256) {
                    float zv[8];
                    load8_z(p, b, k, zv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss += zv[i] * zv[i];
                }
                ss = warp_sum(ss);
                inv = rsqrtf(ss / (float)p.K + p.eps);
            }
            float sc = 1.0f;
            if (p.act_dtype == B200Q_BF16) {
                float mx = 0.0f;
                for (int k = lane * 8; k < p.K; k += 256) {
                    float v[8];
                    load8_act(p, b, k, inv, false, v);
#pragma unroll
                    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(v[i]));
                }
                mx = warp_max(mx);
                int ex = 0;
                if (mx > 0.0f && mx < INFINITY) frexpf(mx, &ex);
                ex = max(-100, min(114, ex - 14));
                sc = exp2f((float)ex);
            }
            if (lane == 0) {
                xscale[b] = sc;
                xscale[B + b] = inv;
            }
        }
        named_bar_sync(1, kConsumerThreads);
    }

    // ---- stage activations of [xk0, xk0+xkn) as fp16 in tensor-core operand order, then per-group sums ----
    auto stage_x = [&](int xk0, int xkn, bool write_side) {
        const int chunks = xkn / 8;
#pragma unroll 2
        for (int i = ctid; i < B * chunks; i += kConsumerThreads) {
            const int b = i / chunks;
            const int kk = (i - b * chunks) * 8;
            float v[8];
            const float inv = need_row_pass ? xscale[B + b] : 1.0f;
            const float down = need_row_pass ? 1.0f / xscale[b] : 1.0f;
            load8_act(p, b, xk0 + kk, inv, write_side, v);
            __half h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(v[j] * down);
            uint4 out;
            if (BITS == 4) {
                // order of the codes of one weight word as the tensor core sees them: (0,4) (1,5) (2,6) (3,7)
                out.x = __half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[4]) << 16);
                out.y = __half_as_ushort(h[1]) | ((uint32_t)__half_as_ushort(h[5]) << 16);
                out.z = __half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[6]) << 16);
                out.w = __half_as_ushort(h[3]) | ((uint32_t)__half_as_ushort(h[7]) << 16);
            } else {
                out.x = __half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
                out.y = __half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
                out.z = __half_as_ushort(h[4]) | ((uint32_t)__half_as_ushort(h[5]) << 16);
                out.w = __half_as_ushort(h[6]) | ((uint32_t)__half_as_ushort(h[7]) << 16);
            }
            *reinterpret_cast<uint4*>(xs + (size_t)b * p.xstride + (size_t)kk * 2) = out;
        }
        named_bar_sync(1, kConsumerThreads);
        // {M, X} per (group, batch column): X = sum of the group's activations, M = sum of offset * activation
        // (offset 1024 for low nibbles / bytes, 64 for high nibbles); zeros for padding groups and columns.
        const int gc = xkn >> LOGG;
        const int gpad = (gc + kUnitGroups - 1) / kUnitGroups * kUnitGroups;
        for (int i = ctid; i < gpad * BC; i += kConsumerThreads) {
            const int gi = i / BC;
            const int b = i - gi * BC;
            float se = 0.0f, so = 0.0f;
            if (gi < gc && b < B) {
                const uint8_t* src = xs + (size_t)b * p.xstride + (size_t)(gi << LOGG) * 2;
#pragma unroll
                for (int j = 0; j < G / 8; ++j) {
                    const uint4 u = *reinterpret_cast<const uint4*>(src + 16 * j);
                    const __half2 h0 = *reinterpret_cast<const __half2*>(&u.x);
                    const __half2 h1 = *reinterpret_cast<const __half2*>(&u.y);
                    const __half2 h2 = *reinterpret_cast<const __half2*>(&u.z);
                    const __half2 h3 = *reinterpret_cast<const __half2*>(&u.w);
                    const float a0 = __low2float(h0) + __high2float(h0), a1 = __low2float(h1) + __high2float(h1);
                    const float a2 = __low2float(h2) + __high2float(h2), a3 = __low2float(h3) + __high2float(h3);
                    if (BITS == 4) {            // words 0 and 2 hold even k, 1 and 3 odd k
                        se += a0 + a2;
                        so += a1 + a3;
                    } else {
                        se += (a0 + a1) + (a2 + a3);
                    }
                }
            }
            xmx[i] = make_float2(1024.0f * se + OFF_ODD * so, se + so);
        }
        named_bar_sync(1, kConsumerThreads);
    };

    // ---- this warp's units: global unit number = stage number * nu + index in stage, dealt modulo 16 ----
    struct Unit { int S, i, tl, m, c; bool valid; };
    struct Meta { uint32_t s[2][MW], z[2][MW]; };
    const int NU = p.nu;

    bool ok = true;
    int c_slot = 0;
    uint32_t c_phase = 0;
    uint32_t ph16 = 0;                          // (units before the current activation chunk) mod 16

    // column bookkeeping of this lane: as B operand it feeds column g, as accumulator owner columns 2t, 2t+1
    const int my_js = g / NB;                   // group slot of column g within a pass
    const int my_b = g % NB;                    // batch row of column g (first column tile)
    const int goff = NB <= 2 ? 2 * t : (NB == 4 ? 4 * (t >> 1) : 0);   // first group of this lane's scale words

#pragma unroll 1
    for (int xc = 0; xc < n_xc; ++xc) {
        const int xk0 = xc * p.xk;
        const int xkn = min(p.xk, p.K - xk0);
        if (xc > 0) named_bar_sync(1, kConsumerThreads);     // everyone is done with the previous chunk
        stage_x(xk0, xkn, cta == 0);

        const int c_begin = xc * cpx;
        const int c_end = min(p.n_kc, c_begin + cpx);
        const int nS = n_tiles * MATS * (c_end - c_begin);

        auto units_in = [&](int c) { return (min(p.kc, p.K - c * p.kc) + UK - 1) / UK; };
        auto normalize = [&](Unit& u) {
            for (;;) {
                while (u.i >= NU) {
                    u.i -= NU;
                    ++u.S;
                    if (++u.c == c_end) {
                        u.c = c_begin;
                        if (++u.m == MATS) { u.m = 0; ++u.tl; }
                    }
                }
                if (u.S >= nS) { u.valid = false; return; }
                if (u.i < units_in(u.c)) { u.valid = true; return; }
                u.i += 16;
            }
        };
        auto load_meta = [&](const Unit& u, Meta& mt) {
            const int gi0 = (u.c * p.kc + u.i * UK) >> LOGG;           // first group of the unit
            const void* sp = (MATS == 2 && u.m != 0) ? p.s[1] : p.s[0];
            const void* zp = (MATS == 2 && u.m != 0) ? p.z[1] : p.z[0];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = min(r_lo + u.tl * kTileRows + g + 8 * rr, p.N - 1);
                const int64_t e = (int64_t)row * Gn + gi0 + goff;
                if (p.meta_vec && gi0 + kUnitGroups <= Gn) {
                    const __half* sh = reinterpret_cast<const __half*>(sp) + e;
                    const __half* zh = reinterpret_cast<const __half*>(zp) + e;
                    if constexpr (MW == 1) {
                        mt.s[rr][0] = __ldg(reinterpret_cast<const uint32_t*>(sh));
                        mt.z[rr][0] = zp != nullptr ? __ldg(reinterpret_cast<const uint32_t*>(zh)) : 0u;
                    } else if constexpr (MW == 2) {
                        const uint2 a = __ldg(reinterpret_cast<const uint2*>(sh));
                        mt.s[rr][0] = a.x; mt.s[rr][1] = a.y;
                        uint2 c2 = make_uint2(0u, 0u);
                        if (zp != nullptr) c2 = __ldg(reinterpret_cast<const uint2*>(zh));
                        mt.z[rr][0] = c2.x; mt.z[rr][1] = c2.y;
                    } else {
                        const uint4 a = __ldg(reinterpret_cast<const uint4*>(sh));
                        mt.s[rr][0] = a.x; mt.s[rr][1] = a.y; mt.s[rr][2] = a.z; mt.s[rr][3] = a.w;
                        uint4 c4 = make_uint4(0u, 0u, 0u, 0u);
                        if (zp != nullptr) c4 = __ldg(reinterpret_cast<const uint4*>(zh));
                        mt.z[rr][0] = c4.x; mt.z[rr][1] = c4.y; mt.z[rr][2] = c4.z; mt.z[rr][3] = c4.w;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < MW; ++j) {
                        uint32_t sw = 0u, zw = 0u;
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int gidx = gi0 + goff + 2 * j + hh;
                            if (gidx < Gn) {
                                const int64_t ee = (int64_t)row * Gn + gidx;
                                sw |= (uint32_t)__half_as_ushort(__float2half_rn(load_as_f32(sp, p.scale_dtype, ee))) << (16 * hh);
                                if (zp != nullptr)
                                    zw |= (uint32_t)__half_as_ushort(__float2half_rn(load_as_f32(zp, p.scale_dtype, ee))) << (16 * hh);
                            }
                        }
                        mt.s[rr][j] = sw;
                        mt.z[rr][j] = zw;
                    }
                }
            }
        };

        // ---- one unit: 16 rows x 8 groups of stage `slot` ----
        auto process_unit = [&](int slot, const Unit& u, const Meta& mt, int ps) {
            const int k_in_stage = u.i * UK;
            const int kcur = min(p.kc, p.K - u.c * p.kc);
            const int ng = min(kUnitGroups, (kcur - k_in_stage) >> LOGG);
            const uint8_t* aw = ring + (size_t)slot * p.stage_bytes + (size_t)g * p.row_stride + (size_t)u.i * (kUnitGroups * GB) + t * LB;
            const uint8_t* aw8 = aw + (size_t)8 * p.row_stride;
            const int kl = u.c * p.kc + k_in_stage - xk0;                 // k of the unit inside the staged activations
            const int gi = kl >> LOGG;
            const uint8_t* xz = xzero + t * XB;
            const uint8_t* xrow[NT];
            bool bvalid[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int b = nt * 8 + my_b;
                bvalid[nt] = b < B;
                xrow[nt] = xs + (size_t)min(b, B - 1) * p.xstride + (size_t)kl * 2 + t * XB;
            }
            float y[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) y[nt][i] = 0.0f;

#pragma unroll
            for (int pass = 0; pass < NP; ++pass) {
                float acc[NT][2][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int a = 0; a < 2; ++a)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[nt][a][i] = 0.0f;
#pragma unroll
                for (int js = 0; js < GS; ++js) {
                    const int gl = js * NP + pass;               // group of the unit handled by slot js in this pass
                    if (gl < ng) {
                        uint32_t wa[NW], wb[NW];
                        load_words<NW>(aw + gl * GB, wa);
                        load_words<NW>(aw8 + gl * GB, wb);
                        const uint8_t* xb[NT];
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) xb[nt] = ((my_js == js && bvalid[nt]) ? xrow[nt] : xz) + gl * (G * 2);
                        if constexpr (BITS == 4) {
#pragma unroll
                            for (int wd = 0; wd < NW; ++wd) {
                                const uint32_t a_lo = wa[wd], b_lo = wb[wd];
                                const uint32_t a_hi = a_lo >> 8, b_hi = b_lo >> 8;
                                const uint32_t aL0 = lop3_and_or(a_lo, 0x000F000Fu, 0x64006400u), aH0 = lop3_and_or(a_lo, 0x00F000F0u, 0x54005400u);
                                const uint32_t bL0 = lop3_and_or(b_lo, 0x000F000Fu, 0x64006400u), bH0 = lop3_and_or(b_lo, 0x00F000F0u, 0x54005400u);
                                const uint32_t aL1 = lop3_and_or(a_hi, 0x000F000Fu, 0x64006400u), aH1 = lop3_and_or(a_hi, 0x00F000F0u, 0x54005400u);
                                const uint32_t bL1 = lop3_and_or(b_hi, 0x000F000Fu, 0x64006400u), bH1 = lop3_and_or(b_hi, 0x00F000F0u, 0x54005400u);
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt) {
                                    const uint4 xv = *reinterpret_cast<const uint4*>(xb[nt] + wd * 16);
                                    mma_m16n8k16(acc[nt][0], aL0, bL0, aH0, bH0, xv.x, xv.y);
                                    mma_m16n8k16(acc[nt][1], aL1, bL1, aH1, bH1, xv.z, xv.w);
                                }
                            }
                        } else {
#pragma unroll
                            for (int wp = 0; wp < NW / 2; ++wp) {
                                const uint32_t a0 = prmt(wa[2 * wp], 0x64646464u, 0x4140u), a1 = prmt(wa[2 * wp], 0x64646464u, 0x4342u);
                                const uint32_t b0 = prmt(wb[2 * wp], 0x64646464u, 0x4140u), b1 = prmt(wb[2 * wp], 0x64646464u, 0x4342u);
                                const uint32_t a2 = prmt(wa[2 * wp + 1], 0x64646464u, 0x4140u), a3 = prmt(wa[2 * wp + 1], 0x64646464u, 0x4342u);
                                const uint32_t b2 = prmt(wb[2 * wp + 1], 0x64646464u, 0x4140u), b3 = prmt(wb[2 * wp + 1], 0x64646464u, 0x4342u);
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt) {
                                    const uint4 xv = *reinterpret_cast<const uint4*>(xb[nt] + wp * 16);
                                    mma_m16n8k16(acc[nt][0], a0, b0, a1, b1, xv.x, xv.y);
                                    mma_m16n8k16(acc[nt][1], a2, b2, a3, b3, xv.z, xv.w);
                                }
                            }
                        }
                    }
                }
                // affine part of the groups of this pass: y += s * (c - M - z * X)
                {
                    // accumulator columns 2t, 2t+1: two groups (NB == 1) or two batch rows of one group
                    const int gl_c = NB == 1 ? 2 * t : ((2 * t) / NB) * NP + pass;
                    const int b0 = NB == 1 ? 0 : (2 * t) % NB;
                    float s0[2], s1[2], z0[2], z1[2];
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        if constexpr (NB == 1) {
                            s0[rr] = half_lo(mt.s[rr][0]); s1[rr] = half_hi(mt.s[rr][0]);
                            z0[rr] = half_lo(mt.z[rr][0]); z1[rr] = half_hi(mt.z[rr][0]);
                        } else {
                            const uint32_t sw = mt.s[rr][pass >> 1], zw = mt.z[rr][pass >> 1];
                            s0[rr] = s1[rr] = (pass & 1) ? half_hi(sw) : half_lo(sw);
                            z0[rr] = z1[rr] = (pass & 1) ? half_hi(zw) : half_lo(zw);
                        }
                    }
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int e = NB == 1 ? (gi + gl_c) : ((gi + gl_c) * BC + nt * 8 + b0);
                        const float4 mx = *reinterpret_cast<const float4*>(xmx + e);   // {M, X} of column 2t, {M, X} of 2t+1
#pragma unroll
                        for (int rr = 0; rr < 2; ++rr) {
                            float v0 = acc[nt][0][2 * rr] + acc[nt][1][2 * rr];
                            float v1 = acc[nt][0][2 * rr + 1] + acc[nt][1][2 * rr + 1];
                            v0 = fmaf(-z0[rr], mx.y, v0 - mx.x);
                            v1 = fmaf(-z1[rr], mx.w, v1 - mx.z);
                            y[nt][2 * rr] = fmaf(s0[rr], v0, y[nt][2 * rr]);
                            y[nt][2 * rr + 1] = fmaf(s1[rr], v1, y[nt][2 * rr + 1]);
                        }
                    }
                }
            }

            // ---- fold the lanes that hold pieces of the same (row, batch row), add into this warp's slot ----
            float* dst = part + ((((size_t)ps * MATS + u.m) * kConsumerWarps + cw) * kTileRows) * BC;
            if constexpr (NB == 1) {
                float v0 = y[0][0] + y[0][1], v1 = y[0][2] + y[0][3];
                v0 += __shfl_xor_sync(0xffffffffu, v0, 1); v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
                v0 += __shfl_xor_sync(0xffffffffu, v0, 2); v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
                if (t == 0) {
                    dst[g] += v0;
                    dst[g + 8] += v1;
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float v = y[nt][i];
                        if constexpr (NB == 2) v += __shfl_xor_sync(0xffffffffu, v, 1);
                        if constexpr (NB <= 4) v += __shfl_xor_sync(0xffffffffu, v, 2);
                        y[nt][i] = v;
                    }
                    const bool writer = NB == 2 ? (t == 0) : (NB == 4 ? (t < 2) : true);
                    if (writer) {
                        const int col = nt * 8 + (2 * t) % NB;
                        float2* d0 = reinterpret_cast<float2*>(dst + (size_t)g * BC + col);
                        float2* d1 = reinterpret_cast<float2*>(dst + (size_t)(g + 8) * BC + col);
                        float2 a = *d0, b2 = *d1;
                        a.x += y[nt][0]; a.y += y[nt][1];
                        b2.x += y[nt][2]; b2.y += y[nt][3];
                        *d0 = a; *d1 = b2;
                    }
                }
            }
        };

        Unit cur = {0, (int)((cw - ph16) & 15u), 0, 0, c_begin, true};
        normalize(cur);
        Meta mcur;
        if (cur.valid) load_meta(cur, mcur);
        int S = 0;
#pragma unroll 1
        for (int tl = 0; tl < n_tiles; ++tl) {
            const int ps = tl % nslot;
            if (xc == 0 && tl >= nslot)
                ok = mbar_wait_bounded(&slot_free[ps], (uint32_t)(tl / nslot - 1) & 1u, &g_device_status, EV_GEMV_EMPTY_WAIT,
                                       ok ? kWaitLimit : 64u) && ok;
#pragma unroll 1
            for (int mc = 0; mc < MATS * (c_end - c_begin); ++mc, ++S) {
                const int slot = c_slot;
                ok = mbar_wait_bounded(&full[slot], c_phase, &g_device_status, EV_GEMV_FULL_WAIT, ok ? kWaitLimit : 64u) && ok;
                if (++c_slot == p.stages) { c_slot = 0; c_phase ^= 1; }
#pragma unroll 1
                while (cur.valid && cur.S == S) {
                    Unit nxt = cur;
                    nxt.i += 16;
                    normalize(nxt);
                    Meta mnext;
                    if (nxt.valid) load_meta(nxt, mnext);
                    process_unit(slot, cur, mcur, ps);
                    cur = nxt;
                    if (nxt.valid) mcur = mnext;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);
            }
            if (xc == n_xc - 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&tile_done[ps]);
            }
        }
        ph16 = (ph16 + (uint32_t)nS * (uint32_t)NU) & 15u;
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

template <int BITS, int LOGG, int NB, int NT, bool GATE_UP>
int launch_fast(GemvParams& p, cudaStream_t stream) {
    constexpr int MATS = GATE_UP ? 2 : 1;
    constexpr int G = 1 << LOGG;
    constexpr int UK = kUnitGroups * G;
    constexpr int LB = G * BITS / 32;
    constexpr int BC = NB * NT;
    const int sms = sm_count();
    const uint32_t smem_cap = (uint32_t)max_smem_optin();

    // k per stage: per-row copies of about 2 KB, a whole number of units
    int kc = tuning_get("gemv.stage_k");
    if (kc <= 0) {
        const int target_bytes = 2048;
        const int n = std::max(1, (p.row_bytes + target_bytes / 2) / target_bytes);
        kc = (p.K + n - 1) / n;
    }
    kc = std::max(UK, (kc + UK - 1) / UK * UK);
    p.kc = kc;
    p.n_kc = (p.K + kc - 1) / kc;
    p.nu = kc / UK;

    const int64_t tiles = (p.N + kTileRows - 1) / kTileRows;
    int grid = (int)std::max<int64_t>(1, std::min<int64_t>(sms, tiles));
    p.rows_lo = p.N / grid;
    p.rem = p.N % grid;
    const int max_tiles = (p.rows_lo + (p.rem ? 1 : 0) + kTileRows - 1) / kTileRows;

    p.meta_vec = p.scale_dtype == B200Q_F16 && (p.Gn % 8 == 0) && aligned16(p.s[0]) &&
                 (p.z[0] == nullptr || aligned16(p.z[0])) &&
                 (MATS == 1 || (aligned16(p.s[1]) && (p.z[1] == nullptr || aligned16(p.z[1]))));
    // stage rows are padded so that the 8 rows a warp reads at once fall into different banks
    const uint32_t row_pad = LB == 32 ? 16 : 4 * LB;
    p.row_stride = align_up((uint32_t)(kc * BITS / 8), 128) + row_pad;
    p.stage_bytes = align_up(kTileRows * p.row_stride, 128);
    const uint32_t x_pad = G == 32 ? 64 : 16;

    // activation chunk: the whole K when it leaves room for a useful ring, else a whole number of stages
    uint32_t off = 0;
    bool fits = false;
    const uint32_t budgets[3] = {96 * 1024, 48 * 1024, 24 * 1024};
    for (int bi = 0; bi < 3 && !fits; ++bi) {
        int xk = p.n_kc * kc;
        if ((size_t)xk * p.B * 2 > budgets[bi]) xk = std::max(1, (int)(budgets[bi] / ((size_t)p.B * 2 * kc))) * kc;
        const int n_xc = (p.K + xk - 1) / xk;
        if (n_xc == 1 && bi != 0) break;      // nothing new to try
        p.xk = xk;
        p.n_xc = n_xc;
        p.nslot = n_xc == 1 ? std::min(2, max_tiles) : max_tiles;
        if (p.nslot > kMaxSlots) return B200Q_ERR_UNSUPPORTED;
        p.xstride = align_up((uint32_t)xk * 2, 128) + x_pad;
        off = align_up((2 * kMaxStages + 2 * kMaxSlots) * sizeof(uint64_t), 128);
        p.off_xs = off;     off += align_up((uint32_t)p.B * p.xstride, 128);
        p.off_xzero = off;  off += align_up((uint32_t)UK * 2, 128);
        p.off_xmx = off;    off += align_up((uint32_t)(xk / G + kUnitGroups) * BC * 8, 128);
        p.off_xscale = off; off += align_up((uint32_t)p.B * 2 * 4, 128);
        p.off_part = off;   off += align_up((uint32_t)p.nslot * MATS * kConsumerWarps * kTileRows * BC * 4, 128);
        p.off_ring = off;
        fits = off + 3ull * p.stage_bytes <= smem_cap;
    }
    if (!fits) return B200Q_ERR_UNSUPPORTED;

    // ring depth: everything the CTA will ever stream if that is little, else as deep as shared memory allows
    const int total_stages = max_tiles * MATS * p.n_kc;
    int stages = tuning_get("gemv.stages");
    if (stages <= 0) stages = kMaxStages;
    stages = std::min({stages, kMaxStages, std::max(2, total_stages)});
    while (stages > 2 && off + (uint64_t)stages * p.stage_bytes > smem_cap) --stages;
    p.stages = stages;
    const uint64_t total = off + (uint64_t)stages * p.stage_bytes;

    auto kernel = qgemv_kernel<BITS, LOGG, NB, NT, GATE_UP>;
    static bool configured[64] = {};   // per instantiation and device; a race only repeats the call
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_cap) != cudaSuccess)
            return B200Q_ERR_LAUNCH;
        configured[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning_get("no_pdl") ? 0 : 1;
    if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return B200Q_ERR_LAUNCH;
    return finish_launch();
}

template <int BITS, int LOGG, bool GATE_UP>
int dispatch_cols(GemvParams& p, cudaStream_t stream) {
    if (p.B <= 1) return launch_fast<BITS, LOGG, 1, 1, GATE_UP>(p, stream);
    if (p.B <= 2) return launch_fast<BITS, LOGG, 2, 1, GATE_UP>(p, stream);
    if (p.B <= 4) return launch_fast<BITS, LOGG, 4, 1, GATE_UP>(p, stream);
    if (p.B <= 8) return launch_fast<BITS, LOGG, 8, 1, GATE_UP>(p, stream);
    return launch_fast<BITS, LOGG, 8, 2, GATE_UP>(p, stream);
}

template <int BITS>
int dispatch_bits(GemvParams& p, bool gate_up, cudaStream_t stream) {
    int logG = 0;
    while ((1 << logG) < p.G) ++logG;
    if (gate_up) {
        if (logG == 5) return dispatch_cols<BITS, 5, true>(p, stream);
        if (logG == 6) return dispatch_cols<BITS, 6, true>(p, stream);
        return dispatch_cols<BITS, 7, true>(p, stream);
    }
    if (logG == 5) return dispatch_cols<BITS, 5, false>(p, stream);
    if (logG == 6) return dispatch_cols<BITS, 6, false>(p, stream);
    return dispatch_cols<BITS, 7, false>(p, stream);
}

}  // namespace
}  // namespace b200q
