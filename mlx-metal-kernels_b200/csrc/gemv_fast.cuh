// Weight-streaming quantized matvec / skinny GEMM for decode (sm_100a): the tensor-core kernel.
//
//   y[b, n] = sum_k x[b, k] * (code[n, k] - zero[n, k/G]) * scale[n, k/G]          b < B <= 16
//
// Design (one CTA per SM: 16 consumer warps, three producer warps, one epilogue warp):
//   * output rows are dealt out evenly to the CTAs; a CTA walks its rows in tiles of 16 (one
//     tensor-core M tile).
//   * the producer warps stream each tile through a ring of shared-memory stages with 1-D bulk
//     copies (TMA engine) signalled on mbarriers: one copy per weight row and k-chunk, sized
//     about 2 KB because the copy engine needs >= 2 KB per copy to saturate HBM; the copies of a
//     stage are shared by the producer warps (issuing one costs a warp about 40 ns).  They start
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
#include <type_traits>

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
__device__ __forceinline__ void words_to_f32(const uint32_t (&w)[4], int dtype, float (&v)[8]) {
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
// The kernel's input rows: plain, or (tensor-parallel exchange in packet form) packets that are polled until they carry
// the sequence number `xs.seq16`.  After a wait ran out the following loads give up quickly.
// PACKETS is a template parameter of the kernel: the polling loop next to the plain loads cost the single-GPU decode
// step 6 % (registers, code layout), so kernels that read plain rows are compiled without it.
struct XSource { uint32_t seq16, limit; };
template <bool PACKETS>
__device__ __forceinline__ void load8_x(const void* base, int dtype, int64_t idx, XSource& xs, float (&v)[8]) {
    if constexpr (!PACKETS) {
        load8_raw(base, dtype, idx, v);
        return;
    }
    uint32_t w[4];
    if (!tp_load8_packets(base, idx, xs.seq16, xs.limit, w)) {
        atomicMax(&g_device_status, (int)EV_PEER_WAIT);
        xs.limit = 64u;
    }
    words_to_f32(w, dtype, v);
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
template <bool PACKETS>
__device__ __forceinline__ void load8_z(const GemvParams& p, int b, int k, XSource& xs, float (&zv)[8]) {
    load8_x<PACKETS>(p.x, p.act_dtype, (int64_t)b * p.K + k, xs, zv);
    if (p.res_in != nullptr) {
        float r[8];
        load8_raw(p.res_in, p.act_dtype, (int64_t)b * p.K + k, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) zv[i] = round_act(zv[i] + r[i], p.act_dtype);
    }
}
// the activation row the matvec sees: x itself, or cast(z * inv_rms * w)
template <bool PACKETS>
__device__ __forceinline__ void load8_act(const GemvParams& p, int b, int k, float inv_rms, bool write_side, XSource& xs,
                                          float (&v)[8]) {
    if (p.norm_w == nullptr) {
        load8_x<PACKETS>(p.x, p.act_dtype, (int64_t)b * p.K + k, xs, v);
        return;
    }
    float zv[8];
    load8_z<PACKETS>(p, b, k, xs, zv);
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

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds_f128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
template <int NWORDS>
__device__ __forceinline__ void lds_words(uint32_t addr, uint32_t (&w)[NWORDS]) {
    if constexpr (NWORDS == 1) {
        w[0] = lds_u32(addr);
    } else if constexpr (NWORDS == 2) {
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(addr));
    } else {
#pragma unroll
        for (int i = 0; i < NWORDS / 4; ++i) {
            const uint4 u = lds_u128(addr + 16 * i);
            w[4 * i] = u.x; w[4 * i + 1] = u.y; w[4 * i + 2] = u.z; w[4 * i + 3] = u.w;
        }
    }
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// BITS: code width.  LOGG: log2(group size) in {5, 6, 7}.  NB: tensor-core columns per quantisation group
// (batch rows rounded up to 1, 2, 4, 8).  NT: column tiles (2 only with NB == 8: 9..16 batch rows).
template <int BITS, int LOGG, int NB, int NT, bool GATE_UP, bool PACKETS>
__global__ void __launch_bounds__(kThreads, kMinCtasPerSm) qgemv_kernel(const __grid_constant__ GemvParams p) {
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
    constexpr float OFF_ODD = BITS == 4 ? 64.0f : 1024.0f;
    static_assert(NT == 1 || NB == 8, "two column tiles only with eight batch columns per group");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    uint64_t* tile_done = empty + kMaxStages;      // [kMaxSlots] all consumer warps have added their share
    uint64_t* slot_free = tile_done + kMaxSlots;   // [kMaxSlots] the epilogue has read (and zeroed) the slot

    const int cta = blockIdx.x;
    // Rows of this CTA: either one contiguous range (rows dealt evenly), or every gridDim-th tile of 16 rows.
    const bool interleave = p.interleave != 0;
    const int total_tiles = (p.N + kTileRows - 1) / kTileRows;
    const int r_lo = interleave ? cta * kTileRows : cta * p.rows_lo + min(cta, p.rem);
    const int r_cnt = p.rows_lo + (cta < p.rem ? 1 : 0);
    const int r_hi = interleave ? p.N : r_lo + r_cnt;
    const int tile_step = interleave ? (int)gridDim.x * kTileRows : kTileRows;
    const int n_tiles = interleave ? (total_tiles - cta + (int)gridDim.x - 1) / (int)gridDim.x : (r_cnt + kTileRows - 1) / kTileRows;
    const int n_xc = p.n_xc;
    const int cpx = p.xk / p.kc;                   // stages per (matrix, tile, activation chunk)
    const int units_per_visit = cpx * p.nu;        // units (incl. absent ones of a short last chunk) per such visit
    const int nslot = p.nslot;
    const int B = p.B;
    const int Gn = p.Gn;

    float* part = reinterpret_cast<float*>(smem + p.off_part);     // [nslot][MATS][16 warps][16 rows][BC]
    uint8_t* xzero = smem + p.off_xzero;
    // barrier set-up spread over threads (one barrier each), fenced by the thread that also owns full[0]
    if ((int)threadIdx.x < p.stages) {
        mbar_init(&full[threadIdx.x], kProducerWarps);
        mbar_init(&empty[threadIdx.x], kConsumerWarps);
    } else if ((int)threadIdx.x >= 32 && (int)threadIdx.x < 32 + nslot) {
        mbar_init(&tile_done[threadIdx.x - 32], kConsumerWarps);
        mbar_init(&slot_free[threadIdx.x - 32], 1);
    }
    if (threadIdx.x < 64) mbar_fence_init();
    for (int i = threadIdx.x; i < nslot * MATS * kConsumerWarps * kTileRows * BC; i += kThreads) part[i] = 0.0f;
    for (int i = threadIdx.x; i < UK * 2 / 4; i += kThreads) reinterpret_cast<uint32_t*>(xzero)[i] = 0u;
    __syncthreads();
    pdl_launch_dependents();

    uint8_t* ring = smem + p.off_ring;
    uint8_t* mbuf = smem + p.off_meta;             // [meta_depth][scales | zeros][16 rows][Gn] halves
    const uint32_t mbuf_half = (uint32_t)kTileRows * Gn * 2;   // bytes of one of the four arrays

    // Producer and consumers walk the stages in the same order: activation chunk, tile, matrix, k-chunk.
    if (warp >= kFirstProducerWarp && warp < kFirstProducerWarp + kProducerWarps) {
        const int pw = warp - kFirstProducerWarp;
        bool ok = true;
        int slot = 0;
        uint32_t phase = 1;
        bool first_pass = true;
        int q = 0;                                  // (tile, matrix) visits so far
        for (int xc = 0; xc < n_xc; ++xc) {
            const int c_begin = xc * cpx;
            const int c_end = min(p.n_kc, c_begin + cpx);
            for (int tl = 0; tl < n_tiles; ++tl) {
                const int row0 = r_lo + tl * tile_step;
                const int rows = min(kTileRows, r_hi - row0);
                for (int m = 0; m < MATS; ++m, ++q) {
                    const void* sp = (MATS == 2 && m != 0) ? p.s[1] : p.s[0];
                    const void* zp = (MATS == 2 && m != 0) ? p.z[1] : p.z[0];
                    const uint8_t* wp = (MATS == 2 && m != 0) ? p.w[1] : p.w[0];
                    for (int c = c_begin; c < c_end; ++c) {
                        if (!first_pass)
                            ok = mbar_wait_bounded(&empty[slot], phase, &g_device_status, EV_GEMV_EMPTY_WAIT,
                                                   ok ? kWaitLimit : 64u) && ok;
                        const int k0 = c * p.kc;
                        const int kcur = min(p.kc, p.K - k0);
                        const uint32_t bytes_row = (uint32_t)(kcur * BITS / 8);
                        uint8_t* stage = ring + (size_t)slot * p.stage_bytes;
                        // the scales / zero points of the (tile, matrix) ride on the barrier of its first stage; their
                        // buffers form a ring deep enough that the buffer being overwritten belongs to a tile whose
                        // stages have all been released (meta_depth >= stages / stages-per-tile + 1)
                        const bool with_meta = p.meta_vec && c == c_begin;
                        const uint32_t meta_bytes = (uint32_t)rows * Gn * 2;
                        // copy number ci of the stage: 0..15 one weight row each, 16 / 17 the scales / zero points;
                        // producer warp pw issues ci = pw, pw + kProducerWarps, ... (one per lane)
                        const int ci = pw + kProducerWarps * lane;
                        uint8_t* dst = nullptr;
                        const uint8_t* src = nullptr;
                        uint32_t nbytes = 0;
                        if (ci < rows) {
                            src = wp + (size_t)(row0 + ci) * p.row_bytes + (size_t)k0 * BITS / 8;
                            dst = stage + (size_t)ci * p.row_stride;
                            nbytes = bytes_row;
                        } else if (with_meta && ci == 16) {
                            src = reinterpret_cast<const uint8_t*>(sp) + (size_t)row0 * Gn * 2;
                            dst = mbuf + (size_t)(q % p.meta_depth) * 2 * mbuf_half;
                            nbytes = meta_bytes;
                        } else if (with_meta && ci == 17 && zp != nullptr) {
                            src = reinterpret_cast<const uint8_t*>(zp) + (size_t)row0 * Gn * 2;
                            dst = mbuf + (size_t)(q % p.meta_depth) * 2 * mbuf_half + mbuf_half;
                            nbytes = meta_bytes;
                        }
                        const uint32_t warp_bytes = __reduce_add_sync(0xffffffffu, nbytes);
                        if (lane == 0) mbar_arrive_expect_tx(&full[slot], warp_bytes);
                        __syncwarp();
                        if (nbytes != 0) bulk_g2s(dst, src, nbytes, &full[slot]);
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
        const uint32_t out_seq16 = (p.tp_out.world > 0 && p.tp_out.packets) ? tp_seq16(tp_writer_seq(p.tp_out)) : 0u;
        bool ok = true;
        for (int tl = 0; tl < n_tiles; ++tl) {
            const int ps = tl % nslot;
            ok = mbar_wait_bounded(&tile_done[ps], (uint32_t)(tl / nslot) & 1u, &g_device_status, EV_GEMV_FULL_WAIT,
                                   ok ? kWaitLimit : 64u) && ok;
            const int row0 = r_lo + tl * tile_step;
            const int rows = min(kTileRows, r_hi - row0);
            float* slot_base = part + (size_t)ps * MATS * kConsumerWarps * kTileRows * BC;
            for (int it = lane; it < kTileRows * BC; it += 32) {
                const int r = it & (kTileRows - 1);
                const int b = it >> 4;
                float val[MATS];
#pragma unroll
                for (int m = 0; m < MATS; ++m) {
                    float* src = slot_base + ((size_t)m * kConsumerWarps * kTileRows + r) * BC + b;
                    // Slot j holds k-spans j, j + 16, ... of the (tile, matrix) visit (the consumers index their slots by
                    // span, not by warp): summing the slots in order adds a row's spans in k order, whatever CTA or
                    // GPU holds the row.
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
                    // tensor-parallel exchange: the value goes to column block `rank` of every rank's full rows
                    auto store_peers = [&](float v) {
                        const int64_t of = (int64_t)b * p.N * p.tp_out.world + (int64_t)p.tp_out.rank * p.N + row0 + r;
                        const unsigned short bits16 = p.act_dtype == B200Q_F16 ? __half_as_ushort(__float2half_rn(v))
                                                                               : __bfloat16_as_ushort(__float2bfloat16_rn(v));
                        if (p.tp_out.packets) {
                            const uint32_t pk = tp_packet(bits16, out_seq16);
#pragma unroll 1
                            for (int peer = 0; peer < p.tp_out.world; ++peer)
                                st_volatile_u32(reinterpret_cast<uint32_t*>(p.tp_out.full[peer]) + of, pk);
                            return;
                        }
#pragma unroll 1
                        for (int peer = 0; peer < p.tp_out.world; ++peer)
                            reinterpret_cast<unsigned short*>(p.tp_out.full[peer])[of] = bits16;
                    };
                    if (GATE_UP) {
                        if (p.gate_out != nullptr) store(p.gate_out, val[0]);
                        if (p.up_out != nullptr) store(p.up_out, val[MATS - 1]);
                        if (p.act_out != nullptr || p.tp_out.world > 0) {
                            const float gte = val[0];
                            const float silu = gte / (1.0f + expf(-gte));
                            if (p.act_out != nullptr) store(p.act_out, silu * val[MATS - 1]);
                            if (p.tp_out.world > 0) store_peers(silu * val[MATS - 1]);
                        }
                    } else {
                        float v = val[0];
                        if (p.residual != nullptr) v = load_as_f32(p.residual, p.act_dtype, o) + v;
                        if (p.y != nullptr) store(p.y, v);
                        if (p.tp_out.world > 0) store_peers(v);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&slot_free[ps]);
        }
        if (p.tp_out.world > 0) {
            if (p.tp_out.packets) tp_finish_writer_packets(p.tp_out, lane);
            else tp_finish_writer(p.tp_out, lane);
        }
        return;
    }

    // ---------------------------------- consumer warps -----------------------------------------
    const int cw = warp;
    const int ctid = threadIdx.x;               // 0 .. kConsumerThreads-1
    const int g = lane >> 2;
    const int t = lane & 3;

    uint8_t* xs = smem + p.off_xs;                                    // [B] rows of xstride bytes, fp16, operand order
    float2* xmx = reinterpret_cast<float2*>(smem + p.off_xmx);        // [groups of the chunk (+ padding)][BC] {M, X}

    // per-lane constants.  As B operand this lane feeds column g, as accumulator owner columns 2t, 2t+1.
    const int my_js = g / NB;                   // group slot of column g within a pass
    const int my_b = g % NB;                    // batch row of column g (first column tile)
    const uint32_t ring_u = smem_u32(ring);
    const uint32_t a_lane = (uint32_t)g * p.row_stride + t * LB;
    const uint32_t a_row8 = 8u * p.row_stride;
    const uint32_t xz_u = smem_u32(xzero) + t * XB;
    const uint32_t xmx_u = smem_u32(xmx);
    const uint32_t mbuf_u = smem_u32(mbuf);
    uint32_t x_lane[NT];
    bool bvalid[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int b = nt * 8 + my_b;
        bvalid[nt] = b < B;
        x_lane[nt] = smem_u32(xs) + (uint32_t)min(b, B - 1) * p.xstride + t * XB;
    }
    // accumulator columns 2t, 2t+1: two groups (NB == 1) or two batch rows of one group
    const int jc = NB == 1 ? 0 : (2 * t) / NB;  // group slot of this lane's accumulator columns
    const int b0 = NB == 1 ? 0 : (2 * t) % NB;  // their first batch row
    const uint32_t meta_lane = (uint32_t)(g * Gn + (NB == 1 ? 2 * t : jc * NP)) * 2;   // byte offset inside a scales array
    const uint32_t meta_row8 = (uint32_t)8 * Gn * 2;
    float* part_lane = part;


    pdl_wait();   // activations belong to the previous kernel until here
    XSource xsrc = {0u, p.tp_in.spin_limit ? p.tp_in.spin_limit : kTpSpinLimit};
    if (PACKETS) {
        // packet form: nothing to wait for here, every load of the rows checks its own packets
        xsrc.seq16 = tp_seq16(*reinterpret_cast<const volatile uint32_t*>(p.tp_in.epoch));
    } else if (p.tp_in.world > 0) {
        // the activations are an exchange buffer filled by all ranks: wait for every source rank's flag
        if (ctid < p.tp_in.world && !tp_wait_source(p.tp_in, ctid)) atomicMax(&g_device_status, (int)EV_PEER_WAIT);
        named_bar_sync(1, kConsumerThreads);
    }

    // per batch row: inv_rms (norm prologue) and the power of two that maps bf16 rows into fp16 range
    if (need_row_pass) {
        float* scratch = xscale + 2 * B;                      // [2][consumer warps] partial sums / maxima
        if (B <= 4) {
            // few rows: every consumer thread takes part in each row (fixed-order sums: bitwise reproducible)
            for (int b = 0; b < B; ++b) {
                float inv = 1.0f;
                if (p.norm_w != nullptr) {
                    float ss = 0.0f;
                    for (int k = ctid * 8; k < p.K; k += kConsumerThreads * 8) {
                        float zv[8];
                        load8_z<PACKETS>(p, b, k, xsrc, zv);
#pragma unroll
                        for (int i = 0; i < 8; ++i) ss += zv[i] * zv[i];
                    }
                    ss = warp_sum(ss);
                    if (lane == 0) scratch[cw] = ss;
                    named_bar_sync(1, kConsumerThreads);
                    float tot = 0.0f;
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; ++w) tot += scratch[w];
                    inv = rsqrtf(tot / (float)p.K + p.eps);
                }
                float sc = 1.0f;
                if (p.act_dtype == B200Q_BF16) {
                    float mx = 0.0f;
                    for (int k = ctid * 8; k < p.K; k += kConsumerThreads * 8) {
                        float v[8];
                        load8_act<PACKETS>(p, b, k, inv, false, xsrc, v);
#pragma unroll
                        for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(v[i]));
                    }
                    mx = warp_max(mx);
                    if (lane == 0) scratch[kConsumerWarps + cw] = mx;
                    named_bar_sync(1, kConsumerThreads);
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; ++w) mx = fmaxf(mx, scratch[kConsumerWarps + w]);
                    int ex = 0;
                    if (mx > 0.0f && mx < INFINITY) frexpf(mx, &ex);
                    ex = max(-100, min(114, ex - 14));
                    sc = exp2f((float)ex);
                }
                if (ctid == 0) {
                    xscale[b] = sc;
                    xscale[B + b] = inv;
                }
                named_bar_sync(1, kConsumerThreads);          // scratch may be reused, xscale is visible
            }
        } else {
            for (int b = cw; b < B; b += kConsumerWarps) {
                float inv = 1.0f;
                if (p.norm_w != nullptr) {
                    float ss = 0.0f;
                    for (int k = lane * 8; k < p.K; k += 256) {
                        float zv[8];
                        load8_z<PACKETS>(p, b, k, xsrc, zv);
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
                        load8_act<PACKETS>(p, b, k, inv, false, xsrc, v);
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
    }
    // ---- stage activations of [xk0, xk0+xkn) as fp16 in tensor-core operand order, with their per-group sums ----
    auto stage_x = [&](int xk0, int xkn, bool write_side) {
        constexpr int CPG = G / 8;                 // 8-value blocks per group: the lanes that share a group
        const int chunks = xkn / 8;
        const int total = B * chunks;
        const int gc = xkn >> LOGG;
        const int gpad = (gc + kUnitGroups - 1) / kUnitGroups * kUnitGroups;
        // zeros for padding groups and unused batch columns
        for (int i = ctid; i < gpad * BC; i += kConsumerThreads) {
            const int gi = i / BC;
            if (gi >= gc || i - gi * BC >= B) xmx[i] = make_float2(0.0f, 0.0f);
        }
#pragma unroll 1
        for (int base = 0; base < total; base += kConsumerThreads) {   // same trip count for every thread (shuffles below)
            const int i = base + ctid;
            const bool live = i < total;
            const int b = live ? i / chunks : 0;
            const int ci = live ? i - b * chunks : 0;
            float se = 0.0f, so = 0.0f;
            if (live) {
                const int kk = ci * 8;
                float v[8];
                const float inv = need_row_pass ? xscale[B + b] : 1.0f;
                const float down = need_row_pass ? 1.0f / xscale[b] : 1.0f;
                load8_act<PACKETS>(p, b, xk0 + kk, inv, write_side, xsrc, v);
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
                    se = (__half2float(h[0]) + __half2float(h[2])) + (__half2float(h[4]) + __half2float(h[6]));
                    so = (__half2float(h[1]) + __half2float(h[3])) + (__half2float(h[5]) + __half2float(h[7]));
                } else {
                    out.x = __half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
                    out.y = __half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
                    out.z = __half_as_ushort(h[4]) | ((uint32_t)__half_as_ushort(h[5]) << 16);
                    out.w = __half_as_ushort(h[6]) | ((uint32_t)__half_as_ushort(h[7]) << 16);
                    se = ((__half2float(h[0]) + __half2float(h[1])) + (__half2float(h[2]) + __half2float(h[3]))) +
                         ((__half2float(h[4]) + __half2float(h[5])) + (__half2float(h[6]) + __half2float(h[7])));
                }
                *reinterpret_cast<uint4*>(xs + (size_t)b * p.xstride + (size_t)kk * 2) = out;
            }
            // {M, X} per (group, batch column): X = sum of the group's activations, M = sum of offset * activation
            // (offset 1024 for low nibbles / bytes, 64 for high nibbles).  The CPG blocks of a group sit in
            // adjacent lanes (rows hold a whole number of groups), summed in a fixed order.
#pragma unroll
            for (int o = 1; o < CPG; o <<= 1) {
                se += __shfl_xor_sync(0xffffffffu, se, o);
                so += __shfl_xor_sync(0xffffffffu, so, o);
            }
            if (live && (ci & (CPG - 1)) == 0) xmx[(ci / CPG) * BC + b] = make_float2(1024.0f * se + OFF_ODD * so, se + so);
        }
        named_bar_sync(1, kConsumerThreads);
    };

    bool ok = true;
    int c_slot = 0;
    uint32_t c_phase = 0;
    int mb_idx = 0;                             // scale / zero-point buffer of the current (tile, matrix) visit

    // ---- one unit: 16 rows x 8 groups ----
    //   a_u    shared address of this lane's bytes of the unit's first group (row g)
    //   xoff   byte offset of the unit inside a staged activation row
    //   gi     first group of the unit inside the staged chunk;  gabs: inside the whole row
    auto process_unit = [&](auto full_c, uint32_t a_u, uint32_t xoff, int gi, int gabs, int ng, uint32_t mb_u,
                            int m, int row0, float* dst, bool has_z) {
        constexpr bool FULL = decltype(full_c)::value;
        float y[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) y[nt][i] = 0.0f;

        // The unit's 8 groups in execution order e = pass * GS + slot; the operands of group e + 1 are
        // fetched from shared memory before the tensor-core work of group e is issued.
        constexpr int NXV = BITS == 4 ? NW : NW / 2;          // 16-byte activation loads per group and column tile
        constexpr bool PIPE = LOGG <= 6 && NT == 1 && !(BITS == 8 && NB >= 4);   // (elsewhere: not enough registers)
        struct Operands { uint32_t wa[NW], wb[NW]; };
        auto fetch = [&](int e, Operands& o) {
            const int pass = e / GS, js = e % GS;
            const int gl = js * NP + pass;                   // group of the unit handled by slot js in this pass
            lds_words<NW>(a_u + gl * GB, o.wa);
            lds_words<NW>(a_u + a_row8 + gl * GB, o.wb);
        };
        auto present = [&](int e) { return FULL || ((e % GS) * NP + e / GS) < ng; };
        Operands ops[PIPE ? 2 : 1];
        if (PIPE) fetch(0, ops[0]);       // group 0 always exists
        // with 4 or 8 batch columns per group a lane meets NB consecutive groups of its two rows, one per pass:
        // their scales / zero points are fetched once per unit as vectors
        uint32_t mvec_s[2][NB >= 4 ? NB / 2 : 1], mvec_z[2][NB >= 4 ? NB / 2 : 1];
        if constexpr (NB >= 4) {
            if (p.meta_vec) {
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const uint32_t ma = mb_u + meta_lane + rr * meta_row8 + (uint32_t)gabs * 2;
                    lds_words<NB / 2>(ma, mvec_s[rr]);
                    if (has_z) {
                        lds_words<NB / 2>(ma + mbuf_half, mvec_z[rr]);
                    } else {
#pragma unroll
                        for (int i = 0; i < NB / 2; ++i) mvec_z[rr][i] = 0u;
                    }
                }
            }
        }

#pragma unroll
        for (int pass = 0; pass < NP; ++pass) {
            // two accumulators shorten the dependent MMA chain of a pass; with one group per pass (NB == 8) the chain
            // is four instructions anyway and one accumulator saves its zeroing and the final add
            constexpr int NACC = NB == 8 ? 1 : 2;
            float acc[NT][NACC][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int a = 0; a < NACC; ++a)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[nt][a][i] = 0.0f;
            // This lane's column belongs to one group of the pass (slot my_js): only that group's activations
            // are fetched; for the other groups of the pass the lane feeds zeros.
            uint4 xr[NT][NXV];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t xb = bvalid[nt] ? x_lane[nt] + xoff + (uint32_t)(my_js * NP + pass) * (G * 2) : xz_u;
#pragma unroll
                for (int v = 0; v < NXV; ++v) xr[nt][v] = lds_u128(xb + v * 16);
            }
#pragma unroll
            for (int js = 0; js < GS; ++js) {
                const int e = pass * GS + js;
                const bool mine = GS == 1 || my_js == js;
                if (PIPE && e + 1 < kUnitGroups && present(e + 1)) fetch(e + 1, ops[(e + 1) & 1]);
                if (present(e)) {
                    if (!PIPE) fetch(e, ops[0]);
                    const Operands& o = ops[PIPE ? (e & 1) : 0];
                    if constexpr (BITS == 4) {
#pragma unroll
                        for (int wd = 0; wd < NW; ++wd) {
                            const uint32_t a_lo = o.wa[wd], b_lo = o.wb[wd];
                            const uint32_t a_hi = a_lo >> 8, b_hi = b_lo >> 8;
                            const uint32_t aL0 = lop3_and_or(a_lo, 0x000F000Fu, 0x64006400u), aH0 = lop3_and_or(a_lo, 0x00F000F0u, 0x54005400u);
                            const uint32_t bL0 = lop3_and_or(b_lo, 0x000F000Fu, 0x64006400u), bH0 = lop3_and_or(b_lo, 0x00F000F0u, 0x54005400u);
                            const uint32_t aL1 = lop3_and_or(a_hi, 0x000F000Fu, 0x64006400u), aH1 = lop3_and_or(a_hi, 0x00F000F0u, 0x54005400u);
                            const uint32_t bL1 = lop3_and_or(b_hi, 0x000F000Fu, 0x64006400u), bH1 = lop3_and_or(b_hi, 0x00F000F0u, 0x54005400u);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                const uint4 xq = xr[nt][wd];
                                const uint4 xv = make_uint4(mine ? xq.x : 0u, mine ? xq.y : 0u, mine ? xq.z : 0u, mine ? xq.w : 0u);
                                mma_m16n8k16(acc[nt][0], aL0, bL0, aH0, bH0, xv.x, xv.y);
                                mma_m16n8k16(acc[nt][NACC - 1], aL1, bL1, aH1, bH1, xv.z, xv.w);
                            }
                        }
                    } else {
#pragma unroll
                        for (int wp = 0; wp < NW / 2; ++wp) {
                            const uint32_t a0 = prmt(o.wa[2 * wp], 0x64646464u, 0x4140u), a1 = prmt(o.wa[2 * wp], 0x64646464u, 0x4342u);
                            const uint32_t c0 = prmt(o.wb[2 * wp], 0x64646464u, 0x4140u), c1 = prmt(o.wb[2 * wp], 0x64646464u, 0x4342u);
                            const uint32_t a2 = prmt(o.wa[2 * wp + 1], 0x64646464u, 0x4140u), a3 = prmt(o.wa[2 * wp + 1], 0x64646464u, 0x4342u);
                            const uint32_t c2 = prmt(o.wb[2 * wp + 1], 0x64646464u, 0x4140u), c3 = prmt(o.wb[2 * wp + 1], 0x64646464u, 0x4342u);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                const uint4 xq = xr[nt][wp];
                                const uint4 xv = make_uint4(mine ? xq.x : 0u, mine ? xq.y : 0u, mine ? xq.z : 0u, mine ? xq.w : 0u);
                                mma_m16n8k16(acc[nt][0], a0, c0, a1, c1, xv.x, xv.y);
                                mma_m16n8k16(acc[nt][NACC - 1], a2, c2, a3, c3, xv.z, xv.w);
                            }
                        }
                    }
                }
            }
            // affine part of the groups of this pass: y += s * (c - M - z * X)
            {
                float s0[2], s1[2], z0[2], z1[2];
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    if (p.meta_vec) {
                        const uint32_t ma = mb_u + meta_lane + rr * meta_row8 + (uint32_t)gabs * 2;
                        if constexpr (NB == 1) {
                            const uint32_t sw = lds_u32(ma);
                            s0[rr] = half_bits_to_float(sw & 0xFFFFu); s1[rr] = half_bits_to_float(sw >> 16);
                            if (has_z) {
                                const uint32_t zw = lds_u32(ma + mbuf_half);
                                z0[rr] = half_bits_to_float(zw & 0xFFFFu); z1[rr] = half_bits_to_float(zw >> 16);
                            } else {
                                z0[rr] = z1[rr] = 0.0f;
                            }
                        } else if constexpr (NB >= 4) {
                            const uint32_t sw = mvec_s[rr][pass >> 1], zw = mvec_z[rr][pass >> 1];
                            s0[rr] = s1[rr] = half_bits_to_float((pass & 1) ? sw >> 16 : sw & 0xFFFFu);
                            z0[rr] = z1[rr] = half_bits_to_float((pass & 1) ? zw >> 16 : zw & 0xFFFFu);
                        } else {
                            s0[rr] = s1[rr] = half_bits_to_float(lds_u16(ma + pass * 2));
                            z0[rr] = z1[rr] = has_z ? half_bits_to_float(lds_u16(ma + mbuf_half + pass * 2)) : 0.0f;
                        }
                    } else {
                        // scales in another dtype or layout: read them where they lie, widened to fp32 (exact), as the
                        // reference does with scales.astype(float32)
                        const void* sp = (MATS == 2 && m != 0) ? p.s[1] : p.s[0];
                        const void* zp = (MATS == 2 && m != 0) ? p.z[1] : p.z[0];
                        const int row = min(row0 + g + 8 * rr, p.N - 1);
                        const int ga = gabs + (NB == 1 ? 2 * t : jc * NP + pass);
                        const int64_t e = (int64_t)row * Gn + ga;
                        s0[rr] = ga < Gn ? load_as_f32(sp, p.scale_dtype, e) : 0.0f;
                        z0[rr] = (ga < Gn && zp != nullptr) ? load_as_f32(zp, p.scale_dtype, e) : 0.0f;
                        if constexpr (NB == 1) {
                            s1[rr] = ga + 1 < Gn ? load_as_f32(sp, p.scale_dtype, e + 1) : 0.0f;
                            z1[rr] = (ga + 1 < Gn && zp != nullptr) ? load_as_f32(zp, p.scale_dtype, e + 1) : 0.0f;
                        } else {
                            s1[rr] = s0[rr];
                            z1[rr] = z0[rr];
                        }
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int e = NB == 1 ? (gi + 2 * t) : ((gi + jc * NP + pass) * BC + nt * 8 + b0);
                    const float4 mx = lds_f128(xmx_u + (uint32_t)e * 8);   // {M, X} of column 2t, {M, X} of 2t+1
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        float v0 = acc[nt][0][2 * rr], v1 = acc[nt][0][2 * rr + 1];
                        if constexpr (NACC == 2) { v0 += acc[nt][1][2 * rr]; v1 += acc[nt][1][2 * rr + 1]; }
                        v0 = fmaf(-z0[rr], mx.y, v0 - mx.x);
                        v1 = fmaf(-z1[rr], mx.w, v1 - mx.z);
                        y[nt][2 * rr] = fmaf(s0[rr], v0, y[nt][2 * rr]);
                        y[nt][2 * rr + 1] = fmaf(s1[rr], v1, y[nt][2 * rr + 1]);
                    }
                }
            }
        }

        // ---- fold the lanes that hold pieces of the same (row, batch row), add into this warp's slot ----
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
                    const int col = nt * 8 + b0;
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

#pragma unroll 1
    for (int xc = 0; xc < n_xc; ++xc) {
        const int xk0 = xc * p.xk;
        const int xkn = min(p.xk, p.K - xk0);
        if (xc > 0) named_bar_sync(1, kConsumerThreads);     // everyone is done with the previous chunk
        stage_x(xk0, xkn, cta == 0);

        const int c_begin = xc * cpx;
        const int c_end = min(p.n_kc, c_begin + cpx);
        // All counters below are advanced incrementally: a consumer warp touches every stage, most of them
        // without finding a unit of its own, so the per-stage bookkeeping has to stay a handful of instructions.
        int visit_rot = 0;                         // ((tile * MATS + matrix) * units_per_visit) mod consumer warps
        int ps = 0;                                // result slot of the tile and the parity of its slot_free barrier
        uint32_t sf_parity = 0;                    // (tile / nslot - 1) & 1, meaningful from tile nslot on
        int row0 = r_lo;
        const int nu_stage = p.nu;
        const uint32_t part_slot_stride = (uint32_t)MATS * kConsumerWarps * kTileRows * BC;
        const uint32_t part_mat_stride = (uint32_t)kConsumerWarps * kTileRows * BC;
        float* dst_tile = part_lane;
#pragma unroll 1
        for (int tl = 0; tl < n_tiles; ++tl) {
            if (xc == 0 && tl >= nslot)
                ok = mbar_wait_bounded(&slot_free[ps], sf_parity, &g_device_status, EV_GEMV_EMPTY_WAIT,
                                       ok ? kWaitLimit : 64u) && ok;
#pragma unroll 1
            for (int m = 0; m < MATS; ++m) {
                // units of a visit are dealt to the warps starting at warp visit_rot
                int first_unit = cw - visit_rot;
                if (first_unit < 0) first_unit += kConsumerWarps;
                visit_rot += units_per_visit % kConsumerWarps;
                if (visit_rot >= kConsumerWarps) visit_rot -= kConsumerWarps;
                const uint32_t mb_u = mbuf_u + (uint32_t)mb_idx * 2 * mbuf_half;
                const bool has_z = ((MATS == 2 && m != 0) ? p.z[1] : p.z[0]) != nullptr;
                // this warp's slot of the visit = the position of its first k-span
                float* dst = dst_tile + (MATS == 2 && m != 0 ? part_mat_stride : 0u) + (uint32_t)first_unit * (kTileRows * BC);
                int k0 = c_begin * p.kc;
#pragma unroll 1
                for (int c = c_begin; c < c_end; ++c, k0 += p.kc) {
                    const int slot = c_slot;
                    ok = mbar_wait_bounded(&full[slot], c_phase, &g_device_status, EV_GEMV_FULL_WAIT, ok ? kWaitLimit : 64u) && ok;
                    if (++c_slot == p.stages) { c_slot = 0; c_phase ^= 1; }
                    const int groups = min(p.kc, p.K - k0) >> LOGG;          // groups in this stage
#pragma unroll 1
                    for (int i = first_unit; i * kUnitGroups < groups; i += kConsumerWarps) {
                        const int ng = min(kUnitGroups, groups - i * kUnitGroups);
                        const uint32_t a_u = ring_u + (uint32_t)slot * p.stage_bytes + a_lane + (uint32_t)i * (kUnitGroups * GB);
                        const int kl = k0 + i * UK - xk0;
                        const int gabs = (k0 + i * UK) >> LOGG;
                        if (ng == kUnitGroups)
                            process_unit(std::true_type{}, a_u, (uint32_t)kl * 2, kl >> LOGG, gabs, ng, mb_u, m, row0, dst, has_z);
                        else
                            process_unit(std::false_type{}, a_u, (uint32_t)kl * 2, kl >> LOGG, gabs, ng, mb_u, m, row0, dst, has_z);
                    }
                    // index of this warp's first unit in the next stage: units are numbered through the stages
                    first_unit -= nu_stage;
                    while (first_unit < 0) first_unit += kConsumerWarps;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[slot]);
                }
                if (++mb_idx == p.meta_depth) mb_idx = 0;
            }
            if (xc == n_xc - 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&tile_done[ps]);
            }
            row0 += tile_step;
            dst_tile += part_slot_stride;
            if (++ps == nslot) { ps = 0; dst_tile = part_lane; if (tl >= nslot) sf_parity ^= 1; }
        }
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
    uint32_t smem_cap = (uint32_t)max_smem_optin();
    if (kMinCtasPerSm > 1) smem_cap = std::min<uint32_t>(smem_cap, smem_cap / kMinCtasPerSm - 1024u);   // room for co-resident CTAs
    const int cap_kb = tuning_get("gemv.smem_kb");
    if (cap_kb > 0) smem_cap = std::min<uint32_t>(smem_cap, (uint32_t)cap_kb * 1024u);

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
    p.interleave = tuning_get("gemv.interleave");
    const int max_tiles = p.interleave ? (int)((tiles + grid - 1) / grid) : (p.rows_lo + (p.rem ? 1 : 0) + kTileRows - 1) / kTileRows;

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
        // result slots: a consumer warp may start tile t only after the epilogue of tile t - nslot, so a
        // handful of slots keeps the tiles (often a single stage each) flowing
        const int slot_bytes = MATS * kConsumerWarps * kTileRows * BC * 4;
        p.nslot = n_xc == 1 ? std::min(max_tiles, std::max(2, std::min(8, (32 * 1024) / slot_bytes))) : max_tiles;
        if (p.nslot > kMaxSlots) return B200Q_ERR_UNSUPPORTED;
        p.xstride = align_up((uint32_t)xk * 2, 128) + x_pad;
        off = align_up((2 * kMaxStages + 2 * kMaxSlots) * sizeof(uint64_t), 128);
        p.off_xs = off;     off += align_up((uint32_t)p.B * p.xstride, 128);
        p.off_xzero = off;  off += align_up((uint32_t)UK * 2, 128);
        p.off_xmx = off;    off += align_up((uint32_t)(xk / G + kUnitGroups) * BC * 8, 128);
        p.off_xscale = off; off += align_up((uint32_t)(p.B * 2 + kConsumerWarps * 2) * 4, 128);
        p.off_part = off;   off += align_up((uint32_t)p.nslot * MATS * kConsumerWarps * kTileRows * BC * 4, 128);
        // Ring depth and the buffers for scales / zero points are chosen together.  The scales of a (tile,
        // matrix) ride on its first stage and are overwritten meta_depth (tile, matrix) visits later, which is
        // safe once all stages of the old visit have been released: meta_depth >= ceil(stages / cpass) + 1.
        const int cpass = std::min(p.n_kc, xk / kc);
        const int total_stages = max_tiles * MATS * p.n_kc;   // everything the CTA will ever stream
        int want = tuning_get("gemv.stages");
        if (want <= 0) want = kMaxStages;
        want = std::min({want, kMaxStages, std::max(2, total_stages)});
        const uint32_t meta_one = p.meta_vec ? (uint32_t)2 * kTileRows * p.Gn * 2 : 0;
        for (int st = want; st >= 2 && !fits; --st) {
            const int depth = (st + cpass - 1) / cpass + 1;
            const uint32_t ring_off = off + align_up((uint32_t)depth * meta_one, 128);
            if (ring_off + (uint64_t)st * p.stage_bytes > smem_cap) continue;
            if (st < 3 && st < want) break;                   // too shallow to stream: try a smaller activation chunk
            p.stages = st;
            p.meta_depth = depth;
            p.off_meta = off;
            p.off_ring = ring_off;
            fits = true;
        }
    }
    if (!fits) return B200Q_ERR_UNSUPPORTED;
    const uint64_t total = p.off_ring + (uint64_t)p.stages * p.stage_bytes;

    // input rows in packet form (fused tensor-parallel exchange): its own instantiation, batches of up to 4 rows
    const bool packets = p.tp_in.world > 0 && p.tp_in.packets;
    auto kernel = qgemv_kernel<BITS, LOGG, NB, NT, GATE_UP, false>;
    if (packets) {
        if constexpr (NB <= 4 && NT == 1) kernel = qgemv_kernel<BITS, LOGG, NB, NT, GATE_UP, true>;
        else return B200Q_ERR_UNSUPPORTED;
    }
    static bool configured[2][64] = {};   // per instantiation and device; a race only repeats the call
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[packets][dev & 63]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_cap) != cudaSuccess)
            return B200Q_ERR_LAUNCH;
        configured[packets][dev & 63] = true;
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
