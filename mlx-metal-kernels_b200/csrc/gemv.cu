// Weight-streaming quantized matvec / skinny GEMM for decode (sm_100a).
//
//   y[b, n] = sum_k x[b, k] * (code[n, k] - zero[n, k/G]) * scale[n, k/G]          b < B <= 16
//
// Design (one CTA per SM, 16 consumer warps + 1 producer warp):
//   * output rows are dealt out evenly to the CTAs; a CTA walks its rows in tiles of 16 (one
//     tensor-core M tile).
//   * the producer warp streams each tile through a ring of shared-memory stages with 1-D bulk
//     copies (TMA engine) signalled on mbarriers: one copy per weight row and k-chunk, sized
//     about 2 KB because the copy engine needs >= 2 KB per copy to saturate HBM (measured: 512 B
//     copies top out near 2.2 TB/s, 2 KB copies reach 7.2 TB/s), plus one copy each for the
//     tile's scales and zero points, which are contiguous over rows.  The producer starts before
//     griddepcontrol.wait: weights do not depend on the previous kernel.
//   * consumers dequantise in registers, fp16 via lop3/prmt + one HFMA2 per two codes, and feed
//     mma.sync.m16n8k16 with the WEIGHTS as the A operand (16 output rows) and the <= 8
//     activation rows as the B operand, accumulating in fp32.  The k order inside an instruction
//     is permuted so that every thread consumes the 16 bytes it loaded; the activations are
//     staged once per CTA in the matching order.
//   * zero points: the integer part rint(zero) is folded into the dequant constant, so the fp16
//     weight fed to the tensor core is (code - rint(zero)) * scale rounded once; the fractional
//     part and the rounding error of the constant are added back in fp32 in the epilogue through
//     per-group sums of the activations.
//   * 16 warps split K; partial tiles are reduced through shared memory in a fixed order
//     (bitwise reproducible), then clamp / round / optional residual add or SwiGLU.
//   * optional prologue: x := rmsnorm(x + residual) recomputed by every CTA from L2.
//
// Shapes outside the fast path (K not a multiple of 128 (q4) / 64 (q8), group size not a
// multiple of 32 / 16, unaligned pointers, B > 16 per launch) run the generic kernel at the
// bottom, which follows the reference arithmetic literally.
#include "common.cuh"

#include <algorithm>
#include <cmath>

namespace b200q {

B200Q_DEFINE_STATUS_WORD(gemv_read_status)

namespace {

constexpr int kConsumerWarps = 16;           // the reduction below assumes 16
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kTileRows = 16;
constexpr int kMaxBlockTiles = 4;             // tiles of a row block (one constants pass, one reduction)
constexpr int kRowPad = 64;                   // stage row stride = chunk bytes + 64: conflict-free 16-byte reads
constexpr uint32_t kWaitLimit = 1u << 21;
constexpr int kMaxStages = 8;
constexpr int kMaxGroupsPerLane = 8;          // groups per row <= 256 on the fast path

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
    int kc;                 // k per ring stage
    int n_kc;               // stages per (matrix, tile)
    int stages;
    int xk;                 // k per staged activation chunk (multiple of kc)
    int block_tiles;        // tiles per row block (1 unless the activations need several chunks)
    int logG;               // group size is a power of two on the fast path
    int dbg;                // measurement probes: bit 0 = skip the tensor-core work, bit 1 = do not wait for data
    int meta_by_tma;        // scales / zeros are fp16 and 16-byte aligned per tile: bulk-copied with the tile
    int rows_lo, rem;       // CTA c owns rows_lo (+1 if c < rem) rows
    uint32_t off_xperm, off_xsum, off_xscale, off_slots, off_red, off_meta, off_ring;
    uint32_t stage_bytes, row_stride, slots_buf_elems, red_buf_elems;
};

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

template <int BITS, int NT, bool GATE_UP, int GPL>
__global__ void __launch_bounds__(kThreads, 1) qgemv_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MATS = GATE_UP ? 2 : 1;
    constexpr int KS = BITS == 4 ? 128 : 64;     // k covered by the 64 bytes a quad reads from one row
    constexpr int NMMA = BITS == 4 ? 8 : 4;      // tensor-core instructions per k-step and tile
    constexpr int CH = NMMA / 2;                 // 16-byte activation chunks per k-step, thread and batch row
    constexpr int KT = KS / 4;                   // k owned by one thread of a quad in a k-step
    constexpr int MAXTB = kMaxBlockTiles / (MATS * NT);   // accumulator tiles kept in registers: 16 floats in all

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    uint64_t* meta_full = empty + kMaxStages;    // [2]
    uint64_t* meta_empty = meta_full + 2;        // [2]

    const int cta = blockIdx.x;
    const int r_lo = cta * p.rows_lo + min(cta, p.rem);
    const int r_cnt = p.rows_lo + (cta < p.rem ? 1 : 0);
    const int r_hi = r_lo + r_cnt;
    const int n_tiles = (r_cnt + kTileRows - 1) / kTileRows;
    const int TB = p.block_tiles;
    const int TBR = TB * kTileRows;              // rows of a full row block
    const int n_rb = (n_tiles + TB - 1) / TB;
    const int n_xc = (p.K + p.xk - 1) / p.xk;
    const int kc_per_xc = p.xk / p.kc;           // ring stages per (matrix, tile, activation chunk)
    const int Gn = p.Gn;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&meta_full[s], 1);
            mbar_init(&meta_empty[s], kConsumerWarps);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    uint8_t* ring = smem + p.off_ring;
    uint8_t* raw_meta = smem + p.off_meta;       // [2 buffers][MATS][scales | zeros][TBR][Gn] halves
    const uint32_t raw_mat_bytes = (uint32_t)2 * TBR * Gn * 2;
    const uint32_t raw_buf_bytes = MATS * raw_mat_bytes;

    // Both sides walk the stages in the same order: row block, activation chunk, tile, matrix, k-chunk.
    if (warp == kConsumerWarps) {
        // ------------------------------ producer warp ------------------------------------------
        bool ok = true;
        int p_slot = 0;
        uint32_t p_phase = 1;
        bool first_pass = true;
        for (int rb = 0; rb < n_rb; ++rb) {
            const int brow0 = r_lo + rb * TBR;
            const int brows = min(TBR, r_hi - brow0);
            if (p.meta_by_tma) {
                // scales / zero points of the whole row block: contiguous over rows, one copy each
                const int mb = rb & 1;
                if (rb >= 2)
                    ok = mbar_wait_bounded(&meta_empty[mb], ((rb >> 1) - 1) & 1, &g_device_status, EV_GEMV_EMPTY_WAIT,
                                           ok ? kWaitLimit : 64u) && ok;
                const uint32_t bytes = (uint32_t)brows * Gn * 2;
                if (lane == 0) {
                    uint32_t tx = 0;
                    for (int m = 0; m < MATS; ++m) tx += bytes * (p.z[m] != nullptr ? 2 : 1);
                    mbar_arrive_expect_tx(&meta_full[mb], tx);
                }
                __syncwarp();
                if (lane < 2 * MATS) {
                    const int m = lane >> 1;
                    const bool is_z = lane & 1;
                    const void* src = is_z ? p.z[m] : p.s[m];
                    if (src != nullptr)
                        bulk_g2s(raw_meta + mb * raw_buf_bytes + m * raw_mat_bytes + (is_z ? TBR * Gn * 2 : 0),
                                 reinterpret_cast<const uint8_t*>(src) + (size_t)brow0 * Gn * 2, bytes, &meta_full[mb]);
                }
            }
            for (int xc = 0; xc < n_xc; ++xc) {
                const int c_begin = xc * kc_per_xc;
                const int c_end = min(p.n_kc, c_begin + kc_per_xc);
                for (int tl = rb * TB; tl < min(n_tiles, (rb + 1) * TB); ++tl) {
                    const int row0 = r_lo + tl * kTileRows;
                    const int rows = min(kTileRows, r_hi - row0);
                    for (int m = 0; m < MATS; ++m) {
                        for (int c = c_begin; c < c_end; ++c) {
                            const int slot = p_slot;
                            if (!first_pass && !(p.dbg & 2))
                                ok = mbar_wait_bounded(&empty[slot], p_phase, &g_device_status, EV_GEMV_EMPTY_WAIT,
                                                       ok ? kWaitLimit : 64u) && ok;
                            if (p.dbg & 2) { if (++p_slot == p.stages) p_slot = 0; continue; }
                            if (++p_slot == p.stages) { p_slot = 0; p_phase ^= 1; first_pass = false; }
                            const int k0 = c * p.kc;
                            const int kcur = min(p.kc, p.K - k0);
                            const uint32_t bytes_row = (uint32_t)(kcur * BITS / 8);
                            uint8_t* stage = ring + (size_t)slot * p.stage_bytes;
                            if (lane == 0) mbar_arrive_expect_tx(&full[slot], bytes_row * rows);
                            __syncwarp();
                            if (lane < rows) {
                                const uint8_t* src = p.w[m] + (size_t)(row0 + lane) * p.row_bytes + (size_t)k0 * BITS / 8;
                                bulk_g2s(stage + (size_t)lane * p.row_stride, src, bytes_row, &full[slot]);
                            }
                        }
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------- consumer warps -----------------------------------------
    const int cw = warp;
    const int ctid = threadIdx.x;               // 0 .. kConsumerThreads-1
    const int g = lane >> 2;
    const int t = lane & 3;
    const int B = p.B;

    uint8_t* xperm = smem + p.off_xperm;
    float* xsum_e = reinterpret_cast<float*>(smem + p.off_xsum);      // [Gn][B] sums over even k (all k for q8)
    float* xsum_o = xsum_e + Gn * B;                                  // [Gn][B] sums over odd k
    float* xscale = reinterpret_cast<float*>(smem + p.off_xscale);    // [B]: 2^e ; [B..2B): inv_rms
    uint2* slots_base = reinterpret_cast<uint2*>(smem + p.off_slots); // [2][MATS][TBR][Gn] dequant constants
    float* red_base = reinterpret_cast<float*>(smem + p.off_red);     // [2]{ red [MATS][TBR][B][W] ; corr [MATS][TBR][B] }
    const bool has_zero = (p.z[0] != nullptr) || (MATS == 2 && p.z[1] != nullptr);

    // Dequant constants of one (row, group): the kernel computes fp16((off + q) * s + c) with
    // c = fp16(-(off + zr) * s), zr = rint(zero), off = 1024 (even k / q8) or 64 (odd k, q4): the
    // fused multiply-add rounds (q - zr) * s + e once, where e = c + (off + zr) * s is the (exactly
    // known) rounding error of c.  The zero-point term of the epilogue uses (ke, ko) = (z - zr) * s + e,
    // formed here in fp16: e is the rounding error of an fp16 product and therefore exact in fp16,
    // (z - zr) is exact, and only the small product (z - zr) * s is rounded.
    auto make_slot = [&](__half s16, __half z16, float& ke, float& ko) -> uint2 {
        const __half2 z2 = __half2half2(z16);
        const __half2 s2 = __half2half2(s16);
        const __half2 zr2 = __hmax2(__hmin2(h2rint(z2), __float2half2_rn(512.0f)), __float2half2_rn(-512.0f));
        const __half2 a2 = __hadd2(zr2, __halves2half2(__float2half_rn(1024.0f), __float2half_rn(64.0f)));
        const __half2 c2 = __hneg2(__hmul2(a2, s2));                                    // (c1024, c64)
        const __half2 k2 = __hfma2(__hsub2(z2, zr2), s2, __hfma2(a2, s2, c2));          // (ke, ko)
        ke = __low2float(k2);
        ko = __high2float(k2);
        uint2 v;
        v.x = (uint32_t)__half_as_ushort(s16) | ((uint32_t)__half_as_ushort(__low2half(c2)) << 16);
        v.y = (uint32_t)__half_as_ushort(__high2half(c2));
        return v;
    };

    pdl_wait();   // activations (and the output buffers) belong to the previous kernel until here

    // per batch row: inv_rms (norm prologue) and the power-of-two that maps bf16 rows into fp16 range
    const bool need_row_pass = (p.norm_w != nullptr) || (p.act_dtype == B200Q_BF16);
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
    const int logG = p.logG;
    if (has_zero && n_xc > 1) {
        // per-group sums of the activations exactly as the tensor cores will see them (scaled, fp16):
        // over even k and odd k separately for q4 (the two nibble positions use different offsets).
        // (When all activations are staged at once the sums are taken from shared memory below.)
        for (int i = ctid; i < Gn * B; i += kConsumerThreads) {
            const int gi = i / B;
            const int b = i - gi * B;
            const float inv = need_row_pass ? xscale[B + b] : 1.0f;
            const float down = need_row_pass ? 1.0f / xscale[b] : 1.0f;
            float se = 0.0f, so = 0.0f;
            for (int kk = gi << logG; kk < ((gi + 1) << logG); kk += 8) {
                float v[8];
                load8_act(p, b, kk, inv, false, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float h = __half2float(__float2half_rn(v[j] * down));
                    if (BITS == 4 && (j & 1)) so += h; else se += h;
                }
            }
            xsum_e[i] = se;
            xsum_o[i] = so;
        }
        named_bar_sync(1, kConsumerThreads);
    }

    // ---- stage activations of [xk0, xk0+xkn) in tensor-core operand order ----
    auto stage_x = [&](int xk0, int xkn, bool write_side) {
                const int chunks = xkn / 8;
#pragma unroll 4
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
                    const int ksx = kk / KS;
                    const int rem = kk - ksx * KS;
                    const int tt = rem / KT;
                    const int c = (rem - tt * KT) / 8;
                    uint4 out;
                    if (BITS == 4) {
                        // nibble order of one weight word after dequantisation: (0,4) (1,5) (2,6) (3,7)
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
                    *reinterpret_cast<uint4*>(xperm + ((uint32_t)((ksx * CH + c) * B + b) * 4 + tt) * 16) = out;
                }
    };
    if (n_xc == 1) {
        stage_x(0, p.K, cta == 0);
        named_bar_sync(1, kConsumerThreads);
        if (has_zero) {
            // per-group sums of the staged (fp16) activations for the zero-point term
            for (int i = ctid; i < Gn * B; i += kConsumerThreads) {
                const int gi = i / B;
                const int b = i - gi * B;
                float se = 0.0f, so = 0.0f;
                for (int kk = gi << logG; kk < ((gi + 1) << logG); kk += 8) {
                    const int ksx = kk / KS;
                    const int rem = kk - ksx * KS;
                    const int tt = rem / KT;
                    const int c = (rem - tt * KT) / 8;
                    const uint4 u = *reinterpret_cast<const uint4*>(xperm + ((uint32_t)((ksx * CH + c) * B + b) * 4 + tt) * 16);
                    const __half2 h0 = *reinterpret_cast<const __half2*>(&u.x);
                    const __half2 h1 = *reinterpret_cast<const __half2*>(&u.y);
                    const __half2 h2 = *reinterpret_cast<const __half2*>(&u.z);
                    const __half2 h3 = *reinterpret_cast<const __half2*>(&u.w);
                    const float a0 = __low2float(h0) + __high2float(h0), a1 = __low2float(h1) + __high2float(h1);
                    const float a2 = __low2float(h2) + __high2float(h2), a3 = __low2float(h3) + __high2float(h3);
                    if (BITS == 4) {            // registers 0 and 2 hold even k, 1 and 3 odd k
                        se += a0 + a2;
                        so += a1 + a3;
                    } else {
                        se += (a0 + a1) + (a2 + a3);
                    }
                }
                xsum_e[i] = se;
                xsum_o[i] = so;
            }
            named_bar_sync(1, kConsumerThreads);
        }
    }

    bool ok = true;
    int buf = 0;
    const float fmax_act = p.act_dtype == B200Q_F16 ? 65504.0f : 3.3895313892515355e38f;
    // per-thread constants of the inner loop
    const uint32_t w_off = (uint32_t)g * p.row_stride + t * 16;       // this thread's 16 bytes inside a stage row
    const uint32_t w_off8 = 8 * p.row_stride;
    const uint32_t x_step = (uint32_t)B * 64;                         // bytes between consecutive activation chunks
    const uint32_t x_lane = (uint32_t)t * 16;
    uint32_t x_nt[NT];                                                // byte offset of this lane's batch row per n-tile
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) x_nt[nt] = (uint32_t)min(nt * 8 + g, B - 1) * 64;
    const int n_stages = p.stages;
    const uint32_t stage_bytes = p.stage_bytes;
    int c_slot = 0;                  // ring slot and phase parity of the stage the consumer is at
    uint32_t c_phase = 0;

#pragma unroll 1
    for (int rb = 0; rb < n_rb; ++rb, buf ^= 1) {
        const int tile_begin = rb * TB;
        const int tile_end = min(n_tiles, tile_begin + TB);
        const int brow0 = r_lo + rb * TBR;
        const int block_rows = min(TBR, r_hi - brow0);
        uint2* slots = slots_base + (uint32_t)buf * p.slots_buf_elems;    // [MATS][TBR][Gn]
        float* red = red_base + (uint32_t)buf * p.red_buf_elems;          // [MATS][TBR][B][W] then corr [MATS][TBR][B]
        float* corr = red + (uint32_t)MATS * TBR * B * kConsumerWarps;

        // ---- dequant constants and zero-point term of the row block: warp per row, lanes over groups ----
        {
            const int mb = rb & 1;
            const __half* raw = reinterpret_cast<const __half*>(raw_meta + mb * raw_buf_bytes);
            if (p.meta_by_tma)
                ok = mbar_wait_bounded(&meta_full[mb], (rb >> 1) & 1, &g_device_status, EV_GEMV_FULL_WAIT,
                                       ok ? kWaitLimit : 64u) && ok;
            for (int rr = cw; rr < block_rows; rr += kConsumerWarps) {
#pragma unroll
                for (int m = 0; m < MATS; ++m) {
                    const bool hz = p.z[m] != nullptr;
                    const __half* rs = raw + (uint32_t)m * 2 * TBR * Gn + (uint32_t)rr * Gn;
                    const __half* rz = rs + (uint32_t)TBR * Gn;
                    const int64_t grow = (int64_t)(brow0 + rr) * Gn;
                    uint2* dst = slots + ((uint32_t)m * TBR + rr) * Gn;
                    // lane owns groups lane, lane + 32, ... (GPL of them: template parameter = ceil(Gn / 32) rounded up)
                    float ke[GPL], ko[GPL];
#pragma unroll
                    for (int j = 0; j < GPL; ++j) {
                        const int gi = lane + 32 * j;
                        ke[j] = ko[j] = 0.0f;
                        if (gi < Gn) {
                            __half s16, z16 = __ushort_as_half(0);
                            if (p.meta_by_tma) {
                                s16 = rs[gi];
                                if (hz) z16 = rz[gi];
                            } else {
                                s16 = __float2half_rn(load_as_f32(p.s[m], p.scale_dtype, grow + gi));
                                if (hz) z16 = __float2half_rn(load_as_f32(p.z[m], p.scale_dtype, grow + gi));
                            }
                            dst[gi] = make_slot(s16, z16, ke[j], ko[j]);
                        }
                    }
                    if (has_zero) {
                        // zero-point term of this row for every batch row: sum over groups of ke*Xe + ko*Xo
#pragma unroll 1
                        for (int b = 0; b < B; ++b) {
                            float part = 0.0f;
                            if (hz) {
#pragma unroll
                                for (int j = 0; j < GPL; ++j) {
                                    const int gi = lane + 32 * j;
                                    if (gi < Gn) part = fmaf(ke[j], xsum_e[gi * B + b], fmaf(ko[j], xsum_o[gi * B + b], part));
                                }
                            }
                            part = warp_sum(part);
                            if (lane == 0) corr[((uint32_t)m * TBR + rr) * B + b] = part;
                        }
                    }
                }
            }
            __syncwarp();
            if (p.meta_by_tma && lane == 0) mbar_arrive(&meta_empty[mb]);
        }

        // two accumulator sets per tile: consecutive tensor-core instructions do not depend on each other
        float acc[MATS][MAXTB][NT][4], acc2[MATS][MAXTB][NT][4];
#pragma unroll
        for (int m = 0; m < MATS; ++m)
#pragma unroll
            for (int tb = 0; tb < MAXTB; ++tb)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[m][tb][nt][i] = acc2[m][tb][nt][i] = 0.0f;

#pragma unroll 1
        for (int xc = 0; xc < n_xc; ++xc) {
            const int xk0 = xc * p.xk;
            const int xkn = min(p.xk, p.K - xk0);
            if (n_xc > 1) {
                named_bar_sync(1, kConsumerThreads);   // everyone is done with the previous chunk
                stage_x(xk0, xkn, cta == 0 && rb == 0);
            }
            if (xc == 0 || n_xc > 1) named_bar_sync(1, kConsumerThreads);   // constants / activations visible

            const int c_begin = xc * kc_per_xc;
            const int c_end = min(p.n_kc, c_begin + kc_per_xc);
#pragma unroll
            for (int tb = 0; tb < MAXTB; ++tb) {
                if (tile_begin + tb < tile_end) {
#pragma unroll
                    for (int m = 0; m < MATS; ++m) {
                        const uint2* slotsA = slots + ((uint32_t)m * TBR + tb * kTileRows + g) * Gn;
                        const uint2* slotsB = slotsA + 8 * Gn;
#pragma unroll 1
                        for (int c = c_begin; c < c_end; ++c) {
                            const int slot = c_slot;
                            if (!(p.dbg & 2))
                                ok = mbar_wait_bounded(&full[slot], c_phase, &g_device_status, EV_GEMV_FULL_WAIT,
                                                       ok ? kWaitLimit : 64u) && ok;
                            if (++c_slot == n_stages) { c_slot = 0; c_phase ^= 1; }
                            const int k0 = c * p.kc;
                            const int kcur = min(p.kc, p.K - k0);
                            const int nks = (p.dbg & 1) ? 0 : kcur / KS;
                            const uint8_t* stage_w = ring + (uint32_t)slot * stage_bytes + w_off;
                            const uint8_t* xbase = xperm + (uint32_t)((k0 - xk0) / KS) * CH * x_step + x_lane;
#pragma unroll 1
                            for (int ksl = cw; ksl < nks; ksl += kConsumerWarps) {
                                const int gi = (k0 + ksl * KS + t * KT) >> logG;
                                const uint8_t* pa = stage_w + ksl * 64;
                                const uint4 ua = *reinterpret_cast<const uint4*>(pa);
                                const uint4 ub = *reinterpret_cast<const uint4*>(pa + w_off8);
                                const uint2 ka = slotsA[gi];
                                const uint2 kb = slotsB[gi];
                                ScaleRegs sa, sb;
                                sa.s2 = prmt(ka.x, ka.x, 0x1010); sa.c1024 = prmt(ka.x, ka.x, 0x3232); sa.c64 = prmt(ka.y, ka.y, 0x1010);
                                sb.s2 = prmt(kb.x, kb.x, 0x1010); sb.c1024 = prmt(kb.x, kb.x, 0x3232); sb.c64 = prmt(kb.y, kb.y, 0x1010);
                                const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w};
                                const uint32_t wb[4] = {ub.x, ub.y, ub.z, ub.w};
                                const uint8_t* xk = xbase + (uint32_t)ksl * CH * x_step;
#pragma unroll
                                for (int ch = 0; ch < CH; ++ch) {
                                    // A fragments of MMA 2ch and 2ch+1
                                    uint32_t a[2][4];
                                    if (BITS == 4) {
                                        uint32_t va[4], vb[4];
                                        dequant_q4_word(wa[ch], sa, va);
                                        dequant_q4_word(wb[ch], sb, vb);
                                        a[0][0] = va[0]; a[0][1] = vb[0]; a[0][2] = va[1]; a[0][3] = vb[1];
                                        a[1][0] = va[2]; a[1][1] = vb[2]; a[1][2] = va[3]; a[1][3] = vb[3];
                                    } else {
                                        uint32_t va[2], vb[2];
                                        dequant_q8_word(wa[2 * ch], sa, va);
                                        dequant_q8_word(wb[2 * ch], sb, vb);
                                        a[0][0] = va[0]; a[0][1] = vb[0]; a[0][2] = va[1]; a[0][3] = vb[1];
                                        dequant_q8_word(wa[2 * ch + 1], sa, va);
                                        dequant_q8_word(wb[2 * ch + 1], sb, vb);
                                        a[1][0] = va[0]; a[1][1] = vb[0]; a[1][2] = va[1]; a[1][3] = vb[1];
                                    }
#pragma unroll
                                    for (int nt = 0; nt < NT; ++nt) {
                                        // columns >= B read a clamped (valid) batch row; their results are never stored
                                        const uint4 u = *reinterpret_cast<const uint4*>(xk + ch * x_step + x_nt[nt]);
                                        mma_m16n8k16(acc[m][tb][nt], a[0][0], a[0][1], a[0][2], a[0][3], u.x, u.y);
                                        mma_m16n8k16(acc2[m][tb][nt], a[1][0], a[1][1], a[1][2], a[1][3], u.z, u.w);
                                    }
                                }
                            }
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&empty[slot]);
                        }
                    }
                }
            }
        }

        // ---- partial tiles -> shared memory, layout [m][row][b][warp] ----
#pragma unroll
        for (int m = 0; m < MATS; ++m)
#pragma unroll
            for (int tb = 0; tb < MAXTB; ++tb)
                if (tile_begin + tb < tile_end) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int rr = tb * kTileRows + g + (i >> 1) * 8;
                            const int b = nt * 8 + 2 * t + (i & 1);
                            if (b < B) red[((((uint32_t)m * TBR + rr) * B + b) << 4) + cw] = acc[m][tb][nt][i] + acc2[m][tb][nt][i];
                        }
                }
        named_bar_sync(1, kConsumerThreads);

        // ---- reduction over the warps (fixed order: xor tree inside 16 lanes) + epilogue.  red / corr /
        //      slots are double-buffered, so the next row block may start while slower warps are here. ----
        const int items = block_rows * B;            // (row, batch row) pairs of this block
        for (int base = 0; base < items; base += kConsumerThreads / 16) {
            const int item = base + (ctid >> 4);
            const int w = ctid & 15;
            const bool live = item < items;
            const int rr = live ? item / B : 0;
            const int b = live ? item - rr * B : 0;
            float val[MATS];
#pragma unroll
            for (int m = 0; m < MATS; ++m) {
                float s = live ? red[((((uint32_t)m * TBR + rr) * B + b) << 4) + w] : 0.0f;
                s += __shfl_xor_sync(0xffffffffu, s, 8);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                if (has_zero && live) s -= corr[((uint32_t)m * TBR + rr) * B + b];
                if (need_row_pass) s *= xscale[b];
                val[m] = round_act(fminf(fmaxf(s, -fmax_act), fmax_act), p.act_dtype);
            }
            if (live && w == 0) {
                const int64_t o = (int64_t)b * p.N + brow0 + rr;
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
    }
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
inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

template <int BITS, int NT, bool GATE_UP, int GPL>
int launch_fast(GemvParams& p, cudaStream_t stream) {
    constexpr int MATS = GATE_UP ? 2 : 1;
    constexpr int KS = BITS == 4 ? 128 : 64;
    const int sms = sm_count();
    const uint32_t smem_cap = (uint32_t)max_smem_optin();

    // k per stage: per-row copies of about 2 KB, whole k-steps and whole groups
    const int unit = std::max(KS, p.G);
    p.logG = 0;
    while ((1 << p.logG) < p.G) ++p.logG;
    int kc = tuning_get("gemv.stage_k");
    if (kc <= 0) {
        const int target_bytes = 2048;
        const int n = std::max(1, (p.row_bytes + target_bytes / 2) / target_bytes);
        kc = (p.K + n - 1) / n;
    }
    kc = std::min(p.K, std::max(unit, (kc + unit - 1) / unit * unit));
    p.kc = kc;
    p.n_kc = (p.K + kc - 1) / kc;

    int grid = (int)std::min<int64_t>(sms, (p.N + kTileRows - 1) / kTileRows);
    const int ctas_per_sm = tuning_get("gemv.ctas_per_sm");
    if (ctas_per_sm > 1) grid = (int)std::min<int64_t>((int64_t)sms * ctas_per_sm, (p.N + kTileRows - 1) / kTileRows);
    grid = std::max(grid, 1);
    p.rows_lo = p.N / grid;
    p.rem = p.N % grid;
    const int max_tiles = (p.rows_lo + (p.rem ? 1 : 0) + kTileRows - 1) / kTileRows;

    // scales / zeros ride along with the first stage of every tile when they are fp16 and every tile
    // starts on a 16-byte boundary
    p.meta_by_tma = p.scale_dtype == B200Q_F16 && (p.Gn % 8 == 0) && aligned16(p.s[0]) &&
                    (p.z[0] == nullptr || aligned16(p.z[0])) &&
                    (MATS == 1 || (aligned16(p.s[1]) && (p.z[1] == nullptr || aligned16(p.z[1]))));
    p.row_stride = (uint32_t)(kc * BITS / 8) + kRowPad;
    p.stage_bytes = align_up(kTileRows * p.row_stride, 128);

    // Tiles per row block (amortises the constants pass and the reduction) and the activation chunk
    // (whole K when it fits the budget, else a multiple of kc): first choice that leaves room for a
    // two-stage ring.
    uint32_t off = 0;
    bool fits = false;
    const uint32_t budgets[3] = {64 * 1024, 32 * 1024, 16 * 1024};
    for (int tb_try = std::min(max_tiles, kMaxBlockTiles / (MATS * NT)); tb_try >= 1 && !fits; --tb_try) {
        const uint32_t tbr = (uint32_t)tb_try * kTileRows;
        // keep the double-buffered constants and reduction scratch moderate
        if (tb_try > 1 && (2u * MATS * tbr * p.Gn * 8 > 64 * 1024 || 2u * (kConsumerWarps + 1) * MATS * tbr * p.B * 4 > 48 * 1024))
            continue;
        for (int bi = 0; bi < 3 && !fits; ++bi) {
            int xk = p.n_kc * kc;
            if ((size_t)p.K * p.B * 2 > budgets[bi]) xk = std::max(1, (int)(budgets[bi] / ((size_t)p.B * 2 * kc))) * kc;
            const int n_xc = (p.K + xk - 1) / xk;
            if (n_xc == 1 && bi != 0) continue;   // nothing new to try
            p.xk = xk;
            p.block_tiles = tb_try;
            p.slots_buf_elems = (uint32_t)MATS * tbr * p.Gn;
            p.red_buf_elems = (uint32_t)(kConsumerWarps + 1) * MATS * tbr * p.B;
            off = align_up((2 * kMaxStages + 4) * sizeof(uint64_t), 128);
            p.off_xperm = off;  off += align_up((uint32_t)xk * p.B * 2, 128);
            p.off_xsum = off;   off += align_up((uint32_t)2 * p.Gn * p.B * 4, 128);
            p.off_xscale = off; off += align_up((uint32_t)p.B * 2 * 4, 128);
            p.off_slots = off;  off += align_up(2 * p.slots_buf_elems * 8, 128);
            p.off_red = off;    off += align_up(2 * p.red_buf_elems * 4, 128);
            p.off_meta = off;   off += p.meta_by_tma ? align_up(2u * MATS * 2 * tbr * p.Gn * 2, 128) : 0;
            p.off_ring = off;
            fits = off + 2ull * p.stage_bytes <= smem_cap;
        }
    }
    if (!fits) return B200Q_ERR_UNSUPPORTED;

    // ring depth: everything the CTA will ever stream if that is small (keeps two CTAs resident per SM, so
    // the next kernel's prefetch overlaps this kernel's tail), else as deep as shared memory allows
    const int total_stages = max_tiles * MATS * p.n_kc;
    p.logG = 0;
    while ((1 << p.logG) < p.G) ++p.logG;
    p.dbg = tuning_get("gemv.dbg");
    int stages = tuning_get("gemv.stages");
    if (stages <= 0) stages = kMaxStages;
    stages = std::min({stages, kMaxStages, std::max(2, total_stages)});
    while (stages > 2 && off + (uint64_t)stages * p.stage_bytes > smem_cap) --stages;
    p.stages = stages;
    const uint64_t total = off + (uint64_t)stages * p.stage_bytes;

    auto kernel = qgemv_kernel<BITS, NT, GATE_UP, GPL>;
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

template <bool GATE_UP>
int launch_generic(const GemvParams& p, int bits, cudaStream_t stream) {
    const int warps = 8;
    const int grid = (int)((p.N + warps - 1) / warps);
    qgemv_generic_kernel<GATE_UP><<<grid, warps * 32, 0, stream>>>(p, bits);
    return finish_launch();
}

// The generic kernel has no norm prologue: the caller runs the stand-alone rmsnorm kernel first when
// the fast path does not apply.
bool fast_path_ok(const GemvParams& p, int bits) {
    const int ks = bits == 4 ? 128 : 64;
    const int kt = ks / 4;
    if (tuning_get("gemv.force_generic")) return false;
    if (p.K % ks != 0 || p.G % kt != 0 || p.K % p.G != 0 || (p.G & (p.G - 1)) != 0) return false;
    if (p.B > 16 || p.Gn > 32 * kMaxGroupsPerLane) return false;
    if ((size_t)p.Gn * kTileRows * 8 * 2 * (p.w[1] ? 2 : 1) > 64 * 1024) return false;
    if (!aligned16(p.x) || !aligned16(p.w[0]) || (p.w[1] != nullptr && !aligned16(p.w[1]))) return false;
    if (p.res_in != nullptr && !aligned16(p.res_in)) return false;
    if (p.z_out != nullptr && !aligned16(p.z_out)) return false;
    if (p.normed_out != nullptr && !aligned16(p.normed_out)) return false;
    if (p.row_bytes % 16 != 0) return false;
    return true;
}

template <int BITS, int NT, bool GATE_UP>
int dispatch_gpl(GemvParams& p, cudaStream_t stream) {
    const int gpl = (p.Gn + 31) / 32;      // groups of one row handled per lane in the constants pass
    if (gpl <= 1) return launch_fast<BITS, NT, GATE_UP, 1>(p, stream);
    if (gpl <= 2) return launch_fast<BITS, NT, GATE_UP, 2>(p, stream);
    if (gpl <= 4) return launch_fast<BITS, NT, GATE_UP, 4>(p, stream);
    return launch_fast<BITS, NT, GATE_UP, 8>(p, stream);
}

template <bool GATE_UP>
int dispatch_fast(int bits, GemvParams& p, cudaStream_t stream) {
    if (bits == 4) return p.B <= 8 ? dispatch_gpl<4, 1, GATE_UP>(p, stream) : dispatch_gpl<4, 2, GATE_UP>(p, stream);
    return p.B <= 8 ? dispatch_gpl<8, 1, GATE_UP>(p, stream) : dispatch_gpl<8, 2, GATE_UP>(p, stream);
}

}  // namespace

// Declared in api.cu
int rmsnorm_residual_launch(const void* x, const void* residual, const void* weight, void* y, void* z_out,
                            int64_t rows, int64_t D, float eps, int dtype, int w_dtype, cudaStream_t stream);

int qmatvec_impl(int bits, const void* x, const uint8_t* codes, const void* scales, const void* zeros,
                 const void* residual, void* y, int B, int64_t N, int64_t K, int group_size, int act_dtype,
                 int scale_dtype, const void* residual_in, const void* norm_weight, int norm_w_dtype, float eps,
                 void* z_out, void* normed_out, cudaStream_t stream) {
    if ((bits != 4 && bits != 8) || x == nullptr || codes == nullptr || scales == nullptr || y == nullptr)
        return B200Q_ERR_BAD_ARG;
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
    for (int b0 = 0; b0 < B; b0 += 16) {
        GemvParams p = {};
        const int bn = std::min(16, B - b0);
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
        int rc = fast_path_ok(p, bits) ? dispatch_fast<false>(bits, p, stream) : B200Q_ERR_UNSUPPORTED;
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
    }
    return B200Q_OK;
}

int gate_up_impl(int bits, const void* x, const uint8_t* gate_codes, const uint8_t* up_codes, const void* gate_scales,
                 const void* up_scales, const void* gate_zeros, const void* up_zeros, void* gate_out, void* up_out,
                 void* act_out, const void* residual_in, const void* norm_weight, float eps, void* z_out,
                 void* normed_out, int rows, int64_t N, int64_t K, int group_size, int act_dtype, int scale_dtype,
                 int norm_w_dtype, cudaStream_t stream) {
    if ((bits != 4 && bits != 8) || x == nullptr || gate_codes == nullptr || up_codes == nullptr ||
        gate_scales == nullptr || up_scales == nullptr)
        return B200Q_ERR_BAD_ARG;
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
    for (int b0 = 0; b0 < rows; b0 += 16) {
        GemvParams p = {};
        const int bn = std::min(16, rows - b0);
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
        int rc;
        rc = fast_path_ok(p, bits) ? dispatch_fast<true>(bits, p, stream) : B200Q_ERR_UNSUPPORTED;
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
    }
    return B200Q_OK;
}

}  // namespace b200q
