// Weight-streaming quantized matvec / skinny GEMM for decode (sm_100a).
//
//   y[b, n] = sum_k x[b, k] * (code[n, k] - zero[n, k/G]) * scale[n, k/G]          b < B <= 16
//
// Design (one CTA per SM slot, 8 consumer warps + 1 producer warp):
//   * output rows are dealt out evenly to the CTAs; a CTA walks its rows in blocks of 32.
//   * the producer warp streams the block's weight rows through a ring of shared-memory stages
//     with 1-D bulk copies (TMA engine, one copy per row and k-chunk) signalled on mbarriers.  It
//     starts before griddepcontrol.wait: weights do not depend on the previous kernel.
//   * consumers dequantise in registers, fp16(code*scale) via lop3/prmt + one HFMA2 per two
//     codes, and feed mma.sync.m16n8k16 with the WEIGHTS as the A operand (16 output rows) and
//     the <= 8 activation rows as the B operand, accumulating in fp32.  The k order inside an
//     instruction is permuted so that every thread consumes the 16 bytes it loaded; the
//     activations are staged once per CTA in the matching order.
//   * zero points: the integer part rint(zero) is folded into the dequant constant, so the fp16
//     weight fed to the tensor core is (code - rint(zero)) * scale rounded once; the fractional
//     part and the rounding error of the constant are added back in fp32 in the epilogue through
//     per-group sums of the activations.
//   * warps split K; partial tiles are reduced through shared memory in a fixed order
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

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kRowTiles = 2;                  // 16-row MMA tiles per row block
constexpr int kRowBlock = kRowTiles * 16;
constexpr int kRowPad = 64;                   // stage row stride = chunk bytes + 64: conflict-free 16-byte reads
constexpr uint32_t kWaitLimit = 1u << 21;
constexpr int kMaxStages = 12;

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
    int stages;
    int xk;                 // k per staged activation chunk (multiple of kc)
    int rows_lo, rem;       // CTA c owns rows_lo (+1 if c < rem) rows
    uint32_t off_xperm, off_xsum, off_xscale, off_scales, off_corr, off_red, off_ring;
    uint32_t stage_bytes, row_stride;
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

template <int BITS, int NT, bool GATE_UP>
__global__ void __launch_bounds__(kThreads, 1) qgemv_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MATS = GATE_UP ? 2 : 1;
    constexpr int KS = BITS == 4 ? 128 : 64;     // k covered by the 64 bytes a quad reads from one row
    constexpr int NMMA = BITS == 4 ? 8 : 4;      // tensor-core instructions per k-step and tile
    constexpr int CH = NMMA / 2;                 // 16-byte activation chunks per k-step, thread and batch row
    constexpr int KT = KS / 4;                   // k owned by one thread of a quad in a k-step

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;

    const int cta = blockIdx.x;
    const int r_lo = cta * p.rows_lo + min(cta, p.rem);
    const int r_cnt = p.rows_lo + (cta < p.rem ? 1 : 0);
    const int r_hi = r_lo + r_cnt;
    const int n_rb = (r_cnt + kRowBlock - 1) / kRowBlock;
    const int rb_rows = n_rb > 0 ? (r_cnt + n_rb - 1) / n_rb : 0;   // balanced row blocks
    const int n_st = (p.K + p.kc - 1) / p.kc;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    uint8_t* ring = smem + p.off_ring;

    if (warp == kConsumerWarps) {
        // ------------------------------ producer warp ------------------------------------------
        uint32_t it = 0;
        bool ok = true;
        for (int rb = 0; rb < n_rb; ++rb) {
            const int row0 = r_lo + rb * rb_rows;
            const int rows = min(rb_rows, r_hi - row0);
            for (int st = 0; st < n_st; ++st, ++it) {
                const int slot = it % p.stages;
                if (it >= (uint32_t)p.stages) {
                    const uint32_t parity = ((it / p.stages) - 1) & 1;
                    ok = mbar_wait_bounded(&empty[slot], parity, &g_device_status, EV_GEMV_EMPTY_WAIT,
                                           ok ? kWaitLimit : 64u) && ok;
                }
                const int k0 = st * p.kc;
                const int kcur = min(p.kc, p.K - k0);
                const uint32_t bytes_row = (uint32_t)(kcur * BITS / 8);
                if (lane == 0) mbar_arrive_expect_tx(&full[slot], bytes_row * rows * MATS);
                __syncwarp();
                uint8_t* stage = ring + (size_t)slot * p.stage_bytes;
                for (int i = lane; i < rows * MATS; i += 32) {
                    const int m = i / rows;
                    const int r = i - m * rows;
                    const uint8_t* src = p.w[m] + (size_t)(row0 + r) * p.row_bytes + (size_t)k0 * BITS / 8;
                    bulk_g2s(stage + (size_t)(m * kRowBlock + r) * p.row_stride, src, bytes_row, &full[slot]);
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
    float* xsum = reinterpret_cast<float*>(smem + p.off_xsum);        // [2][Gn][B]: even-k / odd-k sums per group
    float* xscale = reinterpret_cast<float*>(smem + p.off_xscale);    // [B]: 2^e ; [B..2B): inv_rms
    uint2* slots = reinterpret_cast<uint2*>(smem + p.off_scales);     // [MATS][kRowBlock][Gn] dequant constants
    __half* zr16 = reinterpret_cast<__half*>(smem + p.off_corr);      // [MATS][kRowBlock][Gn] integer part of zero
    float* red = reinterpret_cast<float*>(smem + p.off_red);          // [W][MATS][kRowBlock][B]
    const bool has_zero = (p.z[0] != nullptr) || (MATS == 2 && p.z[1] != nullptr);
    float* xsum_e = xsum;
    float* xsum_o = xsum + p.Gn * B;

    // Dequant constants of one (row, group): the kernel computes fp16((off + q) * s + c) with
    // c = fp16(-(off + zr) * s), zr = rint(zero), off = 1024 (even k / q8) or 64 (odd k, q4): the
    // fused multiply-add rounds (q - zr) * s + e once, where e = c + (off + zr) * s is the (exactly
    // known) rounding error of c.  e and the fractional part of the zero point go into the fp32
    // correction term of the epilogue.
    auto build_slot = [&](int m, int r, int gi, int row) {
        const float sf = __half2float(__float2half_rn(load_as_f32(p.s[m], p.scale_dtype, (int64_t)row * p.Gn + gi)));
        float zr = 0.0f, dz = 0.0f;
        if (p.z[m] != nullptr) {
            const float z = load_as_f32(p.z[m], p.scale_dtype, (int64_t)row * p.Gn + gi);
            zr = fminf(fmaxf(rintf(z), -512.0f), 512.0f);
            dz = z - zr;
        }
        const __half s16 = __float2half_rn(sf);
        const __half c1024 = __float2half_rn(-(1024.0f + zr) * sf);
        const __half c64 = __float2half_rn(-(64.0f + zr) * sf);
        uint2 v;
        v.x = (uint32_t)__half_as_ushort(s16) | ((uint32_t)__half_as_ushort(c1024) << 16);
        v.y = (uint32_t)__half_as_ushort(c64) | ((uint32_t)__half_as_ushort(__float2half_rn(dz)) << 16);
        slots[(m * kRowBlock + r) * p.Gn + gi] = v;
        zr16[(m * kRowBlock + r) * p.Gn + gi] = __float2half_rn(zr);
    };
    auto stage_slots = [&](int row0, int rows) {
        for (int m = 0; m < MATS; ++m)
            for (int i = ctid; i < rows * p.Gn; i += kConsumerThreads) {
                const int r = i / p.Gn;
                build_slot(m, r, i - r * p.Gn, row0 + r);
            }
    };

    // Scales and zero points do not depend on the previous kernel either: convert the first row
    // block's constants before waiting on it.
    {
        const int rows0 = min(rb_rows, r_cnt);
        stage_slots(r_lo, rows0);
    }

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

    uint32_t it = 0;
    bool ok = true;
    const int n_xc = (p.K + p.xk - 1) / p.xk;
    const int st_per_xc = p.xk / p.kc;
    const float fmax_act = p.act_dtype == B200Q_F16 ? 65504.0f : 3.3895313892515355e38f;

    for (int rb = 0; rb < n_rb; ++rb) {
        const int row0 = r_lo + rb * rb_rows;
        const int rows = min(rb_rows, r_hi - row0);
        if (rb > 0) stage_slots(row0, rows);     // (row block 0 was converted before the wait)

        float acc[MATS][kRowTiles][NT][4];
#pragma unroll
        for (int m = 0; m < MATS; ++m)
#pragma unroll
            for (int rt = 0; rt < kRowTiles; ++rt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[m][rt][nt][i] = 0.0f;

        for (int xc = 0; xc < n_xc; ++xc) {
            const int xk0 = xc * p.xk;
            const int xkn = min(p.xk, p.K - xk0);
            if (n_xc > 1 || rb == 0) {
                if (n_xc > 1) named_bar_sync(1, kConsumerThreads);   // everyone is done with the previous chunk
                // ---- stage activations of [xk0, xk0+xkn) in tensor-core operand order ----
                const int chunks = xkn / 8;
                for (int i = ctid; i < B * chunks; i += kConsumerThreads) {
                    const int b = i / chunks;
                    const int kk = (i - b * chunks) * 8;
                    float v[8];
                    const float inv = need_row_pass ? xscale[B + b] : 1.0f;
                    const float down = need_row_pass ? 1.0f / xscale[b] : 1.0f;
                    load8_act(p, b, xk0 + kk, inv, cta == 0 && rb == 0, v);
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
                    *reinterpret_cast<uint4*>(xperm + ((size_t)((ksx * CH + c) * B + b) * 4 + tt) * 16) = out;
                }
                named_bar_sync(1, kConsumerThreads);
                if (has_zero && rb == 0) {
                    // per-group sums of the staged (fp16) activations for the zero-point term; read again
                    // only after the reduction barrier at the end of the row block
                    const int g0 = xk0 / p.G;
                    const int gn = xkn / p.G;
                    for (int i = ctid; i < gn * B; i += kConsumerThreads) {
                        const int gi = i / B;
                        const int b = i - gi * B;
                        float se = 0.0f, so = 0.0f;
                        for (int kk = gi * p.G; kk < (gi + 1) * p.G; kk += 8) {
                            const int ksx = kk / KS;
                            const int rem = kk - ksx * KS;
                            const int tt = rem / KT;
                            const int c = (rem - tt * KT) / 8;
                            const uint4 u = *reinterpret_cast<const uint4*>(
                                xperm + ((size_t)((ksx * CH + c) * B + b) * 4 + tt) * 16);
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
                        xsum_e[(g0 + gi) * B + b] = se;
                        xsum_o[(g0 + gi) * B + b] = so;
                    }
                }
            } else if (xc == 0) {
                named_bar_sync(1, kConsumerThreads);   // constants of this row block are visible
            }

            const int st_begin = xc * st_per_xc;
            const int st_end = min(n_st, st_begin + st_per_xc);
            for (int st = st_begin; st < st_end; ++st, ++it) {
                const int slot = it % p.stages;
                ok = mbar_wait_bounded(&full[slot], (it / p.stages) & 1, &g_device_status, EV_GEMV_FULL_WAIT,
                                       ok ? kWaitLimit : 64u) && ok;
                const int k0 = st * p.kc;
                const int kcur = min(p.kc, p.K - k0);
                const int nks = kcur / KS;
                const uint8_t* stage = ring + (size_t)slot * p.stage_bytes;
                for (int ksl = cw; ksl < nks; ksl += kConsumerWarps) {
                    const int kg = k0 + ksl * KS;
                    const int ksx = (kg - xk0) / KS;
                    const int gi = (kg + t * KT) / p.G;
                    uint32_t bf[NT == 1 ? CH : 1][4];
                    if (NT == 1) {
#pragma unroll
                        for (int c = 0; c < CH; ++c) {
                            uint4 u = make_uint4(0, 0, 0, 0);
                            if (g < B)
                                u = *reinterpret_cast<const uint4*>(xperm + ((size_t)((ksx * CH + c) * B + g) * 4 + t) * 16);
                            bf[c][0] = u.x; bf[c][1] = u.y; bf[c][2] = u.z; bf[c][3] = u.w;
                        }
                    }
#pragma unroll
                    for (int rt = 0; rt < kRowTiles; ++rt) {
                        if (rt * 16 < rows) {
#pragma unroll
                            for (int m = 0; m < MATS; ++m) {
                                const int rowA = m * kRowBlock + rt * 16 + g;
                                const uint8_t* pa = stage + (size_t)rowA * p.row_stride + ksl * 64 + t * 16;
                                const uint4 ua = *reinterpret_cast<const uint4*>(pa);
                                const uint4 ub = *reinterpret_cast<const uint4*>(pa + 8 * p.row_stride);
                                const uint2 ka = slots[rowA * p.Gn + gi];
                                const uint2 kb = slots[(rowA + 8) * p.Gn + gi];
                                ScaleRegs sa, sb;
                                sa.s2 = prmt(ka.x, ka.x, 0x1010); sa.c1024 = prmt(ka.x, ka.x, 0x3232); sa.c64 = prmt(ka.y, ka.y, 0x1010);
                                sb.s2 = prmt(kb.x, kb.x, 0x1010); sb.c1024 = prmt(kb.x, kb.x, 0x3232); sb.c64 = prmt(kb.y, kb.y, 0x1010);
                                const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w};
                                const uint32_t wb[4] = {ub.x, ub.y, ub.z, ub.w};
#pragma unroll
                                for (int c = 0; c < CH; ++c) {
                                    // A fragments of MMA 2c and 2c+1
                                    uint32_t a[2][4];
                                    if (BITS == 4) {
                                        uint32_t va[4], vb[4];
                                        dequant_q4_word(wa[c], sa, va);
                                        dequant_q4_word(wb[c], sb, vb);
                                        a[0][0] = va[0]; a[0][1] = vb[0]; a[0][2] = va[1]; a[0][3] = vb[1];
                                        a[1][0] = va[2]; a[1][1] = vb[2]; a[1][2] = va[3]; a[1][3] = vb[3];
                                    } else {
                                        uint32_t va[2], vb[2];
                                        dequant_q8_word(wa[2 * c], sa, va);
                                        dequant_q8_word(wb[2 * c], sb, vb);
                                        a[0][0] = va[0]; a[0][1] = vb[0]; a[0][2] = va[1]; a[0][3] = vb[1];
                                        dequant_q8_word(wa[2 * c + 1], sa, va);
                                        dequant_q8_word(wb[2 * c + 1], sb, vb);
                                        a[1][0] = va[0]; a[1][1] = vb[0]; a[1][2] = va[1]; a[1][3] = vb[1];
                                    }
#pragma unroll
                                    for (int nt = 0; nt < NT; ++nt) {
                                        uint32_t b0, b1, b2, b3;
                                        if (NT == 1) {
                                            b0 = bf[c][0]; b1 = bf[c][1]; b2 = bf[c][2]; b3 = bf[c][3];
                                        } else {
                                            uint4 u = make_uint4(0, 0, 0, 0);
                                            const int bb = nt * 8 + g;
                                            if (bb < B)
                                                u = *reinterpret_cast<const uint4*>(
                                                    xperm + ((size_t)((ksx * CH + c) * B + bb) * 4 + t) * 16);
                                            b0 = u.x; b1 = u.y; b2 = u.z; b3 = u.w;
                                        }
                                        mma_m16n8k16(acc[m][rt][nt], a[0][0], a[0][1], a[0][2], a[0][3], b0, b1);
                                        mma_m16n8k16(acc[m][rt][nt], a[1][0], a[1][1], a[1][2], a[1][3], b2, b3);
                                    }
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);
            }
        }

        // ---- cross-warp reduction (fixed order) ----
#pragma unroll
        for (int m = 0; m < MATS; ++m)
#pragma unroll
            for (int rt = 0; rt < kRowTiles; ++rt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int r = rt * 16 + g + (i >> 1) * 8;
                        const int b = nt * 8 + 2 * t + (i & 1);
                        if (b < B) red[((cw * MATS + m) * kRowBlock + r) * B + b] = acc[m][rt][nt][i];
                    }
        named_bar_sync(1, kConsumerThreads);

        // ---- epilogue: one warp per output row.  Lanes first split the groups of the row for the
        //      zero-point term, then lane b finishes batch row b. ----
        for (int r = cw; r < rows; r += kConsumerWarps) {
            float val[MATS];
#pragma unroll
            for (int m = 0; m < MATS; ++m) {
                float mine = 0.0f;       // correction for batch row == lane
                if (has_zero && p.z[m] != nullptr) {
                    float part[NT * 8];
#pragma unroll
                    for (int b = 0; b < NT * 8; ++b) part[b] = 0.0f;
                    for (int gi = lane; gi < p.Gn; gi += 32) {
                        const uint2 k = slots[(m * kRowBlock + r) * p.Gn + gi];
                        const float sf = __half2float(__ushort_as_half((unsigned short)(k.x & 0xFFFF)));
                        const float c1024 = __half2float(__ushort_as_half((unsigned short)(k.x >> 16)));
                        const float c64 = __half2float(__ushort_as_half((unsigned short)(k.y & 0xFFFF)));
                        const float dz = __half2float(__ushort_as_half((unsigned short)(k.y >> 16)));
                        const float zr = __half2float(zr16[(m * kRowBlock + r) * p.Gn + gi]);
                        const float base = dz * sf;
                        const float ke = base + fmaf(1024.0f + zr, sf, c1024);
                        const float ko = base + fmaf(64.0f + zr, sf, c64);
#pragma unroll
                        for (int b = 0; b < NT * 8; ++b)
                            if (b < B) part[b] = fmaf(ke, xsum_e[gi * B + b], fmaf(ko, xsum_o[gi * B + b], part[b]));
                    }
#pragma unroll
                    for (int b = 0; b < NT * 8; ++b) {
                        if (b < B) {
                            const float s = warp_sum(part[b]);
                            if (lane == b) mine = s;
                        }
                    }
                }
                float s = 0.0f;
                if (lane < B) {
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; ++w) s += red[((w * MATS + m) * kRowBlock + r) * B + lane];
                    s -= mine;
                    if (need_row_pass) s *= xscale[lane];
                }
                val[m] = round_act(fminf(fmaxf(s, -fmax_act), fmax_act), p.act_dtype);
            }
            if (lane < B) {
                const int64_t o = (int64_t)lane * p.N + row0 + r;
                auto store = [&](void* base, float v) {
                    if (p.act_dtype == B200Q_F16) reinterpret_cast<__half*>(base)[o] = __float2half_rn(v);
                    else reinterpret_cast<__nv_bfloat16*>(base)[o] = __float2bfloat16_rn(v);
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
        named_bar_sync(1, kConsumerThreads);   // red / constants are reused by the next row block
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

template <int BITS, int NT, bool GATE_UP>
int launch_fast(GemvParams& p, cudaStream_t stream) {
    constexpr int MATS = GATE_UP ? 2 : 1;
    constexpr int KS = BITS == 4 ? 128 : 64;
    const int sms = sm_count();
    int ctas_per_sm = tuning_get("gemv.ctas_per_sm");
    if (ctas_per_sm <= 0) ctas_per_sm = 1;
    // k per stage: default 8 k-steps (one per consumer warp)
    int kc = tuning_get("gemv.stage_k");
    if (kc <= 0) kc = KS * kConsumerWarps;
    {
        const int unit = std::max(KS, p.G);   // a stage holds whole k-steps and whole groups
        kc = std::max(unit, kc / unit * unit);
    }
    kc = std::min(kc, p.K);
    int stages = tuning_get("gemv.stages");
    if (stages <= 0) stages = 4;
    stages = std::min(stages, kMaxStages);

    // activation chunk: whole K when it fits the budget, else a multiple of kc
    const uint32_t x_budget = 64 * 1024;
    int xk = p.K;
    if ((size_t)p.K * p.B * 2 > x_budget) {
        xk = (int)(x_budget / (p.B * 2)) / kc * kc;
        if (xk < kc) xk = kc;
    }
    p.kc = kc;
    p.xk = xk;
    p.stages = stages;

    int grid = std::min<int64_t>((int64_t)sms * ctas_per_sm, (p.N + 15) / 16);
    grid = std::max(grid, 1);
    p.rows_lo = p.N / grid;
    p.rem = p.N % grid;

    p.row_stride = (uint32_t)(kc * BITS / 8) + kRowPad;
    p.stage_bytes = MATS * kRowBlock * p.row_stride;
    uint32_t off = 2 * kMaxStages * sizeof(uint64_t);
    off = align_up(off, 128);
    p.off_xperm = off;  off += align_up((uint32_t)xk * p.B * 2, 128);
    p.off_xsum = off;   off += align_up((uint32_t)2 * p.Gn * p.B * 4, 128);
    p.off_xscale = off; off += align_up((uint32_t)p.B * 2 * 4, 128);
    p.off_scales = off; off += align_up((uint32_t)MATS * kRowBlock * p.Gn * 8, 128);   // dequant constants
    p.off_corr = off;   off += align_up((uint32_t)MATS * kRowBlock * p.Gn * 2, 128);   // integer zero points
    p.off_red = off;    off += align_up((uint32_t)kConsumerWarps * MATS * kRowBlock * p.B * 4, 128);
    p.off_ring = off;
    const uint32_t smem_cap = (uint32_t)max_smem_optin();
    while (stages > 2 && off + (uint64_t)stages * p.stage_bytes > smem_cap) --stages;
    p.stages = stages;
    const uint64_t total = off + (uint64_t)stages * p.stage_bytes;
    if (total > smem_cap) return B200Q_ERR_UNSUPPORTED;

    auto kernel = qgemv_kernel<BITS, NT, GATE_UP>;
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

// The generic kernel has no norm prologue: it is run after the stand-alone rmsnorm kernel by the
// caller (see api.cu) when the fast path does not apply.
bool fast_path_ok(const GemvParams& p, int bits) {
    const int ks = bits == 4 ? 128 : 64;
    const int kt = ks / 4;
    if (p.K % ks != 0 || p.G % kt != 0 || p.K % p.G != 0 || (ks * kConsumerWarps) % p.G != 0) return false;
    if (p.B > 16) return false;
    if ((size_t)p.Gn * kRowBlock * 2 * 10 > 96 * 1024) return false;
    if (!aligned16(p.x) || !aligned16(p.w[0]) || (p.w[1] != nullptr && !aligned16(p.w[1]))) return false;
    if (p.res_in != nullptr && !aligned16(p.res_in)) return false;
    if (p.z_out != nullptr && !aligned16(p.z_out)) return false;
    if (p.normed_out != nullptr && !aligned16(p.normed_out)) return false;
    if (p.row_bytes % 16 != 0) return false;
    return true;
}

template <bool GATE_UP>
int dispatch_fast(int bits, GemvParams& p, cudaStream_t stream) {
    if (bits == 4) return p.B <= 8 ? launch_fast<4, 1, GATE_UP>(p, stream) : launch_fast<4, 2, GATE_UP>(p, stream);
    return p.B <= 8 ? launch_fast<8, 1, GATE_UP>(p, stream) : launch_fast<8, 2, GATE_UP>(p, stream);
}

}  // namespace

// Declared in api.cu
int rmsnorm_residual_launch(const void* x, const void* residual, const void* weight, void* y, void* z_out,
                            int64_t rows, int64_t D, float eps, int dtype, int w_dtype, cudaStream_t stream);

int qmatvec_impl(int bits, const void* x, const uint8_t* codes, const void* scales, const void* zeros,
                 const void* residual, void* y, int B, int64_t N, int64_t K, int group_size, int act_dtype,
                 int scale_dtype, cudaStream_t stream) {
    if ((bits != 4 && bits != 8) || x == nullptr || codes == nullptr || scales == nullptr || y == nullptr)
        return B200Q_ERR_BAD_ARG;
    if (B <= 0 || N <= 0 || K <= 0 || group_size <= 0 || !is_act_dtype(act_dtype) || !is_scale_dtype(scale_dtype))
        return B200Q_ERR_BAD_ARG;
    if (N > INT32_MAX || K > INT32_MAX) return B200Q_ERR_UNSUPPORTED;
    const int esz = 2;
    for (int b0 = 0; b0 < B; b0 += 16) {
        GemvParams p = {};
        const int bn = std::min(16, B - b0);
        p.x = reinterpret_cast<const uint8_t*>(x) + (size_t)b0 * K * esz;
        p.w[0] = codes; p.s[0] = scales; p.z[0] = zeros;
        p.residual = residual ? reinterpret_cast<const uint8_t*>(residual) + (size_t)b0 * N * esz : nullptr;
        p.y = reinterpret_cast<uint8_t*>(y) + (size_t)b0 * N * esz;
        p.B = bn; p.N = (int)N; p.K = (int)K; p.G = group_size; p.Gn = (int)((K + group_size - 1) / group_size);
        p.act_dtype = act_dtype; p.scale_dtype = scale_dtype;
        p.row_bytes = bits == 4 ? (int)((K + 1) / 2) : (int)K;
        int rc;
        if (fast_path_ok(p, bits)) rc = dispatch_fast<false>(bits, p, stream);
        else rc = launch_generic<false>(p, bits, stream);
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
        if (fast_path_ok(p, bits)) {
            rc = dispatch_fast<true>(bits, p, stream);
        } else {
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
